// Host-side core of the rollout engine: the KV page pool (all-or-nothing allocation, double-release and range
// checks). Admission, page growth, retraction and the prefix tree live in the Python engine (engine/core.py,
// engine/prefix_cache.py), which overlaps that host work with the decode step in flight.
//
// Reference counterpart: SGLang's scheduler and token-to-KV pool allocator behind the engines that
// miles/backends/sglang_utils/sglang_engine.py:73-152 launches.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <unordered_map>
#include <vector>

namespace py = pybind11;

namespace {

class PagePool {
 public:
  explicit PagePool(int num_pages) : num_pages_(num_pages) {
    if (num_pages < 2) throw std::invalid_argument("the pool needs at least 2 pages (page 0 is reserved)");
    free_.reserve(num_pages - 1);
    for (int p = num_pages - 1; p >= 1; --p) free_.push_back(p);  // page 0: scratch target of dummy writes
  }
  int num_free() const { return static_cast<int>(free_.size()); }
  int num_pages() const { return num_pages_; }
  // all-or-nothing allocation; an empty vector with ok=false means "not enough pages"
  bool alloc(int n, std::vector<int>& out) {
    if (n < 0 || n > num_free()) return false;
    for (int i = 0; i < n; ++i) {
      out.push_back(free_.back());
      free_.pop_back();
    }
    return true;
  }
  void release(const std::vector<int>& pages) {
    for (int p : pages) {
      if (p <= 0 || p >= num_pages_) throw std::out_of_range("released page id out of range");
      free_.push_back(p);
    }
    if (static_cast<int>(free_.size()) > num_pages_ - 1) throw std::logic_error("page released twice");
  }

 private:
  int num_pages_;
  std::vector<int> free_;
};

}  // namespace

void register_engine_core(py::module_& m) {
  py::class_<PagePool>(m, "PagePool")
      .def(py::init<int>())
      .def_property_readonly("num_free", &PagePool::num_free)
      .def_property_readonly("num_pages", &PagePool::num_pages)
      .def("alloc",
           [](PagePool& p, int n) -> py::object {
             std::vector<int> out;
             if (!p.alloc(n, out)) return py::none();
             return py::cast(out);
           })
      .def("release", &PagePool::release);
}
