// Host-side core of the rollout engine: the KV page pool and the continuous-batching planner.
//
// The Python engine drives kernels and owns request objects; the bookkeeping that runs every decode step
// (which requests to admit under the prefill token budget, which pages every running request needs next,
// whom to retract when the pool runs dry) lives here so that a step costs a few microseconds of host time
// instead of Python loops over requests and page lists.
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

struct Seq {
  int64_t rid;
  int len;  // tokens so far (prompt + generated)
  std::vector<int> pages;
  int64_t order;  // admission order; the newest running request is retracted first
};

class Scheduler {
 public:
  Scheduler(int num_pages, int page_size, int max_running, int max_prefill_tokens)
      : pool_(num_pages), page_size_(page_size), max_running_(max_running), max_prefill_tokens_(max_prefill_tokens) {}

  int pages_needed(int tokens) const { return (tokens + page_size_ - 1) / page_size_; }
  int num_free_pages() const { return pool_.num_free(); }
  int num_running() const { return static_cast<int>(running_.size()); }

  // Waiting requests in arrival order as (rid, tokens to prefill). Admits a prefix of them under the slot,
  // token and page limits (a request needs pages for its tokens plus the one it will generate next).
  // Returns [(rid, pages)] of the admitted requests.
  std::vector<std::pair<int64_t, std::vector<int>>> admit(const std::vector<std::pair<int64_t, int>>& waiting) {
    std::vector<std::pair<int64_t, std::vector<int>>> out;
    int tokens = 0;
    for (const auto& w : waiting) {
      if (num_running() >= max_running_) break;
      if (!out.empty() && tokens + w.second > max_prefill_tokens_) break;
      std::vector<int> pages;
      if (!pool_.alloc(pages_needed(w.second + 1), pages)) break;
      Seq s{w.first, w.second, pages, next_order_++};
      index_[w.first] = running_.size();
      running_.push_back(std::move(s));
      out.emplace_back(w.first, running_.back().pages);
      tokens += w.second;
    }
    return out;
  }

  // One decode step is about to append a token to every running request: make sure each owns the page that
  // token lands in. When the pool is empty the newest request is retracted (its pages return to the pool, the
  // caller re-queues it). Returns (grown: [(rid, new page)], retracted: [rid]).
  std::pair<std::vector<std::pair<int64_t, int>>, std::vector<int64_t>> grow_for_decode() {
    std::vector<std::pair<int64_t, int>> grown;
    std::vector<int64_t> retracted;
    size_t i = 0;
    while (i < running_.size()) {
      Seq& s = running_[i];
      const int need = pages_needed(s.len + 1);
      bool dropped_self = false;
      while (static_cast<int>(s.pages.size()) < need) {
        std::vector<int> pg;
        if (pool_.alloc(1, pg)) {
          s.pages.push_back(pg[0]);
          grown.emplace_back(s.rid, pg[0]);
          continue;
        }
        // retract the newest running request
        size_t victim = 0;
        for (size_t j = 1; j < running_.size(); ++j)
          if (running_[j].order > running_[victim].order) victim = j;
        const int64_t vrid = running_[victim].rid;
        const bool self = victim == i;
        retracted.push_back(vrid);
        remove_at(victim);
        if (self) {
          dropped_self = true;
          break;
        }
        if (victim < i) --i;  // the vector shifted under us
      }
      if (!dropped_self) ++i;
    }
    return {grown, retracted};
  }

  void advance(int64_t rid, int tokens = 1) { at(rid).len += tokens; }
  void finish(int64_t rid) { remove_at(index_.at(rid)); }
  std::vector<int> pages_of(int64_t rid) { return at(rid).pages; }
  std::vector<int64_t> running_ids() const {
    std::vector<int64_t> r;
    for (const auto& s : running_) r.push_back(s.rid);
    return r;
  }

 private:
  Seq& at(int64_t rid) { return running_[index_.at(rid)]; }
  void remove_at(size_t i) {
    pool_.release(running_[i].pages);
    index_.erase(running_[i].rid);
    running_.erase(running_.begin() + i);
    for (size_t j = i; j < running_.size(); ++j) index_[running_[j].rid] = j;
  }
  PagePool pool_;
  int page_size_, max_running_, max_prefill_tokens_;
  int64_t next_order_ = 0;
  std::vector<Seq> running_;
  std::unordered_map<int64_t, size_t> index_;
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
  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<int, int, int, int>(), py::arg("num_pages"), py::arg("page_size"), py::arg("max_running"),
           py::arg("max_prefill_tokens"))
      .def("pages_needed", &Scheduler::pages_needed)
      .def_property_readonly("num_free_pages", &Scheduler::num_free_pages)
      .def_property_readonly("num_running", &Scheduler::num_running)
      .def("admit", &Scheduler::admit)
      .def("grow_for_decode", &Scheduler::grow_for_decode)
      .def("advance", &Scheduler::advance, py::arg("rid"), py::arg("tokens") = 1)
      .def("finish", &Scheduler::finish)
      .def("pages_of", &Scheduler::pages_of)
      .def("running_ids", &Scheduler::running_ids);
}
