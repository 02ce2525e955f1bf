// Control-plane primitives that the reference takes from Rust crates: a quorum/heartbeat store (the role of
// torchft's lighthouse for the fault-tolerant trainer cells) and the worker table of the request router (the
// role of sgl-model-gateway: least-inflight selection with failure quarantine). Both are plain thread-safe C++
// state machines; the Python HTTP front-ends (ft/control_server.py, router/router.py) call into them.
//
// Reference counterpart: torchft quorum (miles/backends/megatron_utils/ft/indep_dp.py:24-185,
// miles/ray/train/group.py:332-455) and the router (miles/router/router.py:34-236,
// miles/ray/rollout/router_manager.py:18-77).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace py = pybind11;

namespace {

double now_s() {
  using namespace std::chrono;
  return duration<double>(steady_clock::now().time_since_epoch()).count();
}

// ---------------------------------------------------------------------------------------------- quorum store
// Members heartbeat under a name. The quorum is the sorted list of members whose last heartbeat is younger than
// `timeout_s`; whenever that list changes the quorum id is bumped, and participants rebuild their process groups
// for the new id. `evict` and `join` are the explicit forms (a controller suspending / resuming a cell).
class QuorumStore {
 public:
  explicit QuorumStore(double timeout_s) : timeout_s_(timeout_s) {}

  int64_t heartbeat(const std::string& member, double t = -1.0) {
    std::lock_guard<std::mutex> lk(mu_);
    last_[member] = t >= 0 ? t : now_s();
    evicted_.erase(member);
    return refresh_locked(t);
  }
  int64_t evict(const std::string& member) {
    std::lock_guard<std::mutex> lk(mu_);
    evicted_[member] = true;
    return refresh_locked(-1.0);
  }
  // (quorum id, members) as seen now
  std::pair<int64_t, std::vector<std::string>> quorum(double t = -1.0) {
    std::lock_guard<std::mutex> lk(mu_);
    refresh_locked(t);
    return {id_, members_};
  }
  // rank of `member` in the current quorum, -1 if it is not part of it
  int rank_of(const std::string& member) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = std::find(members_.begin(), members_.end(), member);
    return it == members_.end() ? -1 : static_cast<int>(it - members_.begin());
  }

 private:
  int64_t refresh_locked(double t) {
    const double now = t >= 0 ? t : now_s();
    std::vector<std::string> alive;
    for (const auto& kv : last_)
      if (now - kv.second <= timeout_s_ && !evicted_.count(kv.first)) alive.push_back(kv.first);
    std::sort(alive.begin(), alive.end());
    if (alive != members_) {
      members_ = alive;
      ++id_;
    }
    return id_;
  }
  std::mutex mu_;
  double timeout_s_;
  int64_t id_ = 0;
  std::map<std::string, double> last_;
  std::map<std::string, bool> evicted_;
  std::vector<std::string> members_;
};

// ---------------------------------------------------------------------------------------------- router table
class RouterTable {
 public:
  explicit RouterTable(int max_failures) : max_failures_(max_failures) {}

  void add(const std::string& url) {
    std::lock_guard<std::mutex> lk(mu_);
    workers_.emplace(url, Worker{});
  }
  bool remove(const std::string& url) {
    std::lock_guard<std::mutex> lk(mu_);
    return workers_.erase(url) > 0;
  }
  // Healthy worker with the fewest requests in flight (ties: the one used least recently); "" if none.
  std::string acquire() {
    std::lock_guard<std::mutex> lk(mu_);
    Worker* best = nullptr;
    const std::string* best_url = nullptr;
    for (auto& kv : workers_) {
      Worker& w = kv.second;
      if (w.quarantined) continue;
      if (!best || w.inflight < best->inflight || (w.inflight == best->inflight && w.last_used < best->last_used)) {
        best = &w;
        best_url = &kv.first;
      }
    }
    if (!best) return "";
    ++best->inflight;
    best->last_used = ++clock_;
    ++best->served;
    return *best_url;
  }
  void release(const std::string& url, bool ok) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = workers_.find(url);
    if (it == workers_.end()) return;
    Worker& w = it->second;
    if (w.inflight > 0) --w.inflight;
    report_locked(w, ok);
  }
  // undo an acquire without recording an outcome
  void cancel(const std::string& url) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = workers_.find(url);
    if (it != workers_.end() && it->second.inflight > 0) {
      --it->second.inflight;
      --it->second.served;
    }
  }
  void report_health(const std::string& url, bool ok) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = workers_.find(url);
    if (it != workers_.end()) report_locked(it->second, ok);
  }
  void readmit(const std::string& url) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = workers_.find(url);
    if (it != workers_.end()) {
      it->second.quarantined = false;
      it->second.failures = 0;
    }
  }
  std::vector<std::string> urls(bool healthy_only) {
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<std::string> r;
    for (const auto& kv : workers_)
      if (!healthy_only || !kv.second.quarantined) r.push_back(kv.first);
    return r;
  }
  py::dict snapshot() {
    std::lock_guard<std::mutex> lk(mu_);
    py::dict d;
    for (const auto& kv : workers_)
      d[py::str(kv.first)] = py::make_tuple(kv.second.inflight, kv.second.failures, kv.second.quarantined, kv.second.served);
    return d;
  }

 private:
  struct Worker {
    int inflight = 0;
    int failures = 0;
    bool quarantined = false;
    int64_t last_used = 0;
    int64_t served = 0;
  };
  void report_locked(Worker& w, bool ok) {
    if (ok) {
      w.failures = 0;
    } else if (++w.failures >= max_failures_) {
      w.quarantined = true;
    }
  }
  std::mutex mu_;
  int max_failures_;
  int64_t clock_ = 0;
  std::map<std::string, Worker> workers_;
};

}  // namespace

void register_control_plane(py::module_& m) {
  py::class_<QuorumStore>(m, "QuorumStore")
      .def(py::init<double>(), py::arg("timeout_s") = 30.0)
      .def("heartbeat", &QuorumStore::heartbeat, py::arg("member"), py::arg("t") = -1.0)
      .def("evict", &QuorumStore::evict)
      .def("quorum", &QuorumStore::quorum, py::arg("t") = -1.0)
      .def("rank_of", &QuorumStore::rank_of);
  py::class_<RouterTable>(m, "RouterTable")
      .def(py::init<int>(), py::arg("max_failures") = 3)
      .def("add", &RouterTable::add)
      .def("remove", &RouterTable::remove)
      .def("acquire", &RouterTable::acquire)
      .def("release", &RouterTable::release)
      .def("cancel", &RouterTable::cancel)
      .def("report_health", &RouterTable::report_health)
      .def("readmit", &RouterTable::readmit)
      .def("urls", &RouterTable::urls, py::arg("healthy_only") = true)
      .def("snapshot", &RouterTable::snapshot);
}
