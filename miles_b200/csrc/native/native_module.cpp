// Python module `miles_b200._native`: the host-only runtime pieces (no CUDA, no PyTorch dependency), so that they
// load and are tested on machines without a GPU.
#include <pybind11/pybind11.h>

void register_engine_core(pybind11::module_& m);
void register_control_plane(pybind11::module_& m);

PYBIND11_MODULE(_native, m) {
  m.doc() = "miles_b200 host runtime: engine scheduler / page pool, quorum store, router table";
  register_engine_core(m);
  register_control_plane(m);
}
