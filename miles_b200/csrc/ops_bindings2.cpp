// Bindings of the rollout-engine kernels (paged attention, sampling), RL scans and quantisers.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "launchers.h"

void register_more(pybind11::module_& m) {}
