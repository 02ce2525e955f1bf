// Tagged virtual-memory allocator: device allocations whose physical memory can be released and brought back
// without changing their addresses.
//
// Every allocation reserves a virtual address range (cuMemAddressReserve) and maps freshly created physical
// memory into it (cuMemCreate + cuMemMap). `pause(tag)` unmaps and releases the physical memory of all
// allocations carrying the tag (optionally after copying their contents to host memory), `resume(tag)` creates
// new physical memory at the same addresses (and copies the contents back). Tensors, CUDA graphs and kernels
// that hold the pointers stay valid across a pause/resume cycle, which is what lets a colocated trainer hand its
// memory to the rollout engine and take it back. The functions `mb_vmm_malloc` / `mb_vmm_free` have the
// signature of PyTorch's pluggable allocator, so a `torch.cuda.MemPool` can draw from this arena; the tag that
// new allocations receive is set with `vmm_set_tag`.
//
// The driver entry points are resolved at run time (cudaGetDriverEntryPoint), so the library links against
// the CUDA runtime only.
//
// Reference counterpart: torch_memory_saver (LD_PRELOAD hook over cudaMalloc with cuMemCreate/cuMemMap, pause and
// resume by tag) used by miles/backends/megatron_utils/actor.py:299-341 and ray/train/actor_factory.py:44-60.
#include <cuda.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace py = pybind11;

namespace {

struct Driver {
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*memRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*addrReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addrFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*memUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*setAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  bool ok = false;
};

template <typename F>
bool resolve(const char* name, F& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return false;
  fn = reinterpret_cast<F>(p);
  return true;
}

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.ok = resolve("cuMemCreate", d.memCreate) && resolve("cuMemRelease", d.memRelease) &&
           resolve("cuMemAddressReserve", d.addrReserve) && resolve("cuMemAddressFree", d.addrFree) &&
           resolve("cuMemMap", d.memMap) && resolve("cuMemUnmap", d.memUnmap) && resolve("cuMemSetAccess", d.setAccess) &&
           resolve("cuMemGetAllocationGranularity", d.granularity);
  });
  return d;
}

struct Block {
  size_t size = 0;          // mapped size (multiple of the granularity)
  size_t requested = 0;
  int device = 0;
  std::string tag;
  CUmemGenericAllocationHandle handle = 0;
  bool mapped = false;
  std::vector<char> backup;  // host copy while paused (only when the pause asked for it)
  bool has_backup = false;
};

std::mutex g_mu;
std::map<CUdeviceptr, Block> g_blocks;
std::string g_tag = "default";
std::string g_err;

CUmemAllocationProp prop_for(int device) {
  CUmemAllocationProp p;
  std::memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}

bool map_block(CUdeviceptr va, Block& b) {
  Driver& d = driver();
  const CUmemAllocationProp p = prop_for(b.device);
  if (d.memCreate(&b.handle, b.size, &p, 0) != CUDA_SUCCESS) return false;
  if (d.memMap(va, b.size, 0, b.handle, 0) != CUDA_SUCCESS) {
    d.memRelease(b.handle);
    return false;
  }
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = b.device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.setAccess(va, b.size, &acc, 1) != CUDA_SUCCESS) {
    d.memUnmap(va, b.size);
    d.memRelease(b.handle);
    return false;
  }
  b.mapped = true;
  return true;
}

}  // namespace

extern "C" void* mb_vmm_malloc(ssize_t size, int device, cudaStream_t /*stream*/) {
  Driver& d = driver();
  if (!d.ok || size <= 0) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  cudaSetDevice(device);
  cudaFree(nullptr);  // make sure the primary context exists
  const CUmemAllocationProp p = prop_for(device);
  size_t gran = 0;
  if (d.granularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_MINIMUM) != CUDA_SUCCESS || gran == 0) return nullptr;
  Block b;
  b.requested = static_cast<size_t>(size);
  b.size = (b.requested + gran - 1) / gran * gran;
  b.device = device;
  b.tag = g_tag;
  CUdeviceptr va = 0;
  if (d.addrReserve(&va, b.size, gran, 0, 0) != CUDA_SUCCESS) return nullptr;
  if (!map_block(va, b)) {
    d.addrFree(va, b.size);
    return nullptr;
  }
  g_blocks[va] = std::move(b);
  return reinterpret_cast<void*>(va);
}

extern "C" void mb_vmm_free(void* ptr, ssize_t /*size*/, int /*device*/, cudaStream_t /*stream*/) {
  Driver& d = driver();
  std::lock_guard<std::mutex> lk(g_mu);
  const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(ptr);
  auto it = g_blocks.find(va);
  if (it == g_blocks.end()) return;
  Block& b = it->second;
  if (b.mapped) {
    d.memUnmap(va, b.size);
    d.memRelease(b.handle);
  }
  d.addrFree(va, b.size);
  g_blocks.erase(it);
}

namespace {

void set_tag(const std::string& tag) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_tag = tag;
}

// Releases the physical memory of every mapped allocation with this tag. Returns the number of bytes released.
size_t pause_tag(const std::string& tag, bool keep_contents) {
  Driver& d = driver();
  if (!d.ok) throw std::runtime_error("CUDA virtual memory management is not available");
  cudaDeviceSynchronize();  // nothing may still be using the memory
  std::lock_guard<std::mutex> lk(g_mu);
  size_t released = 0;
  for (auto& kv : g_blocks) {
    Block& b = kv.second;
    if (b.tag != tag || !b.mapped) continue;
    if (keep_contents) {
      b.backup.resize(b.requested);
      if (cudaMemcpy(b.backup.data(), reinterpret_cast<void*>(kv.first), b.requested, cudaMemcpyDeviceToHost) != cudaSuccess)
        throw std::runtime_error("copy to host failed while pausing tag " + tag);
      b.has_backup = true;
    }
    if (d.memUnmap(kv.first, b.size) != CUDA_SUCCESS) throw std::runtime_error("cuMemUnmap failed");
    d.memRelease(b.handle);
    b.mapped = false;
    released += b.size;
  }
  return released;
}

size_t resume_tag(const std::string& tag) {
  Driver& d = driver();
  if (!d.ok) throw std::runtime_error("CUDA virtual memory management is not available");
  std::lock_guard<std::mutex> lk(g_mu);
  size_t mapped = 0;
  for (auto& kv : g_blocks) {
    Block& b = kv.second;
    if (b.tag != tag || b.mapped) continue;
    if (!map_block(kv.first, b)) throw std::runtime_error("out of device memory while resuming tag " + tag);
    if (b.has_backup) {
      if (cudaMemcpy(reinterpret_cast<void*>(kv.first), b.backup.data(), b.requested, cudaMemcpyHostToDevice) != cudaSuccess)
        throw std::runtime_error("copy from host failed while resuming tag " + tag);
      std::vector<char>().swap(b.backup);
      b.has_backup = false;
    }
    mapped += b.size;
  }
  return mapped;
}

py::dict stats() {
  std::lock_guard<std::mutex> lk(g_mu);
  std::map<std::string, std::pair<size_t, size_t>> per;  // tag -> (mapped bytes, paused bytes)
  for (const auto& kv : g_blocks) {
    auto& e = per[kv.second.tag];
    (kv.second.mapped ? e.first : e.second) += kv.second.size;
  }
  py::dict out;
  for (const auto& kv : per) out[py::str(kv.first)] = py::make_tuple(kv.second.first, kv.second.second);
  return out;
}

}  // namespace

void register_vmm(py::module_& m) {
  m.def("vmm_available", [] { return driver().ok; });
  m.def("vmm_set_tag", &set_tag);
  m.def("vmm_pause", &pause_tag, py::arg("tag"), py::arg("keep_contents") = false);
  m.def("vmm_resume", &resume_tag);
  m.def("vmm_stats", &stats);
  m.def("vmm_malloc", [](int64_t size, int device) { return reinterpret_cast<int64_t>(mb_vmm_malloc(size, device, nullptr)); });
  m.def("vmm_free", [](int64_t ptr) { mb_vmm_free(reinterpret_cast<void*>(ptr), 0, 0, nullptr); });
}
