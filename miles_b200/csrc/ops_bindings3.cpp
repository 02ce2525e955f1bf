// Bindings of the symmetric-memory allocator and the expert-parallel exchange kernels.
#include <cmath>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "launchers.h"

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

// Allocates device memory that peers can map; returns (address, 64-byte IPC handle).
std::pair<int64_t, pybind11::bytes> symm_alloc(int64_t nbytes) {
  void* p = nullptr;
  char h[64];
  const int rc = mb::symm_alloc(static_cast<size_t>(nbytes), &p, h);
  TORCH_CHECK(rc == 0, "symm_alloc failed with CUDA error ", rc);
  return {reinterpret_cast<int64_t>(p), pybind11::bytes(h, 64)};
}
int64_t symm_open(const std::string& handle) {
  TORCH_CHECK(handle.size() == 64, "an IPC handle is 64 bytes");
  void* p = nullptr;
  const int rc = mb::symm_open(handle.data(), &p);
  TORCH_CHECK(rc == 0, "symm_open failed with CUDA error ", rc);
  return reinterpret_cast<int64_t>(p);
}
void symm_close(int64_t p) { mb::symm_close(reinterpret_cast<void*>(p)); }
void symm_free(int64_t p) { mb::symm_free(reinterpret_cast<void*>(p)); }

// A non-owning tensor over raw device memory.
at::Tensor tensor_from_ptr(int64_t ptr, std::vector<int64_t> shape, at::ScalarType dtype, int64_t device) {
  auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, device);
  return at::from_blob(reinterpret_cast<void*>(ptr), shape, [](void*) {}, opts);
}

mb::EpPeers make_peers(const std::vector<int64_t>& xrecv, const std::vector<int64_t>& meta, const std::vector<int64_t>& counts,
                       const std::vector<int64_t>& flags, const std::vector<int64_t>& yback, const std::vector<int64_t>& flags2) {
  mb::EpPeers p{};
  const size_t n = xrecv.size();
  TORCH_CHECK(n <= mb::kMaxPeers, "at most ", mb::kMaxPeers, " expert-parallel ranks");
  for (size_t i = 0; i < n; ++i) {
    p.xrecv[i] = reinterpret_cast<void*>(xrecv[i]);
    p.meta[i] = reinterpret_cast<int*>(meta[i]);
    p.counts[i] = reinterpret_cast<int*>(counts[i]);
    p.flags[i] = reinterpret_cast<unsigned long long*>(flags[i]);
    p.yback[i] = reinterpret_cast<void*>(yback[i]);
    p.flags2[i] = reinterpret_cast<unsigned long long*>(flags2[i]);
  }
  return p;
}

void ep_dispatch(const at::Tensor& x, const at::Tensor& ids, const at::Tensor& dest_row, const at::Tensor& offsets,
                 const at::Tensor& send_counts, const std::vector<int64_t>& xrecv, const std::vector<int64_t>& meta,
                 const std::vector<int64_t>& counts, const std::vector<int64_t>& flags, const std::vector<int64_t>& yback,
                 const std::vector<int64_t>& flags2, int64_t me, int64_t experts_per_rank, int64_t row_div, int64_t cap,
                 at::Tensor& ctrl, at::Tensor& status) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.size(-1) % 8 == 0, "bad x");
  const c10::cuda::CUDAGuard guard(x.device());
  mb::EpPeers p = make_peers(xrecv, meta, counts, flags, yback, flags2);
  p.send_counts = send_counts.data_ptr<int>();
  mb::ep_dispatch(x.data_ptr(), ids.data_ptr<int>(), dest_row.data_ptr<int>(), offsets.data_ptr<int>(), p, me, xrecv.size(),
                  experts_per_rank, ids.numel(), row_div, x.size(-1), cap,
                  reinterpret_cast<unsigned long long*>(ctrl.data_ptr<int64_t>()), status.data_ptr<int>(), cur_stream());
}

void ep_wait(const at::Tensor& flags, int64_t nranks, at::Tensor& ctrl, int64_t which, at::Tensor& status) {
  const c10::cuda::CUDAGuard guard(flags.device());
  mb::ep_wait(reinterpret_cast<const unsigned long long*>(flags.data_ptr<int64_t>()), nranks,
              reinterpret_cast<unsigned long long*>(ctrl.data_ptr<int64_t>()), which, status.data_ptr<int>(), cur_stream());
}

void ep_return(const at::Tensor& yp, const at::Tensor& recv_dest_row, const at::Tensor& meta_local, const at::Tensor& counts_local,
               const std::vector<int64_t>& xrecv, const std::vector<int64_t>& meta, const std::vector<int64_t>& counts,
               const std::vector<int64_t>& flags, const std::vector<int64_t>& yback, const std::vector<int64_t>& flags2,
               int64_t me, int64_t cap, at::Tensor& ctrl, at::Tensor& status) {
  TORCH_CHECK(yp.is_cuda() && yp.scalar_type() == at::kBFloat16 && yp.is_contiguous(), "bad yp");
  const c10::cuda::CUDAGuard guard(yp.device());
  mb::EpPeers p = make_peers(xrecv, meta, counts, flags, yback, flags2);
  mb::ep_return(yp.data_ptr(), recv_dest_row.data_ptr<int>(), meta_local.data_ptr<int>(), counts_local.data_ptr<int>(), p, me,
                xrecv.size(), cap, yp.size(-1), reinterpret_cast<unsigned long long*>(ctrl.data_ptr<int64_t>()),
                status.data_ptr<int>(), cur_stream());
}

at::Tensor ep_row_ptrs(const at::Tensor& row_src, const at::Tensor& meta_local, const std::vector<int64_t>& xrecv,
                       const std::vector<int64_t>& meta, const std::vector<int64_t>& counts, const std::vector<int64_t>& flags,
                       const std::vector<int64_t>& yback, const std::vector<int64_t>& flags2, int64_t cap, int64_t H) {
  TORCH_CHECK(row_src.is_cuda() && row_src.scalar_type() == at::kInt && row_src.is_contiguous(), "bad row_src");
  const c10::cuda::CUDAGuard guard(row_src.device());
  mb::EpPeers p = make_peers(xrecv, meta, counts, flags, yback, flags2);
  at::Tensor out = at::empty({row_src.numel()}, row_src.options().dtype(at::kLong));
  mb::ep_row_ptrs(row_src.data_ptr<int>(), meta_local.data_ptr<int>(), p, cap, H, row_src.numel(),
                  reinterpret_cast<unsigned long long*>(out.data_ptr<int64_t>()), cur_stream());
  return out;
}

// slots: [n, slot_elems] bf16 (contiguous); out/residual: the first `out.numel()` elements of a slot's layout.
void sum_slots(const at::Tensor& slots, const c10::optional<at::Tensor>& residual, at::Tensor& out) {
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kBFloat16 && slots.is_contiguous() && slots.dim() == 2, "bad slots");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.numel() % 8 == 0 && out.numel() <= slots.size(1) &&
                  slots.size(1) % 8 == 0, "bad out");
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && residual->numel() == out.numel() && residual->scalar_type() == at::kBFloat16, "bad residual");
  const c10::cuda::CUDAGuard guard(slots.device());
  mb::sum_slots(slots.data_ptr(), slots.size(1), slots.size(0), residual.has_value() ? residual->data_ptr() : nullptr,
                out.data_ptr(), out.numel(), cur_stream());
}

mb::DpPeers make_dp_peers(const std::vector<int64_t>& grad, const std::vector<int64_t>& param, const std::vector<int64_t>& flags,
                          const std::vector<int64_t>& flags2) {
  mb::DpPeers p{};
  TORCH_CHECK(grad.size() <= mb::kMaxPeers && grad.size() == param.size(), "at most ", mb::kMaxPeers, " data-parallel ranks");
  for (size_t i = 0; i < grad.size(); ++i) {
    p.grad[i] = reinterpret_cast<void*>(grad[i]);
    p.param[i] = reinterpret_cast<void*>(param[i]);
    p.flags[i] = reinterpret_cast<unsigned long long*>(flags[i]);
    p.flags2[i] = reinterpret_cast<unsigned long long*>(flags2[i]);
  }
  return p;
}

void peer_signal(const std::vector<int64_t>& grad, const std::vector<int64_t>& param, const std::vector<int64_t>& flags,
                 const std::vector<int64_t>& flags2, int64_t me, at::Tensor& ctrl, int64_t which, bool second) {
  const c10::cuda::CUDAGuard guard(ctrl.device());
  mb::peer_signal(make_dp_peers(grad, param, flags, flags2), me, grad.size(),
                  reinterpret_cast<unsigned long long*>(ctrl.data_ptr<int64_t>()), which, second, cur_stream());
}

// reduced: fp32 [shard]; returns the per-block partial sums of squares (add them up in order for a reproducible norm)
at::Tensor dp_reduce_shard(const std::vector<int64_t>& grad, const std::vector<int64_t>& param, const std::vector<int64_t>& flags,
                           const std::vector<int64_t>& flags2, int64_t lo, at::Tensor& reduced) {
  TORCH_CHECK(reduced.is_cuda() && reduced.scalar_type() == at::kFloat && reduced.is_contiguous(), "bad reduced buffer");
  TORCH_CHECK(lo % 8 == 0 && reduced.numel() % 8 == 0, "shard bounds must be multiples of 8 elements");
  const c10::cuda::CUDAGuard guard(reduced.device());
  const int blocks = mb::dp_reduce_shard_blocks(reduced.numel());
  at::Tensor partial = at::zeros({blocks}, reduced.options());
  mb::dp_reduce_shard(make_dp_peers(grad, param, flags, flags2), grad.size(), lo, reduced.numel(), reduced.data_ptr<float>(),
                      partial.data_ptr<float>(), cur_stream());
  return partial;
}

void dp_adam_push(const std::vector<int64_t>& grad, const std::vector<int64_t>& param, const std::vector<int64_t>& flags,
                  const std::vector<int64_t>& flags2, int64_t me, int64_t lo, const at::Tensor& reduced,
                  const c10::optional<at::Tensor>& master, at::Tensor& m, at::Tensor& v, double lr, double b1, double b2, double eps,
                  double wd, int64_t step, const at::Tensor& grad_scale, const at::Tensor& skip_flag) {
  const int64_t n = reduced.numel();
  TORCH_CHECK(lo % 8 == 0 && n % 8 == 0 && m.numel() == n && v.numel() == n, "piece bounds must be multiples of 8 elements");
  TORCH_CHECK(m.scalar_type() == v.scalar_type() && (m.scalar_type() == at::kFloat || m.scalar_type() == at::kBFloat16), "bad moment dtype");
  const c10::cuda::CUDAGuard guard(reduced.device());
  const float bc1 = 1.0f - static_cast<float>(std::pow(b1, static_cast<double>(step)));
  const float bc2 = 1.0f - static_cast<float>(std::pow(b2, static_cast<double>(step)));
  mb::dp_adam_push(make_dp_peers(grad, param, flags, flags2), me, grad.size(), lo, n, reduced.data_ptr<float>(),
                   master.has_value() ? master->data_ptr<float>() : nullptr, m.data_ptr(), v.data_ptr(),
                   m.scalar_type() == at::kBFloat16, lr, b1, b2, eps, wd, bc1, bc2, grad_scale.data_ptr<float>(),
                   skip_flag.data_ptr<float>(), cur_stream());
}

}  // namespace

void register_comm(pybind11::module_& m) {
  m.def("symm_alloc", &symm_alloc);
  m.def("symm_open", &symm_open);
  m.def("symm_close", &symm_close);
  m.def("symm_free", &symm_free);
  m.def("tensor_from_ptr", &tensor_from_ptr);
  m.def("ep_dispatch", &ep_dispatch);
  m.def("ep_wait", &ep_wait);
  m.def("ep_return", &ep_return);
  m.def("ep_row_ptrs", &ep_row_ptrs);
  m.def("sum_slots", &sum_slots);
  m.def("peer_signal", &peer_signal);
  m.def("dp_reduce_shard", &dp_reduce_shard);
  m.def("dp_adam_push", &dp_adam_push);
  // Per-context preference for a large shared-memory carve-out: decode alternates kernels that use ~200 KB of shared
  // memory with kernels that use none, and without a common preference the SM re-partitions L1 / shared memory in between.
  m.def("device_prefer_shared_memory", [](bool on) {
    return static_cast<int>(cudaDeviceSetCacheConfig(on ? cudaFuncCachePreferShared : cudaFuncCachePreferNone));
  });
}
