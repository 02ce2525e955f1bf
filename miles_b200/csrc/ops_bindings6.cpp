// Bindings of the trainer -> engine weight push (weight_push.cu).
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "launchers.h"

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

// src: the local shard (bf16, any shape, contiguous); segs int64 [nseg, 8]; tensors int64 [nt, 8] (device);
// amax fp32 [slots] or None; bases: the symmetric region base of every rank; counter: one int32 zero on the device.
void weight_push(const at::Tensor& src, const at::Tensor& segs, const at::Tensor& tensors, const c10::optional<at::Tensor>& amax,
                 const std::vector<int64_t>& bases, int64_t flag_off, int64_t me, int64_t flag_mask, int64_t version,
                 at::Tensor& counter, int64_t total_vecs) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kBFloat16 && src.is_contiguous(), "src: contiguous bf16 on the device");
  TORCH_CHECK(segs.is_cuda() && segs.scalar_type() == at::kLong && segs.is_contiguous() && segs.dim() == 2 && segs.size(1) == 8,
              "segs: int64 [nseg, 8] on the device");
  TORCH_CHECK(tensors.is_cuda() && tensors.scalar_type() == at::kLong && tensors.is_contiguous() && tensors.dim() == 2 && tensors.size(1) == 8,
              "tensors: int64 [n, 8] on the device");
  TORCH_CHECK(counter.is_cuda() && counter.scalar_type() == at::kInt && counter.numel() >= 1, "counter: int32 on the device");
  TORCH_CHECK(!bases.empty() && bases.size() <= 8 && me >= 0 && me < static_cast<int64_t>(bases.size()), "1 to 8 ranks");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0 && flag_off % 8 == 0, "16-byte aligned source, 8-byte aligned flags");
  static_assert(sizeof(mb::WeightPushSeg) == 64 && sizeof(mb::WeightPushTensor) == 64, "tables are rows of eight int64");
  const float* am = nullptr;
  if (amax.has_value() && amax->defined()) {
    TORCH_CHECK(amax->is_cuda() && amax->scalar_type() == at::kFloat && amax->is_contiguous(), "amax: fp32 on the device");
    am = amax->data_ptr<float>();
  }
  mb::WeightPushPeers p{};
  for (size_t i = 0; i < bases.size(); ++i) p.base[i] = reinterpret_cast<char*>(bases[i]);
  p.flag_off = flag_off;
  const c10::cuda::CUDAGuard guard(src.device());
  const int rc = mb::weight_push(src.data_ptr(), reinterpret_cast<const mb::WeightPushSeg*>(segs.data_ptr<int64_t>()),
                                 static_cast<int>(segs.size(0)), reinterpret_cast<const mb::WeightPushTensor*>(tensors.data_ptr<int64_t>()),
                                 am, p, static_cast<int>(me), static_cast<unsigned>(flag_mask), static_cast<unsigned long long>(version),
                                 reinterpret_cast<unsigned int*>(counter.data_ptr<int>()), total_vecs, cur_stream());
  TORCH_CHECK(rc == 0, "weight_push: the launch failed");
}

// flags_addr: address of this rank's 8 arrival flags (inside its symmetric region).
void weight_push_wait(int64_t flags_addr, int64_t src_mask, int64_t version, double wait_ms, at::Tensor& status) {
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt, "status: int32 on the device");
  const c10::cuda::CUDAGuard guard(status.device());
  mb::weight_push_wait(reinterpret_cast<const unsigned long long*>(flags_addr), static_cast<unsigned>(src_mask),
                       static_cast<unsigned long long>(version), wait_ms, status.data_ptr<int>(), cur_stream());
}

}  // namespace

void register_weight_push(pybind11::module_& m) {
  m.def("weight_push", &weight_push);
  m.def("weight_push_wait", &weight_push_wait);
}
