// Bindings of the block-scaled (MXFP8 / NVFP4) GEMM and its scale-factor layout kernel.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "gemm.h"

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

// scales: uint8 [rows, S] row-major -> uint8 [ceil(rows/128), ceil(S/4), 512]
at::Tensor sf_swizzle(const at::Tensor& scales) {
  TORCH_CHECK(scales.is_cuda() && scales.scalar_type() == at::kByte && scales.dim() == 2 && scales.is_contiguous(),
              "scales must be a contiguous uint8 CUDA matrix");
  const c10::cuda::CUDAGuard guard(scales.device());
  const int64_t rows = scales.size(0), S = scales.size(1);
  at::Tensor out = at::zeros({(rows + 127) / 128, (S + 3) / 4, 512}, scales.options());
  mb::sf_swizzle(scales.data_ptr<uint8_t>(), out.data_ptr<uint8_t>(), rows, static_cast<int>(S), cur_stream());
  return out;
}

// a: uint8 [M, K or K/2]; b: uint8 [N, ...] (dense) or [G*N, ...] (grouped rows); sfa / sfb: atoms from sf_swizzle.
at::Tensor gemm_mx(const at::Tensor& a, const at::Tensor& sfa, const at::Tensor& b, const at::Tensor& sfb, int64_t kind,
                   double alpha, int64_t n, const c10::optional<at::Tensor>& tile_group,
                   const c10::optional<at::Tensor>& num_m_tiles, const c10::optional<at::Tensor>& status, int64_t block_n,
                   const c10::optional<at::Tensor>& alpha_dev) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kByte && b.scalar_type() == at::kByte, "operands are uint8 CUDA tensors");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && a.size(1) == b.size(1), "operands are [rows, packed K] with equal K");
  TORCH_CHECK(sfa.is_contiguous() && sfb.is_contiguous() && sfa.scalar_type() == at::kByte && sfb.scalar_type() == at::kByte, "scale atoms are contiguous uint8");
  const c10::cuda::CUDAGuard guard(a.device());
  mb::MxGemmProblem p{};
  p.kind = static_cast<int>(kind);
  p.M = static_cast<int>(a.size(0));
  p.K = static_cast<int>(kind == 0 ? a.size(1) : a.size(1) * 2);
  const bool grouped = tile_group.has_value();
  p.N = static_cast<int>(grouped ? n : b.size(0));
  TORCH_CHECK(p.N > 0 && b.size(0) % p.N == 0, "B rows must be a multiple of N");
  p.mode = grouped ? mb::GEMM_GROUPED_ROWS : mb::GEMM_DENSE;
  p.num_groups = static_cast<int>(b.size(0) / p.N);
  p.a = a.data_ptr();
  p.a_rows = a.size(0);
  p.a_pitch_bytes = a.stride(0);
  p.b = b.data_ptr();
  p.b_rows = b.size(0);
  p.b_pitch_bytes = b.stride(0);
  const int64_t kgroups = p.K / (kind == 0 ? 128 : 64);
  TORCH_CHECK(sfa.numel() >= ((a.size(0) + 127) / 128) * kgroups * 512, "sfa is too small for A");
  TORCH_CHECK(sfb.numel() >= ((b.size(0) + 127) / 128) * kgroups * 512, "sfb is too small for B");
  p.sfa = sfa.data_ptr<uint8_t>();
  p.sfb = sfb.data_ptr<uint8_t>();
  at::Tensor out = at::empty({a.size(0), p.N}, a.options().dtype(at::kBFloat16));
  if (grouped) out.zero_();  // rows of tiles that are not live stay defined
  p.c = out.data_ptr();
  p.ldc = p.N;
  p.alpha = static_cast<float>(alpha);
  if (alpha_dev.has_value()) {
    TORCH_CHECK(alpha_dev->is_cuda() && alpha_dev->scalar_type() == at::kFloat && alpha_dev->numel() >= 1, "alpha_dev is a CUDA float scalar");
    p.alpha_dev = alpha_dev->data_ptr<float>();
  }
  if (grouped) {
    TORCH_CHECK(num_m_tiles.has_value() && tile_group->scalar_type() == at::kInt && tile_group->is_contiguous(), "grouped mode needs int32 tile_group and num_m_tiles");
    p.tile_group = tile_group->data_ptr<int>();
    p.num_m_tiles = num_m_tiles->data_ptr<int>();
    p.max_tiles = static_cast<int>(tile_group->numel() / 4);
  }
  p.block_n = static_cast<int>(block_n);
  p.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  const int rc = mb::gemm_mx_launch(p, cur_stream());
  TORCH_CHECK(rc == 0, "gemm_mx: ", mb::gemm_mx_last_error());
  return out;
}

}  // namespace

void register_mx(pybind11::module_& m) {
  m.def("sf_swizzle", &sf_swizzle);
  m.def("gemm_mx", &gemm_mx, pybind11::arg("a"), pybind11::arg("sfa"), pybind11::arg("b"), pybind11::arg("sfb"),
        pybind11::arg("kind"), pybind11::arg("alpha") = 1.0, pybind11::arg("n") = 0, pybind11::arg("tile_group") = pybind11::none(),
        pybind11::arg("num_m_tiles") = pybind11::none(), pybind11::arg("status") = pybind11::none(), pybind11::arg("block_n") = 0, pybind11::arg("alpha_dev") = pybind11::none());
}
