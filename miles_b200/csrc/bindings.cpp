// PyTorch bindings for the sm_100a kernels. Only this file includes the PyTorch headers; every
// kernel lives in a plain CUDA translation unit with a C++ launcher declared in a header.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "gemm.h"
#include "launchers.h"

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

void check_bf16_2d(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bf16");
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, " must be 2-D with a contiguous inner dimension");
}

int* status_ptr(const c10::optional<at::Tensor>& status) {
  if (!status.has_value()) return nullptr;
  TORCH_CHECK(status->is_cuda() && status->scalar_type() == at::kInt, "status must be an int32 CUDA tensor");
  return status->data_ptr<int>();
}

mb::GemmOperand operand(const at::Tensor& t, bool mn_major) {
  mb::GemmOperand o;
  o.ptr = t.data_ptr();
  o.rows = t.size(0);
  o.cols = t.size(1);
  o.ld = t.stride(0);
  o.mn_major = mn_major;
  return o;
}

void fill_out(mb::GemmProblem& p, const at::Tensor& c) {
  TORCH_CHECK(c.is_cuda() && (c.scalar_type() == at::kBFloat16 || c.scalar_type() == at::kFloat),
              "output must be a bf16 or fp32 CUDA tensor");
  TORCH_CHECK(c.stride(-1) == 1, "output must have a contiguous inner dimension");
  p.c = c.data_ptr();
  p.out_fp32 = c.scalar_type() == at::kFloat;
}

void gemm(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool a_mn, bool b_mn, bool accumulate,
          int64_t block_n, const c10::optional<at::Tensor>& status, const std::vector<int64_t>& dest,
          const c10::optional<at::Tensor>& sig_ctrl, const std::vector<int64_t>& sig_flags, int64_t sig_me) {
  check_bf16_2d(a, "a");
  check_bf16_2d(b, "b");
  TORCH_CHECK(c.dim() == 2, "c must be 2-D");
  const c10::cuda::CUDAGuard guard(a.device());
  mb::GemmProblem p{};
  p.mode = mb::GEMM_DENSE;
  p.M = a_mn ? a.size(1) : a.size(0);
  p.K = a_mn ? a.size(0) : a.size(1);
  p.N = b_mn ? b.size(1) : b.size(0);
  const int64_t kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(kb == p.K, "contraction extents differ: ", p.K, " vs ", kb);
  TORCH_CHECK(c.size(0) == p.M && c.size(1) == p.N, "output shape must be [", p.M, ", ", p.N, "]");
  p.a = operand(a, a_mn);
  p.b = operand(b, b_mn);
  fill_out(p, c);
  p.ldc = c.stride(0);
  p.accumulate = accumulate;
  p.status = status_ptr(status);
  p.block_n = static_cast<int>(block_n);
  if (!dest.empty()) {  // replicated output: each destination receives the tile at the offset it has in c
    TORCH_CHECK(dest.size() <= 8, "at most 8 destinations");
    p.n_dest = static_cast<int>(dest.size());
    for (size_t i = 0; i < dest.size(); ++i) p.dest[i] = reinterpret_cast<void*>(dest[i]);
    if (sig_ctrl.has_value()) {
      TORCH_CHECK(sig_ctrl->scalar_type() == at::kLong && sig_ctrl->numel() >= 6 && sig_flags.size() <= 8, "bad signal arguments");
      p.sig_ctrl = reinterpret_cast<unsigned long long*>(sig_ctrl->data_ptr<int64_t>());
      for (size_t i = 0; i < sig_flags.size(); ++i) p.sig_flags[i] = reinterpret_cast<unsigned long long*>(sig_flags[i]);
      p.sig_nranks = static_cast<int>(sig_flags.size());
      p.sig_me = static_cast<int>(sig_me);
    }
  }
  TORCH_CHECK(mb::gemm_bf16_launch(p, cur_stream()) == 0, "gemm: ", mb::gemm_last_error());
}

// a: [rows, K] rows grouped in 128-row tiles; b: [G, N, K] (K-major) or [G, K, N] (MN-major).
void grouped_gemm_rows(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, const at::Tensor& tile_group,
                       const at::Tensor& num_m_tiles, bool b_mn, bool accumulate, int64_t block_n,
                       const c10::optional<at::Tensor>& status, const c10::optional<at::Tensor>& row_ptrs,
                       const c10::optional<at::Tensor>& sig_ctrl, const std::vector<int64_t>& sig_flags, int64_t sig_me) {
  check_bf16_2d(a, "a");
  TORCH_CHECK(b.is_cuda() && b.scalar_type() == at::kBFloat16 && b.dim() == 3 && b.is_contiguous(),
              "b must be a contiguous 3-D bf16 tensor");
  TORCH_CHECK(tile_group.scalar_type() == at::kInt && num_m_tiles.scalar_type() == at::kInt, "tile maps must be int32");
  const c10::cuda::CUDAGuard guard(a.device());
  mb::GemmProblem p{};
  p.mode = mb::GEMM_GROUPED_ROWS;
  p.num_groups = b.size(0);
  p.M = a.size(0);
  p.K = a.size(1);
  p.N = b_mn ? b.size(2) : b.size(1);
  TORCH_CHECK((b_mn ? b.size(1) : b.size(2)) == p.K, "contraction extents differ");
  TORCH_CHECK(tile_group.dim() == 2 && tile_group.size(1) == 4 && num_m_tiles.numel() >= 1, "tile maps must be [tiles, 4] and [2]");
  p.max_tiles = tile_group.size(0);
  TORCH_CHECK(c.dim() == 2 && c.size(0) == p.M && c.size(1) == p.N, "bad output shape");
  p.a = operand(a, false);
  at::Tensor b2 = b.view({b.size(0) * b.size(1), b.size(2)});
  p.b = operand(b2, b_mn);
  fill_out(p, c);
  p.ldc = c.stride(0);
  p.accumulate = accumulate;
  p.tile_group = tile_group.data_ptr<int>();
  p.num_m_tiles = num_m_tiles.data_ptr<int>();
  p.status = status_ptr(status);
  p.block_n = static_cast<int>(block_n);
  if (row_ptrs.has_value()) {  // scattered output: the epilogue stores each row at its own (possibly remote) address
    TORCH_CHECK(row_ptrs->is_cuda() && row_ptrs->scalar_type() == at::kLong && row_ptrs->numel() >= p.M, "row_ptrs must be int64 [M]");
    p.row_ptrs = reinterpret_cast<const unsigned long long*>(row_ptrs->data_ptr<int64_t>());
    if (sig_ctrl.has_value()) {
      TORCH_CHECK(sig_ctrl->scalar_type() == at::kLong && sig_ctrl->numel() >= 6 && sig_flags.size() <= 8, "bad signal arguments");
      p.sig_ctrl = reinterpret_cast<unsigned long long*>(sig_ctrl->data_ptr<int64_t>());
      for (size_t i = 0; i < sig_flags.size(); ++i) p.sig_flags[i] = reinterpret_cast<unsigned long long*>(sig_flags[i]);
      p.sig_nranks = static_cast<int>(sig_flags.size());
      p.sig_me = static_cast<int>(sig_me);
    }
  }
  TORCH_CHECK(mb::gemm_bf16_launch(p, cur_stream()) == 0, "grouped_gemm_rows: ", mb::gemm_last_error());
}

// c[g] (+)= a[rows of g]^T . b[rows of g];  a: [R, M], b: [R, N], c: [G, M, N].
void grouped_gemm_contr(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, const at::Tensor& group_offsets,
                        bool accumulate, int64_t block_n, const c10::optional<at::Tensor>& status) {
  check_bf16_2d(a, "a");
  check_bf16_2d(b, "b");
  TORCH_CHECK(a.size(0) == b.size(0), "a and b must have the same number of rows");
  TORCH_CHECK(c.dim() == 3 && c.is_contiguous(), "c must be a contiguous [G, M, N] tensor");
  TORCH_CHECK(group_offsets.scalar_type() == at::kInt && group_offsets.numel() == c.size(0) + 1, "group_offsets must be int32 [G+1]");
  const c10::cuda::CUDAGuard guard(a.device());
  mb::GemmProblem p{};
  p.mode = mb::GEMM_GROUPED_CONTR;
  p.num_groups = c.size(0);
  p.M = a.size(1);
  p.N = b.size(1);
  p.K = 0;
  TORCH_CHECK(c.size(1) == p.M && c.size(2) == p.N, "bad output shape");
  p.a = operand(a, true);
  p.b = operand(b, true);
  fill_out(p, c);
  p.ldc = c.stride(1);
  p.c_group_stride = c.stride(0);
  p.accumulate = accumulate;
  p.group_offsets = group_offsets.data_ptr<int>();
  p.status = status_ptr(status);
  p.block_n = static_cast<int>(block_n);
  TORCH_CHECK(mb::gemm_bf16_launch(p, cur_stream()) == 0, "grouped_gemm_contr: ", mb::gemm_last_error());
}

}  // namespace

void register_elementwise(pybind11::module_& m);  // ops_bindings.cpp
void register_vmm(pybind11::module_& m);          // vmm_allocator.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.def("gemm", &gemm, "bf16 tcgen05 GEMM: c (+)= a . b^T with selectable operand majors", py::arg("a"), py::arg("b"),
        py::arg("c"), py::arg("a_mn"), py::arg("b_mn"), py::arg("accumulate"), py::arg("block_n"), py::arg("status"),
        py::arg("dest") = std::vector<int64_t>(), py::arg("sig_ctrl") = py::none(),
        py::arg("sig_flags") = std::vector<int64_t>(), py::arg("sig_me") = 0);
  m.def("grouped_gemm_rows", &grouped_gemm_rows, "MoE grouped GEMM over 128-row tiles tagged with a group id", py::arg("a"),
        py::arg("b"), py::arg("c"), py::arg("tile_group"), py::arg("num_m_tiles"), py::arg("b_mn"), py::arg("accumulate"),
        py::arg("block_n"), py::arg("status"), py::arg("row_ptrs") = py::none(), py::arg("sig_ctrl") = py::none(),
        py::arg("sig_flags") = std::vector<int64_t>(), py::arg("sig_me") = 0);
  m.def("grouped_gemm_contr", &grouped_gemm_contr, "MoE weight-gradient GEMM (contraction over each group's rows)");
  register_elementwise(m);
  register_vmm(m);
}
