// Bindings of the low-latency expert-parallel decode exchange (ep_decode.cu).
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "launchers.h"

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

mb::EpLLPeers ll_peers(const std::vector<int64_t>& bases) {
  TORCH_CHECK(!bases.empty() && bases.size() <= static_cast<size_t>(mb::kMaxPeers), "1 to ", mb::kMaxPeers, " expert-parallel ranks");
  mb::EpLLPeers p{};
  for (size_t i = 0; i < bases.size(); ++i) p.base[i] = reinterpret_cast<char*>(bases[i]);
  return p;
}

// layout = [R, Bm, H, K, off_xg, off_ig, off_wg, off_yb, off_flag_a, off_flag_b]
mb::EpLLLayout ll_layout(const std::vector<int64_t>& v) {
  TORCH_CHECK(v.size() == 10, "layout has ten entries");
  mb::EpLLLayout L{};
  L.R = v[0]; L.Bm = v[1]; L.H = v[2]; L.K = v[3];
  L.off_xg = v[4]; L.off_ig = v[5]; L.off_wg = v[6]; L.off_yb = v[7]; L.off_flag_a = v[8]; L.off_flag_b = v[9];
  return L;
}

unsigned long long* ctrl_ptr(at::Tensor& ctrl) {
  TORCH_CHECK(ctrl.is_cuda() && ctrl.scalar_type() == at::kLong && ctrl.numel() >= 8 && ctrl.is_contiguous(), "ctrl: 8 int64 on the device");
  return reinterpret_cast<unsigned long long*>(ctrl.data_ptr<int64_t>());
}

// x [T, H] bf16 (the pre-norm hidden rows when ln_w is given, else already normalised), logits [T, E] fp32.
void ep_ll_send(const at::Tensor& x, const c10::optional<at::Tensor>& ln_w, double eps, const at::Tensor& logits,
                const c10::optional<at::Tensor>& active, const std::vector<int64_t>& bases, const std::vector<int64_t>& layout,
                int64_t me, bool renorm, at::Tensor& ids_out, at::Tensor& w_out, at::Tensor& ctrl) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2, "x: contiguous bf16 [T, H]");
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.is_contiguous() && logits.size(0) == x.size(0), "logits: fp32 [T, E]");
  const mb::EpLLLayout L = ll_layout(layout);
  TORCH_CHECK(x.size(1) == L.H && static_cast<int64_t>(bases.size()) == L.R, "layout does not match the inputs");
  const int T = x.size(0), E = logits.size(1);
  TORCH_CHECK(ids_out.scalar_type() == at::kInt && ids_out.is_contiguous() && ids_out.numel() == static_cast<int64_t>(T) * L.K, "ids_out: int32 [T, K]");
  TORCH_CHECK(w_out.scalar_type() == at::kFloat && w_out.is_contiguous() && w_out.numel() == static_cast<int64_t>(T) * L.K, "w_out: fp32 [T, K]");
  const int* act = nullptr;
  if (active.has_value() && active->defined()) {
    TORCH_CHECK(active->scalar_type() == at::kInt && active->is_contiguous() && active->numel() >= T, "active: int32 [T]");
    act = active->data_ptr<int>();
  }
  const void* lw = nullptr;
  if (ln_w.has_value() && ln_w->defined()) {
    TORCH_CHECK(ln_w->scalar_type() == at::kBFloat16 && ln_w->is_contiguous() && ln_w->numel() == L.H, "ln_w: bf16 [H]");
    lw = ln_w->data_ptr();
  }
  const c10::cuda::CUDAGuard guard(x.device());
  const int rc = mb::ep_ll_send(x.data_ptr(), lw, static_cast<float>(eps), logits.data_ptr<float>(), act, ll_peers(bases), L, me, T, E,
                                renorm, ids_out.data_ptr<int>(), w_out.data_ptr<float>(), ctrl_ptr(ctrl), cur_stream());
  TORCH_CHECK(rc == 0, "ep_ll_send: unsupported sizes (T <= Bm, K <= 16, E <= 256 and divisible by the ranks, H % 8 == 0, H <= 8192)");
}

// Returns [src_rows [R], counts [el], offsets [el+1], dest_row [R*Bm*K], row_src [max_rows], tiles [max_tiles, 4], totals [2]].
// `rows` bounds the rows any source sends in this step (sizes row_src: max_rows = R * rows * K).
std::vector<at::Tensor> ep_ll_plan(int64_t local_base, const std::vector<int64_t>& layout, int64_t me, int64_t E, int64_t rows,
                                   int64_t align, at::Tensor& ctrl, int64_t wait_ns, at::Tensor& status) {
  const mb::EpLLLayout L = ll_layout(layout);
  TORCH_CHECK(E % L.R == 0 && rows >= 1 && rows <= L.Bm && align >= 1, "bad plan sizes");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt, "status: int32 on the device");
  const c10::cuda::CUDAGuard guard(ctrl.device());
  const int el = E / L.R;
  const int64_t max_rows = static_cast<int64_t>(L.R) * rows * L.K + static_cast<int64_t>(el) * (align - 1);
  const int64_t max_tiles = (max_rows + 127) / 128 + el;
  auto o = ctrl.options().dtype(at::kInt);
  at::Tensor src_rows = at::empty({L.R}, o), counts = at::empty({el}, o), offsets = at::empty({el + 1}, o);
  at::Tensor dest = at::empty({static_cast<int64_t>(L.R) * L.Bm * L.K}, o), row_src = at::empty({max_rows}, o);
  at::Tensor tiles = at::empty({max_tiles, 4}, o), totals = at::empty({2}, o);
  const int rc = mb::ep_ll_plan(reinterpret_cast<char*>(local_base), L, me, E, max_rows, max_tiles, align, src_rows.data_ptr<int>(),
                                counts.data_ptr<int>(), offsets.data_ptr<int>(), dest.data_ptr<int>(), row_src.data_ptr<int>(),
                                tiles.data_ptr<int>(), totals.data_ptr<int>(), ctrl_ptr(ctrl), static_cast<unsigned long long>(wait_ns),
                                status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "ep_ll_plan: launch set-up failed (", rc, ")");
  return {src_rows, counts, offsets, dest, row_src, tiles, totals};
}

void ep_ll_return(const at::Tensor& yp, const at::Tensor& dest_row, const at::Tensor& src_rows, const std::vector<int64_t>& bases,
                  const std::vector<int64_t>& layout, int64_t me, int64_t rows, at::Tensor& ctrl) {
  TORCH_CHECK(yp.is_cuda() && yp.scalar_type() == at::kBFloat16 && yp.is_contiguous() && yp.dim() == 2, "yp: contiguous bf16 [rows, H]");
  const mb::EpLLLayout L = ll_layout(layout);
  TORCH_CHECK(yp.size(1) == L.H && dest_row.numel() == static_cast<int64_t>(L.R) * L.Bm * L.K, "layout does not match the inputs");
  const c10::cuda::CUDAGuard guard(yp.device());
  mb::ep_ll_return(yp.data_ptr(), dest_row.data_ptr<int>(), src_rows.data_ptr<int>(), ll_peers(bases), L, me, rows, ctrl_ptr(ctrl),
                   cur_stream());
}

at::Tensor ep_ll_combine(int64_t local_base, const std::vector<int64_t>& layout, const at::Tensor& ids,
                         const c10::optional<at::Tensor>& active, const at::Tensor& residual, int64_t E, at::Tensor& ctrl,
                         int64_t wait_ns, at::Tensor& status) {
  const mb::EpLLLayout L = ll_layout(layout);
  TORCH_CHECK(residual.is_cuda() && residual.scalar_type() == at::kBFloat16 && residual.is_contiguous() && residual.size(1) == L.H,
              "residual: contiguous bf16 [T, H]");
  const int T = residual.size(0);
  TORCH_CHECK(ids.scalar_type() == at::kInt && ids.is_contiguous() && ids.numel() == static_cast<int64_t>(T) * L.K && T <= L.Bm, "ids: int32 [T, K]");
  const int* act = nullptr;
  if (active.has_value() && active->defined()) act = active->data_ptr<int>();
  const c10::cuda::CUDAGuard guard(residual.device());
  at::Tensor out = at::empty_like(residual);
  mb::ep_ll_combine(reinterpret_cast<const char*>(local_base), L, ids.data_ptr<int>(), act, residual.data_ptr(), out.data_ptr(), T, E,
                    ctrl_ptr(ctrl), static_cast<unsigned long long>(wait_ns), status.data_ptr<int>(), cur_stream());
  return out;
}

}  // namespace

void register_ep_ll(pybind11::module_& m) {
  m.def("ep_ll_send", &ep_ll_send);
  m.def("ep_ll_plan", &ep_ll_plan);
  m.def("ep_ll_return", &ep_ll_return);
  m.def("ep_ll_combine", &ep_ll_combine);
}
