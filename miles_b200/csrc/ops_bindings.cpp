// Bindings of the non-GEMM kernels (normalisation, RoPE, SwiGLU, Adam, MoE routing, logprob, ...).
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "launchers.h"

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

#define CHECK_BF16(t) TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kBFloat16 && (t).is_contiguous(), #t " must be a contiguous bf16 CUDA tensor")
#define CHECK_F32(t) TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kFloat && (t).is_contiguous(), #t " must be a contiguous fp32 CUDA tensor")
#define CHECK_I32(t) TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kInt && (t).is_contiguous(), #t " must be a contiguous int32 CUDA tensor")

template <typename T>
T* opt_ptr(const c10::optional<at::Tensor>& t) {
  return t.has_value() ? static_cast<T*>(t->data_ptr()) : nullptr;
}

// y, rstd (and res_out when a residual is given)
std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& res, const at::Tensor& w, double eps) {
  CHECK_BF16(x); CHECK_BF16(w);
  const c10::cuda::CUDAGuard guard(x.device());
  const int H = x.size(-1);
  const int T = x.numel() / H;
  TORCH_CHECK(H % 8 == 0 && w.numel() == H, "hidden size must be a multiple of 8 and match the weight");
  at::Tensor y = at::empty_like(x);
  at::Tensor rstd = at::empty({T}, x.options().dtype(at::kFloat));
  at::Tensor res_out;
  if (res.has_value()) { CHECK_BF16(*res); res_out = at::empty_like(x); }
  mb::rmsnorm_fwd(x.data_ptr(), opt_ptr<void>(res), w.data_ptr(), y.data_ptr(), res.has_value() ? res_out.data_ptr() : nullptr,
                  rstd.data_ptr<float>(), T, H, static_cast<float>(eps), cur_stream());
  if (res.has_value()) return {y, rstd, res_out};
  return {y, rstd};
}

// returns dx; dw (fp32 [H]) is written or accumulated in place
at::Tensor rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd,
                       const c10::optional<at::Tensor>& dres, at::Tensor& dw, bool accumulate_dw) {
  CHECK_BF16(dy); CHECK_BF16(x); CHECK_BF16(w); CHECK_F32(rstd); CHECK_F32(dw);
  const c10::cuda::CUDAGuard guard(x.device());
  const int H = x.size(-1);
  const int T = x.numel() / H;
  at::Tensor dx = at::empty_like(x);
  at::Tensor part = at::empty({mb::rmsnorm_bwd_num_partials(T), H}, x.options().dtype(at::kFloat));
  mb::rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), opt_ptr<void>(dres), dx.data_ptr(),
                  part.data_ptr<float>(), dw.data_ptr<float>(), accumulate_dw, T, H, cur_stream());
  return dx;
}

// qkv [T, (Hq+2Hk)*128] -> q [T,Hq,128], k [T,Hk,128], q_rstd, k_rstd. Optional paged-cache scatter.
std::vector<at::Tensor> qk_norm_rope_fwd(const at::Tensor& qkv, const c10::optional<at::Tensor>& qw,
                                         const c10::optional<at::Tensor>& kw, const at::Tensor& pos, int64_t Hq, int64_t Hk,
                                         double theta, double eps, const c10::optional<at::Tensor>& k_cache,
                                         const c10::optional<at::Tensor>& v_cache, const c10::optional<at::Tensor>& slot_mapping,
                                         bool write_k_out, const c10::optional<at::Tensor>& inv_freq, int64_t rotary_dim) {
  CHECK_BF16(qkv); CHECK_I32(pos);
  TORCH_CHECK(rotary_dim == 128 || rotary_dim == 64, "rotary_dim must be 128 (whole head) or 64 (half of it)");
  if (inv_freq.has_value())
    TORCH_CHECK(inv_freq->is_cuda() && inv_freq->scalar_type() == at::kFloat && inv_freq->numel() == rotary_dim / 2 &&
                    inv_freq->is_contiguous(),
                "inv_freq must be rotary_dim / 2 contiguous fp32 values on the device");
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int T = qkv.size(0);
  TORCH_CHECK(qkv.size(1) == (Hq + 2 * Hk) * 128, "qkv must be [T, (Hq+2Hk)*128]");
  const bool use_norm = qw.has_value();
  at::Tensor q = at::empty({T, Hq, 128}, qkv.options());
  at::Tensor k = write_k_out ? at::empty({T, Hk, 128}, qkv.options()) : at::Tensor();
  at::Tensor qr = use_norm ? at::empty({T, Hq}, qkv.options().dtype(at::kFloat)) : at::Tensor();
  at::Tensor kr = use_norm ? at::empty({T, Hk}, qkv.options().dtype(at::kFloat)) : at::Tensor();
  mb::qk_norm_rope_fwd(qkv.data_ptr(), opt_ptr<void>(qw), opt_ptr<void>(kw), pos.data_ptr<int>(), q.data_ptr(),
                       write_k_out ? k.data_ptr() : nullptr, use_norm ? qr.data_ptr<float>() : nullptr,
                       use_norm ? kr.data_ptr<float>() : nullptr, opt_ptr<void>(k_cache), opt_ptr<void>(v_cache),
                       opt_ptr<int>(slot_mapping), T, Hq, Hk, static_cast<float>(theta), static_cast<float>(eps), use_norm,
                       cur_stream(), opt_ptr<float>(inv_freq), static_cast<int>(rotary_dim));
  return {q, k, qr, kr};
}

std::vector<at::Tensor> qk_norm_rope_fwd_plain(const at::Tensor& qkv, const c10::optional<at::Tensor>& qw,
                                               const c10::optional<at::Tensor>& kw, const at::Tensor& pos, int64_t Hq, int64_t Hk,
                                               double theta, double eps, const c10::optional<at::Tensor>& k_cache,
                                               const c10::optional<at::Tensor>& v_cache,
                                               const c10::optional<at::Tensor>& slot_mapping, bool write_k_out) {
  return qk_norm_rope_fwd(qkv, qw, kw, pos, Hq, Hk, theta, eps, k_cache, v_cache, slot_mapping, write_k_out, c10::nullopt, 128);
}

at::Tensor qk_norm_rope_bwd(const at::Tensor& dq, const at::Tensor& dk, const at::Tensor& dv, const at::Tensor& qkv,
                            const c10::optional<at::Tensor>& qw, const c10::optional<at::Tensor>& kw, const at::Tensor& pos,
                            const c10::optional<at::Tensor>& q_rstd, const c10::optional<at::Tensor>& k_rstd,
                            const c10::optional<at::Tensor>& dqw, const c10::optional<at::Tensor>& dkw, int64_t Hq, int64_t Hk,
                            double theta, const c10::optional<at::Tensor>& inv_freq, int64_t rotary_dim) {
  CHECK_BF16(dq); CHECK_BF16(dk); CHECK_BF16(dv); CHECK_BF16(qkv);
  TORCH_CHECK(rotary_dim == 128 || rotary_dim == 64, "rotary_dim must be 128 (whole head) or 64 (half of it)");
  if (inv_freq.has_value())
    TORCH_CHECK(inv_freq->is_cuda() && inv_freq->scalar_type() == at::kFloat && inv_freq->numel() == rotary_dim / 2 &&
                    inv_freq->is_contiguous(),
                "inv_freq must be rotary_dim / 2 contiguous fp32 values on the device");
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int T = qkv.size(0);
  at::Tensor dqkv = at::empty_like(qkv);
  mb::qk_norm_rope_bwd(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), qkv.data_ptr(), opt_ptr<void>(qw), opt_ptr<void>(kw),
                       pos.data_ptr<int>(), opt_ptr<float>(q_rstd), opt_ptr<float>(k_rstd), dqkv.data_ptr(),
                       opt_ptr<float>(dqw), opt_ptr<float>(dkw), T, Hq, Hk, static_cast<float>(theta), qw.has_value(),
                       cur_stream(), opt_ptr<float>(inv_freq), static_cast<int>(rotary_dim));
  return dqkv;
}

at::Tensor qk_norm_rope_bwd_plain(const at::Tensor& dq, const at::Tensor& dk, const at::Tensor& dv, const at::Tensor& qkv,
                                  const c10::optional<at::Tensor>& qw, const c10::optional<at::Tensor>& kw, const at::Tensor& pos,
                                  const c10::optional<at::Tensor>& q_rstd, const c10::optional<at::Tensor>& k_rstd,
                                  const c10::optional<at::Tensor>& dqw, const c10::optional<at::Tensor>& dkw, int64_t Hq,
                                  int64_t Hk, double theta) {
  return qk_norm_rope_bwd(dq, dk, dv, qkv, qw, kw, pos, q_rstd, k_rstd, dqw, dkw, Hq, Hk, theta, c10::nullopt, 128);
}

at::Tensor swiglu_fwd(const at::Tensor& in) {
  CHECK_BF16(in);
  const c10::cuda::CUDAGuard guard(in.device());
  const int I = in.size(-1) / 2;
  TORCH_CHECK(I % 8 == 0, "intermediate size must be a multiple of 8");
  const long long T = in.numel() / (2 * I);
  auto sizes = in.sizes().vec();
  sizes.back() = I;
  at::Tensor out = at::empty(sizes, in.options());
  mb::swiglu_fwd(in.data_ptr(), out.data_ptr(), T, I, cur_stream());
  return out;
}

at::Tensor swiglu_bwd(const at::Tensor& dout, const at::Tensor& in) {
  CHECK_BF16(dout); CHECK_BF16(in);
  const c10::cuda::CUDAGuard guard(in.device());
  const int I = in.size(-1) / 2;
  const long long T = in.numel() / (2 * I);
  at::Tensor din = at::empty_like(in);
  mb::swiglu_bwd(dout.data_ptr(), in.data_ptr(), din.data_ptr(), T, I, cur_stream());
  return din;
}

void adam_step(at::Tensor& p, const c10::optional<at::Tensor>& master, const at::Tensor& g, at::Tensor& m, at::Tensor& v,
               double lr, double b1, double b2, double eps, double wd, int64_t step,
               const c10::optional<at::Tensor>& grad_scale, const c10::optional<at::Tensor>& skip_flag,
               const c10::optional<at::Tensor>& lo) {
  CHECK_BF16(p);
  TORCH_CHECK(g.is_cuda() && g.is_contiguous() && g.numel() == p.numel(), "bad gradient");
  TORCH_CHECK(m.scalar_type() == v.scalar_type() && m.numel() == p.numel() && v.numel() == p.numel(), "bad moments");
  TORCH_CHECK(m.is_cuda() && v.is_cuda() && m.is_contiguous() && v.is_contiguous(), "moments must be contiguous device tensors");
  void* lo_ptr = nullptr;
  if (lo.has_value() && lo->defined()) {
    TORCH_CHECK(lo->is_cuda() && lo->is_contiguous() && lo->scalar_type() == at::kShort && lo->numel() == p.numel(),
                "lo must be an int16 device tensor of the parameter's size");
    TORCH_CHECK(!(master.has_value() && master->defined()), "pass either master or lo");
    lo_ptr = lo->data_ptr();
  }
  auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  TORCH_CHECK(aligned(p.data_ptr()) && aligned(g.data_ptr()) && aligned(m.data_ptr()) && aligned(v.data_ptr()) &&
              aligned(lo_ptr) && aligned(opt_ptr<float>(master)), "adam_step needs 16-byte aligned buffers");
  const c10::cuda::CUDAGuard guard(p.device());
  const float bc1 = 1.f - std::pow(static_cast<float>(b1), static_cast<float>(step));
  const float bc2 = 1.f - std::pow(static_cast<float>(b2), static_cast<float>(step));
  mb::adam_step(p.data_ptr(), opt_ptr<float>(master), lo_ptr, g.data_ptr(), g.scalar_type() == at::kFloat, m.data_ptr(),
                v.data_ptr(), m.scalar_type() == at::kBFloat16, p.numel(), lr, b1, b2, eps, wd, bc1, bc2,
                opt_ptr<float>(grad_scale), opt_ptr<float>(skip_flag), cur_stream());
}

at::Tensor split_master_join(const at::Tensor& p, const at::Tensor& lo) {
  CHECK_BF16(p);
  TORCH_CHECK(lo.is_cuda() && lo.is_contiguous() && lo.scalar_type() == at::kShort && lo.numel() == p.numel(), "bad lo");
  const c10::cuda::CUDAGuard guard(p.device());
  at::Tensor out = at::empty(p.sizes(), p.options().dtype(at::kFloat));
  mb::split_master_join(p.data_ptr(), lo.data_ptr(), out.data_ptr<float>(), p.numel(), cur_stream());
  return out;
}

void split_master_cut(const at::Tensor& master, at::Tensor& p, at::Tensor& lo) {
  CHECK_BF16(p); CHECK_F32(master);
  TORCH_CHECK(lo.is_cuda() && lo.is_contiguous() && lo.scalar_type() == at::kShort && lo.numel() == p.numel() &&
              master.numel() == p.numel(), "bad lo / master");
  const c10::cuda::CUDAGuard guard(p.device());
  mb::split_master_cut(master.data_ptr<float>(), p.data_ptr(), lo.data_ptr(), p.numel(), cur_stream());
}

void init_normal(at::Tensor& out, int64_t key, double std, int64_t first) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous(), "init_normal needs a contiguous CUDA tensor");
  TORCH_CHECK(out.scalar_type() == at::kFloat || out.scalar_type() == at::kBFloat16, "init_normal fills fp32 or bf16");
  const c10::cuda::CUDAGuard guard(out.device());
  mb::init_normal(out.data_ptr(), out.scalar_type() == at::kFloat, out.numel(), static_cast<unsigned long long>(key), first,
                  static_cast<float>(std), cur_stream());
}

void sumsq(const at::Tensor& g, at::Tensor& out) {
  TORCH_CHECK(g.is_cuda() && g.is_contiguous(), "bad gradient");
  CHECK_F32(out);
  const c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK((reinterpret_cast<uintptr_t>(g.data_ptr()) & 15) == 0, "sumsq needs a 16-byte aligned buffer");
  TORCH_CHECK(g.scalar_type() == at::kFloat || g.scalar_type() == at::kBFloat16, "sumsq takes fp32 or bf16");
  at::Tensor partial = at::empty({mb::sumsq_num_partials(g.numel())}, out.options());
  mb::sumsq(g.data_ptr(), g.scalar_type() == at::kFloat, g.numel(), partial.data_ptr<float>(), out.data_ptr<float>(), cur_stream());
}

// ---------------------------------------------------------------- MoE
std::vector<at::Tensor> moe_router_topk(const at::Tensor& logits, const c10::optional<at::Tensor>& replay_ids, int64_t K,
                                        bool renorm, bool want_probs) {
  CHECK_F32(logits);
  const c10::cuda::CUDAGuard guard(logits.device());
  const int T = logits.size(0), E = logits.size(1);
  TORCH_CHECK(E <= 256 && K <= 16, "router supports at most 256 experts and top-16");
  at::Tensor ids = at::empty({T, K}, logits.options().dtype(at::kInt));
  at::Tensor w = at::empty({T, K}, logits.options());
  at::Tensor probs = want_probs ? at::empty_like(logits) : at::Tensor();
  if (replay_ids.has_value()) CHECK_I32(*replay_ids);
  mb::moe_router_topk(logits.data_ptr<float>(), opt_ptr<int>(replay_ids), ids.data_ptr<int>(), w.data_ptr<float>(),
                      want_probs ? probs.data_ptr<float>() : nullptr, T, E, K, renorm, cur_stream());
  return {ids, w, probs};
}

at::Tensor moe_router_bwd(const at::Tensor& probs, const at::Tensor& ids, const at::Tensor& w, const at::Tensor& dw, bool renorm) {
  CHECK_F32(probs); CHECK_I32(ids); CHECK_F32(w); CHECK_F32(dw);
  const c10::cuda::CUDAGuard guard(probs.device());
  at::Tensor dl = at::empty_like(probs);
  mb::moe_router_bwd(probs.data_ptr<float>(), ids.data_ptr<int>(), w.data_ptr<float>(), dw.data_ptr<float>(),
                     dl.data_ptr<float>(), probs.size(0), probs.size(1), ids.size(1), renorm, cur_stream());
  return dl;
}

// returns counts[E], offsets[E+1], dest_row[T*K], row_src[max_rows], tile_group[max_tiles,4], totals[2]
std::vector<at::Tensor> moe_build_permutation(const at::Tensor& ids, int64_t E, int64_t max_rows, int64_t align) {
  CHECK_I32(ids);
  const c10::cuda::CUDAGuard guard(ids.device());
  const int T = ids.size(0), K = ids.size(1);
  TORCH_CHECK(align >= 1 && max_rows >= 1, "bad permutation sizes");
  const int64_t max_tiles = (max_rows + 127) / 128 + E;
  auto o = ids.options();
  at::Tensor counts = at::empty({E}, o), offsets = at::empty({E + 1}, o), dest = at::empty({T * K}, o);
  at::Tensor src = at::empty({max_rows}, o), tg = at::empty({max_tiles, 4}, o), nt = at::empty({2}, o);
  mb::moe_build_permutation(ids.data_ptr<int>(), T, K, E, max_rows, max_tiles, align, counts.data_ptr<int>(),
                            offsets.data_ptr<int>(), dest.data_ptr<int>(), src.data_ptr<int>(), tg.data_ptr<int>(),
                            nt.data_ptr<int>(), cur_stream());
  return {counts, offsets, dest, src, tg, nt};
}

at::Tensor moe_permute(const at::Tensor& x, const at::Tensor& row_src, const at::Tensor& num_m_tiles, int64_t K) {
  CHECK_BF16(x); CHECK_I32(row_src);
  const c10::cuda::CUDAGuard guard(x.device());
  const int H = x.size(1);
  at::Tensor xp = at::empty({row_src.numel(), H}, x.options());
  mb::moe_permute(x.data_ptr(), row_src.data_ptr<int>(), num_m_tiles.data_ptr<int>(), xp.data_ptr(), row_src.numel(), H, K,
                  cur_stream());
  return xp;
}

at::Tensor moe_combine(const at::Tensor& y_perm, const at::Tensor& dest_row, const c10::optional<at::Tensor>& w, int64_t T, int64_t K,
                       const c10::optional<at::Tensor>& residual) {
  CHECK_BF16(y_perm); CHECK_I32(dest_row);
  const c10::cuda::CUDAGuard guard(y_perm.device());
  const int H = y_perm.size(1);
  at::Tensor out = at::empty({T, H}, y_perm.options());
  mb::moe_combine(y_perm.data_ptr(), dest_row.data_ptr<int>(), opt_ptr<float>(w), opt_ptr<void>(residual), out.data_ptr(), T, K, H,
                  cur_stream());
  return out;
}

std::vector<at::Tensor> moe_combine_bwd(const at::Tensor& dout, const at::Tensor& y_perm, const at::Tensor& row_src,
                                        const at::Tensor& num_m_tiles, const at::Tensor& w) {
  CHECK_BF16(dout); CHECK_BF16(y_perm); CHECK_F32(w);
  const c10::cuda::CUDAGuard guard(dout.device());
  const int H = dout.size(1), K = w.size(1);
  at::Tensor dy = at::empty_like(y_perm);
  at::Tensor dw = at::zeros_like(w);
  mb::moe_combine_bwd(dout.data_ptr(), y_perm.data_ptr(), row_src.data_ptr<int>(), num_m_tiles.data_ptr<int>(),
                      w.data_ptr<float>(), dy.data_ptr(), dw.data_ptr<float>(), row_src.numel(), K, H, cur_stream());
  return {dy, dw};
}

// ---------------------------------------------------------------- logprob / entropy
std::vector<at::Tensor> logprob_entropy_fwd(const at::Tensor& logits, const at::Tensor& targets, double inv_temp) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "logits must be 2-D with contiguous rows");
  CHECK_I32(targets);
  const c10::cuda::CUDAGuard guard(logits.device());
  const bool fp32 = logits.scalar_type() == at::kFloat;
  TORCH_CHECK(fp32 || logits.scalar_type() == at::kBFloat16, "logits must be bf16 or fp32");
  const int T = logits.size(0), V = logits.size(1);
  auto o = logits.options().dtype(at::kFloat);
  at::Tensor lp = at::empty({T}, o), ent = at::empty({T}, o), lse = at::empty({T}, o), px = at::empty({T}, o);
  mb::logprob_entropy_fwd(logits.data_ptr(), fp32, targets.data_ptr<int>(), lp.data_ptr<float>(), ent.data_ptr<float>(),
                          lse.data_ptr<float>(), px.data_ptr<float>(), T, V, logits.stride(0), inv_temp, cur_stream());
  return {lp, ent, lse, px};
}

// Returns dlogits as bf16 [T, V]; for bf16 logits the result overwrites the input buffer.
at::Tensor logprob_entropy_bwd(at::Tensor& logits, const at::Tensor& targets, const at::Tensor& lse, const at::Tensor& px,
                               const c10::optional<at::Tensor>& dlp, const c10::optional<at::Tensor>& dent, double inv_temp) {
  const c10::cuda::CUDAGuard guard(logits.device());
  const bool fp32 = logits.scalar_type() == at::kFloat;
  at::Tensor out = fp32 ? at::empty(logits.sizes(), logits.options().dtype(at::kBFloat16)) : logits;
  mb::logprob_entropy_bwd(logits.data_ptr(), fp32, targets.data_ptr<int>(), lse.data_ptr<float>(), px.data_ptr<float>(),
                          opt_ptr<float>(dlp), opt_ptr<float>(dent), out.data_ptr(), logits.size(0), logits.size(1),
                          logits.stride(0), out.stride(0), inv_temp, cur_stream());
  return out;
}

}  // namespace

void register_more(pybind11::module_& m);  // ops_bindings2.cpp

void register_elementwise(pybind11::module_& m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("qk_norm_rope_fwd", &qk_norm_rope_fwd_plain);
  m.def("qk_norm_rope_bwd", &qk_norm_rope_bwd_plain);
  m.def("qk_norm_rope_fwd_scaled", &qk_norm_rope_fwd);  // + optional inv_freq table (scaled rotary embeddings), rotary_dim
  m.def("qk_norm_rope_bwd_scaled", &qk_norm_rope_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("adam_step", &adam_step, pybind11::arg("p"), pybind11::arg("master"), pybind11::arg("g"), pybind11::arg("m"), pybind11::arg("v"), pybind11::arg("lr"),
        pybind11::arg("b1"), pybind11::arg("b2"), pybind11::arg("eps"), pybind11::arg("wd"), pybind11::arg("step"), pybind11::arg("grad_scale") = pybind11::none(),
        pybind11::arg("skip_flag") = pybind11::none(), pybind11::arg("lo") = pybind11::none());
  m.def("split_master_join", &split_master_join);
  m.def("split_master_cut", &split_master_cut);
  m.def("sumsq", &sumsq);
  m.def("init_normal", &init_normal, pybind11::arg("out"), pybind11::arg("key"), pybind11::arg("std"), pybind11::arg("first") = 0);
  m.def("moe_router_topk", &moe_router_topk);
  m.def("moe_router_bwd", &moe_router_bwd);
  m.def("moe_build_permutation", &moe_build_permutation);
  m.def("moe_permute", &moe_permute);
  m.def("moe_combine", &moe_combine, pybind11::arg("y_perm"), pybind11::arg("dest_row"), pybind11::arg("w"), pybind11::arg("T"),
        pybind11::arg("K"), pybind11::arg("residual") = c10::optional<at::Tensor>());
  m.def("moe_combine_bwd", &moe_combine_bwd);
  m.def("logprob_entropy_fwd", &logprob_entropy_fwd);
  m.def("logprob_entropy_bwd", &logprob_entropy_bwd);
  register_more(m);
}
