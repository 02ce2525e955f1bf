// Bindings of the rollout-engine kernels (paged attention, sampling), RL scans and quantisers.
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

// logits [B, V] (bf16/fp32) -> (token int32 [B], logprob fp32 [B]); per-row parameters are optional tensors.
void sample_rows(const at::Tensor& logits, const c10::optional<at::Tensor>& temperature,
                 const c10::optional<at::Tensor>& top_k, const c10::optional<at::Tensor>& top_p,
                 const c10::optional<at::Tensor>& seeds, const c10::optional<at::Tensor>& step, at::Tensor& out_token,
                 at::Tensor& out_logprob) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "logits must be 2-D with contiguous rows");
  const bool fp32 = logits.scalar_type() == at::kFloat;
  TORCH_CHECK(fp32 || logits.scalar_type() == at::kBFloat16, "logits must be bf16 or fp32");
  CHECK_I32(out_token); CHECK_F32(out_logprob);
  if (seeds.has_value()) TORCH_CHECK(seeds->scalar_type() == at::kLong && seeds->is_cuda(), "seeds must be int64 CUDA");
  const c10::cuda::CUDAGuard guard(logits.device());
  mb::sample_rows(logits.data_ptr(), fp32, logits.size(0), logits.size(1), logits.stride(0), opt_ptr<float>(temperature),
                  opt_ptr<int>(top_k), opt_ptr<float>(top_p),
                  reinterpret_cast<const unsigned long long*>(opt_ptr<int64_t>(seeds)), opt_ptr<int>(step),
                  out_token.data_ptr<int>(), out_logprob.data_ptr<float>(), cur_stream());
}

// q [B, Hq, 128]; caches [slots, Hk, 128]; block_table [B, max_pages]; out [B, Hq, 128]; scratch fp32.
void paged_decode_attention(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                            const at::Tensor& block_table, const at::Tensor& seq_lens, at::Tensor& out, at::Tensor& scratch,
                            int64_t page_size, int64_t num_splits, double scale, const c10::optional<at::Tensor>& status) {
  CHECK_BF16(q); CHECK_BF16(k_cache); CHECK_BF16(v_cache); CHECK_I32(block_table); CHECK_I32(seq_lens); CHECK_BF16(out); CHECK_F32(scratch);
  const int B = q.size(0), Hq = q.size(1), Hk = k_cache.size(1);
  TORCH_CHECK(q.size(2) == 128 && k_cache.size(2) == 128, "head_dim must be 128");
  const int G = Hq / Hk;
  TORCH_CHECK(Hq % Hk == 0 && (G == 1 || G == 2 || G == 4 || G == 8), "unsupported GQA group size");
  TORCH_CHECK(scratch.numel() >= static_cast<int64_t>(B) * Hq * num_splits * 130, "scratch too small");
  const c10::cuda::CUDAGuard guard(q.device());
  int* st = nullptr;
  if (status.has_value() && status->defined()) {
    CHECK_I32((*status));
    st = status->data_ptr<int>();
  }
  const int e = mb::paged_decode_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr<int>(),
                                           seq_lens.data_ptr<int>(), out.data_ptr(), scratch.data_ptr<float>(), B, Hq, Hk,
                                           page_size, block_table.size(1), num_splits, scale, cur_stream(), k_cache.size(0), st);
  TORCH_CHECK(e == 0, "paged_decode_attention launch failed: ", cudaGetErrorString(static_cast<cudaError_t>(e)));
}

// q [Tq, Hq, 128], k/v [Tkv, Hk, 128] (last dim contiguous, arbitrary row pitch); tiles int32 [n, 4].
std::vector<at::Tensor> flash_attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& tiles,
                                       double scale, const c10::optional<at::Tensor>& status) {
  CHECK_I32(tiles);
  for (const at::Tensor* t : {&q, &k, &v}) TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kBFloat16, "q/k/v must be bf16 CUDA tensors");
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && q.size(2) == 128 && k.size(2) == 128 && v.size(2) == 128,
              "q/k/v must be [rows, heads, 128]");
  TORCH_CHECK(q.stride(2) == 1 && k.stride(2) == 1 && v.stride(2) == 1 && q.stride(1) == 128 && k.stride(1) == 128 &&
                  v.stride(1) == 128, "heads must be packed along each row");
  TORCH_CHECK(tiles.is_contiguous() && tiles.dim() == 2 && tiles.size(1) == 4, "tiles must be contiguous [n, 4]");
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t Tq = q.size(0), Hq = q.size(1), Hk = k.size(1);
  at::Tensor out = at::empty({Tq, Hq, 128}, q.options());
  at::Tensor lse = at::empty({Hq, Tq}, q.options().dtype(at::kFloat));
  int* st = nullptr;
  if (status.has_value()) { CHECK_I32((*status)); st = status->data_ptr<int>(); }
  const int rc = mb::flash_attn_fwd(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                                    out.data_ptr(), lse.data_ptr<float>(), tiles.data_ptr<int>(), tiles.size(0), Tq,
                                    k.size(0), Hq, Hk, 128, scale, st, cur_stream());
  TORCH_CHECK(rc == 0, mb::flash_attn_last_error());
  return {out, lse};
}

// Backward of the causal self-attention over packed sequences. Returns {dq, dk, dv}.
std::vector<at::Tensor> flash_attn_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o,
                                       const at::Tensor& d_o, const at::Tensor& lse, const at::Tensor& blocks, double scale,
                                       const c10::optional<at::Tensor>& status) {
  CHECK_I32(blocks);
  for (const at::Tensor* t : {&q, &k, &v, &o, &d_o})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kBFloat16 && t->dim() == 3 && t->size(2) == 128 && t->stride(2) == 1 &&
                    t->stride(1) == 128, "q/k/v/o/d_o must be bf16 [rows, heads, 128] with heads packed along each row");
  TORCH_CHECK(o.is_contiguous() && d_o.is_contiguous(), "o and d_o must be contiguous");
  CHECK_F32(lse);
  const int64_t T = q.size(0), Hq = q.size(1), Hk = k.size(1);
  TORCH_CHECK(k.size(0) == T && v.size(0) == T && o.size(0) == T && d_o.size(0) == T && o.size(1) == Hq && d_o.size(1) == Hq &&
                  v.size(1) == Hk && lse.size(0) == Hq && lse.size(1) == T, "shape mismatch");
  TORCH_CHECK(blocks.is_contiguous() && blocks.dim() == 2 && blocks.size(1) == 4, "blocks must be contiguous [n, 4]");
  const c10::cuda::CUDAGuard guard(q.device());
  at::Tensor dq = at::empty({T, Hq, 128}, q.options());
  at::Tensor dk = at::empty({T, Hk, 128}, q.options()), dv = at::empty({T, Hk, 128}, q.options());
  at::Tensor scratch = at::empty({T * Hq * 128 + 2 * Hq * T}, q.options().dtype(at::kFloat));
  int* st = nullptr;
  if (status.has_value()) { CHECK_I32((*status)); st = status->data_ptr<int>(); }
  const int rc = mb::flash_attn_bwd(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), o.data_ptr(),
                                    d_o.data_ptr(), d_o.stride(0), lse.data_ptr<float>(), blocks.data_ptr<int>(), blocks.size(0),
                                    T, Hq, Hk, 128, scale, scratch.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                    st, cur_stream());
  TORCH_CHECK(rc == 0, mb::flash_attn_bwd_last_error());
  return {dq, dk, dv};
}

// ---- small-batch decode kernels (T <= 8)
void small_gemv(const at::Tensor& x, const c10::optional<at::Tensor>& norm_w, double eps, const at::Tensor& W,
                const c10::optional<at::Tensor>& residual, at::Tensor& out, const c10::optional<at::Tensor>& status) {
  CHECK_BF16(x); CHECK_BF16(W);
  const int T = x.size(0), K = x.size(1), N = W.size(0);
  TORCH_CHECK(T >= 1 && T <= 64 && W.size(1) == K && K % 32 == 0 && N % 16 == 0, "small_gemv: need 1 <= T <= 64, K % 32 == 0, N % 16 == 0");
  TORCH_CHECK(T <= 8 || !norm_w.has_value(), "small_gemv: the folded RMSNorm is available for at most 8 rows");
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.size(0) == T && out.size(1) == N, "small_gemv: bad output shape");
  const bool f32 = out.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || out.scalar_type() == at::kBFloat16, "small_gemv: output must be fp32 or bf16");
  if (norm_w.has_value()) CHECK_BF16((*norm_w));
  if (residual.has_value()) { CHECK_BF16((*residual)); TORCH_CHECK(residual->numel() == out.numel(), "small_gemv: residual shape"); }
  const c10::cuda::CUDAGuard guard(x.device());
  mb::small_gemv(x.data_ptr(), T, norm_w.has_value() ? norm_w->data_ptr() : nullptr, eps, W.data_ptr(), N, K,
                 residual.has_value() ? residual->data_ptr() : nullptr, out.data_ptr(), f32,
                 status.has_value() ? status->data_ptr<int>() : nullptr, cur_stream());
}

void router_small(const at::Tensor& logits, int64_t K, bool renorm, at::Tensor& ids, at::Tensor& w, at::Tensor& active,
                  at::Tensor& pair_count, at::Tensor& pair_list) {
  CHECK_F32(logits); CHECK_I32(ids); CHECK_F32(w); CHECK_I32(active); CHECK_I32(pair_count); CHECK_I32(pair_list);
  const int T = logits.size(0), E = logits.size(1);
  TORCH_CHECK(T >= 1 && T <= 8 && E <= 1024 && K <= 32 && K <= E, "router_small: unsupported shape");
  TORCH_CHECK(ids.numel() >= T * K && w.numel() >= T * K && active.numel() >= E + 1 && pair_count.numel() >= E && pair_list.numel() >= 8 * E,
              "router_small: output buffers too small");
  const c10::cuda::CUDAGuard guard(logits.device());
  mb::router_small(logits.data_ptr<float>(), T, E, K, renorm, ids.data_ptr<int>(), w.data_ptr<float>(), active.data_ptr<int>(),
                   pair_count.data_ptr<int>(), pair_list.data_ptr<int>(), cur_stream());
}

void moe_small_up(const at::Tensor& x, const at::Tensor& norm_w, double eps, const at::Tensor& W1, const at::Tensor& active,
                  const at::Tensor& pair_count, const at::Tensor& pair_list, int64_t max_active, int64_t K, at::Tensor& act,
                  const c10::optional<at::Tensor>& status) {
  CHECK_BF16(x); CHECK_BF16(norm_w); CHECK_BF16(W1); CHECK_BF16(act);
  const int H = x.size(1), I = W1.size(1) / 2;
  TORCH_CHECK(W1.dim() == 3 && W1.size(2) == H && H % 32 == 0 && I % 8 == 0 && act.size(1) == 2 * I, "moe_small_up: unsupported shape");
  TORCH_CHECK((2 * I) % 16 == 0, "moe_small_up: 2I must be a multiple of 16");
  const c10::cuda::CUDAGuard guard(x.device());
  mb::moe_small_up(x.data_ptr(), norm_w.data_ptr(), eps, W1.data_ptr(), active.data_ptr<int>(), pair_count.data_ptr<int>(),
                   pair_list.data_ptr<int>(), max_active, H, I, K, act.data_ptr(),
                   status.has_value() ? status->data_ptr<int>() : nullptr, cur_stream());
}

void moe_small_down(const at::Tensor& act, const at::Tensor& W2, const at::Tensor& active, const at::Tensor& pair_count,
                    const at::Tensor& pair_list, int64_t max_active, at::Tensor& y, const c10::optional<at::Tensor>& status) {
  CHECK_BF16(act); CHECK_BF16(W2); CHECK_BF16(y);
  const int I = act.size(1) / 2, H = W2.size(1);
  TORCH_CHECK(W2.dim() == 3 && W2.size(2) == I && H % 16 == 0 && I % 32 == 0 && y.size(1) == H, "moe_small_down: unsupported shape");
  const c10::cuda::CUDAGuard guard(act.device());
  mb::moe_small_down(act.data_ptr(), W2.data_ptr(), active.data_ptr<int>(), pair_count.data_ptr<int>(), pair_list.data_ptr<int>(),
                     max_active, H, I, y.data_ptr(), status.has_value() ? status->data_ptr<int>() : nullptr, cur_stream());
}

std::vector<at::Tensor> gae(const at::Tensor& rewards, const at::Tensor& values, const at::Tensor& cu, double gamma, double lam) {
  CHECK_F32(rewards); CHECK_F32(values); CHECK_I32(cu);
  const c10::cuda::CUDAGuard guard(rewards.device());
  at::Tensor adv = at::zeros_like(rewards), ret = at::zeros_like(rewards);
  mb::gae_reverse_scan(rewards.data_ptr<float>(), values.data_ptr<float>(), cu.data_ptr<int>(), adv.data_ptr<float>(),
                       ret.data_ptr<float>(), cu.numel() - 1, gamma, lam, cur_stream());
  return {adv, ret};
}

std::vector<at::Tensor> quant_mxfp8(const at::Tensor& x) {
  CHECK_BF16(x);
  const int64_t cols = x.size(-1), rows = x.numel() / cols;
  TORCH_CHECK(cols % 32 == 0, "last dim must be a multiple of 32 for MXFP8");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor q = at::empty(x.sizes(), x.options().dtype(at::kByte));
  auto ssz = x.sizes().vec(); ssz.back() = cols / 32;
  at::Tensor sc = at::empty(ssz, x.options().dtype(at::kByte));
  mb::quant_mxfp8(x.data_ptr(), q.data_ptr<uint8_t>(), sc.data_ptr<uint8_t>(), rows, cols, cur_stream());
  return {q, sc};
}
at::Tensor dequant_mxfp8(const at::Tensor& q, const at::Tensor& sc) {
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t cols = q.size(-1), rows = q.numel() / cols;
  at::Tensor x = at::empty(q.sizes(), q.options().dtype(at::kBFloat16));
  mb::dequant_mxfp8(q.data_ptr<uint8_t>(), sc.data_ptr<uint8_t>(), x.data_ptr(), rows, cols, cur_stream());
  return x;
}
at::Tensor absmax(const at::Tensor& x) {
  CHECK_BF16(x);
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::zeros({1}, x.options().dtype(at::kFloat));
  mb::absmax(x.data_ptr(), x.numel(), out.data_ptr<float>(), cur_stream());
  return out;
}
// returns packed uint8 [.., cols/2], e4m3 block scales as uint8 [.., cols/16]; `global_amax` fp32 [1] on device
std::vector<at::Tensor> quant_nvfp4(const at::Tensor& x, const at::Tensor& global_amax) {
  CHECK_BF16(x); CHECK_F32(global_amax);
  const int64_t cols = x.size(-1), rows = x.numel() / cols;
  TORCH_CHECK(cols % 16 == 0, "last dim must be a multiple of 16 for NVFP4");
  const c10::cuda::CUDAGuard guard(x.device());
  auto qsz = x.sizes().vec(); qsz.back() = cols / 2;
  auto ssz = x.sizes().vec(); ssz.back() = cols / 16;
  at::Tensor q = at::empty(qsz, x.options().dtype(at::kByte)), sc = at::empty(ssz, x.options().dtype(at::kByte));
  mb::quant_nvfp4(x.data_ptr(), q.data_ptr<uint8_t>(), sc.data_ptr<uint8_t>(), global_amax.data_ptr<float>(), rows, cols, cur_stream());
  return {q, sc};
}
at::Tensor dequant_nvfp4(const at::Tensor& q, const at::Tensor& sc, const at::Tensor& global_amax) {
  const c10::cuda::CUDAGuard guard(q.device());
  auto xsz = q.sizes().vec(); xsz.back() *= 2;
  at::Tensor x = at::empty(xsz, q.options().dtype(at::kBFloat16));
  const int64_t cols = xsz.back(), rows = x.numel() / cols;
  mb::dequant_nvfp4(q.data_ptr<uint8_t>(), sc.data_ptr<uint8_t>(), global_amax.data_ptr<float>(), x.data_ptr(), rows, cols, cur_stream());
  return x;
}
std::vector<at::Tensor> quant_fp8_block128(const at::Tensor& x, bool ue8m0) {
  CHECK_BF16(x);
  TORCH_CHECK(x.dim() == 2, "expected a 2-D weight");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), cols = x.size(1);
  at::Tensor q = at::empty({rows, cols}, x.options().dtype(at::kByte));
  at::Tensor sc = at::empty({(rows + 127) / 128, (cols + 127) / 128}, x.options().dtype(at::kFloat));
  mb::quant_fp8_block128(x.data_ptr(), q.data_ptr<uint8_t>(), sc.data_ptr<float>(), rows, cols, ue8m0, cur_stream());
  return {q, sc};
}
std::vector<at::Tensor> fake_int4_quant(const at::Tensor& x, int64_t gr, int64_t gc, bool sym) {
  CHECK_BF16(x);
  TORCH_CHECK(x.dim() == 2 && gr > 0 && gc > 0 && (gr * gc) % 32 == 0, "group must hold a multiple of 32 elements");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), cols = x.size(1);
  at::Tensor y = at::empty_like(x);
  at::Tensor sc = at::empty({(rows + gr - 1) / gr, (cols + gc - 1) / gc}, x.options());
  at::Tensor zp = at::zeros_like(sc);
  mb::fake_int4_quant(x.data_ptr(), y.data_ptr(), sc.data_ptr(), zp.data_ptr(), rows, cols, gr, gc, sym, cur_stream());
  return {y, sc, zp};
}

}  // namespace

void register_comm(pybind11::module_& m);  // ops_bindings3.cpp
void register_mx(pybind11::module_& m);    // ops_bindings4.cpp
void register_ep_ll(pybind11::module_& m); // ops_bindings5.cpp
void register_weight_push(pybind11::module_& m); // ops_bindings6.cpp

void register_more(pybind11::module_& m) {
  register_comm(m);
  register_mx(m);
  register_ep_ll(m);
  register_weight_push(m);
  m.def("sample_rows", &sample_rows);
  m.def("paged_decode_attention", &paged_decode_attention, pybind11::arg("q"), pybind11::arg("k_cache"), pybind11::arg("v_cache"),
        pybind11::arg("block_table"), pybind11::arg("seq_lens"), pybind11::arg("out"), pybind11::arg("scratch"),
        pybind11::arg("page_size"), pybind11::arg("num_splits"), pybind11::arg("scale"), pybind11::arg("status") = pybind11::none());
  m.def("flash_attn_fwd", &flash_attn_fwd);
  m.def("flash_attn_bwd", &flash_attn_bwd);
  m.def("small_gemv", &small_gemv);
  m.def("router_small", &router_small);
  m.def("moe_small_up", &moe_small_up);
  m.def("moe_small_down", &moe_small_down);
  m.def("gae", &gae);
  m.def("quant_mxfp8", &quant_mxfp8);
  m.def("dequant_mxfp8", &dequant_mxfp8);
  m.def("absmax", &absmax);
  m.def("quant_nvfp4", &quant_nvfp4);
  m.def("dequant_nvfp4", &dequant_nvfp4);
  m.def("quant_fp8_block128", &quant_fp8_block128);
  m.def("fake_int4_quant", &fake_int4_quant);
}
