// C++ launchers of the non-GEMM sm_100a kernels. Pointers are device pointers; every launcher is
// asynchronous on the given stream and performs no allocation.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mb {

// ---- elementwise.cu
void rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, float* rstd, int T, int H,
                 float eps, cudaStream_t s);
int rmsnorm_bwd_num_partials(int T);
void rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                 float* dw_partial, float* dw, bool accumulate_dw, int T, int H, cudaStream_t s);
void qk_norm_rope_fwd(const void* qkv, const void* qw, const void* kw, const int* pos, void* q_out, void* k_out,
                      float* q_rstd, float* k_rstd, void* k_cache, void* v_cache, const int* slot_mapping, int T,
                      int Hq, int Hk, float theta, float eps, bool use_norm, cudaStream_t s, const float* inv_freq = nullptr,
                      int rotary_dim = 128);
void qk_norm_rope_bwd(const void* dq, const void* dk, const void* dv, const void* qkv, const void* qw, const void* kw,
                      const int* pos, const float* q_rstd, const float* k_rstd, void* dqkv, float* dqw, float* dkw,
                      int T, int Hq, int Hk, float theta, bool use_norm, cudaStream_t s, const float* inv_freq = nullptr,
                      int rotary_dim = 128);
void swiglu_fwd(const void* in, void* out, long long T, int I, cudaStream_t s);
void swiglu_bwd(const void* dout, const void* in, void* din, long long T, int I, cudaStream_t s);
// Fused Adam(W) on a bf16 flat buffer. The fp32 master is `master` (fp32 array), or the pair (p, lo) with `lo` a
// signed 16-bit remainder per element (see elementwise.cu), or absent. Pointers 16-byte aligned.
void adam_step(void* p, float* master, void* lo, const void* g, bool g_fp32, void* m, void* v, bool mv_bf16, long long n,
               float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, const float* grad_scale,
               const float* skip_flag, cudaStream_t s);
void split_master_join(const void* p, const void* lo, float* out, long long n, cudaStream_t s);
void split_master_cut(const float* master, void* p, void* lo, long long n, cudaStream_t s);
int sumsq_num_partials(long long n);
void sumsq(const void* g, bool g_fp32, long long n, float* partial, float* out, cudaStream_t s);
// out[i] = std * N(key, first + i), a counter-based generator: independent of how the logical tensor is sharded.
void init_normal(void* out, bool fp32, long long n, unsigned long long key, long long first, float std, cudaStream_t s);

// ---- moe.cu
// Router: softmax over E experts (fp32 logits), top-k, optional renormalisation of the k weights.
// With `replay_ids` the expert choice is taken from it (rollout routing replay) and only the weights
// are recomputed from the current logits.
void moe_router_topk(const float* logits, const int* replay_ids, int* topk_ids, float* topk_w, float* probs_out,
                     int T, int E, int K, bool renorm, cudaStream_t s);
// Deterministic counting sort of the T*K (token, slot) pairs by expert. Rows of each expert are padded
// to a multiple of `align`; outputs: dest_row[T*K], row_src[max_rows] (-1 for padding), expert_offsets[E+1]
// (padded), tile_group[max_tiles][4] = {expert, row0, rows, 0}, num_m_tiles[2] = {tiles, live rows},
// expert_counts[E].
void moe_build_permutation(const int* topk_ids, int T, int K, int E, int max_rows, int max_tiles, int align,
                           int* expert_counts, int* expert_offsets, int* dest_row, int* row_src, int* tile_group,
                           int* num_m_tiles, cudaStream_t s);
void moe_permute(const void* x, const int* row_src, const int* num_m_tiles, void* x_perm, int max_rows, int H, int K,
                 cudaStream_t s);
// out[t] = (residual[t] +) sum_k w[t,k] * y_perm[dest_row[t,k]]
void moe_combine(const void* y_perm, const int* dest_row, const float* topk_w, const void* residual, void* out, int T,
                 int K, int H, cudaStream_t s);
// dy_perm[row] = w * dout[token]; dw[t,k] = <dout[t], y_perm[row]>; padding rows are zeroed.
void moe_combine_bwd(const void* dout, const void* y_perm, const int* row_src, const int* num_m_tiles,
                     const float* topk_w, void* dy_perm, float* dtopk_w, int max_rows, int K, int H, cudaStream_t s);
// dx[t] = sum_k dx_perm[dest_row[t,k]]
void moe_unpermute_sum(const void* dx_perm, const int* dest_row, void* dx, int T, int K, int H, cudaStream_t s);
// Backward of softmax->topk->renorm wrt the router logits.
void moe_router_bwd(const float* probs, const int* topk_ids, const float* topk_w, const float* dtopk_w, float* dlogits,
                    int T, int E, int K, bool renorm, cudaStream_t s);

// ---- logprob.cu
// Row-wise online softmax statistics over bf16 or fp32 logits scaled by 1/temperature:
// logprob of `target`, entropy, and (kept for the backward) row max and log-sum-exp.
void logprob_entropy_fwd(const void* logits, bool fp32, const int* targets, float* logprob, float* entropy, float* lse,
                         float* psum_x, int T, int V, long long ld, float inv_temp, cudaStream_t s);
// dlogits = inv_temp * ( dlp * (onehot - p) - dH * p * (x - sum p x) ), written as bf16 with row pitch ld_out
// (in place is allowed for bf16 logits).
void logprob_entropy_bwd(const void* logits, bool fp32, const int* targets, const float* lse, const float* psum_x,
                         const float* dlogprob, const float* dentropy, void* dlogits, int T, int V, long long ld,
                         long long ld_out, float inv_temp, cudaStream_t s);

// ---- sampling.cu
// Per-row temperature / top-k / top-p sampling with a counter-based RNG; returns the token and its
// logprob under the temperature-scaled full distribution.
void sample_rows(const void* logits, bool fp32, int T, int V, long long ld, const float* temperature, const int* top_k,
                 const float* top_p, const unsigned long long* seeds, const int* step, int* out_token, float* out_logprob,
                 cudaStream_t s);

// ---- attention.cu
// Returns the CUDA error code of its own launches (0 = ok). `num_slots` = rows of the cache (0: unchecked page ids),
// `status` (device int or null) receives 8 / 9 for a length / page id outside the tables.
int paged_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                           const int* seq_lens, void* out, float* scratch, int B, int Hq, int Hk, int page_size,
                           int max_pages, int num_splits, float scale, cudaStream_t s, long long num_slots = 0,
                           int* status = nullptr);

// ---- attention_fwd.cu
// Causal variable-length attention forward on tcgen05. q/k/v are bf16 [rows, heads, 128] views with row pitches
// q_ld/k_ld/v_ld (elements); `tiles` is int32 [num_tiles][4] = {q_row0, q_rows (<=128), kv_row0, q_pos0}: the
// tile covers query rows q_row0.. of the q tensor, whose sequence starts at row kv_row0 of k/v and whose first
// query sits at position q_pos0 of that sequence. out bf16 [Tq, Hq, 128]; lse fp32 [Hq, Tq] (natural log) or
// null. Returns 0, or -1 with flash_attn_last_error() set.
int flash_attn_fwd(const void* q, long long q_ld, const void* k, long long k_ld, const void* v, long long v_ld,
                   void* out, float* lse, const int* tiles, int num_tiles, long long Tq, long long Tkv, int Hq, int Hk,
                   int head_dim, float scale, int* status, cudaStream_t stream);
const char* flash_attn_last_error();
// attention_bwd.cu: causal varlen backward for self-attention over packed sequences (keys = queries' own tokens).
// q, o, d_o [T, Hq, 128] (o and d_o contiguous), k, v [T, Hk, 128] (row pitches in elements); lse fp32 [Hq, T] from the
// forward; blocks int32 [n, 4] = {first key row, keys (<= 128), position of the first key in its sequence, row one past
// the sequence}; scratch fp32 [T*Hq*128 + 2*Hq*T]; dq [T, Hq, 128], dk / dv [T, Hk, 128] bf16 contiguous.
int flash_attn_bwd(const void* q, long long q_ld, const void* k, long long k_ld, const void* v, long long v_ld, const void* o,
                   const void* d_o, long long do_ld, const float* lse, const int* blocks, int num_blocks, long long T, int Hq,
                   int Hk, int head_dim, float scale, float* scratch, void* dq, void* dk, void* dv, int* status,
                   cudaStream_t stream);
const char* flash_attn_bwd_last_error();

// ---- decode_stream.cu / decode_small.cu (at most 8 tokens: persistent weight-streaming mma.sync kernel fed by
// bulk asynchronous copies, RMSNorm folded in; `status` receives a code if a bounded wait gives up)
void small_gemv(const void* x, int T, const void* norm_w, float eps, const void* W, int N, int K, const void* residual,
                void* out, bool out_fp32, int* status, cudaStream_t s);
void router_small(const float* logits, int T, int E, int K, bool renorm, int* topk_ids, float* topk_w, int* active,
                  int* pair_count, int* pair_list, cudaStream_t s);
// gu[pair, 2I] = W1[e] . norm(x[pair / K]) for the experts listed in `active` (count in active[0])
void moe_small_up(const void* x, const void* norm_w, float eps, const void* W1, const int* active, const int* pair_count,
                  const int* pair_list, int max_active, int H, int I, int K, void* gu, int* status, cudaStream_t s);
// y[pair, H] = W2[e] . (silu(gu[pair, :I]) * gu[pair, I:])
void moe_small_down(const void* gu, const void* W2, const int* active, const int* pair_count, const int* pair_list,
                    int max_active, int H, int I, void* y, int* status, cudaStream_t s);

// ---- rl.cu
void gae_reverse_scan(const float* rewards, const float* values, const int* cu_seqlens, float* adv, float* ret,
                      int num_seqs, float gamma, float lam, cudaStream_t s);

// ---- quant.cu
void quant_mxfp8(const void* x, uint8_t* q, uint8_t* scales, long long rows, long long cols, cudaStream_t s);
void dequant_mxfp8(const uint8_t* q, const uint8_t* scales, void* x, long long rows, long long cols, cudaStream_t s);
void quant_nvfp4(const void* x, uint8_t* q, uint8_t* block_scales, const float* global_amax, long long rows,
                 long long cols, cudaStream_t s);
void dequant_nvfp4(const uint8_t* q, const uint8_t* block_scales, const float* global_amax, void* x, long long rows,
                   long long cols, cudaStream_t s);
void absmax(const void* x, long long n, float* out, cudaStream_t s);
void quant_fp8_block128(const void* x, uint8_t* q, float* scales, long long rows, long long cols, bool ue8m0,
                        cudaStream_t s);
void fake_int4_quant(const void* x, void* y, void* scale, void* zero, long long rows, long long cols, int group_rows,
                     int group_cols, bool symmetric, cudaStream_t s);

// ---- ep_comm.cu: expert-parallel exchange over NVLink peer memory
constexpr int kMaxPeers = 8;
struct EpPeers {
  void* xrecv[kMaxPeers];                 // peer receive regions [nranks][cap][H] bf16
  int* meta[kMaxPeers];                   // per received row: (local expert, source slot)
  int* counts[kMaxPeers];                 // [nranks] rows sent by each source
  unsigned long long* flags[kMaxPeers];   // [nranks] dispatch arrival epochs
  void* yback[kMaxPeers];                 // peer return regions [T*K][H] bf16
  unsigned long long* flags2[kMaxPeers];  // [nranks] return arrival epochs
  const int* send_counts;                 // local: true number of entries bound for each rank
};
void ep_dispatch(const void* x, const int* ids, const int* dest_row, const int* offsets, const EpPeers& peers, int me,
                 int nranks, int experts_per_rank, int n_entries, int row_div, int H, int cap, unsigned long long* ctrl,
                 int* status, cudaStream_t s);
void ep_wait(const unsigned long long* flags, int nranks, unsigned long long* ctrl, int which, int* status, cudaStream_t s);
void sum_slots(const void* slots, long long slot_elems, int n, const void* residual, void* out, long long elems,
               cudaStream_t s);
void ep_row_ptrs(const int* row_src, const int* meta, const EpPeers& peers, int cap, int H, int max_rows,
                 unsigned long long* out, cudaStream_t s);
void ep_return(const void* yp, const int* recv_dest_row, const int* meta, const int* counts, const EpPeers& peers, int me,
               int nranks, int cap, int H, unsigned long long* ctrl, int* status, cudaStream_t s);

// ---- ep_decode.cu (low-latency expert-parallel exchange for decode steps)
struct EpLLPeers {
  char* base[kMaxPeers];  // every rank's mapping of the symmetric region (own rank included)
};
struct EpLLLayout {       // identical on all ranks; offsets in bytes from the region base
  int R, Bm, H, K;        // ranks, max rows per rank and step, hidden size, experts per token
  long long off_xg;       // [R][Bm][H] bf16   gathered (normalised) rows, by source rank
  long long off_ig;       // [R][Bm][K] int32  their expert ids (-1: padding row)
  long long off_wg;       // [R][Bm][K] fp32   their gate weights
  long long off_yb;       // [R][Bm][H] bf16   partial sums returned by each owner rank for this rank's rows
  long long off_flag_a;   // [R] u64 (epoch << 32 | rows)  arrival of a source's rows
  long long off_flag_b;   // [R] u64 (epoch << 32)         arrival of an owner's partial sums
};
size_t ep_ll_plan_smem(const EpLLLayout& L, int E);
int ep_ll_send(const void* x, const void* ln_w, float eps, const float* logits, const int* active, const EpLLPeers& peers,
               const EpLLLayout& L, int me, int T, int E, bool renorm, int* ids_out, float* w_out, unsigned long long* ctrl,
               cudaStream_t s);
int ep_ll_plan(char* local, const EpLLLayout& L, int me, int E, int max_rows, int max_tiles, int align, int* src_rows,
               int* counts, int* offsets, int* dest_row, int* row_src, int* tiles, int* totals, unsigned long long* ctrl,
               unsigned long long wait_ns, int* status, cudaStream_t s);
void ep_ll_return(const void* yp, const int* dest_row, const int* src_rows, const EpLLPeers& peers, const EpLLLayout& L, int me,
                  int rows_hint, unsigned long long* ctrl, cudaStream_t s);
void ep_ll_combine(const char* local, const EpLLLayout& L, const int* ids, const int* active, const void* residual, void* out,
                   int T, int E, unsigned long long* ctrl, unsigned long long wait_ns, int* status, cudaStream_t s);

// ---- dp_adam.cu (gradient reduce-scatter + partitioned Adam + parameter all-gather over peer memory)
struct DpPeers {
  void* grad[kMaxPeers];                  // fp32 flat gradient buffers of all data-parallel ranks
  void* param[kMaxPeers];                 // bf16 flat parameter buffers
  unsigned long long* flags[kMaxPeers];   // [nranks] "gradients final" epochs
  unsigned long long* flags2[kMaxPeers];  // [nranks] "parameters pushed" epochs
};
void peer_signal(const DpPeers& peers, int me, int nranks, unsigned long long* ctrl, int which, bool second, cudaStream_t s);
int dp_reduce_shard_blocks(long long shard_elems);
void dp_reduce_shard(const DpPeers& peers, int nranks, long long lo, long long shard_elems, float* reduced, float* partial,
                     cudaStream_t s);
void dp_adam_push(const DpPeers& peers, int me, int nranks, long long lo, long long n, const float* reduced, float* master,
                  void* m, void* v, bool mv_bf16, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                  const float* grad_scale, const float* skip_flag, cudaStream_t s);

int symm_alloc(size_t nbytes, void** ptr, char* handle64);
int symm_open(const char* handle64, void** ptr);
int symm_close(void* ptr);
int symm_free(void* ptr);

// ---- trainer -> engine weight push (weight_push.cu). The tables are int64 rows so that the host builds them as tensors.
struct WeightPushSeg {      // one 2-D slab of the local shard
  long long src_off;        // element offset in the source buffer (multiple of 8)
  long long rows, cols;     // cols % 8 == 0 (bf16), % 128 (MXFP8), % 64 (NVFP4)
  long long src_ld;         // source leading dimension in elements (multiple of 8)
  long long tensor;         // row of the tensor table
  long long dst_row0, dst_col0;  // position of the slab inside the destination tensor
  long long peer_mask;      // ranks that receive the slab
};
struct WeightPushTensor {   // one destination tensor, at the same offsets inside every rank's symmetric region
  long long val_off;        // byte offset of the values
  long long sf_off;         // byte offset of the scale-factor atoms (quantised modes)
  long long ld;             // destination leading dimension in elements (= K for the quantised modes)
  long long mode;           // 0 bf16, 1 MXFP8, 2 NVFP4
  long long amax_slot;      // NVFP4: index of the per-tensor amax
  long long pad[3];
};
struct WeightPushPeers {
  char* base[8];
  long long flag_off;       // byte offset of the 8 arrival flags (u64) inside every region
};
int weight_push(const void* src, const WeightPushSeg* segs, int nseg, const WeightPushTensor* tensors, const float* amax,
                const WeightPushPeers& peers, int me, unsigned flag_mask, unsigned long long version, unsigned int* counter,
                long long total_vecs, cudaStream_t s);
void weight_push_wait(const unsigned long long* flags, unsigned src_mask, unsigned long long version, double wait_ms, int* status,
                      cudaStream_t s);

}  // namespace mb
