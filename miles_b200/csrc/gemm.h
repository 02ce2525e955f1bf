// Host API of the tcgen05 bf16 GEMM family (dense, grouped-by-rows, grouped-by-contraction).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb {

enum GemmMode : int {
  GEMM_DENSE = 0,          // C[M,N] = A . B^T
  GEMM_GROUPED_ROWS = 1,   // every row tile of A (<= 128 rows, listed in tile_group) picks the B slab of its group
  GEMM_GROUPED_CONTR = 2,  // C_g[M,N] = sum over the rows of group g (MoE wgrad)
};

// Operand description. A "K-major" operand is a row-major [mn, k] matrix (contraction contiguous);
// an "MN-major" operand is a row-major [k, mn] matrix (contraction strided).
struct GemmOperand {
  const void* ptr;
  long long rows;  // outer extent of the row-major matrix in memory
  long long cols;  // inner (contiguous) extent
  long long ld;    // elements between rows
  bool mn_major;
};

struct GemmProblem {
  int mode;
  int M, N, K;  // logical problem per group (K ignored in GEMM_GROUPED_CONTR)
  GemmOperand a, b;
  void* c;
  long long ldc;
  long long c_group_stride;  // elements between per-group outputs (mode 2)
  bool out_fp32;
  bool accumulate;           // C += A.B^T instead of C =
  int num_groups;
  const int* tile_group;     // mode 1: [max_tiles][4] = {group, first row, rows to compute, 0} per row tile
  const int* num_m_tiles;    // mode 1: device scalar with the number of live row tiles
  int max_tiles;             // mode 1: capacity of tile_group
  const int* group_offsets;  // mode 2: [num_groups+1] row offsets, multiples of 64
  int* status;               // device status word (0 = ok); may be null
  int block_n;               // 0 = choose, else 128 or 256
  int max_ctas;              // 0 = all SMs
  // Scattered output (bf16, no accumulate): row r of C is stored at byte address row_ptrs[r] (0 = drop the row)
  // instead of c + r*ldc. The addresses may lie in other GPUs' memory mapped into this process: the epilogue then
  // is the expert-parallel return transfer (plain 16-byte P2P stores, tile by tile, while later tiles compute).
  const unsigned long long* row_ptrs;
  // With row_ptrs: after every CTA has stored its tiles and fenced at system scope, the last CTA to finish writes
  // epoch = sig_ctrl[2] + 1 to sig_flags[d][sig_me] for every rank d (release) and stores it to sig_ctrl[2];
  // sig_ctrl[5] is the arrival counter (left at zero). Null sig_ctrl = no signalling.
  unsigned long long* sig_ctrl;
  unsigned long long* sig_flags[8];
  int sig_nranks, sig_me;
  // Replicated output (bf16, no accumulate): the tile is stored at the same offset into each of dest[0..n_dest)
  // instead of c. With dest[d] = slot `me` of rank d's partial-sum buffer this turns a row-parallel projection into
  // GEMM + all-gather of partial sums in one kernel (a tensor-parallel all-reduce once the slots are added up);
  // signalling as above.
  void* dest[8];
  int n_dest;
};

// Block-scaled GEMM (gemm_mx.cu): C[M,N] (bf16) = alpha * A . B^T, both operands K-major packed values with
// scale-factor atoms (see sf_swizzle). kind 0 = MXFP8 (K % 128 == 0), kind 1 = NVFP4 (K % 256 == 0, two values per byte).
struct MxGemmProblem {
  int kind;
  int mode;  // GEMM_DENSE or GEMM_GROUPED_ROWS (row tiles start on 128-row boundaries; B holds num_groups slabs of N rows)
  int M, N, K;
  const void* a;
  long long a_rows, a_pitch_bytes;
  const void* b;
  long long b_rows, b_pitch_bytes;
  const uint8_t* sfa;
  const uint8_t* sfb;
  void* c;
  long long ldc;
  float alpha;
  const float* alpha_dev;  // optional device scalar multiplied into alpha
  int num_groups;
  const int* tile_group;
  const int* num_m_tiles;
  int max_tiles;
  int* status;
  int block_n;  // 0 = choose, else 128 or 256
};
int gemm_mx_launch(const MxGemmProblem& p, cudaStream_t stream);
const char* gemm_mx_last_error();
// Row-major scale factors [rows, S] -> 512-byte atoms [ceil(rows/128)][ceil(S/4)] in the layout the block-scaled MMA
// reads from TMEM; `out` must be zero-filled and hold ceil(rows/128) * ceil(S/4) * 512 bytes.
void sf_swizzle(const uint8_t* in, uint8_t* out, long long rows, int S, cudaStream_t s);

// Launches on `stream`. Returns 0 or a negative host-side error code (bad argument / driver error).
int gemm_bf16_launch(const GemmProblem& p, cudaStream_t stream);
const char* gemm_last_error();

}  // namespace mb
