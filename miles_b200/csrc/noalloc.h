// Allocation-free C entry point of the paged decode attention.
//
// This entry point has no counterpart in the reference framework. It exists for hosts that drive
// decode attention of this library but cannot obtain device memory at call time: a C/C++ serving loop
// that links the shared object without PyTorch's caching allocator, or a rollout process that has
// already handed every free byte of the device to the KV-cache pool (a static memory fraction), where
// a cudaMalloc for the split-KV partial results would either fail or stall the device.
//
// The split-KV partials live in a fixed array in device global memory that is part of the library
// image: MB_NOALLOC_SCRATCH_FLOATS floats (16 MiB) on every GPU that loads the library, held until
// the process exits. Nothing is allocated or freed by the call, by this library or by a library it
// calls.
//
// Rules for callers:
//   * B * Hq * num_splits * 130 must not exceed MB_NOALLOC_SCRATCH_FLOATS; larger requests are refused
//     with MB_NOALLOC_ERR_TOO_LARGE and nothing is launched.
//   * The first call on each device looks up the device address of the array (with that device current).
//     Make that first call outside of any stream capture.
//   * All calls on a device share the one array and it keeps whatever the previous call left in it. No
//     part of it has to start at zero: each call overwrites every partial slot before it reads it. Two
//     calls whose kernels may overlap on the GPU (different streams, no ordering) race on the array;
//     order them on one stream or with events.
//   * seq_lens and block_table are read on the device and are not trusted: a length below zero or beyond
//     max_pages * page_size is clamped (status 8), and a page id that is negative or whose last row lies
//     beyond num_slots is treated as a page of zeros instead of being read (status 9). `status` is an
//     optional device int the kernel writes the first such code into (pass NULL to ignore); the host
//     decides when to read it.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MB_NOALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)

enum {
  MB_NOALLOC_OK = 0,
  MB_NOALLOC_ERR_BAD_ARG = -1,     // null pointer, non-positive extent, unsupported head configuration
  MB_NOALLOC_ERR_TOO_LARGE = -2,   // B * Hq * num_splits * 130 floats do not fit the built-in scratch
  MB_NOALLOC_ERR_CUDA = -3,        // a CUDA runtime call failed (symbol lookup or launch)
};

// q [B, Hq, 128] bf16; k_cache / v_cache [slots, Hk, 128] bf16 with slot = page * page_size + offset;
// block_table [B, max_pages] int32; seq_lens [B] int32; out [B, Hq, 128] bf16. Hq / Hk in {1, 2, 4, 8}.
// num_slots = rows of k_cache / v_cache (pages * page_size); status = device int or NULL (see above).
// Asynchronous on `stream`. Returns MB_NOALLOC_OK or one of the codes above;
// mb_noalloc_last_error() describes the most recent failure of the calling thread.
__attribute__((visibility("default"))) int mb_paged_decode_attention_noalloc(
    const void* q, const void* k_cache, const void* v_cache, const int* block_table, const int* seq_lens, void* out,
    int B, int Hq, int Hk, int page_size, int max_pages, int num_splits, float scale, long long num_slots, int* status,
    cudaStream_t stream);

__attribute__((visibility("default"))) const char* mb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
