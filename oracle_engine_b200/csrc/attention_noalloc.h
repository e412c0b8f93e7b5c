// oe_attn_mma_bf16_noalloc: decode / prompt attention over the paged cache for callers
// that must not allocate device memory.
//
// This entry point has no counterpart in the reference engine (which runs on the CPU and
// has no device memory at all).  It exists for hosts that drive this library from a
// context where cudaMalloc is off limits: a real-time or safety-certified control loop
// whose memory is fixed at start-up, a plugin running inside another application's CUDA
// memory pool, or a step that is being replayed while device allocation is forbidden.
// Such callers own every buffer they pass in; what they cannot provide is the float32
// scratch that the split-key decode path needs between its two kernels.  This variant
// keeps that scratch in a fixed array inside the library's device image instead.
//
// Same arguments and results as oe_attn_mma_bf16 (csrc/attention_mma.cu) without the
// `partial` pointer.  Differences a caller has to know:
//   * The scratch is OE_ATTN_NOALLOC_MAX_FLOATS float32 values (8 MiB).  Every GPU on which
//     the library is loaded holds that array until the process exits.  The attention library
//     is built once per head size, so a process that loads the libraries of several head
//     sizes holds one such array per head size and GPU.
//   * A call needs n_tokens * H * n_splits * (head_dim + 2) floats when n_splits > 1 (and
//     none otherwise).  A call that needs more is refused with OE_ERR_SCRATCH_TOO_SMALL
//     before anything is launched; oe_attn_mma_error_string() gives the text.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and keeps it.  Make that first call
//     outside any stream capture, and from one thread: the look-up takes no lock (two
//     threads that both make a first call would both store the same address).
//   * Nothing in the array has to start at zero: each call writes every partial it later
//     reads.  All calls of a head size share one array, so two calls that may overlap on the GPU
//     (different streams without an ordering between them) race; keep them on one stream
//     or order them with events.
//   * It calls no cudaMalloc, cudaFree or other allocating routine.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#define OE_ATTN_NOALLOC_MAX_FLOATS (2ll << 20)
#define OE_ERR_SCRATCH_TOO_SMALL 100002

#ifdef __cplusplus
extern "C" {
#endif

int oe_attn_mma_bf16_noalloc(__nv_bfloat16* out, const __nv_bfloat16* q, long long q_stride,
                             const __nv_bfloat16* cache, const int* tables, int max_pages, const int* cu_q,
                             const int* seq_start, const int* seq_qlen, const int* tok_seq, int n_seqs,
                             int n_tokens, int max_qlen, int H, int KVH, int window, float scale, int n_splits,
                             cudaStream_t stream);

const char* oe_attn_mma_error_string(int code);

#ifdef __cplusplus
}
#endif
