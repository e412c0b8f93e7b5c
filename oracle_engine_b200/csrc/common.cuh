// Shared helpers of the hand-written sm_100a kernels.
//
// Every exported entry point is `extern "C"`, takes raw device pointers, sizes and a
// cudaStream_t, launches on that stream and returns a cudaError_t-compatible int
// (0 = launched).  Sizes a kernel cannot take are refused on the host side with
// OE_ERR_UNSUPPORTED before anything is launched; nothing falls back to another path.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#define OE_ERR_UNSUPPORTED 100001   // size or option outside what the kernel takes
#define OE_PAGE 64                  // tokens per cache page

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of this library is launched with the
// programmatic-stream-serialization attribute: it may start while the kernel before it in
// the stream is still draining, does whatever does not depend on that kernel (set-up,
// prefetch of weights), and calls pdl_wait() before it first touches memory that an
// earlier kernel of the stream may have written (or may still read, for buffers it
// overwrites).  pdl_wait() returns when every earlier kernel has completed and its
// writes are visible.  Every kernel calls it, so completion is transitive along the
// stream.  pdl_launch_dependents() lets the next kernel be scheduled early.
// A kernel that starts early must read what earlier kernels wrote through the coherent path:
// pointers to such data are NOT `const __restrict__` (which lets the compiler use the read-only
// cache, valid only for data that does not change while the kernel is resident); weights and
// the step's integer tables, written before the step's first kernel, may be.
// Set OE_PDL=0 in the environment to launch without the attribute.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#ifndef __CUDA_ARCH__
static inline int oe_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("OE_PDL");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v;
}
#endif

template <typename... KArgs, typename... Args>
static inline int oe_launch_ex(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                               Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
#ifndef __CUDA_ARCH__
    attr[0].val.programmaticStreamSerializationAllowed = early ? oe_pdl_enabled() : 0;
#endif
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with clusters of cluster_x consecutive CTAs along x (the grid's x is a multiple of it).
template <typename... KArgs, typename... Args>
static inline int oe_launch_cluster(void (*kernel)(KArgs...), unsigned cluster_x, dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
#ifndef __CUDA_ARCH__
    attr[0].val.programmaticStreamSerializationAllowed = oe_pdl_enabled();
#endif
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster_x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// early = true: the kernel may start before the one before it has finished (see above).
template <typename... KArgs, typename... Args>
static inline int oe_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    return oe_launch_ex(true, kernel, grid, block, smem, st, args...);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block in a fixed order (warp shuffles, then warp 0 over the warp totals);
// every thread gets the result.  `red` holds 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

// Address of token `pos` of one (cache entry, K-or-V, kv head) in the paged cache.
// Storage of one cache entry: [n_pages][2][kv_heads][OE_PAGE][head_dim].
// Returns the element offset from the entry's base, or -1 if the page is not mapped.
__device__ __forceinline__ long long page_row_offset(const int* __restrict__ table_row, int pos,
                                                     int which, int kvh, int kv_heads, int head_dim) {
    const int page = table_row[pos / OE_PAGE];
    if (page < 0) return -1;
    return ((((long long)page * 2 + which) * kv_heads + kvh) * OE_PAGE + (pos % OE_PAGE)) * head_dim;
}
