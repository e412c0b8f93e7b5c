// Row-wise kernels around the matrix products: embedding gather, RMSNorm, rotary
// position encoding fused with the cache write, SwiGLU, row gather.
//
// The residual stream is float32 in both precisions; T is the activation / weight /
// cache type (float for the 32-bit path, bf16 for serving).  All arithmetic is float32.
// Every row is computed by itself in a fixed order, so a row's result does not depend on
// which other rows are in the batch.
#include "common.cuh"

// ---------------------------------------------------------------------------------------
// x[t, :] = table[ids[t], :]            (reference: core/model.cpp:352-358)
// An id outside [0, vocab) writes zeros and raises *err (the reference clamps to 0 with a
// warning; here it is an error the host reports).
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(float* __restrict__ x, const T* __restrict__ table,
                                    const int* __restrict__ ids, int D, int vocab, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* xr = x + (size_t)t * D;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && err) atomicExch(err, 1);
        for (int d = threadIdx.x; d < D; d += blockDim.x) xr[d] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) xr[d] = to_f32(row[d]);
}

// ---------------------------------------------------------------------------------------
// y = (x * 1/sqrt(mean(x^2) + eps)) * w      (reference: core/ops.cpp:149-195)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_kernel(T* y, const float* x,
                               const float* __restrict__ w, int D, float eps) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* xr = x + (size_t)blockIdx.x * D;
    T* yr = y + (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) { const float v = xr[d]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float s = 1.f / sqrtf(ss / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) yr[d] = from_f32<T>((xr[d] * s) * w[d]);
}

// The same with 16-byte loads, for D a multiple of 4: each thread keeps its first chunks in
// registers, so the row is read once.  The order of the sum is fixed by D and the block
// size, not by the batch.
constexpr int OE_RMSNORM_ROWS_MIN = 1024;    // from this many rows the bfloat16 norm of up to 4096 columns runs a warp per row
template <typename T> struct Out4;
template <> struct Out4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) { *(float4*)p = make_float4(a, b, c, d); }
};
template <> struct Out4<bf16> {
    static __device__ __forceinline__ void store(bf16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        *(uint2*)p = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
    }
};

template <typename T, int NT>
__global__ void __launch_bounds__(NT)
rmsnorm_vec_kernel(T* y, const float* x, const float* __restrict__ w, int D, float eps) {
    __shared__ float red[32];
    constexpr int KEEP = 4;
    pdl_launch_dependents();
    pdl_wait();
    const float4* xr = (const float4*)(x + (size_t)blockIdx.x * D);
    const float4* wr = (const float4*)w;
    T* yr = y + (size_t)blockIdx.x * D;
    const int n4 = D / 4;
    float4 keep[KEEP];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < KEEP; j++) {
        const int i = threadIdx.x + j * NT;
        keep[j] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += keep[j].x * keep[j].x + keep[j].y * keep[j].y + keep[j].z * keep[j].z + keep[j].w * keep[j].w;
    }
    for (int i = threadIdx.x + KEEP * NT; i < n4; i += NT) {
        const float4 v = xr[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss, red);
    const float s = 1.f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int j = 0; j < KEEP; j++) {
        const int i = threadIdx.x + j * NT;
        if (i < n4) {
            const float4 g = wr[i];
            Out4<T>::store(yr + 4 * i, (keep[j].x * s) * g.x, (keep[j].y * s) * g.y, (keep[j].z * s) * g.z, (keep[j].w * s) * g.w);
        }
    }
    for (int i = threadIdx.x + KEEP * NT; i < n4; i += NT) {
        const float4 v = xr[i], g = wr[i];
        Out4<T>::store(yr + 4 * i, (v.x * s) * g.x, (v.y * s) * g.y, (v.z * s) * g.z, (v.w * s) * g.w);
    }
}

// Many rows (a prompt step): one WARP per row, no barrier, the whole row (KEEP x 32 float4) in
// registers with all its loads in flight at once, so that the kernel runs at memory speed
// instead of at the latency of one block's load, reduce, store.  Its sum has another
// order than the block kernel's; both are float32 sums of the same squares.
template <typename T, int KEEP>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(T* y, const float* x, const float* __restrict__ w, int rows, int D, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float4* xr = (const float4*)(x + (size_t)r * D);
    const float4* wr = (const float4*)w;
    T* yr = y + (size_t)r * D;
    const int n4 = D / 4;
    float4 keep[KEEP];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < KEEP; j++) {
        const int i = lane + j * 32;
        keep[j] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < KEEP; j++)
        ss += keep[j].x * keep[j].x + keep[j].y * keep[j].y + keep[j].z * keep[j].z + keep[j].w * keep[j].w;
    for (int i = lane + KEEP * 32; i < n4; i += 32) {
        const float4 v = xr[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float s = 1.f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int j = 0; j < KEEP; j++) {
        const int i = lane + j * 32;
        if (i < n4) {
            const float4 g = wr[i];
            Out4<T>::store(yr + 4 * i, (keep[j].x * s) * g.x, (keep[j].y * s) * g.y, (keep[j].z * s) * g.z, (keep[j].w * s) * g.w);
        }
    }
    for (int i = lane + KEEP * 32; i < n4; i += 32) {
        const float4 v = xr[i], g = wr[i];
        Out4<T>::store(yr + 4 * i, (v.x * s) * g.x, (v.y * s) * g.y, (v.z * s) * g.z, (v.w * s) * g.w);
    }
}

// ---------------------------------------------------------------------------------------
// Rotary encoding of q and k (rotate-half pairs (i, i+hd/2)) at each token's absolute
// position, from a float32 cos/sin table [max_pos, hd/2]; q is rotated in place, rotated
// k and v go to the token's row of the paged cache.
// (reference: core/ops.cpp:440-485 and the cache write core/model.cpp:405-408, 596-602)
// qkv row: [H*hd | KVH*hd | KVH*hd] when has_kv, else [H*hd] only.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride,
                                     const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                     T* __restrict__ cache, const int* __restrict__ tables, int max_pages,
                                     const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                     int H, int KVH, int hd, int has_kv, int rotate) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    if (b < 0) return;
    const int pos = tok_pos[t];
    const int half = hd / 2;
    T* row = qkv + (size_t)t * row_stride;
    const float* cs = cos_tab + (size_t)pos * half;
    const float* sn = sin_tab + (size_t)pos * half;
    for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        T* p = row + h * hd;
        const float x0 = to_f32(p[i]), x1 = to_f32(p[i + half]);
        if (rotate) {
            const float c = cs[i], s = sn[i];
            p[i] = from_f32<T>(x0 * c - x1 * s);
            p[i + half] = from_f32<T>(x0 * s + x1 * c);
        }
    }
    if (!has_kv) return;
    const int* trow = tables + (size_t)b * max_pages;
    const T* krow = row + H * hd;
    const T* vrow = krow + KVH * hd;
    for (int idx = threadIdx.x; idx < KVH * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        const long long ko = page_row_offset(trow, pos, 0, h, KVH, hd);
        const long long vo = page_row_offset(trow, pos, 1, h, KVH, hd);
        if (ko < 0) continue;
        const float x0 = to_f32(krow[h * hd + i]), x1 = to_f32(krow[h * hd + i + half]);
        if (rotate) {
            const float c = cs[i], s = sn[i];
            cache[ko + i] = from_f32<T>(x0 * c - x1 * s);
            cache[ko + i + half] = from_f32<T>(x0 * s + x1 * c);
        } else {
            cache[ko + i] = from_f32<T>(x0);
            cache[ko + i + half] = from_f32<T>(x1);
        }
        cache[vo + i] = vrow[h * hd + i];
        cache[vo + i + half] = vrow[h * hd + i + half];
    }
}

// The same with 16-byte accesses: a work item is VEC consecutive pairs (i, i + hd/2) of one
// head.  Needs hd/2 and the row stride to be multiples of VEC = 16 / sizeof(T).
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) { const float4 t = *(const float4*)p; v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *(float4*)p = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
        const uint4 t = *(const uint4*)p;
        const uint32_t r[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int j = 0; j < 4; j++) { const __nv_bfloat162 h = *(const __nv_bfloat162*)&r[j]; v[2 * j] = __low2float(h); v[2 * j + 1] = __high2float(h); }
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
        uint32_t r[4];
#pragma unroll
        for (int j = 0; j < 4; j++) { __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]); r[j] = *(uint32_t*)&h; }
        *(uint4*)p = make_uint4(r[0], r[1], r[2], r[3]);
    }
};

template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, int row_stride,
                                         const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                         T* __restrict__ cache, const int* __restrict__ tables, int max_pages,
                                         const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                         int H, int KVH, int hd, int has_kv, int rotate) {
    constexpr int V = Vec16<T>::N;
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    if (b < 0) return;
    const int pos = tok_pos[t];
    const int half = hd / 2, per_head = half / V;
    T* row = qkv + (size_t)t * row_stride;
    const float* cs = cos_tab + (size_t)pos * half;
    const float* sn = sin_tab + (size_t)pos * half;
    const int n_q = H * per_head, n_k = has_kv ? KVH * per_head : 0;
    const int* trow = tables + (size_t)b * max_pages;
    for (int idx = threadIdx.x; idx < n_q + n_k; idx += blockDim.x) {
        const bool is_k = idx >= n_q;
        const int h = (is_k ? idx - n_q : idx) / per_head, i = ((is_k ? idx - n_q : idx) % per_head) * V;
        const T* src = row + (size_t)(is_k ? H + h : h) * hd;
        float x0[V], x1[V], y0[V], y1[V];
        Vec16<T>::load(src + i, x0);
        Vec16<T>::load(src + i + half, x1);
        if (rotate) {
            // i is a multiple of V and the table's rows are hd/2 floats: 16-byte loads
            float c[V], s[V];
#pragma unroll
            for (int j = 0; j < V; j += 4) {
                const float4 c4 = *(const float4*)(cs + i + j), s4 = *(const float4*)(sn + i + j);
                c[j] = c4.x; c[j + 1] = c4.y; c[j + 2] = c4.z; c[j + 3] = c4.w;
                s[j] = s4.x; s[j + 1] = s4.y; s[j + 2] = s4.z; s[j + 3] = s4.w;
            }
#pragma unroll
            for (int j = 0; j < V; j++) {
                y0[j] = x0[j] * c[j] - x1[j] * s[j];
                y1[j] = x0[j] * s[j] + x1[j] * c[j];
            }
        } else {
#pragma unroll
            for (int j = 0; j < V; j++) { y0[j] = x0[j]; y1[j] = x1[j]; }
        }
        if (!is_k) {
            if (rotate) {
                Vec16<T>::store(row + (size_t)h * hd + i, y0);
                Vec16<T>::store(row + (size_t)h * hd + i + half, y1);
            }
        } else {
            const long long ko = page_row_offset(trow, pos, 0, h, KVH, hd);
            const long long vo = page_row_offset(trow, pos, 1, h, KVH, hd);
            if (ko < 0) continue;
            Vec16<T>::store(cache + ko + i, y0);
            Vec16<T>::store(cache + ko + i + half, y1);
            const T* vsrc = row + (size_t)(H + KVH + h) * hd;
            *(uint4*)(cache + vo + i) = *(const uint4*)(vsrc + i);
            *(uint4*)(cache + vo + i + half) = *(const uint4*)(vsrc + i + half);
        }
    }
}

// The same for many tokens (a prompt step): a block takes TPB tokens and first brings their whole rows
// (q, k and v: one contiguous run each) into shared memory with 16-byte asynchronous copies, so that
// what a block has in flight is bounded by its shared memory, not by its registers; then it rotates out
// of shared memory.  With a block per token and the values in registers the SMs had about 40 KB in
// flight each and the kernel ran at 0.55-0.6 of the memory's rate.
__device__ __forceinline__ void stage16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
template <typename T, int TPB>
__global__ void __launch_bounds__(256)
rope_kv_write_staged_kernel(T* __restrict__ qkv, int row_stride,
                            const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                            T* __restrict__ cache, const int* __restrict__ tables, int max_pages,
                            const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, int n_tokens,
                            int H, int KVH, int hd, int has_kv, int rotate) {
    constexpr int V = Vec16<T>::N;
    extern __shared__ __align__(16) uint8_t staged[];
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * TPB;
    const int width = (H + (has_kv ? 2 * KVH : 0)) * hd;          // elements of a row that are used
    const int chunks = width / V;                                  // 16-byte pieces of a row
    const int row_bytes = chunks * 16;
#pragma unroll
    for (int j = 0; j < TPB; j++) {
        if (t0 + j >= n_tokens) break;
        const T* src = qkv + (size_t)(t0 + j) * row_stride;
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) stage16(staged + (size_t)j * row_bytes + c * 16, src + c * V);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    int seq[TPB], place[TPB];
#pragma unroll
    for (int j = 0; j < TPB; j++) {
        const bool in = t0 + j < n_tokens;
        seq[j] = in ? tok_seq[t0 + j] : -1;
        place[j] = in ? tok_pos[t0 + j] : 0;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const int half = hd / 2, per_head = half / V;
    const int n_q = H * per_head, n_k = has_kv ? KVH * per_head : 0;
#pragma unroll
    for (int j = 0; j < TPB; j++) {
        if (seq[j] < 0) continue;
        const int pos = place[j];
        const T* srow = reinterpret_cast<const T*>(staged + (size_t)j * row_bytes);
        T* row = qkv + (size_t)(t0 + j) * row_stride;
        const float* cs = cos_tab + (size_t)pos * half;
        const float* sn = sin_tab + (size_t)pos * half;
        const int* trow = tables + (size_t)seq[j] * max_pages;
        for (int idx = threadIdx.x; idx < n_q + n_k; idx += blockDim.x) {
            const bool is_k = idx >= n_q;
            const int h = (is_k ? idx - n_q : idx) / per_head, i = ((is_k ? idx - n_q : idx) % per_head) * V;
            if (!is_k && !rotate) continue;                        // q stays as it is
            const T* src = srow + (size_t)(is_k ? H + h : h) * hd;
            float x0[V], x1[V], y0[V], y1[V];
            Vec16<T>::load(src + i, x0);
            Vec16<T>::load(src + i + half, x1);
            if (rotate) {
                float c[V], sv[V];
#pragma unroll
                for (int e = 0; e < V; e += 4) {
                    const float4 c4 = *(const float4*)(cs + i + e), s4 = *(const float4*)(sn + i + e);
                    c[e] = c4.x; c[e + 1] = c4.y; c[e + 2] = c4.z; c[e + 3] = c4.w;
                    sv[e] = s4.x; sv[e + 1] = s4.y; sv[e + 2] = s4.z; sv[e + 3] = s4.w;
                }
#pragma unroll
                for (int e = 0; e < V; e++) {
                    y0[e] = x0[e] * c[e] - x1[e] * sv[e];
                    y1[e] = x0[e] * sv[e] + x1[e] * c[e];
                }
            } else {
#pragma unroll
                for (int e = 0; e < V; e++) { y0[e] = x0[e]; y1[e] = x1[e]; }
            }
            if (!is_k) {
                Vec16<T>::store(row + (size_t)h * hd + i, y0);
                Vec16<T>::store(row + (size_t)h * hd + i + half, y1);
            } else {
                const long long ko = page_row_offset(trow, pos, 0, h, KVH, hd);
                const long long vo = page_row_offset(trow, pos, 1, h, KVH, hd);
                if (ko < 0) continue;
                Vec16<T>::store(cache + ko + i, y0);
                Vec16<T>::store(cache + ko + i + half, y1);
                const T* vsrc = srow + (size_t)(H + KVH + h) * hd;
                *(uint4*)(cache + vo + i) = *(const uint4*)(vsrc + i);
                *(uint4*)(cache + vo + i + half) = *(const uint4*)(vsrc + i + half);
            }
        }
    }
}

// Many tokens and rows that fit: the staged kernel with as many tokens per block as 40 KB of shared memory hold.
#define OE_ROPE_STAGED_MIN_TOKENS 512
template <typename T>
static int rope_staged(bool& done, T* qkv, int row_stride, const float* cos_tab, const float* sin_tab, T* cache,
                       const int* tables, int max_pages, const int* tok_seq, const int* tok_pos, int n_tokens, int H,
                       int KVH, int hd, int has_kv, int rotate, cudaStream_t st) {
    done = false;
    if (n_tokens < OE_ROPE_STAGED_MIN_TOKENS) return 0;
    const size_t row_bytes = (size_t)(H + (has_kv ? 2 * KVH : 0)) * hd * sizeof(T);
    const size_t budget = 40 * 1024;
#define OE_ROPE_STAGED(TPB)                                                                                          \
    if (row_bytes * TPB <= budget) {                                                                                  \
        done = true;                                                                                                  \
        return oe_launch(rope_kv_write_staged_kernel<T, TPB>, dim3((n_tokens + TPB - 1) / TPB), dim3(256),            \
                         row_bytes * TPB, st, qkv, row_stride, cos_tab, sin_tab, cache, tables, max_pages, tok_seq,    \
                         tok_pos, n_tokens, H, KVH, hd, has_kv, rotate);                                              \
    }
    OE_ROPE_STAGED(4)
    OE_ROPE_STAGED(2)
    OE_ROPE_STAGED(1)
#undef OE_ROPE_STAGED
    return 0;
}

// ---------------------------------------------------------------------------------------
// a = g / (1 + exp(-g)) * u, with gu = [g | u] per row   (reference: core/model.cpp:638-641)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(T* out, const T* gu, int FF, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / FF, c = i % FF;
        const float g = to_f32(gu[r * 2 * FF + c]);
        const float u = to_f32(gu[r * 2 * FF + FF + c]);
        out[i] = from_f32<T>((g / (1.f + expf(-g))) * u);
    }
}

__global__ void gather_rows_f32_kernel(float* out, const float* x,
                                       const int* __restrict__ rows, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = rows[blockIdx.x];
    for (int d = threadIdx.x; d < D; d += blockDim.x)
        out[(size_t)blockIdx.x * D + d] = x[(size_t)r * D + d];
}

// ---------------------------------------------------------------------------------------
// exported entry points
// ---------------------------------------------------------------------------------------
#define LAUNCH_CHECK() return (int)cudaGetLastError()

extern "C" {

int oe_embed_gather_f32(float* x, const float* table, const int* ids, int n_tokens, int D, int vocab,
                        int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    const int launch_rc = oe_launch(embed_gather_kernel<float>, dim3(n_tokens), dim3(256), 0, st, x, table, ids, D, vocab, err);
    return launch_rc;
}
int oe_embed_gather_bf16(float* x, const bf16* table, const int* ids, int n_tokens, int D, int vocab,
                         int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    const int launch_rc = oe_launch(embed_gather_kernel<bf16>, dim3(n_tokens), dim3(256), 0, st, x, table, ids, D, vocab, err);
    return launch_rc;
}

int oe_rmsnorm_f32(float* y, const float* x, const float* w, int rows, int D, float eps, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (D % 4 == 0 && !(((uintptr_t)y | (uintptr_t)x | (uintptr_t)w) & 15))
        return oe_launch(rmsnorm_vec_kernel<float, 256>, dim3(rows), dim3(256), 0, st, y, x, w, D, eps);
    const int launch_rc = oe_launch(rmsnorm_kernel<float>, dim3(rows), dim3(256), 0, st, y, x, w, D, eps);
    return launch_rc;
}
int oe_rmsnorm_bf16(bf16* y, const float* x, const float* w, int rows, int D, float eps, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (D % 4 == 0 && !(((uintptr_t)x | (uintptr_t)w) & 15) && !((uintptr_t)y & 7)) {
        // a prompt step's rows: a warp per row (measured at 4,096 x 3072: 18.3 us with a block per row)
        if (rows >= OE_RMSNORM_ROWS_MIN && D <= 4096) {
            const dim3 grid((rows + 7) / 8);
            if (D <= 2048) return oe_launch(rmsnorm_rows_kernel<bf16, 16>, grid, dim3(256), 0, st, y, x, w, rows, D, eps);
            if (D <= 3072) return oe_launch(rmsnorm_rows_kernel<bf16, 24>, grid, dim3(256), 0, st, y, x, w, rows, D, eps);
            return oe_launch(rmsnorm_rows_kernel<bf16, 32>, grid, dim3(256), 0, st, y, x, w, rows, D, eps);
        }
        // 512 threads a row: inside the 28-layer decode step 1.4 % faster than 256 at 8 sequences (128: 4 % slower)
        return oe_launch(rmsnorm_vec_kernel<bf16, 512>, dim3(rows), dim3(512), 0, st, y, x, w, D, eps);
    }
    const int launch_rc = oe_launch(rmsnorm_kernel<bf16>, dim3(rows), dim3(256), 0, st, y, x, w, D, eps);
    return launch_rc;
}

int oe_rope_kv_write_f32(float* qkv, int row_stride, const float* cos_tab, const float* sin_tab,
                         float* cache, const int* tables, int max_pages, const int* tok_seq,
                         const int* tok_pos, int n_tokens, int H, int KVH, int hd, int has_kv, int rotate,
                         cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (hd % 2) return OE_ERR_UNSUPPORTED;
    if ((hd / 2) % 4 == 0 && row_stride % 4 == 0 && !(((uintptr_t)qkv | (uintptr_t)cache | (uintptr_t)cos_tab | (uintptr_t)sin_tab) & 15)) {
        bool done;
        const int rc = rope_staged<float>(done, qkv, row_stride, cos_tab, sin_tab, cache, tables, max_pages, tok_seq, tok_pos,
                                  n_tokens, H, KVH, hd, has_kv, rotate, st);
        if (done) return rc;
        return oe_launch(rope_kv_write_vec_kernel<float>, dim3(n_tokens), dim3(256), 0, st, qkv, row_stride, cos_tab, sin_tab,
                         cache, tables, max_pages, tok_seq, tok_pos, H, KVH, hd, has_kv, rotate);
    }
    const int launch_rc = oe_launch(rope_kv_write_kernel<float>, dim3(n_tokens), dim3(256), 0, st, qkv, row_stride, cos_tab, sin_tab, cache, tables,
                                                           max_pages, tok_seq, tok_pos, H, KVH, hd, has_kv, rotate);
    return launch_rc;
}
int oe_rope_kv_write_bf16(bf16* qkv, int row_stride, const float* cos_tab, const float* sin_tab,
                          bf16* cache, const int* tables, int max_pages, const int* tok_seq,
                          const int* tok_pos, int n_tokens, int H, int KVH, int hd, int has_kv, int rotate,
                          cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (hd % 2) return OE_ERR_UNSUPPORTED;
    if ((hd / 2) % 8 == 0 && row_stride % 8 == 0 && !(((uintptr_t)qkv | (uintptr_t)cache | (uintptr_t)cos_tab | (uintptr_t)sin_tab) & 15)) {
        bool done;
        const int rc = rope_staged<bf16>(done, qkv, row_stride, cos_tab, sin_tab, cache, tables, max_pages, tok_seq, tok_pos,
                                  n_tokens, H, KVH, hd, has_kv, rotate, st);
        if (done) return rc;
        return oe_launch(rope_kv_write_vec_kernel<bf16>, dim3(n_tokens), dim3(256), 0, st, qkv, row_stride, cos_tab, sin_tab,
                         cache, tables, max_pages, tok_seq, tok_pos, H, KVH, hd, has_kv, rotate);
    }
    const int launch_rc = oe_launch(rope_kv_write_kernel<bf16>, dim3(n_tokens), dim3(256), 0, st, qkv, row_stride, cos_tab, sin_tab, cache, tables,
                                                          max_pages, tok_seq, tok_pos, H, KVH, hd, has_kv, rotate);
    return launch_rc;
}

int oe_swiglu_f32(float* out, const float* gu, int rows, int FF, cudaStream_t st) {
    const size_t total = (size_t)rows * FF;
    if (total == 0) return 0;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    const int launch_rc = oe_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, st, out, gu, FF, total);
    return launch_rc;
}
int oe_swiglu_bf16(bf16* out, const bf16* gu, int rows, int FF, cudaStream_t st) {
    const size_t total = (size_t)rows * FF;
    if (total == 0) return 0;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    const int launch_rc = oe_launch(swiglu_kernel<bf16>, dim3(blocks), dim3(256), 0, st, out, gu, FF, total);
    return launch_rc;
}

int oe_gather_rows_f32(float* out, const float* x, const int* rows, int n_rows, int D, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    const int launch_rc = oe_launch(gather_rows_f32_kernel, dim3(n_rows), dim3(256), 0, st, out, x, rows, D);
    return launch_rc;
}

}  // extern "C"
