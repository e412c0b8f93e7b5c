// Token selection on the device: first-maximum argmax, and the reference's sampling
// chain  repeat penalty -> temperature -> softmax -> top-k -> top-p -> draw
// (core/sampler.cpp:15-27, 35-39, 48-86, 91-97), one block per row of float32 logits.
//
// Differences from the reference, on purpose:
//  * the draw is one uniform per (sequence, draw number) from a counter-based generator
//    kept in the per-sequence state (the reference seeds std::mt19937 from the clock,
//    core/engine.cpp:109-111), and the kept tokens are walked in index order, which gives
//    the same distribution as walking them by probability;
//  * top-k and top-p are applied as probability thresholds found by bisection over the
//    bit patterns, so tokens whose probability equals the cut exactly are all kept.
// The logits row is overwritten (the reference's sampler also works in place).
#include "common.cuh"

namespace {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ float uniform_from_counter(unsigned long long seed, unsigned long long counter) {
    unsigned long long z = seed + (counter + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// First maximum of a row (strict >, lowest index wins ties; core/ops.cpp:490-497).
__device__ int block_argmax(const float* x, int V, float* s_val, int* s_idx) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = x[i];
        if (v > best || bi == 0x7fffffff) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = lane < nw ? s_val[lane] : -INFINITY;
        bi = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) s_idx[0] = bi;
    }
    __syncthreads();
    const int r = s_idx[0];
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_rows_kernel(const float* logits, int* out, int V) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = block_argmax(logits + (size_t)blockIdx.x * V, V, s_val, s_idx);
    if (threadIdx.x == 0) out[blockIdx.x] = r;
}

// Two-stage first-maximum for wide rows: each block takes one slice of a row, then one warp
// per row combines the slices (lowest index wins ties, as in block_argmax).
constexpr int ARGMAX_SLICES = 32;

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* logits, float* part_val, int* part_idx, int V) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y, slice = blockIdx.x;
    const int per = (V + ARGMAX_SLICES - 1) / ARGMAX_SLICES;
    const int lo = slice * per, hi = min(V, lo + per);
    const float* x = logits + (size_t)row * V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = x[i];
        if (v > best || bi == 0x7fffffff) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = lane < (int)(blockDim.x >> 5) ? s_val[lane] : -INFINITY;
        bi = lane < (int)(blockDim.x >> 5) ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) { part_val[row * ARGMAX_SLICES + slice] = best; part_idx[row * ARGMAX_SLICES + slice] = bi; }
    }
}

__global__ void argmax_final_kernel(const float* part_val, const int* part_idx, int* out) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, lane = threadIdx.x;
    float best = part_val[row * ARGMAX_SLICES + lane];
    int bi = part_idx[row * ARGMAX_SLICES + lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) out[row] = bi;
}

struct SampleState {
    const long long* rng_seed;   // [slots]
    int* rng_counter;            // [slots] draws made so far
    int* hist;                   // [slots, hist_cap] ring of recorded tokens
    int* hist_count;             // [slots] tokens recorded so far
    int hist_cap;
};

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(float* __restrict__ logits, int* __restrict__ out, const int* __restrict__ row_slot,
                   int V, float temperature, int top_k, float top_p, float repeat_pen, int repeat_last,
                   SampleState st, int record) {
    __shared__ float red[32];
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ float s_scan[SAMPLE_THREADS];
    __shared__ int s_pick;
    pdl_launch_dependents();
    pdl_wait();
    const int slot = row_slot[blockIdx.x];
    if (slot < 0) { if (threadIdx.x == 0) out[blockIdx.x] = -1; return; }
    float* x = logits + (size_t)blockIdx.x * V;
    const int tid = threadIdx.x;

    // 1. repeat penalty over the last `repeat_last` recorded tokens, in order
    if (repeat_pen > 1.f && st.hist != nullptr) {
        if (tid == 0) {
            const int count = st.hist_count[slot];
            int n = count < repeat_last ? count : repeat_last;
            if (n > st.hist_cap) n = st.hist_cap;
            const int* ring = st.hist + (size_t)slot * st.hist_cap;
            for (int j = count - n; j < count; j++) {
                const int id = ring[j % st.hist_cap];
                if (id < 0 || id >= V) continue;
                const float v = x[id];
                x[id] = v > 0.f ? v / repeat_pen : v * repeat_pen;
            }
        }
        __syncthreads();
    }

    int token;
    if (temperature <= 0.f) {
        token = block_argmax(x, V, s_val, s_idx);
    } else {
        // 2. temperature, 3. softmax (probabilities stored in place)
        const float inv_t = (temperature == 1.f) ? 1.f : 1.f / temperature;
        float mx = -INFINITY;
        for (int i = tid; i < V; i += blockDim.x) { const float v = x[i] * inv_t; x[i] = v; mx = fmaxf(mx, v); }
        mx = block_max(mx, red);
        float sum = 0.f;
        for (int i = tid; i < V; i += blockDim.x) { const float e = expf(x[i] - mx); x[i] = e; sum += e; }
        sum = block_sum(sum, red);
        const float inv = 1.f / sum;
        for (int i = tid; i < V; i += blockDim.x) x[i] *= inv;
        __syncthreads();

        // 4. top-k: largest threshold with at least k probabilities at or above it
        unsigned thr = 0u;
        if (top_k > 0 && top_k < V) {
            for (int bit = 30; bit >= 0; bit--) {
                const unsigned cand = thr | (1u << bit);
                float cnt = 0.f;
                for (int i = tid; i < V; i += blockDim.x) cnt += (__float_as_uint(x[i]) >= cand) ? 1.f : 0.f;
                cnt = block_sum(cnt, red);
                if (cnt >= (float)top_k) thr = cand;
            }
        }
        // 5. top-p within those: largest threshold whose kept mass reaches top_p
        if (top_p < 1.f) {
            unsigned thp = 0u;
            for (int bit = 30; bit >= 0; bit--) {
                const unsigned cand = thp | (1u << bit);
                const unsigned eff = cand > thr ? cand : thr;
                float mass = 0.f;
                for (int i = tid; i < V; i += blockDim.x) mass += (__float_as_uint(x[i]) >= eff) ? x[i] : 0.f;
                mass = block_sum(mass, red);
                if (mass >= top_p) thp = cand;
            }
            if (thp > thr) thr = thp;
        }
        // 6. draw: first kept index (ascending) whose running mass exceeds u * kept mass
        const int chunk = (V + blockDim.x - 1) / blockDim.x;
        const int i0 = tid * chunk, i1 = (i0 + chunk < V) ? i0 + chunk : V;
        float local = 0.f;
        for (int i = i0; i < i1; i++) local += (__float_as_uint(x[i]) >= thr) ? x[i] : 0.f;
        s_scan[tid] = local;
        if (tid == 0) s_pick = -1;
        __syncthreads();
        if (tid == 0) {
            float run = 0.f;
            for (int t = 0; t < (int)blockDim.x; t++) { const float v = s_scan[t]; s_scan[t] = run; run += v; }
            red[0] = run;
        }
        __syncthreads();
        const float total = red[0];
        const float u = uniform_from_counter((unsigned long long)st.rng_seed[slot],
                                             (unsigned long long)st.rng_counter[slot]);
        const float r = u * total;
        const float excl = s_scan[tid];
        const float next = (tid + 1 < (int)blockDim.x) ? s_scan[tid + 1] : total;
        if (local > 0.f && excl <= r && r < next) {
            float run = excl;
            int pick = -1, last = -1;
            for (int i = i0; i < i1; i++) {
                if (__float_as_uint(x[i]) >= thr) {
                    last = i;
                    run += x[i];
                    if (run > r) { pick = i; break; }
                }
            }
            s_pick = pick >= 0 ? pick : last;
        }
        __syncthreads();
        if (s_pick < 0) {
            // r fell at or beyond the total through rounding: the last kept index
            int last = -1;
            for (int i = i0; i < i1; i++) if (__float_as_uint(x[i]) >= thr && x[i] > 0.f) last = i;
            if (last >= 0) atomicMax(&s_pick, last);
            __syncthreads();
        }
        token = s_pick;
    }
    if (tid == 0) {
        out[blockIdx.x] = token;
        if (record) {
            if (temperature > 0.f) st.rng_counter[slot] += 1;
            if (st.hist != nullptr) {
                const int c = st.hist_count[slot];
                st.hist[(size_t)slot * st.hist_cap + (c % st.hist_cap)] = token;
                st.hist_count[slot] = c + 1;
            }
        }
    }
}

}  // namespace

extern "C" {

// Wide rows in two stages; scratch: rows * 32 floats and rows * 32 ints.
int oe_argmax_rows_wide(const float* logits, int* out, float* part_val, int* part_idx, int rows, int V, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (V <= 0 || rows > 65535) return OE_ERR_UNSUPPORTED;
    int rc = oe_launch(argmax_partial_kernel, dim3(ARGMAX_SLICES, rows), dim3(256), 0, st, logits, part_val, part_idx, V);
    if (rc) return rc;
    return oe_launch(argmax_final_kernel, dim3(rows), dim3(32), 0, st, (const float*)part_val, (const int*)part_idx, out);
}

int oe_argmax_rows(const float* logits, int* out, int rows, int V, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (V <= 0) return OE_ERR_UNSUPPORTED;
    const int launch_rc = oe_launch(argmax_rows_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, st, logits, out, V);
    return launch_rc;
}

int oe_sample_rows(float* logits, int* out, const int* row_slot, int rows, int V, float temperature,
                   int top_k, float top_p, float repeat_pen, int repeat_last, const long long* rng_seed,
                   int* rng_counter, int* hist, int* hist_count, int hist_cap, int record,
                   cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0 || (hist != nullptr && hist_cap <= 0)) return OE_ERR_UNSUPPORTED;
    SampleState st{rng_seed, rng_counter, hist, hist_count, hist_cap};
    const int launch_rc = oe_launch(sample_rows_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, out, row_slot, V, temperature, top_k, top_p,
                                                            repeat_pen, repeat_last, st, record);
    return launch_rc;
}

}  // extern "C"
