// Grouped-query attention of every token of a step over its sequence's paged cache:
// one code path for prompts and for single decoded tokens.
//
// One warp per (token, query head).  Keys are taken in chunks of 32 whose boundaries lie
// at absolute key positions (multiples of 32), with an online softmax in float32, so the
// result for a token depends only on its query and on the keys 0..pos of its sequence,
// not on how the tokens were cut into steps or batched.  This is the attention of the
// 32-bit path and of head sizes the tensor-core kernels do not take (any head_dim that
// is a multiple of 2 up to 256).
// Reference: core/model.cpp:411-435 (decode) and :605-626 (prefill): query head h reads
// KV head h / (H/KVH); s_t = (q.k_t)/sqrt(hd) for keys t <= pos; softmax; o = sum s_t v_t.
// `window` > 0 restricts the keys to pos-window < t <= pos (0 = all keys).
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_paged_kernel(T* out, const T* q, int q_stride,
                  const T* cache, const int* __restrict__ tables, int max_pages,
                  const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                  int n_tokens, int H, int KVH, int hd, int window, float scale) {
    extern __shared__ float qs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    float* qs = qs_all + warp * hd;
    T* o = out + (size_t)t * H * hd + (size_t)h * hd;
    const int b = tok_seq[t];
    if (b < 0) {                                   // padding row
        for (int d = lane; d < hd; d += 32) o[d] = from_f32<T>(0.f);
        return;
    }
    const int pos = tok_pos[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int kvh = h / (H / KVH);
    const int* trow = tables + (size_t)b * max_pages;
    const T* qr = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_f32(qr[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; i++) acc[i] = 0.f;

    for (int c0 = (lo / 32) * 32; c0 <= pos; c0 += 32) {
        const int key = c0 + lane;
        const bool valid = key >= lo && key <= pos;
        float s = -INFINITY;
        if (valid) {
            const long long off = page_row_offset(trow, key, 0, kvh, KVH, hd);
            if (off >= 0) {
                const T* kr = cache + off;
                float dot = 0.f;
                for (int d = 0; d < hd; d++) dot = fmaf(qs[d], to_f32(kr[d]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float alpha = expf(m - m_new);
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_HD / 32; i++) acc[i] *= alpha;
        const int jmax = (pos - c0 < 31) ? pos - c0 : 31;
        for (int j = 0; j <= jmax; j++) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (c0 + j < lo) continue;
            const long long voff = page_row_offset(trow, c0 + j, 1, kvh, KVH, hd);
            if (voff < 0) continue;
            const T* vr = cache + voff;
#pragma unroll
            for (int i = 0; i < MAX_HD / 32; i++) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; i++) {
        const int d = lane + 32 * i;
        if (d < hd) o[d] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T>
int launch(T* out, const T* q, int q_stride, const T* cache, const int* tables, int max_pages,
           const int* tok_seq, const int* tok_pos, int n_tokens, int H, int KVH, int hd, int window,
           float scale, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || hd > MAX_HD || (hd % 2) || H % KVH) return OE_ERR_UNSUPPORTED;
    const long long items = (long long)n_tokens * H;
    const long long blocks = (items + WARPS - 1) / WARPS;
    if (blocks > 2147483647LL) return OE_ERR_UNSUPPORTED;
    const int launch_rc = oe_launch(attn_paged_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), WARPS * hd * sizeof(float), st, 
        out, q, q_stride, cache, tables, max_pages, tok_seq, tok_pos, n_tokens, H, KVH, hd, window, scale);
    return launch_rc;
}

}  // namespace

extern "C" {
int oe_attn_paged_f32(float* out, const float* q, int q_stride, const float* cache, const int* tables,
                      int max_pages, const int* tok_seq, const int* tok_pos, int n_tokens, int H, int KVH,
                      int hd, int window, float scale, cudaStream_t st) {
    return launch<float>(out, q, q_stride, cache, tables, max_pages, tok_seq, tok_pos, n_tokens, H, KVH, hd,
                         window, scale, st);
}
int oe_attn_paged_bf16(bf16* out, const bf16* q, int q_stride, const bf16* cache, const int* tables,
                       int max_pages, const int* tok_seq, const int* tok_pos, int n_tokens, int H, int KVH,
                       int hd, int window, float scale, cudaStream_t st) {
    return launch<bf16>(out, q, q_stride, cache, tables, max_pages, tok_seq, tok_pos, n_tokens, H, KVH, hd,
                        window, scale, st);
}
}
