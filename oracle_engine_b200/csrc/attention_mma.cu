// bf16 grouped-query attention over the paged cache on the tensor cores, for prompts
// (causal, ragged batches) and for decoded tokens (split over the keys), compiled for one
// head size: -DOE_HD=<head_dim>, a multiple of 16 up to 256.
//
// A CTA works on one (sequence, KV head) and a tile of query rows; a row is a (token,
// query head of the group) pair, so the G = H/KVH query heads that share a KV head also
// share every K/V tile the CTA loads.  Each warp owns 16 rows.  Key blocks are cache
// pages (64 keys): a page's K and V panels are contiguous [64][head_dim] and are staged
// in shared memory with cp.async, double buffered.  S = Q K^T and O += P V run on
// mma.sync m16n8k16 (bf16 in, float32 accumulate) with ldmatrix fragments; the softmax is
// online, in float32 (running maximum and sum per row).  Causal mask: key <= the row's
// absolute position; window > 0 keeps only the last `window` keys.
// For decoded tokens the page range of a sequence is split over `n_splits` CTAs; each
// writes an unnormalised partial (o, m, l) and attn_merge_kernel combines them in split
// order.
// Reference: core/model.cpp:411-435 and :605-626 (scores, softmax, weighted values).
#include "common.cuh"

#ifndef OE_HD
#define OE_HD 128
#endif

namespace {

constexpr int HD = OE_HD;
constexpr int BN = OE_PAGE;                     // keys per block = one page
constexpr int ROW_BYTES = HD * 2 + 16;          // padded row: ldmatrix without bank conflicts
constexpr int TILE_BYTES = BN * ROW_BYTES;
constexpr int KS = HD / 16;                     // k-steps of Q K^T; pairs of 8-wide output tiles of P V
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head_dim must be a multiple of 16 up to 256");

struct AttnArgs {
    bf16* out;                 // [T, H*HD]
    const bf16* q;             // rows of q_stride elements, head h at h*HD
    long long q_stride;
    const bf16* cache;         // one cache entry [pages][2][KVH][64][HD]
    const int* tables;         // [B, max_pages]
    int max_pages;
    const int* cu_q;           // [B+1] first packed row of each sequence
    const int* seq_start;      // [B] cache length before the step
    const int* seq_qlen;       // [B]
    int H, KVH, window;
    float scale_log2;          // scale * log2(e)
    int tokens_per_tile;
    int n_splits;
    float* partial;            // [T, H, n_splits, HD + 2] when n_splits > 1
    // fused decode (every sequence brings one token): q is the raw fused qkv row, the kernel
    // rotates q (and the new k) itself, writes the new k, v to the cache and the CTA that
    // finishes last merges the splits
    int fused;
    const float* cos_tab;      // [max_pos, HD/2] or null (no rotation)
    const float* sin_tab;
    bf16* cache_w;             // the cache entry, writable, when this call stores the new k, v; else null
    int* counters;             // [B * KVH] zeros (n_splits > 1)
    int stages;                // K/V tiles staged ahead: 2 (double buffer) or 1
    int cluster;               // warps kernel: CTAs (a thread-block cluster) that share one (sequence, KV head)
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&h;
}

// Stages the K and V panels of `page` for KV head `kvh` into shared memory.
template <int NTHREADS>
__device__ __forceinline__ void load_page(uint8_t* ks, uint8_t* vs, const bf16* cache, int page, int kvh, int KVH) {
    const bf16* kg = cache + (((size_t)page * 2 + 0) * KVH + kvh) * (size_t)(BN * HD);
    const bf16* vg = cache + (((size_t)page * 2 + 1) * KVH + kvh) * (size_t)(BN * HD);
    constexpr int CHUNKS = BN * HD / 8;                 // 16-byte chunks per panel
    for (int c = threadIdx.x; c < CHUNKS; c += NTHREADS) {
        const int row = c / (HD / 8), col = c % (HD / 8);
        cp_async16(ks + row * ROW_BYTES + col * 16, kg + (size_t)c * 8);
        cp_async16(vs + row * ROW_BYTES + col * 16, vg + (size_t)c * 8);
    }
}

template <int NWARPS, int STAGES>
__global__ void __launch_bounds__(NWARPS * 32, NWARPS == 4 ? 2 : 1)
attn_mma_kernel(const AttnArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_launch_dependents();
    // The kernel before this one (or, for a layer that reads another layer's cache, an earlier
    // one) wrote this step's keys and values into the cache, unless this kernel writes them
    // itself; see below.
    const bool own_kv = a.fused && a.cache_w != nullptr;
    if (!own_kv) pdl_wait();
    const int b = blockIdx.z, kvh = blockIdx.y;
    const int qlen = a.seq_qlen[b];
    if (qlen <= 0) {
        // a padding sequence: like every CTA of this kernel it leaves only after the kernel before has
        // finished (CTAs that left at once made the decode step of 5 to 7 sequences, padded to 8, 15 %
        // slower than that of 8)
        if (own_kv) pdl_wait();
        return;
    }
    const int start = a.seq_start[b];
    const int G = a.H / a.KVH;
    const int tpt = a.tokens_per_tile;
    const int n_q_tiles = (qlen + tpt - 1) / tpt;
    const int q_tile = a.n_splits > 1 ? 0 : blockIdx.x;
    const int split = a.n_splits > 1 ? blockIdx.x : 0;
    if (q_tile >= n_q_tiles) {
        if (own_kv) pdl_wait();                  // as above
        return;
    }
    const int t0 = q_tile * tpt;
    const int nt = min(tpt, qlen - t0);
    const int pos_lo = start + t0, pos_hi = start + t0 + nt - 1;
    const int key_lo = a.window > 0 ? max(0, pos_lo - a.window + 1) : 0;
    int j_lo = key_lo / BN, j_hi = pos_hi / BN;
    if (a.n_splits > 1) {
        const int per = (j_hi - j_lo + a.n_splits) / a.n_splits;
        j_lo = j_lo + split * per;
        j_hi = min(j_hi, j_lo + per - 1);
    }
    const int* trow = a.tables + (size_t)b * a.max_pages;
    const int n_blocks = j_hi - j_lo + 1;
    if (own_kv) {
        // The first tile holds keys and values of earlier steps (and the stale row of the new
        // token, replaced below): its load overlaps the end of the kernel before this one, from
        // which only the new token's q, k and v come.
        if (n_blocks > 0) load_page<NWARPS * 32>(smem, smem + TILE_BYTES, a.cache, trow[j_lo], kvh, a.KVH);
        cp_async_commit();
        pdl_wait();
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int row0 = warp * 16 + gid;                   // this thread's rows: row0 and row0 + 8
    const long long packed0 = a.cu_q[b] + t0;

    int tok[2], pos[2], head[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = row0 + i * 8;
        tok[i] = r / G;
        head[i] = kvh * G + r % G;
        valid[i] = tok[i] < nt;
        pos[i] = start + t0 + tok[i];
    }

    // Q fragments (A operand), kept in registers for the whole kernel
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (valid[i]) {
                const bf16* qr = a.q + (packed0 + tok[i]) * a.q_stride + (size_t)head[i] * HD + ks * 16 + tig * 2;
                qf[ks][i] = *(const uint32_t*)qr;
                qf[ks][i + 2] = *(const uint32_t*)(qr + 8);
            } else {
                qf[ks][i] = 0u;
                qf[ks][i + 2] = 0u;
            }
        }
    }

    if (a.fused && a.cos_tab != nullptr) {
        // rotate-half pairs (d, d + HD/2) sit in the same lane, KS/2 k-steps apart
#pragma unroll
        for (int ks = 0; ks < KS / 2; ks++) {
#pragma unroll
            for (int x = 0; x < 4; x++) {
                const int i = x & 1;
                const int d = ks * 16 + tig * 2 + (x >> 1) * 8;
                const float2 cs = *(const float2*)(a.cos_tab + (size_t)pos[i] * (HD / 2) + d);
                const float2 sn = *(const float2*)(a.sin_tab + (size_t)pos[i] * (HD / 2) + d);
                const __nv_bfloat162 lo = *(__nv_bfloat162*)&qf[ks][x];
                const __nv_bfloat162 hi = *(__nv_bfloat162*)&qf[ks + KS / 2][x];
                const float x0a = __low2float(lo), x0b = __high2float(lo), x1a = __low2float(hi), x1b = __high2float(hi);
                qf[ks][x] = pack_bf16(x0a * cs.x - x1a * sn.x, x0b * cs.y - x1b * sn.y);
                qf[ks + KS / 2][x] = pack_bf16(x0a * sn.x + x1a * cs.x, x0b * sn.y + x1b * cs.y);
            }
        }
    }

    float oacc[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; n++) { oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    if (!own_kv) {
        if (n_blocks > 0) load_page<NWARPS * 32>(smem, smem + TILE_BYTES, a.cache, trow[j_lo], kvh, a.KVH);
        cp_async_commit();
    }
    for (int it = 0; it < n_blocks; it++) {
        const int j = j_lo + it;
        constexpr bool dbl = STAGES > 1;
        uint8_t* ks_cur = smem + (size_t)(dbl ? (it & 1) : 0) * 2 * TILE_BYTES;
        uint8_t* vs_cur = ks_cur + TILE_BYTES;
        if (dbl && it + 1 < n_blocks) {
            uint8_t* nxt = smem + (size_t)((it + 1) & 1) * 2 * TILE_BYTES;
            load_page<NWARPS * 32>(nxt, nxt + TILE_BYTES, a.cache, trow[j + 1], kvh, a.KVH);
        }
        cp_async_commit();
        if (dbl) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();

        if (a.fused && a.cache_w != nullptr && j == pos_hi / BN) {
            // this CTA holds the page of the new token: rotate its key, store key and value
            // in the cache, and put them into the staged tile as well
            const int r = pos_hi % BN;
            const bf16* krow = a.q + packed0 * a.q_stride + (size_t)(a.H + kvh) * HD;
            const bf16* vrow = krow + (size_t)a.KVH * HD;
            const size_t page = (size_t)trow[j];
            bf16* kc = a.cache_w + ((page * 2 + 0) * a.KVH + kvh) * (size_t)(BN * HD) + (size_t)r * HD;
            bf16* vc = a.cache_w + ((page * 2 + 1) * a.KVH + kvh) * (size_t)(BN * HD) + (size_t)r * HD;
            bf16* ksm = (bf16*)(ks_cur + r * ROW_BYTES);
            bf16* vsm = (bf16*)(vs_cur + r * ROW_BYTES);
            for (int d = threadIdx.x; d < HD / 2; d += blockDim.x) {
                float k0 = __bfloat162float(krow[d]), k1 = __bfloat162float(krow[d + HD / 2]);
                if (a.cos_tab != nullptr) {
                    const float c = a.cos_tab[(size_t)pos_hi * (HD / 2) + d], sn = a.sin_tab[(size_t)pos_hi * (HD / 2) + d];
                    const float r0 = k0 * c - k1 * sn, r1 = k0 * sn + k1 * c;
                    k0 = r0; k1 = r1;
                }
                const bf16 b0 = __float2bfloat16_rn(k0), b1 = __float2bfloat16_rn(k1);
                const bf16 v0 = vrow[d], v1 = vrow[d + HD / 2];
                kc[d] = b0; kc[d + HD / 2] = b1; ksm[d] = b0; ksm[d + HD / 2] = b1;
                vc[d] = v0; vc[d + HD / 2] = v1; vsm[d] = v0; vsm[d + HD / 2] = v1;
            }
            __syncthreads();
        }

        // S = Q K^T for this warp's 16 rows and the block's 64 keys
        float sacc[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; n++) { sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f; }
        {
            // K fragments of the next k-step are loaded while the current one multiplies
            const int m = lane >> 3, r = lane & 7;
            const uint8_t* kbase = ks_cur + ((m >> 1) * 8 + r) * ROW_BYTES + (m & 1) * 16;
            uint32_t kb[2][BN / 16][4];
#pragma unroll
            for (int np = 0; np < BN / 16; np++) ldmatrix_x4(kb[0][np], kbase + np * 16 * ROW_BYTES);
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                if (ks + 1 < KS) {
#pragma unroll
                    for (int np = 0; np < BN / 16; np++)
                        ldmatrix_x4(kb[(ks + 1) & 1][np], kbase + np * 16 * ROW_BYTES + (ks + 1) * 32);
                }
#pragma unroll
                for (int np = 0; np < BN / 16; np++) {
                    mma_bf16(sacc[2 * np], qf[ks], kb[ks & 1][np][0], kb[ks & 1][np][1]);
                    mma_bf16(sacc[2 * np + 1], qf[ks], kb[ks & 1][np][2], kb[ks & 1][np][3]);
                }
            }
        }
        // scale, mask, online softmax
        float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < BN / 8; n++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = e >> 1;
                const int key = j * BN + n * 8 + tig * 2 + (e & 1);
                const bool ok = valid[i] && key <= pos[i] && (a.window <= 0 || key > pos[i] - a.window);
                const float s = ok ? sacc[n][e] * a.scale_log2 : -INFINITY;
                sacc[n][e] = s;
                rmax[i] = fmaxf(rmax[i], s);
            }
        }
        float alpha[2], m_use[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            rmax[i] = fmaxf(rmax[i], __shfl_xor_sync(0xffffffffu, rmax[i], 1));
            rmax[i] = fmaxf(rmax[i], __shfl_xor_sync(0xffffffffu, rmax[i], 2));
            const float m_new = fmaxf(m_run[i], rmax[i]);
            m_use[i] = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[i] = exp2f(m_run[i] - m_use[i]);
            m_run[i] = m_new;
        }
        float rsum[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < BN / 8; n++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = exp2f(sacc[n][e] - m_use[e >> 1]);
                sacc[n][e] = p;
                rsum[e >> 1] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < 2; i++) l_run[i] = l_run[i] * alpha[i] + rsum[i];
#pragma unroll
        for (int n = 0; n < HD / 8; n++) {
            oacc[n][0] *= alpha[0]; oacc[n][1] *= alpha[0];
            oacc[n][2] *= alpha[1]; oacc[n][3] *= alpha[1];
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < BN / 16; kk++) {
            uint32_t pa[4];
            pa[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
            pa[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
            pa[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
            pa[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
            {
                const int m = lane >> 3, r = lane & 7;
                const uint8_t* vbase = vs_cur + (kk * 16 + (m & 1) * 8 + r) * ROW_BYTES + (m >> 1) * 16;
                uint32_t vb[2][4];
                ldmatrix_x4_trans(vb[0], vbase);
#pragma unroll
                for (int dp = 0; dp < KS; dp++) {
                    if (dp + 1 < KS) ldmatrix_x4_trans(vb[(dp + 1) & 1], vbase + (dp + 1) * 32);
                    mma_bf16(oacc[2 * dp], pa, vb[dp & 1][0], vb[dp & 1][1]);
                    mma_bf16(oacc[2 * dp + 1], pa, vb[dp & 1][2], vb[dp & 1][3]);
                }
            }
        }
        __syncthreads();
        if (!dbl && it + 1 < n_blocks)
            load_page<NWARPS * 32>(smem, smem + TILE_BYTES, a.cache, trow[j + 1], kvh, a.KVH);
    }
    cp_async_wait<0>();

#pragma unroll
    for (int i = 0; i < 2; i++) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    if (a.n_splits <= 1) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (!valid[i]) continue;
            const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
            bf16* o = a.out + (packed0 + tok[i]) * (long long)(a.H * HD) + (size_t)head[i] * HD + tig * 2;
#pragma unroll
            for (int n = 0; n < HD / 8; n++)
                *(uint32_t*)(o + n * 8) = pack_bf16(oacc[n][2 * i] * inv, oacc[n][2 * i + 1] * inv);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (!valid[i]) continue;
            float* p = a.partial + (((packed0 + tok[i]) * a.H + head[i]) * a.n_splits + split) * (long long)(HD + 2);
#pragma unroll
            for (int n = 0; n < HD / 8; n++) {
                p[n * 8 + tig * 2] = oacc[n][2 * i];
                p[n * 8 + tig * 2 + 1] = oacc[n][2 * i + 1];
            }
            if (tig == 0) { p[HD] = m_run[i]; p[HD + 1] = l_run[i]; }
        }
        if (a.fused) {
            // the CTA of this (sequence, KV head) that finishes last merges the splits, in split order
            __shared__ int s_last;
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) s_last = (atomicAdd(&a.counters[b * a.KVH + kvh], 1) == a.n_splits - 1) ? 1 : 0;
            __syncthreads();
            if (s_last) {
                __threadfence();
                // weights of every (head, split) first, then all value loads of a thread at once
                float* s_m = (float*)(smem + (size_t)STAGES * 2 * TILE_BYTES);
                float* s_l = s_m + 64 * 32;
                const int ns = a.n_splits;
                const float* pbase = a.partial + ((packed0 * a.H + (long long)kvh * G) * ns) * (long long)(HD + 2);
                for (int idx = threadIdx.x; idx < G * ns; idx += blockDim.x) {
                    s_m[idx] = __ldcg(pbase + (size_t)idx * (HD + 2) + HD);
                    s_l[idx] = __ldcg(pbase + (size_t)idx * (HD + 2) + HD + 1);
                }
                __syncthreads();
                for (int gh = threadIdx.x; gh < G; gh += blockDim.x) {
                    float m = -INFINITY, l = 0.f;
                    for (int sp = 0; sp < ns; sp++) m = fmaxf(m, s_m[gh * ns + sp]);
                    for (int sp = 0; sp < ns; sp++)
                        if (s_m[gh * ns + sp] != -INFINITY) l += s_l[gh * ns + sp] * exp2f(s_m[gh * ns + sp] - m);
                    const float inv = l > 0.f ? 1.f / l : 0.f;
                    for (int sp = 0; sp < ns; sp++)
                        s_l[gh * ns + sp] = (s_m[gh * ns + sp] != -INFINITY) ? exp2f(s_m[gh * ns + sp] - m) * inv : 0.f;
                }
                __syncthreads();
                bf16* obase = a.out + packed0 * (long long)(a.H * HD) + (size_t)kvh * G * HD;
                const int total = G * HD;
                for (int i0 = threadIdx.x; i0 < total; i0 += 4 * blockDim.x) {
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int idx = i0 + u * blockDim.x;
                        if (idx < total) {
                            const int gh = idx / HD, d = idx % HD;
#pragma unroll 8
                            for (int sp = 0; sp < ns; sp++)
                                acc[u] += s_l[gh * ns + sp] * __ldcg(pbase + (size_t)(gh * ns + sp) * (HD + 2) + d);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int idx = i0 + u * blockDim.x;
                        if (idx < total) obase[idx] = __float2bfloat16_rn(acc[u]);
                    }
                }
                if (threadIdx.x == 0) a.counters[b * a.KVH + kvh] = 0;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Decoded tokens, one CTA per (sequence, KV head), the WARPS of the CTA split the keys.
// Every warp holds the same 16 query rows (the G heads of the group for the one new token),
// walks half pages (32 keys) warp, warp + NW, ... of the sequence through a double buffer of
// its own (cp.async, no CTA-wide barrier in the loop) and keeps its own running softmax; at
// the end the warps' partial results are added in warp order through shared memory.  The
// kernel also rotates q and the new token's k and writes k and v to the cache (as the fused
// path of attn_mma_kernel does), so a decode step needs one attention launch and no scratch
// in global memory.  For batches whose (sequence, KV head) pairs alone give enough CTAs.
// ---------------------------------------------------------------------------------------
constexpr int TB = 32;                          // keys per tile of a warp
constexpr int TB_BYTES = TB * ROW_BYTES;
constexpr int WARP_STAGE_BYTES = 2 * TB_BYTES;  // K and V

__device__ __forceinline__ void load_half_page(uint8_t* ks, uint8_t* vs, const bf16* cache, int page, int half, int kvh, int KVH, int lane) {
    const bf16* kg = cache + (((size_t)page * 2 + 0) * KVH + kvh) * (size_t)(BN * HD) + (size_t)half * TB * HD;
    const bf16* vg = cache + (((size_t)page * 2 + 1) * KVH + kvh) * (size_t)(BN * HD) + (size_t)half * TB * HD;
    constexpr int CHUNKS = TB * HD / 8;
#pragma unroll
    for (int c0 = 0; c0 < CHUNKS; c0 += 32) {
        const int c = c0 + lane;
        const int row = c / (HD / 8), col = c % (HD / 8);
        cp_async16(ks + row * ROW_BYTES + col * 16, kg + (size_t)c * 8);
        cp_async16(vs + row * ROW_BYTES + col * 16, vg + (size_t)c * 8);
    }
}

// NW warps, each with a ring of ST tiles: ST - 1 tiles of every warp are on their way from memory
// while one is multiplied.  What a kernel like this streams is (bytes in flight) / (memory
// latency), so the ring is as deep as shared memory allows: few warps with deep rings where many
// CTAs share an SM (a large batch), many warps where a CTA has an SM to itself.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Every thread of every CTA of the cluster calls it.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// A float at this CTA's shared-memory address `p`, read from the CTA of rank `rank` of the cluster.
__device__ __forceinline__ float ld_peer_f32(const float* p, uint32_t rank) {
    uint32_t addr;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"((uint32_t)__cvta_generic_to_shared(p)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

template <int NW, int ST>
__global__ void __launch_bounds__(NW * 32, 1)
attn_decode_warps_kernel(const AttnArgs a) {
    constexpr int WARP_BYTES = ST * WARP_STAGE_BYTES;
    static_assert(ST >= 2 && (NW + 1) * 16 * (HD + 2) * 4 <= NW * WARP_BYTES, "the merge scratch shares the staging buffers");
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_launch_dependents();
    // A layer that reads another layer's cache finds the new token's key there, written by an
    // earlier kernel of this step: it waits first.  Otherwise this kernel writes that key itself.
    const bool own_kv = a.cache_w != nullptr;
    if (!own_kv) pdl_wait();
    const int b = blockIdx.z, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int G = a.H / a.KVH;
    const int qlen = a.seq_qlen[b];
    const long long packed0 = a.cu_q[b];
    if (qlen <= 0) {
        // A padding sequence: its row is never read.  Like every CTA of this kernel it leaves only after
        // the kernel before has finished: with padding CTAs that left at once the decode step of 5 to 7
        // sequences (padded to 8) took 1.98-2.04 ms against 1.72 ms for 8; with the wait 1.69-1.70 ms.
        if (own_kv) pdl_wait();
        return;
    }
    const int pos = a.seq_start[b];                          // the new token's position
    const int key_lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int hp_lo = key_lo / TB, hp_hi = pos / TB;
    const int* trow = a.tables + (size_t)b * a.max_pages;
    uint8_t* mine = smem + (size_t)warp * WARP_BYTES;
    // Few sequences with long contexts: the CTAs of a thread-block cluster (gridDim.x of them) share the
    // pair's tiles, warp gw of NW x CR taking every (NW x CR)-th, and rank 0 adds up through the
    // cluster's shared memory: twice or four times the SMs stream one sequence's keys.
    const int CR = a.cluster, rank = CR > 1 ? (int)cluster_ctarank() : 0;
    const int gw = rank * NW + warp, stride = NW * CR;

    // this warp's first tiles are requested before anything else
    const int n_my = hp_lo + gw <= hp_hi ? (hp_hi - hp_lo - gw) / stride + 1 : 0;
    // (the whole ring: nothing is being multiplied yet)
#pragma unroll
    for (int pre = 0; pre < ST; pre++) {
        if (pre < n_my) {
            const int hp = hp_lo + gw + pre * stride;
            uint8_t* st = mine + (size_t)pre * WARP_STAGE_BYTES;
            load_half_page(st, st + TB_BYTES, a.cache, trow[hp >> 1], hp & 1, kvh, a.KVH, lane);
        }
        cp_async_commit();
    }
    // Up to here only the step's tables and keys and values of earlier steps were read, which no
    // kernel of this step writes (the stale row of the new token is replaced below): those loads
    // overlap the end of the kernel before this one.  The new token's q, k and v come from that kernel.
    if (own_kv) pdl_wait();

    // The warp that will meet the new token's tile asks for that token's k and v now, with q, rotates
    // the key and stores both in the cache; the values wait in registers for the tile.
    constexpr int NEW_IT = (HD / 2 + 31) / 32;
    const bool owner = a.cache_w != nullptr && n_my > 0 && (hp_hi - hp_lo - gw) % stride == 0;
    bf16 new_k0[NEW_IT], new_k1[NEW_IT], new_v0[NEW_IT], new_v1[NEW_IT];
    if (owner) {
        const bf16* krow = a.q + packed0 * a.q_stride + (size_t)(a.H + kvh) * HD;
        const bf16* vrow = krow + (size_t)a.KVH * HD;
        float kf0[NEW_IT], kf1[NEW_IT], cs[NEW_IT], sn[NEW_IT];
#pragma unroll
        for (int u = 0; u < NEW_IT; u++) {
            const int d = lane + u * 32;
            if (d < HD / 2) {
                kf0[u] = __bfloat162float(krow[d]); kf1[u] = __bfloat162float(krow[d + HD / 2]);
                new_v0[u] = vrow[d]; new_v1[u] = vrow[d + HD / 2];
                cs[u] = a.cos_tab != nullptr ? a.cos_tab[(size_t)pos * (HD / 2) + d] : 1.f;
                sn[u] = a.cos_tab != nullptr ? a.sin_tab[(size_t)pos * (HD / 2) + d] : 0.f;
            }
        }
        const size_t page = (size_t)trow[pos / BN];
        bf16* kc = a.cache_w + ((page * 2 + 0) * a.KVH + kvh) * (size_t)(BN * HD) + (size_t)(pos % BN) * HD;
        bf16* vc = a.cache_w + ((page * 2 + 1) * a.KVH + kvh) * (size_t)(BN * HD) + (size_t)(pos % BN) * HD;
#pragma unroll
        for (int u = 0; u < NEW_IT; u++) {
            const int d = lane + u * 32;
            if (d < HD / 2) {
                float k0 = kf0[u], k1 = kf1[u];
                if (a.cos_tab != nullptr) {
                    const float r0 = k0 * cs[u] - k1 * sn[u], r1 = k0 * sn[u] + k1 * cs[u];
                    k0 = r0; k1 = r1;
                }
                new_k0[u] = __float2bfloat16_rn(k0); new_k1[u] = __float2bfloat16_rn(k1);
                kc[d] = new_k0[u]; kc[d + HD / 2] = new_k1[u];
                vc[d] = new_v0[u]; vc[d + HD / 2] = new_v1[u];
            }
        }
    }

    bool valid[2];
    int head[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = gid + i * 8;
        valid[i] = r < G;
        head[i] = kvh * G + (valid[i] ? r : 0);
    }
    // Q fragments (A operand): rows gid and gid + 8 are heads of the group
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (valid[i]) {
                const bf16* qr = a.q + packed0 * a.q_stride + (size_t)head[i] * HD + ks * 16 + tig * 2;
                qf[ks][i] = *(const uint32_t*)qr;
                qf[ks][i + 2] = *(const uint32_t*)(qr + 8);
            } else {
                qf[ks][i] = 0u;
                qf[ks][i + 2] = 0u;
            }
        }
    }
    if (a.cos_tab != nullptr) {
        // rotate-half pairs (d, d + HD/2) sit in the same lane, KS/2 k-steps apart
#pragma unroll
        for (int ks = 0; ks < KS / 2; ks++) {
#pragma unroll
            for (int x = 0; x < 4; x++) {
                const int d = ks * 16 + tig * 2 + (x >> 1) * 8;
                const float2 cs = *(const float2*)(a.cos_tab + (size_t)pos * (HD / 2) + d);
                const float2 sn = *(const float2*)(a.sin_tab + (size_t)pos * (HD / 2) + d);
                const __nv_bfloat162 lo = *(__nv_bfloat162*)&qf[ks][x];
                const __nv_bfloat162 hi = *(__nv_bfloat162*)&qf[ks + KS / 2][x];
                const float x0a = __low2float(lo), x0b = __high2float(lo), x1a = __low2float(hi), x1b = __high2float(hi);
                qf[ks][x] = pack_bf16(x0a * cs.x - x1a * sn.x, x0b * cs.y - x1b * sn.y);
                qf[ks + KS / 2][x] = pack_bf16(x0a * sn.x + x1a * cs.x, x0b * sn.y + x1b * cs.y);
            }
        }
    }

    float oacc[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; n++) { oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    int stage = 0;                                          // it % ST
    for (int it = 0; it < n_my; it++) {
        const int hp = hp_lo + gw + it * stride;
        uint8_t* ks_cur = mine + (size_t)stage * WARP_STAGE_BYTES;
        uint8_t* vs_cur = ks_cur + TB_BYTES;
        cp_async_wait<ST - 1>();
        __syncwarp();
        if (hp == hp_hi && a.cache_w != nullptr) {
            // the tile of the new token: its row in the cache was stale when the tile was requested
            const int r = pos % TB;
            bf16* ksm = (bf16*)(ks_cur + r * ROW_BYTES);
            bf16* vsm = (bf16*)(vs_cur + r * ROW_BYTES);
#pragma unroll
            for (int u = 0; u < NEW_IT; u++) {
                const int d = lane + u * 32;
                if (d < HD / 2) {
                    ksm[d] = new_k0[u]; ksm[d + HD / 2] = new_k1[u];
                    vsm[d] = new_v0[u]; vsm[d + HD / 2] = new_v1[u];
                }
            }
            __syncwarp();
        }

        // S = Q K^T for the 16 rows and the tile's 32 keys
        float sacc[TB / 8][4];
#pragma unroll
        for (int n = 0; n < TB / 8; n++) { sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f; }
        {
            const int m = lane >> 3, r = lane & 7;
            const uint8_t* kbase = ks_cur + ((m >> 1) * 8 + r) * ROW_BYTES + (m & 1) * 16;
            uint32_t kb[2][TB / 16][4];
#pragma unroll
            for (int np = 0; np < TB / 16; np++) ldmatrix_x4(kb[0][np], kbase + np * 16 * ROW_BYTES);
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                if (ks + 1 < KS) {
#pragma unroll
                    for (int np = 0; np < TB / 16; np++)
                        ldmatrix_x4(kb[(ks + 1) & 1][np], kbase + np * 16 * ROW_BYTES + (ks + 1) * 32);
                }
#pragma unroll
                for (int np = 0; np < TB / 16; np++) {
                    mma_bf16(sacc[2 * np], qf[ks], kb[ks & 1][np][0], kb[ks & 1][np][1]);
                    mma_bf16(sacc[2 * np + 1], qf[ks], kb[ks & 1][np][2], kb[ks & 1][np][3]);
                }
            }
        }
        float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < TB / 8; n++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = e >> 1;
                const int key = hp * TB + n * 8 + tig * 2 + (e & 1);
                const bool ok = valid[i] && key <= pos && key >= key_lo;
                const float sv = ok ? sacc[n][e] * a.scale_log2 : -INFINITY;
                sacc[n][e] = sv;
                rmax[i] = fmaxf(rmax[i], sv);
            }
        }
        float alpha[2], m_use[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            rmax[i] = fmaxf(rmax[i], __shfl_xor_sync(0xffffffffu, rmax[i], 1));
            rmax[i] = fmaxf(rmax[i], __shfl_xor_sync(0xffffffffu, rmax[i], 2));
            const float m_new = fmaxf(m_run[i], rmax[i]);
            m_use[i] = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[i] = exp2f(m_run[i] - m_use[i]);
            m_run[i] = m_new;
        }
        float rsum[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < TB / 8; n++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = exp2f(sacc[n][e] - m_use[e >> 1]);
                sacc[n][e] = p;
                rsum[e >> 1] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < 2; i++) l_run[i] = l_run[i] * alpha[i] + rsum[i];
#pragma unroll
        for (int n = 0; n < HD / 8; n++) {
            oacc[n][0] *= alpha[0]; oacc[n][1] *= alpha[0];
            oacc[n][2] *= alpha[1]; oacc[n][3] *= alpha[1];
        }
#pragma unroll
        for (int kk = 0; kk < TB / 16; kk++) {
            uint32_t pa[4];
            pa[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
            pa[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
            pa[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
            pa[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
            const int m = lane >> 3, r = lane & 7;
            const uint8_t* vbase = vs_cur + (kk * 16 + (m & 1) * 8 + r) * ROW_BYTES + (m >> 1) * 16;
            uint32_t vb[2][4];
            ldmatrix_x4_trans(vb[0], vbase);
#pragma unroll
            for (int dp = 0; dp < KS; dp++) {
                if (dp + 1 < KS) ldmatrix_x4_trans(vb[(dp + 1) & 1], vbase + (dp + 1) * 32);
                mma_bf16(oacc[2 * dp], pa, vb[dp & 1][0], vb[dp & 1][1]);
                mma_bf16(oacc[2 * dp + 1], pa, vb[dp & 1][2], vb[dp & 1][3]);
            }
        }
        __syncwarp();                                       // every lane has read the stage: refill it
        if (it + ST < n_my) {
            const int hn = hp + ST * stride;
            load_half_page(ks_cur, vs_cur, a.cache, trow[hn >> 1], hn & 1, kvh, a.KVH, lane);
        }
        cp_async_commit();
        stage = stage + 1 == ST ? 0 : stage + 1;
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; i++) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    // the warps' partial results, added in warp order
    __syncthreads();                                        // every warp has left its staging buffers
    float* part = (float*)smem;                             // [NW][G][HD + 2]
#pragma unroll
    for (int i = 0; i < 2; i++) {
        if (!valid[i]) continue;
        float* p = part + ((size_t)warp * G + gid + i * 8) * (HD + 2);
#pragma unroll
        for (int n = 0; n < HD / 8; n++) {
            p[n * 8 + tig * 2] = oacc[n][2 * i];
            p[n * 8 + tig * 2 + 1] = oacc[n][2 * i + 1];
        }
        if (tig == 0) { p[HD] = m_run[i]; p[HD + 1] = l_run[i]; }
    }
    __syncthreads();
    bf16* obase = a.out + packed0 * (long long)(a.H * HD) + (size_t)kvh * G * HD;
    float* cpart = part + (size_t)NW * G * (HD + 2);       // [G][HD + 2]: this CTA's sum, for the cluster
    for (int idx = threadIdx.x; idx < G * HD; idx += NW * 32) {
        const int gh = idx / HD, d = idx % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) m = fmaxf(m, part[((size_t)w * G + gh) * (HD + 2) + HD]);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            const float* p = part + ((size_t)w * G + gh) * (HD + 2);
            if (p[HD] != -INFINITY) {
                const float wgt = exp2f(p[HD] - m);
                l += p[HD + 1] * wgt;
                o += p[d] * wgt;
            }
        }
        if (CR == 1) {
            obase[idx] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        } else {
            cpart[(size_t)gh * (HD + 2) + d] = o;
            if (d == 0) { cpart[(size_t)gh * (HD + 2) + HD] = m; cpart[(size_t)gh * (HD + 2) + HD + 1] = l; }
        }
    }
    if (CR > 1) {
        cluster_sync_all();                                 // every CTA's sum is in its shared memory
        if (rank == 0) {
            for (int idx = threadIdx.x; idx < G * HD; idx += NW * 32) {
                const int gh = idx / HD, d = idx % HD;
                const float* row = cpart + (size_t)gh * (HD + 2);
                float mr[8], lr[8], orr[8];
                float m = -INFINITY;
#pragma unroll
                for (int r = 0; r < 8; r++) {
                    if (r >= CR) break;
                    mr[r] = ld_peer_f32(row + HD, (uint32_t)r);
                    lr[r] = ld_peer_f32(row + HD + 1, (uint32_t)r);
                    orr[r] = ld_peer_f32(row + d, (uint32_t)r);
                    m = fmaxf(m, mr[r]);
                }
                float l = 0.f, o = 0.f;
#pragma unroll
                for (int r = 0; r < 8; r++) {              // in rank order
                    if (r >= CR) break;
                    if (mr[r] != -INFINITY) {
                        const float wgt = exp2f(mr[r] - m);
                        l += lr[r] * wgt;
                        o += orr[r] * wgt;
                    }
                }
                obase[idx] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
            }
        }
        cluster_sync_all();                                 // nobody leaves while its shared memory is read
    }
}

// out[row, head] = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m), splits taken in order.
__global__ void attn_merge_kernel(bf16* out, const float* partial,
                                  const int* __restrict__ tok_seq, int H, int n_splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    bf16* o = out + ((size_t)t * H + h) * HD;
    if (tok_seq[t] < 0) {
        for (int d = threadIdx.x; d < HD; d += blockDim.x) o[d] = __float2bfloat16_rn(0.f);
        return;
    }
    const float* p = partial + ((size_t)t * H + h) * n_splits * (HD + 2);
    float m = -INFINITY;
    for (int s = 0; s < n_splits; s++) m = fmaxf(m, p[s * (HD + 2) + HD]);
    float l = 0.f;
    for (int s = 0; s < n_splits; s++) {
        const float ms = p[s * (HD + 2) + HD];
        if (ms != -INFINITY) l += p[s * (HD + 2) + HD + 1] * exp2f(ms - m);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; s++) {
            const float ms = p[s * (HD + 2) + HD];
            if (ms != -INFINITY) acc += p[s * (HD + 2) + d] * exp2f(ms - m);
        }
        o[d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int NWARPS, int STAGES>
int launch_staged(const AttnArgs& a, int n_seqs, int grid_x, cudaStream_t st) {
    const size_t smem = (size_t)STAGES * 2 * TILE_BYTES + (a.fused && a.n_splits > 1 ? 2 * 64 * 32 * sizeof(float) : 0);
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_mma_kernel<NWARPS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)(STAGES * 2 * TILE_BYTES + 2 * 64 * 32 * sizeof(float)));
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    dim3 grid(grid_x, a.KVH, n_seqs);
    const int launch_rc = oe_launch(attn_mma_kernel<NWARPS, STAGES>, dim3(grid), dim3(NWARPS * 32), smem, st, a);
    return launch_rc;
}

template <int NWARPS>
int launch(const AttnArgs& a, int n_seqs, int grid_x, cudaStream_t st) {
    if (NWARPS == 1 && a.stages == 1) return launch_staged<NWARPS, 1>(a, n_seqs, grid_x, st);
    return launch_staged<NWARPS, 2>(a, n_seqs, grid_x, st);
}

// One-warp CTAs (decoded tokens).  A large batch, where each CTA walks all pages of its
// sequence: a single staged page per CTA lets twice as many CTAs share an SM, which hides
// a page's load behind the other CTAs' work (measured 38 vs 44 us at batch 64).  A small
// batch split over the keys: few pages per CTA, the double buffer wins (11 vs 13 us at 8).
int decode_stages(int n_splits) { return n_splits > 1 ? 2 : 1; }

}  // namespace

extern "C" {

int oe_attn_mma_head_dim() { return HD; }

// How many CTAs of the one-warp decode kernel with a double buffer (the form that splits the keys)
// an SM holds; <= 0 on error.
int oe_attn_mma_decode_ctas_per_sm() {
    const size_t smem = (size_t)2 * 2 * TILE_BYTES;
    if (cudaFuncSetAttribute(attn_mma_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(2 * 2 * TILE_BYTES + 2 * 64 * 32 * sizeof(float))) != cudaSuccess) return 0;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_mma_kernel<1, 2>, 32, smem) != cudaSuccess) return 0;
    return n;
}

// Floats of scratch the split path needs for a step of n_tokens rows.
long long oe_attn_mma_partial_floats(int n_tokens, int H, int n_splits) {
    return (long long)n_tokens * H * n_splits * (HD + 2);
}

// max_qlen: the most tokens any sequence brings (sizes the grid); n_splits > 1 only when
// every sequence's tokens fit one tile (decode).  zero_rows: tok_seq for the merge kernel.
int oe_attn_mma_bf16(bf16* out, const bf16* q, long long q_stride, const bf16* cache, const int* tables, int max_pages,
                     const int* cu_q, const int* seq_start, const int* seq_qlen, const int* tok_seq, int n_seqs,
                     int n_tokens, int max_qlen, int H, int KVH, int window, float scale, int n_splits, float* partial,
                     cudaStream_t st) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (H % KVH || ((uintptr_t)q & 3) || (q_stride & 1)) return OE_ERR_UNSUPPORTED;
    const int G = H / KVH;
    if (G > 64) return OE_ERR_UNSUPPORTED;
    AttnArgs a;
    a.out = out; a.q = q; a.q_stride = q_stride; a.cache = cache; a.tables = tables; a.max_pages = max_pages;
    a.cu_q = cu_q; a.seq_start = seq_start; a.seq_qlen = seq_qlen; a.H = H; a.KVH = KVH; a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.partial = partial;
    a.fused = 0; a.cos_tab = nullptr; a.sin_tab = nullptr; a.cache_w = nullptr; a.counters = nullptr;
    a.stages = 2; a.cluster = 1;
    // rows per sequence tile: 16 per warp; few rows (decode) use fewer warps
    const long long rows_needed = (long long)max_qlen * G;
    int nwarps = rows_needed <= 16 ? 1 : (rows_needed <= 32 ? 2 : 4);
    while (nwarps * 16 < G) nwarps *= 2;
    a.tokens_per_tile = (nwarps * 16) / G;
    const int n_q_tiles = (max_qlen + a.tokens_per_tile - 1) / a.tokens_per_tile;
    if (n_splits > 1 && (n_q_tiles > 1 || partial == nullptr)) n_splits = 1;
    a.n_splits = n_splits < 1 ? 1 : n_splits;
    if (nwarps == 1 && max_qlen == 1) a.stages = decode_stages(a.n_splits);
    const int grid_x = a.n_splits > 1 ? a.n_splits : n_q_tiles;
    int rc;
    if (nwarps == 1) rc = launch<1>(a, n_seqs, grid_x, st);
    else if (nwarps == 2) rc = launch<2>(a, n_seqs, grid_x, st);
    else rc = launch<4>(a, n_seqs, grid_x, st);
    if (rc) return rc;
    if (a.n_splits > 1) {
        const int launch_rc = oe_launch(attn_merge_kernel, dim3(n_tokens, H), dim3(HD >= 128 ? 128 : 64), 0, st, out, partial, tok_seq, H, a.n_splits);
        rc = launch_rc;
    }
    return rc;
}

// Decode step in one kernel: every sequence brings ONE token.  qkv rows are the fused
// projection [H*HD | KVH*HD | KVH*HD] before rotation; the kernel rotates q and the new k
// (cos/sin float32 [max_pos, HD/2], null = no rotation), stores k and v at the token's
// position when has_kv is set (else the row holds queries only and the cache already has
// the key), attends, and merges the splits.  counters: n_seqs * KVH zeroed ints.
int oe_attn_decode_fused_bf16(bf16* out, const bf16* qkv, long long qkv_stride, const float* cos_tab,
                              const float* sin_tab, bf16* cache, int has_kv, const int* tables, int max_pages,
                              const int* cu_q, const int* seq_start, const int* seq_qlen, int n_seqs, int H, int KVH,
                              int window, float scale, int n_splits, float* partial, int* counters, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (H % KVH || ((uintptr_t)qkv & 3) || (qkv_stride & 1) || (HD % 32)) return OE_ERR_UNSUPPORTED;
    const int G = H / KVH;
    if (G > 64) return OE_ERR_UNSUPPORTED;
    if (n_splits > 32 || (n_splits > 1 && (partial == nullptr || counters == nullptr))) return OE_ERR_UNSUPPORTED;
    AttnArgs a;
    a.out = out; a.q = qkv; a.q_stride = qkv_stride; a.cache = cache; a.tables = tables; a.max_pages = max_pages;
    a.cu_q = cu_q; a.seq_start = seq_start; a.seq_qlen = seq_qlen; a.H = H; a.KVH = KVH; a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.partial = partial;
    a.fused = 1; a.cos_tab = cos_tab; a.sin_tab = sin_tab; a.cache_w = has_kv ? cache : nullptr; a.counters = counters;
    int nwarps = G <= 16 ? 1 : (G <= 32 ? 2 : 4);
    a.tokens_per_tile = (nwarps * 16) / G;
    a.n_splits = n_splits < 1 ? 1 : n_splits;
    a.stages = nwarps == 1 ? decode_stages(a.n_splits) : 2; a.cluster = 1;
    if (nwarps == 1) return launch<1>(a, n_seqs, a.n_splits, st);
    if (nwarps == 2) return launch<2>(a, n_seqs, a.n_splits, st);
    return launch<4>(a, n_seqs, a.n_splits, st);
}

// The same decode step with the warps of a CTA splitting the keys (attn_decode_warps_kernel):
// one launch, no scratch.  Needs G = H/KVH <= 16.  shape = warps * 16 + ring depth; the forms
// built here: 6 x 2 (a CTA fills an SM: up to about two CTAs for every SM), 4 x 3 (the same with
// a deeper ring), 2 x 3 (two CTAs an SM) and 1 x 3 (four CTAs an SM: large batches).  0: 6 x 2.
// cluster: 1, or how many CTAs (a thread-block cluster, up to 8) share one (sequence, KV head).
// Returns OE_ERR_UNSUPPORTED for a form that is not built or does not fit an SM at this head size.
int oe_attn_decode_warps_bf16(bf16* out, const bf16* qkv, long long qkv_stride, const float* cos_tab,
                              const float* sin_tab, bf16* cache, int has_kv, const int* tables, int max_pages,
                              const int* cu_q, const int* seq_start, const int* seq_qlen, int n_seqs, int H, int KVH,
                              int window, float scale, int shape, int cluster, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (H % KVH || ((uintptr_t)qkv & 3) || (qkv_stride & 1) || (HD % 32)) return OE_ERR_UNSUPPORTED;
    const int G = H / KVH;
    if (G > 16 || n_seqs > 65535) return OE_ERR_UNSUPPORTED;
    AttnArgs a;
    a.out = out; a.q = qkv; a.q_stride = qkv_stride; a.cache = cache; a.tables = tables; a.max_pages = max_pages;
    a.cu_q = cu_q; a.seq_start = seq_start; a.seq_qlen = seq_qlen; a.H = H; a.KVH = KVH; a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.partial = nullptr; a.fused = 1; a.cos_tab = cos_tab; a.sin_tab = sin_tab; a.cache_w = has_kv ? cache : nullptr;
    a.counters = nullptr; a.tokens_per_tile = 1; a.n_splits = 1; a.stages = 2;
    if (cluster < 1 || cluster > 8) return OE_ERR_UNSUPPORTED;
    a.cluster = cluster;
    if (shape == 0) shape = 6 * 16 + 2;
    if (shape == 6 * 16 + 2 && 6 * 2 * WARP_STAGE_BYTES > 220 * 1024) shape = 3 * 16 + 2;    // large heads
#define OE_WARPS_LAUNCH(NW, ST)                                                                                    \
    if (shape == NW * 16 + ST) {                                                                                  \
        constexpr size_t smem = (size_t)NW * ST * WARP_STAGE_BYTES;                                               \
        if (smem > 220 * 1024) return OE_ERR_UNSUPPORTED;                                                         \
        static bool attr_set = false;                                                                             \
        if (!attr_set) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(attn_decode_warps_kernel<NW, ST>,                                \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
            if (e != cudaSuccess) return (int)e;                                                                  \
            attr_set = true;                                                                                      \
        }                                                                                                         \
        if (cluster > 1)                                                                                          \
            return oe_launch_cluster(attn_decode_warps_kernel<NW, ST>, (unsigned)cluster, dim3(cluster, KVH, n_seqs), \
                                     dim3(NW * 32), smem, st, a);                                                  \
        return oe_launch(attn_decode_warps_kernel<NW, ST>, dim3(1, KVH, n_seqs), dim3(NW * 32), smem, st, a);     \
    }
    OE_WARPS_LAUNCH(6, 2)
    OE_WARPS_LAUNCH(3, 2)
    OE_WARPS_LAUNCH(4, 3)
    OE_WARPS_LAUNCH(2, 3)
    OE_WARPS_LAUNCH(1, 3)
#undef OE_WARPS_LAUNCH
    return OE_ERR_UNSUPPORTED;
}

// Bytes of shared memory one CTA of a form takes (how many share an SM follows from it).
int oe_attn_decode_warps_smem(int shape) { return (shape / 16) * (shape % 16) * WARP_STAGE_BYTES; }

}  // extern "C"

// ---------------------------------------------------------------------------------------
// The entry point that allocates nothing (see attention_noalloc.h).
// ---------------------------------------------------------------------------------------
#include "attention_noalloc.h"

namespace {
// Split-key partials of one call; shared by all calls on this device.
static __device__ __align__(256) float g_noalloc_scratch[OE_ATTN_NOALLOC_MAX_FLOATS];
// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device
// address; the address is looked up once per device and kept here.
float* g_noalloc_addr[64] = {nullptr};
}  // namespace

extern "C" {

int oe_attn_mma_bf16_noalloc(bf16* out, const bf16* q, long long q_stride, const bf16* cache, const int* tables,
                             int max_pages, const int* cu_q, const int* seq_start, const int* seq_qlen,
                             const int* tok_seq, int n_seqs, int n_tokens, int max_qlen, int H, int KVH, int window,
                             float scale, int n_splits, cudaStream_t stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (n_splits < 1) n_splits = 1;
    if (n_splits > 1 && oe_attn_mma_partial_floats(n_tokens, H, n_splits) > OE_ATTN_NOALLOC_MAX_FLOATS)
        return OE_ERR_SCRATCH_TOO_SMALL;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return OE_ERR_UNSUPPORTED;
    if (g_noalloc_addr[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);      // first call on this device
        if (e != cudaSuccess) return (int)e;
        g_noalloc_addr[dev] = p;
    }
    return oe_attn_mma_bf16(out, q, q_stride, cache, tables, max_pages, cu_q, seq_start, seq_qlen, tok_seq, n_seqs,
                            n_tokens, max_qlen, H, KVH, window, scale, n_splits, g_noalloc_addr[dev], stream);
}

const char* oe_attn_mma_error_string(int code) {
    if (code == 0) return "ok";
    if (code == OE_ERR_SCRATCH_TOO_SMALL)
        return "the call needs more split-key scratch than the library's fixed array holds "
               "(n_tokens * H * n_splits * (head_dim + 2) floats > OE_ATTN_NOALLOC_MAX_FLOATS); "
               "use fewer splits or fewer tokens per call";
    if (code == OE_ERR_UNSUPPORTED) return "sizes or alignment outside what the attention kernel takes";
    return cudaGetErrorString((cudaError_t)code);
}

}  // extern "C"
