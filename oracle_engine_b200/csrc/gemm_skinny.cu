// out[M,N] (+)= A[M,K] . W[N,K]^T for a handful of tokens (M <= 16): the decode step's
// matrix products, which only have to stream the weights once at memory speed.
//
// A CTA of 8 warps owns 16 weight rows; the warps split K between them.  Every lane
// reads its rows with 16-byte loads that bypass L1 (each row is read in runs of 128
// contiguous bytes), the few activation rows come through L1/L2, and the products run on
// mma.sync m16n8k16 (weights are the 16-row operand, tokens the 8 columns) with float32
// accumulators.  The k indices inside an instruction are permuted the same way for both
// operands, so that each lane's 8 consecutive bf16 of a row feed two instructions
// without any shuffle.  The 8 partial tiles of a CTA are added in warp order through
// shared memory: no workspace, no atomics, the same bits every time.  Nothing is staged
// in shared memory and there is no tensor-memory set-up, so the kernel's fixed cost is a
// launch plus one memory round trip; with 16 rows per CTA there are enough CTAs (N/16)
// to keep every SM streaming.  The tensor-memory kernel (gemm_tcgen05.cu) takes over for
// more than 16 tokens, where the weights' tile is reused enough to need it.
// Epilogues: bf16 store, float32 store, float32 accumulate (residual), and SwiGLU on
// interleaved gate/up rows.  Reference role: gemv_q (core/gguf_parser.cpp:868-911).
#include "common.cuh"

namespace {

constexpr int ROWS = 16;          // weight rows per CTA
constexpr int CHUNK = 64;         // k per chunk: 4 lanes x 16 consecutive bf16

__device__ __forceinline__ uint4 ld_weight(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: 8-token tiles, 1 (M <= 8) or 2 (M <= 16); WARPS: warps per CTA (they split K);
// UNROLL: 64-wide k chunks whose weight loads a warp has in flight at once.
template <int NT, int WARPS, int UNROLL>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(void* C, const bf16* A, const bf16* __restrict__ W,
                   int M, int N, int K, long long lda, long long ldc, int out_kind, int late_trigger) {
    __shared__ float red[WARPS][ROWS][8 * NT + 1];
    __shared__ float total[ROWS][8 * NT + 1];
    if (!late_trigger) pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * ROWS;
    const bool rv0 = row0 + g < N, rv1 = row0 + g + 8 < N;
    const bf16* w0 = W + (size_t)(rv0 ? row0 + g : 0) * K;
    const bf16* w1 = W + (size_t)(rv1 ? row0 + g + 8 : 0) * K;
    const int n_chunks = (K + CHUNK - 1) / CHUNK;
    const int per = (n_chunks + WARPS - 1) / WARPS;
    const int c_begin = warp * per;
    const int c_end = min(n_chunks, c_begin + per);

    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; n++) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    bool waited = false;

    for (int c = c_begin; c < c_end; c += UNROLL) {
        uint4 wa[UNROLL][2], wb[UNROLL][2];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int k8 = (c + u) * CHUNK + t * 16 + hh * 8;
                const bool kv = (c + u) < c_end && k8 < K;
                wa[u][hh] = (kv && rv0) ? ld_weight(w0 + k8) : zero;
                wb[u][hh] = (kv && rv1) ? ld_weight(w1 + k8) : zero;
            }
        }
        if (!waited) { pdl_wait(); waited = true; }      // activations come from the kernel before
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int k8 = (c + u) * CHUNK + t * 16 + hh * 8;
                const bool kv = (c + u) < c_end && k8 < K;
#pragma unroll
                for (int n = 0; n < NT; n++) {
                    const int tok = n * 8 + g;
                    uint4 x = zero;
                    if (kv && tok < M) x = *(const uint4*)(A + (size_t)tok * lda + k8);
                    mma_bf16(acc[n], wa[u][hh].x, wb[u][hh].x, wa[u][hh].y, wb[u][hh].y, x.x, x.y);
                    mma_bf16(acc[n], wa[u][hh].z, wb[u][hh].z, wa[u][hh].w, wb[u][hh].w, x.z, x.w);
                }
            }
        }
    }
    if (!waited) pdl_wait();
    // late_trigger: the kernel after this one may be scheduled only now, when this CTA has streamed
    // its weights, so that its CTAs do not sit on the SMs while this kernel still needs them
    if (late_trigger) pdl_launch_dependents();

    // add the warps' partial tiles in warp order
#pragma unroll
    for (int n = 0; n < NT; n++) {
        red[warp][g][n * 8 + t * 2] = acc[n][0];
        red[warp][g][n * 8 + t * 2 + 1] = acc[n][1];
        red[warp][g + 8][n * 8 + t * 2] = acc[n][2];
        red[warp][g + 8][n * 8 + t * 2 + 1] = acc[n][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS * 8 * NT; idx += WARPS * 32) {
        const int r = idx % ROWS, tok = idx / ROWS;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) s += red[w][r][tok];
        total[r][tok] = s;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS * 8 * NT; idx += WARPS * 32) {
        const int r = idx % ROWS, tok = idx / ROWS;
        const int row = row0 + r;
        if (tok >= M || row >= N) continue;
        const float v = total[r][tok];
        if (out_kind == 0) ((bf16*)C)[(size_t)tok * ldc + row] = __float2bfloat16_rn(v);
        else if (out_kind == 1) ((float*)C)[(size_t)tok * ldc + row] = v;
        else if (out_kind == 2) ((float*)C)[(size_t)tok * ldc + row] += v;
        else if (!(r & 1)) {
            const float up = total[r + 1][tok];
            ((bf16*)C)[(size_t)tok * ldc + (row >> 1)] = __float2bfloat16_rn((v / (1.f + expf(-v))) * up);
        }
    }
}

}  // namespace

extern "C" {

int oe_gemm_skinny_supported(const void* A, const void* W, int M, int N, int K, long long lda) {
    if (M <= 0 || M > 16 || N <= 0 || K <= 0) return 0;
    if ((K % 8) || (lda % 8)) return 0;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return 0;
    return 1;
}

// out_kind: 0 bf16, 1 float32, 2 float32 accumulate, 3 bf16 silu(gate)*up on interleaved rows (C is [M, N/2]).
// early: bit 0 start early, bit 1 trigger late (see below).
int oe_gemm_skinny_bf16(void* C, const bf16* A, const bf16* W, int M, int N, int K, long long lda, long long ldc,
                        int out_kind, int early, cudaStream_t st) {
    if (!oe_gemm_skinny_supported(A, W, M, N, K, lda)) return OE_ERR_UNSUPPORTED;
    if (out_kind < 0 || out_kind > 3 || (out_kind == 3 && (N & 1))) return OE_ERR_UNSUPPORTED;
    const int blocks = (N + ROWS - 1) / ROWS;
    // early bit 0: the kernel may start (and request its first weights) while the kernel before it
    // drains.  early bit 1: this kernel releases the kernel after it only when its CTAs have
    // streamed their weights (else at its top).  Measured on B200 in a decode step of the 3B
    // shape, 8 sequences (1.768 ms with qkv and o starting early, every trigger at the top):
    // gate/up or down starting early behind kernels that trigger at their top cost 20-50 %
    // (their very many CTAs sit on the SMs while the kernel before still needs them); with o,
    // gate/up and down starting early AND triggering late, qkv starting early and triggering at
    // its top (the attention kernel asks for its keys meanwhile): 1.736 ms.  Varied one at a time
    // from there (timed steps of 1.714 ms, the device idle before them): only down triggering at its
    // top is as fast or faster (1 sequence 1.606 -> 1.577 ms); o starting early and triggering at its
    // top: 2.44 ms.  The caller decides.
    // Warps and loads in flight per shape: matrices with many rows do best with small CTAs, long rows
    // with more loads in flight.
#define OE_SKINNY_LAUNCH(NT, WARPS, UNROLL)                                                                        \
    return oe_launch_ex((early & 1) != 0, gemm_skinny_kernel<NT, WARPS, UNROLL>, dim3(blocks), dim3(WARPS * 32), 0, st, C, A, \
                        W, M, N, K, lda, ldc, out_kind, (early >> 1) & 1)
    if (M > 8) {
        // 9 to 16 tokens, chosen inside the 28-layer decode step (16 sequences: 2.11 ms with 8 warps x 3 loads
        // for every shape, 1.96 ms with these)
        if (blocks >= 4 * 148) OE_SKINNY_LAUNCH(2, 4, 4);
        if (blocks >= 256) OE_SKINNY_LAUNCH(2, 8, 2);
        OE_SKINNY_LAUNCH(2, 8, 3);
    }
    // up to 8 tokens, chosen shape by shape inside the 28-layer decode step (8 sequences: 1.713 ms with the
    // forms a sweep of the kernels alone had given, 4 warps x 3 loads for very many rows, 8 x 3 for long rows,
    // 8 x 2 else; 1.670 ms with these)
    if (blocks >= 256) OE_SKINNY_LAUNCH(1, 4, 4);
    if (K > 4096) OE_SKINNY_LAUNCH(1, 8, 4);
    OE_SKINNY_LAUNCH(1, 8, 2);
#undef OE_SKINNY_LAUNCH
}

}  // extern "C"
