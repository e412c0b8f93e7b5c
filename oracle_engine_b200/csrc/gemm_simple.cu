// C[M,N] (+)= A[M,K] . W[N,K]^T on the CUDA cores, float32 accumulation.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced-
// precision mode) and the product for shapes the tensor-core kernels refuse.  Every
// output element is one chain of fused multiply-adds over k = 0..K-1 in that order, so
// its value does not depend on M, on the tile it falls in, or on what else is in the
// batch: the 32-bit logits are identical under every way of cutting the work.
// Role of the reference's `ops::matmul` / `gemm_q` (core/ops.cpp:207-289,
// core/gguf_parser.cpp:919-997): out[m,n] = A[m,k] . B[n,k]^T.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// MODE 0: C = acc (type TC);  MODE 1: C += acc (TC must be float: the residual stream)
template <typename TA, typename TC, int MODE>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(TC* C, const TA* A, const TA* __restrict__ W,
               int M, int N, int K, long long lda, long long ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lr = tid / 4, lk = (tid % 4) * 4;      // loader: row lr, k lk..lk+3

    pdl_launch_dependents();
    pdl_wait();
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + lk + j;
            const int am = m0 + lr, wn = n0 + lr;
            As[lk + j][lr] = (am < M && k < K) ? to_f32(A[(size_t)am * lda + k]) : 0.f;
            Ws[lk + j][lr] = (wn < N && k < K) ? to_f32(W[(size_t)wn * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; j++) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            TC* p = C + (size_t)m * ldc + n;
            if (MODE == 1) *p = from_f32<TC>(to_f32(*p) + acc[i][j]);
            else *p = from_f32<TC>(acc[i][j]);
        }
    }
}

template <typename TA, typename TC, int MODE>
int launch(TC* C, const TA* A, const TA* W, int M, int N, int K, long long lda, long long ldc,
           cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return OE_ERR_UNSUPPORTED;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return OE_ERR_UNSUPPORTED;
    const int launch_rc = oe_launch(gemm_nt_kernel<TA, TC, MODE>, dim3(grid), dim3(256), 0, st, C, A, W, M, N, K, lda, ldc);
    return launch_rc;
}

}  // namespace

extern "C" {
// out_kind: 0 = same type as the inputs, 1 = float32 store, 2 = float32 accumulate (C += A.W^T)
int oe_gemm_simple_f32(void* C, const float* A, const float* W, int M, int N, int K, long long lda,
                       long long ldc, int out_kind, cudaStream_t st) {
    if (out_kind == 2) return launch<float, float, 1>((float*)C, A, W, M, N, K, lda, ldc, st);
    return launch<float, float, 0>((float*)C, A, W, M, N, K, lda, ldc, st);
}
int oe_gemm_simple_bf16(void* C, const bf16* A, const bf16* W, int M, int N, int K, long long lda,
                        long long ldc, int out_kind, cudaStream_t st) {
    if (out_kind == 2) return launch<bf16, float, 1>((float*)C, A, W, M, N, K, lda, ldc, st);
    if (out_kind == 1) return launch<bf16, float, 0>((float*)C, A, W, M, N, K, lda, ldc, st);
    return launch<bf16, bf16, 0>((bf16*)C, A, W, M, N, K, lda, ldc, st);
}
}
