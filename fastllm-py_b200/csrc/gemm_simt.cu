// C[M, N] = A[M, K] * W[N, K]^T on CUDA cores with float accumulation: the
// matrix product of the true 32-bit path (no tensor-core mode drops mantissa
// bits here), and the product for any operand types the tensor-core kernel
// does not take (a weight stored in 32-bit under bfloat16 activations).
//
// fastllm-py calls cuBLAS for `x @ w.T` (fastllm_py/model.py:63).  This kernel
// is slower and has one property cuBLAS lacks: each output element is one
// thread's sum over k = 0..K-1 in that order, whatever M is, so a token's
// result does not depend on how many other tokens share the step.
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TA* __restrict__ A, long lda,
                                                        const TW* __restrict__ W, long ldw,
                                                        TC* __restrict__ C, long ldc, int M, int N,
                                                        int K) {
    pdl_wait();
    pdl_trigger();
    __shared__ float As[GS_BK][GS_BM + 1];
    __shared__ float Ws[GS_BK][GS_BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += GS_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx >> 4, c = idx & 15;
            const bool kin = (k0 + c) < K;
            As[c][r] = (kin && m0 + r < M) ? to_f32<TA>(A[(long)(m0 + r) * lda + k0 + c]) : 0.0f;
            Ws[c][r] = (kin && n0 + r < N) ? to_f32<TW>(W[(long)(n0 + r) * ldw + k0 + c]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GS_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(long)m * ldc + n] = from_f32<TC>(acc[i][j]);
        }
    }
}

FL_API int fl_gemm_simt(const void* A, int a_dtype, long lda, const void* W, int w_dtype, long ldw,
                        void* C, int c_dtype, long ldc, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(a_dtype, TA, FL_DISPATCH(w_dtype, TW, FL_DISPATCH(c_dtype, TC,
        return fl_launch(gemm_simt_kernel<TA, TW, TC>, grid, dim3(256), 0, stream, (const TA*)A, lda,
                         (const TW*)W, ldw, (TC*)C, ldc, M, N, K))));
    return 0;
}
