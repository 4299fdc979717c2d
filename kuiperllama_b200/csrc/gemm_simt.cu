// C[M, N] = A[M, K] * W[N, K]^T with plain 32-bit FMA arithmetic: every size, every
// alignment.  It is the matrix product of the true 32-bit path (no tensor-core mode of any
// kind) and the fallback of the bfloat16 path for shapes that the tensor-core kernel
// refuses (a K whose row stride is no multiple of 16 bytes).
//
// y = W x as in ExiledOfCode/KuiperLLama's matmul_kernel_cu_fp32 (matmul_kernel.cu:6-54):
// weights are [out, in] row-major and there is no bias.  There one CTA reduces one output
// row of a single vector; here a 64 x 64 tile of outputs is accumulated over K in steps of
// 16, each output in one thread in ascending k, so the value of an output does not depend
// on how many rows M the call has.
#include "common.cuh"

namespace kl {

constexpr int GS_BM = 64, GS_BN = 64, GS_BK = 16, GS_THREADS = 256;

template <typename TI, typename TO>
__global__ void __launch_bounds__(GS_THREADS)
gemm_simt_kernel(const TI* __restrict__ A, int lda, const TI* __restrict__ W, int ldw, TO* __restrict__ C, int ldc,
                 int M, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float As[GS_BK][GS_BM + 4];
    __shared__ float Ws[GS_BK][GS_BN + 4];
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;      // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GS_BK) {
        // 64 x 16 elements of each operand, 4 per thread
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = threadIdx.x + r * GS_THREADS;          // 0 .. 1023
            const int row = e / GS_BK, kk = e % GS_BK;
            const int gm = m0 + row, gn = n0 + row, gk = k0 + kk;
            As[kk][row] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[kk][row] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
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
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = from_f32<TO>(acc[i][j]);
        }
    }
}

}  // namespace kl

using namespace kl;

// in_dtype: dtype of A and W; out_dtype: dtype of C (float32 output of bfloat16 operands is
// what the classifier uses for logits).
KL_API int kl_gemm_simt(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                        int in_dtype, int out_dtype, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KL_OK;
    if (K <= 0) return KL_ERR_BAD_SIZE;
    const dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
    if (grid.y > 65535) return KL_ERR_BAD_SIZE;
    if (in_dtype == KL_F32 && out_dtype == KL_F32)
        launch_kernel(gemm_simt_kernel<float, float>, grid, GS_THREADS, 0, stream, (const float*)A, lda, (const float*)W, ldw,
                                                                        (float*)C, ldc, M, N, K);
    else if (in_dtype == KL_BF16 && out_dtype == KL_BF16)
        launch_kernel(gemm_simt_kernel<bf16, bf16>, grid, GS_THREADS, 0, stream, (const bf16*)A, lda, (const bf16*)W, ldw,
                                                                      (bf16*)C, ldc, M, N, K);
    else if (in_dtype == KL_BF16 && out_dtype == KL_F32)
        launch_kernel(gemm_simt_kernel<bf16, float>, grid, GS_THREADS, 0, stream, (const bf16*)A, lda, (const bf16*)W, ldw,
                                                                       (float*)C, ldc, M, N, K);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
