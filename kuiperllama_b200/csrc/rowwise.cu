// Row-wise kernels: embedding gather, RMSNorm fused with the residual add, SwiGLU.
//
// The residual stream is float32 in every run, so the sum x + delta and the norm's
// statistics are computed and kept in 32 bits; `T` is the compute dtype of the run
// (float in the true 32-bit path, bfloat16 in serving).
//
// Formulas as in ExiledOfCode/KuiperLLama: emb_kernel.cu:15-20 (gather),
// rmsnorm_kernel.cu:70-106 (out = w * x * rsqrt(mean(x^2) + eps)), swiglu_kernel.cu:18-21
// (silu(a) * b), add_kernel.cu:4-12 (x + delta); eps is an argument here, not a build flag.
#include "common.cuh"

namespace kl {

// out[t, :] = table[ids[t], :] as float32.  An id outside [0, vocab) writes zeros and sets
// *error_flag (KuiperLLama skips such a row silently, emb_kernel.cu:11-13).
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                 int hidden, int vocab, int* __restrict__ error_flag) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(error_flag, 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(row[i]);
}

// One CTA per output row r.  Source row s = rows ? rows[r] : r.
//   x = residual[s] (+ delta[s] if delta);  if (!rows && delta) residual[s] = x;
//   out[r] = weight * x * rsqrt(mean(x^2) + eps)
// With `rows` the residual is not written back: it is the read of a few rows before the
// classifier.  The row is kept in registers between the two passes (hidden <= 256 * 32),
// else it is read twice.
template <typename T, int THREADS, int PER_THREAD>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* x = residual + (size_t)s * hidden;
    const T* d = delta ? delta + (size_t)s * hidden : nullptr;
    T* o = out + (size_t)r * hidden;
    const bool write_back = (rows == nullptr) && (delta != nullptr);
    float v[PER_THREAD];
    float ss = 0.f;
    const bool in_regs = hidden <= THREADS * PER_THREAD;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < PER_THREAD; ++j) {
            const int i = threadIdx.x + j * THREADS;
            float a = 0.f;
            if (i < hidden) {
                a = x[i];
                if (d) a += to_f32(d[i]);
                if (write_back) x[i] = a;
            }
            v[j] = a;
            ss += a * a;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += THREADS) {
            float a = x[i];
            if (d) a += to_f32(d[i]);
            if (write_back) x[i] = a;
            ss += a * a;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < PER_THREAD; ++j) {
            const int i = threadIdx.x + j * THREADS;
            if (i < hidden) o[i] = from_f32<T>(weight[i] * (v[j] * inv));
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += THREADS) {
            float a = x[i];
            if (d && !write_back) a += to_f32(d[i]);
            o[i] = from_f32<T>(weight[i] * (a * inv));
        }
    }
}

// out[t, i] = silu(gu[t, i]) * gu[t, inter + i]; gu is [tokens, 2 * inter] (gate columns first).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int tokens, int inter) {
    const size_t n = (size_t)tokens * inter;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inter;
        const int i = (int)(idx - t * inter);
        const float g = to_f32(gu[t * 2 * inter + i]);
        const float u = to_f32(gu[t * 2 * inter + inter + i]);
        out[idx] = from_f32<T>(g * (1.0f / (1.0f + expf(-g))) * u);
    }
}

}  // namespace kl

using namespace kl;

KL_API int kl_embedding(const int* ids, int n_tokens, const void* table, int table_dtype, int vocab, int hidden,
                        float* out, int* error_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return KL_OK;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == KL_F32)
        embedding_kernel<float><<<n_tokens, threads, 0, stream>>>(ids, (const float*)table, out, hidden, vocab, error_flag);
    else if (table_dtype == KL_BF16)
        embedding_kernel<bf16><<<n_tokens, threads, 0, stream>>>(ids, (const bf16*)table, out, hidden, vocab, error_flag);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_add_rmsnorm(float* residual, const void* delta, const float* weight, void* out, const int* rows,
                          int n_rows, int hidden, float eps, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return KL_OK;
    constexpr int THREADS = 256, PER = 32;
    if (dtype == KL_F32)
        add_rmsnorm_kernel<float, THREADS, PER><<<n_rows, THREADS, 0, stream>>>(residual, (const float*)delta, weight,
                                                                               (float*)out, rows, hidden, eps);
    else if (dtype == KL_BF16)
        add_rmsnorm_kernel<bf16, THREADS, PER><<<n_rows, THREADS, 0, stream>>>(residual, (const bf16*)delta, weight,
                                                                              (bf16*)out, rows, hidden, eps);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_swiglu(const void* gate_up, void* out, int tokens, int inter, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return KL_OK;
    const size_t n = (size_t)tokens * inter;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
    if (dtype == KL_F32)
        swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, tokens, inter);
    else if (dtype == KL_BF16)
        swiglu_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, tokens, inter);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
