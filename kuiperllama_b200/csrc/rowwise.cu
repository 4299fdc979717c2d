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

// out[t, :] = scale * table[ids[t], :] as float32 (scale 1 for a plain gather).  An id outside
// [0, vocab) writes zeros and sets *error_flag (KuiperLLama skips such a row silently,
// emb_kernel.cu:11-13).
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                 int hidden, int vocab, float scale, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(error_flag, 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = scale * to_f32(row[i]);
}

// One CTA per output row r.  Source row s = rows ? rows[r] : r.
//   x = residual[s] + delta[s] (+ partial[0][s] + partial[1][s] + ... in ascending order)
//   if (!rows && something was added) residual[s] = x
//   out[r] = weight * x * rsqrt(mean(x^2) + eps)
// `delta` is in the compute dtype; `partials` are float32 partial sums [n_partials][rows][hidden]
// of a product whose K range was cut (their sum is the delta).  With `rows` the residual is
// not written back: it is the read of a few rows before the classifier.  Rows are processed
// four floats at a time when hidden is a multiple of 4; a row that fits THREADS * 4 * VPT
// floats stays in registers between the two passes, else it is recomputed.
template <typename T> struct Delta4;
template <> struct Delta4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Delta4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS, 1)
add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ partials,
                   int n_partials, size_t partial_stride, const float* __restrict__ weight, T* __restrict__ out,
                   const int* __restrict__ rows, int hidden, float eps) {
    pdl_launch_dependents();
    // The norm's weight is written by no kernel: where a row fits the registers it is fetched before
    // this grid waits for the kernel before it.
    // (only in the form for few rows, THREADS = 1024: with many rows the registers are worth more as occupancy)
    constexpr bool FEW = THREADS >= 1024;
    float4 wreg[FEW ? VPT : 1];
    const bool fits = FEW && (hidden & 3) == 0 && (hidden >> 2) <= THREADS * VPT;
    if (fits) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i4 = threadIdx.x + j * THREADS;
            wreg[j] = i4 < (hidden >> 2) ? *reinterpret_cast<const float4*>(weight + 4 * i4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* x = residual + (size_t)s * hidden;
    const T* d = delta ? delta + (size_t)s * hidden : nullptr;
    const float* p = n_partials > 0 ? partials + (size_t)s * hidden : nullptr;
    T* o = out + (size_t)r * hidden;
    const bool adds = d != nullptr || p != nullptr;
    const bool write_back = rows == nullptr && adds;
    float ss = 0.f;
    if ((hidden & 3) == 0) {
        const int n4 = hidden >> 2;
        auto value = [&](int i4) {
            float4 a = *reinterpret_cast<const float4*>(x + 4 * i4);
            if (d) { const float4 b = Delta4<T>::load(d + 4 * i4); a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
            // eight pieces (few rows) are requested at a time, one trip to memory instead of eight, and added in ascending order
            constexpr int ZB = FEW ? 8 : 2;
            for (int z0 = 0; z0 < n_partials; z0 += ZB) {
                float4 b[ZB];
#pragma unroll
                for (int zz = 0; zz < ZB; ++zz)
                    b[zz] = z0 + zz < n_partials ? *reinterpret_cast<const float4*>(p + (size_t)(z0 + zz) * partial_stride + 4 * i4)
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int zz = 0; zz < ZB; ++zz)
                    if (z0 + zz < n_partials) { a.x += b[zz].x; a.y += b[zz].y; a.z += b[zz].z; a.w += b[zz].w; }
            }
            return a;
        };
        float4 v[VPT];
        const bool in_regs = n4 <= THREADS * VPT;
        if (in_regs) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int i4 = threadIdx.x + j * THREADS;
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i4 < n4) {
                    a = value(i4);
                    if (write_back) *reinterpret_cast<float4*>(x + 4 * i4) = a;
                }
                v[j] = a;
                ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            }
        } else {
            for (int i4 = threadIdx.x; i4 < n4; i4 += THREADS) {
                const float4 a = value(i4);
                ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            }
        }
        ss = block_sum(ss, scratch);
        const float inv = rsqrtf(ss / (float)hidden + eps);
        if (in_regs) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int i4 = threadIdx.x + j * THREADS;
                if (i4 < n4) {
                    const float4 w = FEW ? wreg[FEW ? j : 0] : *reinterpret_cast<const float4*>(weight + 4 * i4);
                    const float4 a = v[j];
                    Delta4<T>::store(o + 4 * i4, make_float4(w.x * (a.x * inv), w.y * (a.y * inv), w.z * (a.z * inv), w.w * (a.w * inv)));
                }
            }
        } else {
            for (int i4 = threadIdx.x; i4 < n4; i4 += THREADS) {
                const float4 a = value(i4);                      // the residual is still unchanged: recompute, then write
                const float4 w = *reinterpret_cast<const float4*>(weight + 4 * i4);
                Delta4<T>::store(o + 4 * i4, make_float4(w.x * (a.x * inv), w.y * (a.y * inv), w.z * (a.z * inv), w.w * (a.w * inv)));
                if (write_back) *reinterpret_cast<float4*>(x + 4 * i4) = a;
            }
        }
    } else {
        auto value = [&](int i) {
            float a = x[i];
            if (d) a += to_f32(d[i]);
            for (int z = 0; z < n_partials; ++z) a += p[(size_t)z * partial_stride + i];
            return a;
        };
        for (int i = threadIdx.x; i < hidden; i += THREADS) { const float a = value(i); ss += a * a; }
        ss = block_sum(ss, scratch);
        const float inv = rsqrtf(ss / (float)hidden + eps);
        for (int i = threadIdx.x; i < hidden; i += THREADS) {
            const float a = value(i);
            o[i] = from_f32<T>(weight[i] * (a * inv));
            if (write_back) x[i] = a;
        }
    }
}

// out[t, i] = silu(gu[t, i]) * gu[t, inter + i]; gu is [tokens, 2 * inter] (gate columns first).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int tokens, int inter) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)tokens * inter;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inter;
        const int i = (int)(idx - t * inter);
        const float g = to_f32(gu[t * 2 * inter + i]);
        const float u = to_f32(gu[t * 2 * inter + inter + i]);
        out[idx] = from_f32<T>(g * (1.0f / (1.0f + expf(-g))) * u);
    }
}

// Logits in place: x = scale * x, then, with a soft cap c > 0, x = c * tanh(x / c).
__global__ void logit_transform_kernel(float* __restrict__ logits, long long ld, int rows, int vocab, float scale, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)rows * vocab;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / vocab;
        float* p = logits + r * ld + (idx - r * vocab);
        float x = *p * scale;
        if (cap > 0.f) x = cap * tanhf(x / cap);
        *p = x;
    }
}

}  // namespace kl

using namespace kl;

KL_API int kl_logit_transform(float* logits, long long ld, int rows, int vocab, float scale, float softcap, cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0) return KL_OK;
    if (softcap < 0.f || ld < vocab) return KL_ERR_BAD_SIZE;
    const int threads = 256;
    launch_kernel(logit_transform_kernel, kl::strided_grid((size_t)rows * vocab, threads, 16), threads, 0, stream, logits, ld, rows,
                  vocab, scale, softcap);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_embedding(const int* ids, int n_tokens, const void* table, int table_dtype, int vocab, int hidden,
                        float scale, float* out, int* error_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return KL_OK;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == KL_F32)
        launch_kernel(embedding_kernel<float>, n_tokens, threads, 0, stream, ids, (const float*)table, out, hidden, vocab, scale, error_flag);
    else if (table_dtype == KL_BF16)
        launch_kernel(embedding_kernel<bf16>, n_tokens, threads, 0, stream, ids, (const bf16*)table, out, hidden, vocab, scale, error_flag);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// delta: compute dtype [rows, hidden] or null; partials: float32 [n_partials, rows_total, hidden]
// or null (partial_stride = rows_total * hidden elements).
KL_API int kl_add_rmsnorm(float* residual, const void* delta, const float* partials, int n_partials,
                          long long partial_stride, const float* weight, void* out, const int* rows, int n_rows,
                          int hidden, float eps, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return KL_OK;
    if (n_partials < 0 || (n_partials > 0 && partials == nullptr)) return KL_ERR_BAD_SIZE;
    // few rows: more threads per row, so that a step of a handful of tokens is not one slow CTA each
    const bool wide = n_rows <= 256 && hidden >= 2048;
#define KL_NORM(T, THREADS, VPT)                                                                                        \
    launch_kernel(add_rmsnorm_kernel<T, THREADS, VPT>, n_rows, THREADS, 0, stream, residual, (const T*)delta, partials, n_partials, \
        (size_t)partial_stride, weight, (T*)out, rows, hidden, eps)
    // many rows: a row in registers of 256 threads, four or eight float4 each (fewer registers, more CTAs per SM)
    const bool narrow = hidden <= 256 * 4 * 4;
    if (dtype == KL_F32) { if (wide) KL_NORM(float, 1024, 2); else if (narrow) KL_NORM(float, 256, 4); else KL_NORM(float, 256, 8); }
    else if (dtype == KL_BF16) { if (wide) KL_NORM(bf16, 1024, 2); else if (narrow) KL_NORM(bf16, 256, 4); else KL_NORM(bf16, 256, 8); }
    else return KL_ERR_BAD_DTYPE;
#undef KL_NORM
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_swiglu(const void* gate_up, void* out, int tokens, int inter, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return KL_OK;
    const size_t n = (size_t)tokens * inter;
    const int threads = 256;
    const int blocks = kl::strided_grid(n, threads, 16);
    if (dtype == KL_F32)
        launch_kernel(swiglu_kernel<float>, blocks, threads, 0, stream, (const float*)gate_up, (float*)out, tokens, inter);
    else if (dtype == KL_BF16)
        launch_kernel(swiglu_kernel<bf16>, blocks, threads, 0, stream, (const bf16*)gate_up, (bf16*)out, tokens, inter);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
