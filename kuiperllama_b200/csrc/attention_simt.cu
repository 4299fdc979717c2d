// Causal grouped-query attention over the paged cache, plain SIMT arithmetic in 32 bits.
//
// This is the kernel of the true 32-bit path (prefill and decode) and the fallback of the
// bfloat16 path for sizes and options that the tensor-core kernels refuse (a window, a
// head size that is no multiple of 16 on their list).  One CTA of four warps per
// (token, query head).  Query token t of slot s at position p reads keys lo..p of that
// slot, lo = max(0, p - window + 1) with a window, else 0.  Head h reads kv head
// h / (H / KV); score = (q . k) * scale; softmax with the maximum subtracted; o = sum p v
// (ExiledOfCode/KuiperLLama mha_kernel.cu:61,74-106; there one CTA per head loops over one
// sequence and the scores pass through global memory).
//
// Keys are cut into chunks of 32 by absolute position and the chunks are dealt to the warps
// round-robin, so the order of every sum depends only on the token's own position: the
// result does not change with the way tokens are cut into steps or batched.
#include "common.cuh"

namespace kl {

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_PER_LANE = 8;      // head_dim <= 256

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ k, const float* __restrict__ q, int hd);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ k, const float* __restrict__ q, int hd) {
    float s = 0.f;
    for (int i = 0; i < hd; i += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(k + i);
        s += kv.x * q[i] + kv.y * q[i + 1] + kv.z * q[i + 2] + kv.w * q[i + 3];
    }
    return s;
}
template <>
__device__ __forceinline__ float dot_row<bf16>(const bf16* __restrict__ k, const float* __restrict__ q, int hd) {
    float s = 0.f;
    for (int i = 0; i < hd; i += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(k + i);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(p[j]);
            s += f.x * q[i + 2 * j] + f.y * q[i + 2 * j + 1];
        }
    }
    return s;
}

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                      const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                      const int* __restrict__ block_table, int blocks_per_seq,
                      const int* __restrict__ positions, const int* __restrict__ token_slot,
                      int H, int KV, int hd, float scale, int window) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    float* q_s = smem;                               // [hd]
    float* m_s = q_s + hd;                           // [ATT_WARPS]
    float* l_s = m_s + ATT_WARPS;                    // [ATT_WARPS]
    float* acc_s = l_s + ATT_WARPS;                  // [ATT_WARPS][hd]

    const int t = blockIdx.x, h = blockIdx.y;
    const int slot = token_slot[t];
    if (slot < 0) return;                            // a padding row: nothing is written
    const int pos = positions[t];
    const int g = h / (H / KV);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) q_s[i] = to_f32(qrow[i]);
    __syncthreads();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float m = -INFINITY, l = 0.f;
    float acc[ATT_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < ATT_MAX_PER_LANE; ++i) acc[i] = 0.f;

    const int* table = block_table + (size_t)slot * blocks_per_seq;
    for (int c = lo / 32 + warp; c * 32 <= pos; c += ATT_WARPS) {
        const int base = c * 32;                                     // 32 keys inside one page
        const int page = table[base / PAGE];
        const size_t page_off = (((size_t)page * KV + g) * PAGE + (base % PAGE)) * (size_t)hd;
        const int key = base + lane;
        const bool valid = key >= lo && key <= pos;
        float s = -INFINITY;
        if (valid) s = dot_row<T>(k_cache + page_off + (size_t)lane * hd, q_s, hd) * scale;
        const float m_new = fmaxf(m, warp_max(s));                   // finite: the chunk holds a valid key
        const float corr = expf(m - m_new);                          // exp(-inf) = 0 at the first chunk
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < ATT_MAX_PER_LANE; ++i) acc[i] *= corr;
        const int j_lo = max(lo - base, 0), j_hi = min(pos - base, 31);
        const T* vbase = v_cache + page_off;
        for (int j = j_lo; j <= j_hi; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const T* vrow = vbase + (size_t)j * hd;
#pragma unroll
            for (int i = 0; i < ATT_MAX_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] += pj * to_f32(vrow[d]);
            }
        }
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int i = 0; i < ATT_MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc_s[warp * hd + d] = acc[i];
    }
    __syncthreads();
    float M = m_s[0];
#pragma unroll
    for (int w = 1; w < ATT_WARPS; ++w) M = fmaxf(M, m_s[w]);
    float L = 0.f;
    float wgt[ATT_WARPS];
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        wgt[w] = m_s[w] == -INFINITY ? 0.f : expf(m_s[w] - M);
        L += l_s[w] * wgt[w];
    }
    T* orow = out + ((size_t)t * H + h) * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) o += acc_s[w * hd + d] * wgt[w];
        orow[d] = from_f32<T>(o / L);
    }
}

}  // namespace kl

using namespace kl;

// q: rows of q_stride elements, head h at column h * hd.  out: [tokens, H * hd].
KL_API int kl_attention_simt(const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,
                             const int* block_table, int blocks_per_seq, const int* positions,
                             const int* token_slot, int n_tokens, int H, int KV, int hd, float scale, int window,
                             int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return KL_OK;
    if (hd % 16 || hd > 32 * ATT_MAX_PER_LANE || hd <= 0 || KV <= 0 || H % KV) return KL_ERR_BAD_SIZE;
    if (H > 65535) return KL_ERR_BAD_SIZE;
    const dim3 grid(n_tokens, H);
    const size_t smem = (size_t)(hd + 2 * ATT_WARPS + ATT_WARPS * hd) * sizeof(float);
    if (dtype == KL_F32)
        launch_kernel(attention_simt_kernel<float>, grid, ATT_WARPS * 32, smem, stream, (const float*)q, q_stride, (float*)out,
            (const float*)k_cache, (const float*)v_cache, block_table, blocks_per_seq, positions, token_slot, H, KV,
            hd, scale, window);
    else if (dtype == KL_BF16)
        launch_kernel(attention_simt_kernel<bf16>, grid, ATT_WARPS * 32, smem, stream, (const bf16*)q, q_stride, (bf16*)out,
            (const bf16*)k_cache, (const bf16*)v_cache, block_table, blocks_per_seq, positions, token_slot, H, KV,
            hd, scale, window);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
