// Decode attention in bfloat16: one new token per sequence against its paged cache, the keys
// of every sequence cut over several CTAs (split-KV) so that a single long context fills
// the machine, and the query heads of one kv group handled together so that every key and
// value is read once for the whole group.
//
// Per head: s_t = (q . k_t) * scale for t <= pos, softmax with the maximum subtracted,
// o = sum p_t v_t, all in 32 bits (ExiledOfCode/KuiperLLama mha_kernel.cu:61,74-106, where
// one CTA per head walks the whole sequence and the scores go through global memory).
//
// Grid (sequence, kv head x head tile, split).  A sequence of n keys gives each of the S
// splits ceil(n / S) keys rounded up to whole pages, so the grid does not depend on the
// lengths (it can be captured in a CUDA graph) and an empty split only records that.  LPK
// lanes share one key, each holding eight of its dimensions (one 16-byte load); a
// lane group takes four keys per turn.  Partial results (max, sum, unnormalised output) of
// the lane groups are merged in the warp, the warps in shared memory, the splits by a second
// kernel, always in the same order.
#include "common.cuh"

namespace kl {

constexpr int DA_WARPS = 4;
constexpr int DA_KEYS = 4;            // keys a lane group handles per turn

template <int N>
__device__ __forceinline__ void load_bf16(const bf16* __restrict__ p, float (&out)[N]) {
#pragma unroll
    for (int i = 0; i < N; i += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            out[i + 2 * j] = f.x;
            out[i + 2 * j + 1] = f.y;
        }
    }
}

// partial_o: [rows, H, S, HD] float32; partial_ml: [rows, H, S, 2] (max, sum).
template <int HD, int LPK, int GT>
__global__ void __launch_bounds__(DA_WARPS * 32)
decode_attention_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out,
                        const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                        const int* __restrict__ block_table, int blocks_per_seq,
                        const int* __restrict__ positions, const int* __restrict__ token_slot,
                        float* __restrict__ partial_o, float* __restrict__ partial_ml,
                        int H, int KV, float scale, int window) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int DPL = HD / LPK;                 // dimensions per lane
    constexpr int KPW = 32 / LPK;                 // lane groups (keys in flight) per warp
    static_assert(DPL == 8, "a lane holds 8 dimensions: one 16-byte load per key");
    __shared__ float sm_m[DA_WARPS][GT], sm_l[DA_WARPS][GT];
    __shared__ float sm_o[DA_WARPS][GT][HD];

    const int row = blockIdx.x;
    const int slot = token_slot[row];
    if (slot < 0) return;                                        // a padding row
    const int group = H / KV;
    const int tiles = (group + GT - 1) / GT;
    const int g = blockIdx.y / tiles, ht = blockIdx.y % tiles;
    const int S = gridDim.z, z = blockIdx.z;
    const int pos = positions[row];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    // this split's keys: whole pages, counted from the first page that holds a visible key
    const int first = (lo / PAGE) * PAGE;
    const int span = pos + 1 - first;
    const int chunk = ((span + S - 1) / S + PAGE - 1) / PAGE * PAGE;
    const int k_begin = max(first + z * chunk, lo);
    const int k_end = min(first + (z + 1) * chunk, pos + 1);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LPK, kg = lane / LPK;                 // position in the lane group, lane group in the warp
    const int h0 = g * group + ht * GT;                          // first query head of this CTA
    const int heads = min(GT, group - ht * GT);

    float qv[GT][DPL];
#pragma unroll
    for (int i = 0; i < GT; ++i) {
        if (i < heads) load_bf16<DPL>(q + (size_t)row * q_stride + (size_t)(h0 + i) * HD + sub * DPL, qv[i]);
        else {
#pragma unroll
            for (int d = 0; d < DPL; ++d) qv[i][d] = 0.f;
        }
    }
    float m[GT], l[GT], acc[GT][DPL];
#pragma unroll
    for (int i = 0; i < GT; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[i][d] = 0.f;
    }
    const int* table = block_table + (size_t)slot * blocks_per_seq;
    constexpr int STRIDE = DA_WARPS * KPW * DA_KEYS;             // keys the CTA covers per turn
    for (int base = k_begin - (k_begin % DA_KEYS); base < k_end; base += STRIDE) {
        const int k0 = base + (warp * KPW + kg) * DA_KEYS;       // this lane group's four consecutive keys
        float kf[DA_KEYS][DPL], vf[DA_KEYS][DPL];
        bool valid[DA_KEYS];
#pragma unroll
        for (int j = 0; j < DA_KEYS; ++j) {
            const int key = k0 + j;
            valid[j] = key >= k_begin && key < k_end;
            if (valid[j]) {
                const size_t off = (((size_t)table[key / PAGE] * KV + g) * PAGE + (key % PAGE)) * HD + sub * DPL;
                load_bf16<DPL>(k_cache + off, kf[j]);
                load_bf16<DPL>(v_cache + off, vf[j]);
            }
        }
#pragma unroll
        for (int i = 0; i < GT; ++i) {
            float s[DA_KEYS];
            float smax = -INFINITY;
#pragma unroll
            for (int j = 0; j < DA_KEYS; ++j) {
                float d = 0.f;
                if (valid[j]) {
#pragma unroll
                    for (int e = 0; e < DPL; ++e) d = fmaf(qv[i][e], kf[j][e], d);
                }
#pragma unroll
                for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                s[j] = valid[j] ? d * scale : -INFINITY;
                smax = fmaxf(smax, s[j]);
            }
            if (smax == -INFINITY) continue;                     // none of the four keys is visible (same for the lane group)
            const float m_new = fmaxf(m[i], smax);
            const float corr = __expf(m[i] - m_new);             // exp(-inf) = 0 the first time
            float p[DA_KEYS];
            float psum = 0.f;
#pragma unroll
            for (int j = 0; j < DA_KEYS; ++j) { p[j] = valid[j] ? __expf(s[j] - m_new) : 0.f; psum += p[j]; }
            l[i] = l[i] * corr + psum;
            m[i] = m_new;
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                float a = acc[i][e] * corr;
#pragma unroll
                for (int j = 0; j < DA_KEYS; ++j)
                    if (valid[j]) a = fmaf(p[j], vf[j][e], a);
                acc[i][e] = a;
            }
        }
    }
    // merge the lane groups of the warp (lanes with equal `sub` hold the same dimensions)
#pragma unroll
    for (int i = 0; i < GT; ++i) {
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) {
            const float m_o = __shfl_xor_sync(0xffffffffu, m[i], o);
            const float l_o = __shfl_xor_sync(0xffffffffu, l[i], o);
            const float m_new = fmaxf(m[i], m_o);
            const float c_self = m[i] == -INFINITY ? 0.f : __expf(m[i] - m_new);
            const float c_other = m_o == -INFINITY ? 0.f : __expf(m_o - m_new);
            l[i] = l[i] * c_self + l_o * c_other;
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                const float a_o = __shfl_xor_sync(0xffffffffu, acc[i][e], o);
                acc[i][e] = acc[i][e] * c_self + a_o * c_other;
            }
            m[i] = m_new;
        }
        if (kg == 0) {
            if (sub == 0) { sm_m[warp][i] = m[i]; sm_l[warp][i] = l[i]; }
#pragma unroll
            for (int e = 0; e < DPL; ++e) sm_o[warp][i][sub * DPL + e] = acc[i][e];
        }
    }
    __syncthreads();
    // merge the warps; thread t owns (head t / HD..., dimension): GT * HD outputs over 128 threads
    for (int idx = threadIdx.x; idx < heads * HD; idx += DA_WARPS * 32) {
        const int i = idx / HD, d = idx % HD;
        float M = sm_m[0][i];
#pragma unroll
        for (int w = 1; w < DA_WARPS; ++w) M = fmaxf(M, sm_m[w][i]);
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < DA_WARPS; ++w) {
            const float c = sm_m[w][i] == -INFINITY ? 0.f : __expf(sm_m[w][i] - M);
            L += sm_l[w][i] * c;
            o += sm_o[w][i][d] * c;
        }
        const int h = h0 + i;
        if (S == 1) {
            out[((size_t)row * H + h) * HD + d] = __float2bfloat16_rn(o / L);
        } else {
            const size_t pi = ((size_t)row * H + h) * S + z;
            partial_o[pi * HD + d] = o;
            if (d == 0) { partial_ml[pi * 2] = M; partial_ml[pi * 2 + 1] = L; }
        }
    }
}

template <int HD>
__global__ void decode_combine_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                      const int* __restrict__ token_slot, bf16* __restrict__ out, int H, int S) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, h = blockIdx.y;
    if (token_slot[row] < 0) return;
    const size_t base = ((size_t)row * H + h) * S;
    float M = -INFINITY;
    for (int z = 0; z < S; ++z) M = fmaxf(M, partial_ml[(base + z) * 2]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float L = 0.f, o = 0.f;
        for (int z = 0; z < S; ++z) {
            const float mz = partial_ml[(base + z) * 2];
            const float c = mz == -INFINITY ? 0.f : __expf(mz - M);
            L += partial_ml[(base + z) * 2 + 1] * c;
            o += partial_o[(base + z) * HD + d] * c;
        }
        out[((size_t)row * H + h) * HD + d] = __float2bfloat16_rn(o / L);
    }
}

template <int HD, int LPK>
static int launch_decode(const bf16* q, int q_stride, bf16* out, const bf16* k, const bf16* v, const int* table,
                         int bps, const int* positions, const int* token_slot, float* po, float* pml, int rows, int H,
                         int KV, float scale, int window, int S, cudaStream_t stream) {
    const int group = H / KV;
    const int gt = group >= 3 ? 4 : group;                      // 1, 2 or 4 heads per CTA
    const int tiles = (group + gt - 1) / gt;
    const dim3 grid(rows, KV * tiles, S);
    if (grid.y > 65535 || grid.z > 65535) return KL_ERR_BAD_SIZE;
#define KL_DA_LAUNCH(GT)                                                                                              \
    launch_kernel(decode_attention_kernel<HD, LPK, GT>, grid, DA_WARPS * 32, 0, stream, q, q_stride, out, k, v, table, bps,        \
        positions, token_slot, po, pml, H, KV, scale, window)
    if (gt == 1) KL_DA_LAUNCH(1);
    else if (gt == 2) KL_DA_LAUNCH(2);
    else KL_DA_LAUNCH(4);
#undef KL_DA_LAUNCH
    KL_LAUNCH_CHECK();
    if (S > 1) {
        launch_kernel(decode_combine_kernel<HD>, dim3(rows, H), HD < 128 ? 32 : 128, 0, stream, po, pml, token_slot, out, H, S);
        KL_LAUNCH_CHECK();
    }
    return KL_OK;
}

}  // namespace kl

using namespace kl;

// One query token per row.  Head sizes 16, 32, 64, 128 and 256; others: KL_ERR_BAD_SIZE (the
// caller then uses the plain attention kernel).  With splits > 1 the caller provides
// partial_o [rows, H, splits, hd] and partial_ml [rows, H, splits, 2] float32 scratch.
KL_API int kl_attention_decode(const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,
                               const int* block_table, int blocks_per_seq, const int* positions,
                               const int* token_slot, float* partial_o, float* partial_ml, int rows, int H, int KV,
                               int hd, float scale, int window, int splits, cudaStream_t stream) {
    if (rows <= 0) return KL_OK;
    if (KV <= 0 || H % KV || splits < 1) return KL_ERR_BAD_SIZE;
    if (splits > 1 && (partial_o == nullptr || partial_ml == nullptr)) return KL_ERR_BAD_SIZE;
    if (q_stride % 8 || ((uintptr_t)q & 15)) return KL_ERR_BAD_ALIGN;
#define KL_DA(HD, LPK)                                                                                                \
    return launch_decode<HD, LPK>((const bf16*)q, q_stride, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache,     \
                                  block_table, blocks_per_seq, positions, token_slot, partial_o, partial_ml, rows, H,  \
                                  KV, scale, window, splits, stream)
    switch (hd) {
        case 16: KL_DA(16, 2);
        case 32: KL_DA(32, 4);
        case 64: KL_DA(64, 8);
        case 128: KL_DA(128, 16);
        case 256: KL_DA(256, 32);
        default: return KL_ERR_BAD_SIZE;
    }
#undef KL_DA
}

// ------------------------------------------------------------------------------------------
// The variant that allocates nothing (see attention_decode_noalloc.h for who needs it and why).
#include "attention_decode_noalloc.h"
#include <stdio.h>

// Scratch for the splits' partial results.  In host code this name is only a stand-in for the
// device symbol, not a device address: the address is asked for once per device below.
static __device__ __align__(256) float g_decode_noalloc_scratch[KL_DECODE_NOALLOC_FLOATS];

static constexpr int KL_MAX_DEVICES = 64;
static float* g_decode_noalloc_ptr[KL_MAX_DEVICES] = {nullptr};

KL_API int kl_attention_decode_noalloc(const void* q, int q_stride, void* out, const void* k_cache,
                                       const void* v_cache, const int* block_table, int blocks_per_seq,
                                       const int* positions, const int* token_slot, int rows, int H, int KV, int hd,
                                       float scale, int window, int splits, cudaStream_t stream) {
    if (rows <= 0) return KL_OK;
    if (splits < 1 || H <= 0 || hd <= 0) return KL_ERR_BAD_SIZE;
    const long long need = (long long)rows * H * splits * (hd + 2);
    if (need > (long long)KL_DECODE_NOALLOC_FLOATS) {
        fprintf(stderr, "[kuiperllama_b200] kl_attention_decode_noalloc: rows %d x heads %d x splits %d x (head_dim %d + 2) = "
                        "%lld float32 values of scratch exceed the built-in %d; use fewer splits or kl_attention_decode\n",
                rows, H, splits, hd, need, KL_DECODE_NOALLOC_FLOATS);
        return KL_ERR_BAD_SIZE;
    }
    int dev = -1;
    KL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= KL_MAX_DEVICES) return KL_ERR_SETUP;
    if (g_decode_noalloc_ptr[dev] == nullptr) {
        // First call on this device (it is the current one): the array's address there.
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_decode_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            fprintf(stderr, "[kuiperllama_b200] kl_attention_decode_noalloc: cudaGetSymbolAddress failed: %s\n",
                    cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : KL_ERR_SETUP;
        }
        g_decode_noalloc_ptr[dev] = p;
    }
    float* partial_o = g_decode_noalloc_ptr[dev];                       // [rows, H, splits, hd]
    float* partial_ml = partial_o + (size_t)rows * H * splits * hd;     // [rows, H, splits, 2]
    return kl_attention_decode(q, q_stride, out, k_cache, v_cache, block_table, blocks_per_seq, positions, token_slot,
                               partial_o, partial_ml, rows, H, KV, hd, scale, window, splits, stream);
}
