// Rotary position encoding fused with the cache write.
//
// For every token of the step: rotate its query heads in place, rotate its key heads and
// store them in the paged cache, and store its value heads unrotated.  Pairs are
// (j, j + rot/2) inside each head (the half-split layout of HF weights, as
// ExiledOfCode/KuiperLLama's Llama-3 build rotates them, rope_kernel.cu:5-36; its CPU twin
// cpu/rope_kernel.cpp:25-41).  The angle is float(position) * inv_freq[j] in 32 bits with
// sincosf; inv_freq comes from the configuration (theta and scaling are not constants here,
// unlike rope_kernel.cu:42,128).  Every thread checks its own bounds (the reference guard
// `idx > total_pairs`, rope_kernel.cu:13, lets one thread past the end).
#include "common.cuh"

namespace kl {

// qkv: [tokens, (H + 2 KV) * hd], query heads first, then key heads, then value heads.
// With n_partials > 0 the projections arrive as float32 partial sums
// [n_partials][tokens][(H + 2 KV) * hd] of a product whose K range was cut: they are added in
// ascending order here, rotated in float32, and qkv only receives the rotated queries.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const float* __restrict__ partials, int n_partials,
                                     size_t partial_stride, const float* __restrict__ inv_freq, int rot,
                                     const int* __restrict__ positions, const int* __restrict__ token_slot,
                                     const int* __restrict__ block_table, int blocks_per_seq,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     int H, int KV, int hd, int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;                                   // a padding row
    const int pos = positions[t];
    const int width = (H + 2 * KV) * hd;
    T* row = qkv + (size_t)t * width;
    const float* prow = n_partials > 0 ? partials + (size_t)t * width : nullptr;
    auto value = [&](int idx) {                             // element idx of this token's q|k|v row, in float32
        if (prow == nullptr) return to_f32(row[idx]);
        float a = 0.f;
        int z = 0;
        for (; z + 4 <= n_partials; z += 4) {               // four loads in flight, added in ascending order
            const float p0 = prow[(size_t)z * partial_stride + idx], p1 = prow[(size_t)(z + 1) * partial_stride + idx];
            const float p2 = prow[(size_t)(z + 2) * partial_stride + idx], p3 = prow[(size_t)(z + 3) * partial_stride + idx];
            a = (((a + p0) + p1) + p2) + p3;
        }
        for (; z < n_partials; ++z) a += prow[(size_t)z * partial_stride + idx];
        return a;
    };
    const int half = hd / 2;                                // work items per head: hd/2 pairs of lanes
    const int rhalf = rot / 2;
    if (prow != nullptr && rot != hd) {
        // partial or no rotation: first put the summed row down, then go on as without partials
        for (int idx = threadIdx.x; idx < width; idx += blockDim.x) {
            float a = 0.f;
            for (int z = 0; z < n_partials; ++z) a += prow[(size_t)z * partial_stride + idx];
            row[idx] = from_f32<T>(a);
        }
        prow = nullptr;
        __syncthreads();
    }
    // Full rotation (the usual case): the CTAs of a token (gridDim.y of them) share its work
    // items, first the (head, j) pairs of queries and keys (element j and element j + hd/2 are
    // handled together, so each thread owns what it reads and writes), then the value elements.
    const int n_qk = (H + KV) * half;
    if constexpr (sizeof(T) == 2) {
        if (rot == hd && prow == nullptr && (half & 7) == 0) {
            // bfloat16 rows without partial sums (prefill): eight pairs per thread, 16-byte accesses
            const int h8 = half >> 3;                       // groups of eight pairs per head
            const int n_qk8 = (H + KV) * h8;
            const int total = n_qk8 + (write_kv ? KV * hd / 8 : 0);
            for (int w = blockIdx.y * blockDim.x + threadIdx.x; w < total; w += gridDim.y * blockDim.x) {
                if (w < n_qk8) {
                    const int head = w / h8, j0 = (w - head * h8) << 3;
                    if (head >= H && !write_kv) continue;
                    T* h = row + (size_t)head * hd;
                    uint4 ra = *reinterpret_cast<const uint4*>(h + j0), rb = *reinterpret_cast<const uint4*>(h + j0 + half);
                    __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&ra);
                    __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&rb);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 a = __bfloat1622float2(pa[e]), b = __bfloat1622float2(pb[e]);
                        float s0, c0, s1, c1;
                        sincosf((float)pos * inv_freq[j0 + 2 * e], &s0, &c0);
                        sincosf((float)pos * inv_freq[j0 + 2 * e + 1], &s1, &c1);
                        pa[e] = __floats2bfloat162_rn(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
                        pb[e] = __floats2bfloat162_rn(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
                    }
                    T* dst = head < H ? h : (T*)k_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, head - H, KV, hd);
                    *reinterpret_cast<uint4*>(dst + j0) = ra;
                    *reinterpret_cast<uint4*>(dst + j0 + half) = rb;
                } else {
                    const int idx = (w - n_qk8) << 3;
                    const int g = idx / hd, e = idx - g * hd;
                    T* dst = (T*)v_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, g, KV, hd);
                    *reinterpret_cast<uint4*>(dst + e) = *reinterpret_cast<const uint4*>(row + (size_t)(H + KV) * hd + idx);
                }
            }
            return;
        }
    }
    if (rot == hd) {
        const int total = n_qk + (write_kv ? KV * hd : 0);
        for (int w = blockIdx.y * blockDim.x + threadIdx.x; w < total; w += gridDim.y * blockDim.x) {
            if (w < n_qk) {
                const int head = w / half;
                const int j = w - head * half;
                if (head >= H && !write_kv) continue;
                const float a = value(head * hd + j), b = value(head * hd + j + half);
                float sn, cs;
                sincosf((float)pos * inv_freq[j], &sn, &cs);
                const float v0 = a * cs - b * sn, v1 = b * cs + a * sn;
                if (head < H) {
                    T* h = row + (size_t)head * hd;
                    h[j] = from_f32<T>(v0);
                    h[j + half] = from_f32<T>(v1);
                } else {
                    T* dst = k_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, head - H, KV, hd);
                    dst[j] = from_f32<T>(v0);
                    dst[j + half] = from_f32<T>(v1);
                }
            } else {
                const int idx = w - n_qk;
                const int g = idx / hd, e = idx - g * hd;
                T* dst = v_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, g, KV, hd);
                dst[e] = from_f32<T>(value((H + KV) * hd + idx));
            }
        }
        return;
    }
    {
        // Partial or absent rotation (one CTA per token): pairs (j, j + rot/2) for j < rot/2; the
        // rest passes through.
        const int n_pairs = (H + KV) * rhalf;
        for (int idx = threadIdx.x; idx < n_pairs; idx += blockDim.x) {
            const int head = idx / rhalf;
            const int j = idx - head * rhalf;
            T* h = row + (size_t)head * hd;
            float s, c;
            sincosf((float)pos * inv_freq[j], &s, &c);
            const float a = to_f32(h[j]), b = to_f32(h[j + rhalf]);
            h[j] = from_f32<T>(a * c - b * s);
            h[j + rhalf] = from_f32<T>(b * c + a * s);
        }
        __syncthreads();
        if (write_kv) {
            for (int idx = threadIdx.x; idx < KV * hd; idx += blockDim.x) {
                const int g = idx / hd, e = idx - g * hd;
                T* dst = k_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, g, KV, hd);
                dst[e] = row[(size_t)(H + g) * hd + e];
            }
        }
    }
    if (write_kv) {
        for (int idx = threadIdx.x; idx < KV * hd; idx += blockDim.x) {
            const int g = idx / hd, e = idx - g * hd;
            T* dst = v_cache + cache_row_offset(block_table, blocks_per_seq, slot, pos, g, KV, hd);
            dst[e] = from_f32<T>(value((H + KV) * hd + idx));
        }
    }
}

}  // namespace kl

using namespace kl;

KL_API int kl_rope_kv_write(void* qkv, const float* partials, int n_partials, long long partial_stride,
                            const float* inv_freq, int rotary_dim, const int* positions,
                            const int* token_slot, const int* block_table, int blocks_per_seq, void* k_cache,
                            void* v_cache, int n_tokens, int H, int KV, int hd, int write_kv, int dtype,
                            cudaStream_t stream) {
    if (n_tokens <= 0) return KL_OK;
    if (hd % 2 || rotary_dim % 2 || rotary_dim > hd || rotary_dim < 0) return KL_ERR_BAD_SIZE;
    if (rotary_dim > 0 && inv_freq == nullptr) return KL_ERR_BAD_SIZE;
    if (n_partials < 0 || (n_partials > 0 && partials == nullptr)) return KL_ERR_BAD_SIZE;
    const int work = (H + KV) * hd / 2 + (write_kv ? KV * hd : 0);
    const int threads = work >= 1024 ? 256 : (work >= 256 ? 128 : 64);
    // full rotation: a token's work is spread over several CTAs (one item per thread; rows of
    // bfloat16 without partial sums take eight items per thread)
    const bool vec = dtype == KL_BF16 && n_partials == 0 && rotary_dim == hd && (hd % 16) == 0 &&
                     (((H + 2 * KV) * hd) % 8) == 0 && ((uintptr_t)qkv & 15) == 0;
    const int items = vec ? (work + 7) / 8 : work;
    const int ctas = rotary_dim == hd ? (items + threads - 1) / threads : 1;
    if (dtype == KL_F32)
        launch_kernel(rope_kv_write_kernel<float>, dim3(n_tokens, ctas), threads, 0, stream, (float*)qkv, partials, n_partials,
            (size_t)partial_stride, inv_freq, rotary_dim, positions,
            token_slot, block_table, blocks_per_seq, (float*)k_cache, (float*)v_cache, H, KV, hd, write_kv);
    else if (dtype == KL_BF16)
        launch_kernel(rope_kv_write_kernel<bf16>, dim3(n_tokens, ctas), threads, 0, stream, (bf16*)qkv, partials, n_partials,
            (size_t)partial_stride, inv_freq, rotary_dim, positions,
            token_slot, block_table, blocks_per_seq, (bf16*)k_cache, (bf16*)v_cache, H, KV, hd, write_kv);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}
