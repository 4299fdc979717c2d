// Picking the next token of every row of a [rows, vocab] float32 logits matrix on the device.
//
// * argmax: the largest logit, the lowest index among equals, as ExiledOfCode/KuiperLLama's
//   sampler (argmax_sampler.cpp:5-13, argmax_kernel.cu:13-18); one CTA per row here, and the
//   result stays on the device for the next step.
// * temperature (and top-k): p = softmax(logits / T) over the logits that are not below the
//   k-th largest (KuiperLLama has this only in tools/model.py:327-339), then an inverse-CDF
//   draw with u from a counter-based generator keyed by (seed, request id, step), so that a
//   request's tokens do not depend on what else is in the batch.
#include "common.cuh"

namespace kl {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ unsigned int ordered_key(float v) {
    const unsigned int b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);       // ascending in v
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_rows_kernel(const float* __restrict__ logits, size_t row_stride, int vocab, int* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* x = logits + (size_t)blockIdx.x * row_stride;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = x[i];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        const int nwarps = blockDim.x >> 5;
        best = lane < nwarps ? sv[lane] : -INFINITY;
        best_i = lane < nwarps ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        // all logits NaN or -inf: index 0
        if (lane == 0) out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
    }
}

// Two-stage argmax for wide rows: grid (chunks, rows) writes each chunk's best (value, index),
// then one warp per row picks among the chunks.  Ties go to the lower index in both stages.
constexpr int ARGMAX_CHUNK = 4096;

__global__ void __launch_bounds__(256)
argmax_chunks_kernel(const float* __restrict__ logits, size_t row_stride, int vocab, float* __restrict__ best_v,
                     int* __restrict__ best_i) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sv[8];
    __shared__ int si[8];
    const int row = blockIdx.y, chunk = blockIdx.x;
    const float* x = logits + (size_t)row * row_stride;
    const int begin = chunk * ARGMAX_CHUNK, end = min(begin + ARGMAX_CHUNK, vocab);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = x[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
        best_v[(size_t)row * gridDim.x + chunk] = best;
        best_i[(size_t)row * gridDim.x + chunk] = bi;
    }
}

__global__ void argmax_pick_kernel(const float* __restrict__ best_v, const int* __restrict__ best_i, int chunks,
                                   int* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < chunks; c += 32) {
        const float v = best_v[(size_t)row * chunks + c];
        const int i = best_i[(size_t)row * chunks + c];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

// The uniform draw in [0, 1) of (seed, request, step): a 64-bit mix, top 24 bits.
__device__ __forceinline__ float uniform_from_counter(unsigned long long seed, unsigned long long request,
                                                      unsigned long long step) {
    unsigned long long z = seed * 0x9E3779B97F4A7C15ull + request * 0xBF58476D1CE4E5B9ull +
                           step * 0x94D049BB133111EBull + 0x2545F4914F6CDD1Dull;
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// Four consecutive logits of a row starting at element i (a multiple of 4); elements past the
// vocabulary read as -inf.  `vec`: the row starts on a 16-byte boundary, so one load does it.
__device__ __forceinline__ float4 load4(const float* __restrict__ x, int i, int vocab, bool vec) {
    if (vec && i + 3 < vocab) return *reinterpret_cast<const float4*>(x + i);
    float4 v;
    v.x = i < vocab ? x[i] : -INFINITY;
    v.y = i + 1 < vocab ? x[i + 1] : -INFINITY;
    v.z = i + 2 < vocab ? x[i + 2] : -INFINITY;
    v.w = i + 3 < vocab ? x[i + 3] : -INFINITY;
    return v;
}

constexpr int SAMPLE_TILE = SAMPLE_THREADS * 4;       // logits a CTA reads per pass over its threads
constexpr int SAMPLE_MAX_TILES = 256;                 // rows of up to 2^20 logits

// One CTA per row.  Every pass reads the row in tiles of 4,096 consecutive logits, thread t taking
// the four at 4 t, so that loads are coalesced and a warp owns 128 consecutive logits of a tile:
//   1. with top-k, the k-th largest logit as an ordered key, by four passes of an 8-bit radix
//      select over shared-memory histograms;
//   2. the maximum;
//   3. sum of exp((x - max) / T) over the kept logits per (tile, warp), then per tile and in all,
//      added in index order in float64;
//   4. the (tile, warp) whose stretch of the cumulative sum holds u * total, and inside that warp
//      the first logit at which the running sum passes it.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, size_t row_stride, int vocab, float temperature, int top_k,
                   unsigned long long seed, const int* __restrict__ request_ids, const int* __restrict__ steps,
                   int* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float fscratch[33];
    __shared__ unsigned int hist[256];
    __shared__ unsigned int sel_prefix, sel_remaining;
    __shared__ float warp_sums[SAMPLE_MAX_TILES][32];
    __shared__ double tile_sums[SAMPLE_MAX_TILES];
    __shared__ int pick_tile, pick_warp, pick_last, chosen;
    __shared__ double pick_base, pick_target;
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* x = logits + (size_t)row * row_stride;
    const bool vec = (((uintptr_t)x) & 15) == 0;
    const float inv_t = 1.0f / temperature;
    const int n_tiles = (vocab + SAMPLE_TILE - 1) / SAMPLE_TILE;

    // 1. threshold of the top-k cut as an ordered key; 0 keeps everything
    unsigned int th = 0u;
    if (top_k > 0 && top_k < vocab) {
        if (threadIdx.x == 0) { sel_prefix = 0u; sel_remaining = (unsigned int)top_k; }
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (threadIdx.x < 256) hist[threadIdx.x] = 0u;
            __syncthreads();
            const unsigned int prefix = sel_prefix;
            const unsigned int mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int t = 0; t < n_tiles; ++t) {
                const int i = t * SAMPLE_TILE + threadIdx.x * 4;
                const float4 v = load4(x, i, vocab, vec);
                const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const unsigned int key = ordered_key(e[j]);
                    if (i + j < vocab && (key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
                }
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                // the bin that holds the k-th largest among the keys with this prefix, from the top
                unsigned int remaining = sel_remaining, b = 255u;
                for (;; --b) {
                    if (hist[b] >= remaining || b == 0u) break;
                    remaining -= hist[b];
                }
                sel_prefix = prefix | (b << shift);
                sel_remaining = remaining;
            }
            __syncthreads();
        }
        th = sel_prefix;
    }

    // 2. the maximum (the largest logit is always kept)
    float m = -INFINITY;
    for (int t = 0; t < n_tiles; ++t) {
        const float4 v = load4(x, t * SAMPLE_TILE + threadIdx.x * 4, vocab, vec);
        m = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    }
    m = block_max(m, fscratch) * inv_t;

    // 3. sums per (tile, warp)
    auto weight = [&](float v, int i) -> float {
        return (i < vocab && ordered_key(v) >= th) ? expf(v * inv_t - m) : 0.f;
    };
    for (int t = 0; t < n_tiles; ++t) {
        const int i = t * SAMPLE_TILE + threadIdx.x * 4;
        const float4 v = load4(x, i, vocab, vec);
        float s = (weight(v.x, i) + weight(v.y, i + 1)) + (weight(v.z, i + 2) + weight(v.w, i + 3));
        s = warp_sum(s);
        if (lane == 0) warp_sums[t][warp] = s;
    }
    if (threadIdx.x == 0) chosen = -1;
    __syncthreads();
    if (threadIdx.x < n_tiles) {
        double s = 0.0;
        for (int w = 0; w < 32; ++w) s += (double)warp_sums[threadIdx.x][w];
        tile_sums[threadIdx.x] = s;
    }
    __syncthreads();

    // 4. where u * total falls
    if (threadIdx.x == 0) {
        double total = 0.0;
        for (int t = 0; t < n_tiles; ++t) total += tile_sums[t];
        const double target = (double)uniform_from_counter(seed, (unsigned long long)request_ids[row],
                                                           (unsigned long long)steps[row]) * total;
        double run = 0.0;
        int pt = -1, pw = -1;
        for (int t = 0; t < n_tiles && pt < 0; ++t) {
            if (tile_sums[t] > 0.0 && target < run + tile_sums[t]) {
                for (int w = 0; w < 32 && pw < 0; ++w) {
                    const double s = (double)warp_sums[t][w];
                    if (s > 0.0 && target < run + s) pw = w;
                    else run += s;
                }
                if (pw >= 0) pt = t;
                // else rounding: the warp sums of this tile end below the target; go on with the next tile
            } else {
                run += tile_sums[t];
            }
        }
        int last = 0;
        if (pt < 0) {                                       // rounding put the target past the end: the last kept logit of all
            last = 1;
            for (int t = n_tiles - 1; t >= 0 && pt < 0; --t)
                for (int w = 31; w >= 0 && pt < 0; --w)
                    if (warp_sums[t][w] > 0.f) { pt = t; pw = w; }
            if (pt < 0) { pt = 0; pw = 0; }
        }
        pick_tile = pt; pick_warp = pw; pick_base = run; pick_target = target; pick_last = last;
    }
    __syncthreads();
    if (warp == pick_warp) {
        const double target = pick_target;
        const int i = pick_tile * SAMPLE_TILE + threadIdx.x * 4;
        const float4 v = load4(x, i, vocab, vec);
        const float e[4] = {weight(v.x, i), weight(v.y, i + 1), weight(v.z, i + 2), weight(v.w, i + 3)};
        // inclusive running sums in index order: lanes in order, four logits inside a lane
        double mine = ((double)e[0] + (double)e[1]) + ((double)e[2] + (double)e[3]);
        double incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double other = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += other;
        }
        double run = pick_base + (incl - mine);
        int pick = -1, last_kept = -1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (e[j] > 0.f) {
                last_kept = i + j;
                run += (double)e[j];
                if (pick < 0 && run > target && !pick_last) pick = i + j;
            }
        }
        // the first lane with a pick wins; else the warp's last kept logit
        const unsigned int has = __ballot_sync(0xffffffffu, pick >= 0);
        const unsigned int kept = __ballot_sync(0xffffffffu, last_kept >= 0);
        int result;
        if (has) result = __shfl_sync(0xffffffffu, pick, __ffs(has) - 1);
        else if (kept) result = __shfl_sync(0xffffffffu, last_kept, 31 - __clz(kept));
        else result = 0;
        if (lane == 0) chosen = result;
    }
    __syncthreads();
    if (threadIdx.x == 0) out[row] = chosen < 0 ? 0 : chosen;
}

// out[row] = log softmax(logits[row])[tokens[row]] = x[token] - max - log(sum exp(x - max)), in
// float32; a token outside the vocabulary gives -inf.  (KuiperLLama's Python model has the same
// softmax over the last position's logits, tools/model.py:327-339.)
__global__ void __launch_bounds__(SAMPLE_THREADS)
token_logprob_kernel(const float* __restrict__ logits, size_t row_stride, int vocab, const int* __restrict__ tokens,
                     float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const float* x = logits + (size_t)blockIdx.x * row_stride;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, x[i]);
    m = block_max(m, scratch);
    float s = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) s += expf(x[i] - m);
    s = block_sum(s, scratch);
    if (threadIdx.x == 0) {
        const int t = tokens[blockIdx.x];
        out[blockIdx.x] = (t >= 0 && t < vocab) ? (x[t] - m) - logf(s) : -INFINITY;
    }
}

}  // namespace kl

using namespace kl;

KL_API int kl_token_logprob(const float* logits, long long row_stride, int rows, int vocab, const int* tokens, float* out,
                            cudaStream_t stream) {
    if (rows <= 0) return KL_OK;
    if (vocab <= 0) return KL_ERR_BAD_SIZE;
    launch_kernel(token_logprob_kernel, rows, SAMPLE_THREADS, 0, stream, logits, (size_t)row_stride, vocab, tokens, out);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// Chunks a row is cut into by the two-stage argmax (the caller sizes scratch with it).
KL_API int kl_argmax_chunks(int vocab) { return (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK; }

// scratch_v / scratch_i: [rows, kl_argmax_chunks(vocab)] float32 / int32, or null for the
// single-stage kernel (one CTA per row).
KL_API int kl_argmax_rows(const float* logits, long long row_stride, int rows, int vocab, int* out, float* scratch_v,
                          int* scratch_i, cudaStream_t stream) {
    if (rows <= 0) return KL_OK;
    if (vocab <= 0) return KL_ERR_BAD_SIZE;
    if (scratch_v == nullptr || scratch_i == nullptr || rows > 65535) {
        launch_kernel(argmax_rows_kernel, rows, SAMPLE_THREADS, 0, stream, logits, (size_t)row_stride, vocab, out);
        KL_LAUNCH_CHECK();
        return KL_OK;
    }
    const int chunks = (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    launch_kernel(argmax_chunks_kernel, dim3(chunks, rows), 256, 0, stream, logits, (size_t)row_stride, vocab, scratch_v, scratch_i);
    KL_LAUNCH_CHECK();
    launch_kernel(argmax_pick_kernel, rows, 32, 0, stream, scratch_v, scratch_i, chunks, out);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// temperature > 0.  top_k <= 0 or >= vocab: no cut.
KL_API int kl_sample_rows(const float* logits, long long row_stride, int rows, int vocab, float temperature,
                          int top_k, unsigned long long seed, const int* request_ids, const int* steps, int* out,
                          cudaStream_t stream) {
    if (rows <= 0) return KL_OK;
    if (vocab <= 0 || !(temperature > 0.f) || vocab > SAMPLE_TILE * SAMPLE_MAX_TILES) return KL_ERR_BAD_SIZE;
    launch_kernel(sample_rows_kernel, rows, SAMPLE_THREADS, 0, stream, logits, (size_t)row_stride, vocab, temperature, top_k,
                                                            seed, request_ids, steps, out);
    KL_LAUNCH_CHECK();
    return KL_OK;
}
