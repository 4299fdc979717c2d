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

__device__ __forceinline__ int block_count(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int t = lane < nwarps ? scratch[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, size_t row_stride, int vocab, float temperature, int top_k,
                   unsigned long long seed, const int* __restrict__ request_ids, const int* __restrict__ steps,
                   int* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float fscratch[33];
    __shared__ int iscratch[33];
    __shared__ double part[SAMPLE_THREADS];
    __shared__ int chosen;
    __shared__ double total_s;
    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * row_stride;
    const float inv_t = 1.0f / temperature;

    // threshold of the top-k cut as an ordered key; 0 keeps everything
    unsigned int th = 0u;
    if (top_k > 0 && top_k < vocab) {
        // the largest key K with count(key >= K) >= top_k, bit by bit from the top
        unsigned int k = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int trial = k | (1u << bit);
            int c = 0;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += ordered_key(x[i]) >= trial;
            if (block_count(c, iscratch) >= top_k) k = trial;
        }
        th = k;
    }
    float m = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, x[i]);
    m = block_max(m, fscratch) * inv_t;

    // every thread owns one contiguous segment, so the cumulative sum runs in index order
    const int per = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = min(threadIdx.x * per, vocab), end = min(begin + per, vocab);
    double s = 0.0;
    for (int i = begin; i < end; ++i)
        if (ordered_key(x[i]) >= th) s += (double)expf(x[i] * inv_t - m);
    part[threadIdx.x] = s;
    if (threadIdx.x == 0) chosen = -1;
    __syncthreads();
    if (threadIdx.x == 0) {                                  // exclusive scan of 1024 partial sums
        double run = 0.0;
        for (int i = 0; i < blockDim.x; ++i) { const double p = part[i]; part[i] = run; run += p; }
        part[0] = 0.0;
        total_s = run;
    }
    __syncthreads();
    const double total = total_s;
    const double target = (double)uniform_from_counter(seed, (unsigned long long)request_ids[row],
                                                       (unsigned long long)steps[row]) * total;
    const double excl = part[threadIdx.x];
    if (s > 0.0 && excl <= target && target < excl + s) {
        double run = excl;
        int pick = -1, last_kept = -1;
        for (int i = begin; i < end && pick < 0; ++i) {
            if (ordered_key(x[i]) >= th) {
                last_kept = i;
                run += (double)expf(x[i] * inv_t - m);
                if (run > target) pick = i;
            }
        }
        chosen = pick >= 0 ? pick : last_kept;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int c = chosen;
        if (c < 0) {                                         // rounding put the target past the end: last kept token
            for (int i = vocab - 1; i >= 0 && c < 0; --i)
                if (ordered_key(x[i]) >= th && expf(x[i] * inv_t - m) > 0.f) c = i;
            if (c < 0) c = 0;
        }
        out[row] = c;
    }
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
    if (vocab <= 0 || !(temperature > 0.f)) return KL_ERR_BAD_SIZE;
    launch_kernel(sample_rows_kernel, rows, SAMPLE_THREADS, 0, stream, logits, (size_t)row_stride, vocab, temperature, top_k,
                                                            seed, request_ids, steps, out);
    KL_LAUNCH_CHECK();
    return KL_OK;
}
