// Causal grouped-query attention of a prefill step on the fifth-generation tensor cores
// (bfloat16, head size 128): both products of flash attention as tcgen05.mma with their
// results in tensor memory.
//
// Per head: s_t = (q . k_t) * scale for lo <= t <= pos, softmax with the maximum subtracted,
// o = sum p_t v_t (ExiledOfCode/KuiperLLama mha_kernel.cu:61,74-106: one CTA per head, one
// token, scalar FMAs).
//
// A CTA owns 128 query rows of one sequence and one kv head; a row is (token, head of the kv
// group).  Warp 0 loads with TMA: the queries once (a 3-D box over [token, head, dim]), then
// key blocks of two cache pages (128 keys) into a two-stage ring, keys and values as 64-wide
// swizzled slabs.  Warp 1 issues the MMAs: S = Q K^T (M 128, N keys, K 128) into one of two
// score buffers in tensor memory, and O_j = P_j V_j (M 128, N 128, K keys; V is the MN-major
// operand, straight from its [key][dim] rows) into one of two output buffers.  Warps 2..5 are
// the softmax: thread r owns row r.  It reads its scores from tensor memory twice (maximum,
// then exp2 and sum), writes the probabilities as bfloat16 into a swizzled shared-memory
// tile for the second product, and adds the finished O_j of the block before into its
// float32 accumulator in registers with the correction of that block.  The score buffer,
// the probability tile and the output buffer are double so that the products of block j + 1
// run while block j is in the softmax.
//
// Every wait is bounded, as in gemm_tcgen05.cu.
#include "tcgen05.cuh"
#include "tma_host.cuh"

namespace kl {

constexpr int AT_ROWS = 128;             // query rows per CTA = UMMA M
constexpr int AT_HD = 128;               // head size
constexpr int AT_THREADS = 192;
constexpr uint32_t AT_SLAB = AT_ROWS * 128;            // bytes of a [128 rows][64 elements] swizzled slab
constexpr uint32_t AT_Q_BYTES = 2 * AT_SLAB;           // 32 KB
constexpr uint32_t AT_K_BYTES = 2 * AT_SLAB;           // [128 keys][128 dims] as two slabs
constexpr uint32_t AT_P_BYTES = 2 * AT_SLAB;           // [128 rows][128 keys] as two slabs

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 : : "r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// MN-major operand with the 128-byte swizzle: rows (k) of 128 bytes hold 64 consecutive
// elements of the MN dimension; 8 rows are 1024 bytes apart (stride byte offset); the next 64
// MN elements are `lbo` bytes away (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// D float32, A and B bfloat16, A K-major, B K-major (b_mn = 0) or MN-major (1), M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_ab(int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

struct AttnArgs {
    bf16* out;                 // [rows, H * 128]
    const int* block_table;
    int blocks_per_seq;
    const int* cu_tokens;
    const int* seq_slots;
    const int* seq_starts;
    const int* seq_new;
    int H, KV, Gp;
    float scale_log2;
    int* status;
};

__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, AttnArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_sm = smem;
    uint8_t* k_sm = q_sm + AT_Q_BYTES;                    // [2 stages]
    uint8_t* v_sm = k_sm + 2 * AT_K_BYTES;                // [2 stages]
    uint8_t* p_sm = v_sm + 2 * AT_K_BYTES;                // [2]
    uint64_t* bars = (uint64_t*)(p_sm + 2 * AT_P_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;                         // [2]
    uint64_t* kv_empty = bars + 3;                        // [2]
    uint64_t* s_full = bars + 5;                          // [2]
    uint64_t* p_ready = bars + 7;                         // [2]
    uint64_t* o_full = bars + 9;                          // [2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 11);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y, g = blockIdx.z;
    const int H = args.H, KV = args.KV, Gp = args.Gp, G = H / KV;
    const int BT = AT_ROWS / Gp;
    const int T = args.seq_new[b];
    // long tiles first (CTAs are handed out in ascending blockIdx.x)
    const int t0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BT;
    if (t0 >= T) return;
    const int start = args.seq_starts[b], slot = args.seq_slots[b], row0 = args.cu_tokens[b];
    const int max_pos = start + min(T, t0 + BT) - 1;
    const int n_pages = max_pos / PAGE + 1;
    const int n_blocks = (n_pages + 1) / 2;
    const int* table = args.block_table + (size_t)slot * args.blocks_per_seq;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); mbar_init(&s_full[i], 1);
            mbar_init(&p_ready[i], 4); mbar_init(&o_full[i], 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0 && lane == 0) { prefetch_tmap(&map_q); prefetch_tmap(&map_k); prefetch_tmap(&map_v); }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                                           // q, and this step's keys and values, come from the kernels before

    if (warp == 0) {
        // ---------------------------------------------------------------- loads
        if (elect_one()) {
            mbar_expect_tx(q_full, AT_Q_BYTES);
            tma_load_3d(q_sm, &map_q, q_full, 0, g * G, row0 + t0);
            tma_load_3d(q_sm + AT_SLAB, &map_q, q_full, 64, g * G, row0 + t0);
            int issued = 0;
            for (int j = 0; j < n_blocks; ++j) {
                const int s = j & 1;
                if (j >= 2 && !mbar_wait(&kv_empty[s], ((j >> 1) - 1) & 1, abort_flag, args.status, 11)) break;
                const int pages = min(2, n_pages - 2 * j);
                mbar_expect_tx(&kv_full[s], pages * 2 * (PAGE * 128 * 2));
                for (int pg = 0; pg < pages; ++pg) {
                    const int y = (table[2 * j + pg] * KV + g) * PAGE;
                    for (int h = 0; h < 2; ++h) {
                        tma_load_2d(k_sm + s * AT_K_BYTES + h * AT_SLAB + pg * (PAGE * 128), &map_k, &kv_full[s], h * 64, y);
                        tma_load_2d(v_sm + s * AT_K_BYTES + h * AT_SLAB + pg * (PAGE * 128), &map_v, &kv_full[s], h * 64, y);
                    }
                }
                issued = j + 1;
            }
            if (*abort_flag)
                for (int j = max(0, issued - 2); j < issued; ++j)
                    for (uint32_t t = 0; t < (1u << 20) && !mbar_try_wait(&kv_full[j & 1], (j >> 1) & 1); ++t) {}
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issue
        if (elect_one()) {
            bool ok = mbar_wait(q_full, 0, abort_flag, args.status, 12);
            auto issue_s = [&](int j) {                   // S_j = Q K_j^T into score buffer j & 1
                const int s = j & 1;
                if (!mbar_wait(&kv_full[s], (j >> 1) & 1, abort_flag, args.status, 13)) return false;
                tc_fence_after();
                const int keys = min(2, n_pages - 2 * j) * PAGE;
                const uint32_t idesc = umma_idesc_ab(keys, 0);
#pragma unroll
                for (int ks = 0; ks < AT_HD / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * AT_SLAB + (ks & 3) * 32;
                    umma_bf16(tmem_base + s * 128, smem_desc_sw128(smem_u32(q_sm + off)),
                              smem_desc_sw128(smem_u32(k_sm + s * AT_K_BYTES + off)), idesc, ks > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[s]);
                return true;
            };
            if (ok && n_blocks > 0) ok = issue_s(0);
            for (int j = 0; j < n_blocks && ok; ++j) {
                const int s = j & 1;
                if (j + 1 < n_blocks) { ok = issue_s(j + 1); if (!ok) break; }
                ok = mbar_wait(&p_ready[s], (j >> 1) & 1, abort_flag, args.status, 14);
                if (!ok) break;
                tc_fence_after();
                const int keys = min(2, n_pages - 2 * j) * PAGE;
                const uint32_t idesc = umma_idesc_ab(AT_HD, 1);
                for (int kk = 0; kk < keys / 16; ++kk) {  // O_j = P_j V_j into output buffer j & 1
                    const uint32_t poff = (kk >> 2) * AT_SLAB + (kk & 3) * 32;
                    umma_bf16(tmem_base + 256 + s * 128, smem_desc_sw128(smem_u32(p_sm + s * AT_P_BYTES + poff)),
                              smem_desc_sw128_mn(smem_u32(v_sm + s * AT_K_BYTES + kk * 2048), AT_SLAB), idesc, kk > 0 ? 1u : 0u);
                }
                umma_commit(&o_full[s]);
                umma_commit(&kv_empty[s]);
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax and output: thread r owns row r
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int tl = t0 + r / Gp, hh = r % Gp;
        const bool valid = tl < T && hh < G;
        const int pos = valid ? start + tl : -1;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float acc[AT_HD];
#pragma unroll
        for (int d = 0; d < AT_HD; ++d) acc[d] = 0.f;
        float m = -INFINITY, l = 0.f, corr_prev = 1.f;
        bool ok = true;
        for (int j = 0; j < n_blocks && ok; ++j) {
            const int s = j & 1;
            ok = mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag, args.status, 15);
            if (!ok) break;
            tc_fence_after();
            const int keys = min(2, n_pages - 2 * j) * PAGE;
            const int key0 = 2 * j * PAGE;
            // The same for all lanes of the warp: the tensor-memory loads below are warp-wide
            // instructions and must not sit in branches that lanes take differently.
            const bool need_mask = key0 + keys - 1 > start + t0 || __any_sync(0xffffffffu, !valid);
            // pass 1: the row's maximum of the raw scores (the scale is positive: it commutes with max)
            float mx = -INFINITY;
            uint32_t c32[32];
            if (need_mask) {
                for (int c = 0; c < keys; c += 32) {
                    tmem_ld32(lane_base + s * 128 + c, c32);
                    tmem_ld_wait();
                    const int visible = pos - key0 - c;            // elements 0..visible are seen
#pragma unroll
                    for (int e = 0; e < 32; ++e) mx = fmaxf(mx, e <= visible ? __uint_as_float(c32[e]) : -INFINITY);
                }
            } else {
                for (int c = 0; c < keys; c += 32) {
                    tmem_ld32(lane_base + s * 128 + c, c32);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; e += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(c32[e]), __uint_as_float(c32[e + 1])));
                }
            }
            const float m_new = fmaxf(m, mx * args.scale_log2);
            const float muse = m_new == -INFINITY ? 0.f : m_new;
            const float corr = fast_exp2(m - muse);
            // pass 2: probabilities exp2(score * scale - max), their sum, and the bfloat16 tile for
            // the second product
            float sum = 0.f;
            uint8_t* prow = p_sm + s * AT_P_BYTES + r * 128;
            for (int c = 0; c < keys; c += 32) {
                tmem_ld32(lane_base + s * 128 + c, c32);
                tmem_ld_wait();
                uint32_t packed[16];
                const int visible = need_mask ? pos - key0 - c : 32;
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float p0 = fast_exp2(fmaf(__uint_as_float(c32[e]), args.scale_log2, -muse));
                    float p1 = fast_exp2(fmaf(__uint_as_float(c32[e + 1]), args.scale_log2, -muse));
                    if (need_mask) {
                        if (e > visible) p0 = 0.f;
                        if (e + 1 > visible) p1 = 0.f;
                    }
                    sum += p0 + p1;
                    __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
                    packed[e >> 1] = *reinterpret_cast<uint32_t*>(&pr);
                }
                // 32 keys = four 16-byte chunks of the row's slab (64 keys per slab)
                uint8_t* slab = prow + (c >> 6) * AT_SLAB;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = ((c & 63) >> 3) + q4;
                    *reinterpret_cast<uint4*>(slab + ((chunk ^ (r & 7)) << 4)) =
                        make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
                }
            }
            l = l * corr + sum;
            m = m_new;
            fence_proxy_async();                          // the tile is read by the tensor core (async proxy)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[s]);
            // the block before: its output is complete (or will be soon); add it with its correction
            if (j > 0) {
                const int sp = (j - 1) & 1;
                ok = mbar_wait(&o_full[sp], ((j - 1) >> 1) & 1, abort_flag, args.status, 16);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < AT_HD; c += 32) {
                    tmem_ld32(lane_base + 256 + sp * 128 + c, c32);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[c + e] = acc[c + e] * corr_prev + __uint_as_float(c32[e]);
                }
                // corr_prev was the correction of block j - 1; blocks before it are scaled by it too (done above),
                // and from now on everything accumulated is in the scale of block j - 1's maximum
            }
            corr_prev = corr;
        }
        if (ok && n_blocks > 0) {
            const int j = n_blocks - 1, sp = j & 1;
            ok = mbar_wait(&o_full[sp], (j >> 1) & 1, abort_flag, args.status, 17);
            if (ok) {
                tc_fence_after();
                uint32_t c32[32];
                const float inv = 1.f / l;
                bf16* orow = args.out + ((size_t)(row0 + tl) * H + (g * G + hh)) * AT_HD;
#pragma unroll
                for (int c = 0; c < AT_HD; c += 32) {
                    tmem_ld32(lane_base + 256 + sp * 128 + c, c32);
                    tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int x = 0; x < 4; ++x) {
                                const float a0 = (acc[c + e + 2 * x] * corr_prev + __uint_as_float(c32[e + 2 * x])) * inv;
                                const float a1 = (acc[c + e + 2 * x + 1] * corr_prev + __uint_as_float(c32[e + 2 * x + 1])) * inv;
                                __nv_bfloat162 pr = __floats2bfloat162_rn(a0, a1);
                                w[x] = *reinterpret_cast<uint32_t*>(&pr);
                            }
                            *reinterpret_cast<uint4*>(orow + c + e) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace kl

using namespace kl;

// Prefill attention of a ragged batch (see kl_attention_mma for the arguments' meaning).  Head
// size 128, group sizes that divide 128, no window; q rows 16-byte aligned.  Others:
// KL_ERR_BAD_SIZE / KL_ERR_BAD_ALIGN, and the caller takes the mma.sync kernel.
KL_API int kl_attention_tcgen05(const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,
                                long long n_cache_rows, const int* block_table, int blocks_per_seq, const int* cu_tokens,
                                const int* seq_slots, const int* seq_starts, const int* seq_new, int n_seqs, int max_new,
                                int n_rows, int H, int KV, int hd, float scale, int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return KL_OK;
    if (hd != AT_HD || KV <= 0 || H % KV) return KL_ERR_BAD_SIZE;
    const int G = H / KV;
    int Gp = 1;
    while (Gp < G) Gp <<= 1;
    if (Gp > 128) return KL_ERR_BAD_SIZE;
    if (q_stride % 8 || ((uintptr_t)q & 15)) return KL_ERR_BAD_ALIGN;
    const int BT = AT_ROWS / Gp;
    CUtensorMap mq, mk, mv;
    int rc;
    {
        const long long dims[3] = {hd, H, n_rows}, strides[2] = {hd, q_stride};
        const int box[3] = {64, Gp, BT};
        if ((rc = tma_make_map(&mq, q, 3, dims, strides, box)) != KL_OK) return rc;
    }
    {
        const long long dims[2] = {hd, n_cache_rows}, strides[1] = {hd};
        const int box[2] = {64, PAGE};
        if ((rc = tma_make_map(&mk, k_cache, 2, dims, strides, box)) != KL_OK) return rc;
        if ((rc = tma_make_map(&mv, v_cache, 2, dims, strides, box)) != KL_OK) return rc;
    }
    AttnArgs args{(bf16*)out, block_table, blocks_per_seq, cu_tokens, seq_slots, seq_starts, seq_new, H, KV, Gp,
                  scale * 1.4426950408889634f, status};
    const dim3 grid((max_new + BT - 1) / BT, n_seqs, KV);
    if (grid.y > 65535 || grid.z > 65535) return KL_ERR_BAD_SIZE;
    constexpr size_t smem = AT_Q_BYTES + 4 * AT_K_BYTES + 2 * AT_P_BYTES + 11 * 8 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        KL_CUDA(cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    launch_kernel(attention_tcgen05_kernel, grid, AT_THREADS, smem, stream, mq, mk, mv, args);
    KL_LAUNCH_CHECK();
    return KL_OK;
}
