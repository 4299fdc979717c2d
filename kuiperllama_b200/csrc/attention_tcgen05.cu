// Causal grouped-query attention of a prefill step on the fifth-generation tensor cores
// (bfloat16, head sizes 64 and 128): both products of flash attention as tcgen05.mma with their
// results in tensor memory.
//
// Per head: s_t = (q . k_t) * scale for lo <= t <= pos, softmax with the maximum subtracted,
// o = sum p_t v_t (ExiledOfCode/KuiperLLama mha_kernel.cu:61,74-106: one CTA per head, one
// token, scalar FMAs).
//
// A CTA owns two tiles of 128 query rows of one sequence and one kv head; a row is (token, head
// of the kv group).  Warp 0 loads with TMA: the queries once (3-D boxes over [token, head, dim]),
// then key blocks of two cache pages (128 keys) into a two-stage ring, keys and values as 64-wide
// swizzled slabs.  Warp 1 issues the MMAs: S = Q K^T (M 128, N keys, K head size) into the tile's score
// columns of tensor memory, and O += P V (M 128, N head size, K keys) into the tile's output columns,
// where P is read from tensor memory (the A operand) and V is the MN-major B operand, straight
// from its [key][dim] rows.  Warps 2..5 are the softmax of tile 0, warps 6..9 of tile 1: thread r
// owns row r of its tile.  It reads its 128 scores from tensor memory, takes exp2 against a
// reference maximum, and writes the probabilities back as packed bfloat16 over the scores' first
// 64 columns.  The output stays in tensor memory over all key blocks; a row is rescaled there
// (tcgen05.ld, multiply, tcgen05.st) only when its maximum has grown by more than 2^8 since the
// reference was set, which is rare after the first blocks.  While one tile is in the softmax
// the tensor core works on the other tile's products.
//
// Every wait is bounded, as in gemm_tcgen05.cu.
#include "tcgen05.cuh"
#include "tma_host.cuh"

namespace kl {

constexpr int AT_ROWS = 128;             // query rows per CTA = UMMA M
constexpr int AT_THREADS = 320;          // warp 0 loads, warp 1 issues, warps 2..5 and 6..9: softmax of tiles 0 and 1
constexpr uint32_t AT_SLAB = AT_ROWS * 128;            // bytes of a [128 rows][64 elements] swizzled slab
constexpr float AT_RESCALE = 8.0f;                     // a row is rescaled when its maximum grew by more (log2 units)

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 : : "r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// sm_100 forms that halve the softmax's instruction count: a maximum of three, and float32 pairs
// (two lanes of one 64-bit register) for multiply-add and add.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 : : "r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 : : "r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// A from tensor memory: row = lane, two bfloat16 along K per 32-bit column (the lower half is the
// lower k), so the 16 k of one instruction are 8 columns.
__device__ __forceinline__ void umma_bf16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 : : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
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

// HD: head size, 64 or 128 (one or two 64-wide slabs per row of queries, keys and values).
template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, AttnArgs args) {
    constexpr int AT_HD = HD;
    constexpr int SLABS = HD / 64;
    constexpr uint32_t AT_Q_BYTES = SLABS * AT_SLAB;      // one tile's queries
    constexpr uint32_t AT_K_BYTES = SLABS * AT_SLAB;      // [128 keys][HD dims] as 64-wide slabs
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_sm = smem;                                 // [2 tiles]
    uint8_t* k_sm = q_sm + 2 * AT_Q_BYTES;                // [2 stages]
    uint8_t* v_sm = k_sm + 2 * AT_K_BYTES;                // [2 stages]
    uint64_t* bars = (uint64_t*)(v_sm + 2 * AT_K_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;                         // [2 stages] a key block has landed
    uint64_t* kv_empty = bars + 3;                        // [2 stages] every product that reads it is done
    uint64_t* s_full = bars + 5;                          // [2 tiles] the tile's scores of a block are complete
    uint64_t* p_ready = bars + 7;                         // [2 tiles] its probabilities are in tensor memory (and its output rescaled)
    uint64_t* o_done = bars + 9;                          // [2 tiles] its output holds the block
    uint32_t* tmem_slot = (uint32_t*)(bars + 11);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y, g = blockIdx.x;
    const int H = args.H, KV = args.KV, Gp = args.Gp, G = H / KV;
    const int BT = AT_ROWS / Gp;                          // tokens per tile
    const int T = args.seq_new[b];
    // Long tiles first: CTAs are handed out with blockIdx.x fastest and blockIdx.z slowest, so the
    // token tile is z (descending) and every kv head's and sequence's longest tiles start before
    // anybody's short ones.
    const int t0 = ((int)gridDim.z - 1 - (int)blockIdx.z) * 2 * BT;
    if (t0 >= T) return;
    const int n_tiles = t0 + BT < T ? 2 : 1;
    const int start = args.seq_starts[b], slot = args.seq_slots[b], row0 = args.cu_tokens[b];
    // pages and key blocks (two pages) that each tile reads: tile 1 reads at least as many as tile 0
    int n_pages[2], n_blocks[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int max_pos = start + min(T, t0 + (t + 1) * BT) - 1;
        n_pages[t] = t < n_tiles ? max_pos / PAGE + 1 : 0;
        n_blocks[t] = (n_pages[t] + 1) / 2;
    }
    const int all_pages = n_pages[n_tiles - 1], all_blocks = n_blocks[n_tiles - 1];
    const int* table = args.block_table + (size_t)slot * args.blocks_per_seq;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); mbar_init(&s_full[i], 1);
            mbar_init(&p_ready[i], 4); mbar_init(&o_done[i], 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0 && lane == 0) { prefetch_tmap(&map_q); prefetch_tmap(&map_k); prefetch_tmap(&map_v); }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;                // columns: scores 0 | scores 1 | output 0 | output 1, 128 each
    pdl_wait();                                           // q, and this step's keys and values, come from the kernels before

    if (warp == 0) {
        // ---------------------------------------------------------------- loads
        if (elect_one()) {
            mbar_expect_tx(q_full, n_tiles * AT_Q_BYTES);
            for (int t = 0; t < n_tiles; ++t) {
                for (int h = 0; h < SLABS; ++h)
                    tma_load_3d(q_sm + t * AT_Q_BYTES + h * AT_SLAB, &map_q, q_full, h * 64, g * G, row0 + t0 + t * BT);
            }
            int issued = 0;
            for (int j = 0; j < all_blocks; ++j) {
                const int s = j & 1;
                if (j >= 2 && !mbar_wait(&kv_empty[s], ((j >> 1) - 1) & 1, abort_flag, args.status, 11)) break;
                const int pages = min(2, all_pages - 2 * j);
                mbar_expect_tx(&kv_full[s], pages * 2 * SLABS * (PAGE * 128));
                for (int pg = 0; pg < pages; ++pg) {
                    const int y = (table[2 * j + pg] * KV + g) * PAGE;
                    for (int h = 0; h < SLABS; ++h) {
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
            auto issue_s = [&](int t, int j) {            // S = Q_t K_j^T into the tile's score columns
                const int s = j & 1;
                if (!mbar_wait(&kv_full[s], (j >> 1) & 1, abort_flag, args.status, 13)) return false;
                tc_fence_after();
                const int keys = min(2, n_pages[t] - 2 * j) * PAGE;
                const uint32_t idesc = umma_idesc_ab(keys, 0);
#pragma unroll
                for (int ks = 0; ks < AT_HD / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * AT_SLAB + (ks & 3) * 32;
                    umma_bf16(tmem_base + t * 128, smem_desc_sw128(smem_u32(q_sm + t * AT_Q_BYTES + off)),
                              smem_desc_sw128(smem_u32(k_sm + s * AT_K_BYTES + off)), idesc, ks > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[t]);
                return true;
            };
            for (int t = 0; t < n_tiles && ok; ++t) ok = issue_s(t, 0);
            for (int j = 0; j < all_blocks && ok; ++j) {
                const int s = j & 1;
                for (int t = 0; t < n_tiles && ok; ++t) {
                    if (j >= n_blocks[t]) continue;
                    ok = mbar_wait(&p_ready[t], j & 1, abort_flag, args.status, 14);
                    if (!ok) break;
                    tc_fence_after();
                    const int keys = min(2, n_pages[t] - 2 * j) * PAGE;
                    const uint32_t idesc = umma_idesc_ab(AT_HD, 1);
                    for (int kk = 0; kk < keys / 16; ++kk)     // O_t += P_t V_j: P from tensor memory, 8 columns per 16 keys
                        umma_bf16_ta(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8,
                                     smem_desc_sw128_mn(smem_u32(v_sm + s * AT_K_BYTES + kk * 2048), AT_SLAB), idesc,
                                     (j > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(&o_done[t]);
                    if (t == n_tiles - 1) umma_commit(&kv_empty[s]);      // the last product that reads this stage
                    if (j + 1 < n_blocks[t]) ok = issue_s(t, j + 1);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax and output: thread r owns row r of its tile
        const int tile = (warp - 2) >> 2;
        const int quarter = warp & 3;                     // the tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;
        const int tt0 = t0 + tile * BT;
        const int tl = tt0 + r / Gp, hh = r % Gp;
        const bool valid = tile < n_tiles && tl < T && hh < G;
        const int pos = valid ? start + tl : -1;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_bits + tile * 128;
        const uint32_t o_addr = tmem_base + lane_bits + 256 + tile * 128;
        const int nb = tile < n_tiles ? n_blocks[tile] : 0;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nb && ok; ++j) {
            ok = mbar_wait(&s_full[tile], j & 1, abort_flag, args.status, 15);
            if (!ok) break;
            tc_fence_after();
            const int keys = min(2, n_pages[tile] - 2 * j) * PAGE;      // 64 or 128, the same for the whole tile
            const int key0 = 2 * j * PAGE;
            const int limit = pos - key0;                               // scores 0..limit of this block are visible
            // The same for all lanes of the warp: the tensor-memory loads and stores below are warp-wide
            // instructions and must not sit in branches that lanes take differently.
            const bool need_mask = __any_sync(0xffffffffu, limit < keys - 1);
            // two passes over the scores, 64 at a time (tensor-memory loads are cheap, registers are not)
            uint32_t sc[2][32];
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains: a warp has little else to hide latency behind
#pragma unroll
            for (int h = 0; h < 2; ++h)
                if (h * 64 < keys) {
                    tmem_ld32(s_addr + h * 64, sc[0]);
                    tmem_ld32(s_addr + h * 64 + 32, sc[1]);
                    tmem_ld_wait();
                    if (need_mask) {
#pragma unroll
                        for (int q = 0; q < 2; ++q)
#pragma unroll
                            for (int e = 0; e < 32; ++e)
                                mx4[e & 3] = fmaxf(mx4[e & 3], h * 64 + q * 32 + e <= limit ? __uint_as_float(sc[q][e]) : -INFINITY);
                    } else {
#pragma unroll
                        for (int q = 0; q < 2; ++q)
#pragma unroll
                            for (int e = 0; e < 32; e += 2)
                                mx4[(e >> 1) & 3] = max3(mx4[(e >> 1) & 3], __uint_as_float(sc[q][e]), __uint_as_float(sc[q][e + 1]));
                    }
                }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * args.scale_log2;   // the scale is positive: it commutes with max
            // the reference maximum moves only when the row's maximum has outgrown it by 2^AT_RESCALE
            float m_new = m_ref, factor = 1.f;
            if (j == 0 || mx > m_ref + AT_RESCALE) {
                m_new = fmaxf(m_ref, mx);
                factor = m_new == -INFINITY ? 1.f : fast_exp2(m_ref - m_new);     // 0 when nothing was seen before
            }
            const float muse = m_new == -INFINITY ? 0.f : m_new;
            uint64_t sum4[4] = {0ull, 0ull, 0ull, 0ull};                  // four chains of float32 pairs
            const uint64_t scale2 = pack2(args.scale_log2, args.scale_log2), shift2 = pack2(-muse, -muse);
#pragma unroll
            for (int h = 0; h < 2; ++h)
                if (h * 64 < keys) {
                    tmem_ld32(s_addr + h * 64, sc[0]);
                    tmem_ld32(s_addr + h * 64 + 32, sc[1]);
                    tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        uint32_t packed[16];
#pragma unroll
                        for (int e = 0; e < 32; e += 2) {
                            float x0, x1;
                            unpack2(fma2(pack2(__uint_as_float(sc[q][e]), __uint_as_float(sc[q][e + 1])), scale2, shift2), x0, x1);
                            float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                            if (need_mask) {
                                if (h * 64 + q * 32 + e > limit) p0 = 0.f;
                                if (h * 64 + q * 32 + e + 1 > limit) p1 = 0.f;
                            }
                            sum4[(e >> 1) & 3] = add2(sum4[(e >> 1) & 3], pack2(p0, p1));
                            __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
                            packed[e >> 1] = *reinterpret_cast<uint32_t*>(&pr);
                        }
                        // over scores that this thread has read already: column (h * 64 + q * 32) / 2 lies behind the reads
                        tmem_st16(s_addr + h * 32 + q * 16, packed);
                    }
                }
            float sum_lo, sum_hi;
            unpack2(add2(add2(sum4[0], sum4[1]), add2(sum4[2], sum4[3])), sum_lo, sum_hi);
            l = l * factor + (sum_lo + sum_hi);
            m_ref = m_new;
            if (j > 0) {
                // the output so far is complete (the scores of this block were issued after it); rescale if a row asks
                ok = mbar_wait(&o_done[tile], (j - 1) & 1, abort_flag, args.status, 16);
                if (!ok) break;
                tc_fence_after();
                if (__any_sync(0xffffffffu, factor != 1.f)) {
                    uint32_t c32[32];
#pragma unroll
                    for (int c = 0; c < AT_HD; c += 32) {
                        tmem_ld32(o_addr + c, c32);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) c32[e] = __float_as_uint(__uint_as_float(c32[e]) * factor);
                        tmem_st32(o_addr + c, c32);
                    }
                }
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[tile]);
        }
        if (ok && nb > 0) {
            ok = mbar_wait(&o_done[tile], (nb - 1) & 1, abort_flag, args.status, 17);
            if (ok) {
                tc_fence_after();
                uint32_t c32[32];
                const float inv = 1.f / l;
                bf16* orow = args.out + ((size_t)(row0 + tl) * H + (g * G + hh)) * AT_HD;
#pragma unroll
                for (int c = 0; c < AT_HD; c += 32) {
                    tmem_ld32(o_addr + c, c32);
                    tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int x = 0; x < 4; ++x) {
                                __nv_bfloat162 pr = __floats2bfloat162_rn(__uint_as_float(c32[e + 2 * x]) * inv,
                                                                          __uint_as_float(c32[e + 2 * x + 1]) * inv);
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

namespace kl {
template <int HD>
static int launch_attention_tcgen05(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& args,
                                    dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = (size_t)(2 + 4) * (HD / 64) * AT_SLAB + 11 * 8 + 16 + 1024;     // two query tiles, two stages of keys and of values
    static bool configured = false;
    if (!configured) {
        KL_CUDA(cudaFuncSetAttribute(attention_tcgen05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    launch_kernel(attention_tcgen05_kernel<HD>, grid, AT_THREADS, smem, stream, mq, mk, mv, args);
    KL_LAUNCH_CHECK();
    return KL_OK;
}
}  // namespace kl

// Prefill attention of a ragged batch (see kl_attention_mma for the arguments' meaning).  Head
// sizes 64 and 128, group sizes that divide 128, no window; q rows 16-byte aligned.  Others:
// KL_ERR_BAD_SIZE / KL_ERR_BAD_ALIGN, and the caller takes the mma.sync kernel.
KL_API int kl_attention_tcgen05(const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,
                                long long n_cache_rows, const int* block_table, int blocks_per_seq, const int* cu_tokens,
                                const int* seq_slots, const int* seq_starts, const int* seq_new, int n_seqs, int max_new,
                                int n_rows, int H, int KV, int hd, float scale, int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return KL_OK;
    if ((hd != 64 && hd != 128) || KV <= 0 || H % KV) return KL_ERR_BAD_SIZE;
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
    const dim3 grid(KV, n_seqs, (max_new + 2 * BT - 1) / (2 * BT));          // two tiles of BT tokens per CTA
    if (grid.y > 65535 || grid.z > 65535) return KL_ERR_BAD_SIZE;
    return hd == 128 ? launch_attention_tcgen05<128>(mq, mk, mv, args, grid, stream)
                     : launch_attention_tcgen05<64>(mq, mk, mv, args, grid, stream);
}
