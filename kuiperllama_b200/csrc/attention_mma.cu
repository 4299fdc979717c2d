// Causal grouped-query attention over the paged cache on the tensor cores (bfloat16 operands,
// float32 scores, softmax and accumulation): the prefill kernel of the bfloat16 path, and its
// decode kernel for large batches.
//
// Per head: s_t = (q . k_t) * scale for lo <= t <= pos, softmax with the maximum subtracted,
// o = sum p_t v_t (ExiledOfCode/KuiperLLama mha_kernel.cu:61,74-106: there one CTA per head,
// one token, scalar FMAs, scores through global memory).
//
// A CTA owns 16 * WM query rows of one sequence and one kv head; a row is (token, head of the
// kv group), so the group's heads share every key and value that is loaded.  Keys and values
// come a cache page (64 keys) or half a page at a time through cp.async into a ring of
// shared-memory stages (NS stages of SK keys: template parameters), XOR-swizzled so that
// ldmatrix is free of bank conflicts.  Each warp keeps its
// 16 rows' queries as mma.sync A fragments, multiplies them with the page's keys (B fragments
// by ldmatrix), runs the online softmax on the score fragments in registers, and multiplies
// the probabilities (converted in place to A fragments) with the values (ldmatrix.trans).
// With WN > 1 (decode: few rows) the warps of a CTA split each stage's keys instead of the
// rows and merge their results in shared memory; with splits > 1 the pages of a sequence are
// cut over blockIdx.z and the pieces are merged by a second kernel or, in the decode step's
// fused form, by the last CTA of the sequence to finish.  The decode layout comes as four warps
// on whole pages (two stages, three CTAs per SM; or three stages, two per SM) and as light CTAs
// of two warps on half pages (three stages of 16 KB at a head size of 128: four CTAs per SM),
// taken where three per SM would leave CTAs for a second round.
#include "common.cuh"

namespace kl {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D (16x8, float32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit alone (two units in the last place; 2^-inf = 0): the softmax takes it
// some ten times per warp and page, where exp2f costs four instructions each.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// SK keys of one kv head, [SK][HD] (a cache page or half of one), into a swizzled stage: the
// 16-byte chunk c of key row r lands at chunk c ^ (r & 7) of that row.
template <int HD, int THREADS, int SK>
__device__ __forceinline__ void load_keys(bf16* stage, const bf16* __restrict__ src) {
    constexpr int CHUNKS = HD / 8;                       // 16-byte chunks per row
    constexpr int ROWS_PER_TURN = THREADS / CHUNKS;      // rows that the CTA covers with one copy per thread
    static_assert(THREADS % CHUNKS == 0 && SK % ROWS_PER_TURN == 0, "load_keys: thread layout");
    const int r0 = threadIdx.x / CHUNKS, c = threadIdx.x % CHUNKS;
    if constexpr (ROWS_PER_TURN % 8 == 0) {
        // A thread keeps its chunk column; its rows are a multiple of 8 apart, so the swizzle term is
        // the same in every turn and the addresses differ by compile-time constants.
        const uint32_t dst = smem_addr(stage + r0 * HD + ((c ^ (r0 & 7)) << 3));
        const bf16* from = src + r0 * HD + (c << 3);
#pragma unroll
        for (int t = 0; t < SK / ROWS_PER_TURN; ++t)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                         ::"r"(dst + (uint32_t)(t * ROWS_PER_TURN * HD * 2)), "l"(from + t * ROWS_PER_TURN * HD) : "memory");
    } else {
#pragma unroll
        for (int t = 0; t < SK / ROWS_PER_TURN; ++t) {
            const int r = r0 + t * ROWS_PER_TURN;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                         ::"r"(smem_addr(stage + r * HD + ((c ^ (r & 7)) << 3))), "l"(src + r * HD + (c << 3)) : "memory");
        }
    }
}

// What a decode step may fold into the attention kernel (one token per sequence): the sum of
// the q/k/v product's float32 pieces, the rotation of q and k, the write of the new key and
// value into the cache (by the CTA whose pages end at the token's position), and the merge of a
// sequence's splits (by the last of its CTAs to finish; `counters` are zero between launches).
struct DecodeFuse {
    int enabled;
    const float* partials;        // [n_partials][rows][(H + 2 KV) * HD] float32, or null
    int n_partials;
    size_t partial_stride;
    const bf16* qkv;              // [rows][(H + 2 KV) * HD] bfloat16 when there are no partials
    const float* inv_freq;        // [HD / 2]
    bf16* k_cache_w;              // the cache, writable
    bf16* v_cache_w;
    int* counters;                // [rows * KV], zero
};

// The decode step's token of one sequence, for one kv group: its q (the group's G heads) into q_sm
// [G][HD], and with `writes_token` its k and v into the cache at element offset `dst`.  The values are
// the sum of the q/k/v product's float32 pieces (or the bfloat16 qkv row), q and k rotated by the angles
// whose cos and sin are in rot_cs / rot_sn [HD / 2] (k by `k_position` itself where it differs from q's).
// Work is cut into items of four neighbouring elements (and their four rotation partners), one per
// thread and turn, and an item's loads are all requested before any is used: the CTA waits for
// memory once.
template <int HD, int THREADS>
__device__ __forceinline__ void make_token_qkv(const DecodeFuse& fuse, bf16* q_sm, const float* rot_cs, const float* rot_sn,
                                               int G, int H, int KV, int g, size_t q_row, size_t kv_row, bool writes_token,
                                               size_t dst, bool k_at_q_position, int k_position) {
    const int width = (H + 2 * KV) * HD;
    constexpr int QI = HD / 8;                       // items per head: HD / 2 pairs, four at a time
    const int n_q = G * QI, n_k = writes_token ? QI : 0, n_v = writes_token ? HD / 4 : 0;
    // A CTA of fewer than 128 threads takes two items per thread and turn (and four pieces at a time
    // instead of eight), so that it still waits for memory once.
    constexpr int IT = THREADS >= 128 ? 1 : 2, PC = 8 / IT;
    const int n_items = n_q + n_k + n_v;
    for (int base = 0; base < n_items; base += IT * THREADS) {
        bool live[IT], is_q[IT], is_k[IT], rot[IT];
        int hh[IT], j[IT];
        size_t off[IT];
        float4 x[IT], y[IT];
#pragma unroll
        for (int e = 0; e < IT; ++e) {
            const int item = base + e * THREADS + threadIdx.x;
            live[e] = item < n_items;
            is_q[e] = item < n_q;
            is_k[e] = !is_q[e] && item < n_q + n_k;
            hh[e] = is_q[e] ? item / QI : 0;
            j[e] = is_q[e] ? (item % QI) * 4 : (is_k[e] ? (item - n_q) * 4 : (item - n_q - n_k) * 4);
            const int col = is_q[e] ? (g * G + hh[e]) * HD + j[e] : (is_k[e] ? (H + g) * HD + j[e] : (H + KV + g) * HD + j[e]);
            off[e] = (is_q[e] ? q_row : kv_row) * width + col;
            rot[e] = is_q[e] || is_k[e];
            x[e] = y[e] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (fuse.n_partials == 0) {
#pragma unroll
            for (int e = 0; e < IT; ++e) {
                if (!live[e]) continue;
                const uint2 rx = *reinterpret_cast<const uint2*>(fuse.qkv + off[e]);
                const float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rx.x));
                const float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rx.y));
                x[e] = make_float4(x01.x, x01.y, x23.x, x23.y);
                if (rot[e]) {
                    const uint2 ry = *reinterpret_cast<const uint2*>(fuse.qkv + off[e] + HD / 2);
                    const float2 y01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ry.x));
                    const float2 y23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ry.y));
                    y[e] = make_float4(y01.x, y01.y, y23.x, y23.y);
                }
            }
        } else {
            for (int z0 = 0; z0 < fuse.n_partials; z0 += PC) {     // pieces are added in ascending order
                float4 px[IT][PC], py[IT][PC];
#pragma unroll
                for (int e = 0; e < IT; ++e) {
#pragma unroll
                    for (int zz = 0; zz < PC; ++zz) {
                        const float* p = fuse.partials + (size_t)(z0 + zz) * fuse.partial_stride + off[e];
                        const bool in = live[e] && z0 + zz < fuse.n_partials;
                        px[e][zz] = in ? __ldcg(reinterpret_cast<const float4*>(p)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        py[e][zz] = (in && rot[e]) ? __ldcg(reinterpret_cast<const float4*>(p + HD / 2)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
#pragma unroll
                for (int e = 0; e < IT; ++e) {
#pragma unroll
                    for (int zz = 0; zz < PC; ++zz) {
                        x[e].x += px[e][zz].x; x[e].y += px[e][zz].y; x[e].z += px[e][zz].z; x[e].w += px[e][zz].w;
                        y[e].x += py[e][zz].x; y[e].y += py[e][zz].y; y[e].z += py[e][zz].z; y[e].w += py[e][zz].w;
                    }
                }
            }
        }
#pragma unroll
        for (int e = 0; e < IT; ++e) {
            if (!live[e]) continue;
            uint2 lo_half, hi_half;                  // elements j..j+3 and their partners j + HD / 2 ..
            if (rot[e]) {
                float sn[4], cs[4];
                if (is_q[e] || k_at_q_position) {            // a decode step's one token: q and k share the position
                    const float4 c4 = *reinterpret_cast<const float4*>(rot_cs + j[e]), s4 = *reinterpret_cast<const float4*>(rot_sn + j[e]);
                    cs[0] = c4.x; cs[1] = c4.y; cs[2] = c4.z; cs[3] = c4.w;
                    sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
                } else {
                    const float4 f = *reinterpret_cast<const float4*>(fuse.inv_freq + j[e]);
                    const float angle = (float)k_position;
                    sincosf(angle * f.x, &sn[0], &cs[0]);
                    sincosf(angle * f.y, &sn[1], &cs[1]);
                    sincosf(angle * f.z, &sn[2], &cs[2]);
                    sincosf(angle * f.w, &sn[3], &cs[3]);
                }
                lo_half.x = pack_bf16(x[e].x * cs[0] - y[e].x * sn[0], x[e].y * cs[1] - y[e].y * sn[1]);
                lo_half.y = pack_bf16(x[e].z * cs[2] - y[e].z * sn[2], x[e].w * cs[3] - y[e].w * sn[3]);
                hi_half.x = pack_bf16(y[e].x * cs[0] + x[e].x * sn[0], y[e].y * cs[1] + x[e].y * sn[1]);
                hi_half.y = pack_bf16(y[e].z * cs[2] + x[e].z * sn[2], y[e].w * cs[3] + x[e].w * sn[3]);
            } else {
                lo_half.x = pack_bf16(x[e].x, x[e].y);
                lo_half.y = pack_bf16(x[e].z, x[e].w);
                hi_half = lo_half;
            }
            if (is_q[e]) {
                *reinterpret_cast<uint2*>(q_sm + hh[e] * HD + j[e]) = lo_half;
                *reinterpret_cast<uint2*>(q_sm + hh[e] * HD + j[e] + HD / 2) = hi_half;
            } else if (is_k[e]) {
                *reinterpret_cast<uint2*>(fuse.k_cache_w + dst + j[e]) = lo_half;
                *reinterpret_cast<uint2*>(fuse.k_cache_w + dst + j[e] + HD / 2) = hi_half;
            } else {
                *reinterpret_cast<uint2*>(fuse.v_cache_w + dst + j[e]) = lo_half;
            }
        }
    }
}

// SK: keys per stage, a cache page (64) or half of one.  Half pages with two warps make a CTA of the
// decode layout light enough (48 KB of stages at a head size of 128) for four of them on an SM, or
// with two stages (32 KB) for six.
template <int HD, int WM, int WN, int NS, int SK>
__global__ void __launch_bounds__(32 * WM * WN, SK < PAGE ? (NS == 2 ? 6 : 4) : (NS == 2 ? ((HD == 64 && WN > 1) ? 4 : 3) : 2))   // half pages: six CTAs of two stages or four of three; whole pages, NS = 2: three CTAs per SM (168 registers, 3 x 64 KB of stages), four in the decode layout with a head size of 64
attention_mma_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out,
                     const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                     const int* __restrict__ block_table, int blocks_per_seq,
                     const int* __restrict__ cu_tokens, const int* __restrict__ seq_slots,
                     const int* __restrict__ seq_starts, const int* __restrict__ seq_new,
                     float* __restrict__ part_o, float* __restrict__ part_ml,
                     int H, int KV, int Gp, float scale_log2, int window, int S, DecodeFuse fuse) {
    pdl_launch_dependents();
    // The fused decode form reads only what earlier steps left (the batch's index arrays, the
    // block table, old cache pages) until it has requested its first page; then it waits.
    if (!fuse.enabled) pdl_wait();
    constexpr int THREADS = 32 * WM * WN;
    constexpr int ROWS = 16 * WM;
    constexpr int KPW = SK / WN;                         // keys of a stage that one warp handles
    constexpr int UPP = PAGE / SK;                       // stages ("units") per cache page
    static_assert(PAGE % SK == 0 && KPW % 16 == 0, "attention_mma_kernel: keys per stage and warp");
    constexpr int NT = KPW / 8;                          // score tiles (8 keys each) per warp
    constexpr int KS = HD / 16;                          // k steps of q . k
    constexpr int ON = HD / 8;                           // output tiles (8 dims each)
    extern __shared__ __align__(128) uint8_t smem_raw[];
    bf16* k_stage = reinterpret_cast<bf16*>(smem_raw);                   // [NS][SK][HD]
    bf16* v_stage = k_stage + NS * SK * HD;                              // [NS][SK][HD]

    const int b = blockIdx.y;
    const int g = blockIdx.z % KV, z = blockIdx.z / KV;
    const int G = H / KV;
    const int BT = ROWS / Gp;                            // tokens per CTA
    const int T = seq_new[b];
    // Tiles late in a sequence read the most keys: they are started first (CTAs are handed out
    // in ascending blockIdx.x), so the short ones fill the machine's tail.
    const int t0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BT;
    if (t0 >= T) return;
    const int start = seq_starts[b], slot = seq_slots[b], row0 = cu_tokens[b];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warp_m = warp % WM, warp_n = warp / WM;
    const int quad = lane >> 2, tq = lane & 3;

    // this thread's two rows (quad and quad + 8 of the warp's 16)
    int tok[2], head[2], pos[2], lo[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp_m * 16 + quad + 8 * i;
        const int tl = t0 + r / Gp, hh = r % Gp;
        valid[i] = tl < T && hh < G;
        tok[i] = row0 + tl;
        head[i] = g * G + hh;
        pos[i] = valid[i] ? start + tl : -1;
        lo[i] = (window > 0 && valid[i]) ? max(0, pos[i] - window + 1) : 0;
    }
    // pages this CTA reads
    const int last_tok = min(T, t0 + BT) - 1;
    const int max_pos = start + last_tok;
    const int min_lo = window > 0 ? max(0, start + t0 - window + 1) : 0;
    const int first_page = min_lo / PAGE, n_pages = max_pos / PAGE - first_page + 1;
    const int per = (n_pages + S - 1) / S;
    const int p_begin = first_page + z * per, p_end = min(first_page + n_pages, p_begin + per);
    const int* table = block_table + (size_t)slot * blocks_per_seq;
    const int full_below = start + t0;                   // keys <= this are visible to every valid row (no window)

    // Units of SK keys this CTA reads: its pages, without what lies wholly behind the last position.
    const int u_begin = p_begin * UPP, u_end = min(p_end * UPP, max_pos / SK + 1);
    auto issue = [&](int unit, int st) {
        const size_t off = (((size_t)table[unit / UPP] * KV + g) * PAGE + (unit % UPP) * SK) * HD;
        load_keys<HD, THREADS, SK>(k_stage + st * SK * HD, k_cache + off);
        load_keys<HD, THREADS, SK>(v_stage + st * SK * HD, v_cache + off);
        cp_async_commit();
    };
    const bool writes_token = fuse.enabled && p_begin < p_end && p_end == first_page + n_pages;
    // Units are requested NS - 1 ahead, one cp.async group per unit in key order.  The fused
    // decode form requests what it can before it waits for the kernel before it: every unit but
    // the one this CTA is about to write the new token into.
    int next = u_begin, groups = 0;
    // The fused form's rotation: cos and sin of the token's position times every frequency, made once per
    // CTA before the wait (position and frequencies are known by then), so that the rotation of q and k
    // costs no sincosf on the path between the kernel ahead and the first page (it took 0.9 us of 7.6 at 8
    // sequences and 1.7 us per round at 64, every item computing its four anew).
    __shared__ __align__(16) float rot_cs[HD / 2];
    __shared__ __align__(16) float rot_sn[HD / 2];
    if (fuse.enabled) {
        const int limit = writes_token ? max_pos / SK : u_end;
        while (groups < NS - 1 && next < limit) { issue(next, (next - u_begin) % NS); ++next; ++groups; }
        for (int f = threadIdx.x; f < HD / 2; f += THREADS) sincosf((float)(start + t0) * fuse.inv_freq[f], &rot_sn[f], &rot_cs[f]);
        pdl_wait();
        __syncthreads();
    }
    // query fragments
    uint32_t qa[KS][4];
    if (fuse.enabled) {
        // The token's q (this group's heads), and in the CTA whose pages end at the token also its k
        // and v, are made here: the sum of the product's pieces, rotated.
        __shared__ __align__(16) bf16 q_sm[16 * HD];
        const size_t dst = writes_token ? (((size_t)table[max_pos / PAGE] * KV + g) * PAGE + (max_pos % PAGE)) * HD : 0;
        make_token_qkv<HD, THREADS>(fuse, q_sm, rot_cs, rot_sn, G, H, KV, g, (size_t)(row0 + t0), (size_t)row0, writes_token, dst,
                                    max_pos == start + t0, max_pos);
        __syncthreads();                                 // q_sm is whole; the CTA's own copies below read the new cache rows
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                uint32_t x0 = 0u, x1 = 0u;
                if (valid[i]) {
                    const bf16* p = q_sm + (quad + 8 * i) * HD + ks * 16 + 2 * tq;       // row r = head r of the group (Gp rows per token)
                    x0 = *reinterpret_cast<const uint32_t*>(p);
                    x1 = *reinterpret_cast<const uint32_t*>(p + 8);
                }
                qa[ks][i] = x0;
                qa[ks][2 + i] = x1;
            }
        }
    } else
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t x0 = 0u, x1 = 0u;
            if (valid[i]) {
                const bf16* p = q + (size_t)tok[i] * q_stride + (size_t)head[i] * HD + ks * 16 + 2 * tq;
                x0 = *reinterpret_cast<const uint32_t*>(p);
                x1 = *reinterpret_cast<const uint32_t*>(p + 8);
            }
            qa[ks][i] = x0;
            qa[ks][2 + i] = x1;
        }
    }
    float o[ON][4];
#pragma unroll
    for (int n = 0; n < ON; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    while (groups < NS - 1) {
        if (next < u_end) { issue(next, (next - u_begin) % NS); ++next; } else cp_async_commit();
        ++groups;
    }
    for (int pi = u_begin; pi < u_end; ++pi) {
        const int st = (pi - u_begin) % NS;
        if (next < u_end) { issue(next, (next - u_begin) % NS); ++next; } else cp_async_commit();
        cp_async_wait<NS - 1>();                         // all but the NS - 1 newest groups: unit pi has landed
        __syncthreads();
        const bf16* ks_ = k_stage + st * SK * HD;
        const bf16* vs_ = v_stage + st * SK * HD;
        const int key0 = pi * SK + warp_n * KPW;         // first key of this warp's share
        float s[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        if (key0 <= max_pos) {                           // the warp's keys are not all in the future
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int n2 = 0; n2 < NT / 2; ++n2) {
                    const int r = warp_n * KPW + n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
                    const int c = ks * 2 + ((lane >> 3) & 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(smem_addr(ks_ + r * HD + ((c ^ (r & 7)) << 3)), b0, b1, b2, b3);
                    mma_bf16(s[2 * n2], qa[ks], b0, b1);
                    mma_bf16(s[2 * n2 + 1], qa[ks], b2, b3);
                }
            }
            // scale, mask, online softmax
            const bool need_mask = key0 + KPW - 1 > full_below || window > 0 || !valid[0] || !valid[1];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int i = c >> 1;
                    float v = s[n][c] * scale_log2;
                    if (need_mask) {
                        const int kp = key0 + n * 8 + 2 * tq + (c & 1);
                        if (kp > pos[i] || kp < lo[i]) v = -INFINITY;
                    }
                    s[n][c] = v;
                    mx[i] = fmaxf(mx[i], v);
                }
            }
            float corr[2], muse[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m[i], mx[i]);
                muse[i] = m_new == -INFINITY ? 0.f : m_new;
                corr[i] = fast_exp2(m[i] - muse[i]);     // 0 when nothing was seen before
                m[i] = m_new;
                l[i] *= corr[i];
            }
            if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {      // most blocks after the first leave the maxima alone
#pragma unroll
                for (int n = 0; n < ON; ++n) { o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1]; }
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float p = fast_exp2(s[n][c] - muse[c >> 1]);
                    s[n][c] = p;
                    l[c >> 1] += p;
                }
            }
            // probabilities as A fragments, times the values
#pragma unroll
            for (int kk = 0; kk < KPW / 16; ++kk) {
                uint32_t pa[4];
                pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < ON / 2; ++n2) {
                    const int r = warp_n * KPW + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    const int c = n2 * 2 + (lane >> 4);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(smem_addr(vs_ + r * HD + ((c ^ (r & 7)) << 3)), b0, b1, b2, b3);
                    mma_bf16(o[2 * n2], pa, b0, b1);
                    mma_bf16(o[2 * n2 + 1], pa, b2, b3);
                }
            }
        }
        __syncthreads();                                 // the stage may be overwritten by the next prefetch
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    if constexpr (WN > 1) {
        // merge the warps that shared the rows: through shared memory (the stages are free now)
        constexpr int OS = HD + 8;                                   // row stride of sm_o: rows 8 banks apart
        float* sm_m = reinterpret_cast<float*>(smem_raw);            // [WN][ROWS]
        float* sm_l = sm_m + WN * ROWS;                              // [WN][ROWS]
        float* sm_o = sm_l + WN * ROWS;                              // [WN][ROWS][OS]
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!valid[i]) continue;                                 // rows of padding are never read
            const int r = warp_m * 16 + quad + 8 * i;
            if (tq == 0) { sm_m[warp_n * ROWS + r] = m[i]; sm_l[warp_n * ROWS + r] = l[i]; }
#pragma unroll
            for (int n = 0; n < ON; ++n)
                *reinterpret_cast<float2*>(sm_o + ((size_t)warp_n * ROWS + r) * OS + n * 8 + 2 * tq) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
        }
        __syncthreads();
        const int n_rows = min(BT, T - t0) * Gp;                     // rows of the tile that belong to tokens
        for (int item = threadIdx.x; item < n_rows * (HD / 4); item += THREADS) {
            const int r = item / (HD / 4), d = (item % (HD / 4)) * 4;
            const int tl = t0 + r / Gp, hh = r % Gp;
            if (hh >= G) continue;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < WN; ++w) M = fmaxf(M, sm_m[w * ROWS + r]);
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < WN; ++w) {
                const float mw = sm_m[w * ROWS + r];
                const float c = mw == -INFINITY ? 0.f : exp2f(mw - M);
                L += sm_l[w * ROWS + r] * c;
                const float4 v = *reinterpret_cast<const float4*>(sm_o + ((size_t)w * ROWS + r) * OS + d);
                acc.x += v.x * c; acc.y += v.y * c; acc.z += v.z * c; acc.w += v.w * c;
            }
            const size_t orow = (size_t)(row0 + tl) * H + (g * G + hh);
            if (S == 1) {
                const float inv = 1.f / L;
                *reinterpret_cast<uint2*>(out + orow * HD + d) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
            } else {
                *reinterpret_cast<float4*>(part_o + (orow * S + z) * HD + d) = acc;
                if (d == 0) *reinterpret_cast<float2*>(part_ml + (orow * S + z) * 2) = make_float2(M, L);
            }
        }
        if (fuse.enabled && S > 1) {
            // The last of the sequence's CTAs (for this kv head) to get here merges the pieces.
            __shared__ int is_last;
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const int done = atomicAdd(&fuse.counters[b * KV + g], 1);
                is_last = done == S - 1;
                if (is_last) fuse.counters[b * KV + g] = 0;      // zero again for the next launch
            }
            __syncthreads();
            if (is_last) {
                __threadfence();
                // four output elements per thread and turn; eight pieces are requested at a time and merged
                // into a running maximum, sum and output, in ascending order
                for (int item = threadIdx.x; item < G * (HD / 4); item += THREADS) {
                    const int hh = item / (HD / 4), d = (item % (HD / 4)) * 4;
                    const size_t orow = (size_t)row0 * H + (g * G + hh);
                    float M = -INFINITY, L = 0.f;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int z0 = 0; z0 < S; z0 += 8) {
                        float2 ml[8];
                        float4 po[8];
#pragma unroll
                        for (int zz = 0; zz < 8; ++zz) {
                            const bool in = z0 + zz < S;
                            ml[zz] = in ? __ldcg(reinterpret_cast<const float2*>(part_ml + (orow * S + z0 + zz) * 2)) : make_float2(-INFINITY, 0.f);
                            po[zz] = in ? __ldcg(reinterpret_cast<const float4*>(part_o + (orow * S + z0 + zz) * HD + d)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                        float Mc = M;
#pragma unroll
                        for (int zz = 0; zz < 8; ++zz) Mc = fmaxf(Mc, ml[zz].x);
                        const float keep = M == -INFINITY ? 0.f : exp2f(M - Mc);     // Mc is finite when M is
                        L *= keep; acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
#pragma unroll
                        for (int zz = 0; zz < 8; ++zz) {
                            const float c = ml[zz].x == -INFINITY ? 0.f : exp2f(ml[zz].x - Mc);
                            L += ml[zz].y * c;
                            acc.x += po[zz].x * c; acc.y += po[zz].y * c; acc.z += po[zz].z * c; acc.w += po[zz].w * c;
                        }
                        M = Mc;
                    }
                    const float inv = 1.f / L;
                    *reinterpret_cast<uint2*>(out + orow * HD + d) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
                }
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!valid[i]) continue;
            const size_t orow = (size_t)tok[i] * H + head[i];
            if (S == 1) {
                const float inv = 1.f / l[i];
#pragma unroll
                for (int n = 0; n < ON; ++n)
                    *reinterpret_cast<uint32_t*>(out + orow * HD + n * 8 + 2 * tq) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
            } else {
#pragma unroll
                for (int n = 0; n < ON; ++n)
                    *reinterpret_cast<float2*>(part_o + (orow * S + z) * HD + n * 8 + 2 * tq) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
                if (tq == 0) { part_ml[(orow * S + z) * 2] = m[i]; part_ml[(orow * S + z) * 2 + 1] = l[i]; }
            }
        }
    }
}

// Merge the pieces of a split sequence: maxima and sums are in the exp2 domain of the kernel above.
template <int HD>
__global__ void attention_mma_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                             bf16* __restrict__ out, int H, int S) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t orow = (size_t)blockIdx.x * H + blockIdx.y;
    float M = -INFINITY;
    for (int z = 0; z < S; ++z) M = fmaxf(M, part_ml[(orow * S + z) * 2]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float L = 0.f, acc = 0.f;
        for (int z = 0; z < S; ++z) {
            const float mz = part_ml[(orow * S + z) * 2];
            const float c = mz == -INFINITY ? 0.f : exp2f(mz - M);
            L += part_ml[(orow * S + z) * 2 + 1] * c;
            acc += part_o[(orow * S + z) * HD + d] * c;
        }
        out[orow * HD + d] = __float2bfloat16_rn(acc / L);
    }
}

template <int HD, int WM, int WN, int NS, int SK = PAGE>
static int launch_mma(const bf16* q, int q_stride, bf16* out, const bf16* k, const bf16* v, const int* table, int bps,
                      const int* cu, const int* slots, const int* starts, const int* news, float* po, float* pml,
                      int n_seqs, int max_new, int n_rows, int H, int KV, float scale, int window, int S,
                      const DecodeFuse& fuse, cudaStream_t stream) {
    const int G = H / KV;
    int Gp = 1;
    while (Gp < G) Gp <<= 1;
    constexpr int ROWS = 16 * WM;
    if (Gp > ROWS) return KL_ERR_BAD_SIZE;
    const int BT = ROWS / Gp;
    const dim3 grid((max_new + BT - 1) / BT, n_seqs, KV * S);
    if (grid.y > 65535 || grid.z > 65535) return KL_ERR_BAD_SIZE;
    size_t smem = (size_t)2 * NS * SK * HD * sizeof(bf16);
    if (WN > 1) smem = max(smem, (size_t)(2 * WN * ROWS + WN * ROWS * (HD + 8)) * sizeof(float));
    static bool configured = false;
    if (!configured) {
        KL_CUDA(cudaFuncSetAttribute(attention_mma_kernel<HD, WM, WN, NS, SK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        // all of the SM's memory as shared memory: the kernel's data come through cp.async, and how many CTAs fit decides its speed
        KL_CUDA(cudaFuncSetAttribute(attention_mma_kernel<HD, WM, WN, NS, SK>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
        configured = true;
    }
    launch_kernel(attention_mma_kernel<HD, WM, WN, NS, SK>, grid, 32 * WM * WN, smem, stream, q, q_stride, out, k, v, table, bps, cu, slots,
        starts, news, po, pml, H, KV, Gp, scale * 1.4426950408889634f, window, S, fuse);
    KL_LAUNCH_CHECK();
    if (S > 1 && !fuse.enabled) {
        launch_kernel(attention_mma_combine_kernel<HD>, dim3(n_rows, H), HD <= 64 ? 32 : 64, 0, stream, po, pml, out, H, S);
        KL_LAUNCH_CHECK();
    }
    return KL_OK;
}

}  // namespace kl

using namespace kl;

// Attention of a ragged batch: sequence b brings seq_new[b] tokens (rows cu_tokens[b] ... of q
// and out) that start at position seq_starts[b] of slot seq_slots[b]; its keys and values are
// already in the cache.  max_new is the largest seq_new (host copy, sizes the grid); n_rows the
// number of packed rows.  few_rows != 0 picks the layout for decode (one token per sequence:
// the warps of a CTA split the keys).  Head sizes 64 and 128; others KL_ERR_BAD_SIZE.
static int attention_mma_dispatch(const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,
                            const int* block_table, int blocks_per_seq, const int* cu_tokens, const int* seq_slots,
                            const int* seq_starts, const int* seq_new, float* part_o, float* part_ml, int n_seqs,
                            int max_new, int n_rows, int H, int KV, int hd, float scale, int window, int splits,
                            int few_rows, const DecodeFuse& fuse, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return KL_OK;
    if (KV <= 0 || H % KV || splits < 1) return KL_ERR_BAD_SIZE;
    if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return KL_ERR_BAD_SIZE;
    if (q_stride % 2 || ((uintptr_t)q & 3)) return KL_ERR_BAD_ALIGN;
#define KL_MMA(HD, WM, WN, NS)                                                                                        \
    return launch_mma<HD, WM, WN, NS>((const bf16*)q, q_stride, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache,     \
                                  block_table, blocks_per_seq, cu_tokens, seq_slots, seq_starts, seq_new, part_o,      \
                                  part_ml, n_seqs, max_new, n_rows, H, KV, scale, window, splits, fuse, stream)
#define KL_MMA5(HD, WM, WN, NS, SK)                                                                                   \
    return launch_mma<HD, WM, WN, NS, SK>((const bf16*)q, q_stride, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache, \
                                  block_table, blocks_per_seq, cu_tokens, seq_slots, seq_starts, seq_new, part_o,      \
                                  part_ml, n_seqs, max_new, n_rows, H, KV, scale, window, splits, fuse, stream)
    // Decode: three CTAs of two stages fit an SM, or two CTAs of three stages.  A CTA's time is set by
    // its chain of pages either way, so what counts is how many rounds of CTAs the grid needs: three
    // stages where they do not add a round (64 sequences of 8 kv heads: 2 rounds both ways, 47 against 53 us).
    const int sms = kl::sm_count();
    if (sms <= 0) return KL_ERR_SETUP;
    if (hd == 128 && few_rows) {
        const long long ctas = (long long)n_seqs * KV * splits;
        const long long rounds2 = (ctas + 3 * sms - 1) / (3 * sms), rounds3 = (ctas + 2 * sms - 1) / (2 * sms);
        // More CTAs than three per SM: light CTAs (two warps, half pages, three stages), four to an SM.
        static const int light = getenv("KL_ATTN_LIGHT") ? atoi(getenv("KL_ATTN_LIGHT")) : 1;
        // Light CTAs of two stages (32 KB, 168 registers) fit six to an SM: taken where that saves rounds
        // over four of three stages (each of its rounds moves fewer bytes at a time; measured on the 8B
        // shape: one round against two and two against three are faster, three against four is not).
        const long long rounds4 = (ctas + 4 * sms - 1) / (4 * sms), rounds6 = (ctas + 6 * sms - 1) / (6 * sms);
        if (rounds2 > 1 && light && rounds6 * 7 < rounds4 * 5) KL_MMA5(128, 1, 2, 2, 32);
        if (rounds2 > 1 && light) KL_MMA5(128, 1, 2, 3, 32);
        if (rounds2 > 1 && rounds3 <= rounds2) KL_MMA(128, 1, 4, 3);
    }
    if (hd == 128) { if (few_rows) KL_MMA(128, 1, 4, 2); else KL_MMA(128, 4, 1, 2); }
    if (hd == 64) { if (few_rows) KL_MMA(64, 1, 4, 2); else KL_MMA(64, 4, 1, 2); }
#undef KL_MMA
#undef KL_MMA5
    return KL_ERR_BAD_SIZE;
}

KL_API int kl_attention_mma(const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,
                            const int* block_table, int blocks_per_seq, const int* cu_tokens, const int* seq_slots,
                            const int* seq_starts, const int* seq_new, float* part_o, float* part_ml, int n_seqs,
                            int max_new, int n_rows, int H, int KV, int hd, float scale, int window, int splits,
                            int few_rows, cudaStream_t stream) {
    DecodeFuse none;
    memset(&none, 0, sizeof(none));
    return attention_mma_dispatch(q, q_stride, out, k_cache, v_cache, block_table, blocks_per_seq, cu_tokens, seq_slots,
                                  seq_starts, seq_new, part_o, part_ml, n_seqs, max_new, n_rows, H, KV, hd, scale, window,
                                  splits, few_rows, none, stream);
}

// A whole decode step's attention in one kernel: one token per sequence, rows in sequence
// order.  The q/k/v projections come as `qkv` (bfloat16 [rows, (H + 2 KV) * hd]) or as
// float32 pieces `partials` [n_partials, rows, width]; the kernel rotates q and k (full
// rotation, inv_freq [hd / 2]), writes the token's key and value into the cache, attends, and
// merges the splits itself (`counters`: int32 [rows * KV], zero, left zero).
KL_API int kl_attention_decode_fused(const void* qkv, const float* partials, int n_partials, long long partial_stride,
                                     const float* inv_freq, void* out, void* k_cache, void* v_cache,
                                     const int* block_table, int blocks_per_seq, const int* cu_tokens,
                                     const int* seq_slots, const int* seq_starts, const int* seq_new, float* part_o,
                                     float* part_ml, int* counters, int n_seqs, int H, int KV, int hd, float scale,
                                     int window, int splits, cudaStream_t stream) {
    if (n_seqs <= 0) return KL_OK;
    if (inv_freq == nullptr || counters == nullptr || (n_partials == 0 && qkv == nullptr)) return KL_ERR_BAD_SIZE;
    DecodeFuse fuse;
    fuse.enabled = 1;
    fuse.partials = partials;
    fuse.n_partials = n_partials;
    fuse.partial_stride = (size_t)partial_stride;
    fuse.qkv = (const bf16*)qkv;
    fuse.inv_freq = inv_freq;
    fuse.k_cache_w = (bf16*)k_cache;
    fuse.v_cache_w = (bf16*)v_cache;
    fuse.counters = counters;
    return attention_mma_dispatch(out /* unused as q */, 8, out, k_cache, v_cache, block_table, blocks_per_seq, cu_tokens,
                                  seq_slots, seq_starts, seq_new, part_o, part_ml, n_seqs, 1, n_seqs, H, KV, hd, scale,
                                  window, splits, 1, fuse, stream);
}
