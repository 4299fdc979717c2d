// C = A * W^T in bfloat16 on the fifth-generation tensor cores of sm_100a.
//
// Operands are K-major bfloat16 matrices ([rows, K] row-major): TMA (cp.async.bulk.tensor.2d,
// 128-byte swizzle, no multicast) stages 128 x 64 and BN x 64 tiles in shared memory through
// a ring of mbarrier-guarded stages; one elected thread issues tcgen05.mma (kind::f16,
// M = 128, N = BN, K = 16) with the float32 accumulator in tensor memory; four warps read it
// back with tcgen05.ld and store.  Warp roles: warp 0 loads, warp 1 allocates tensor memory
// and issues the MMAs, warps 2..5 are the epilogue (their index mod 4 picks the quarter of
// the 128 tensor-memory lanes that each may read).
//
// Ways of laying a product on tiles:
//   * tokens as rows (prefill): A = activations [M, K], B = weights [N, K]; out[m, n] in bfloat16
//     or float32.  Tiles of 256 x 256 worked by pairs of CTAs as one (gemm_pair_kernel, cta_group::2)
//     where the token count suits, else tiles of 128 x 256 by single CTAs.
//   * weights as rows (decode, few tokens): A = weights [N, K], B = activations [M <= 64, K],
//     tile 128 x {16, 32, 64}; the K range may be cut over blockIdx.z, each cut writing
//     float32 partial sums [z, M, N] that the caller's reduction adds in a fixed order.  Every
//     weight is read from HBM exactly once per product.
//
// This replaces ExiledOfCode/KuiperLLama's matmul_kernel_cu_fp32 (matmul_kernel.cu:6-54), a
// float32 GEMV with one CTA per output row.  Same contract: y = W x, W [out, in], no bias.
//
// Every wait is bounded: a wait that runs out sets a status word that the host reads, the
// roles stop, the CTA waits (bounded) for its own copies in flight, frees its tensor memory
// and returns.
#include "tcgen05.cuh"
#include "tma_host.cuh"

namespace kl {

constexpr int TC_BM = 128;            // tile rows = UMMA M
constexpr int TC_BK = 64;             // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int TC_THREADS = 192;

// ------------------------------------------------------------------------------------------ the kernel

struct GemmArgs {
    void* out;          // bf16 or float32
    long long ld_out;   // elements between rows of out
    long long split_stride;  // elements between the partial results of two k cuts (weights-as-rows only)
    int rows_a;         // valid rows of the A operand (tile rows)
    int rows_b;         // valid rows of the B operand (tile columns)
    int k_blocks;       // ceil(K / 64)
    int out_f32;        // 1: float32 output, 0: bfloat16
    int* status;        // device status word, 0 = fine
    int tiles_m;        // tokens-as-rows: tiles along the tokens and along the output features;
    int tiles_n;        //   blockIdx.x walks them in groups of TC_GROUP_M token tiles (see tile_of)
    int swiglu;         // 1: the B (or A) operand's rows alternate 64 gate rows and 64 up rows; the
                        //    epilogue writes silu(gate) * up, half as many output features, bf16
    // Weights-as-rows only, for the few tokens of a decode step (see "the residual stream inside
    // the products" below).
    const float* scale_ss;    // every token's result is multiplied by rsqrt(sum / K + scale_eps), the sum
    int scale_ss_n;           //   given in pieces [scale_ss_n][64] by the product before (the 1 / rms of a
    float scale_eps;          //   norm whose weight is already in the activations)
    int K;
    float* sink;              // the split's partial sums are added into this residual stream [rows_b, rows_a]
    float* sink_ss;           //   by the last CTA of each row tile, which also leaves sum(x^2) of its
    int* sink_counters;       //   128 columns per row in sink_ss[tile][64]; counters are zero between launches
    const float* sink_w;      // with sink: the next norm's weight [rows_a], and where bf16(x * w) of the new
    __nv_bfloat16* sink_scaled;   //   rows goes [rows_b, rows_a] (the next product's activations); may be null
};

// Tile order for tokens-as-rows: all the feature tiles of a group of TC_GROUP_M token tiles
// before the next group, token tiles fastest.  CTAs that run at the same time then share a few
// weight tiles and a few token tiles, and both stay in L2 instead of being streamed from HBM
// once per token tile.
constexpr int TC_GROUP_M = 16;
__device__ __forceinline__ void tile_of(int id, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int per_group = TC_GROUP_M * tiles_n;
    const int group = id / per_group, in = id - group * per_group;
    const int first = group * TC_GROUP_M;
    const int gm = min(TC_GROUP_M, tiles_m - first);
    tm = first + in % gm;
    tn = in / gm;
}
// silu(g) * u with one exponential and one reciprocal, both of the special-function unit (a full
// division takes a slow path whenever exp(-g) overflows, and this runs 16,384 times per tile beside
// the products).  For g far below zero the denominator is huge or infinite and the quotient 0, as it should be.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// Tokens-as-rows: 32 accumulator columns of one token row to the output (columns n0 .. n0 + 31).
__device__ __forceinline__ void store_row_chunk(const GemmArgs& args, int row, int n0, const uint32_t (&r)[32]) {
    const bool full_n = n0 + 32 <= args.rows_b;
    if (args.out_f32) {
        float* o = (float*)args.out + (size_t)row * args.ld_out + n0;
        if (full_n && (args.ld_out & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        } else {
            for (int j = 0; j < 32; ++j)
                if (n0 + j < args.rows_b) o[j] = __uint_as_float(r[j]);
        }
    } else {
        __nv_bfloat16* o = (__nv_bfloat16*)args.out + (size_t)row * args.ld_out + n0;
        if (full_n && (args.ld_out & 7) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                uint4 v;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(o + j) = v;
            }
        } else {
            for (int j = 0; j < 32; ++j)
                if (n0 + j < args.rows_b) o[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
        }
    }
}
// The same with the SwiGLU epilogue: 32 gate columns and their 32 up columns give the output features f0 .. f0 + 31.
__device__ __forceinline__ void store_row_chunk_swiglu(const GemmArgs& args, int row, int f0, const uint32_t (&rg)[32],
                                                       const uint32_t (&ru)[32]) {
    const int half_n = args.rows_b / 2;
    __nv_bfloat16* o = (__nv_bfloat16*)args.out + (size_t)row * args.ld_out + f0;
    if (f0 + 32 <= half_n && (args.ld_out & 7) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 pr = __floats2bfloat162_rn(
                    silu_mul(__uint_as_float(rg[j + 2 * e]), __uint_as_float(ru[j + 2 * e])),
                    silu_mul(__uint_as_float(rg[j + 2 * e + 1]), __uint_as_float(ru[j + 2 * e + 1])));
                w[e] = *reinterpret_cast<uint32_t*>(&pr);
            }
            *reinterpret_cast<uint4*>(o + j) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        for (int j = 0; j < 32; ++j)
            if (f0 + j < half_n)
                o[j] = __float2bfloat16_rn(silu_mul(__uint_as_float(rg[j]), __uint_as_float(ru[j])));
    }
}

template <int BN, int STAGES, bool WEIGHT_ROWS>
__global__ void __launch_bounds__(TC_THREADS, WEIGHT_ROWS ? 2 : 1)      // weights-as-rows: two CTAs share an SM
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmArgs args) {
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
    constexpr uint32_t ACC_COLS = BN < 32 ? 32 : BN;      // columns of one accumulator
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;          // two accumulators: one is drained while the other is filled
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);     // swizzled tiles want 1024-byte alignment
    uint8_t* tiles_a = smem;
    uint8_t* tiles_b = smem + STAGES * A_BYTES;
    uint64_t* full = (uint64_t*)(tiles_b + STAGES * B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;                  // [2] an accumulator is complete
    uint64_t* acc_empty = acc_full + 2;                   // [2] an accumulator has been read out
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // A CTA takes the tiles blockIdx.x, blockIdx.x + gridDim.x, ... (tokens-as-rows: one CTA per
    // SM walks many tiles; weights-as-rows: the grid has one CTA per tile).
    const int n_tiles = WEIGHT_ROWS ? (int)gridDim.x : args.tiles_m * args.tiles_n;
    auto tile_at = [&](int t, int& ta, int& tb) {
        // weights-as-rows: tiles_m token tiles of BN tokens per weight tile, neighbours in the grid, so
        // that the CTAs that share a weight tile ask for it at about the same time (one trip to HBM)
        if constexpr (WEIGHT_ROWS) { ta = t / args.tiles_m; tb = t - ta * args.tiles_m; }
        else tile_of(t, args.tiles_m, args.tiles_n, ta, tb);
    };
    // k range of this CTA (cut over blockIdx.z)
    const int per = (args.k_blocks + gridDim.z - 1) / gridDim.z;
    const int kb0 = blockIdx.z * per;
    const int kb1 = min(args.k_blocks, kb0 + per);
    const int nkb = max(kb1 - kb0, 0);

    pdl_launch_dependents();                    // the next kernel in the stream may set itself up while this one runs
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0 && lane == 0) { prefetch_tmap(&map_a); prefetch_tmap(&map_b); }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (elect_one()) {
            int issued = 0;                                   // k blocks requested so far, over all tiles
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                int tile_a, tile_b;
                tile_at(t, tile_a, tile_b);
                int first = 0;
                if (issued == 0) {
                    // Weights are written by no kernel, so their tiles for the first stages are requested
                    // before this grid waits for the kernel before it; the activations come after.
                    const int pre = min(nkb, STAGES);
                    for (int i = 0; i < pre; ++i) {
                        mbar_expect_tx(&full[i], A_BYTES + B_BYTES);
                        if constexpr (WEIGHT_ROWS) tma_load_2d(tiles_a + i * A_BYTES, &map_a, &full[i], (kb0 + i) * TC_BK, tile_a * TC_BM);
                        else tma_load_2d(tiles_b + i * B_BYTES, &map_b, &full[i], (kb0 + i) * TC_BK, tile_b * BN);
                    }
                    pdl_wait();
                    for (int i = 0; i < pre; ++i) {
                        if constexpr (WEIGHT_ROWS) tma_load_2d(tiles_b + i * B_BYTES, &map_b, &full[i], (kb0 + i) * TC_BK, tile_b * BN);
                        else tma_load_2d(tiles_a + i * A_BYTES, &map_a, &full[i], (kb0 + i) * TC_BK, tile_a * TC_BM);
                    }
                    issued = first = pre;
                }
                for (int i = first; i < nkb; ++i) {
                    const int s = issued % STAGES;
                    if (issued >= STAGES && !mbar_wait(&empty[s], ((issued / STAGES) - 1) & 1, abort_flag, args.status, 1)) { ok = false; break; }
                    mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                    tma_load_2d(tiles_a + s * A_BYTES, &map_a, &full[s], (kb0 + i) * TC_BK, tile_a * TC_BM);
                    tma_load_2d(tiles_b + s * B_BYTES, &map_b, &full[s], (kb0 + i) * TC_BK, tile_b * BN);
                    ++issued;
                }
            }
            if (issued == 0) pdl_wait();
            if (*abort_flag) {
                // Wait (bounded) for this CTA's own copies in flight before shared memory goes away.
                for (int i = max(0, issued - STAGES); i < issued; ++i)
                    for (uint32_t t = 0; t < (1u << 20) && !mbar_try_wait(&full[i % STAGES], (i / STAGES) & 1); ++t) {}
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc = umma_idesc(BN);
            // No stage can fill before the kernel ahead has finished (the activations are requested
            // after the loader's own wait), so wait for it here too: the bounded polls below then
            // count this kernel's own progress only.
            pdl_wait();
            bool ok = true;
            int it = 0, lt = 0;                               // k blocks consumed, tiles done (both over all tiles)
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++lt) {
                const int buf = lt & 1, use = lt >> 1;
                if (use > 0) {                                // the epilogue must have read this accumulator out
                    ok = mbar_wait(&acc_empty[buf], (use - 1) & 1, abort_flag, args.status, 4);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t tmem_acc = tmem_base + buf * ACC_COLS;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, args.status, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = smem_desc_sw128(smem_u32(tiles_a + s * A_BYTES));
                    const uint64_t db = smem_desc_sw128(smem_u32(tiles_b + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)      // 16 bf16 = 32 bytes along the swizzled row: +2 in 16-byte units
                        umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty[s]);                   // the stage is free once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[buf]);                  // arrives when every MMA above is done (or at once if none)
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue: warps 2..5
        const int quarter = warp & 3;                         // the 32 tensor-memory lanes this warp may read
        pdl_wait();                                           // before this grid writes anything
        constexpr int TOKENS = BN > 64 ? BN : 64;
        static_assert(!WEIGHT_ROWS || TOKENS <= 128, "one epilogue thread per token sets its factor");
        __shared__ float inv_rms[TOKENS];                     // weights-as-rows: the factor of every token (column)
        if constexpr (WEIGHT_ROWS) {
            const int et = threadIdx.x - 64;                  // 0..127 among the epilogue threads
            if (et < TOKENS) {
                float f = 1.0f;
                if (args.scale_ss != nullptr) {
                    float ss = 0.f;
                    if (et < args.rows_b && et < 64)
                        for (int j = 0; j < args.scale_ss_n; ++j) ss += args.scale_ss[j * 64 + et];
                    f = rsqrtf(ss / (float)args.K + args.scale_eps);
                }
                inv_rms[et] = f;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        int lt = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++lt) {
        int tile_a, tile_b;
        tile_at(t, tile_a, tile_b);
        const int buf = lt & 1;
        const bool ok = mbar_wait(&acc_full[buf], (lt >> 1) & 1, abort_flag, args.status, 3) && !*abort_flag;
        tc_fence_after();
        const int row = tile_a * TC_BM + quarter * 32 + lane;              // row of the A operand
        const uint32_t taddr = tmem_base + buf * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
        if constexpr (WEIGHT_ROWS) {
            if (args.swiglu) {
                // Tile rows 0..63 are gate features, 64..127 the up rows of the same features.  The
                // warps that hold the up rows pass them through shared memory (the stages are
                // free: every MMA has read them) to the warps that hold the gate rows.
                float* xch = reinterpret_cast<float*>(tiles_a);            // [BN tokens][64 features]
                const int f = (quarter & 1) * 32 + lane;                   // feature within the tile
                uint32_t r[16];
                if (ok && quarter >= 2) {
                    // The loops over the chunks of 16 tokens stay rolled: a CTA runs its epilogue once, and
                    // unrolled for 64 tokens most of its time went to instruction fetches (64 sequences of the
                    // 8B shape: 4.94 ms per decode step unrolled, 4.53 ms rolled).
#pragma unroll 1
                    for (int c = 0; c < BN; c += 16) {
                        if (nkb > 0) { tmem_ld16(taddr + c, r); tmem_ld_wait(); }
                        else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) r[j] = 0u;
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) xch[(c + j) * 64 + f] = __uint_as_float(r[j]) * inv_rms[c + j];
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");             // the four epilogue warps, whatever happened
                if (ok && quarter < 2) {
                    const int feature = tile_a * 64 + f;
                    __nv_bfloat16* outb = (__nv_bfloat16*)args.out;
#pragma unroll 1
                    for (int c = 0; c < BN; c += 16) {
                        if (nkb > 0) { tmem_ld16(taddr + c, r); tmem_ld_wait(); }
                        else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) r[j] = 0u;
                        }
                        if (feature < args.rows_a / 2) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int m = c + j, token = tile_b * BN + m;
                                if (token < args.rows_b)
                                    outb[(size_t)token * args.ld_out + feature] =
                                        __float2bfloat16_rn(silu_mul(__uint_as_float(r[j]) * inv_rms[m], xch[m * 64 + f]));
                            }
                        }
                    }
                }
            } else if (ok) {
                // tile rows are output features n, tile columns are tokens m: out[z][m][n]
                float* out = (float*)args.out + (size_t)blockIdx.z * args.split_stride;
                __nv_bfloat16* outb = (__nv_bfloat16*)args.out;
                uint32_t r[16];
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    if (nkb > 0) { tmem_ld16(taddr + c, r); tmem_ld_wait(); }
                    else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = 0u;
                    }
                    const int token0 = tile_b * BN + c;
                    if (row < args.rows_a && args.out_f32) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (token0 + j < args.rows_b) out[(size_t)(token0 + j) * args.ld_out + row] = __uint_as_float(r[j]) * inv_rms[c + j];
                    } else if (row < args.rows_a) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (token0 + j < args.rows_b)
                                outb[(size_t)(token0 + j) * args.ld_out + row] = __float2bfloat16_rn(__uint_as_float(r[j]) * inv_rms[c + j]);
                    }
                }
            }
            if (args.sink != nullptr) {
                // The last CTA of this row tile (over the k cuts) adds all pieces, in ascending order, into
                // the residual stream and leaves the sum of squares of its 128 columns for every row.
                __shared__ int last_flag;
                __shared__ float ss_part[4][64];
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    const int done = atomicAdd(&args.sink_counters[tile_a], 1);
                    last_flag = done == (int)gridDim.z - 1;
                    if (last_flag) args.sink_counters[tile_a] = 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (last_flag) {
                    __threadfence();
                    // Four rows at a time and four pieces at a time, so that 16 loads are in flight per
                    // thread; every sum still runs over the pieces in ascending order.
                    const float* part = (const float*)args.out + row;
                    float* stream = args.sink + row;
                    const bool live = row < args.rows_a;
                    const int Z = (int)gridDim.z;
                    const float nw = (live && args.sink_scaled != nullptr) ? args.sink_w[row] : 0.f;
                    for (int m0 = 0; m0 < args.rows_b; m0 += 4) {
                        float x[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            x[j] = (live && m0 + j < args.rows_b) ? stream[(size_t)(m0 + j) * args.rows_a] : 0.f;
                        for (int z0 = 0; z0 < Z; z0 += 4) {
                            float p[4][4];
#pragma unroll
                            for (int zz = 0; zz < 4; ++zz)
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    p[zz][j] = (live && z0 + zz < Z && m0 + j < args.rows_b)
                                        ? __ldcg(part + (size_t)(z0 + zz) * args.split_stride + (size_t)(m0 + j) * args.ld_out) : 0.f;
#pragma unroll
                            for (int zz = 0; zz < 4; ++zz)
#pragma unroll
                                for (int j = 0; j < 4; ++j) x[j] += p[zz][j];
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (live && m0 + j < args.rows_b) {
                                stream[(size_t)(m0 + j) * args.rows_a] = x[j];
                                if (args.sink_scaled != nullptr)
                                    args.sink_scaled[(size_t)(m0 + j) * args.rows_a + row] = __float2bfloat16_rn(x[j] * nw);
                            }
                            const float sq = warp_sum(x[j] * x[j]);
                            if (lane == 0 && m0 + j < 64) ss_part[quarter][m0 + j] = sq;
                        }
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const int et = threadIdx.x - 64;
                    if (et < args.rows_b)
                        args.sink_ss[tile_a * 64 + et] = (ss_part[0][et] + ss_part[1][et]) + (ss_part[2][et] + ss_part[3][et]);
                }
            }
        } else if (ok) {
            if (args.swiglu) {
                // tile columns: 64 gate, 64 up, 64 gate, 64 up -> 128 outputs silu(gate) * up per row
                uint32_t rg[32], ru[32];
#pragma unroll 1
                for (int c = 0; c < BN / 2; c += 32) {                     // c: output column within the tile
                    const int f0 = tile_b * (BN / 2) + c;
                    if (f0 >= args.rows_b / 2) break;
                    const int col = (c / 64) * 128 + (c % 64);             // gate column in the accumulator
                    if (nkb > 0) { tmem_ld32(taddr + col, rg); tmem_ld32(taddr + col + 64, ru); tmem_ld_wait(); }
                    else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) { rg[j] = 0u; ru[j] = 0u; }
                    }
                    if (row < args.rows_a) store_row_chunk_swiglu(args, row, f0, rg, ru);
                }
            } else {
                // tile rows are tokens m, tile columns are output features n: out[m][n]
                uint32_t r[32];
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    const int n0 = tile_b * BN + c;
                    if (n0 >= args.rows_b) break;             // uniform across the warp
                    if (nkb > 0) { tmem_ld32(taddr + c, r); tmem_ld_wait(); }
                    else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = 0u;
                    }
                    if (row < args.rows_a) store_row_chunk(args, row, n0, r);
                }
            }
        }
        // this accumulator may be filled again once all four warps have read it out
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        if (!ok) break;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------ pairs of CTAs (prefill)
// Tokens as rows with tiles of 256 tokens x 256 features worked by two CTAs of a cluster as one
// (cta_group::2).  Each CTA stages its own 128 token rows and 128 of the tile's 256 weight rows, the
// CTA of even rank issues MMAs of M = 256, N = 256 that read both CTAs' shared memory and fill both
// CTAs' tensor memory (each keeps its 128 rows of the result).  Per 64 k a CTA then takes 32 KB of
// operands from L2 instead of 48 KB for the same products, and that traffic is what bounds the
// single-CTA kernel above (and costs energy, which bounds the whole prefill step).  TMA loads are
// plain per-CTA loads that report to the even CTA's barrier; the MMA's completion is committed to
// both CTAs' barriers.  Persistent: pair p walks the tiles p, p + pairs, ...; two accumulators of 256
// columns, one drained by both CTAs' epilogue warps while the other is filled.
template <int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmArgs args) {
    constexpr int BN = 256;
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = (BN / 2) * TC_BK * 2;
    constexpr uint32_t STAGE_TX = 2u * (A_BYTES + B_BYTES);
    constexpr uint32_t ACC_COLS = BN, TMEM_COLS = 2 * ACC_COLS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles_a = smem;
    uint8_t* tiles_b = smem + STAGES * A_BYTES;
    uint64_t* full = (uint64_t*)(tiles_b + STAGES * B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_tiles = args.tiles_m * args.tiles_n;              // tiles of 256 x 256
    const int nkb = args.k_blocks;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }   // 4 epilogue warps of each CTA
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0 && lane == 0) { prefetch_tmap(&map_a); prefetch_tmap(&map_b); }
    if (warp == 1) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                               // the other CTA's barriers exist before anything reports to them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t rank = cluster_ctarank();

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        if (elect_one()) {
            int issued = 0;
            bool ok = true;
            for (int t = pair; t < n_tiles && ok; t += n_pairs) {
                int tm, tn;
                tile_of(t, args.tiles_m, args.tiles_n, tm, tn);
                const int row_a = tm * 2 * TC_BM + (int)rank * TC_BM, row_b = tn * BN + (int)rank * (BN / 2);
                int first = 0;
                if (issued == 0) {
                    // weights before this grid waits for the kernel ahead, activations after
                    const int pre = min(nkb, STAGES);
                    for (int i = 0; i < pre; ++i) {
                        if (rank == 0) mbar_expect_tx(&full[i], STAGE_TX);
                        tma_load_2d_pair(tiles_b + i * B_BYTES, &map_b, mapa(smem_u32(&full[i]), 0), i * TC_BK, row_b);
                    }
                    pdl_wait();
                    for (int i = 0; i < pre; ++i)
                        tma_load_2d_pair(tiles_a + i * A_BYTES, &map_a, mapa(smem_u32(&full[i]), 0), i * TC_BK, row_a);
                    issued = first = pre;
                }
                for (int i = first; i < nkb; ++i) {
                    const int s = issued % STAGES;
                    if (issued >= STAGES && !mbar_wait(&empty[s], ((issued / STAGES) - 1) & 1, abort_flag, args.status, 1)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(&full[s], STAGE_TX);
                    const uint32_t bar = mapa(smem_u32(&full[s]), 0);
                    tma_load_2d_pair(tiles_a + s * A_BYTES, &map_a, bar, i * TC_BK, row_a);
                    tma_load_2d_pair(tiles_b + s * B_BYTES, &map_b, bar, i * TC_BK, row_b);
                    ++issued;
                }
            }
            if (issued == 0) pdl_wait();
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (the even CTA, for both)
        if (rank == 0 && elect_one()) {
            constexpr uint32_t idesc = umma_idesc(BN, 2 * TC_BM);
            pdl_wait();
            bool ok = true;
            int it = 0, lt = 0;
            for (int t = pair; t < n_tiles && ok; t += n_pairs, ++lt) {
                const int buf = lt & 1, use = lt >> 1;
                if (use > 0) {                                // both CTAs' epilogues must have read this accumulator out
                    ok = mbar_wait(&acc_empty[buf], (use - 1) & 1, abort_flag, args.status, 4);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t tmem_acc = tmem_base + buf * ACC_COLS;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, args.status, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = smem_desc_sw128(smem_u32(tiles_a + s * A_BYTES));
                    const uint64_t db = smem_desc_sw128(smem_u32(tiles_b + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_bf16_pair(tmem_acc, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty[s], 3);           // the stage is free in both CTAs once these MMAs have read it
                }
                if (!ok) break;
                umma_commit_pair(&acc_full[buf], 3);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue: warps 2..5 of both CTAs, 128 rows each
        const int quarter = warp & 3;
        pdl_wait();
        int lt = 0;
        for (int t = pair; t < n_tiles; t += n_pairs, ++lt) {
            int tm, tn;
            tile_of(t, args.tiles_m, args.tiles_n, tm, tn);
            const int buf = lt & 1;
            const bool ok = mbar_wait(&acc_full[buf], (lt >> 1) & 1, abort_flag, args.status, 3) && !*abort_flag;
            tc_fence_after();
            const int row = tm * 2 * TC_BM + (int)rank * TC_BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + buf * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            if (ok && args.swiglu) {
                uint32_t rg[32], ru[32];
#pragma unroll 1
                for (int c = 0; c < BN / 2; c += 32) {
                    const int f0 = tn * (BN / 2) + c;
                    if (f0 >= args.rows_b / 2) break;
                    const int col = (c / 64) * 128 + (c % 64);
                    if (nkb > 0) { tmem_ld32(taddr + col, rg); tmem_ld32(taddr + col + 64, ru); tmem_ld_wait(); }
                    else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) { rg[j] = 0u; ru[j] = 0u; }
                    }
                    if (row < args.rows_a) store_row_chunk_swiglu(args, row, f0, rg, ru);
                }
            } else if (ok) {
                uint32_t r[32];
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    const int n0 = tn * BN + c;
                    if (n0 >= args.rows_b) break;
                    if (nkb > 0) { tmem_ld32(taddr + c, r); tmem_ld_wait(); }
                    else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = 0u;
                    }
                    if (row < args.rows_a) store_row_chunk(args, row, n0, r);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&acc_empty[buf]), 0));
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                 // neither CTA leaves (or frees tensor memory) while the other may still reach into it
    if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------ host side

// A tensor map over a [rows, cols] bf16 matrix with `ld` elements between rows; box = 64
// columns x box_rows rows.
static int make_map(CUtensorMap* out, const void* ptr, int rows, int cols, long long ld, int box_rows) {
    const long long dims[2] = {cols, rows}, strides[1] = {ld};
    const int box[2] = {TC_BK, box_rows};
    return tma_make_map(out, ptr, 2, dims, strides, box);
}

template <int BN, int STAGES, bool WEIGHT_ROWS>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& args, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        KL_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, WEIGHT_ROWS>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    launch_kernel(gemm_tcgen05_kernel<BN, STAGES, WEIGHT_ROWS>, grid, TC_THREADS, smem, stream, ma, mb, args);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// KL_GEMM_PAIRS=0 in the environment keeps every CTA on its own (for comparisons).
static bool pairs_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("KL_GEMM_PAIRS");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

static int launch_pairs(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& args, int grid_x, cudaStream_t stream) {
    constexpr int STAGES = 6;
    constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + 128 * TC_BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        KL_CUDA(cudaFuncSetAttribute(gemm_pair_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    launch_kernel_clustered(gemm_pair_kernel<STAGES>, 2, dim3(grid_x, 1, 1), TC_THREADS, smem, stream, ma, mb, args);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

static bool aligned_operand(const void* p, long long ld, int K) {
    return ((uintptr_t)p & 15) == 0 && (ld % 8) == 0 && (K % 8) == 0 && K > 0;
}

}  // namespace kl

using namespace kl;

// out[M, N] = a[M, K] * w[N, K]^T, tokens as tile rows (any M).  out is bf16 (out_f32 = 0) or
// float32.  Needs 16-byte aligned bases and row strides (K % 8 == 0): else KL_ERR_BAD_ALIGN.
KL_API int kl_gemm_tcgen05(const void* a, long long lda, const void* w, long long ldw, void* out, long long ldo, int M,
                           int N, int K, int out_f32, int swiglu, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KL_OK;
    if (swiglu && (out_f32 || N % 128)) return KL_ERR_BAD_SIZE;
    if (!aligned_operand(a, lda, K) || !aligned_operand(w, ldw, K)) return KL_ERR_BAD_ALIGN;
    CUtensorMap ma, mb;
    int rc;
    if ((rc = make_map(&ma, a, M, K, lda, TC_BM)) != KL_OK) return rc;
    // Pairs of CTAs on tiles of 256 tokens where that wastes no rows to speak of: an even number of
    // 128-token tiles, or so many tokens that half a tile of padding is little.
    if (pairs_enabled() && (((M + TC_BM - 1) / TC_BM) % 2 == 0 || M >= 1024)) {
        const int sms2 = kl::sm_count();
        if (sms2 <= 1) return KL_ERR_SETUP;
        if ((rc = make_map(&mb, w, N, K, ldw, 128)) != KL_OK) return rc;
        const int tiles_m2 = (M + 2 * TC_BM - 1) / (2 * TC_BM), tiles_n2 = (N + 255) / 256;
        if ((long long)tiles_m2 * tiles_n2 > 0x3fffffffLL) return KL_ERR_BAD_SIZE;
        GemmArgs pargs{out, ldo, 0, M, N, (K + TC_BK - 1) / TC_BK, out_f32, status, tiles_m2, tiles_n2, swiglu};
        return launch_pairs(ma, mb, pargs, 2 * min(tiles_m2 * tiles_n2, sms2 / 2), stream);
    }
    if ((rc = make_map(&mb, w, N, K, ldw, 256)) != KL_OK) return rc;
    const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + 255) / 256;
    GemmArgs args{out, ldo, 0, M, N, (K + TC_BK - 1) / TC_BK, out_f32, status, tiles_m, tiles_n, swiglu};
    if ((long long)tiles_m * tiles_n > 0x7fffffffLL) return KL_ERR_BAD_SIZE;
    const int sms = kl::sm_count();
    if (sms <= 0) return KL_ERR_SETUP;
    const int tiles = tiles_m * tiles_n;
    const int grid_x = min(tiles, sms);               // one CTA per SM walks the tiles
    dim3 grid(grid_x, 1, 1);
    return launch<256, 4, false>(ma, mb, args, grid, stream);
}

// Few tokens (M <= 512): weights as tile rows (beyond 64 tokens: up to four tiles of 128 tokens per
// weight tile), the K range cut into `splits` pieces.
// splits == 1: out[M, N] directly (bf16 or float32).  splits > 1: out is float32
// [splits, M, N] partial sums (out_f32 must be 1) for the caller to add.
//
// The residual stream inside the products (decode steps).  With `sink` (float32 [M, N]; out must be
// the float32 pieces, any splits >= 1) the last CTA of every 128-column tile adds the pieces into
// `sink` in ascending order, writes the tile's sum of squares per row to sink_ss[tile][64] and, with
// `sink_scaled` (bf16 [M, N]), the new rows times `sink_w` [N] (the weight of the norm that follows);
// `sink_counters` (int32 [tiles]) are zero before and after.  With `scale_ss` (float32
// [scale_ss_n][64], pieces of every token's sum of squares) every token's result is multiplied by
// rsqrt(sum / K + scale_eps): with activations x * w this is the product of the normalised rows,
// norm(x) = w * x / rms(x).  Together they remove the add-and-normalise kernel between two products.
KL_API int kl_gemm_tcgen05_skinny(const void* a, long long lda, const void* w, long long ldw, void* out, long long ldo,
                                  int M, int N, int K, int splits, int out_f32, int swiglu, const float* scale_ss,
                                  int scale_ss_n, float scale_eps, float* sink, float* sink_ss, int* sink_counters,
                                  const float* sink_w, void* sink_scaled, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KL_OK;
    if (M > 512) return KL_ERR_BAD_SIZE;
    if (M > 64 && (scale_ss != nullptr || sink != nullptr)) return KL_ERR_BAD_SIZE;     // the folded norm: one tile of tokens
    if (swiglu && (splits != 1 || out_f32 || N % 128)) return KL_ERR_BAD_SIZE;
    if (!aligned_operand(w, ldw, K) || !aligned_operand(a, lda, K)) return KL_ERR_BAD_ALIGN;
    if (scale_ss != nullptr && scale_ss_n < 1) return KL_ERR_BAD_SIZE;
    if (sink != nullptr && (!out_f32 || swiglu || sink_ss == nullptr || sink_counters == nullptr || ldo != N ||
                            (sink_scaled != nullptr && sink_w == nullptr))) return KL_ERR_BAD_SIZE;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    if (splits < 1 || splits > k_blocks || splits > 65535) return KL_ERR_BAD_SIZE;
    if (splits > 1 && !out_f32) return KL_ERR_BAD_DTYPE;
    // More than 64 tokens: tiles of 128 tokens (a stage holds 16 KB of weights and 16 KB of tokens; with
    // two tiles of 64 tokens side by side the weights cross from L2 to the SMs twice).  KL_SKINNY_BN128=0: tiles of 64.
    static const int wide = getenv("KL_SKINNY_BN128") ? atoi(getenv("KL_SKINNY_BN128")) : 1;
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : ((M <= 64 || !wide) ? 64 : 128));
    CUtensorMap ma, mb;
    int rc;
    if ((rc = make_map(&ma, w, N, K, ldw, TC_BM)) != KL_OK) return rc;
    if ((rc = make_map(&mb, a, M, K, lda, bn)) != KL_OK) return rc;
    const int token_tiles = (M + bn - 1) / bn;
    GemmArgs args{out, ldo, (long long)M * ldo, N, M, k_blocks, out_f32, status, token_tiles, 0, swiglu,
                  scale_ss, scale_ss_n, scale_eps, K, sink, sink_ss, sink_counters, sink_w, (__nv_bfloat16*)sink_scaled};
    dim3 grid(((N + TC_BM - 1) / TC_BM) * token_tiles, 1, splits);
    // A grid of at most one CTA per SM (small matrices) gives each CTA the whole of the SM's shared
    // memory as stages: what a CTA has in flight bounds what it streams (96 KB over the 1.5 us a tile
    // takes to arrive are 64 GB/s).  Otherwise two CTAs share an SM, so that one's epilogue overlaps
    // the other's loads.
    const int sms = kl::sm_count();
    if (sms <= 0) return KL_ERR_SETUP;
    if ((long long)grid.x * splits <= sms) {
        if (bn == 16) return launch<16, 12, true>(ma, mb, args, grid, stream);
        if (bn == 32) return launch<32, 10, true>(ma, mb, args, grid, stream);
        if (bn == 64) return launch<64, 8, true>(ma, mb, args, grid, stream);
        return launch<128, 6, true>(ma, mb, args, grid, stream);
    }
    if (bn == 128) return launch<128, 3, true>(ma, mb, args, grid, stream);
    if (bn == 16) return launch<16, 6, true>(ma, mb, args, grid, stream);
    if (bn == 32) return launch<32, 5, true>(ma, mb, args, grid, stream);
    return launch<64, 4, true>(ma, mb, args, grid, stream);
}

namespace kl {
// out[m, n] = sum over z of partial[z, m, n], added in ascending z.
template <typename TO>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, int M, int N, TO* __restrict__ out,
                                     long long ldo) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)M * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int z = 0; z < splits; ++z) acc += partial[(size_t)z * total + i];
        const size_t m = i / N, n = i - m * N;
        out[m * ldo + n] = from_f32<TO>(acc);
    }
}
}  // namespace kl

KL_API int kl_splitk_reduce(const float* partial, int splits, int M, int N, void* out, long long ldo, int out_f32,
                            cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KL_OK;
    const size_t total = (size_t)M * N;
    const int threads = 256;
    const int blocks = kl::strided_grid(total, threads, 8);
    if (out_f32) launch_kernel(kl::splitk_reduce_kernel<float>, blocks, threads, 0, stream, partial, splits, M, N, (float*)out, ldo);
    else launch_kernel(kl::splitk_reduce_kernel<kl::bf16>, blocks, threads, 0, stream, partial, splits, M, N, (kl::bf16*)out, ldo);
    KL_LAUNCH_CHECK();
    return KL_OK;
}
