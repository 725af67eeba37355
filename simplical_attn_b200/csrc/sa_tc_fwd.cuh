// Forward 2-simplicial attention on the sm_100a tensor cores (tcgen05 MMA, accumulators in tensor
// memory, K1/V1 window tiles staged by TMA).  Replaces the reference's
// two_simplicial_attn_fwd_kernel (simplicial/kernels.py:11-171).
//
// Formulation.  A query i and a K2 position k = i - delta (delta in [0, w2)) form one "virtual
// row" r = (i, delta) with the operand row  A[r, :] = Q_i * (K2_k + k2_bias)  (elementwise, formed
// on chip).  Then
//     S[r, j] = A[r, :] . K1[j, :]                      tensor-core GEMM, K = D
//     P[r, j] = exp2(S * scale*log2e - m_r)             online softmax per virtual row
//     T[r, :] = sum_j P[r, j] * V1[j, :]                tensor-core GEMM, K = j
//     O_i     = sum_delta w_r * (V2_k + v2_bias) * T[r, :] / L_i        epilogue merge over delta
// so the main loop is flash attention over the K1 window with 128-row tiles of virtual rows.
//
// A block works on "units" of 2 row tiles (2 x 128 virtual rows = 2 * 128/DW consecutive queries,
// DW = w2 rounded up to a power of two).  Both row tiles stream through the same K1/V1 column
// tiles (128 K1 rows each; the last tile of a unit is only as wide as needed, in steps of 16).
//
// Warps: 0-3 softmax/epilogue group of row tile 0, 4-7 the same for row tile 1, warp 8 issues the
// TMA loads, warp 9 issues the MMAs.  Tensor memory: S0 | S1 (128 fp32 columns each, P overwrites
// S in place as packed bf16) | T0 | T1 (D columns each).
#pragma once

#include "sa_ptx.cuh"

namespace sa {
namespace tc {

constexpr int kRowTile = 128;          // virtual rows per row tile = tensor-memory lanes
constexpr int kColTile = 128;          // K1/V1 rows per column tile
constexpr int kNumRowTiles = 2;        // row tiles per unit
constexpr int kStages = 2;             // K1/V1 ring depth
constexpr int kFwdThreads = 384;       // 2 softmax groups, TMA warp (8), MMA warp (9), 2 idle warps
constexpr float kRescaleThreshold = 8.0f;   // log2 units; below it the running maximum is kept

struct FwdTcParams {
    KParams k;
    int dw_log2;          // DW = 1 << dw_log2 delta slots per query
    int num_qblocks;      // ceil(N / queries per unit)
    long num_units;       // B * H * num_qblocks
    DeviceStatus* status;
    uint64_t wait_limit_ns;   // bound of every device-side wait
};

template <int HD>
struct FwdSmem {
    static constexpr int kSlabs = HD / 64;                       // 64-element slabs per tile
    static constexpr int kTileBytes = kRowTile * HD * 2;         // one [128 x HD] bf16 tile
    static constexpr int kSlabBytes = kRowTile * 128;
    // byte offsets from the 1024-aligned base
    static constexpr int kA = 0;                                 // 2 row tiles
    static constexpr int kK1 = kA + kNumRowTiles * kTileBytes;   // kStages tiles
    static constexpr int kV1 = kK1 + kStages * kTileBytes;       // kStages tiles
    static constexpr int kStats = kV1 + kStages * kTileBytes;    // m, l: 2 groups x 128 x 2 floats
    static constexpr int kBars = kStats + kNumRowTiles * kRowTile * 2 * 4;
    static constexpr int kNumBars = 4 * kStages + 7 * kNumRowTiles;
    static constexpr int kMisc = kBars + kNumBars * 8;           // tmem base, abort flag
    static constexpr int kScratch = kMisc + 16;                  // only used when HD == 64
    static constexpr int kScratchBytes = (HD == 64) ? kNumRowTiles * kRowTile * 32 * 4 : 0;
    static constexpr int kTotal = kScratch + kScratchBytes;
    static constexpr int kAlloc = (kTotal + 1024 > 120 * 1024) ? kTotal + 1024 : 120 * 1024;   // > half an SM: one block per SM
};

// Unit -> (batch, head, first query, column range).
struct UnitGeom {
    int b, h, hk, i0;
    int col_start;     // first K1/V1 buffer row the unit needs
    int ntiles;        // column tiles
    int last_width;    // width of the last tile, multiple of 16
};

__device__ __forceinline__ UnitGeom unit_geom(const FwdTcParams& P, long u) {
    const KParams& p = P.k;
    UnitGeom g;
    const int qpb = (kNumRowTiles * kRowTile) >> P.dw_log2;
    const int qb = (int)(u % P.num_qblocks);
    const long bh = u / P.num_qblocks;
    g.h = (int)(bh % p.H);
    g.b = (int)(bh / p.H);
    g.hk = g.h / p.G;
    g.i0 = qb * qpb;
    const int i_last = min(g.i0 + qpb, p.N) - 1;
    g.col_start = max(0, g.i0 + p.halo1 - p.w1 + 1);
    const int ncols = i_last + p.halo1 - g.col_start + 1;
    g.ntiles = (ncols + kColTile - 1) / kColTile;
    g.last_width = ((ncols - (g.ntiles - 1) * kColTile) + 15) & ~15;
    return g;
}

// BIAS = false: both biases are zero, every bias add folds away.
template <int HD, bool BIAS>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_tc_kernel(const __grid_constant__ FwdTcParams P, const __grid_constant__ CUtensorMap map_k1,
              const __grid_constant__ CUtensorMap map_v1, const __nv_bfloat16* __restrict__ q,
              const __nv_bfloat16* __restrict__ k2, const __nv_bfloat16* __restrict__ v2,
              __nv_bfloat16* __restrict__ o, float* __restrict__ lse) {
    using L = FwdSmem<HD>;
    using namespace ptx;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const KParams& p = P.k;
    const float k2_bias = BIAS ? p.k2_bias : 0.f, v2_bias = BIAS ? p.v2_bias : 0.f;

    uint64_t* bars = (uint64_t*)(smem + L::kBars);
    uint64_t* k1_full = bars;                       // [kStages]
    uint64_t* k1_empty = bars + kStages;
    uint64_t* v1_full = bars + 2 * kStages;
    uint64_t* v1_empty = bars + 3 * kStages;
    uint64_t* a_ready = bars + 4 * kStages;         // [kNumRowTiles]
    uint64_t* s_ready = a_ready + kNumRowTiles;
    uint64_t* o_ready = s_ready + kNumRowTiles;
    uint64_t* p_ready = o_ready + kNumRowTiles;     // [kNumRowTiles][4]: P of one 32-column chunk stored
    uint32_t* tmem_base_slot = (uint32_t*)(smem + L::kMisc);
    volatile int* abort_flag = (volatile int*)(smem + L::kMisc + 4);
    const WaitCtx wctx{abort_flag, P.status, P.wait_limit_ns};

    const int tid = threadIdx.x;
    SA_PROF_T0(t_life);
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&k1_full[s], 1);
            mbar_init(&k1_empty[s], 1);
            mbar_init(&v1_full[s], 1);
            mbar_init(&v1_empty[s], 1);
        }
        for (int r = 0; r < kNumRowTiles; ++r) {
            mbar_init(&a_ready[r], kRowTile);
            mbar_init(&s_ready[r], 1);
            for (int c = 0; c < 4; ++c) mbar_init(&p_ready[4 * r + c], kRowTile);
            mbar_init(&o_ready[r], 1);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 9) {
        tmem_alloc(tmem_base_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const uint32_t tmem_s[2] = {tmem_base, tmem_base + 128};
    const uint32_t tmem_t[2] = {tmem_base + 256, tmem_base + 256 + HD};

    const int DW = 1 << P.dw_log2;
    const int qpt = kRowTile >> P.dw_log2;          // queries per row tile

    if (warp == 8) {
        // ------------------------------------------------------------------ TMA producer
        reg_dealloc<72>();
        if (lane == 0) {
            prefetch_tensormap(&map_k1);
            prefetch_tensormap(&map_v1);
            uint32_t g = 0;                           // running column-tile counter (ring position)
            for (long u = blockIdx.x; u < P.num_units; u += gridDim.x) {
                const UnitGeom ug = unit_geom(P, u);
                for (int t = 0; t < ug.ntiles; ++t, ++g) {
                    const int s = g % kStages;
                    const uint32_t ph = (g / kStages) & 1;
                    const int row = ug.col_start + t * kColTile;
                    mbar_wait(&k1_empty[s], ph ^ 1, wctx, 1);
                    mbar_arrive_expect_tx(&k1_full[s], L::kTileBytes);
#pragma unroll
                    for (int sl = 0; sl < L::kSlabs; ++sl)
                        tma_load_4d(smem + L::kK1 + s * L::kTileBytes + sl * L::kSlabBytes, &map_k1, &k1_full[s], sl * 64,
                                    row, ug.hk, ug.b);
                    mbar_wait(&v1_empty[s], ph ^ 1, wctx, 2);
                    mbar_arrive_expect_tx(&v1_full[s], L::kTileBytes);
#pragma unroll
                    for (int sl = 0; sl < L::kSlabs; ++sl)
                        tma_load_4d(smem + L::kV1 + s * L::kTileBytes + sl * L::kSlabBytes, &map_v1, &v1_full[s], sl * 64,
                                    row, ug.hk, ug.b);
                }
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        reg_dealloc<72>();
        {
            const uint32_t leader = elect_one();      // the whole warp runs the loop; one lane issues
            const uint32_t idesc_pv = make_idesc(128, HD, false, true);
            const uint32_t idesc_s_full = make_idesc(128, kColTile, false, false);
            uint32_t g = 0;          // ring position of the unit's first tile
            uint32_t nu = 0;         // units done (phase of a_ready / o_ready)
            uint32_t ns[2] = {0, 0}; // S tiles issued per row tile (phase of s_ready / p_ready)
            for (long u = blockIdx.x; u < P.num_units; u += gridDim.x, ++nu) {
                const UnitGeom ug = unit_geom(P, u);
                auto width_of = [&](int t) { return t == ug.ntiles - 1 ? ug.last_width : kColTile; };
                auto issue_s = [&](int r, int t) {
                    const int s = (g + t) % kStages;
                    const uint32_t idesc_s = (t == ug.ntiles - 1) ? make_idesc(128, ug.last_width, false, false) : idesc_s_full;
                    const uint64_t da = desc_kmajor(smem_base + L::kA + r * L::kTileBytes, 0);
                    const uint64_t db = desc_kmajor(smem_base + L::kK1 + s * L::kTileBytes, 0);
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk) {
                        const uint32_t off = ((kk >> 2) * L::kSlabBytes + (kk & 3) * 32) >> 4;
                        mma_ss(leader, tmem_s[r], da + off, db + off, idesc_s, kk > 0);
                    }
                    tc_commit(leader, &s_ready[r]);
                };
                // P arrives in two halves of 64 columns (four k-steps each): the MMAs of a chunk are issued as
                // soon as it is stored, while the softmax group works on the next one.
                auto issue_pv = [&](int r, int t, uint32_t parity, uint32_t gt) {
                    const int s = (g + t) % kStages;
                    const uint64_t db = desc_mnmajor(smem_base + L::kV1 + s * L::kTileBytes, L::kSlabBytes);
                    const int ksteps = (t != ug.ntiles - 1) ? kColTile / 16 : ug.last_width / 16;
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        mbar_wait(&p_ready[4 * r + c], parity, wctx, 5);
                        if (c == 0 && r == 0) mbar_wait(&v1_full[gt % kStages], (gt / kStages) & 1, wctx, 6);
                        tc_fence_after();
#pragma unroll
                        for (int kk = 4 * c; kk < 4 * c + 4; ++kk)
                            if (kk < ksteps) mma_ts(leader, tmem_t[r], tmem_s[r] + kk * 8, db + kk * (2048 >> 4), idesc_pv, t > 0 || kk > 0);
                    }
                };
                // prologue: S(0) of both row tiles
                mbar_wait(&k1_full[g % kStages], (g / kStages) & 1, wctx, 3);
                for (int r = 0; r < kNumRowTiles; ++r) {
                    mbar_wait(&a_ready[r], nu & 1, wctx, 4);
                    tc_fence_after();
                    issue_s(r, 0);
                }
                tc_commit(leader, &k1_empty[g % kStages]);
                for (int t = 0; t < ug.ntiles; ++t) {
                    const uint32_t gt = g + t;
                    for (int r = 0; r < kNumRowTiles; ++r) {
                        SA_PROF_T0(t_pv);
                        issue_pv(r, t, ns[r] & 1, gt);
                        ++ns[r];
                        SA_PROF_ADD(30, t_pv);
                        if (r == kNumRowTiles - 1) tc_commit(leader, &v1_empty[gt % kStages]);
                        if (t + 1 < ug.ntiles) {
                            if (r == 0) {
                                mbar_wait(&k1_full[(gt + 1) % kStages], ((gt + 1) / kStages) & 1, wctx, 7);
                                tc_fence_after();
                            }
                            SA_PROF_T0(t_s);
                            issue_s(r, t + 1);
                            SA_PROF_ADD(31, t_s);
                            if (r == kNumRowTiles - 1) tc_commit(leader, &k1_empty[(gt + 1) % kStages]);
                        } else {
                            tc_commit(leader, &o_ready[r]);
                        }
                    }
                }
                g += ug.ntiles;
            }
        }
        __syncwarp();
    } else if (warp >= 10) {
        reg_dealloc<72>();
    } else {
        // ------------------------------------------------------------------ softmax / epilogue groups
        reg_alloc<216>();
        const int r = warp >> 2;                     // row tile of this group
        const int row = tid & 127;                   // virtual row = tensor-memory lane
        const uint32_t lane_addr = ((uint32_t)(row & ~31)) << 16;   // lane base of this warp
        const int qq = row >> P.dw_log2;
        const int delta = row & (DW - 1);
        uint8_t* a_tile = smem + L::kA + r * L::kTileBytes;
        float* scratch = (HD == 64) ? (float*)(smem + L::kScratch + r * kRowTile * 32 * 4) : (float*)a_tile;
        float* m_s = (float*)(smem + L::kStats) + r * 2 * kRowTile;
        float* l_s = m_s + kRowTile;
        const float c2 = p.scale * kLog2e;
        uint32_t nu = 0, ns = 0;
        for (long u = blockIdx.x; u < P.num_units; u += gridDim.x, ++nu) {
            const UnitGeom ug = unit_geom(P, u);
            const int i = ug.i0 + r * qpt + qq;
            const int kb = i + p.halo2 - delta;                    // K2/V2 buffer row
            const bool row_valid = (i < p.N) && (delta < p.w2) && (kb >= 0);
            // ---- form A_r: row (i, delta) = Q_i * (K2_{i-delta} + bias) as bf16, 128-byte swizzled
            SA_PROF_T0(t_form);
            form_query_tile<HD, BIAS>(a_tile, L::kSlabBytes, row, ug.i0 + r * qpt, P.dw_log2, p.N, p.w2, p.halo2,
                                      q + ug.b * p.q.b + ug.h * p.q.h, p.q.n, k2 + ug.b * p.k2.b + ug.hk * p.k2.h, p.k2.n, k2_bias);
            fence_proxy_async_smem();
            mbar_arrive(&a_ready[r]);
            SA_PROF_ADD(10 + r, t_form);
            SA_PROF_T0(t_loop);
            // ---- main loop over column tiles
            // Valid buffer rows of this virtual row: [jlo, jhi] (empty for an invalid row).
            const int jhi = row_valid ? i + p.halo1 : -1;
            const int jlo = row_valid ? max(0, i + p.halo1 - p.w1 + 1) : 0;
            float m = -INFINITY, l = 0.f;
            for (int t = 0; t < ug.ntiles; ++t, ++ns) {
                const int width = (t == ug.ntiles - 1) ? ug.last_width : kColTile;
                const int tile0 = ug.col_start + t * kColTile;
                const int lo = jlo - tile0, hi = jhi - tile0;        // valid tile-relative columns [lo, hi]
                mbar_wait(&s_ready[r], ns & 1, wctx, 8);
                tc_fence_after();
                SA_PROF_T0(t_sm);
                const uint32_t s_addr = tmem_s[r] + lane_addr;
                // a tile is "full" when every column is inside every row's window: no masks needed
                bool full = (width == kColTile) && __all_sync(0xffffffffu, lo <= 0 && hi >= kColTile - 1);
                if (!full && width == kColTile && __all_sync(0xffffffffu, lo <= 16 && hi >= kColTile - 1)) {
                    // The first tile of a unit: only the first few columns lie before the window of some rows.
                    // Overwrite those scores with a large negative number (their P becomes exactly 0) and
                    // treat the tile as full.
                    uint32_t e16[16];
                    tmem_ld16(s_addr, e16);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 16; ++e) e16[e] = (e < lo) ? __float_as_uint(-1e30f) : e16[e];
                    tmem_st16(s_addr, e16);
                    tmem_wait_st();
                    full = true;
                }
                float lsum = 0.f;
                // running maximum, lazily updated: returns the factor the row's T and l must be scaled by
                auto update_max = [&](float tmax) {
                    float factor = 1.f;
                    bool rescale = false;
                    if (tmax > m + kRescaleThreshold || (m == -INFINITY && tmax > -INFINITY)) {
                        rescale = (m != -INFINITY);
                        factor = rescale ? ex2(m - tmax) : 1.f;
                        m = tmax;
                    }
                    if (__any_sync(0xffffffffu, rescale)) {
                        l *= factor;
                        const uint32_t t_addr = tmem_t[r] + lane_addr;
#pragma unroll
                        for (int c0 = 0; c0 < HD; c0 += 32) {
                            uint32_t tv[32];
                            tmem_ld32(t_addr + c0, tv);
                            tmem_wait_ld();
#pragma unroll
                            for (int e = 0; e < 32; ++e) tv[e] = __float_as_uint(__uint_as_float(tv[e]) * factor);
                            tmem_st32(t_addr + c0, tv);
                        }
                    }
                };
                if (full) {
                    // two passes over tensor memory, 32 columns at a time, the next chunk's load in flight
                    // while the current one is processed (keeps the live registers at two chunks)
                    uint32_t v[2][32];
                    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    tmem_ld32(s_addr, v[0]);
#pragma unroll
                    for (int cch = 0; cch < 4; ++cch) {
                        tmem_wait_ld();
                        if (cch + 1 < 4) tmem_ld32(s_addr + 32 * (cch + 1), v[(cch + 1) & 1]);
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
#pragma unroll
                            for (int x = 0; x < 4; ++x)
                                mx[x] = max3(mx[x], __uint_as_float(v[cch & 1][e + x]), __uint_as_float(v[cch & 1][e + 4 + x]));
                        }
                    }
                    SA_PROF_ADD(20 + r, t_sm);
                    SA_PROF_T0(t_p2);
                    tmem_ld32(s_addr, v[0]);                  // issued before the (rare) rescale so its latency overlaps
                    update_max(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * c2);
                    // packed two-wide fp32 arithmetic: one FMA and one add per pair of columns
                    float2 ls = make_float2(0.f, 0.f);
                    const float2 c2v = make_float2(c2, c2), nm = make_float2(-m, -m);
#pragma unroll
                    for (int cch = 0; cch < 4; ++cch) {
                        tmem_wait_ld();
                        if (cch + 1 < 4) tmem_ld32(s_addr + 32 * (cch + 1), v[(cch + 1) & 1]);
                        uint32_t pk[16];
#pragma unroll
                        for (int e = 0; e < 32; e += 2) {
                            const float2 x = __ffma2_rn(make_float2(__uint_as_float(v[cch & 1][e]), __uint_as_float(v[cch & 1][e + 1])), c2v, nm);
                            const float2 pr = make_float2(ex2(x.x), ex2(x.y));
                            ls = __fadd2_rn(ls, pr);
                            pk[e >> 1] = pack_bf16(pr.x, pr.y);
                        }
                        // chunk cch of P (16 packed columns) lands on S columns that have been read already
                        tmem_st16(s_addr + 16 * cch, pk);
                        if (cch & 1) {       // a half tile of P is complete
                            tmem_wait_st();
                            tc_fence_before();
                            mbar_arrive(&p_ready[4 * r + (cch >> 1)]);
                        }
                    }
                    lsum = ls.x + ls.y;
                    SA_PROF_ADD(22 + r, t_p2);
                } else {
                    // pass 1: row maximum of the valid columns
                    float tmax = -INFINITY;
                    for (int c0 = 0; c0 < width; c0 += 32) {
                        uint32_t v[32];
                        tmem_ld32(s_addr + c0, v);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const int c = c0 + e;
                            if (c >= lo && c <= hi) tmax = fmaxf(tmax, __uint_as_float(v[e]));
                        }
                    }
                    update_max(tmax * c2);                                 // -inf stays -inf (c2 > 0)
                    // pass 2: P = exp2(S*c2 - m), packed bf16 over the S columns already consumed
                    const float msafe = (m == -INFINITY) ? 0.f : m;
                    for (int c0 = 0; c0 < width; c0 += 32) {
                        uint32_t v[32];
                        tmem_ld32(s_addr + c0, v);
                        tmem_wait_ld();
                        uint32_t pk[16];
#pragma unroll
                        for (int e = 0; e < 32; e += 2) {
                            const int c = c0 + e;
                            float p0 = ex2(fmaf(__uint_as_float(v[e]), c2, -msafe));
                            float p1 = ex2(fmaf(__uint_as_float(v[e + 1]), c2, -msafe));
                            p0 = (c >= lo && c <= hi) ? p0 : 0.f;
                            p1 = (c + 1 >= lo && c + 1 <= hi) ? p1 : 0.f;
                            lsum += p0 + p1;
                            pk[e >> 1] = pack_bf16(p0, p1);
                        }
                        tmem_st16(s_addr + (c0 >> 1), pk);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(&p_ready[4 * r]);
                    mbar_arrive(&p_ready[4 * r + 1]);
                    SA_PROF_ADD((t == 0 ? 24 : 26) + r, t_sm);
                }
                l += lsum;
                SA_PROF_ADD(16 + r, t_sm);
            }
            // ---- epilogue: merge the delta rows of each query
            SA_PROF_ADD(12 + r, t_loop);
            SA_PROF_T0(t_epi);
            float mq, lq;
            if (P.dw_log2 <= 5) {
                // the delta rows of a query are DW consecutive lanes of one warp: merge by register exchange
                mq = m;
                for (int sft = DW >> 1; sft >= 1; sft >>= 1) mq = fmaxf(mq, __shfl_xor_sync(0xffffffffu, mq, sft));
                lq = (m > -INFINITY) ? ex2(m - mq) * l : 0.f;
                for (int sft = DW >> 1; sft >= 1; sft >>= 1) lq += __shfl_xor_sync(0xffffffffu, lq, sft);
            } else {
                m_s[row] = m;
                l_s[row] = l;
                named_barrier_sync(1 + r, kRowTile);
                mq = -INFINITY;
                for (int d2 = 0; d2 < DW; ++d2) mq = fmaxf(mq, m_s[(qq << P.dw_log2) + d2]);
                lq = 0.f;
                for (int d2 = 0; d2 < DW; ++d2) {
                    const float mm = m_s[(qq << P.dw_log2) + d2];
                    if (mm > -INFINITY) lq += ex2(mm - mq) * l_s[(qq << P.dw_log2) + d2];
                }
            }
            const float wrow = (m > -INFINITY) ? ex2(m - mq) / lq : 0.f;
            const __nv_bfloat16* v2row = v2 + ug.b * p.v2.b + (long)max(kb, 0) * p.v2.n + ug.hk * p.v2.h;
            const uint32_t t_addr = tmem_t[r] + lane_addr;
            if (P.dw_log2 >= 5) {
                // this row's V2 values, fetched while the last MMAs of the unit are still running
                uint32_t vw[HD / 2];
#pragma unroll
                for (int e = 0; e < HD / 2; ++e) vw[e] = 0u;
                if (row_valid) load_bf16_words<HD>(v2row, vw);
                mbar_wait(&o_ready[r], nu & 1, wctx, 9);
                tc_fence_after();
                // a warp holds 32 consecutive deltas of one query: sum them by a register exchange;
                // lane L ends up with column L of each 32-column chunk
                const int wq = row >> 5;                      // warp within the group
                const int wpq = DW >> 5;                      // warps per query
                float* part = scratch;                        // [4 warps][HD] when a query spans several warps
                float tot[HD / 32];
#pragma unroll
                for (int cch = 0; cch < HD / 32; ++cch) {
                    uint32_t v[32];
                    tmem_ld32(t_addr + 32 * cch, v);
                    tmem_wait_ld();
                    float y[32];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        // rows that are not valid have T = 0 exactly (their P is 0) and wrow = 0: no select needed
                        const uint32_t w = vw[16 * cch + (e >> 1)];
                        float2 x2 = make_float2(bf16_lo(w), bf16_hi(w));
                        if (BIAS) x2 = __fadd2_rn(x2, make_float2(v2_bias, v2_bias));
                        const float2 y2 = __fmul2_rn(make_float2(__uint_as_float(v[e]), __uint_as_float(v[e + 1])),
                                                     __fmul2_rn(x2, make_float2(wrow, wrow)));
                        y[e] = y2.x;
                        y[e + 1] = y2.y;
                    }
                    tot[cch] = warp_transpose_reduce<32>(y, lane);
                }
                if (wpq == 1) {
                    if (i < p.N) {
                        __nv_bfloat16* orow = o + ug.b * p.o.b + (long)i * p.o.n + ug.h * p.o.h;
#pragma unroll
                        for (int cch = 0; cch < HD / 32; ++cch) orow[32 * cch + lane] = __float2bfloat16_rn(tot[cch]);
                    }
                } else {
#pragma unroll
                    for (int cch = 0; cch < HD / 32; ++cch) part[wq * HD + 32 * cch + lane] = tot[cch];
                    named_barrier_sync(1 + r, kRowTile);
                    for (int idx = row; idx < qpt * HD; idx += kRowTile) {
                        const int q2 = idx / HD, col = idx % HD;
                        float acc = 0.f;
                        for (int w2i = 0; w2i < wpq; ++w2i) acc += part[(q2 * wpq + w2i) * HD + col];
                        const int i2 = ug.i0 + r * qpt + q2;
                        if (i2 < p.N) o[ug.b * p.o.b + (long)i2 * p.o.n + ug.h * p.o.h + col] = __float2bfloat16_rn(acc);
                    }
                    named_barrier_sync(1 + r, kRowTile);
                }
            } else {
            mbar_wait(&o_ready[r], nu & 1, wctx, 9);
            tc_fence_after();
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(t_addr + c0, v);
                tmem_wait_ld();
                uint32_t vw[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) vw[e] = 0u;
                if (row_valid) load_bf16_words<32>(v2row + c0, vw);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const float vf = (e & 1) ? bf16_hi(vw[e >> 1]) : bf16_lo(vw[e >> 1]);
                    const float val = row_valid ? __uint_as_float(v[e]) * wrow * (vf + v2_bias) : 0.f;
                    scratch[row * 32 + (e ^ (row & 31))] = val;
                }
                named_barrier_sync(1 + r, kRowTile);
                for (int idx = row; idx < qpt * 32; idx += kRowTile) {
                    const int q2 = idx >> 5, e = idx & 31;
                    const int i2 = ug.i0 + r * qpt + q2;
                    float acc = 0.f;
                    for (int d2 = 0; d2 < DW; ++d2) {
                        const int rr = (q2 << P.dw_log2) + d2;
                        acc += scratch[rr * 32 + (e ^ (rr & 31))];
                    }
                    if (i2 < p.N) o[ug.b * p.o.b + (long)i2 * p.o.n + ug.h * p.o.h + c0 + e] = __float2bfloat16_rn(acc);
                }
                named_barrier_sync(1 + r, kRowTile);
            }
            }
            if (delta == 0 && i < p.N) lse[((long)ug.b * p.H + ug.h) * p.N + i] = (mq + log2f(lq)) * kLn2;
            SA_PROF_ADD(14 + r, t_epi);
            tc_fence_before();
        }
    }
    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    SA_PROF_LIFE(t_life);
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace tc
}  // namespace sa
