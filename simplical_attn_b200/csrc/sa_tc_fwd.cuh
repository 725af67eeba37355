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
// tiles (64 K1 rows each, a four-stage TMA ring; the last tile of a unit is only as wide as needed,
// in steps of 16).
//
// Warps: 0-3 softmax group of row tile 0, 4-7 the same for row tile 1; 8-11 the auxiliary group,
// which forms the A tiles of the NEXT unit while the current one is in its last column tiles and
// merges / writes the results of the unit that just finished, so that neither operand formation nor
// the epilogue ever stops the tensor cores; warps 12 and 13 issue the MMAs of row tile 0 and 1 (two
// issuers: the row tiles are independent streams, neither waits behind the other's barriers); warp
// 14 issues the TMA loads.  Tensor memory: two 64-column S buffers per row tile (S of the next tile
// is computed while the softmax works on the current one; P overwrites S in place as packed 16-bit
// values) | T0 | T1 (D columns each).
#pragma once

#include <type_traits>

#include "sa_ptx.cuh"

// Column pairs out of every eight whose exponential the forward takes on the FMA pipe (0: all on the
// special-function unit).  Measured on B200 with this kernel: 3 of 8 is 10 % slower than 0 -- the softmax
// warps are short of issue slots, not of special-function throughput -- so the default is 0.
#ifndef SA_FWD_POLY_OF_8
#define SA_FWD_POLY_OF_8 0
#endif
// Registers per thread of the softmax groups, the auxiliary group and the MMA / TMA warps (multiples of 8).
#ifndef SA_FWD_REGS_SM
#define SA_FWD_REGS_SM 152
#define SA_FWD_REGS_AUX 144
#define SA_FWD_REGS_REST 64
#endif

namespace sa {
namespace tc {

constexpr int kRowTile = 128;          // virtual rows per row tile = tensor-memory lanes
constexpr int kSubTile = 64;           // columns of one S tile = K1/V1 rows of one TMA stage
constexpr int kNumRowTiles = 2;        // row tiles per unit
constexpr int kStages = 4;             // K1/V1 ring depth
constexpr int kFwdThreads = 512;       // 2 softmax groups, auxiliary group, MMA warps (12, 13), TMA warp (14), 1 idle warp
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
    static constexpr int kTileBytes = kRowTile * HD * 2;         // one [128 x HD] bf16 A tile
    static constexpr int kSlabBytes = kRowTile * 128;
    static constexpr int kStageBytes = kSubTile * HD * 2;        // one [64 x HD] bf16 K1 or V1 stage
    static constexpr int kStageSlab = kSubTile * 128;
    // byte offsets from the 1024-aligned base
    static constexpr int kA = 0;                                 // 2 row tiles
    static constexpr int kK1 = kA + kNumRowTiles * kTileBytes;   // kStages stages
    static constexpr int kV1 = kK1 + kStages * kStageBytes;      // kStages stages
    static constexpr int kStats = kV1 + kStages * kStageBytes;   // m, l: 2 row tiles x 128 x 2 floats
    static constexpr int kBars = kStats + kNumRowTiles * kRowTile * 2 * 4;
    static constexpr int kNumBars = 4 * kStages + 14 * kNumRowTiles;
    static constexpr int kMisc = kBars + kNumBars * 8;           // tmem base, abort flag
    static constexpr int kScratch = kMisc + 16;                  // epilogue staging of one row tile: [128][16] floats
    static constexpr int kScratchBytes = kRowTile * 16 * 4;
    static_assert(kRowTile * 16 >= 4 * HD, "the staging buffer also holds 4 partial rows of HD floats");
    static constexpr int kTotal = kScratch + kScratchBytes;
    static constexpr int kAlloc = (kTotal + 1024 > 120 * 1024) ? kTotal + 1024 : 120 * 1024;   // > half an SM: one block per SM
    static_assert(kAlloc <= 227 * 1024, "more dynamic shared memory than a block can have");
};

// Unit -> (batch, head, first query, column range).
struct UnitGeom {
    int b, h, hk, i0;
    int col_start;     // first K1/V1 buffer row the unit needs
    int nsub;          // 64-column S sub-tiles (one TMA stage each)
    int last_width;    // width of the last sub-tile, multiple of 16
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
    g.nsub = (ncols + kSubTile - 1) / kSubTile;
    g.last_width = ((ncols - (g.nsub - 1) * kSubTile) + 15) & ~15;
    return g;
}

// exp2 on the FMA pipe: round to the nearest integer n by the magic-number add, a cubic for
// 2^f on f in [-0.5, 0.5] (near-minimax, relative error 7.5e-5, far below the bf16 rounding of P), n added into the
// exponent field.  The argument is clamped at -125 (the result is then 2^-125, nothing beside the
// row's largest term 2^0..2^8).  Two values at a time: the packed fp32 instructions.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    x.x = fmaxf(x.x, -125.f);
    x.y = fmaxf(x.y, -125.f);
    const float2 magic = make_float2(12582912.f, 12582912.f);
    const float2 xf = __fadd2_rn(x, magic);
    const float2 r = __fadd2_rn(xf, make_float2(-12582912.f, -12582912.f));
    const float2 f = __fadd2_rn(x, make_float2(-r.x, -r.y));
    float2 p = __ffma2_rn(make_float2(0.05517165f, 0.05517165f), f, make_float2(0.24261113f, 0.24261113f));
    p = __ffma2_rn(p, f, make_float2(0.69326097f, 0.69326097f));
    p = __ffma2_rn(p, f, make_float2(0.99992806f, 0.99992806f));
    return make_float2(__uint_as_float(__float_as_uint(p.x) + (__float_as_uint(xf.x) << 23)),
                       __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(xf.y) << 23)));
}

// BIAS = false: both biases are zero, every bias add folds away.  F16: the tensors are IEEE half instead of bf16
// (same kernels; only the element encoding and the MMA's operand format differ).
template <int HD, bool BIAS, bool F16 = false>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_tc_kernel(const __grid_constant__ FwdTcParams P, const __grid_constant__ CUtensorMap map_k1,
              const __grid_constant__ CUtensorMap map_v1, const __nv_bfloat16* __restrict__ q,
              const __nv_bfloat16* __restrict__ k2, const __nv_bfloat16* __restrict__ v2,
              __nv_bfloat16* __restrict__ o, float* __restrict__ lse) {
    using L = FwdSmem<HD>;
    using namespace ptx;
    using E = El<F16>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const KParams& p = P.k;
    const float k2_bias = BIAS ? p.k2_bias : 0.f, v2_bias = BIAS ? p.v2_bias : 0.f;

    uint64_t* bars = (uint64_t*)(smem + L::kBars);
    uint64_t* k1_full = bars;                       // [kStages] TMA landed
    uint64_t* k1_empty = bars + kStages;            //           both row tiles' S MMAs have read the stage
    uint64_t* v1_full = bars + 2 * kStages;
    uint64_t* v1_empty = bars + 3 * kStages;
    uint64_t* a_ready = bars + 4 * kStages;         // [kNumRowTiles] A tile formed (auxiliary group -> MMA warp)
    uint64_t* a_free = a_ready + kNumRowTiles;      //                the unit's last S MMAs have read it (MMA warp -> auxiliary group)
    uint64_t* o_ready = a_free + kNumRowTiles;      //                T final (MMA warp -> auxiliary group)
    uint64_t* t_free = o_ready + kNumRowTiles;      //                T read out (auxiliary group -> MMA warp)
    uint64_t* st_ready = t_free + kNumRowTiles;     //                m, l of the unit stored (softmax group -> auxiliary group)
    uint64_t* st_free = st_ready + kNumRowTiles;    //                m, l consumed (auxiliary group -> softmax group)
    uint64_t* s_ready = st_free + kNumRowTiles;     // [kNumRowTiles][2] S sub-tile in buffer b computed (MMA warp -> softmax group)
    uint64_t* p_ready = s_ready + 2 * kNumRowTiles; // [kNumRowTiles][2] P of buffer b stored (softmax group -> MMA warp)
    uint64_t* pv_done = p_ready + 2 * kNumRowTiles; // [kNumRowTiles] a P.V sub-tile has been accumulated (MMA warp -> softmax group)
    uint32_t* tmem_base_slot = (uint32_t*)(smem + L::kMisc);
    volatile int* abort_flag = (volatile int*)(smem + L::kMisc + 4);
    const WaitCtx wctx{abort_flag, P.status, P.wait_limit_ns};

    const int tid = threadIdx.x;
    SA_PROF_T0(t_life);
    SA_TR_DECL();
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&k1_full[s], 1);
            mbar_init(&k1_empty[s], kNumRowTiles);
            mbar_init(&v1_full[s], 1);
            mbar_init(&v1_empty[s], kNumRowTiles);
        }
        for (int r = 0; r < kNumRowTiles; ++r) {
            // barriers a 128-thread group arrives on count one (elected) arrival per warp
            mbar_init(&a_ready[r], 4);
            mbar_init(&a_free[r], 1);
            mbar_init(&o_ready[r], 1);
            mbar_init(&pv_done[r], 1);
            mbar_init(&t_free[r], 4);
            mbar_init(&st_ready[r], 4);
            mbar_init(&st_free[r], 4);
            for (int c = 0; c < 2; ++c) {
                mbar_init(&s_ready[2 * r + c], 1);
                mbar_init(&p_ready[2 * r + c], 4);
            }
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 12) {
        tmem_alloc(tmem_base_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    // S buffers: row tile r, buffer b at column (2r + b) * 64; T accumulators behind them
    const uint32_t tmem_t[2] = {tmem_base + 256, tmem_base + 256 + HD};

    const int DW = 1 << P.dw_log2;
    const int qpt = kRowTile >> P.dw_log2;          // queries per row tile
    // One arrival per warp: every lane has finished (and fenced) its own part, the warp converges, lane 0 arrives.
    auto warp_arrive = [&](uint64_t* bar) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
    };

    // Register pool of the block: what it was launched with, 512 x 128 >= 128 x (2 x softmax groups + auxiliary group
    // + MMA / TMA warps), at the register counts above.  Registers the launch left unused on the multiprocessor do NOT
    // belong to the block: an increase beyond the block's own pool never returns.
    static_assert(2 * 128 * SA_FWD_REGS_SM + 128 * SA_FWD_REGS_AUX + 128 * SA_FWD_REGS_REST <= kFwdThreads * 128, "register pool of the block");
    if (warp == 14) {
        // ------------------------------------------------------------------ TMA producer
        reg_dealloc<SA_FWD_REGS_REST>();
        if (lane == 0) {
            prefetch_tensormap(&map_k1);
            prefetch_tensormap(&map_v1);
            uint32_t g = 0;                           // running column-tile counter (ring position)
            for (long u = blockIdx.x; u < P.num_units; u += gridDim.x) {
                const UnitGeom ug = unit_geom(P, u);
                for (int t = 0; t < ug.nsub; ++t, ++g) {
                    const int s = g % kStages;
                    const uint32_t ph = (g / kStages) & 1;
                    const int row = ug.col_start + t * kSubTile;
                    mbar_wait(&k1_empty[s], ph ^ 1, wctx, 1);
                    mbar_arrive_expect_tx(&k1_full[s], L::kStageBytes);
#pragma unroll
                    for (int sl = 0; sl < L::kSlabs; ++sl)
                        tma_load_4d(smem + L::kK1 + s * L::kStageBytes + sl * L::kStageSlab, &map_k1, &k1_full[s], sl * 64,
                                    row, ug.hk, ug.b);
                    mbar_wait(&v1_empty[s], ph ^ 1, wctx, 2);
                    mbar_arrive_expect_tx(&v1_full[s], L::kStageBytes);
#pragma unroll
                    for (int sl = 0; sl < L::kSlabs; ++sl)
                        tma_load_4d(smem + L::kV1 + s * L::kStageBytes + sl * L::kStageSlab, &map_v1, &v1_full[s], sl * 64,
                                    row, ug.hk, ug.b);
                }
            }
        }
        __syncwarp();
    } else if (warp == 12 || warp == 13) {
        // ------------------------------------------------------------------ MMA issuer of row tile r
        reg_dealloc<SA_FWD_REGS_REST>();
        {
            const int r = warp - 12;
            const uint32_t leader = elect_one();      // the whole warp runs the loop; one lane issues
            const uint32_t idesc_pv = make_idesc(128, HD, false, true, F16);
            const uint32_t idesc_s_full = make_idesc(128, kSubTile, false, false, F16);
            const uint32_t a_addr = smem_base + L::kA + r * L::kTileBytes;
            const uint32_t tmem_sb = tmem_base + 2 * r * kSubTile;     // this row tile's two S buffers
            uint32_t g = 0;          // ring position of the unit's first stage
            uint32_t nu = 0;         // units done (phase of a_ready / o_ready / t_free)
            uint32_t gs = 0;         // sub-tiles before this unit: sub-tile s uses S buffer (gs + s) & 1
            UnitGeom ug = unit_geom(P, blockIdx.x < P.num_units ? blockIdx.x : 0);
            for (long u = blockIdx.x; u < P.num_units; u += gridDim.x, ++nu) {
                // S sub-tile sub = A . K1[64 rows]^T into buffer (gs + sub) & 1.  The buffer is free: the P.V MMAs
                // that read it (sub-tile sub - 2) were issued by this warp before, and the tensor cores run in order.
                auto issue_s = [&](int sub) {
                    const uint32_t gt = g + sub;
                    const int st = gt % kStages;
                    mbar_wait(&k1_full[st], (gt / kStages) & 1, wctx, 3);
                    tc_fence_after();
                    const int b = (gs + sub) & 1;
                    const uint32_t idesc_s = (sub == ug.nsub - 1) ? make_idesc(128, ug.last_width, false, false, F16) : idesc_s_full;
                    const uint64_t da = desc_kmajor(a_addr, 0);
                    const uint64_t db = desc_kmajor(smem_base + L::kK1 + st * L::kStageBytes, 0);
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk) {
                        const uint32_t offa = ((kk >> 2) * L::kSlabBytes + (kk & 3) * 32) >> 4;
                        const uint32_t offb = ((kk >> 2) * L::kStageSlab + (kk & 3) * 32) >> 4;
                        mma_ss(leader, tmem_sb + b * kSubTile, da + offa, db + offb, idesc_s, kk > 0);
                    }
                    tc_commit(leader, &s_ready[2 * r + b]);
                    tc_commit(leader, &k1_empty[st]);
                    if (sub == ug.nsub - 1) tc_commit(leader, &a_free[r]);                          // the A tile may be overwritten
                };
                SA_TR(r, 1);
                mbar_wait(&a_ready[r], nu & 1, wctx, 4);
                SA_TR(r, 2);
                tc_fence_after();
                issue_s(0);
                if (ug.nsub > 1) issue_s(1);
                SA_TR(r, 3);
                // the next unit's geometry, computed while the softmax group works on the first sub-tile
                const UnitGeom ug_next = unit_geom(P, u + gridDim.x < P.num_units ? u + gridDim.x : u);
                for (int sub = 0; sub < ug.nsub; ++sub) {
                    const uint32_t gt = g + sub;
                    const int st = gt % kStages;
                    const uint32_t n = gs + sub;                           // running sub-tile number of this row tile
                    const int b = n & 1;
                    const uint64_t db = desc_mnmajor(smem_base + L::kV1 + st * L::kStageBytes, L::kStageSlab);
                    const int ksteps = (sub != ug.nsub - 1) ? kSubTile / 16 : ug.last_width / 16;
                    SA_PROF_T0(t_pv);
                    mbar_wait(&p_ready[2 * r + b], (n >> 1) & 1, wctx, 5);
                    SA_TR(r, 20);
                    mbar_wait(&v1_full[st], (gt / kStages) & 1, wctx, 6);
                    // the previous unit's T has been read out by the auxiliary group
                    if (sub == 0 && nu > 0) mbar_wait(&t_free[r], (nu - 1) & 1, wctx, 10);
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < kSubTile / 16; ++kk)
                        if (kk < ksteps)
                            mma_ts(leader, tmem_t[r], tmem_sb + b * kSubTile + kk * 8, db + kk * (2048 >> 4), idesc_pv, sub > 0 || kk > 0);
                    tc_commit(leader, &pv_done[r]);
                    SA_PROF_ADD(30, t_pv);
                    SA_TR(r, 30);
                    tc_commit(leader, &v1_empty[st]);
                    if (sub + 2 < ug.nsub) {
                        SA_PROF_T0(t_s);
                        issue_s(sub + 2);
                        SA_PROF_ADD(31, t_s);
                        SA_TR(r, 40);
                    }
                    if (sub == ug.nsub - 1) tc_commit(leader, &o_ready[r]);
                }
                g += ug.nsub;
                gs += ug.nsub;
                ug = ug_next;
            }
        }
        __syncwarp();
    } else if (warp == 15) {
        reg_dealloc<SA_FWD_REGS_REST>();
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ auxiliary group: operand formation ahead of the
        // softmax groups, merge over delta and output behind them
        reg_alloc<SA_FWD_REGS_AUX>();
        const int row = tid & 127;                   // virtual row = tensor-memory lane
        const uint32_t lane_addr = ((uint32_t)(row & ~31)) << 16;
        const int qq = row >> P.dw_log2;
        const int delta = row & (DW - 1);
        float* scratch = (float*)(smem + L::kScratch);
        // Operand formation in two steps: the loads of a unit's Q and K2 rows are issued a whole unit ahead
        // (form_load, into registers), the products are written once the tile is free (form_store).  DWL is
        // the compile-time number of delta slots per query (log2) for 16, 32 and 64 slots, 0 for any other
        // count (those load when they store).
        auto aux_body = [&](auto dwl_c) {
        constexpr int DWL = decltype(dwl_c)::value;
        constexpr int kFormRegs = DWL != 0 ? ProductTileShape<HD, DWL != 0 ? DWL : 5>::NREGS : 1;
        uint4 fr0[kFormRegs], fr1[kFormRegs];
        // (written out rather than wrapped in lambdas: register arrays captured by reference end up in local memory)
#define SA_FWD_FORM_LOAD(UG)                                                                                              \
        if constexpr (DWL != 0) {                                                                                         \
            const __nv_bfloat16* xb_ = q + (UG).b * p.q.b + (UG).h * p.q.h;                                               \
            const __nv_bfloat16* yb_ = k2 + (UG).b * p.k2.b + (UG).hk * p.k2.h;                                           \
            load_product_tile_shared<HD, DWL>(fr0, row, (UG).i0, p.N, p.halo2, xb_, p.q.n, yb_, p.k2.n);                  \
            load_product_tile_shared<HD, DWL>(fr1, row, (UG).i0 + qpt, p.N, p.halo2, xb_, p.q.n, yb_, p.k2.n);            \
        }
#define SA_FWD_FORM_STORE(UG, R, FR)                                                                                      \
        {                                                                                                                 \
            SA_PROF_T0(t_form);                                                                                           \
            if (warp == 8) SA_TR(2, 50 + (R));                                                                            \
            uint8_t* tile_ = smem + L::kA + (R) * L::kTileBytes;                                                          \
            const int i0_ = (UG).i0 + (R) * qpt;                                                                          \
            if constexpr (DWL != 0) {                                                                                     \
                store_product_tile_shared<HD, DWL, BIAS, F16>(tile_, L::kSlabBytes, row, i0_, p.N, p.w2, p.halo2, FR, k2_bias); \
            } else {                                                                                                      \
                form_product_tile<HD, 128, 128, BIAS, F16>(tile_, L::kSlabBytes, row, (long)i0_ << P.dw_log2, P.dw_log2, p.N, p.w2, \
                                                      p.halo2, q + (UG).b * p.q.b + (UG).h * p.q.h, p.q.n,                \
                                                      k2 + (UG).b * p.k2.b + (UG).hk * p.k2.h, p.k2.n, k2_bias);          \
            }                                                                                                             \
            fence_proxy_async_smem();                                                                                     \
            warp_arrive(&a_ready[R]);                                                                                     \
            if (warp == 8) SA_TR(2, 52 + (R));                                                                            \
            SA_PROF_ADD(10 + (R), t_form);                                                                                \
        }
        uint32_t nu = 0;
        long u = blockIdx.x;
        if (u < P.num_units) {
            const UnitGeom ug = unit_geom(P, u);
            SA_FWD_FORM_LOAD(ug);
            SA_FWD_FORM_STORE(ug, 0, fr0);
            SA_FWD_FORM_STORE(ug, 1, fr1);
            const UnitGeom un = unit_geom(P, u + gridDim.x < P.num_units ? u + gridDim.x : u);
            SA_FWD_FORM_LOAD(un);
        }
        for (; u < P.num_units; u += gridDim.x, ++nu) {
            const UnitGeom ug = unit_geom(P, u);
            // ---- A tiles of the next unit, as soon as this unit's last S MMAs have read the current ones
            if (u + gridDim.x < P.num_units) {
                const UnitGeom un = unit_geom(P, u + gridDim.x);
                mbar_wait(&a_free[0], nu & 1, wctx, 11);
                SA_FWD_FORM_STORE(un, 0, fr0);
                mbar_wait(&a_free[1], nu & 1, wctx, 11);
                SA_FWD_FORM_STORE(un, 1, fr1);
            }
            // ---- epilogue of this unit: merge the delta rows of each query
            for (int r = 0; r < kNumRowTiles; ++r) {
                SA_PROF_T0(t_epi);
                const int i = ug.i0 + r * qpt + qq;
                const int kb = i + p.halo2 - delta;                    // K2/V2 buffer row
                const bool row_valid = (i < p.N) && (delta < p.w2) && (kb >= 0);
                const float* m_s = (const float*)(smem + L::kStats) + r * 2 * kRowTile;
                const float* l_s = m_s + kRowTile;
                const __nv_bfloat16* v2row = v2 + ug.b * p.v2.b + (long)max(kb, 0) * p.v2.n + ug.hk * p.v2.h;
                const uint32_t t_addr = tmem_t[r] + lane_addr;
                // this row's V2 values (first 32-column chunk), fetched while the last MMAs of the unit are still running
                uint32_t vw[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) vw[e] = 0u;
                if (row_valid) load_bf16_words<32>(v2row, vw);
                if (warp == 8) SA_TR(2, 60 + r);
                mbar_wait(&st_ready[r], nu & 1, wctx, 12);
                if (warp == 8) SA_TR(2, 62 + r);
                const float m = m_s[row], l = l_s[row];
                float mq, lq;
                if (P.dw_log2 <= 5) {
                    // the delta rows of a query are DW consecutive lanes of one warp: merge by register exchange
                    mq = m;
                    for (int sft = DW >> 1; sft >= 1; sft >>= 1) mq = fmaxf(mq, __shfl_xor_sync(0xffffffffu, mq, sft));
                    lq = (m > -INFINITY) ? ex2(m - mq) * l : 0.f;
                    for (int sft = DW >> 1; sft >= 1; sft >>= 1) lq += __shfl_xor_sync(0xffffffffu, lq, sft);
                } else {
                    mq = -INFINITY;
                    for (int d2 = 0; d2 < DW; ++d2) mq = fmaxf(mq, m_s[(qq << P.dw_log2) + d2]);
                    lq = 0.f;
                    for (int d2 = 0; d2 < DW; ++d2) {
                        const float mm = m_s[(qq << P.dw_log2) + d2];
                        if (mm > -INFINITY) lq += ex2(mm - mq) * l_s[(qq << P.dw_log2) + d2];
                    }
                }
                const float wrow = (m > -INFINITY) ? ex2(m - mq) / lq : 0.f;
                mbar_wait(&o_ready[r], nu & 1, wctx, 9);
                if (warp == 8) SA_TR(2, 64 + r);
                tc_fence_after();
                if constexpr (DWL == 4) {
                    // a warp holds the 16 deltas of two queries, one per half warp: sum them by a register exchange
                    // within each half, 16 columns at a time; lane L ends up with column (L % 16) of its half's query
                    uint32_t v[16], cur[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) cur[e] = vw[e];
                    tmem_ld16(t_addr, v);
                    __nv_bfloat16* orow = o + ug.b * p.o.b + (long)min(i, p.N - 1) * p.o.n + ug.h * p.o.h;
#pragma unroll
                    for (int ch = 0; ch < HD / 16; ++ch) {
                        uint32_t vn[8];                           // the next chunk's V2 values are in flight under this one's reduction
#pragma unroll
                        for (int e = 0; e < 8; ++e) vn[e] = 0u;
                        if (ch + 1 < HD / 16 && row_valid) load_bf16_words<16>(v2row + 16 * (ch + 1), vn);
                        tmem_wait_ld();
                        if (ch == HD / 16 - 1) {                  // T has been read: the next unit's first P.V may overwrite it
                            tc_fence_before();
                            warp_arrive(&t_free[r]);
                        }
                        float y[16];
#pragma unroll
                        for (int e = 0; e < 16; e += 2) {
                            const uint32_t w = cur[e >> 1];
                            float2 x2 = make_float2(E::lo(w), E::hi(w));
                            if (BIAS) x2 = __fadd2_rn(x2, make_float2(v2_bias, v2_bias));
                            const float2 y2 = __fmul2_rn(make_float2(__uint_as_float(v[e]), __uint_as_float(v[e + 1])),
                                                         __fmul2_rn(x2, make_float2(wrow, wrow)));
                            y[e] = y2.x;
                            y[e + 1] = y2.y;
                        }
                        if (ch + 1 < HD / 16) tmem_ld16(t_addr + 16 * (ch + 1), v);
                        const float tot = half_warp_transpose_reduce<16>(y, lane);
                        if (i < p.N) E::st(&orow[16 * ch + (lane & 15)], tot);
#pragma unroll
                        for (int e = 0; e < 8; ++e) cur[e] = vn[e];
                    }
                } else if (DWL >= 5 || P.dw_log2 >= 5) {
                    // a warp holds 32 consecutive deltas of one query: sum them by a register exchange;
                    // lane L ends up with column L of each 32-column chunk
                    const int wq = row >> 5;                      // warp within the group
                    const int wpq = DW >> 5;                      // warps per query
                    float* part = scratch;                        // [4 warps][HD] when a query spans several warps
                    float tot[HD / 32];
                    uint32_t v[32];                               // the next chunk's tensor-memory load is in flight under this one's reduction
                    tmem_ld32(t_addr, v);
#pragma unroll
                    for (int cch = 0; cch < HD / 32; ++cch) {
                        uint32_t vn[16];                          // ... and so are the next chunk's V2 values
#pragma unroll
                        for (int e = 0; e < 16; ++e) vn[e] = 0u;
                        if (cch + 1 < HD / 32 && row_valid) load_bf16_words<32>(v2row + 32 * (cch + 1), vn);
                        tmem_wait_ld();
                        if (cch == HD / 32 - 1) {                 // T has been read: the next unit's first P.V may overwrite it
                            tc_fence_before();
                            warp_arrive(&t_free[r]);
                        }
                        float y[32];
#pragma unroll
                        for (int e = 0; e < 32; e += 2) {
                            // rows that are not valid have T = 0 exactly (their P is 0) and wrow = 0: no select needed
                            const uint32_t w = vw[e >> 1];
                            float2 x2 = make_float2(E::lo(w), E::hi(w));
                            if (BIAS) x2 = __fadd2_rn(x2, make_float2(v2_bias, v2_bias));
                            const float2 y2 = __fmul2_rn(make_float2(__uint_as_float(v[e]), __uint_as_float(v[e + 1])),
                                                         __fmul2_rn(x2, make_float2(wrow, wrow)));
                            y[e] = y2.x;
                            y[e + 1] = y2.y;
                        }
                        if (cch + 1 < HD / 32) tmem_ld32(t_addr + 32 * (cch + 1), v);
                        tot[cch] = warp_transpose_reduce<32>(y, lane);
#pragma unroll
                        for (int e = 0; e < 16; ++e) vw[e] = vn[e];
                    }
                    if (wpq == 1) {
                        if (i < p.N) {
                            __nv_bfloat16* orow = o + ug.b * p.o.b + (long)i * p.o.n + ug.h * p.o.h;
#pragma unroll
                            for (int cch = 0; cch < HD / 32; ++cch) E::st(&orow[32 * cch + lane], tot[cch]);
                        }
                    } else {
#pragma unroll
                        for (int cch = 0; cch < HD / 32; ++cch) part[wq * HD + 32 * cch + lane] = tot[cch];
                        named_barrier_sync(1, kRowTile);
                        for (int idx = row; idx < qpt * HD; idx += kRowTile) {
                            const int q2 = idx / HD, col = idx % HD;
                            float acc = 0.f;
                            for (int w2i = 0; w2i < wpq; ++w2i) acc += part[(q2 * wpq + w2i) * HD + col];
                            const int i2 = ug.i0 + r * qpt + q2;
                            if (i2 < p.N) E::st(&o[ug.b * p.o.b + (long)i2 * p.o.n + ug.h * p.o.h + col], acc);
                        }
                        named_barrier_sync(1, kRowTile);
                    }
                } else {
                    // several queries per warp: 16 columns at a time through the staging buffer
                    for (int c0 = 0; c0 < HD; c0 += 16) {
                        uint32_t v[16];
                        tmem_ld16(t_addr + c0, v);
                        tmem_wait_ld();
                        if (c0 + 16 >= HD) {
                            tc_fence_before();
                            warp_arrive(&t_free[r]);
                        }
                        uint32_t vw16[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) vw16[e] = 0u;
                        if (row_valid) load_bf16_words<16>(v2row + c0, vw16);
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const float vf = (e & 1) ? E::hi(vw16[e >> 1]) : E::lo(vw16[e >> 1]);
                            const float val = row_valid ? __uint_as_float(v[e]) * wrow * (vf + v2_bias) : 0.f;
                            scratch[row * 16 + (e ^ (row & 15))] = val;
                        }
                        named_barrier_sync(1, kRowTile);
                        for (int idx = row; idx < qpt * 16; idx += kRowTile) {
                            const int q2 = idx >> 4, e = idx & 15;
                            const int i2 = ug.i0 + r * qpt + q2;
                            float acc = 0.f;
                            for (int d2 = 0; d2 < DW; ++d2) {
                                const int rr = (q2 << P.dw_log2) + d2;
                                acc += scratch[rr * 16 + (e ^ (rr & 15))];
                            }
                            if (i2 < p.N) E::st(&o[ug.b * p.o.b + (long)i2 * p.o.n + ug.h * p.o.h + c0 + e], acc);
                        }
                        named_barrier_sync(1, kRowTile);
                    }
                }
                if (delta == 0 && i < p.N) lse[((long)ug.b * p.H + ug.h) * p.N + i] = (mq + log2f(lq)) * kLn2;
                warp_arrive(&st_free[r]);             // m, l of this unit are no longer needed
                if (warp == 8) SA_TR(2, 66 + r);
                SA_PROF_ADD(14 + r, t_epi);
            }
            // ---- start the loads of the unit after next.  Unconditional (past the end: this unit's rows once
            // more, never used), so that the registers are defined on every path and do not stay live across
            // the epilogue above.
            {
                const long u2 = u + 2 * (long)gridDim.x;
                const UnitGeom un2 = unit_geom(P, u2 < P.num_units ? u2 : u);
                SA_FWD_FORM_LOAD(un2);
            }
        }
#undef SA_FWD_FORM_LOAD
#undef SA_FWD_FORM_STORE
        };      // aux_body
        switch (P.dw_log2) {
            case 4: aux_body(std::integral_constant<int, 4>{}); break;
            case 5: aux_body(std::integral_constant<int, 5>{}); break;
            case 6: aux_body(std::integral_constant<int, 6>{}); break;
            default: aux_body(std::integral_constant<int, 0>{});
        }
    } else {
        // ------------------------------------------------------------------ softmax groups
        reg_alloc<SA_FWD_REGS_SM>();
        const int r = warp >> 2;                     // row tile of this group
        const int row = tid & 127;                   // virtual row = tensor-memory lane
        const uint32_t lane_addr = ((uint32_t)(row & ~31)) << 16;
        const int qq = row >> P.dw_log2;
        const int delta = row & (DW - 1);
        float* m_s = (float*)(smem + L::kStats) + r * 2 * kRowTile;
        float* l_s = m_s + kRowTile;
        const float c2 = p.scale * kLog2e;
        const uint32_t tmem_sb = tmem_base + 2 * r * kSubTile + lane_addr;     // this row tile's two S buffers, this warp's lanes
        uint32_t nu = 0, gs = 0;                     // units done; sub-tiles before this unit
        for (long u = blockIdx.x; u < P.num_units; u += gridDim.x, ++nu) {
            const UnitGeom ug = unit_geom(P, u);
            const int i = ug.i0 + r * qpt + qq;
            const int kb = i + p.halo2 - delta;                    // K2/V2 buffer row
            const bool row_valid = (i < p.N) && (delta < p.w2) && (kb >= 0);
            SA_PROF_T0(t_loop);
            // ---- main loop over 64-column sub-tiles
            // Valid buffer rows of this virtual row: [jlo, jhi] (empty for an invalid row).
            const int jhi = row_valid ? i + p.halo1 : -1;
            const int jlo = row_valid ? max(0, i + p.halo1 - p.w1 + 1) : 0;
            float m = -INFINITY, l = 0.f;
            for (int sub = 0; sub < ug.nsub; ++sub) {
                const uint32_t n = gs + sub;
                const int b = n & 1;
                const int width = (sub == ug.nsub - 1) ? ug.last_width : kSubTile;
                const int tile0 = ug.col_start + sub * kSubTile;
                const int lo = jlo - tile0, hi = jhi - tile0;        // valid tile-relative columns [lo, hi]
                mbar_wait(&s_ready[2 * r + b], (n >> 1) & 1, wctx, 8);
                SA_TR(3 + warp, 70);
                tc_fence_after();
                SA_PROF_T0(t_sm);
                const uint32_t s_addr = tmem_sb + b * kSubTile;
                // Running maximum, lazily updated.  When it moves, T and l are scaled down; T is being
                // accumulated into by the P.V MMAs of the previous sub-tile, which must have finished first.
                auto update_max = [&](float tmax) {
                    float factor = 1.f;
                    bool rescale = false;
                    if (tmax > m + kRescaleThreshold || (m == -INFINITY && tmax > -INFINITY)) {
                        rescale = (m != -INFINITY);
                        factor = rescale ? ex2(m - tmax) : 1.f;
                        m = tmax;
                    }
                    if (__any_sync(0xffffffffu, rescale)) {
                        // n P.V commits precede this sub-tile; at least n - 1 are known complete (S of this sub-tile was
                        // issued after them): wait for the n-th
                        if (n > 0) mbar_wait(&pv_done[r], (n - 1) & 1, wctx, 14);
                        tc_fence_after();
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
                // a sub-tile is "full" when every column is inside every row's window: no masks needed
                const bool full = (width == kSubTile) && __all_sync(0xffffffffu, lo <= 0 && hi >= kSubTile - 1);
                // or nearly: only the first few columns lie before the window of some rows (a unit's first sub-tile)
                const bool head_masked = !full && (width == kSubTile) && __all_sync(0xffffffffu, lo <= 16 && hi >= kSubTile - 1);
                float lsum = 0.f;
                if (full || head_masked) {
                    // the whole sub-tile in registers: one pass over tensor memory
                    uint32_t v0[32], v1[32];
                    tmem_ld32(s_addr, v0);
                    tmem_ld32(s_addr + 32, v1);
                    tmem_wait_ld();
                    if (head_masked) {
                        // scores before a row's window become a large negative number: their P is exactly 0 (or 2^-125)
#pragma unroll
                        for (int e = 0; e < 16; ++e) v0[e] = (e < lo) ? __float_as_uint(-1e30f) : v0[e];
                    }
                    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
                            mx[x] = max3(mx[x], __uint_as_float(v0[e + x]), __uint_as_float(v0[e + 4 + x]));
                            mx[x] = max3(mx[x], __uint_as_float(v1[e + x]), __uint_as_float(v1[e + 4 + x]));
                        }
                    }
                    SA_PROF_ADD(20 + r, t_sm);
                    SA_TR(3 + warp, 71);
                    SA_PROF_T0(t_p2);
                    update_max(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * c2);
                    // packed two-wide fp32 arithmetic: one FMA and one add per pair of columns
                    float2 ls = make_float2(0.f, 0.f);
                    const float2 c2v = make_float2(c2, c2), nm = make_float2(-m, -m);
                    uint32_t pk[32];
#pragma unroll
                    for (int e = 0; e < 64; e += 2) {
                        const uint32_t s0 = e < 32 ? v0[e] : v1[e - 32], s1 = e < 32 ? v0[e + 1] : v1[e - 31];
                        const float2 x = __ffma2_rn(make_float2(__uint_as_float(s0), __uint_as_float(s1)), c2v, nm);
                        // The special-function unit and the FMA pipe share the exponentials: SA_FWD_POLY_OF_8 of every eight
                        // column pairs take the polynomial.
                        const float2 pr = ((e >> 1) & 7) < SA_FWD_POLY_OF_8 ? exp2_poly2(x) : make_float2(ex2(x.x), ex2(x.y));
                        ls = __fadd2_rn(ls, pr);
                        pk[e >> 1] = E::pack(pr.x, pr.y);
                    }
                    // P (32 packed columns) overwrites the first half of the S buffer
                    tmem_st32(s_addr, pk);
                    tmem_wait_st();
                    tc_fence_before();
                    warp_arrive(&p_ready[2 * r + b]);
                    SA_TR(3 + warp, 72);
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
                            pk[e >> 1] = E::pack(p0, p1);
                        }
                        tmem_st16(s_addr + (c0 >> 1), pk);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    warp_arrive(&p_ready[2 * r + b]);
                    SA_PROF_ADD((sub == 0 ? 24 : 26) + r, t_sm);
                }
                l += lsum;
                SA_PROF_ADD(16 + r, t_sm);
            }
            SA_PROF_ADD(12 + r, t_loop);
            // ---- hand the row statistics to the auxiliary group (once it has consumed the previous unit's)
            if (nu > 0) mbar_wait(&st_free[r], (nu - 1) & 1, wctx, 13);
            m_s[row] = m;
            l_s[row] = l;
            warp_arrive(&st_ready[r]);
            SA_TR(3 + warp, 74);
            gs += ug.nsub;
        }
    }
    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    SA_PROF_LIFE(t_life);
    if (warp == 12) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace tc
}  // namespace sa
