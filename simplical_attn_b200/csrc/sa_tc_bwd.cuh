// Backward 2-simplicial attention on the sm_100a tensor cores.  Replaces the reference's
// compute_D_kernel, two_simplicial_attn_bwd_kv1_kernel and two_simplicial_attn_bwd_kv2_kernel
// (simplicial/kernels.py:569-571, :175-382, :386-566) without atomics.
//
// Virtual rows as in the forward: rho = i * DW + delta (DW = w2 rounded up to a power of two),
// k = i - delta,  A[rho,:] = Q_i * (K2_k + k2_bias),  C[rho,:] = dO_i * (V2_k + v2_bias).  With
//   S = A K1^T,  P = exp2(S*scale*log2e - LSE2_i),  dP = C V1^T,  dS = P * (dP - Delta_i)
// the gradients are
//   dV1 = P^T C          dK1 = scale * dS^T A                              ("column" kernel)
//   G = dS K1,  U = P V1                                                   ("row" kernel)
//   dQ_i = scale * sum_delta G[rho] * (K2_k + bias)
//   dK2_k = scale * sum_i G[(i, i-k)] * Q_i        dV2_k = sum_i U[(i, i-k)] * dO_i
//
// Three launches plus a tiny one:
//   1. prep_kernel      Delta_i = dO_i . O_i and LSE2_i = LSE_i * log2e                (fp32)
//   2. bwd_col_kernel   a block owns 128 K1/V1 rows of one KV head, streams 128-row tiles of A and C
//                       (formed on chip by two producer warpgroups) for every query head of the
//                       group, accumulates dV1 and dK1 in tensor memory and writes them once.
//   3. bwd_row_kernel / bwd_row2_kernel
//                       a block owns a run of consecutive queries of one query head; per 128-row
//                       tile it streams 64-row K1/V1 tiles by TMA, accumulates U and G in tensor
//                       memory, merges G over delta into dQ and adds the per-K2-row sums of G*Q and
//                       U*dO into fp32 partial buffers in the workspace (plain read-modify-write:
//                       a row is only ever touched by one block, in program order).  The second
//                       form (16, 32 or 64 delta slots per query, D = 128) has separate warpgroups that
//                       form the operands and run the epilogue, see there.
//   4. kv2_reduce_kernel sums those partials over the query heads of a group and over run
//                       boundaries and writes dK2, dV2.
//
// Row kernels: S and dP tiles (128 lanes x 64 columns) are double buffered in tensor memory; the softmax
// groups turn a buffer into P and dS (16-bit, in place) while the tensor cores work on the other buffer
// (bwd_row_kernel: one group per buffer; bwd_row2_kernel: both groups split every tile's columns); P and dS
// then feed the two accumulating MMAs from tensor memory.  Column kernel: one 128-column S^T / dP^T pair,
// both softmax groups split its columns and hand P^T / dS^T to the MMA warp in 16-column chunks.
#pragma once

#include <type_traits>

#include "sa_ptx.cuh"

namespace sa {
namespace tc {

constexpr int kColThreads = 640;      // column kernel: 2 softmax groups, 2 producer groups, MMA warp (16), TMA warp (17), 2 idle
constexpr int kRowThreads = 384;      // row kernel: 2 softmax groups, MMA warp (8), TMA warp (9), 2 idle warps
constexpr int kStreamRows = 64;        // rows of a streamed tile = columns of an S / dP tile
constexpr int kColTileRows = 128;      // column kernel: virtual rows per streamed tile (columns of S^T)
constexpr int kColStages = 2;          // ... and its ring depth
constexpr int kRowStages = 3;          // ... of the row kernel (its dK2/dV2 ring needs the room)

struct BwdTcParams {
    KParams k;
    int dw_log2;
    // column kernel
    int num_jtiles;          // ceil(n1 / 128)
    long num_col_items;      // B * Hkv * num_jtiles
    // row kernel
    int units_per_run;       // 128-row tiles per run
    int num_runs;            // runs per (b, h)
    long num_row_items;      // B * H * num_runs
    const float* lse2;       // [B,H,N]
    const float* delta;      // [B,H,N]
    float* ws_full_k2;       // [B,H,N,D]   fp32 partial dK2 of rows k = i + halo2
    float* ws_full_v2;
    float* ws_head_k2;       // [B,H,num_runs,w2-1,D]  partials for the rows just before a run
    float* ws_head_v2;
    DeviceStatus* status;
    uint64_t wait_limit_ns;  // bound of every device-side wait
};

template <int HD, int NS = kRowStages>
struct BwdSmem {
    static constexpr int kSlabs = HD / 64;
    static constexpr int kBigTile = 128 * HD * 2;            // stationary tile  [128 x HD]
    static constexpr int kBigSlab = 128 * 128;
    static constexpr int kSmallTile = kStreamRows * HD * 2;  // streamed tile    [64 x HD]
    static constexpr int kSmallSlab = kStreamRows * 128;
    static constexpr int kStat0 = 0;                         // K1 (column kernel) / A (row kernel)
    static constexpr int kStat1 = kBigTile;                  // V1 / C
    static constexpr int kStream = 2 * kBigTile;             // NS x (tile0 | tile1)
    static constexpr int kMeta = kStream + NS * 2 * kSmallTile;   // per stage: 64 lse2 + 64 delta
    static constexpr int kBars = kMeta + NS * 128 * 4;
    static constexpr int kNumBars = 2 * NS + 14;
    static constexpr int kMisc = kBars + kNumBars * 8;
    static constexpr int kTotal = kMisc + 16;
    static constexpr int kRing = kTotal;                     // row kernel: 2 x ring_rows x HD floats (optional)
    static constexpr int kAlloc = (kTotal + 1024 > 120 * 1024) ? kTotal + 1024 : 120 * 1024;
    static constexpr int kMaxDynamic = 227 * 1024;
};

// ------------------------------------------------------------------------------------------------
// 1. Delta and LSE2
// ------------------------------------------------------------------------------------------------
template <bool F16>
__global__ void __launch_bounds__(128)
prep_kernel(KParams p, const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
            const float* __restrict__ lse, float* __restrict__ lse2, float* __restrict__ delta) {
    const long row = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= (long)p.B * p.H * p.N) return;
    const int i = (int)(row % p.N);
    const int h = (int)((row / p.N) % p.H);
    const int b = (int)(row / p.N / p.H);
    const __nv_bfloat16* orow = o + b * p.o.b + (long)i * p.o.n + h * p.o.h;
    const __nv_bfloat16* drow = d_o + b * p.d_o.b + (long)i * p.d_o.n + h * p.d_o.h;
    float s = 0.f;
    for (int d = lane * 2; d < p.D; d += 64) {
        const float2 a = ptx::El<F16>::ld2(orow + d);
        const float2 c = ptx::El<F16>::ld2(drow + d);
        s = fmaf(a.x, c.x, s);
        s = fmaf(a.y, c.y, s);
    }
    s = warp_sum(s);
    if (lane == 0) {
        delta[row] = s;
        lse2[row] = lse[row] * kLog2e;
    }
}

// P = mask ? exp2(s*c2 - lse2) : 0 and dS = P * (dp - delta) for W columns, packed to bf16.
// MASKED selects per-column validity through lo/hi (tile-relative valid column range).
template <bool MASKED, int W = 32, bool F16 = false>
__device__ __forceinline__ void softmax_bwd_chunk(const uint32_t (&s)[W], const uint32_t (&dp)[W], int c0, int lo, int hi,
                                                  float c2, float lse2, float delta, uint32_t (&pp)[W / 2], uint32_t (&ds)[W / 2]) {
    // packed two-wide fp32 arithmetic (one instruction per pair of columns)
    const float2 c2v = make_float2(c2, c2), nl = make_float2(-lse2, -lse2), nd = make_float2(-delta, -delta);
#pragma unroll
    for (int e = 0; e < W; e += 2) {
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), c2v, nl);
        float2 pr = make_float2(ptx::ex2(x.x), ptx::ex2(x.y));
        if (MASKED) {
            const int c = c0 + e;
            pr.x = (c >= lo && c <= hi) ? pr.x : 0.f;
            pr.y = (c + 1 >= lo && c + 1 <= hi) ? pr.y : 0.f;
        }
        float2 d = __fmul2_rn(pr, __fadd2_rn(make_float2(__uint_as_float(dp[e]), __uint_as_float(dp[e + 1])), nd));
        if (MASKED) {      // a masked column may hold stale tensor-memory contents (NaN): select, never multiply
            const int c = c0 + e;
            d.x = (c >= lo && c <= hi) ? d.x : 0.f;
            d.y = (c + 1 >= lo && c + 1 <= hi) ? d.y : 0.f;
        }
        pp[e >> 1] = ptx::El<F16>::pack(pr.x, pr.y);
        ds[e >> 1] = ptx::El<F16>::pack(d.x, d.y);
    }
}

// ------------------------------------------------------------------------------------------------
// 2. Column kernel: dK1, dV1
// ------------------------------------------------------------------------------------------------
struct ColItem {
    int b, hk, j0;        // first K1/V1 buffer row of the block's 128-row tile
    int tt_lo, ntq;       // first streamed tile (128 virtual rows each) and tiles per query head
};

__device__ __forceinline__ ColItem col_item(const BwdTcParams& P, long it) {
    const KParams& p = P.k;
    ColItem c;
    const int jt = (int)(it % P.num_jtiles);
    const long bh = it / P.num_jtiles;
    c.hk = (int)(bh % p.Hkv);
    c.b = (int)(bh / p.Hkv);
    c.j0 = jt * 128;
    // queries whose K1 window meets rows [j0, j0+128)
    const int i_lo = max(0, c.j0 - p.halo1);
    const int i_hi = min(p.N - 1, c.j0 + 127 - p.halo1 + p.w1 - 1);
    if (i_hi < i_lo) {
        c.tt_lo = 0;
        c.ntq = 0;
    } else {
        const long r_lo = (long)i_lo << P.dw_log2, r_hi = ((long)(i_hi + 1) << P.dw_log2);   // [r_lo, r_hi)
        c.tt_lo = (int)(r_lo / kColTileRows);
        c.ntq = (int)((r_hi + kColTileRows - 1) / kColTileRows) - c.tt_lo;
    }
    return c;
}


// Barrier block shared by the two big kernels.
struct BwdBars {
    uint64_t* st_full;     // [stages] streamed tile ready
    uint64_t* st_empty;    // [stages] streamed tile consumed (tcgen05.commit)
    uint64_t* sdp_ready;   // [2] S and dP of buffer b computed (commit)
    uint64_t* pds_ready;   // [2] P and dS of buffer b stored (128 arrivals)
    uint64_t* stat_full;   // stationary tiles ready
    uint64_t* stat_empty;  // stationary tiles no longer read (commit)
    uint64_t* acc_ready;   // accumulators final (commit)
    uint64_t* acc_free;    // accumulators read out (256 arrivals)
};

template <int NS>
__device__ __forceinline__ BwdBars bwd_bars(uint64_t* b) {
    return BwdBars{b, b + NS, b + 2 * NS, b + 2 * NS + 2, b + 2 * NS + 4, b + 2 * NS + 5, b + 2 * NS + 6, b + 2 * NS + 7};
}

// The MMAs of one streamed tile.  `X`, `Y`: stationary tiles [128 x HD]; `W`, `Z`: streamed tiles
// [64 x HD] of which the first `width` rows count.
//   S_b  = X W^T,   dP_b = Y Z^T              (issue_sdp)
//   acc1 += P_b Z,  acc2 += dS_b W            (issue_acc; P_b, dS_b read from tensor memory)
// The issuing thread is a single lane, so every integer instruction between two MMAs delays the
// tensor pipe: descriptors are built once per tile from the tile's address and only advanced by
// constants (a descriptor's low bits hold the address in 16-byte units, and no operand here ends
// beyond 256 KiB, so adding to the 64-bit value never carries out of the address field).
template <int HD>
__device__ __forceinline__ void issue_sdp(uint32_t leader, uint32_t tm_s, uint32_t tm_dp, uint32_t x, uint32_t y, uint32_t w, uint32_t z,
                                          uint32_t idesc) {
    using L = BwdSmem<HD>;
    const uint64_t dx = ptx::desc_kmajor(x, 0), dy = ptx::desc_kmajor(y, 0);
    const uint64_t dw = ptx::desc_kmajor(w, 0), dz = ptx::desc_kmajor(z, 0);
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk)
        ptx::mma_ss(leader, tm_s, dx + (((kk >> 2) * L::kBigSlab + (kk & 3) * 32) >> 4),
                    dw + (((kk >> 2) * L::kSmallSlab + (kk & 3) * 32) >> 4), idesc, kk > 0);
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk)
        ptx::mma_ss(leader, tm_dp, dy + (((kk >> 2) * L::kBigSlab + (kk & 3) * 32) >> 4),
                    dz + (((kk >> 2) * L::kSmallSlab + (kk & 3) * 32) >> 4), idesc, kk > 0);
}

// SPLIT: P and dS of a tile were written by two groups, each into the first 16 columns of its own 32-column half
// of the buffer (k-steps 0, 1 at columns 0..15, k-steps 2, 3 at columns 32..47); otherwise packed at columns 0..31.
template <int HD, bool SPLIT = false, bool F16 = false>
__device__ __forceinline__ void issue_acc(uint32_t leader, uint32_t tm_acc1, uint32_t tm_acc2, uint32_t tm_p, uint32_t tm_ds, uint32_t w,
                                          uint32_t z, int ksteps, bool accumulate) {
    using L = BwdSmem<HD>;
    const uint32_t idesc = ptx::make_idesc(128, HD, false, true, F16);
    const uint64_t dw = ptx::desc_mnmajor(w, L::kSmallSlab), dz = ptx::desc_mnmajor(z, L::kSmallSlab);
    auto col = [](int kk) { return SPLIT ? (kk >> 1) * 32 + (kk & 1) * 8 : kk * 8; };
    if (ksteps == kStreamRows / 16) {
#pragma unroll
        for (int kk = 0; kk < kStreamRows / 16; ++kk)
            ptx::mma_ts(leader, tm_acc1, tm_p + col(kk), dz + kk * (2048 >> 4), idesc, accumulate || kk > 0);
#pragma unroll
        for (int kk = 0; kk < kStreamRows / 16; ++kk)
            ptx::mma_ts(leader, tm_acc2, tm_ds + col(kk), dw + kk * (2048 >> 4), idesc, accumulate || kk > 0);
    } else {
        for (int kk = 0; kk < ksteps; ++kk)
            ptx::mma_ts(leader, tm_acc1, tm_p + col(kk), dz + kk * (2048 >> 4), idesc, accumulate || kk > 0);
        for (int kk = 0; kk < ksteps; ++kk)
            ptx::mma_ts(leader, tm_acc2, tm_ds + col(kk), dw + kk * (2048 >> 4), idesc, accumulate || kk > 0);
    }
}

// Shared-memory plan of the column kernel: the block's K1 and V1 rows, then kColStages pairs of
// streamed tiles (A | C, 128 virtual rows each), per-stage LSE2 / Delta of the tile's queries.
template <int HD>
struct ColSmem {
    static constexpr int kSlabs = HD / 64;
    static constexpr int kTile = 128 * HD * 2;
    static constexpr int kSlab = 128 * 128;
    static constexpr int kK1 = 0;
    static constexpr int kV1 = kTile;
    static constexpr int kStream = 2 * kTile;
    static constexpr int kMeta = kStream + kColStages * 2 * kTile;
    static constexpr int kBars = kMeta + kColStages * 256 * 4;
    static constexpr int kNumBars = 2 * kColStages + 10;
    static constexpr int kMisc = kBars + kNumBars * 8;
    static constexpr int kTotal = kMisc + 16;
    static constexpr int kAlloc = (kTotal + 1024 > 120 * 1024) ? kTotal + 1024 : 120 * 1024;
};

// One streamed tile covers 128 virtual rows, so S^T and dP^T are single 128x128 tiles: the MMAs run
// with N = 128 (a 128x64 tile costs almost as much: the 128-row stationary operand is re-read from
// shared memory either way) and in long bursts.  S^T / dP^T are not double buffered (tensor memory
// is full: 128 + 128 + 2 x 128 accumulator columns); instead both softmax groups work on the same
// tile, group g on columns [64g, 64g + 64), and write P / dS back inside their own column range.
// Registers per thread of the column kernel's softmax groups, producers and remaining warps (multiples of 8).
#ifndef SA_COL_SM
#define SA_COL_SM 96
#define SA_COL_PR 112
#define SA_COL_REST 64
#endif
static_assert(128 * (2 * SA_COL_SM + 2 * SA_COL_PR + SA_COL_REST) <= 640 * 96 && SA_COL_SM >= 96 && SA_COL_PR >= 96,
              "register pool of the column kernel's block");
template <int HD, bool BIAS, bool F16 = false>
__global__ void __launch_bounds__(kColThreads, 1)
bwd_col_kernel(const __grid_constant__ BwdTcParams P, const __grid_constant__ CUtensorMap map_k1,
               const __grid_constant__ CUtensorMap map_v1, const __nv_bfloat16* __restrict__ q,
               const __nv_bfloat16* __restrict__ k2, const __nv_bfloat16* __restrict__ v2,
               const __nv_bfloat16* __restrict__ d_o, __nv_bfloat16* __restrict__ dk1, __nv_bfloat16* __restrict__ dv1) {
    using L = ColSmem<HD>;
    using namespace ptx;
    using E = El<F16>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const KParams& p = P.k;
    uint64_t* bars = (uint64_t*)(smem + L::kBars);
    uint64_t* st_full = bars;                         // [kColStages] A and C of a tile formed (256 arrivals)
    uint64_t* st_empty = bars + kColStages;           // [kColStages] tile consumed (commit)
    uint64_t* sdp_ready = bars + 2 * kColStages;      // S^T, dP^T computed (commit)
    uint64_t* pds_ready = sdp_ready + 6;              // [4] P^T, dS^T of the k-th 16-column chunk of both groups stored (256 arrivals)
    uint64_t* stat_full = sdp_ready + 2;              // K1, V1 landed (TMA)
    uint64_t* stat_empty = sdp_ready + 3;             // K1, V1 no longer read (commit)
    uint64_t* acc_ready = sdp_ready + 4;              // dV1, dK1 final (commit)
    uint64_t* acc_free = sdp_ready + 5;               // dV1, dK1 read out (256 arrivals)
    uint32_t* tmem_slot = (uint32_t*)(smem + L::kMisc);
    volatile int* abort_flag = (volatile int*)(smem + L::kMisc + 4);
    const WaitCtx wctx{abort_flag, P.status, P.wait_limit_ns};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    SA_PROF_T0(t_life);
    SA_TR_DECL();
    if (tid == 0) {
        for (int s = 0; s < kColStages; ++s) {
            mbar_init(&st_full[s], 8);         // one arrival per producer warp
            mbar_init(&st_empty[s], 1);
        }
        mbar_init(sdp_ready, 1);
        for (int k = 0; k < 4; ++k) mbar_init(&pds_ready[k], 8);      // one arrival per softmax warp
        mbar_init(stat_full, 1);
        mbar_init(stat_empty, 1);
        mbar_init(acc_ready, 1);
        mbar_init(acc_free, 8);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 16) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dv1 = tmem_base + 256, tm_dk1 = tmem_base + 384;
    auto warp_arrive = [&](uint64_t* bar) {      // every lane has finished and fenced its part; lane 0 arrives for the warp
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
    };

    if (warp < 8) {
        // ---------------------------------------------------------------- softmax groups + epilogue
        // Register pool of the block: 640 x 96 = 128 x (2 x softmax groups + 2 x producers + MMA / TMA group) at the
        // counts SA_COL_*: an increase beyond the block's own pool would never return.
        reg_alloc<SA_COL_SM>();
        const int grp = warp >> 2;
        const int row = tid & 127;                       // tensor-memory lane = K1/V1 row of the block's tile
        const uint32_t lane_addr = ((uint32_t)(row & ~31)) << 16;
        const float c2 = p.scale * kLog2e;
        uint32_t n_items = 0, g_base = 0;
        for (long it = blockIdx.x; it < P.num_col_items; it += gridDim.x) {
            const ColItem ci = col_item(P, it);
            const int jb = ci.j0 + row;
            const int nt = ci.ntq * p.G;
            for (int t = 0; t < nt; ++t) {
                const uint32_t g = g_base + t;
                const int stage = (int)(g % kColStages);
                const float* m_lse = (const float*)(smem + L::kMeta) + stage * 256;
                const float* m_delta = m_lse + 128;
                const long rho0 = (long)(ci.tt_lo + (t % ci.ntq)) * kColTileRows;
                const int iq0 = (int)(rho0 >> P.dw_log2);
                mbar_wait(sdp_ready, g & 1, wctx, 20);
                if ((warp & 3) == 0) SA_TR(1 + grp, 52);
                tc_fence_after();
                SA_PROF_T0(t_csm);
                if (P.dw_log2 >= 4) {
                    // 16 columns (virtual rows) at a time, each chunk within one query; the next chunk's
                    // tensor-memory loads are in flight while the current one is processed.  A step whose
                    // columns all lie inside the window of every row of the warp needs no masks.
                    const int i_first = (int)((rho0 + 64 * grp) >> P.dw_log2), i_last = (int)((rho0 + 64 * grp + 63) >> P.dw_log2);
                    const bool step_full = __all_sync(0xffffffffu, jb <= i_first + p.halo1 && jb >= i_last + p.halo1 - p.w1 + 1);
                    auto run_step = [&](auto masked_tag) {
                        constexpr bool MASKED = decltype(masked_tag)::value;
                        uint32_t s[2][16], dp[2][16];
                        tmem_ld16(tm_s + lane_addr + 64 * grp, s[0]);
                        tmem_ld16(tm_dp + lane_addr + 64 * grp, dp[0]);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int c0 = 64 * grp + 16 * k;
                            tmem_wait_ld();
                            if (k + 1 < 4) {
                                tmem_ld16(tm_s + lane_addr + c0 + 16, s[(k + 1) & 1]);
                                tmem_ld16(tm_dp + lane_addr + c0 + 16, dp[(k + 1) & 1]);
                            }
                            const int i = (int)((rho0 + c0) >> P.dw_log2);
                            const bool valid = !MASKED || ((jb <= i + p.halo1) && (jb >= i + p.halo1 - p.w1 + 1));
                            uint32_t pp[8], ds[8];
                            softmax_bwd_chunk<MASKED, 16, F16>(s[k & 1], dp[k & 1], 0, valid ? 0 : 1, valid ? 15 : 0, c2, m_lse[i - iq0],
                                                          m_delta[i - iq0], pp, ds);
                            // packed P^T / dS^T of columns [64g + 16k, +16) go to tensor-memory columns 64g + 8k ...
                            tmem_st8(tm_s + lane_addr + 64 * grp + 8 * k, pp);
                            tmem_st8(tm_dp + lane_addr + 64 * grp + 8 * k, ds);
                            // the accumulating MMAs of this chunk start while the next one is processed
                            tmem_wait_st();
                            tc_fence_before();
                            warp_arrive(&pds_ready[k]);
                        }
                    };
                    if (step_full) run_step(std::false_type{});
                    else run_step(std::true_type{});
                } else {
#pragma unroll 1
                    for (int cc = 0; cc < 64; cc += 16) {
                        const int c0 = 64 * grp + cc;
                        uint32_t s[16], dp[16], pp[8], ds[8];
                        tmem_ld16(tm_s + lane_addr + c0, s);
                        tmem_ld16(tm_dp + lane_addr + c0, dp);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 16; e += 2) {
                            float pv[2], dv[2];
#pragma unroll
                            for (int x = 0; x < 2; ++x) {
                                const int i = (int)((rho0 + c0 + e + x) >> P.dw_log2);
                                const bool valid = (jb <= i + p.halo1) && (jb >= i + p.halo1 - p.w1 + 1);
                                const float pe = ex2(fmaf(__uint_as_float(s[e + x]), c2, -m_lse[i - iq0]));
                                pv[x] = valid ? pe : 0.f;
                                dv[x] = valid ? pe * (__uint_as_float(dp[e + x]) - m_delta[i - iq0]) : 0.f;
                            }
                            pp[e >> 1] = E::pack(pv[0], pv[1]);
                            ds[e >> 1] = E::pack(dv[0], dv[1]);
                        }
                        tmem_st8(tm_s + lane_addr + 64 * grp + (cc >> 1), pp);
                        tmem_st8(tm_dp + lane_addr + 64 * grp + (cc >> 1), ds);
                        tmem_wait_st();
                        tc_fence_before();
                        warp_arrive(&pds_ready[cc >> 4]);
                    }
                }
                SA_PROF_ADD(28, t_csm);
                if ((warp & 3) == 0) SA_TR(1 + grp, 53);
            }
            g_base += nt;
            // epilogue: group 0 writes dV1, group 1 writes dK1 (times scale)
            __nv_bfloat16* out = grp == 0 ? dv1 : dk1;
            const sa_strides st = grp == 0 ? p.dv1 : p.dk1;
            const float mult = grp == 0 ? 1.f : p.scale;
            if (nt > 0) {
                mbar_wait(acc_ready, n_items & 1, wctx, 21);
                ++n_items;
                tc_fence_after();
            }
            const uint32_t acc = (grp == 0 ? tm_dv1 : tm_dk1) + lane_addr;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t v[32];
                if (nt > 0) {
                    tmem_ld32(acc + c0, v);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = 0u;
                }
                if (out != nullptr && jb < p.n1) {
                    uint4* dst = (uint4*)(out + ci.b * st.b + (long)jb * st.n + ci.hk * st.h + c0);
#pragma unroll
                    for (int x = 0; x < 4; ++x)
                        dst[x] = make_uint4(E::pack(__uint_as_float(v[8 * x]) * mult, __uint_as_float(v[8 * x + 1]) * mult),
                                            E::pack(__uint_as_float(v[8 * x + 2]) * mult, __uint_as_float(v[8 * x + 3]) * mult),
                                            E::pack(__uint_as_float(v[8 * x + 4]) * mult, __uint_as_float(v[8 * x + 5]) * mult),
                                            E::pack(__uint_as_float(v[8 * x + 6]) * mult, __uint_as_float(v[8 * x + 7]) * mult));
                }
            }
            if (nt > 0) {
                tc_fence_before();
                warp_arrive(acc_free);
            }
        }
    } else if (warp < 16) {
        // ---------------------------------------------------------------- producers: group 0 forms A, group 1 forms C
        reg_alloc<SA_COL_PR>();
        const int grp = (warp - 8) >> 2;
        const int row = tid & 127;
        // DWL: compile-time log2 of the delta slots per query for 16, 32 and 64 slots (the operand rows of a tile are
        // then loaded one tile ahead, into registers, and multiplied and stored once the stage is free); 0: any other
        // count (those load when they store).
        auto producer_body = [&](auto dwl_c) {
        constexpr int DWL = decltype(dwl_c)::value;
        constexpr int kFormRegs = DWL != 0 ? ProductTileShape<HD, DWL != 0 ? DWL : 5>::NREGS : 1;
        uint4 fr[kFormRegs];
        float meta_lse = INFINITY, meta_delta = 0.f;
        uint32_t g_base = 0;
        const int nq = max(1, kColTileRows >> P.dw_log2);
        const bool meta_thread = grp == 0 && row < nq;
        // loads of tile t of item ci (rows of Q / dO and of K2 / V2, and the LSE2 / Delta of the tile's queries)
#define SA_COL_LOAD(CI, T)                                                                                                \
        {                                                                                                                 \
            const int h_ = (CI).hk * p.G + (T) / (CI).ntq;                                                                \
            const long rho0_ = (long)((CI).tt_lo + ((T) % (CI).ntq)) * kColTileRows;                                      \
            const int iq0_ = (int)(rho0_ >> P.dw_log2);                                                                   \
            if constexpr (DWL != 0) {                                                                                     \
                const __nv_bfloat16* xb_ = grp == 0 ? q + (CI).b * p.q.b + h_ * p.q.h : d_o + (CI).b * p.d_o.b + h_ * p.d_o.h; \
                const __nv_bfloat16* yb_ = grp == 0 ? k2 + (CI).b * p.k2.b + (CI).hk * p.k2.h : v2 + (CI).b * p.v2.b + (CI).hk * p.v2.h; \
                load_product_tile_shared<HD, DWL>(fr, row, iq0_, p.N, p.halo2, xb_, grp == 0 ? p.q.n : p.d_o.n, yb_,      \
                                                  grp == 0 ? p.k2.n : p.v2.n);                                            \
            }                                                                                                             \
            meta_lse = INFINITY;                                                                                          \
            meta_delta = 0.f;                                                                                             \
            if (meta_thread && iq0_ + row < p.N) {                                                                        \
                const long li_ = ((long)(CI).b * p.H + h_) * p.N + iq0_ + row;                                            \
                meta_lse = P.lse2[li_];                                                                                   \
                meta_delta = P.delta[li_];                                                                                \
            }                                                                                                             \
        }
        for (long it = blockIdx.x; it < P.num_col_items; it += gridDim.x) {
            const ColItem ci = col_item(P, it);
            const int nt = ci.ntq * p.G;
            if (nt > 0) SA_COL_LOAD(ci, 0);
            for (int t = 0; t < nt; ++t) {
                const uint32_t g = g_base + t;
                const int stage = (int)(g % kColStages);
                const int h = ci.hk * p.G + t / ci.ntq;
                const long rho0 = (long)(ci.tt_lo + (t % ci.ntq)) * kColTileRows;
                uint8_t* tile = smem + L::kStream + (stage * 2 + grp) * L::kTile;
                mbar_wait(&st_empty[stage], ((g / kColStages) & 1) ^ 1, wctx, 22);
                if ((warp & 3) == 0) SA_TR(3 + grp, 50);
                SA_PROF_T0(t_cform);
                const float bias = BIAS ? (grp == 0 ? p.k2_bias : p.v2_bias) : 0.f;
                const int iq0 = (int)(rho0 >> P.dw_log2);
                if constexpr (DWL != 0) {
                    store_product_tile_shared<HD, DWL, BIAS, F16>(tile, L::kSlab, row, iq0, p.N, p.w2, p.halo2, fr, bias);
                } else {
                    const __nv_bfloat16* xb = grp == 0 ? q + ci.b * p.q.b + h * p.q.h : d_o + ci.b * p.d_o.b + h * p.d_o.h;
                    const __nv_bfloat16* yb = grp == 0 ? k2 + ci.b * p.k2.b + ci.hk * p.k2.h : v2 + ci.b * p.v2.b + ci.hk * p.v2.h;
                    form_product_tile<HD, kColTileRows, 128, BIAS, F16>(tile, L::kSlab, row, rho0, P.dw_log2, p.N, p.w2, p.halo2, xb,
                                                                   grp == 0 ? p.q.n : p.d_o.n, yb, grp == 0 ? p.k2.n : p.v2.n, bias);
                }
                if (meta_thread) {
                    float* m_lse = (float*)(smem + L::kMeta) + stage * 256;
                    m_lse[row] = meta_lse;
                    m_lse[128 + row] = meta_delta;
                }
                fence_proxy_async_smem();
                warp_arrive(&st_full[stage]);
                if ((warp & 3) == 0) SA_TR(3 + grp, 51);
                SA_PROF_ADD(37 + grp, t_cform);
                // the next tile's rows start travelling now (past the item's end: this tile's once more, never used, so
                // that the registers are defined on every path)
                {
                    const int tn = t + 1 < nt ? t + 1 : t;
                    SA_COL_LOAD(ci, tn);
                }
            }
            g_base += nt;
        }
#undef SA_COL_LOAD
        };      // producer_body
        switch (P.dw_log2) {
            case 4: producer_body(std::integral_constant<int, 4>{}); break;
            case 5: producer_body(std::integral_constant<int, 5>{}); break;
            case 6: producer_body(std::integral_constant<int, 6>{}); break;
            default: producer_body(std::integral_constant<int, 0>{});
        }
    } else if (warp == 16) {
        // ---------------------------------------------------------------- MMA issuer
        reg_dealloc<SA_COL_REST>();
        {
            const uint32_t leader = elect_one();      // the whole warp runs the loop; one lane issues
            uint32_t g_base = 0, n_items = 0;
            const uint32_t idesc_sd = make_idesc(128, kColTileRows, false, false, F16);
            const uint32_t idesc_acc = make_idesc(128, HD, false, true, F16);
            const uint64_t d_k1 = desc_kmajor(smem_base + L::kK1, 0), d_v1 = desc_kmajor(smem_base + L::kV1, 0);
            for (long it = blockIdx.x; it < P.num_col_items; it += gridDim.x) {
                const ColItem ci = col_item(P, it);
                const int nt = ci.ntq * p.G;
                if (nt == 0) continue;
                mbar_wait(stat_full, n_items & 1, wctx, 23);
                if (n_items > 0) mbar_wait(acc_free, (n_items - 1) & 1, wctx, 24);
                tc_fence_after();
                for (int t = 0; t < nt; ++t) {
                    const uint32_t g = g_base + t;
                    const int stage = (int)(g % kColStages);
                    const uint32_t a_t = smem_base + L::kStream + stage * 2 * L::kTile, c_t = a_t + L::kTile;
                    const uint64_t d_a = desc_kmajor(a_t, 0), d_c = desc_kmajor(c_t, 0);
                    const uint64_t d_am = desc_mnmajor(a_t, L::kSlab), d_cm = desc_mnmajor(c_t, L::kSlab);
                    SA_TR(0, 1);
                    mbar_wait(&st_full[stage], (g / kColStages) & 1, wctx, 25);
                    SA_TR(0, 2);
                    tc_fence_after();
                    // S^T = K1 A^T,  dP^T = V1 C^T
                    SA_PROF_T0(t_ci1);
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk) {
                        const uint32_t off = ((kk >> 2) * L::kSlab + (kk & 3) * 32) >> 4;
                        mma_ss(leader, tm_s, d_k1 + off, d_a + off, idesc_sd, kk > 0);
                    }
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk) {
                        const uint32_t off = ((kk >> 2) * L::kSlab + (kk & 3) * 32) >> 4;
                        mma_ss(leader, tm_dp, d_v1 + off, d_c + off, idesc_sd, kk > 0);
                    }
                    tc_commit(leader, sdp_ready);
                    SA_TR(0, 3);
                    SA_PROF_ADD(29, t_ci1);
                    SA_PROF_T0(t_ci2);
                    // dV1 += P^T-tile C-tile,  dK1 += dS^T-tile A-tile   (K = 128 virtual rows: 8 steps of 16).
                    // Chunk k of both softmax groups (k-steps k and 4 + k) is issued as soon as it is stored.
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        mbar_wait(&pds_ready[k], g & 1, wctx, 26);
                        SA_TR(0, 10 + k);
                        tc_fence_after();
#pragma unroll
                        for (int gq = 0; gq < 2; ++gq) {
                            const int kk = 4 * gq + k;
                            mma_ts(leader, tm_dv1, tm_s + gq * 64 + k * 8, d_cm + kk * (2048 >> 4), idesc_acc, t > 0 || k > 0 || gq > 0);
                        }
#pragma unroll
                        for (int gq = 0; gq < 2; ++gq) {
                            const int kk = 4 * gq + k;
                            mma_ts(leader, tm_dk1, tm_dp + gq * 64 + k * 8, d_am + kk * (2048 >> 4), idesc_acc, t > 0 || k > 0 || gq > 0);
                        }
                    }
                    tc_commit(leader, &st_empty[stage]);
                    SA_TR(0, 4);
                    SA_PROF_ADD(36, t_ci2);
                }
                tc_commit(leader, acc_ready);
                tc_commit(leader, stat_empty);
                g_base += nt;
                ++n_items;
            }
        }
        __syncwarp();
    } else if (warp == 17) {
        // ---------------------------------------------------------------- TMA: the block's K1 / V1 rows
        reg_dealloc<SA_COL_REST>();
        if (lane == 0) {
            prefetch_tensormap(&map_k1);
            prefetch_tensormap(&map_v1);
            uint32_t n = 0;
            for (long it = blockIdx.x; it < P.num_col_items; it += gridDim.x) {
                const ColItem ci = col_item(P, it);
                if (ci.ntq == 0) continue;
                mbar_wait(stat_empty, (n & 1) ^ 1, wctx, 27);
                mbar_arrive_expect_tx(stat_full, 2 * L::kTile);
#pragma unroll
                for (int sl = 0; sl < L::kSlabs; ++sl) {
                    tma_load_4d(smem + L::kK1 + sl * L::kSlab, &map_k1, stat_full, sl * 64, ci.j0, ci.hk, ci.b);
                    tma_load_4d(smem + L::kV1 + sl * L::kSlab, &map_v1, stat_full, sl * 64, ci.j0, ci.hk, ci.b);
                }
                ++n;
            }
        }
        __syncwarp();
    } else {
        reg_dealloc<SA_COL_REST>();
    }
    tc_fence_before();
    __syncthreads();
    SA_PROF_LIFE(t_life);
    if (warp == 16) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------------------------------------
// 3. Row kernel: dQ and the per-query-head partial sums of dK2, dV2
// ------------------------------------------------------------------------------------------------
struct RowUnit {
    int i0;            // first query of the 128-row tile
    int col_start;     // first K1/V1 buffer row needed
    int nt;            // streamed 64-row tiles
    int last_width;    // width of the last one (multiple of 16)
};

__device__ __forceinline__ RowUnit row_unit(const BwdTcParams& P, int i0) {
    const KParams& p = P.k;
    RowUnit u;
    const int qpt = 128 >> P.dw_log2;
    u.i0 = i0;
    const int i_last = min(i0 + qpt, p.N) - 1;
    u.col_start = max(0, i0 + p.halo1 - p.w1 + 1);
    const int ncols = i_last + p.halo1 - u.col_start + 1;
    u.nt = (ncols + kStreamRows - 1) / kStreamRows;
    u.last_width = ((ncols - (u.nt - 1) * kStreamRows) + 15) & ~15;
    return u;
}

struct RowItem {
    int b, h, hk, run, i_run0, i_run1;     // queries [i_run0, i_run1)
};

__device__ __forceinline__ RowItem row_item(const BwdTcParams& P, long it) {
    const KParams& p = P.k;
    RowItem r;
    r.run = (int)(it % P.num_runs);
    const long bh = it / P.num_runs;
    r.h = (int)(bh % p.H);
    r.b = (int)(bh / p.H);
    r.hk = r.h / p.G;
    const int runq = P.units_per_run * (128 >> P.dw_log2);
    r.i_run0 = r.run * runq;
    r.i_run1 = min(p.N, r.i_run0 + runq);
    return r;
}

// Loads CW consecutive fp32 accumulator columns of this thread's tensor-memory lane.
template <int CW>
__device__ __forceinline__ void tmem_ld_cw(uint32_t addr, uint32_t (&v)[CW]) {
    if constexpr (CW == 32) ptx::tmem_ld32(addr, v);
    else if constexpr (CW == 16) ptx::tmem_ld16(addr, v);
    else ptx::tmem_ld8(addr, v);
    ptx::tmem_wait_ld();
}


// Index into a ring of fp32 rows [slot][HD + 2]: with this row pitch the same column pair of 32
// consecutive rows falls into different banks for 8-byte accesses, a column offset known at compile
// time stays an immediate in the address, and rows stay 8-byte aligned.
template <int HD>
__device__ __forceinline__ int ring_index(int slot, int col) {
    return slot * (HD + 2) + col;
}

template <int HD, int NS, bool TWOQ, bool BIAS, bool F16 = false>
__global__ void __launch_bounds__(kRowThreads, 1)
bwd_row_kernel(const __grid_constant__ BwdTcParams P, const __grid_constant__ CUtensorMap map_k1,
               const __grid_constant__ CUtensorMap map_v1, const __nv_bfloat16* __restrict__ q,
               const __nv_bfloat16* __restrict__ k2, const __nv_bfloat16* __restrict__ v2,
               const __nv_bfloat16* __restrict__ d_o, __nv_bfloat16* __restrict__ dq, int need_kv2, int ring_rows) {
    using L = BwdSmem<HD, NS>;
    using namespace ptx;
    using E = El<F16>;
    constexpr int CW = HD / 4;                            // epilogue chunk width
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const KParams& p = P.k;
    const BwdBars B = bwd_bars<NS>((uint64_t*)(smem + L::kBars));
    uint32_t* tmem_slot = (uint32_t*)(smem + L::kMisc);
    volatile int* abort_flag = (volatile int*)(smem + L::kMisc + 4);
    const WaitCtx wctx{abort_flag, P.status, P.wait_limit_ns};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    SA_PROF_T0(t_life);
    SA_TR_DECL();
    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&B.st_full[s], 1);
            mbar_init(&B.st_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&B.sdp_ready[b], 1);
            mbar_init(&B.pds_ready[b], 128);
        }
        mbar_init(B.stat_full, 256);       // A and C formed by the two softmax groups
        mbar_init(B.stat_empty, 1);
        mbar_init(B.acc_ready, 1);
        mbar_init(B.acc_free, 256);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 8) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tm_s[2] = {tmem_base, tmem_base + 64};
    const uint32_t tm_dp[2] = {tmem_base + 128, tmem_base + 192};
    const uint32_t tm_u = tmem_base + 256, tm_g = tmem_base + 384;     // U = P V1, G = dS K1
    const int DW = 1 << P.dw_log2;
    const int qpt = 128 >> P.dw_log2;

    if (warp < 8) {
        // ---------------------------------------------------------------- softmax groups + epilogue
        reg_alloc<216>();
        const int grp = warp >> 2;
        const int row = tid & 127;
        const uint32_t lane_addr = ((uint32_t)(row & ~31)) << 16;
        const int qq = row >> P.dw_log2;
        const int dlt = row & (DW - 1);
        const float c2 = p.scale * kLog2e;
        uint8_t* my_tile = smem + (grp == 0 ? L::kStat0 : L::kStat1);      // group 0 forms A, group 1 forms C
        float* scr_a = (float*)my_tile;                   // [128][CW] fp32, column index XOR-swizzled by the row
        float* scr_b = scr_a + 128 * CW;
        // fp32 accumulators of the dK2 (group 0) / dV2 (group 1) rows currently within reach of the
        // block's queries, one slot per row modulo ring_rows; ring_rows == 0: not enough shared memory
        float* ring = (float*)(smem + L::kRing) + grp * ring_rows * (HD + 2);
        for (int x = row; x < ring_rows * (HD + 2); x += 128) ring[x] = 0.f;
        named_barrier_sync(1 + grp, 128);
        int flush_lo = 0;
        uint32_t n_mine = 0, n_units = 0;
        for (long it = blockIdx.x; it < P.num_row_items; it += gridDim.x) {
            const RowItem ri = row_item(P, it);
            for (int i0 = ri.i_run0, uidx = 0; i0 < ri.i_run1; i0 += qpt, ++uidx, ++n_units) {
                const RowUnit ru = row_unit(P, i0);
                const int i = i0 + qq;
                const int kb = i + p.halo2 - dlt;
                const bool row_valid = (i < p.N) && (dlt < p.w2) && (kb >= 0);
                const int ic = min(i, p.N - 1), kc = min(max(kb, 0), p.n2 - 1);      // rows that exist (queries past the end are not stored)
                const __nv_bfloat16* q_row = q + ri.b * p.q.b + (long)ic * p.q.n + ri.h * p.q.h;
                const __nv_bfloat16* do_row = d_o + ri.b * p.d_o.b + (long)ic * p.d_o.n + ri.h * p.d_o.h;
                const __nv_bfloat16* k2_row = k2 + ri.b * p.k2.b + (long)kc * p.k2.n + ri.hk * p.k2.h;
                const __nv_bfloat16* v2_row = v2 + ri.b * p.v2.b + (long)kc * p.v2.n + ri.hk * p.v2.h;
                // ---- stationary operand of this group
                SA_PROF_T0(t_form);
                if (grp == 0)
                    form_query_tile<HD, BIAS, F16>(my_tile, L::kBigSlab, row, i0, P.dw_log2, p.N, p.w2, p.halo2,
                                              q + ri.b * p.q.b + ri.h * p.q.h, p.q.n, k2 + ri.b * p.k2.b + ri.hk * p.k2.h, p.k2.n,
                                              BIAS ? p.k2_bias : 0.f);
                else
                    form_query_tile<HD, BIAS, F16>(my_tile, L::kBigSlab, row, i0, P.dw_log2, p.N, p.w2, p.halo2,
                                              d_o + ri.b * p.d_o.b + ri.h * p.d_o.h, p.d_o.n,
                                              v2 + ri.b * p.v2.b + ri.hk * p.v2.h, p.v2.n, BIAS ? p.v2_bias : 0.f);
                fence_proxy_async_smem();
                tc_fence_before();
                mbar_arrive(B.stat_full);
                SA_PROF_ADD(40 + grp, t_form);
                SA_PROF_T0(t_loop);
                const long li = ((long)ri.b * p.H + ri.h) * p.N + ic;
                const float lse2 = P.lse2[li], dlt_i = P.delta[li];
                const int jhi = row_valid ? i + p.halo1 : -1;
                const int jlo = row_valid ? max(0, i + p.halo1 - p.w1 + 1) : 0;
                // ---- column tiles of this group
                for (int t = grp; t < ru.nt; t += 2, ++n_mine) {
                    const int width = (t == ru.nt - 1) ? ru.last_width : kStreamRows;
                    const int tile0 = ru.col_start + t * kStreamRows;
                    const int lo = jlo - tile0, hi = jhi - tile0;
                    const bool full = __all_sync(0xffffffffu, lo <= 0 && hi >= kStreamRows - 1);
                    mbar_wait(&B.sdp_ready[grp], n_mine & 1, wctx, 30);
                    tc_fence_after();
                    SA_PROF_T0(t_rsm);
#pragma unroll 1
                    for (int c0 = 0; c0 < width; c0 += 32) {
                        uint32_t s[32], dp[32], pp[16], ds[16];
                        tmem_ld32(tm_s[grp] + lane_addr + c0, s);
                        tmem_ld32(tm_dp[grp] + lane_addr + c0, dp);
                        tmem_wait_ld();
                        if (full) softmax_bwd_chunk<false, 32, F16>(s, dp, c0, lo, hi, c2, lse2, dlt_i, pp, ds);
                        else softmax_bwd_chunk<true, 32, F16>(s, dp, c0, lo, hi, c2, lse2, dlt_i, pp, ds);
                        tmem_st16(tm_s[grp] + lane_addr + (c0 >> 1), pp);
                        tmem_st16(tm_dp[grp] + lane_addr + (c0 >> 1), ds);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(&B.pds_ready[grp]);
                    SA_PROF_ADD(58 + grp, t_rsm);
                }
                // ---- epilogue: group 0 takes G (dQ and dK2 partials), group 1 takes U (dV2 partials)
                const uint32_t acc = (grp == 0 ? tm_g : tm_u) + lane_addr;
                const __nv_bfloat16* y_row = grp == 0 ? q_row : do_row;
                const float mult = grp == 0 ? p.scale : 1.f;
                float* ws_full = grp == 0 ? P.ws_full_k2 : P.ws_full_v2;
                float* ws_head = grp == 0 ? P.ws_head_k2 : P.ws_head_v2;
                const long bh = (long)ri.b * p.H + ri.h;
                const int kb_base = i0 + p.halo2 - (DW - 1);                 // K2 buffer row of kbrel = 0
                const int kb_min = max(0, i0 + p.halo2 - (p.w2 - 1));        // first row any valid delta reaches
                const int kb_max = min(i0 + qpt, p.N) - 1 + p.halo2;
                const int own0 = ri.i_run0 + p.halo2;                        // first row owned by this run
                if (uidx == 0) flush_lo = max(0, own0 - (p.w2 - 1));
                SA_PROF_ADD(42 + grp, t_loop);
                mbar_wait(B.acc_ready, n_units & 1, wctx, 31);
                tc_fence_after();
                SA_PROF_T0(t_epi);
                if ((TWOQ ? P.dw_log2 == 4 : P.dw_log2 >= 5) && (ring_rows > 0 || !need_kv2)) {
                    // ---- a warp holds 32 consecutive deltas of one query (DW >= 32) or all 16 deltas of two
                    // queries (DW = 16): within a query its lanes own distinct K2 rows.  Warp w works on
                    // column chunk (w + phase) % 4, so no two warps touch the same ring columns at the same
                    // time; the delta sum for dQ is a register exchange inside the warp (or half warp).
                    const int wq = row >> 5;
                    constexpr bool two_q = TWOQ;                         // DW = 16: two queries per warp
                    const int part_row = two_q ? (wq * 2 + (lane >> 4)) : wq;
                    float* dq_part = scr_a;                              // [4 partial rows][HD] when a query spans several warps
                    const int ppq = two_q ? 1 : (DW >> 5);               // partial rows (warps) per query
                    __nv_bfloat16* dq_out = dq == nullptr ? nullptr : dq + ri.b * p.dq.b + (long)i0 * p.dq.n + ri.h * p.dq.h;
                    const int slot = row_valid ? kb % max(ring_rows, 1) : 0;
                    // Rows that are not valid (delta >= w2, K2 row before the buffer, query past the end) have
                    // P = dS = 0, hence exact zeros in U and G: they need no masking in the sums below.
                    SA_PROF_ADD(28 + grp, t_epi);
#pragma unroll 1
                    for (int ph = 0; ph < 4; ++ph) {
                        const int c = (wq + ph) & 3;
                        SA_PROF_T0(t_p0);
                        uint32_t yw[CW / 2], xw[CW / 2], g[CW];
                        load_bf16_words<CW>(y_row + c * CW, yw);
                        if (grp == 0) load_bf16_words<CW>(k2_row + c * CW, xw);
                        tmem_ld_cw<CW>(acc + c * CW, g);
                        SA_PROF_ADD(50 + 4 * grp, t_p0);
                        SA_PROF_T0(t_p1);
                        if (grp == 0 && dq != nullptr) {
                            float v[CW];
                            if constexpr (!BIAS) {
#pragma unroll
                                for (int e = 0; e < CW; e += 2) {
                                    const float2 t = __fmul2_rn(make_float2(__uint_as_float(g[e]), __uint_as_float(g[e + 1])),
                                                                make_float2(E::lo(xw[e >> 1]), E::hi(xw[e >> 1])));
                                    v[e] = t.x;
                                    v[e + 1] = t.y;
                                }
                            } else {
#pragma unroll
                                for (int e = 0; e < CW; e += 2) {
                                    v[e] = __uint_as_float(g[e]) * (E::lo(xw[e >> 1]) + p.k2_bias);
                                    v[e + 1] = __uint_as_float(g[e + 1]) * (E::hi(xw[e >> 1]) + p.k2_bias);
                                }
                            }
                            if constexpr (!two_q) {
                                const float tot = warp_transpose_reduce<CW>(v, lane) * mult;
                                if (lane < CW) {
                                    if (ppq == 1) {      // the warp holds the whole query: its dQ columns are final
                                        if (i0 + wq < p.N) E::st(&dq_out[(long)wq * p.dq.n + c * CW + lane], tot);
                                    } else {
                                        dq_part[part_row * HD + c * CW + lane] = tot;
                                    }
                                }
                            } else {
#pragma unroll
                                for (int hb = 0; hb < CW / 16; ++hb) {
                                    float vv[16];
#pragma unroll
                                    for (int e = 0; e < 16; ++e) vv[e] = v[16 * hb + e];
                                    const float tot = half_warp_transpose_reduce16(vv, lane) * mult;
                                    if (i0 + part_row < p.N)
                                        E::st(&dq_out[(long)part_row * p.dq.n + c * CW + 16 * hb + (lane & 15)], tot);
                                }
                            }
                        }
                        SA_PROF_ADD(51 + 4 * grp, t_p1);
                        SA_PROF_T0(t_p2);
                        // ring update, staged (all loads, then all adds, then all stores).  With two queries in
                        // a warp, lanes (q, delta) and (q+1, delta+1) own the same K2 row: the halves take turns.
                        for (int turn = 0; turn < (two_q ? 2 : 1); ++turn) {
                            if (need_kv2 && row_valid && (!two_q || (lane >> 4) == turn)) {
                                float2* rp = (float2*)(ring + ring_index<HD>(slot, c * CW));
                                float2 acc_r[CW / 2];
#pragma unroll
                                for (int e = 0; e < CW / 2; ++e) acc_r[e] = rp[e];
#pragma unroll
                                for (int e = 0; e < CW / 2; ++e)
                                    acc_r[e] = __ffma2_rn(make_float2(__uint_as_float(g[2 * e]), __uint_as_float(g[2 * e + 1])),
                                                          make_float2(E::lo(yw[e]), E::hi(yw[e])), acc_r[e]);
#pragma unroll
                                for (int e = 0; e < CW / 2; ++e) rp[e] = acc_r[e];
                            }
                            if (two_q) __syncwarp();
                        }
                        SA_PROF_ADD(52 + 4 * grp, t_p2);
                        SA_PROF_T0(t_p3);
                        named_barrier_sync(1 + grp, 128);
                        SA_PROF_ADD(53 + 4 * grp, t_p3);
                    }
                    SA_PROF_T0(t_dqf);
                    if (grp == 0 && dq != nullptr && ppq > 1) {
                        // a query spans DW / 32 warps: thread t finishes column t
                        if (row < HD) {
                            for (int q2 = 0; q2 < qpt; ++q2) {
                                float a = 0.f;
                                for (int w2i = 0; w2i < ppq; ++w2i) a += dq_part[(q2 * ppq + w2i) * HD + row];
                                if (i0 + q2 < p.N)
                                    E::st(&dq[ri.b * p.dq.b + (long)(i0 + q2) * p.dq.n + ri.h * p.dq.h + row], a);
                            }
                        }
                        named_barrier_sync(1 + grp, 128);
                    }
                    SA_PROF_ADD(24 + grp, t_dqf);
                } else {
                // ---- general path (several queries per warp, or no room for the ring): stage the scaled
                // rows in shared memory and sum them per output row
#pragma unroll 1
                for (int c = 0; c < HD / CW; ++c) {
                    uint32_t g[CW];
                    tmem_ld_cw<CW>(acc + c * CW, g);
                    uint32_t yw[CW / 2], xw[CW / 2];
                    load_bf16_words<CW>(y_row + c * CW, yw);
                    if (grp == 0) {
                        load_bf16_words<CW>(k2_row + c * CW, xw);
#pragma unroll
                        for (int e = 0; e < CW; ++e) {
                            const float xf = ((e & 1) ? E::hi(xw[e >> 1]) : E::lo(xw[e >> 1])) + (BIAS ? p.k2_bias : 0.f);
                            scr_a[row * CW + (e ^ (row & (CW - 1)))] = row_valid ? __uint_as_float(g[e]) * xf * mult : 0.f;
                        }
                    }
#pragma unroll
                    for (int e = 0; e < CW; ++e) {
                        const float yf = (e & 1) ? E::hi(yw[e >> 1]) : E::lo(yw[e >> 1]);
                        scr_b[row * CW + (e ^ (row & (CW - 1)))] = row_valid ? __uint_as_float(g[e]) * yf : 0.f;
                    }
                    named_barrier_sync(1 + grp, 128);
                    if (grp == 0 && dq != nullptr) {
                        for (int idx = row; idx < qpt * CW; idx += 128) {
                            const int q2 = idx / CW, e = idx % CW;
                            float a = 0.f;
                            for (int d2 = 0; d2 < DW; ++d2) {
                                const int rr = (q2 << P.dw_log2) + d2;
                                a += scr_a[rr * CW + (e ^ (rr & (CW - 1)))];
                            }
                            if (i0 + q2 < p.N)
                                E::st(&dq[ri.b * p.dq.b + (long)(i0 + q2) * p.dq.n + ri.h * p.dq.h + c * CW + e], a);
                        }
                    }
                    if (need_kv2) {
                        const int nrows = DW + qpt - 1;
                        for (int idx = row; idx < nrows * CW; idx += 128) {
                            const int kbrel = idx / CW, e = idx % CW;
                            const int kbt = kb_base + kbrel;
                            if (kbt < kb_min || kbt > kb_max) continue;
                            float a = 0.f;
                            for (int q2 = 0; q2 < qpt; ++q2) {
                                const int d2 = q2 + DW - 1 - kbrel;
                                if (d2 >= 0 && d2 < DW) {
                                    const int rr = (q2 << P.dw_log2) + d2;
                                    a += scr_b[rr * CW + (e ^ (rr & (CW - 1)))];
                                }
                            }
                            if (ring_rows > 0) {
                                ring[ring_index<HD>(kbt % ring_rows, c * CW + e)] += a;
                            } else {
                                // no room for the ring: accumulate in the workspace (this block alone touches the row)
                                float* dst;
                                bool first;
                                if (kbt >= own0) {
                                    dst = ws_full + (bh * p.N + (kbt - p.halo2)) * HD + c * CW + e;
                                    first = kbt >= i0 + p.halo2;
                                } else {
                                    const int slot = kbt - (own0 - (p.w2 - 1));
                                    dst = ws_head + ((bh * P.num_runs + ri.run) * (p.w2 - 1) + slot) * HD + c * CW + e;
                                    first = uidx == 0;
                                }
                                *dst = first ? a * mult : fmaf(a, mult, *dst);
                            }
                        }
                    }
                    named_barrier_sync(1 + grp, 128);
                }
                }
                SA_PROF_T0(t_flush);
                if (need_kv2 && ring_rows > 0) {
                    // rows no later query of the run reaches are final: move them to the workspace, clear the slots
                    const bool last_unit = i0 + qpt >= ri.i_run1;
                    const int f_hi = last_unit ? kb_max + 1 : max(0, i0 + qpt + p.halo2 - (p.w2 - 1));
                    // each warp moves whole rows, a lane four consecutive columns of them
                    for (int kbf = flush_lo + (row >> 5); kbf < f_hi; kbf += 4) {
                        const int slot = kbf % ring_rows;
                        float* dst = (kbf >= own0) ? ws_full + (bh * p.N + (kbf - p.halo2)) * HD
                                                   : ws_head + ((bh * P.num_runs + ri.run) * (p.w2 - 1) + (kbf - (own0 - (p.w2 - 1)))) * HD;
                        float* src = ring + ring_index<HD>(slot, 0);
                        for (int d = lane * 4; d < HD; d += 128) {
                            // the ring holds unscaled sums
                            *(float4*)(dst + d) = make_float4(src[d] * mult, src[d + 1] * mult, src[d + 2] * mult, src[d + 3] * mult);
                            src[d] = 0.f;
                            src[d + 1] = 0.f;
                            src[d + 2] = 0.f;
                            src[d + 3] = 0.f;
                        }
                    }
                    flush_lo = max(flush_lo, f_hi);
                }
                SA_PROF_ADD(26 + grp, t_flush);
                SA_PROF_ADD(44 + grp, t_epi);
                tc_fence_before();
                mbar_arrive(B.acc_free);
            }
        }
    } else if (warp == 8) {
        // ---------------------------------------------------------------- MMA issuer
        reg_dealloc<72>();
        {
            const uint32_t leader = elect_one();      // the whole warp runs the loop; one lane issues
            uint32_t nb[2] = {0, 0}, g_base = 0, n_units = 0;
            const uint32_t idesc_full = make_idesc(128, kStreamRows, false, false, F16);
            const uint32_t a_s = smem_base + L::kStat0, c_s = smem_base + L::kStat1;
            for (long it = blockIdx.x; it < P.num_row_items; it += gridDim.x) {
                const RowItem ri = row_item(P, it);
                for (int i0 = ri.i_run0; i0 < ri.i_run1; i0 += qpt, ++n_units) {
                    const RowUnit ru = row_unit(P, i0);
                    mbar_wait(B.stat_full, n_units & 1, wctx, 32);      // A, C formed (implies last epilogue done)
                    tc_fence_after();
                    SA_PROF_T0(t_mma);
                    for (int t = 0; t <= ru.nt; ++t) {
                        if (t < ru.nt) {
                            const uint32_t g = g_base + t;
                            const int stage = (int)(g % NS), b = t & 1;
                            const int width = (t == ru.nt - 1) ? ru.last_width : kStreamRows;
                            const uint32_t k1_t = smem_base + L::kStream + stage * 2 * L::kSmallTile, v1_t = k1_t + L::kSmallTile;
                            mbar_wait(&B.st_full[stage], (g / NS) & 1, wctx, 33);
                            tc_fence_after();
                            SA_PROF_T0(t_i1);
                            issue_sdp<HD>(leader, tm_s[b], tm_dp[b], a_s, c_s, k1_t, v1_t, width == kStreamRows ? idesc_full : make_idesc(128, width, false, false, F16));
                            tc_commit(leader, &B.sdp_ready[b]);
                            SA_PROF_ADD(47, t_i1);
                        }
                        if (t >= 1) {
                            const int tp = t - 1;
                            const uint32_t g = g_base + tp;
                            const int stage = (int)(g % NS), b = tp & 1;
                            const int width = (tp == ru.nt - 1) ? ru.last_width : kStreamRows;
                            const uint32_t k1_t = smem_base + L::kStream + stage * 2 * L::kSmallTile, v1_t = k1_t + L::kSmallTile;
                            mbar_wait(&B.pds_ready[b], nb[b] & 1, wctx, 34);
                            ++nb[b];
                            tc_fence_after();
                            // U += P V1-tile ; G += dS K1-tile
                            SA_PROF_T0(t_i2);
                            issue_acc<HD, false, F16>(leader, tm_u, tm_g, tm_s[b], tm_dp[b], k1_t, v1_t, width / 16, tp > 0);
                            tc_commit(leader, &B.st_empty[stage]);
                            SA_PROF_ADD(48, t_i2);
                        }
                    }
                    tc_commit(leader, B.acc_ready);
                    SA_PROF_ADD(46, t_mma);
                    g_base += ru.nt;
                }
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ---------------------------------------------------------------- TMA: streamed K1 / V1 tiles
        reg_dealloc<72>();
        if (lane == 0) {
            prefetch_tensormap(&map_k1);
            prefetch_tensormap(&map_v1);
            uint32_t g = 0;
            for (long it = blockIdx.x; it < P.num_row_items; it += gridDim.x) {
                const RowItem ri = row_item(P, it);
                for (int i0 = ri.i_run0; i0 < ri.i_run1; i0 += qpt) {
                    const RowUnit ru = row_unit(P, i0);
                    for (int t = 0; t < ru.nt; ++t, ++g) {
                        const int stage = (int)(g % NS);
                        const int r0 = ru.col_start + t * kStreamRows;
                        uint8_t* k1_t = smem + L::kStream + stage * 2 * L::kSmallTile;
                        uint8_t* v1_t = k1_t + L::kSmallTile;
                        mbar_wait(&B.st_empty[stage], ((g / NS) & 1) ^ 1, wctx, 35);
                        mbar_arrive_expect_tx(&B.st_full[stage], 2 * L::kSmallTile);
#pragma unroll
                        for (int sl = 0; sl < L::kSlabs; ++sl) {
                            tma_load_4d(k1_t + sl * L::kSmallSlab, &map_k1, &B.st_full[stage], sl * 64, r0, ri.hk, ri.b);
                            tma_load_4d(v1_t + sl * L::kSmallSlab, &map_v1, &B.st_full[stage], sl * 64, r0, ri.hk, ri.b);
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else {
        reg_dealloc<72>();
    }
    tc_fence_before();
    __syncthreads();
    SA_PROF_LIFE(t_life);
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------------------------------------
// 3b. Row kernel with separate operand / epilogue warpgroups, for 16, 32 or 64 delta slots per query (w2 in
//     9..64) when the dK2/dV2 ring fits: warps 0-7 run the softmax of every tile, warps 8-15 form the next
//     unit's operands the moment the tensor cores have finished with the current ones and take U and G out of
//     tensor memory (dQ, dK2 ring, dV2 ring) while warps 0-7 already work on the next unit, so neither the
//     operand formation nor the epilogue of a unit interrupts the stream of tiles.  Same workspace contents as
//     bwd_row_kernel; U and G pass through one 16-bit rounding before the final sums.
// ------------------------------------------------------------------------------------------------
// Bytes of one staging buffer of the row kernel with separate epilogue warpgroups: the raw Q and dO rows of a
// unit's queries and the K2 rows of their window (row pitch padded by 16 bytes so that the lanes of a warp, which
// read consecutive rows at the same column, fall into different banks).  Used for 16 and 32 delta slots per query.
constexpr int row2_stage_bytes(int dwl, int hd) {
    return dwl > 5 ? 0 : 2 * (128 >> dwl) * hd * 2 + ((1 << dwl) + (128 >> dwl) - 1) * (hd * 2 + 16);
}

// Registers per thread of the softmax groups, the operand / epilogue groups and the remaining warps of the row
// kernel below (multiples of 8; 128 x (2 SM + 2 EP + REST) must not exceed the block's launch allocation, 640 x 96).
// Measured: the operand / epilogue groups are the ones that need them (their unit of work holds 64 registers of
// accumulator data): 96 / 128 / 32 is 10 % faster at short windows than 104 / 112 / 48 and equal at long ones.
#ifndef SA_R2_SM
#define SA_R2_SM 96
#define SA_R2_EP 128
#define SA_R2_REST 32
#endif
static_assert(128 * (2 * SA_R2_SM + 2 * SA_R2_EP + SA_R2_REST) <= 640 * 96 && SA_R2_SM >= 96 && SA_R2_EP >= 96,
              "register pool of the row kernel's block; an increase must not go below the launch allocation");
constexpr int kRow2Threads = 640;     // softmax groups (0-7), epilogue groups (8-15), MMA issuers (16, 17), TMA (18), 1 idle

template <int HD, int DWL, int NS, bool BIAS, bool F16 = false>
__global__ void __launch_bounds__(kRow2Threads, 1)
bwd_row2_kernel(const __grid_constant__ BwdTcParams P, const __grid_constant__ CUtensorMap map_k1,
                const __grid_constant__ CUtensorMap map_v1, const __nv_bfloat16* __restrict__ q,
                const __nv_bfloat16* __restrict__ k2, const __nv_bfloat16* __restrict__ v2,
                const __nv_bfloat16* __restrict__ d_o, __nv_bfloat16* __restrict__ dq, int need_kv2, int ring_rows) {
    using L = BwdSmem<HD, NS>;
    using namespace ptx;
    using E = El<F16>;
    constexpr int CW = HD / 8;                            // epilogue chunk width: four chunks per half of the columns
    static_assert(DWL >= 4 && DWL <= 6, "16, 32 or 64 delta slots per query");
    constexpr int DW = 1 << DWL, QPT = 128 >> DWL;        // delta slots per query, queries per 128-row unit
    constexpr bool TWO_Q = DWL == 4;                      // a warp holds two queries of 16 deltas each
    constexpr int WPQ = DW > 32 ? DW / 32 : 1;            // warps per query
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const KParams& p = P.k;
    const BwdBars B = bwd_bars<NS>((uint64_t*)(smem + L::kBars));
    uint64_t* const buf_free = (uint64_t*)(smem + L::kBars) + 2 * NS + 8;      // [2] an S / dP buffer's P and dS have been consumed
    // Staging: the groups that form A and C have a unit's Q, dO and K2 rows in registers then; they leave raw copies in
    // shared memory (two buffers, alternating by unit) for the unit's epilogue, which needs the same rows again per
    // column chunk and would otherwise fetch them from global memory.
    constexpr bool STAGE = DWL <= 5;
    constexpr int NWIN = DW + QPT - 1;
    constexpr int K2PITCH = HD * 2 + 16;
    constexpr int kStageBuf = row2_stage_bytes(DWL, HD);
    uint8_t* const stage_base = smem + L::kRing + 2 * ring_rows * (HD + 2) * 4 + 2048;      // behind the rings and the partial dQ rows
    uint32_t* tmem_slot = (uint32_t*)(smem + L::kMisc);
    volatile int* abort_flag = (volatile int*)(smem + L::kMisc + 4);
    const WaitCtx wctx{abort_flag, P.status, P.wait_limit_ns};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    SA_PROF_T0(t_life);
    SA_TR_DECL();
    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&B.st_full[s], 1);
            mbar_init(&B.st_empty[s], 1);
        }
        // (barriers a warp group arrives on count one elected arrival per warp)
        for (int b = 0; b < 2; ++b) {
            mbar_init(&B.sdp_ready[b], 1);
            mbar_init(&B.pds_ready[b], 8);     // both softmax groups: each turns half the columns of a tile into P and dS
        }
        mbar_init(B.stat_full, 8);         // A and C formed by the two operand / epilogue groups
        mbar_init(B.stat_empty, 1);        // the unit's last S / dP MMAs have read A and C
        mbar_init(B.acc_ready, 1);         // U and G final
        mbar_init(B.acc_free, 8);          // U and G read out by the two epilogue groups
        for (int b = 0; b < 2; ++b) {
            mbar_init(&buf_free[b], 1);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 16) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tm_s[2] = {tmem_base, tmem_base + 64};
    const uint32_t tm_dp[2] = {tmem_base + 128, tmem_base + 192};
    const uint32_t tm_u = tmem_base + 256, tm_g = tmem_base + 384;     // U = P V1, G = dS K1

    // Register pool of the block: 640 x 96 = 128 x (2 x softmax groups + 2 x operand / epilogue groups + the rest) at
    // the counts SA_R2_*: an increase beyond the block's own pool would never return.
    if (warp < 8) {
        // ---------------------------------------------------------------- softmax
        // Every column tile (64 columns) is split between the two groups: group g turns columns [32g, 32g + 32)
        // of S and dP into P and dS, so a tile's softmax takes half as long and the accumulating MMAs that wait
        // for it start that much earlier.  P and dS (16-bit) go to columns [32g, 32g + 16) of the S / dP buffer:
        // inside the group's own columns.  The two S / dP buffers alternate over all tiles of the block, not per
        // unit, so that the first tile of a unit never waits for the buffer of the previous unit's last tile.
        reg_alloc<SA_R2_SM>();
        const int grp = warp >> 2;
        const int row = tid & 127;
        const uint32_t lane_addr = ((uint32_t)(row & ~31)) << 16;
        const int qq = row >> DWL;
        const int dlt = row & (DW - 1);
        const float c2 = p.scale * kLog2e;
        auto warp_arrive = [&](uint64_t* bar) {      // every lane has finished and fenced its part; lane 0 arrives for the warp
            __syncwarp();
            if (lane == 0) mbar_arrive(bar);
        };
        uint32_t gt = 0;                             // tiles so far
        for (long it = blockIdx.x; it < P.num_row_items; it += gridDim.x) {
            const RowItem ri = row_item(P, it);
            for (int i0 = ri.i_run0; i0 < ri.i_run1; i0 += QPT) {
                const RowUnit ru = row_unit(P, i0);
                const int i = i0 + qq;
                const int kb = i + p.halo2 - dlt;
                const bool row_valid = (i < p.N) && (dlt < p.w2) && (kb >= 0);
                const int ic = min(i, p.N - 1);
                SA_PROF_T0(t_loop);
                const long li = ((long)ri.b * p.H + ri.h) * p.N + ic;
                const float lse2 = P.lse2[li], dlt_i = P.delta[li];
                const int jhi = row_valid ? i + p.halo1 : -1;
                const int jlo = row_valid ? max(0, i + p.halo1 - p.w1 + 1) : 0;
                for (int t = 0; t < ru.nt; ++t, ++gt) {
                    const int b = gt & 1;
                    const int width = (t == ru.nt - 1) ? ru.last_width : kStreamRows;
                    const int c0 = 32 * grp;                                   // first column of this group's half
                    const int tile0 = ru.col_start + t * kStreamRows;
                    const int lo = jlo - tile0, hi = jhi - tile0;
                    const bool full = __all_sync(0xffffffffu, lo <= c0 && hi >= c0 + 31);
                    mbar_wait(&B.sdp_ready[b], (gt >> 1) & 1, wctx, 30);
                    if ((warp & 3) == 0) SA_TR(1 + grp, 52);
                    tc_fence_after();
                    SA_PROF_T0(t_rsm);
                    if (c0 < width) {
                        uint32_t s[32], dp[32], pp[16], ds[16];
                        tmem_ld32(tm_s[b] + lane_addr + c0, s);
                        tmem_ld32(tm_dp[b] + lane_addr + c0, dp);
                        tmem_wait_ld();
                        if (full) softmax_bwd_chunk<false, 32, F16>(s, dp, c0, lo, hi, c2, lse2, dlt_i, pp, ds);
                        else softmax_bwd_chunk<true, 32, F16>(s, dp, c0, lo, hi, c2, lse2, dlt_i, pp, ds);
                        tmem_st16(tm_s[b] + lane_addr + c0, pp);
                        tmem_st16(tm_dp[b] + lane_addr + c0, ds);
                        tmem_wait_st();
                    }
                    tc_fence_before();
                    warp_arrive(&B.pds_ready[b]);
                    if ((warp & 3) == 0) SA_TR(1 + grp, 53);
                    SA_PROF_ADD(58 + grp, t_rsm);
                }
                SA_PROF_ADD(42 + grp, t_loop);
            }
        }
    } else if (warp < 16) {
        // ---------------------------------------------------------------- operand + epilogue groups
        // Two jobs, interleaved per unit.  (1) Form the NEXT unit's stationary operands as soon as the current
        // unit's last S / dP MMAs have read the old ones: group 0 forms A = Q * K2, group 1 forms C = dO * V2, from
        // rows loaded well before (the softmax groups are still busy with the current unit's last tiles then, and
        // the S / dP MMAs of the next unit can follow the current unit's without a gap).  (2) The current unit's
        // epilogue: group g takes columns [g * HD/2, (g + 1) * HD/2) of all three results (dQ and dK2 from G, dV2
        // from U), so both groups carry the same load and no ring column is shared between them.
        reg_alloc<SA_R2_EP>();
        const int grp = (warp - 8) >> 2;
        const int row = tid & 127;
        const uint32_t lane_addr = ((uint32_t)(row & ~31)) << 16;
        const int qq = row >> DWL;
        const int dlt = row & (DW - 1);
        const int wq = row >> 5;                          // warp within the group
        constexpr int HALF = HD / 2;
        constexpr int NPHG = HALF / CW;                   // phases per group (4 at HD = 128)
        static_assert(NPHG == 4, "one column chunk per warp and phase");
        const int cbase = grp * HALF;
        // fp32 accumulators of the dK2 / dV2 rows currently within reach of the block's queries, one slot
        // per row modulo ring_rows
        float* ring_k = (float*)(smem + L::kRing);
        float* ring_v = ring_k + ring_rows * (HD + 2);
        float* dq_part = ring_v + ring_rows * (HD + 2) + grp * 4 * HALF;     // [4 warps][HALF] when a query spans two warps
        for (int x = row; x < ring_rows * HALF; x += 128) {
            const int idx = ring_index<HD>(x / HALF, cbase + x % HALF);
            ring_k[idx] = 0.f;
            ring_v[idx] = 0.f;
        }
        named_barrier_sync(3 + grp, 128);
        // ---- operand formation: this group's tile, its row and window operands
        uint8_t* const my_tile = smem + (grp == 0 ? L::kStat0 : L::kStat1);
        const __nv_bfloat16* const x_t = grp == 0 ? q : d_o;
        const __nv_bfloat16* const y_t = grp == 0 ? k2 : v2;
        const sa_strides xs = grp == 0 ? p.q : p.d_o, ys = grp == 0 ? p.k2 : p.v2;
        const float bias = BIAS ? (grp == 0 ? p.k2_bias : p.v2_bias) : 0.f;
        // Forms the unit that starts at query f_i0 of item f_ri out of the rows in fr; leaves raw copies of the Q, dO
        // and K2 rows in staging buffer sb for the epilogue (which needs them again, per column chunk).
        long f_it = blockIdx.x;                            // the unit to form next
        RowItem f_ri = row_item(P, f_it < P.num_row_items ? f_it : 0);
        int f_i0 = f_ri.i_run0;
        uint32_t n_formed = 0;
#define SA_ROW2_LOAD(fr)                                                                                              \
        load_product_tile_shared<HD, DWL>(fr, row, f_i0, p.N, p.halo2, x_t + f_ri.b * xs.b + f_ri.h * xs.h, xs.n,      \
                                          y_t + f_ri.b * ys.b + f_ri.hk * ys.h, ys.n)
#define SA_ROW2_FORM(fr)                                                                                              \
        do {                                                                                                          \
            using S = ProductTileShape<HD, DWL>;                                                                      \
            if ((warp & 3) == 0) SA_TR(3 + grp, 50);                                                                  \
            store_product_tile_shared<HD, DWL, BIAS, F16>(my_tile, L::kBigSlab, row, f_i0, p.N, p.w2, p.halo2, fr, bias); \
            if constexpr (STAGE) {                                                                                    \
                uint8_t* const stg_w = stage_base + (n_formed & 1) * kStageBuf;                                       \
                const int c = row % S::C, pr = row / S::C;                                                            \
                if (pr == 0) {                                                                                        \
                    _Pragma("unroll") for (int q2 = 0; q2 < S::NQ; ++q2)                                              \
                        *(uint4*)(stg_w + (grp * QPT + q2) * HD * 2 + c * 16) = fr[q2];                               \
                }                                                                                                     \
                if (grp == 0) {                                                                                       \
                    _Pragma("unroll") for (int k = 0; k < S::PASSES; ++k) {                                           \
                        const int w = pr + k * S::RPP;                                                                \
                        if (w < NWIN) *(uint4*)(stg_w + 2 * QPT * HD * 2 + w * K2PITCH + c * 16) = fr[S::NQ + k];     \
                    }                                                                                                 \
                }                                                                                                     \
            }                                                                                                         \
            fence_proxy_async_smem();                                                                                 \
            tc_fence_before();                                                                                        \
            __syncwarp();                                                                                             \
            if (lane == 0) mbar_arrive(B.stat_full);                                                                  \
            if ((warp & 3) == 0) SA_TR(3 + grp, 51);                                                                  \
            ++n_formed;                                                                                               \
            f_i0 += QPT;                                                                                              \
            if (f_i0 >= f_ri.i_run1) {                                                                                \
                f_it += gridDim.x;                                                                                    \
                f_ri = row_item(P, f_it < P.num_row_items ? f_it : f_it - gridDim.x);                                 \
                f_i0 = f_ri.i_run0;                                                                                   \
            }                                                                                                         \
        } while (0)
        if (f_it < P.num_row_items) {
            uint4 fr[ProductTileShape<HD, DWL>::NREGS];
            SA_ROW2_LOAD(fr);
            SA_ROW2_FORM(fr);
        }
        int flush_lo = 0;
        uint32_t n_units = 0;
        for (long it = blockIdx.x; it < P.num_row_items; it += gridDim.x) {
            const RowItem ri = row_item(P, it);
            for (int i0 = ri.i_run0, uidx = 0; i0 < ri.i_run1; i0 += QPT, ++uidx, ++n_units) {
                {
                    // the next unit's operands (always some unit's rows, so that the loop has one shape); both groups
                    // meet first: the staging buffer about to be rewritten was read by both in the unit before last
                    uint4 fr[ProductTileShape<HD, DWL>::NREGS];
                    SA_ROW2_LOAD(fr);
                    named_barrier_sync(5, 256);
                    if (f_it < P.num_row_items) {
                        mbar_wait(B.stat_empty, n_units & 1, wctx, 37);      // this unit's last S / dP MMAs have read A and C
                        SA_ROW2_FORM(fr);
                    }
                }
                const int i = i0 + qq;
                const int kb = i + p.halo2 - dlt;
                const bool row_valid = (i < p.N) && (dlt < p.w2) && (kb >= 0);
                const int ic = min(i, p.N - 1), kc = min(max(kb, 0), p.n2 - 1);      // rows that exist (queries past the end are not stored)
                const __nv_bfloat16* q_row = q + ri.b * p.q.b + (long)ic * p.q.n + ri.h * p.q.h + cbase;
                const __nv_bfloat16* do_row = d_o + ri.b * p.d_o.b + (long)ic * p.d_o.n + ri.h * p.d_o.h + cbase;
                const __nv_bfloat16* k2_row = k2 + ri.b * p.k2.b + (long)kc * p.k2.n + ri.hk * p.k2.h + cbase;
                const long bh = (long)ri.b * p.H + ri.h;
                const int kb_max = min(i0 + QPT, p.N) - 1 + p.halo2;
                const int own0 = ri.i_run0 + p.halo2;                        // first row owned by this run
                if (uidx == 0) flush_lo = max(0, own0 - (p.w2 - 1));
                const int slot = row_valid ? kb % max(ring_rows, 1) : 0;
                __nv_bfloat16* dq_out = dq == nullptr ? nullptr : dq + ri.b * p.dq.b + (long)i0 * p.dq.n + ri.h * p.dq.h + cbase;
                const uint8_t* stg = nullptr;
                if constexpr (STAGE) stg = stage_base + (n_units & 1) * kStageBuf;
                const int wrow_k2 = qq + DW - 1 - dlt;                       // this lane's K2 row inside the unit's window
                mbar_wait(B.acc_ready, n_units & 1, wctx, 31);
                if ((warp & 3) == 0) SA_TR(3 + grp, 60);
                tc_fence_after();
                SA_PROF_T0(t_epi);
                // U and G leave tensor memory at once, as packed 16-bit pairs held in registers (half the group's columns
                // of both, 64 registers), and the accumulators are handed back to the MMA issuer before any of the sums
                // below: those take several thousand cycles per unit, during which the next unit's accumulating MMAs
                // would otherwise stand still.  The rounding is that of the results themselves (one 16-bit rounding
                // of every addend, before sums of at most w2 of them).
                // A warp holds the 32 deltas of one query (or the 16 deltas of two): within a query the lanes own distinct
                // K2 rows.  In phase ph warp w works on column chunk (w + ph) % 4 of the group's half, so no two warps
                // touch the same ring columns at the same time; register slot ph holds that chunk.  Rows that are not
                // valid have P = dS = 0, hence exact zeros in U and G: they need no masking in the sums.
                uint32_t gp[NPHG][CW / 2], up[NPHG][CW / 2];
#pragma unroll
                for (int ph = 0; ph < NPHG; ++ph) {
                    const int c = ((wq + ph) & 3) * CW;
                    uint32_t g[CW], u[CW];
                    if constexpr (CW == 16) {
                        tmem_ld16(tm_g + lane_addr + cbase + c, g);
                        tmem_ld16(tm_u + lane_addr + cbase + c, u);
                    } else {
                        tmem_ld8(tm_g + lane_addr + cbase + c, g);
                        tmem_ld8(tm_u + lane_addr + cbase + c, u);
                    }
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < CW / 2; ++e) {
                        gp[ph][e] = El<false>::pack(__uint_as_float(g[2 * e]), __uint_as_float(g[2 * e + 1]));
                        up[ph][e] = El<false>::pack(__uint_as_float(u[2 * e]), __uint_as_float(u[2 * e + 1]));
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(B.acc_free);        // the next unit's accumulating MMAs may start
                if ((warp & 3) == 0) SA_TR(3 + grp, 61);
                // ---- dV2 from U
                if (need_kv2) {
#pragma unroll
                    for (int ph = 0; ph < NPHG; ++ph) {
                        const int c = ((wq + ph) & 3) * CW;
                        uint32_t ow[CW / 2];
                        if constexpr (STAGE) load_bf16_words<CW>((const __nv_bfloat16*)(stg + (QPT + qq) * HD * 2) + cbase + c, ow);
                        else load_bf16_words<CW>(do_row + c, ow);
#pragma unroll
                        for (int turn = 0; turn < (TWO_Q ? 2 : 1); ++turn) {
                            // with two queries in a warp, lanes (q, delta) and (q + 1, delta + 1) own the same row: the halves take turns
                            if (row_valid && (!TWO_Q || (lane >> 4) == turn)) {
                                float2* rv = (float2*)(ring_v + ring_index<HD>(slot, cbase + c));
#pragma unroll
                                for (int e = 0; e < CW / 2; ++e)
                                    rv[e] = __ffma2_rn(make_float2(El<false>::lo(up[ph][e]), El<false>::hi(up[ph][e])),
                                                       make_float2(E::lo(ow[e]), E::hi(ow[e])), rv[e]);
                            }
                            if (TWO_Q) __syncwarp();
                        }
                        named_barrier_sync(3 + grp, 128);
                    }
                }
                if ((warp & 3) == 0) SA_TR(3 + grp, 62);
                // ---- dQ and dK2 from G
#pragma unroll
                for (int ph = 0; ph < NPHG; ++ph) {
                    const int c = ((wq + ph) & 3) * CW;
                    uint32_t qw[CW / 2], xw[CW / 2];
                    if constexpr (STAGE) {
                        load_bf16_words<CW>((const __nv_bfloat16*)(stg + qq * HD * 2) + cbase + c, qw);
                        load_bf16_words<CW>((const __nv_bfloat16*)(stg + 2 * QPT * HD * 2 + wrow_k2 * K2PITCH) + cbase + c, xw);
                    } else {
                        load_bf16_words<CW>(q_row + c, qw);
                        load_bf16_words<CW>(k2_row + c, xw);
                    }
                    if (dq != nullptr) {
                        float v[CW];
#pragma unroll
                        for (int e = 0; e < CW; e += 2) {
                            float2 x2 = make_float2(E::lo(xw[e >> 1]), E::hi(xw[e >> 1]));
                            if (BIAS) x2 = __fadd2_rn(x2, make_float2(p.k2_bias, p.k2_bias));
                            const float2 t = __fmul2_rn(make_float2(El<false>::lo(gp[ph][e >> 1]), El<false>::hi(gp[ph][e >> 1])), x2);
                            v[e] = t.x;
                            v[e + 1] = t.y;
                        }
                        if constexpr (!TWO_Q) {
                            const float tot = warp_transpose_reduce<CW>(v, lane) * p.scale;
                            if (WPQ == 1) {
                                if (lane < CW && i0 + wq < p.N) E::st(&dq_out[(long)wq * p.dq.n + c + lane], tot);
                            } else if (lane < CW) {
                                dq_part[wq * HALF + c + lane] = tot;
                            }
                        } else {
                            // each half warp holds the 16 deltas of one query
                            const int qh = wq * 2 + (lane >> 4);
                            const float tot = half_warp_transpose_reduce<CW>(v, lane) * p.scale;
                            if ((lane & 15) < CW && i0 + qh < p.N) E::st(&dq_out[(long)qh * p.dq.n + c + (lane & 15)], tot);
                        }
                    }
#pragma unroll
                    for (int turn = 0; turn < (TWO_Q ? 2 : 1); ++turn) {
                        if (need_kv2 && row_valid && (!TWO_Q || (lane >> 4) == turn)) {
                            float2* rk = (float2*)(ring_k + ring_index<HD>(slot, cbase + c));
#pragma unroll
                            for (int e = 0; e < CW / 2; ++e)
                                rk[e] = __ffma2_rn(make_float2(El<false>::lo(gp[ph][e]), El<false>::hi(gp[ph][e])),
                                                   make_float2(E::lo(qw[e]), E::hi(qw[e])), rk[e]);
                        }
                        if (TWO_Q) __syncwarp();
                    }
                    named_barrier_sync(3 + grp, 128);
                }
                if ((warp & 3) == 0) SA_TR(3 + grp, 65);
                if (WPQ > 1 && dq != nullptr) {
                    // a query spans WPQ warps: add their partial rows (the last phase ended with a barrier)
                    for (int idx = row; idx < QPT * HALF; idx += 128) {
                        const int q2 = idx / HALF, col = idx % HALF;
                        float a = 0.f;
#pragma unroll
                        for (int w = 0; w < WPQ; ++w) a += dq_part[(q2 * WPQ + w) * HALF + col];
                        if (i0 + q2 < p.N) E::st(&dq_out[(long)q2 * p.dq.n + col], a);
                    }
                    named_barrier_sync(3 + grp, 128);     // before the next unit overwrites the partial rows
                }
                if (need_kv2 && ring_rows > 0) {
                    // rows no later query of the run reaches are final: move them to the workspace, clear the slots.
                    // One row per warp and turn; lanes 0-15 move the group's dK2 columns, lanes 16-31 its dV2 columns.
                    const bool last_unit = i0 + QPT >= ri.i_run1;
                    const int f_hi = last_unit ? kb_max + 1 : max(0, i0 + QPT + p.halo2 - (p.w2 - 1));
                    const bool is_v = lane >= 16;
                    float* ring = is_v ? ring_v : ring_k;
                    float* ws_full = is_v ? P.ws_full_v2 : P.ws_full_k2;
                    float* ws_head = is_v ? P.ws_head_v2 : P.ws_head_k2;
                    const float mult = is_v ? 1.f : p.scale;                 // the rings hold unscaled sums
                    for (int kbf = flush_lo + (row >> 5); kbf < f_hi; kbf += 4) {
                        const int fslot = kbf % ring_rows;
                        float* dst = (kbf >= own0) ? ws_full + (bh * p.N + (kbf - p.halo2)) * HD
                                                   : ws_head + ((bh * P.num_runs + ri.run) * (p.w2 - 1) + (kbf - (own0 - (p.w2 - 1)))) * HD;
                        float* src = ring + ring_index<HD>(fslot, 0);
                        const int d = cbase + (lane & 15) * 4;
                        if ((lane & 15) * 4 < HALF) {
                            *(float4*)(dst + d) = make_float4(src[d] * mult, src[d + 1] * mult, src[d + 2] * mult, src[d + 3] * mult);
                            src[d] = 0.f;
                            src[d + 1] = 0.f;
                            src[d + 2] = 0.f;
                            src[d + 3] = 0.f;
                        }
                    }
                    flush_lo = max(flush_lo, f_hi);
                    named_barrier_sync(3 + grp, 128);     // cleared slots are visible before the next unit's updates
                }
                SA_PROF_ADD(44 + grp, t_epi);
                if ((warp & 3) == 0) SA_TR(3 + grp, 66);
            }
        }
    } else if (warp == 16) {
        // ---------------------------------------------------------------- MMA issuer of the S / dP tiles.  Two warps
        // issue MMAs: this one S and dP, warp 17 the accumulating U and G.  One warp alone spends as long on the
        // scalar work between two batches (barriers, descriptors) as the tensor cores need for a batch, and its
        // issue queue is short, so the tensor cores would idle through that work; with two issuers one is always
        // queued up.  The only order the two must keep is on an S / dP buffer: tile t + 2 overwrites what the
        // accumulating MMAs of tile t read (buf_free, completed by the tensor cores themselves).
        reg_dealloc<SA_R2_REST>();
        {
            const uint32_t leader = elect_one();      // the whole warp runs the loop; one lane issues
            uint32_t g_base = 0, n_units = 0;
            const uint32_t idesc_full = make_idesc(128, kStreamRows, false, false, F16);
            const uint32_t a_s = smem_base + L::kStat0, c_s = smem_base + L::kStat1;
            for (long it = blockIdx.x; it < P.num_row_items; it += gridDim.x) {
                const RowItem ri = row_item(P, it);
                for (int i0 = ri.i_run0; i0 < ri.i_run1; i0 += QPT, ++n_units) {
                    const RowUnit ru = row_unit(P, i0);
                    SA_TR(0, 1);
                    mbar_wait(B.stat_full, n_units & 1, wctx, 32);      // A, C formed
                    SA_TR(0, 2);
                    tc_fence_after();
                    for (int t = 0; t < ru.nt; ++t) {
                        const uint32_t g = g_base + t;
                        const int stage = (int)(g % NS), b = g & 1;
                        const int width = (t == ru.nt - 1) ? ru.last_width : kStreamRows;
                        const uint32_t k1_t = smem_base + L::kStream + stage * 2 * L::kSmallTile, v1_t = k1_t + L::kSmallTile;
                        mbar_wait(&B.st_full[stage], (g / NS) & 1, wctx, 33);
                        // the accumulating MMAs of the tile that used this buffer before (two tiles back) have read its P and dS
                        if (g >= 2) mbar_wait(&buf_free[b], ((g >> 1) - 1) & 1, wctx, 39);
                        SA_TR(0, 3);
                        tc_fence_after();
                        issue_sdp<HD>(leader, tm_s[b], tm_dp[b], a_s, c_s, k1_t, v1_t, width == kStreamRows ? idesc_full : make_idesc(128, width, false, false, F16));
                        tc_commit(leader, &B.sdp_ready[b]);
                        if (t == ru.nt - 1) tc_commit(leader, B.stat_empty);     // A and C may be overwritten
                        SA_TR(0, 4);
                    }
                    g_base += ru.nt;
                }
            }
        }
        __syncwarp();
    } else if (warp == 17) {
        // ---------------------------------------------------------------- MMA issuer of the accumulating U and G
        reg_dealloc<SA_R2_REST>();
        {
            const uint32_t leader = elect_one();
            uint32_t g_base = 0, n_units = 0;
            for (long it = blockIdx.x; it < P.num_row_items; it += gridDim.x) {
                const RowItem ri = row_item(P, it);
                for (int i0 = ri.i_run0; i0 < ri.i_run1; i0 += QPT, ++n_units) {
                    const RowUnit ru = row_unit(P, i0);
                    for (int tp = 0; tp < ru.nt; ++tp) {
                        const uint32_t g = g_base + tp;
                        const int stage = (int)(g % NS), b = g & 1;
                        const int width = (tp == ru.nt - 1) ? ru.last_width : kStreamRows;
                        const uint32_t k1_t = smem_base + L::kStream + stage * 2 * L::kSmallTile, v1_t = k1_t + L::kSmallTile;
                        mbar_wait(&B.pds_ready[b], (g >> 1) & 1, wctx, 34);
                        SA_TR(5, 5);
                        // the previous unit's U and G have been read out by the epilogue groups
                        if (tp == 0 && n_units > 0) { mbar_wait(B.acc_free, (n_units - 1) & 1, wctx, 38); SA_TR(5, 6); }
                        tc_fence_after();
                        // U += P V1-tile ; G += dS K1-tile
                        issue_acc<HD, true, F16>(leader, tm_u, tm_g, tm_s[b], tm_dp[b], k1_t, v1_t, width / 16, tp > 0);
                        tc_commit(leader, &buf_free[b]);
                        tc_commit(leader, &B.st_empty[stage]);
                        SA_TR(5, 7);
                    }
                    tc_commit(leader, B.acc_ready);
                    g_base += ru.nt;
                }
            }
        }
    } else if (warp == 18) {
        // ---------------------------------------------------------------- TMA: streamed K1 / V1 tiles
        reg_dealloc<SA_R2_REST>();
        if (lane == 0) {
            prefetch_tensormap(&map_k1);
            prefetch_tensormap(&map_v1);
            uint32_t g = 0;
            for (long it = blockIdx.x; it < P.num_row_items; it += gridDim.x) {
                const RowItem ri = row_item(P, it);
                for (int i0 = ri.i_run0; i0 < ri.i_run1; i0 += QPT) {
                    const RowUnit ru = row_unit(P, i0);
                    for (int t = 0; t < ru.nt; ++t, ++g) {
                        const int stage = (int)(g % NS);
                        const int r0 = ru.col_start + t * kStreamRows;
                        uint8_t* k1_t = smem + L::kStream + stage * 2 * L::kSmallTile;
                        uint8_t* v1_t = k1_t + L::kSmallTile;
                        mbar_wait(&B.st_empty[stage], ((g / NS) & 1) ^ 1, wctx, 35);
                        mbar_arrive_expect_tx(&B.st_full[stage], 2 * L::kSmallTile);
#pragma unroll
                        for (int sl = 0; sl < L::kSlabs; ++sl) {
                            tma_load_4d(k1_t + sl * L::kSmallSlab, &map_k1, &B.st_full[stage], sl * 64, r0, ri.hk, ri.b);
                            tma_load_4d(v1_t + sl * L::kSmallSlab, &map_v1, &B.st_full[stage], sl * 64, r0, ri.hk, ri.b);
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else {
        reg_dealloc<SA_R2_REST>();
    }
    tc_fence_before();
    __syncthreads();
    SA_PROF_LIFE(t_life);
    if (warp == 16) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------------------------------------
// 4. dK2 / dV2 from the fp32 partials: sum over the query heads of a group, add the head partials of
//    the runs that start within w2-1 queries after the row, convert to bf16.
// ------------------------------------------------------------------------------------------------
template <bool F16>
__global__ void __launch_bounds__(256)
kv2_reduce_kernel(BwdTcParams P, __nv_bfloat16* __restrict__ dk2, __nv_bfloat16* __restrict__ dv2) {
    const KParams& p = P.k;
    const int HD = p.D;
    const int cpr = HD / 4;                               // threads per row: four columns (16 bytes of fp32) each
    const long total = (long)p.B * p.n2 * p.Hkv * cpr;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int d = (int)(idx % cpr) * 4;
    const int hk = (int)((idx / cpr) % p.Hkv);
    const int kb = (int)((idx / cpr / p.Hkv) % p.n2);
    const int b = (int)(idx / cpr / p.Hkv / p.n2);
    const int runq = P.units_per_run * (128 >> P.dw_log2);
    const int ip = kb - p.halo2;                          // the query aligned with this row (may be negative)
    // runs r with  r*runq in [ip + 1, ip + w2 - 1]
    int r_lo = (ip + 1 <= 0) ? 0 : (ip + 1 + runq - 1) / runq;
    int r_hi = (ip + p.w2 - 1 < 0) ? -1 : (ip + p.w2 - 1) / runq;
    if (r_hi > P.num_runs - 1) r_hi = P.num_runs - 1;
    float4 ak = make_float4(0.f, 0.f, 0.f, 0.f), av = make_float4(0.f, 0.f, 0.f, 0.f);
    auto add4 = [](float4& a, const float4 t) { a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w; };
    for (int hq = 0; hq < p.G; ++hq) {
        const int h = hk * p.G + hq;
        const long bh = (long)b * p.H + h;
        if (ip >= 0 && ip < p.N) {
            const long o = (bh * p.N + ip) * HD + d;
            if (dk2) add4(ak, __ldcs((const float4*)(P.ws_full_k2 + o)));     // read once: streaming loads
            if (dv2) add4(av, __ldcs((const float4*)(P.ws_full_v2 + o)));
        }
        for (int r = r_lo; r <= r_hi; ++r) {
            const int slot = kb - (r * runq + p.halo2 - (p.w2 - 1));
            const long o = ((bh * P.num_runs + r) * (p.w2 - 1) + slot) * HD + d;
            if (dk2) add4(ak, *(const float4*)(P.ws_head_k2 + o));
            if (dv2) add4(av, *(const float4*)(P.ws_head_v2 + o));
        }
    }
    if (dk2) {
        uint32_t* dst = (uint32_t*)(dk2 + b * p.dk2.b + (long)kb * p.dk2.n + hk * p.dk2.h + d);
        dst[0] = ptx::El<F16>::pack(ak.x, ak.y);
        dst[1] = ptx::El<F16>::pack(ak.z, ak.w);
    }
    if (dv2) {
        uint32_t* dst = (uint32_t*)(dv2 + b * p.dv2.b + (long)kb * p.dv2.n + hk * p.dv2.h + d);
        dst[0] = ptx::El<F16>::pack(av.x, av.y);
        dst[1] = ptx::El<F16>::pack(av.z, av.w);
    }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
struct BwdPlan {
    int dw_log2, qpt, units_per_run, num_runs;
    size_t off_lse2, off_delta, off_full_k2, off_full_v2, off_head_k2, off_head_v2, total;
};

// `sm_count`: multiprocessors of the device the launch will run on (the run length is chosen so that
// there are at least two runs per multiprocessor).
inline BwdPlan bwd_plan(const KParams& k, int sm_count) {
    BwdPlan pl{};
    int l = 0;
    while ((1 << l) < k.w2) ++l;
    pl.dw_log2 = l;
    pl.qpt = 128 >> l;
    const int units = (k.N + pl.qpt - 1) / pl.qpt;
    int upr = 16;
    while (upr > 1 && (long)k.B * k.H * ((units + upr - 1) / upr) < 2 * (long)sm_count) upr >>= 1;
    pl.units_per_run = upr;
    pl.num_runs = (units + upr - 1) / upr;
    auto align = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t bhn = (size_t)k.B * k.H * k.N;
    size_t off = 0;
    pl.off_lse2 = off; off = align(off + bhn * 4);
    pl.off_delta = off; off = align(off + bhn * 4);
    pl.off_full_k2 = off; off = align(off + bhn * k.D * 4);
    pl.off_full_v2 = off; off = align(off + bhn * k.D * 4);
    const size_t head = (size_t)k.B * k.H * pl.num_runs * (size_t)(k.w2 > 1 ? k.w2 - 1 : 1) * k.D * 4;
    pl.off_head_k2 = off; off = align(off + head);
    pl.off_head_v2 = off; off = align(off + head);
    pl.total = off;
    return pl;
}

inline size_t bwd_workspace_bytes(const KParams& k, int sm_count) { return bwd_plan(k, sm_count).total; }

typedef bool (*MakeMapFn)(CUtensorMap*, const void*, int, int, int, int, const sa_strides&, int, bool);

// Returns an sa_status, or -1 when the tensor-core backward does not cover the problem.  F16: the tensors are
// IEEE half instead of bf16.
template <bool F16>
int launch_bwd_t(const KParams& k, const void* q, const void* k1, const void* k2, const void* v1, const void* v2,
                      const void* o, const float* lse, const void* d_o, void* dq, void* dk1, void* dk2, void* dv1,
                      void* dv2, uint8_t* workspace, DeviceStatus* status, cudaStream_t st, int* nlaunch, MakeMapFn make_map,
                      int sm_count, uint64_t wait_limit_ns) {
    const BwdPlan pl = bwd_plan(k, sm_count);
    BwdTcParams P{};
    P.k = k;
    P.dw_log2 = pl.dw_log2;
    P.num_jtiles = (k.n1 + 127) / 128;
    P.num_col_items = (long)k.B * k.Hkv * P.num_jtiles;
    P.units_per_run = pl.units_per_run;
    P.num_runs = pl.num_runs;
    P.num_row_items = (long)k.B * k.H * pl.num_runs;
    float* lse2 = (float*)(workspace + pl.off_lse2);
    float* delta = (float*)(workspace + pl.off_delta);
    P.lse2 = lse2;
    P.delta = delta;
    P.ws_full_k2 = (float*)(workspace + pl.off_full_k2);
    P.ws_full_v2 = (float*)(workspace + pl.off_full_v2);
    P.ws_head_k2 = (float*)(workspace + pl.off_head_k2);
    P.ws_head_v2 = (float*)(workspace + pl.off_head_v2);
    P.status = status;
    P.wait_limit_ns = wait_limit_ns;
    auto bf = [](const void* x) { return (const __nv_bfloat16*)x; };

    const long rows = (long)k.B * k.H * k.N;
    prep_kernel<F16><<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(k, bf(o), bf(d_o), lse, lse2, delta);
    ++*nlaunch;

    const bool has_bias = k.k2_bias != 0.f || k.v2_bias != 0.f;     // selects the kernels that carry the bias adds
    if (dk1 || dv1) {
        CUtensorMap m1, m2;
        if (!make_map(&m1, k1, k.B, k.n1, k.Hkv, k.D, k.k1, 128, F16)) return SA_ERR_BAD_STRIDE;
        if (!make_map(&m2, v1, k.B, k.n1, k.Hkv, k.D, k.v1, 128, F16)) return SA_ERR_BAD_STRIDE;
        const long grid = P.num_col_items < sm_count ? P.num_col_items : sm_count;
        if (k.D == 128) {
            auto kern = has_bias ? bwd_col_kernel<128, true, F16> : bwd_col_kernel<128, false, F16>;
            using LC = ColSmem<128>;
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LC::kAlloc) != cudaSuccess)
                return SA_ERR_LAUNCH;
            kern<<<(unsigned)grid, kColThreads, LC::kAlloc, st>>>(P, m1, m2, bf(q), bf(k2), bf(v2), bf(d_o),
                                                                             (__nv_bfloat16*)dk1, (__nv_bfloat16*)dv1);
        } else {
            auto kern = has_bias ? bwd_col_kernel<64, true, F16> : bwd_col_kernel<64, false, F16>;
            using LC = ColSmem<64>;
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LC::kAlloc) != cudaSuccess)
                return SA_ERR_LAUNCH;
            kern<<<(unsigned)grid, kColThreads, LC::kAlloc, st>>>(P, m1, m2, bf(q), bf(k2), bf(v2), bf(d_o),
                                                                            (__nv_bfloat16*)dk1, (__nv_bfloat16*)dv1);
        }
        ++*nlaunch;
    }
    if (dq || dk2 || dv2) {
        CUtensorMap m1, m2;
        if (!make_map(&m1, k1, k.B, k.n1, k.Hkv, k.D, k.k1, kStreamRows, F16)) return SA_ERR_BAD_STRIDE;
        if (!make_map(&m2, v1, k.B, k.n1, k.Hkv, k.D, k.v1, kStreamRows, F16)) return SA_ERR_BAD_STRIDE;
        const long grid = P.num_row_items < sm_count ? P.num_row_items : sm_count;
        const int need_kv2 = (dk2 || dv2) ? 1 : 0;
        // shared-memory ring of fp32 dK2/dV2 rows beside the tiles: with the 3-stage K1/V1 ring if it fits,
        // else with 2 stages, else none (partials then accumulate in the workspace)
        const int ring_want = (1 << pl.dw_log2) + pl.qpt;
        auto launch_row = [&](auto kern, int k_ring, int k_min, int max_dyn, int hd, int threads = kRowThreads, int extra = 0) -> bool {
            int ring_rows = ring_want;
            int smem = k_ring + 1024 + 2 * ring_rows * (hd + 2) * 4 + extra;
            if (!need_kv2 || smem > max_dyn) { ring_rows = 0; smem = k_ring + 1024 + extra; }
            if (smem < k_min) smem = k_min;
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, max_dyn) != cudaSuccess) return false;
            kern<<<(unsigned)grid, threads, smem, st>>>(P, m1, m2, bf(q), bf(k2), bf(v2), bf(d_o), (__nv_bfloat16*)dq,
                                                        need_kv2, ring_rows);
            return true;
        };
        bool ok;
        if (k.D == 128) {
            using L3 = BwdSmem<128, 3>;
            using L2 = BwdSmem<128, 2>;
            const bool fits3 = L3::kRing + 1024 + 2 * ring_want * 130 * 4 <= L3::kMaxDynamic;
            constexpr int kDqPart = 2048;     // partial dQ rows of the epilogue groups when a query spans two warps
            const bool fits2 = L2::kRing + 1024 + 2 * ring_want * 130 * 4 + kDqPart <= L2::kMaxDynamic;
            const bool fits3x = L3::kRing + 1024 + 2 * ring_want * 130 * 4 + kDqPart <= L3::kMaxDynamic;
            // (16 and 32 delta slots: two staging buffers of raw Q, dO and K2 rows behind the rings)
            const int stage5 = 2 * row2_stage_bytes(5, 128), stage4 = 2 * row2_stage_bytes(4, 128);
            const bool fits5 = L3::kRing + 1024 + 2 * ring_want * 130 * 4 + kDqPart + stage5 <= L3::kMaxDynamic;
            const bool fits4 = L3::kRing + 1024 + 2 * ring_want * 130 * 4 + kDqPart + stage4 <= L3::kMaxDynamic;
            if (pl.dw_log2 == 5 && (fits5 || !need_kv2))     // separate epilogue warpgroups
                ok = launch_row(has_bias ? bwd_row2_kernel<128, 5, 3, true, F16> : bwd_row2_kernel<128, 5, 3, false, F16>, L3::kRing, L3::kAlloc,
                                L3::kMaxDynamic, 128, kRow2Threads, kDqPart + stage5);
            else if (pl.dw_log2 == 4 && (fits4 || !need_kv2))
                ok = launch_row(has_bias ? bwd_row2_kernel<128, 4, 3, true, F16> : bwd_row2_kernel<128, 4, 3, false, F16>, L3::kRing, L3::kAlloc,
                                L3::kMaxDynamic, 128, kRow2Threads, kDqPart + stage4);
            else if (pl.dw_log2 == 6 && (fits3x || !need_kv2))
                ok = launch_row(has_bias ? bwd_row2_kernel<128, 6, 3, true, F16> : bwd_row2_kernel<128, 6, 3, false, F16>, L3::kRing, L3::kAlloc,
                                L3::kMaxDynamic, 128, kRow2Threads, kDqPart);
            else if (pl.dw_log2 == 6 && fits2)
                ok = launch_row(has_bias ? bwd_row2_kernel<128, 6, 2, true, F16> : bwd_row2_kernel<128, 6, 2, false, F16>, L2::kRing, L2::kAlloc,
                                L2::kMaxDynamic, 128, kRow2Threads, kDqPart);
            else if (pl.dw_log2 == 4)
                ok = launch_row(has_bias ? bwd_row_kernel<128, 3, true, true, F16> : bwd_row_kernel<128, 3, true, false, F16>, L3::kRing, L3::kAlloc, L3::kMaxDynamic, 128);
            else
                ok = (fits3 || !need_kv2) ? launch_row(has_bias ? bwd_row_kernel<128, 3, false, true, F16> : bwd_row_kernel<128, 3, false, false, F16>, L3::kRing, L3::kAlloc, L3::kMaxDynamic, 128)
                                          : launch_row(has_bias ? bwd_row_kernel<128, 2, false, true, F16> : bwd_row_kernel<128, 2, false, false, F16>, L2::kRing, L2::kAlloc, L2::kMaxDynamic, 128);
        } else {
            using L3 = BwdSmem<64, 3>;
            using L2 = BwdSmem<64, 2>;
            const bool fits3 = L3::kRing + 1024 + 2 * ring_want * 66 * 4 <= L3::kMaxDynamic;
            constexpr int kDqPart = 2048;     // (the kernel places the staging buffers 2048 bytes behind the rings)
            const int stage5 = 2 * row2_stage_bytes(5, 64), stage4 = 2 * row2_stage_bytes(4, 64);
            const int ring_bytes = 2 * ring_want * 66 * 4;
            const bool fits5 = L3::kRing + 1024 + ring_bytes + kDqPart + stage5 <= L3::kMaxDynamic;
            const bool fits4 = L3::kRing + 1024 + ring_bytes + kDqPart + stage4 <= L3::kMaxDynamic;
            const bool fits6 = L3::kRing + 1024 + ring_bytes + kDqPart <= L3::kMaxDynamic;
            if (pl.dw_log2 == 5 && (fits5 || !need_kv2))     // separate operand / epilogue warpgroups
                ok = launch_row(has_bias ? bwd_row2_kernel<64, 5, 3, true, F16> : bwd_row2_kernel<64, 5, 3, false, F16>, L3::kRing, L3::kAlloc,
                                L3::kMaxDynamic, 64, kRow2Threads, kDqPart + stage5);
            else if (pl.dw_log2 == 4 && (fits4 || !need_kv2))
                ok = launch_row(has_bias ? bwd_row2_kernel<64, 4, 3, true, F16> : bwd_row2_kernel<64, 4, 3, false, F16>, L3::kRing, L3::kAlloc,
                                L3::kMaxDynamic, 64, kRow2Threads, kDqPart + stage4);
            else if (pl.dw_log2 == 6 && (fits6 || !need_kv2))
                ok = launch_row(has_bias ? bwd_row2_kernel<64, 6, 3, true, F16> : bwd_row2_kernel<64, 6, 3, false, F16>, L3::kRing, L3::kAlloc,
                                L3::kMaxDynamic, 64, kRow2Threads, kDqPart);
            else if (pl.dw_log2 == 4)
                ok = launch_row(has_bias ? bwd_row_kernel<64, 3, true, true, F16> : bwd_row_kernel<64, 3, true, false, F16>, L3::kRing, L3::kAlloc, L3::kMaxDynamic, 64);
            else
                ok = (fits3 || !need_kv2) ? launch_row(has_bias ? bwd_row_kernel<64, 3, false, true, F16> : bwd_row_kernel<64, 3, false, false, F16>, L3::kRing, L3::kAlloc, L3::kMaxDynamic, 64)
                                          : launch_row(has_bias ? bwd_row_kernel<64, 2, false, true, F16> : bwd_row_kernel<64, 2, false, false, F16>, L2::kRing, L2::kAlloc, L2::kMaxDynamic, 64);
        }
        if (!ok) return SA_ERR_LAUNCH;
        ++*nlaunch;
        if (need_kv2) {
            const long total = (long)k.B * k.n2 * k.Hkv * (k.D / 4);
            kv2_reduce_kernel<F16><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(P, (__nv_bfloat16*)dk2, (__nv_bfloat16*)dv2);
            ++*nlaunch;
        }
    }
    return cudaGetLastError() == cudaSuccess ? SA_OK : SA_ERR_LAUNCH;
}

// The two element types are compiled in translation units of their own (sa_tc_bwd_bf16.cu, sa_tc_bwd_f16.cu: the
// kernels of one type take minutes to compile, and the units build side by side); everywhere else the
// instantiations are only declared.
#ifndef SA_TC_BWD_INSTANTIATE
extern template int launch_bwd_t<false>(const KParams&, const void*, const void*, const void*, const void*, const void*, const void*,
                                        const float*, const void*, void*, void*, void*, void*, void*, uint8_t*, DeviceStatus*,
                                        cudaStream_t, int*, MakeMapFn, int, uint64_t);
extern template int launch_bwd_t<true>(const KParams&, const void*, const void*, const void*, const void*, const void*, const void*,
                                       const float*, const void*, void*, void*, void*, void*, void*, uint8_t*, DeviceStatus*,
                                       cudaStream_t, int*, MakeMapFn, int, uint64_t);
#endif

inline int launch_bwd(const KParams& k, const void* q, const void* k1, const void* k2, const void* v1, const void* v2,
                      const void* o, const float* lse, const void* d_o, void* dq, void* dk1, void* dk2, void* dv1,
                      void* dv2, uint8_t* workspace, DeviceStatus* status, cudaStream_t st, int* nlaunch, MakeMapFn make_map,
                      int sm_count, uint64_t wait_limit_ns, bool f16) {
    return f16 ? launch_bwd_t<true>(k, q, k1, k2, v1, v2, o, lse, d_o, dq, dk1, dk2, dv1, dv2, workspace, status, st, nlaunch,
                                    make_map, sm_count, wait_limit_ns)
               : launch_bwd_t<false>(k, q, k1, k2, v1, v2, o, lse, d_o, dq, dk1, dk2, dv1, dv2, workspace, status, st, nlaunch,
                                     make_map, sm_count, wait_limit_ns);
}

}  // namespace tc
}  // namespace sa
