// Thin inline-PTX wrappers for the sm_100a features the tensor-core kernels use: mbarriers with
// bounded waits, TMA tiled loads, tensor-memory allocation, tcgen05 MMA / load / store / commit,
// and the shared-memory and instruction descriptors of the tcgen05 MMA.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sa_common.cuh"

namespace sa {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ----------------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One probe of the barrier.  The suspend-time hint lets the hardware park the warp until the phase
// completes (it wakes at once when it does) instead of spinning through issue slots that the
// working warps of the same scheduler need.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}

// Shared by every wait of a block: once any wait has given up, all later waits return at once so
// that the block drains, frees its tensor memory and exits.  `status` points at the DeviceStatus
// word in the caller's workspace.
struct WaitCtx {
    volatile int* abort_flag;    // shared memory
    DeviceStatus* status;        // global memory
    uint64_t limit_ns;           // how long one wait may last before the block gives up
};

#ifdef SA_TRACE
// Trace builds only: block 0 records (clock, event) pairs per role; read back through sa_trace_read.
// (The buffers exist once per translation unit: build sa_api.cu alone with -DSA_TRACE
// -DSA_TC_BWD_INSTANTIATE, which instantiates the backward there too.  The same holds for -DSA_PROFILE.)
// The event counter of a role lives in a register of the recording warp (SA_TR_DECL in the scope of
// the role's code), so that recording costs one store and no load.
__device__ unsigned long long g_trace[16][2048];
__device__ int g_trace_n[16];
#define SA_TR_DECL() int tr_n_ = 0
#define SA_TR(role, ev)                                                                           \
    do {                                                                                          \
        if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && tr_n_ < 2048) {                         \
            sa::ptx::g_trace[role][tr_n_] = ((unsigned long long)clock64() << 8) | (unsigned)(ev); \
            sa::ptx::g_trace_n[role] = ++tr_n_;                                                   \
        }                                                                                         \
    } while (0)
#else
#define SA_TR_DECL() do { } while (0)
#define SA_TR(role, ev) do { } while (0)
#endif

#ifdef SA_PROFILE
// Profiling builds only: cycles block 0 spent in each wait site (indexed by the site id) and how
// often, read back through sa_prof_read.
__device__ unsigned long long g_prof_cycles[64];
__device__ unsigned long long g_prof_count[64];
#endif

#ifdef SA_PROFILE
#define SA_PROF_T0(name) const long long name = clock64()
#define SA_PROF_ADD(site, t0)                                                              \
    do {                                                                                   \
        if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) {                                  \
            atomicAdd(&sa::ptx::g_prof_cycles[(site) & 63], (unsigned long long)(clock64() - (t0))); \
            atomicAdd(&sa::ptx::g_prof_count[(site) & 63], 1ull);                          \
        }                                                                                  \
    } while (0)
// Lifetime of a block in cycles: site 62 = block 0, site 63 = the longest-lived block.
#define SA_PROF_LIFE(t0)                                                                   \
    do {                                                                                   \
        if (threadIdx.x == 0) {                                                            \
            const unsigned long long dt_ = (unsigned long long)(clock64() - (t0));         \
            if (blockIdx.x == 0) { sa::ptx::g_prof_cycles[62] = dt_; sa::ptx::g_prof_count[62] = 1; } \
            atomicMax(&sa::ptx::g_prof_cycles[63], dt_);                                   \
            sa::ptx::g_prof_count[63] = 1;                                                 \
        }                                                                                  \
    } while (0)
#else
#define SA_PROF_T0(name) do { } while (0)
#define SA_PROF_ADD(site, t0) do { } while (0)
#define SA_PROF_LIFE(t0) do { } while (0)
#endif

constexpr uint64_t kWaitLimitNs = 2000000000ull;   // default limit, 2 s: far beyond any legitimate wait in these kernels

// Waits for the phase with the given parity.  Bounded: after ctx.limit_ns it records where it gave
// up, raises the block's abort flag and returns false.
__device__ __forceinline__ bool mbar_wait_impl(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, int where);
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, int where) {
#ifdef SA_PROFILE
    const long long t0 = clock64();
    const bool r = mbar_wait_impl(bar, parity, ctx, where);
    if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) {
        atomicAdd(&g_prof_cycles[where & 63], (unsigned long long)(clock64() - t0));
        atomicAdd(&g_prof_count[where & 63], 1ull);
    }
    return r;
#else
    return mbar_wait_impl(bar, parity, ctx, where);
#endif
}
__device__ __forceinline__ bool mbar_wait_impl(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, int where) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*ctx.abort_flag) return false;
        if ((++spins & 0xff) == 0) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > ctx.limit_ns) {
                *ctx.abort_flag = 1;
                if (atomicCAS(&ctx.status->code, 0, (int)SA_ERR_DEVICE_TIMEOUT) == 0) {
                    ctx.status->where = where;
                    ctx.status->block = (int)blockIdx.x;
                }
                __threadfence();
                return false;
            }
        }
    }
}

// Per-warpgroup register re-allocation: the data-movement warps give registers up, the softmax /
// epilogue warps take them.  N is a multiple of 8; all four warps of an aligned warpgroup execute it.
template <int N>
__device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// Arrives without waiting: the barrier completes once `nthreads` threads have arrived or synchronised on it.
__device__ __forceinline__ void named_barrier_arrive(int id, int nthreads) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ----------------------------------------------------------------------------------------------
// TMA (tiled, 4-d, global -> shared, completion on an mbarrier)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// Coordinates are (d, row, head, batch); d * 2 bytes must be a multiple of 16.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
        : "memory");
}

// ----------------------------------------------------------------------------------------------
// Tensor memory
// ----------------------------------------------------------------------------------------------
// Allocates `ncols` (power of two, 32..512) columns; the base address is written to *smem_dst.
// Must be executed by one full warp.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// The mbarrier receives one arrival once every tcgen05 operation this thread issued before has
// completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// The same, issued by the elected lane of a convergent warp only.
__device__ __forceinline__ void tc_commit(uint32_t leader, uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(smem_u32(bar)), "r"(leader)
        : "memory");
}

// Each lane of the warp reads 8 (16, 32) consecutive 32-bit columns of its own tensor-memory lane
// (lane = 32 * (warp % 4) + laneid, encoded in bits 16.. of `addr`).
__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(addr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(addr)
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t addr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(addr), "r"(v[0]), "r"(v[1]),
                 "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05.mma descriptors (bf16 operands, fp32 accumulate, 128-byte swizzled shared-memory tiles)
//
// A shared-memory operand tile is stored as rows of 128 bytes (64 bf16), eight rows to a 1024-byte
// swizzle atom, the 16-byte chunk index of a row XOR-ed with (row & 7): exactly what a TMA load with
// CU_TENSOR_MAP_SWIZZLE_128B of a {64, rows} box produces.  A tile wider than 64 elements is a
// sequence of such [rows x 64] slabs.
//  * "K-major" use: the 64 elements of a row run along the MMA's K dimension, the rows along M/N.
//  * "MN-major" use: the 64 elements of a row run along M/N, the rows along K.
// The same bytes serve both uses; only the descriptor differs.
// ----------------------------------------------------------------------------------------------
constexpr uint64_t kDescSwizzle128 = 2ull << 61;
constexpr uint64_t kDescVersion = 1ull << 46;

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | kDescVersion | kDescSwizzle128;
}
// K-major: start of a [rows x 64] slab plus k * 32 bytes for the k-th 16-element K step; 8-row
// groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t slab_addr, int kstep_in_slab) {
    return make_smem_desc(slab_addr + (uint32_t)kstep_in_slab * 32u, 16u, 1024u);
}
// MN-major: `addr` is the first of the 16 rows (K) of this step; consecutive 64-element slabs along
// M/N are `slab_bytes` apart, 8-row K groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t slab_bytes) {
    return make_smem_desc(addr, slab_bytes, 1024u);
}

// Instruction descriptor: D fp32 (bits 4-5 = 1), A and B bf16 (bits 7-9, 10-12 = 1), optional
// MN-major A (bit 15) / B (bit 16), N >> 3 at bit 17, M >> 4 at bit 24.
// `f16`: both operands are IEEE half (format 0) instead of bf16 (format 1).
__host__ __device__ __forceinline__ uint32_t make_idesc(int m, int n, bool a_mn_major, bool b_mn_major, bool f16 = false) {
    const uint32_t fmt = f16 ? 0u : 1u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// The MMA-issuing warp runs its whole loop convergently (all 32 lanes wait on the barriers and
// compute the descriptors, which the compiler can then keep in uniform registers) and only the
// tcgen05 instructions themselves are predicated on one elected lane.  A loop executed by a single
// lane inside a divergent branch issues one MMA every ~90 cycles when other warps are busy; the
// convergent form sustains the tensor pipe's 64 cycles per 128x128x16 MMA.
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred;
}

// D[tmem] (+)= A[smem] * B[smem]       (issued by the lane whose `leader` is non-zero)
__device__ __forceinline__ void mma_ss(uint32_t leader, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate), "r"(leader)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]     (A: 128 lanes x K/2 columns, two bf16 per column)
__device__ __forceinline__ void mma_ts(uint32_t leader, uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate), "r"(leader)
        : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// max of three values in one instruction
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}


// bf16 pair held in a 32-bit word -> floats, by bit operations only (a register array reinterpreted
// through a pointer cast tends to be demoted to local memory).
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// The 16-bit element type of the tensor-core kernels: bf16 (F16 = false) or IEEE half (F16 = true).  The
// kernels move elements as raw 16-bit patterns (pointers are typed __nv_bfloat16 for their size only);
// everything that depends on the encoding goes through this struct.
template <bool F16>
struct El {
    // two floats -> one packed word (lo in the low half)
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t r;
        if constexpr (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
    static __device__ __forceinline__ float lo(uint32_t w) {
        if constexpr (F16) {
            float f;
            asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %1;\n\tcvt.f32.f16 %0, l;\n\t}" : "=f"(f) : "r"(w));
            return f;
        } else {
            return __uint_as_float(w << 16);
        }
    }
    static __device__ __forceinline__ float hi(uint32_t w) {
        if constexpr (F16) {
            float f;
            asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %1;\n\tcvt.f32.f16 %0, h;\n\t}" : "=f"(f) : "r"(w));
            return f;
        } else {
            return __uint_as_float(w & 0xffff0000u);
        }
    }
    // one element to / from its 16-bit slot
    static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) {
        if constexpr (F16) *reinterpret_cast<__half*>(p) = __float2half_rn(v);
        else *p = __float2bfloat16_rn(v);
    }
    static __device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) {      // two consecutive elements (4-byte aligned)
        const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
        return make_float2(lo(w), hi(w));
    }
    // elementwise product of two packed pairs, rounded once (exact: the product of two such significands fits fp32)
    static __device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
        uint32_t r;
        if constexpr (F16) asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        else asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
};

// Loads N consecutive bf16 values (N a multiple of 8, 16-byte aligned) as N/2 packed words.
template <int N>
__device__ __forceinline__ void load_bf16_words(const __nv_bfloat16* src, uint32_t (&w)[N / 2]) {
#pragma unroll
    for (int x = 0; x < N / 8; ++x) {
        const uint4 t = ((const uint4*)src)[x];
        w[4 * x] = t.x;
        w[4 * x + 1] = t.y;
        w[4 * x + 2] = t.z;
        w[4 * x + 3] = t.w;
    }
}

// Product of two chunks of 8 elements, x * (y + bias), computed in fp32 and rounded once.
template <bool F16 = false>
__device__ __forceinline__ uint4 mul_chunk(const uint4& xa, const uint4& ya, float bias) {
    using E = El<F16>;
    const uint32_t xw[4] = {xa.x, xa.y, xa.z, xa.w}, yw[4] = {ya.x, ya.y, ya.z, ya.w};
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
        w[e] = E::pack(E::lo(xw[e]) * (E::lo(yw[e]) + bias), E::hi(xw[e]) * (E::hi(yw[e]) + bias));
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// With bias == 0 the product of two bf16 values rounded to bf16 is exactly what the packed bf16
// multiply returns (the product of two 8-bit significands is exact in fp32, one rounding follows).
__device__ __forceinline__ uint32_t hmul2_bf16(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
template <bool F16 = false>
__device__ __forceinline__ uint4 mul_chunk_nobias(const uint4& xa, const uint4& ya) {
    using E = El<F16>;
    return make_uint4(E::mul2(xa.x, ya.x), E::mul2(xa.y, ya.y), E::mul2(xa.z, ya.z), E::mul2(xa.w, ya.w));
}

// BIAS = false: the bias is known to be zero (the common case) and the exact packed-bf16 product is used.
template <int HD, int NROWS, int NTHREADS, bool BIAS, bool F16 = false, int MAXBATCH = 4>
__device__ __forceinline__ void form_product_tile(uint8_t* tile, int slab_bytes, int t, long rho0, int dw_log2, int n_q,
                                                  int w2, int halo2, const __nv_bfloat16* x, int64_t xs,
                                                  const __nv_bfloat16* y, int64_t ys, float bias) {
    constexpr int C = HD / 8;
    constexpr int RPP = NTHREADS / C;            // rows per pass
    constexpr int PASSES = NROWS / RPP;
    static_assert(NROWS % RPP == 0, "tile rows must be a multiple of the rows formed per pass");
    constexpr int BATCH = PASSES < MAXBATCH ? PASSES : MAXBATCH;    // loads in flight per thread: 2 * BATCH 16-byte loads
    static_assert(PASSES % BATCH == 0, "passes must split into whole batches");
    const int c = t % C;
    const int dmask = (1 << dw_log2) - 1;
#pragma unroll 1
    for (int k0 = 0; k0 < PASSES; k0 += BATCH) {
        uint4 xa[BATCH], ya[BATCH];
        bool ok[BATCH];
#pragma unroll
        for (int k = 0; k < BATCH; ++k) {         // loads first: one memory round trip per batch
            const long rho = rho0 + t / C + (k0 + k) * RPP;
            const int i = (int)(rho >> dw_log2);
            const int dlt = (int)(rho & dmask);
            const int kb = i + halo2 - dlt;
            ok[k] = i < n_q && dlt < w2 && kb >= 0;
            if (ok[k]) {                          // read-only path: the rows are re-read by neighbouring tiles
                xa[k] = __ldg((const uint4*)(x + (int64_t)i * xs) + c);
                ya[k] = __ldg((const uint4*)(y + (int64_t)kb * ys) + c);
            }
        }
#pragma unroll
        for (int k = 0; k < BATCH; ++k) {
            const int r = t / C + (k0 + k) * RPP;
            uint4 out = make_uint4(0, 0, 0, 0);
            if (ok[k]) out = BIAS ? mul_chunk<F16>(xa[k], ya[k], bias) : mul_chunk_nobias<F16>(xa[k], ya[k]);
            *(uint4*)(tile + (c >> 3) * slab_bytes + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = out;
        }
    }
}



// Same result as form_product_tile for a 128-row tile whose queries are aligned to it (DW = 1 << DWLOG
// delta slots per query, 128 / DW queries per tile), but every y row (K2 or V2) is loaded once and
// used for all the queries it pairs with: consecutive queries share all but one of their DW rows.
// Window row w (0 <= w < DW + nq - 1) is y row  kb = i0 + halo2 - (DW-1) + w ; it meets query x at
// delta = DW - 1 + x - w.  One round of loads per tile: NQ chunks of x and PASSES chunks of y.
// The work is split in two so that a caller can start the loads long before it may write the tile:
// load_product_tile_shared fills the registers, store_product_tile_shared multiplies and stores.
template <int HD, int DWLOG, int NTHREADS = 128>
struct ProductTileShape {
    static constexpr int C = HD / 8;
    static constexpr int RPP = NTHREADS / C;             // window rows per pass
    static constexpr int DW = 1 << DWLOG;
    static constexpr int NQ = 128 / DW;
    static constexpr int NWIN = DW + NQ - 1;
    static constexpr int PASSES = (NWIN + RPP - 1) / RPP;
    static constexpr int NREGS = NQ + PASSES;            // 16-byte registers per thread
};

template <int HD, int DWLOG, int NTHREADS = 128>
__device__ __forceinline__ void load_product_tile_shared(uint4* regs, int t, int i0, int n_q, int halo2, const __nv_bfloat16* x,
                                                         int64_t xs, const __nv_bfloat16* y, int64_t ys) {
    using S = ProductTileShape<HD, DWLOG, NTHREADS>;
    const int c = t % S::C, pr = t / S::C;
    const int kb_first = i0 + halo2 - (S::DW - 1);
#pragma unroll
    for (int q2 = 0; q2 < S::NQ; ++q2) {
        regs[q2] = make_uint4(0, 0, 0, 0);
        if (i0 + q2 < n_q) regs[q2] = __ldg((const uint4*)(x + (int64_t)(i0 + q2) * xs) + c);
    }
#pragma unroll
    for (int k = 0; k < S::PASSES; ++k) {
        const int w = pr + k * S::RPP;
        const int kb = kb_first + w;
        regs[S::NQ + k] = make_uint4(0, 0, 0, 0);
        // (rows past the end belong to queries past the end of the last tile: they must not be read, and a
        // zero row keeps the product with the zero query row an exact zero whatever lies behind the tensor)
        if (w < S::NWIN && kb >= 0 && kb < n_q + halo2) regs[S::NQ + k] = __ldg((const uint4*)(y + (int64_t)kb * ys) + c);
    }
}

template <int HD, int DWLOG, bool BIAS, bool F16 = false, int NTHREADS = 128>
__device__ __forceinline__ void store_product_tile_shared(uint8_t* tile, int slab_bytes, int t, int i0, int n_q, int w2, int halo2,
                                                          const uint4* regs, float bias) {
    using S = ProductTileShape<HD, DWLOG, NTHREADS>;
    constexpr int C = S::C, RPP = S::RPP, DW = S::DW, NQ = S::NQ, PASSES = S::PASSES;
    const int c = t % C, pr = t / C;
    const int kb_first = i0 + halo2 - (DW - 1);
    // Row r = q2 * DW + delta of the tile, delta = DW - 1 + q2 - w, w = pr + k * RPP.  DW and RPP are
    // multiples of 8, so the swizzle term (r & 7) = (q2 + 7 - pr) & 7 does not depend on the pass:
    // one base address per query, the passes are constant offsets from it.
    static_assert(RPP % 8 == 0 && DW % 8 == 0, "the 128-byte swizzle phase must not depend on the pass");
    const int lim = w2 < DW ? w2 : DW;
    uint8_t* const base = tile + (c >> 3) * slab_bytes + 128 * (DW - 1 - pr);
#pragma unroll
    for (int q2 = 0; q2 < NQ; ++q2) {
        uint8_t* const bq = base + 128 * (DW + 1) * q2 + ((((c & 7) ^ ((q2 + 7 - pr) & 7))) << 4);
        const bool q_ok = i0 + q2 < n_q;
#pragma unroll
        for (int k = 0; k < PASSES; ++k) {
            const int dlt = DW - 1 + q2 - pr - k * RPP;
            if ((unsigned)dlt >= (unsigned)DW) continue;          // this window row does not meet query q2
            // x and y chunks of rows outside the tensors were loaded as zeros: without a bias their
            // product is already the zero the tile needs there
            bool ok = dlt < lim;
            if (BIAS) ok = ok && q_ok && (kb_first + pr + k * RPP >= 0);
            uint4 out = make_uint4(0, 0, 0, 0);
            if (ok) out = BIAS ? mul_chunk<F16>(regs[q2], regs[NQ + k], bias) : mul_chunk_nobias<F16>(regs[q2], regs[NQ + k]);
            *(uint4*)(bq - 128 * RPP * k) = out;
        }
    }
}

template <int HD, int DWLOG, bool BIAS, bool F16 = false, int NTHREADS = 128>
__device__ __forceinline__ void form_product_tile_shared(uint8_t* tile, int slab_bytes, int t, int i0, int n_q, int w2,
                                                         int halo2, const __nv_bfloat16* x, int64_t xs,
                                                         const __nv_bfloat16* y, int64_t ys, float bias) {
    uint4 regs[ProductTileShape<HD, DWLOG, NTHREADS>::NREGS];
    SA_PROF_T0(t_ld);
    load_product_tile_shared<HD, DWLOG, NTHREADS>(regs, t, i0, n_q, halo2, x, xs, y, ys);
#ifdef SA_PROFILE
#pragma unroll
    for (int k = 0; k < ProductTileShape<HD, DWLOG, NTHREADS>::NREGS; ++k) asm volatile("" ::"r"(regs[k].x), "r"(regs[k].w));
    SA_PROF_ADD(60, t_ld);
    SA_PROF_T0(t_st);
#endif
    store_product_tile_shared<HD, DWLOG, BIAS, F16, NTHREADS>(tile, slab_bytes, t, i0, n_q, w2, halo2, regs, bias);
#ifdef SA_PROFILE
    SA_PROF_ADD(61, t_st);
#endif
}

// A 128-row product tile that starts at query i0 (DW = 1 << dw_log2 delta slots per query): the
// shared-window form for 16, 32 and 64 slots (one round of loads), the general form otherwise.
template <int HD, bool BIAS, bool F16 = false>
__device__ __forceinline__ void form_query_tile(uint8_t* tile, int slab_bytes, int t, int i0, int dw_log2, int n_q, int w2,
                                                int halo2, const __nv_bfloat16* x, int64_t xs, const __nv_bfloat16* y,
                                                int64_t ys, float bias) {
    switch (dw_log2) {
        case 4: form_product_tile_shared<HD, 4, BIAS, F16>(tile, slab_bytes, t, i0, n_q, w2, halo2, x, xs, y, ys, bias); break;
        case 5: form_product_tile_shared<HD, 5, BIAS, F16>(tile, slab_bytes, t, i0, n_q, w2, halo2, x, xs, y, ys, bias); break;
        case 6: form_product_tile_shared<HD, 6, BIAS, F16>(tile, slab_bytes, t, i0, n_q, w2, halo2, x, xs, y, ys, bias); break;
        default:
            form_product_tile<HD, 128, 128, BIAS, F16>(tile, slab_bytes, t, (long)i0 << dw_log2, dw_log2, n_q, w2, halo2, x, xs, y, ys, bias);
    }
}

// Sum over the 32 lanes of a warp of CW values per lane (CW = 8, 16 or 32); afterwards lane L holds the
// total of value (L % CW) in v[0].  Lane bits at or above CW are summed plainly, the rest by a halving
// exchange: each step a lane keeps one half of its values and adds the partner's copy of that half
// (31 shuffles for 32 values).
template <int CW>
__device__ __forceinline__ float warp_transpose_reduce(float (&v)[CW], int lane) {
#pragma unroll
    for (int m = 16; m >= CW; m >>= 1) {
#pragma unroll
        for (int j = 0; j < CW; ++j) v[j] += __shfl_xor_sync(0xffffffffu, v[j], m);
    }
#pragma unroll
    for (int s = (CW == 32 ? 16 : CW / 2); s >= 1; s >>= 1) {
        const bool upper = (lane & s) != 0;
#pragma unroll
        for (int j = 0; j < s; ++j) {
            const float send = upper ? v[j] : v[j + s];
            const float keep = upper ? v[j + s] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, s);
        }
    }
    return v[0];
}

// The same within each half of the warp (lanes 0-15 and 16-31 separately), for CW = 8 or 16 values:
// lane L ends up with the total, over its 16-lane half, of value (L % CW).
template <int CW>
__device__ __forceinline__ float half_warp_transpose_reduce(float (&v)[CW], int lane) {
#pragma unroll
    for (int m = 8; m >= CW; m >>= 1) {
#pragma unroll
        for (int j = 0; j < CW; ++j) v[j] += __shfl_xor_sync(0xffffffffu, v[j], m);
    }
#pragma unroll
    for (int s = (CW == 16 ? 8 : CW / 2); s >= 1; s >>= 1) {
        const bool upper = (lane & s) != 0;
#pragma unroll
        for (int j = 0; j < s; ++j) {
            const float send = upper ? v[j] : v[j + s];
            const float keep = upper ? v[j + s] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, s);
        }
    }
    return v[0];
}
__device__ __forceinline__ float half_warp_transpose_reduce16(float (&v)[16], int lane) {
    return half_warp_transpose_reduce<16>(v, lane);
}

// Byte offset of element (row, col) inside a 128-byte-swizzled [rows x 64] bf16 slab.
__device__ __forceinline__ uint32_t swz128_offset(int row, int col) {
    return (uint32_t)row * 128u + ((((uint32_t)col >> 3) ^ ((uint32_t)row & 7u)) << 4) + (((uint32_t)col & 7u) << 1);
}

}  // namespace ptx
}  // namespace sa
