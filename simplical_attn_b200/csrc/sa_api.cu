// C ABI of libsimplicial_attn_b200.so: argument validation, kernel selection and launches.
// Declarations and the reference interfaces they replace: include/simplicial_attn_b200.h.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <atomic>
#include <mutex>

#include "sa_common.cuh"
#include "sa_general.cuh"
#include "sa_tc_bwd.cuh"
#include "sa_tc_fwd.cuh"

namespace {

using sa::KParams;

constexpr size_t kStatusBytes = 256;

std::atomic<uint64_t> g_launches{0};      // kernels launched by this library in this process
std::atomic<uint64_t> g_wait_limit_ns{sa::ptx::kWaitLimitNs};   // bound of every device-side wait (sa_set_wait_limit_ns)

// Scratch of sa_backward_static: lives in the module image, so every GPU that loads the library
// carries these bytes until the process exits.  In host code the symbol is only a handle; the
// device address is looked up once per device (static_scratch below).
constexpr size_t kStaticScratchBytes = 32u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kChunkW2 = 128;      // K2 positions one pass of the tensor-core kernels covers
constexpr int kMaxChunks = 8;      // passes the library is willing to chain (wider windows: general kernels)

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool stride_ok8(const sa_strides& s) { return s.b % 8 == 0 && s.n % 8 == 0 && s.h % 8 == 0; }

int elem_size(int dtype) { return dtype == SA_F32 ? 4 : 2; }

int validate(const sa_params* p) {
    if (!p) return SA_ERR_NULL_POINTER;
    if (p->B < 1 || p->N < 1 || p->H < 1 || p->Hkv < 1 || p->D < 1) return SA_ERR_BAD_SHAPE;
    if (p->H % p->Hkv != 0 || p->w1 < 1 || p->w2 < 1 || p->halo1 < 0 || p->halo2 < 0) return SA_ERR_BAD_SHAPE;
    if (p->dtype < SA_BF16 || p->dtype > SA_F32) return SA_ERR_UNSUPPORTED;
    if (p->D > 256) return SA_ERR_UNSUPPORTED;
    if (p->algo < SA_ALGO_AUTO || p->algo > SA_ALGO_TCGEN05) return SA_ERR_UNSUPPORTED;
    return SA_OK;
}

KParams make_kparams(const sa_params* p) {
    KParams k{};
    k.B = p->B; k.N = p->N; k.H = p->H; k.Hkv = p->Hkv; k.D = p->D; k.G = p->H / p->Hkv;
    k.halo1 = p->halo1; k.halo2 = p->halo2;
    k.n1 = p->N + p->halo1; k.n2 = p->N + p->halo2;
    k.w1 = p->w1 < k.n1 ? p->w1 : k.n1;
    k.w2 = p->w2 < k.n2 ? p->w2 : k.n2;
    k.scale = p->scale; k.k2_bias = p->k2_bias; k.v2_bias = p->v2_bias;
    k.q = p->q; k.k1 = p->k1; k.k2 = p->k2; k.v1 = p->v1; k.v2 = p->v2; k.o = p->o;
    k.d_o = p->d_o; k.dq = p->dq; k.dk1 = p->dk1; k.dk2 = p->dk2; k.dv1 = p->dv1; k.dv2 = p->dv2;
    return k;
}

// Whether the tensor-core kernels cover the problem's shape and dtype (pointer alignment is
// checked at the call).
bool tc_shape_ok(const sa_params* p, bool backward) {
    const KParams k = make_kparams(p);
    if (p->dtype != SA_BF16 && p->dtype != SA_F16) return false;
    if (p->D != 64 && p->D != 128) return false;
    if (k.w2 > kChunkW2 * kMaxChunks) return false;
    if (p->scale <= 0.f) return false;            // the row maximum is taken before scaling
    if (!stride_ok8(p->q) || !stride_ok8(p->k1) || !stride_ok8(p->k2) || !stride_ok8(p->v1) || !stride_ok8(p->v2) ||
        !stride_ok8(p->o))
        return false;
    if (backward && (!stride_ok8(p->d_o) || !stride_ok8(p->dq) || !stride_ok8(p->dk1) || !stride_ok8(p->dk2) ||
                     !stride_ok8(p->dv1) || !stride_ok8(p->dv2)))
        return false;
    return true;
}

int dw_log2_of(int w2) {
    int l = 0;
    while ((1 << l) < w2) ++l;
    return l;
}

// ---- driver entry point for tensor-map encoding (resolved at run time; no link against libcuda)
PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    });
    return fn;
}

// Tensor map over a bf16 (or, with `f16`, IEEE half) [B, rows, heads, D] tensor with (b, n, h) element strides;
// a box is 64 elements of one row by `box_rows` rows, landing 128-byte swizzled.
bool make_map(CUtensorMap* map, const void* base, int B, int rows, int heads, int D, const sa_strides& st, int box_rows,
              bool f16) {
    auto enc = get_encode();
    if (!enc) return false;
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)B};
    // A stride of an extent-1 dimension is never used to form an address; give it a harmless value.
    auto sb = [&](int64_t s, int extent) { return (cuuint64_t)((extent > 1 ? s : (int64_t)D) * 2); };
    cuuint64_t strides[3] = {sb(st.n, rows), sb(st.h, heads), sb(st.b, B)};
    cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Self-test of the bounded wait: one warp waits on an mbarrier that nobody ever arrives on.  The wait
// gives up after `limit_ns`, records SA_ERR_DEVICE_TIMEOUT in the status word and the kernel returns
// by itself: nothing traps, nothing spins without a bound.
__global__ void __launch_bounds__(32) wait_timeout_probe_kernel(sa::DeviceStatus* status, uint64_t limit_ns, int where) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        sa::ptx::mbar_init(&bar, 1);
        abort_flag = 0;
        sa::ptx::fence_mbar_init();
    }
    __syncwarp();
    const sa::ptx::WaitCtx ctx{&abort_flag, status, limit_ns};
    sa::ptx::mbar_wait(&bar, 0, ctx, where);      // phase 0 never completes
    sa::ptx::mbar_wait(&bar, 0, ctx, where + 1);  // after the first wait gave up every later wait falls through
}

// ---- K2 windows wider than one pass of the tensor-core kernels (128 positions).  The window is cut into chunks of
// at most 128 positions; chunk c is an ordinary call whose K2/V2 rows sit 128 c rows further back, which is what a
// halo of halo2 - 128 c rows means (rows before the buffer's start do not exist and are masked as always).  Forward:
// the chunks' outputs are merged by their log-sum-exp.  Backward: with the merged O and LSE every chunk's
// probabilities are already normalised over the whole window, so the chunks' gradients simply add.
int num_chunks(const KParams& k) { return (k.w2 + kChunkW2 - 1) / kChunkW2; }

KParams chunk_params(const KParams& k, int c) {
    KParams kc = k;
    kc.halo2 = k.halo2 - c * kChunkW2;
    kc.n2 = k.N + kc.halo2;
    kc.w2 = k.w2 - c * kChunkW2 < kChunkW2 ? k.w2 - c * kChunkW2 : kChunkW2;
    return kc;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
sa_strides contiguous_strides(int rows, int heads, int D) {
    return sa_strides{(int64_t)rows * heads * D, (int64_t)heads * D, (int64_t)D};
}

// Temporaries of the chunked calls, behind the status word (and, in the backward, the kernels' own workspace).
struct ChunkTemps {
    size_t o, lse, dq, dk1, dv1, dk2, dv2, total;
};
ChunkTemps chunk_temps(const KParams& k, bool backward) {
    ChunkTemps t{};
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t at = off; off += align256(bytes); return at; };
    if (!backward) {
        t.o = take((size_t)k.B * k.N * k.H * k.D * 2);
        t.lse = take((size_t)k.B * k.H * k.N * 4);
    } else {
        t.dq = take((size_t)k.B * k.N * k.H * k.D * 2);
        t.dk1 = take((size_t)k.B * k.n1 * k.Hkv * k.D * 2);
        t.dv1 = take((size_t)k.B * k.n1 * k.Hkv * k.D * 2);
        t.dk2 = take((size_t)k.B * k.n2 * k.Hkv * k.D * 2);
        t.dv2 = take((size_t)k.B * k.n2 * k.Hkv * k.D * 2);
    }
    t.total = off;
    return t;
}

// o = (e^lse o + e^lse_t o_t) / (e^lse + e^lse_t), eight elements per thread; lse is updated afterwards by
// merge_lse_kernel (every thread of a row reads the old value here).
template <typename T>
__global__ void __launch_bounds__(256) merge_o_kernel(T* __restrict__ o, sa_strides so, const float* __restrict__ lse,
                                                      const T* __restrict__ o_t, const float* __restrict__ lse_t, int B, int N,
                                                      int H, int D) {
    const int cpr = D / 8;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)B * N * H * cpr) return;
    const int c = (int)(idx % cpr), h = (int)((idx / cpr) % H), n = (int)((idx / cpr / H) % N), b = (int)(idx / cpr / H / N);
    const long li = ((long)b * H + h) * N + n;
    const float l0 = lse[li], l1 = lse_t[li];
    if (!(l1 > -INFINITY)) return;                     // this chunk holds nothing for the query
    const float m = fmaxf(l0, l1);
    const float w0 = __expf(l0 - m), w1 = __expf(l1 - m), inv = 1.f / (w0 + w1);
    T* dst = o + b * so.b + (long)n * so.n + h * so.h + c * 8;
    const T* src = o_t + (((long)b * N + n) * H + h) * D + c * 8;
    uint4 a = *reinterpret_cast<const uint4*>(dst), t = *reinterpret_cast<const uint4*>(src);
    T* av = reinterpret_cast<T*>(&a);
    const T* tv = reinterpret_cast<const T*>(&t);
#pragma unroll
    for (int e = 0; e < 8; ++e) av[e] = sa::from_f<T>((w0 * sa::to_f<T>(av[e]) + w1 * sa::to_f<T>(tv[e])) * inv);
    *reinterpret_cast<uint4*>(dst) = a;
}

__global__ void __launch_bounds__(256) merge_lse_kernel(float* __restrict__ lse, const float* __restrict__ lse_t, long n) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const float l0 = lse[idx], l1 = lse_t[idx];
    if (!(l1 > -INFINITY)) return;
    const float m = fmaxf(l0, l1);
    lse[idx] = m + __logf(__expf(l0 - m) + __expf(l1 - m));
}

// dst[b, r, h, :] += tmp[b, r, h, :] for r < rows (tmp contiguous [B, rows, heads, D]), eight elements per thread
template <typename T>
__global__ void __launch_bounds__(256) add_rows_kernel(T* __restrict__ dst, sa_strides sd, const T* __restrict__ tmp, int B,
                                                       int rows, int heads, int D) {
    const int cpr = D / 8;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)B * rows * heads * cpr) return;
    const int c = (int)(idx % cpr), h = (int)((idx / cpr) % heads), r = (int)((idx / cpr / heads) % rows),
              b = (int)(idx / cpr / heads / rows);
    T* d = dst + b * sd.b + (long)r * sd.n + h * sd.h + c * 8;
    uint4 a = *reinterpret_cast<const uint4*>(d), t = *reinterpret_cast<const uint4*>(tmp + idx * 8);
    T* av = reinterpret_cast<T*>(&a);
    const T* tv = reinterpret_cast<const T*>(&t);
#pragma unroll
    for (int e = 0; e < 8; ++e) av[e] = sa::from_f<T>(sa::to_f<T>(av[e]) + sa::to_f<T>(tv[e]));
    *reinterpret_cast<uint4*>(d) = a;
}

template <typename T>
void launch_add_rows(void* dst, const sa_strides& sd, const void* tmp, int B, int rows, int heads, int D, cudaStream_t st) {
    const long total = (long)B * rows * heads * (D / 8);
    add_rows_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((T*)dst, sd, (const T*)tmp, B, rows, heads, D);
}

struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    bool attrs_set = false;
};

DeviceInfo& device_info() {
    static DeviceInfo info[64];
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    DeviceInfo& d = info[dev & 63];
    if (d.sm_count == 0) {
        cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    }
    return d;
}

// Device address of g_static_scratch on the current device, resolved on first use per device.
void* static_scratch() {
    static void* addr[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    void*& slot = addr[dev & 63];
    if (slot == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess) return nullptr;
        slot = p;
    }
    return slot;
}

// Multiprocessor count the backward plan is sized for: the current device's, or a B200's when no
// device is available (size queries on a machine without a GPU).
int plan_sm_count() {
    const int n = device_info().sm_count;
    return n > 0 ? n : 148;
}

template <typename Kern>
bool set_smem(Kern kern, int bytes) {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
}

template <bool F16>
int launch_fwd_tc_t(const KParams& k, const void* q, const void* k1, const void* k2, const void* v1, const void* v2, void* o,
                    float* lse, void* workspace, cudaStream_t st) {
    DeviceInfo& dev = device_info();
    if (dev.cc_major != 10) return SA_ERR_NOT_SM100;
    CUtensorMap map_k1, map_v1;
    if (!make_map(&map_k1, k1, k.B, k.n1, k.Hkv, k.D, k.k1, sa::tc::kSubTile, F16)) return SA_ERR_BAD_STRIDE;
    if (!make_map(&map_v1, v1, k.B, k.n1, k.Hkv, k.D, k.v1, sa::tc::kSubTile, F16)) return SA_ERR_BAD_STRIDE;
    sa::tc::FwdTcParams P{};
    P.k = k;
    P.dw_log2 = dw_log2_of(k.w2);
    const int qpb = (sa::tc::kNumRowTiles * sa::tc::kRowTile) >> P.dw_log2;
    P.num_qblocks = (k.N + qpb - 1) / qpb;
    P.num_units = (long)k.B * k.H * P.num_qblocks;
    P.status = reinterpret_cast<sa::DeviceStatus*>(workspace);
    P.wait_limit_ns = g_wait_limit_ns.load();
    const long grid = P.num_units < dev.sm_count ? P.num_units : dev.sm_count;
    const bool has_bias = k.k2_bias != 0.f || k.v2_bias != 0.f;
    auto launch = [&](auto kern, int smem_bytes) {
        if (!set_smem(kern, smem_bytes)) return false;
        kern<<<(unsigned)grid, sa::tc::kFwdThreads, smem_bytes, st>>>(P, map_k1, map_v1, (const __nv_bfloat16*)q,
                                                                       (const __nv_bfloat16*)k2, (const __nv_bfloat16*)v2,
                                                                       (__nv_bfloat16*)o, lse);
        return true;
    };
    bool ok;
    if (k.D == 128)
        ok = has_bias ? launch(sa::tc::fwd_tc_kernel<128, true, F16>, sa::tc::FwdSmem<128>::kAlloc)
                      : launch(sa::tc::fwd_tc_kernel<128, false, F16>, sa::tc::FwdSmem<128>::kAlloc);
    else
        ok = has_bias ? launch(sa::tc::fwd_tc_kernel<64, true, F16>, sa::tc::FwdSmem<64>::kAlloc)
                      : launch(sa::tc::fwd_tc_kernel<64, false, F16>, sa::tc::FwdSmem<64>::kAlloc);
    if (!ok) return SA_ERR_LAUNCH;
    g_launches += 1;
    return cudaGetLastError() == cudaSuccess ? SA_OK : SA_ERR_LAUNCH;
}

int launch_fwd_tc_one(const sa_params* p, const KParams& k, const void* q, const void* k1, const void* k2, const void* v1,
                      const void* v2, void* o, float* lse, void* workspace, cudaStream_t st) {
    return p->dtype == SA_F16 ? launch_fwd_tc_t<true>(k, q, k1, k2, v1, v2, o, lse, workspace, st)
                              : launch_fwd_tc_t<false>(k, q, k1, k2, v1, v2, o, lse, workspace, st);
}

// One pass, or one pass per 128-position chunk of the K2 window merged into o / lse.
int launch_fwd_tc(const sa_params* p, const KParams& k, const void* q, const void* k1, const void* k2, const void* v1,
                  const void* v2, void* o, float* lse, void* workspace, cudaStream_t st) {
    const int nc = num_chunks(k);
    if (nc == 1) return launch_fwd_tc_one(p, k, q, k1, k2, v1, v2, o, lse, workspace, st);
    const ChunkTemps t = chunk_temps(k, false);
    uint8_t* base = static_cast<uint8_t*>(workspace) + kStatusBytes;
    void* o_t = base + t.o;
    float* lse_t = reinterpret_cast<float*>(base + t.lse);
    for (int c = 0; c < nc; ++c) {
        KParams kc = chunk_params(k, c);
        if (c > 0) kc.o = contiguous_strides(k.N, k.H, k.D);
        const int rc = launch_fwd_tc_one(p, kc, q, k1, k2, v1, v2, c == 0 ? o : o_t, c == 0 ? lse : lse_t, workspace, st);
        if (rc != SA_OK) return rc;
        if (c == 0) continue;
        const long total = (long)k.B * k.N * k.H * (k.D / 8);
        if (p->dtype == SA_F16)
            merge_o_kernel<__half><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((__half*)o, k.o, lse, (const __half*)o_t, lse_t,
                                                                                      k.B, k.N, k.H, k.D);
        else
            merge_o_kernel<__nv_bfloat16><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
                (__nv_bfloat16*)o, k.o, lse, (const __nv_bfloat16*)o_t, lse_t, k.B, k.N, k.H, k.D);
        const long rows = (long)k.B * k.H * k.N;
        merge_lse_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(lse, lse_t, rows);
        g_launches += 2;
    }
    return cudaGetLastError() == cudaSuccess ? SA_OK : SA_ERR_LAUNCH;
}

// Workspace of the tensor-core backward: the kernels' own (the largest over the chunks) and, with more than one
// chunk, the temporaries the later chunks' gradients are written to before they are added.
size_t bwd_tc_kernel_workspace(const KParams& k) {
    size_t m = 0;
    for (int c = 0; c < num_chunks(k); ++c) {
        const size_t b = sa::tc::bwd_workspace_bytes(chunk_params(k, c), plan_sm_count());
        m = b > m ? b : m;
    }
    return align256(m);
}

// Returns an sa_status, or -1 when the tensor-core backward declines the problem (nothing has been launched then).
int launch_bwd_tc(const sa_params* p, const KParams& k, const void* q, const void* k1, const void* k2, const void* v1,
                  const void* v2, const void* o, const float* lse, const void* d_o, void* dq, void* dk1, void* dk2, void* dv1,
                  void* dv2, void* workspace, cudaStream_t st) {
    const int nc = num_chunks(k);
    uint8_t* kernel_ws = static_cast<uint8_t*>(workspace) + kStatusBytes;
    sa::DeviceStatus* status = reinterpret_cast<sa::DeviceStatus*>(workspace);
    const bool f16 = p->dtype == SA_F16;
    const ChunkTemps t = chunk_temps(k, true);
    uint8_t* temps = kernel_ws + bwd_tc_kernel_workspace(k);
    for (int c = 0; c < nc; ++c) {
        KParams kc = chunk_params(k, c);
        void *cq = dq, *ck1 = dk1, *ck2 = dk2, *cv1 = dv1, *cv2 = dv2;
        if (c > 0) {
            if (dq) { cq = temps + t.dq; kc.dq = contiguous_strides(k.N, k.H, k.D); }
            if (dk1) { ck1 = temps + t.dk1; kc.dk1 = contiguous_strides(k.n1, k.Hkv, k.D); }
            if (dv1) { cv1 = temps + t.dv1; kc.dv1 = contiguous_strides(k.n1, k.Hkv, k.D); }
            if (dk2) { ck2 = temps + t.dk2; kc.dk2 = contiguous_strides(kc.n2, k.Hkv, k.D); }
            if (dv2) { cv2 = temps + t.dv2; kc.dv2 = contiguous_strides(kc.n2, k.Hkv, k.D); }
        }
        int nlaunch = 0;
        const int rc = sa::tc::launch_bwd(kc, q, k1, k2, v1, v2, o, lse, d_o, cq, ck1, ck2, cv1, cv2, kernel_ws, status, st, &nlaunch,
                                          &make_map, plan_sm_count(), g_wait_limit_ns.load(), f16);
        g_launches += nlaunch;
        if (rc == -1) return c == 0 ? -1 : SA_ERR_UNSUPPORTED;
        if (rc != SA_OK) return rc;
        if (c == 0) continue;
        auto add = [&](void* dst, const sa_strides& sd, void* tmp, int rows, int heads) {
            if (!dst) return;
            if (f16) launch_add_rows<__half>(dst, sd, tmp, k.B, rows, heads, k.D, st);
            else launch_add_rows<__nv_bfloat16>(dst, sd, tmp, k.B, rows, heads, k.D, st);
            g_launches += 1;
        };
        add(dq, k.dq, cq, k.N, k.H);
        add(dk1, k.dk1, ck1, k.n1, k.Hkv);
        add(dv1, k.dv1, cv1, k.n1, k.Hkv);
        add(dk2, k.dk2, ck2, kc.n2, k.Hkv);      // a later chunk reaches only the first n2 - 128 c rows
        add(dv2, k.dv2, cv2, kc.n2, k.Hkv);
    }
    return cudaGetLastError() == cudaSuccess ? SA_OK : SA_ERR_LAUNCH;
}

int resolve(const sa_params* p, bool backward) {
    if (p->algo == SA_ALGO_GENERAL) return SA_ALGO_GENERAL;
    const bool ok = tc_shape_ok(p, backward);
    if (p->algo == SA_ALGO_TCGEN05) return ok ? SA_ALGO_TCGEN05 : -SA_ERR_UNSUPPORTED;
    return ok ? SA_ALGO_TCGEN05 : SA_ALGO_GENERAL;
}

}  // namespace

extern "C" {

int sa_version(void) { return 200; }

uint64_t sa_kernel_launches(void) { return g_launches.load(); }

#ifdef SA_PROFILE
// Profiling builds only: copies and clears the per-wait-site cycle and hit counters of block 0.
int sa_prof_read(unsigned long long* cycles, unsigned long long* counts) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(cycles, sa::ptx::g_prof_cycles, 64 * 8);
    cudaMemcpyFromSymbol(counts, sa::ptx::g_prof_count, 64 * 8);
    unsigned long long z[64] = {0};
    cudaMemcpyToSymbol(sa::ptx::g_prof_cycles, z, 64 * 8);
    cudaMemcpyToSymbol(sa::ptx::g_prof_count, z, 64 * 8);
    return 0;
}
#endif

#ifdef SA_TRACE
int sa_trace_read(unsigned long long* ev, int* n) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(ev, sa::ptx::g_trace, sizeof(unsigned long long) * 16 * 2048);
    cudaMemcpyFromSymbol(n, sa::ptx::g_trace_n, sizeof(int) * 16);
    int z[16] = {0};
    cudaMemcpyToSymbol(sa::ptx::g_trace_n, z, sizeof(z));
    return 0;
}
#endif

const char* sa_strerror(int status) {
    switch (status) {
        case SA_OK: return "ok";
        case SA_ERR_NULL_POINTER: return "a required pointer is NULL";
        case SA_ERR_BAD_SHAPE: return "bad shape: extents must be positive, H % Hkv == 0, windows >= 1, halos >= 0";
        case SA_ERR_BAD_STRIDE: return "bad stride or pointer alignment: the tensor-core kernels need 16-byte aligned rows";
        case SA_ERR_UNSUPPORTED: return "unsupported dtype, head dim, window or kernel choice";
        case SA_ERR_WORKSPACE: return "workspace too small or not 256-byte aligned";
        case SA_ERR_LAUNCH: return "CUDA reported an error at kernel launch";
        case SA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
        case SA_ERR_NOT_SM100: return "the tensor-core kernels need a compute capability 10.x device";
        default: return "unknown status";
    }
}

int sa_resolve_algo(const sa_params* p) {
    const int v = validate(p);
    if (v != SA_OK) return -v;
    return resolve(p, true);
}

size_t sa_forward_workspace_size(const sa_params* p) {
    if (validate(p) != SA_OK || resolve(p, false) != SA_ALGO_TCGEN05) return kStatusBytes;
    const KParams k = make_kparams(p);
    return kStatusBytes + (num_chunks(k) > 1 ? chunk_temps(k, false).total : 0);
}

size_t sa_backward_workspace_size(const sa_params* p) {
    if (validate(p) != SA_OK) return kStatusBytes;
    if (resolve(p, true) != SA_ALGO_TCGEN05) return kStatusBytes;
    const KParams k = make_kparams(p);
    return kStatusBytes + bwd_tc_kernel_workspace(k) + (num_chunks(k) > 1 ? chunk_temps(k, true).total : 0);
}

int sa_read_status_ex(void* workspace, void* stream, int* where, int* block) {
    if (!workspace) return SA_ERR_NULL_POINTER;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    sa::DeviceStatus h{};
    if (cudaMemcpyAsync(&h, workspace, sizeof(h), cudaMemcpyDeviceToHost, st) != cudaSuccess) return SA_ERR_LAUNCH;
    if (cudaStreamSynchronize(st) != cudaSuccess) return SA_ERR_LAUNCH;
    if (h.code != 0) cudaMemsetAsync(workspace, 0, sizeof(h), st);
    if (where) *where = h.where;
    if (block) *block = h.block;
    return h.code;
}

int sa_read_status(void* workspace, void* stream) { return sa_read_status_ex(workspace, stream, nullptr, nullptr); }

int sa_status_relay(const void* workspace, void* device_slot, void* host_slot, void* stream, void* side_stream, void* ev_ready,
                    void* ev_done) {
    if (!workspace || !device_slot || !host_slot || !ev_ready || !ev_done) return SA_ERR_NULL_POINTER;
    cudaStream_t st = static_cast<cudaStream_t>(stream), side = static_cast<cudaStream_t>(side_stream);
    cudaEvent_t ready = static_cast<cudaEvent_t>(ev_ready), done = static_cast<cudaEvent_t>(ev_done);
    const bool ok = cudaMemcpyAsync(device_slot, workspace, sizeof(sa::DeviceStatus), cudaMemcpyDeviceToDevice, st) == cudaSuccess &&
                    cudaEventRecord(ready, st) == cudaSuccess && cudaStreamWaitEvent(side, ready, 0) == cudaSuccess &&
                    cudaMemcpyAsync(host_slot, device_slot, sizeof(sa::DeviceStatus), cudaMemcpyDeviceToHost, side) == cudaSuccess &&
                    cudaEventRecord(done, side) == cudaSuccess;
    return ok ? SA_OK : SA_ERR_LAUNCH;
}

int sa_read_status_static(void* stream) {
    void* scratch = static_scratch();
    if (!scratch) return SA_ERR_LAUNCH;
    return sa_read_status_ex(scratch, stream, nullptr, nullptr);
}

void sa_set_wait_limit_ns(uint64_t limit_ns) { g_wait_limit_ns.store(limit_ns ? limit_ns : sa::ptx::kWaitLimitNs); }

int sa_selftest_wait_timeout(void* workspace, uint64_t limit_ns, void* stream) {
    if (!workspace) return SA_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return SA_ERR_WORKSPACE;
    if (limit_ns == 0 || limit_ns > 100000000ull) return SA_ERR_UNSUPPORTED;      // at most 0.1 s for a test
    wait_timeout_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<sa::DeviceStatus*>(workspace), limit_ns, 90);
    g_launches += 1;
    return cudaGetLastError() == cudaSuccess ? SA_OK : SA_ERR_LAUNCH;
}

int sa_forward(const sa_params* p, const void* q, const void* k1, const void* k2, const void* v1, const void* v2, void* o,
               float* lse, void* workspace, size_t workspace_bytes, void* stream) {
    const int v = validate(p);
    if (v != SA_OK) return v;
    if (!q || !k1 || !k2 || !v1 || !v2 || !o || !lse || !workspace) return SA_ERR_NULL_POINTER;
    if (workspace_bytes < sa_forward_workspace_size(p) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return SA_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const KParams k = make_kparams(p);
    int algo = resolve(p, false);
    if (algo < 0) return -algo;
    if (algo == SA_ALGO_TCGEN05 &&
        !(aligned16(q) && aligned16(k1) && aligned16(k2) && aligned16(v1) && aligned16(v2) && aligned16(o))) {
        if (p->algo == SA_ALGO_TCGEN05) return SA_ERR_BAD_STRIDE;
        algo = SA_ALGO_GENERAL;
    }
    if (algo == SA_ALGO_TCGEN05) return launch_fwd_tc(p, k, q, k1, k2, v1, v2, o, lse, workspace, st);
    const cudaError_t e = sa::general::launch_fwd(p->dtype, k, q, k1, k2, v1, v2, o, lse, st);
    g_launches += 1;
    (void)elem_size;
    return e == cudaSuccess ? SA_OK : SA_ERR_LAUNCH;
}

int sa_backward(const sa_params* p, const void* q, const void* k1, const void* k2, const void* v1, const void* v2,
                const void* o, const float* lse, const void* d_o, void* dq, void* dk1, void* dk2, void* dv1, void* dv2,
                void* workspace, size_t workspace_bytes, void* stream) {
    const int v = validate(p);
    if (v != SA_OK) return v;
    if (!q || !k1 || !k2 || !v1 || !v2 || !o || !lse || !d_o || !workspace) return SA_ERR_NULL_POINTER;
    if (workspace_bytes < sa_backward_workspace_size(p) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return SA_ERR_WORKSPACE;
    if (!dq && !dk1 && !dk2 && !dv1 && !dv2) return SA_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const KParams k = make_kparams(p);
    int algo = resolve(p, true);
    if (algo < 0) return -algo;
    auto al = [](const void* x) { return x == nullptr || aligned16(x); };
    if (algo == SA_ALGO_TCGEN05 && !(aligned16(q) && aligned16(k1) && aligned16(k2) && aligned16(v1) && aligned16(v2) &&
                                     aligned16(o) && aligned16(d_o) && al(dq) && al(dk1) && al(dk2) && al(dv1) && al(dv2))) {
        if (p->algo == SA_ALGO_TCGEN05) return SA_ERR_BAD_STRIDE;
        algo = SA_ALGO_GENERAL;
    }
    if (algo == SA_ALGO_TCGEN05) {
        if (device_info().cc_major != 10) return SA_ERR_NOT_SM100;
        const int rc = launch_bwd_tc(p, k, q, k1, k2, v1, v2, o, lse, d_o, dq, dk1, dk2, dv1, dv2, workspace, st);
        if (rc != -1) return rc;      // -1: the tensor-core backward declines this problem
        if (p->algo == SA_ALGO_TCGEN05) return SA_ERR_UNSUPPORTED;
    }
    const cudaError_t e = sa::general::launch_bwd(p->dtype, k, q, k1, k2, v1, v2, o, lse, d_o, dq, dk1, dk2, dv1, dv2, st);
    g_launches += (dq ? 1 : 0) + ((dk1 || dv1) ? 1 : 0) + ((dk2 || dv2) ? 1 : 0);
    return e == cudaSuccess ? SA_OK : SA_ERR_LAUNCH;
}

int sa_copy_rows_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes, size_t rows,
                       void* stream) {
    if (!dst || !src) return SA_ERR_NULL_POINTER;
    if (row_bytes > dst_pitch || row_bytes > src_pitch) return SA_ERR_BAD_STRIDE;
    const cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, row_bytes, rows, cudaMemcpyDefault,
                                            static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? SA_OK : SA_ERR_LAUNCH;
}

size_t sa_backward_static_capacity(void) { return kStaticScratchBytes; }

int sa_backward_static(const sa_params* p, const void* q, const void* k1, const void* k2, const void* v1, const void* v2,
                       const void* o, const float* lse, const void* d_o, void* dq, void* dk1, void* dk2, void* dv1,
                       void* dv2, void* stream) {
    const int v = validate(p);
    if (v != SA_OK) return v;
    const size_t need = sa_backward_workspace_size(p);
    if (need > kStaticScratchBytes) return SA_ERR_WORKSPACE;      // the built-in scratch is fixed-size
    void* scratch = static_scratch();                             // first call per device resolves the address
    if (!scratch) return SA_ERR_LAUNCH;
    // The scratch keeps what the previous call left.  Nothing in it has to start at zero: the kernels
    // write every partial sum before they read it, and the status word (zero when the library is
    // loaded) is only ever cleared by sa_read_status_static, so that a timeout recorded by an earlier
    // call is not lost.
    return sa_backward(p, q, k1, k2, v1, v2, o, lse, d_o, dq, dk1, dk2, dv1, dv2, scratch, kStaticScratchBytes, stream);
}

}  // extern "C"
