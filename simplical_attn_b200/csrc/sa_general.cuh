// General 2-simplicial attention kernels: CUDA-core fp32 arithmetic for any dtype, head dim
// (<= 256) and window.  One warp owns one output row and accumulates it in registers, so every
// output element is written exactly once, in a fixed order, without atomics.
//
// They cover what the tensor-core kernels do not (fp16/fp32 tensors, head dims other than 64/128,
// very wide K2 windows) and are the on-device cross-check of the tensor-core kernels.
//
// The arithmetic restates the reference's definition (simplicial/reference.py:39-74) with an
// online maximum, and, for the backward, the derivative the reference's backward kernels
// implement (simplicial/kernels.py:175-382 for dQ/dK1/dV1, :386-566 for dK2/dV2).
#pragma once

#include "sa_common.cuh"

namespace sa {
namespace general {

constexpr int kWarpsPerBlock = 4;

// Lane `lane` of a warp holds elements d = lane + 32*e of a D-vector.
template <typename T, int EPL>
__device__ __forceinline__ void load_row(const T* __restrict__ row, int D, int lane, float (&v)[EPL], float bias = 0.f) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        const int d = lane + 32 * e;
        v[e] = d < D ? to_f<T>(row[d]) + bias : 0.f;
    }
}

template <typename T, int EPL>
__device__ __forceinline__ void store_row(T* __restrict__ row, int D, int lane, const float (&v)[EPL]) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        const int d = lane + 32 * e;
        if (d < D) row[d] = from_f<T>(v[e]);
    }
}

template <int EPL>
__device__ __forceinline__ float dot(const float (&a)[EPL], const float (&b)[EPL]) {
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) s = fmaf(a[e], b[e], s);
    return s;
}

// Forward: warp per (b, h, i).
template <typename T, int EPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
fwd_kernel(KParams p, const T* __restrict__ q, const T* __restrict__ k1, const T* __restrict__ k2,
           const T* __restrict__ v1, const T* __restrict__ v2, T* __restrict__ o, float* __restrict__ lse) {
    const long row = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= (long)p.B * p.H * p.N) return;
    const int i = (int)(row % p.N);
    const int h = (int)((row / p.N) % p.H);
    const int b = (int)(row / p.N / p.H);
    const int hk = h / p.G;
    const int D = p.D;

    float qv[EPL];
    load_row<T, EPL>(q + b * p.q.b + (long)i * p.q.n + h * p.q.h, D, lane, qv);
    const int j_hi = i + p.halo1, j_lo = max(0, j_hi - p.w1 + 1);
    const int k_hi = i + p.halo2, k_lo = max(0, k_hi - p.w2 + 1);
    const T* k1h = k1 + b * p.k1.b + hk * p.k1.h;
    const T* v1h = v1 + b * p.v1.b + hk * p.v1.h;
    const T* k2h = k2 + b * p.k2.b + hk * p.k2.h;
    const T* v2h = v2 + b * p.v2.b + hk * p.v2.h;

    float m = -INFINITY, l = 0.f;
    float acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;

    for (int k = k_lo; k <= k_hi; ++k) {
        float a[EPL], t[EPL], v2v[EPL];
        load_row<T, EPL>(k2h + (long)k * p.k2.n, D, lane, a, p.k2_bias);
        load_row<T, EPL>(v2h + (long)k * p.v2.n, D, lane, v2v, p.v2_bias);
#pragma unroll
        for (int e = 0; e < EPL; ++e) { a[e] *= qv[e] * p.scale; t[e] = 0.f; }
        for (int j = j_lo; j <= j_hi; ++j) {
            float k1v[EPL], v1v[EPL];
            load_row<T, EPL>(k1h + (long)j * p.k1.n, D, lane, k1v);
            load_row<T, EPL>(v1h + (long)j * p.v1.n, D, lane, v1v);
            const float s = warp_sum(dot<EPL>(a, k1v));
            if (s > m) {                                  // warp-uniform
                const float corr = __expf(m - s);         // m = -inf gives 0
                l *= corr;
#pragma unroll
                for (int e = 0; e < EPL; ++e) { acc[e] *= corr; t[e] *= corr; }
                m = s;
            }
            const float pv = __expf(s - m);
            l += pv;
#pragma unroll
            for (int e = 0; e < EPL; ++e) t[e] = fmaf(pv, v1v[e], t[e]);
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] = fmaf(t[e], v2v[e], acc[e]);
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] *= inv;
    store_row<T, EPL>(o + b * p.o.b + (long)i * p.o.n + h * p.o.h, D, lane, acc);
    if (lane == 0) lse[((long)b * p.H + h) * p.N + i] = m + logf(l);
}

// Per-query quantities every backward sweep needs: the query row, dO row, Delta = dO.O and LSE.
template <typename T, int EPL>
__device__ __forceinline__ void load_query(const KParams& p, const T* q, const T* o, const T* d_o, const float* lse,
                                           int b, int h, int i, int lane, float (&qv)[EPL], float (&dov)[EPL],
                                           float& delta, float& L) {
    float ov[EPL];
    load_row<T, EPL>(q + b * p.q.b + (long)i * p.q.n + h * p.q.h, p.D, lane, qv);
    load_row<T, EPL>(d_o + b * p.d_o.b + (long)i * p.d_o.n + h * p.d_o.h, p.D, lane, dov);
    load_row<T, EPL>(o + b * p.o.b + (long)i * p.o.n + h * p.o.h, p.D, lane, ov);
    delta = warp_sum(dot<EPL>(dov, ov));
    L = lse[((long)b * p.H + h) * p.N + i];
}

// dQ: warp per (b, h, i).
template <typename T, int EPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
bwd_dq_kernel(KParams p, const T* __restrict__ q, const T* __restrict__ k1, const T* __restrict__ k2,
              const T* __restrict__ v1, const T* __restrict__ v2, const T* __restrict__ o,
              const float* __restrict__ lse, const T* __restrict__ d_o, T* __restrict__ dq) {
    const long row = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= (long)p.B * p.H * p.N) return;
    const int i = (int)(row % p.N);
    const int h = (int)((row / p.N) % p.H);
    const int b = (int)(row / p.N / p.H);
    const int hk = h / p.G;
    const int D = p.D;
    float qv[EPL], dov[EPL], delta, L;
    load_query<T, EPL>(p, q, o, d_o, lse, b, h, i, lane, qv, dov, delta, L);
    const int j_hi = i + p.halo1, j_lo = max(0, j_hi - p.w1 + 1);
    const int k_hi = i + p.halo2, k_lo = max(0, k_hi - p.w2 + 1);
    const T* k1h = k1 + b * p.k1.b + hk * p.k1.h;
    const T* v1h = v1 + b * p.v1.b + hk * p.v1.h;
    const T* k2h = k2 + b * p.k2.b + hk * p.k2.h;
    const T* v2h = v2 + b * p.v2.b + hk * p.v2.h;
    float acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
    for (int k = k_lo; k <= k_hi; ++k) {
        float k2v[EPL], a[EPL], c[EPL], g[EPL];
        load_row<T, EPL>(k2h + (long)k * p.k2.n, D, lane, k2v, p.k2_bias);
        load_row<T, EPL>(v2h + (long)k * p.v2.n, D, lane, c, p.v2_bias);
#pragma unroll
        for (int e = 0; e < EPL; ++e) { a[e] = qv[e] * k2v[e] * p.scale; c[e] *= dov[e]; g[e] = 0.f; }
        for (int j = j_lo; j <= j_hi; ++j) {
            float k1v[EPL], v1v[EPL];
            load_row<T, EPL>(k1h + (long)j * p.k1.n, D, lane, k1v);
            load_row<T, EPL>(v1h + (long)j * p.v1.n, D, lane, v1v);
            const float s = warp_sum(dot<EPL>(a, k1v));
            const float dP = warp_sum(dot<EPL>(c, v1v));
            const float dS = __expf(s - L) * (dP - delta);
#pragma unroll
            for (int e = 0; e < EPL; ++e) g[e] = fmaf(dS, k1v[e], g[e]);
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] = fmaf(g[e], k2v[e] * p.scale, acc[e]);
    }
    store_row<T, EPL>(dq + b * p.dq.b + (long)i * p.dq.n + h * p.dq.h, D, lane, acc);
}

// dK1 and dV1: warp per (b, hkv, K1 buffer row); loops over the group's query heads.
template <typename T, int EPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
bwd_kv1_kernel(KParams p, const T* __restrict__ q, const T* __restrict__ k1, const T* __restrict__ k2,
               const T* __restrict__ v1, const T* __restrict__ v2, const T* __restrict__ o,
               const float* __restrict__ lse, const T* __restrict__ d_o, T* __restrict__ dk1, T* __restrict__ dv1) {
    const long row = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= (long)p.B * p.Hkv * p.n1) return;
    const int jb = (int)(row % p.n1);
    const int hk = (int)((row / p.n1) % p.Hkv);
    const int b = (int)(row / p.n1 / p.Hkv);
    const int D = p.D;
    float k1v[EPL], v1v[EPL], acck[EPL], accv[EPL];
    load_row<T, EPL>(k1 + b * p.k1.b + (long)jb * p.k1.n + hk * p.k1.h, D, lane, k1v);
    load_row<T, EPL>(v1 + b * p.v1.b + (long)jb * p.v1.n + hk * p.v1.h, D, lane, v1v);
#pragma unroll
    for (int e = 0; e < EPL; ++e) { acck[e] = 0.f; accv[e] = 0.f; }
    const T* k2h = k2 + b * p.k2.b + hk * p.k2.h;
    const T* v2h = v2 + b * p.v2.b + hk * p.v2.h;
    const int i_lo = max(0, jb - p.halo1), i_hi = min(p.N - 1, jb - p.halo1 + p.w1 - 1);
    for (int hq = 0; hq < p.G; ++hq) {
        const int h = hk * p.G + hq;
        for (int i = i_lo; i <= i_hi; ++i) {
            float qv[EPL], dov[EPL], delta, L;
            load_query<T, EPL>(p, q, o, d_o, lse, b, h, i, lane, qv, dov, delta, L);
            const int k_hi = i + p.halo2, k_lo = max(0, k_hi - p.w2 + 1);
            for (int k = k_lo; k <= k_hi; ++k) {
                float a[EPL], c[EPL];
                load_row<T, EPL>(k2h + (long)k * p.k2.n, D, lane, a, p.k2_bias);
                load_row<T, EPL>(v2h + (long)k * p.v2.n, D, lane, c, p.v2_bias);
#pragma unroll
                for (int e = 0; e < EPL; ++e) { a[e] *= qv[e] * p.scale; c[e] *= dov[e]; }
                const float s = warp_sum(dot<EPL>(a, k1v));
                const float dP = warp_sum(dot<EPL>(c, v1v));
                const float P = __expf(s - L);
                const float dS = P * (dP - delta);
#pragma unroll
                for (int e = 0; e < EPL; ++e) { acck[e] = fmaf(dS, a[e], acck[e]); accv[e] = fmaf(P, c[e], accv[e]); }
            }
        }
    }
    if (dk1) store_row<T, EPL>(dk1 + b * p.dk1.b + (long)jb * p.dk1.n + hk * p.dk1.h, D, lane, acck);
    if (dv1) store_row<T, EPL>(dv1 + b * p.dv1.b + (long)jb * p.dv1.n + hk * p.dv1.h, D, lane, accv);
}

// dK2 and dV2: warp per (b, hkv, K2 buffer row).
template <typename T, int EPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
bwd_kv2_kernel(KParams p, const T* __restrict__ q, const T* __restrict__ k1, const T* __restrict__ k2,
               const T* __restrict__ v1, const T* __restrict__ v2, const T* __restrict__ o,
               const float* __restrict__ lse, const T* __restrict__ d_o, T* __restrict__ dk2, T* __restrict__ dv2) {
    const long row = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= (long)p.B * p.Hkv * p.n2) return;
    const int kb = (int)(row % p.n2);
    const int hk = (int)((row / p.n2) % p.Hkv);
    const int b = (int)(row / p.n2 / p.Hkv);
    const int D = p.D;
    float k2v[EPL], v2v[EPL], acck[EPL], accv[EPL];
    load_row<T, EPL>(k2 + b * p.k2.b + (long)kb * p.k2.n + hk * p.k2.h, D, lane, k2v, p.k2_bias);
    load_row<T, EPL>(v2 + b * p.v2.b + (long)kb * p.v2.n + hk * p.v2.h, D, lane, v2v, p.v2_bias);
#pragma unroll
    for (int e = 0; e < EPL; ++e) { acck[e] = 0.f; accv[e] = 0.f; }
    const T* k1h = k1 + b * p.k1.b + hk * p.k1.h;
    const T* v1h = v1 + b * p.v1.b + hk * p.v1.h;
    const int i_lo = max(0, kb - p.halo2), i_hi = min(p.N - 1, kb - p.halo2 + p.w2 - 1);
    for (int hq = 0; hq < p.G; ++hq) {
        const int h = hk * p.G + hq;
        for (int i = i_lo; i <= i_hi; ++i) {
            float qv[EPL], dov[EPL], delta, L;
            load_query<T, EPL>(p, q, o, d_o, lse, b, h, i, lane, qv, dov, delta, L);
            float a[EPL], c[EPL], g[EPL], u[EPL];
#pragma unroll
            for (int e = 0; e < EPL; ++e) { a[e] = qv[e] * k2v[e] * p.scale; c[e] = dov[e] * v2v[e]; g[e] = 0.f; u[e] = 0.f; }
            const int j_hi = i + p.halo1, j_lo = max(0, j_hi - p.w1 + 1);
            for (int j = j_lo; j <= j_hi; ++j) {
                float k1v[EPL], v1v[EPL];
                load_row<T, EPL>(k1h + (long)j * p.k1.n, D, lane, k1v);
                load_row<T, EPL>(v1h + (long)j * p.v1.n, D, lane, v1v);
                const float s = warp_sum(dot<EPL>(a, k1v));
                const float dP = warp_sum(dot<EPL>(c, v1v));
                const float P = __expf(s - L);
                const float dS = P * (dP - delta);
#pragma unroll
                for (int e = 0; e < EPL; ++e) { g[e] = fmaf(dS, k1v[e], g[e]); u[e] = fmaf(P, v1v[e], u[e]); }
            }
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                acck[e] = fmaf(g[e], qv[e] * p.scale, acck[e]);
                accv[e] = fmaf(u[e], dov[e], accv[e]);
            }
        }
    }
    if (dk2) store_row<T, EPL>(dk2 + b * p.dk2.b + (long)kb * p.dk2.n + hk * p.dk2.h, D, lane, acck);
    if (dv2) store_row<T, EPL>(dv2 + b * p.dv2.b + (long)kb * p.dv2.n + hk * p.dv2.h, D, lane, accv);
}

template <typename T, int EPL>
cudaError_t launch_fwd_t(const KParams& p, const void* q, const void* k1, const void* k2, const void* v1,
                         const void* v2, void* o, float* lse, cudaStream_t st) {
    const long rows = (long)p.B * p.H * p.N;
    const unsigned blocks = (unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    fwd_kernel<T, EPL><<<blocks, kWarpsPerBlock * 32, 0, st>>>(p, (const T*)q, (const T*)k1, (const T*)k2,
                                                               (const T*)v1, (const T*)v2, (T*)o, lse);
    return cudaGetLastError();
}

template <typename T, int EPL>
cudaError_t launch_bwd_t(const KParams& p, const void* q, const void* k1, const void* k2, const void* v1,
                         const void* v2, const void* o, const float* lse, const void* d_o, void* dq, void* dk1,
                         void* dk2, void* dv1, void* dv2, cudaStream_t st) {
    const int th = kWarpsPerBlock * 32;
    auto nblk = [](long rows) { return (unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock); };
    if (dq) {
        bwd_dq_kernel<T, EPL><<<nblk((long)p.B * p.H * p.N), th, 0, st>>>(
            p, (const T*)q, (const T*)k1, (const T*)k2, (const T*)v1, (const T*)v2, (const T*)o, lse, (const T*)d_o, (T*)dq);
    }
    if (dk1 || dv1) {
        bwd_kv1_kernel<T, EPL><<<nblk((long)p.B * p.Hkv * p.n1), th, 0, st>>>(
            p, (const T*)q, (const T*)k1, (const T*)k2, (const T*)v1, (const T*)v2, (const T*)o, lse, (const T*)d_o,
            (T*)dk1, (T*)dv1);
    }
    if (dk2 || dv2) {
        bwd_kv2_kernel<T, EPL><<<nblk((long)p.B * p.Hkv * p.n2), th, 0, st>>>(
            p, (const T*)q, (const T*)k1, (const T*)k2, (const T*)v1, (const T*)v2, (const T*)o, lse, (const T*)d_o,
            (T*)dk2, (T*)dv2);
    }
    return cudaGetLastError();
}

// Dispatch on dtype and head dim (elements per lane = ceil(D / 32)).
#define SA_GENERAL_DISPATCH(FN, ...)                                                         \
    do {                                                                                     \
        const int epl = (p.D + 31) / 32;                                                     \
        const int key = dtype * 16 + (epl <= 1 ? 1 : epl <= 2 ? 2 : epl <= 4 ? 4 : 8);       \
        switch (key) {                                                                       \
            case 0 * 16 + 1: return FN<__nv_bfloat16, 1>(__VA_ARGS__);                       \
            case 0 * 16 + 2: return FN<__nv_bfloat16, 2>(__VA_ARGS__);                       \
            case 0 * 16 + 4: return FN<__nv_bfloat16, 4>(__VA_ARGS__);                       \
            case 0 * 16 + 8: return FN<__nv_bfloat16, 8>(__VA_ARGS__);                       \
            case 1 * 16 + 1: return FN<__half, 1>(__VA_ARGS__);                              \
            case 1 * 16 + 2: return FN<__half, 2>(__VA_ARGS__);                              \
            case 1 * 16 + 4: return FN<__half, 4>(__VA_ARGS__);                              \
            case 1 * 16 + 8: return FN<__half, 8>(__VA_ARGS__);                              \
            case 2 * 16 + 1: return FN<float, 1>(__VA_ARGS__);                               \
            case 2 * 16 + 2: return FN<float, 2>(__VA_ARGS__);                               \
            case 2 * 16 + 4: return FN<float, 4>(__VA_ARGS__);                               \
            case 2 * 16 + 8: return FN<float, 8>(__VA_ARGS__);                               \
            default: return cudaErrorInvalidValue;                                           \
        }                                                                                    \
    } while (0)

inline cudaError_t launch_fwd(int dtype, const KParams& p, const void* q, const void* k1, const void* k2,
                              const void* v1, const void* v2, void* o, float* lse, cudaStream_t st) {
    SA_GENERAL_DISPATCH(launch_fwd_t, p, q, k1, k2, v1, v2, o, lse, st);
}

inline cudaError_t launch_bwd(int dtype, const KParams& p, const void* q, const void* k1, const void* k2,
                              const void* v1, const void* v2, const void* o, const float* lse, const void* d_o,
                              void* dq, void* dk1, void* dk2, void* dv1, void* dv2, cudaStream_t st) {
    SA_GENERAL_DISPATCH(launch_bwd_t, p, q, k1, k2, v1, v2, o, lse, d_o, dq, dk1, dk2, dv1, dv2, st);
}

}  // namespace general
}  // namespace sa
