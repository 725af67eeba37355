// Shared definitions of the 2-simplicial attention kernels: the device-side problem descriptor and
// the dtype load/store helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/simplicial_attn_b200.h"

namespace sa {

// Problem descriptor handed to every kernel by value.  Windows are already clipped to the row
// counts (a window wider than the buffer behaves like one exactly as wide).
struct KParams {
    int B, N, H, Hkv, D, G;      // G = H / Hkv query heads per KV head
    int w1, w2;                  // effective windows
    int halo1, halo2;            // leading halo rows of K1/V1 and K2/V2
    int n1, n2;                  // rows of K1/V1 (N + halo1) and K2/V2 (N + halo2)
    float scale, k2_bias, v2_bias;
    sa_strides q, k1, k2, v1, v2, o, d_o, dq, dk1, dk2, dv1, dv2;
};

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Device status word kept in the first bytes of the caller's workspace.
struct DeviceStatus {
    int code;        // 0 or SA_ERR_DEVICE_TIMEOUT
    int where;       // id of the wait that gave up
    int block;       // block that recorded it
    int pad;
};

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace sa
