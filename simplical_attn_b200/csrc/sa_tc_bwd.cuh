// Backward 2-simplicial attention on the sm_100a tensor cores.
#pragma once

#include "sa_ptx.cuh"

namespace sa {
namespace tc {

inline size_t bwd_workspace_bytes(const KParams& k) {
    (void)k;
    return 0;
}

// Returns an sa_status, or -1 when the tensor-core backward does not cover the problem.
inline int launch_bwd(const KParams& k, const void* q, const void* k1, const void* k2, const void* v1, const void* v2,
                      const void* o, const float* lse, const void* d_o, void* dq, void* dk1, void* dk2, void* dv1,
                      void* dv2, uint8_t* workspace, DeviceStatus* status, cudaStream_t st, int* nlaunch) {
    return -1;
}

}  // namespace tc
}  // namespace sa
