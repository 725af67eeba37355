// The tensor-core backward for bf16 tensors: this translation unit holds the instantiation, so that it
// compiles beside the other element type's and the rest of the library instead of after them.
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/simplicial_attn_b200.h"
#include "sa_common.cuh"
#define SA_TC_BWD_INSTANTIATE
#include "sa_tc_bwd.cuh"

namespace sa {
namespace tc {

template int launch_bwd_t<false>(const KParams&, const void*, const void*, const void*, const void*, const void*, const void*,
                                 const float*, const void*, void*, void*, void*, void*, void*, uint8_t*, DeviceStatus*, cudaStream_t,
                                 int*, MakeMapFn, int, uint64_t);

}  // namespace tc
}  // namespace sa
