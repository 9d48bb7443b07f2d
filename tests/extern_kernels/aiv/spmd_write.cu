// External-kernel fixture: every SPMD block writes float(block_idx) one cache line apart,
//   out[(base_cl + block_idx) * FLOATS_PER_CACHE_LINE] = float(block_idx)
// (the behaviour of the reference's fixture tests/st/runtime/external_kernel/kernels/aiv/spmd_write.cpp,
// written for CUDA).  The constant comes from a sibling directory through a relative include, so the
// test also shows that the source is compiled where it lies.
//   args[0] = out tensor (INOUT), args[1] = scalar base_cl
#include <cstdint>

#include "pypto_b200_device.h"

#include "../common/cacheline_offset.h"

extern "C" __global__ void kernel_entry(const int64_t* args) {
  float* out = pto_tensor_ptr<float>(args, 0);
  const int32_t base_cl = pto_scalar<int32_t>(args, 1);
  const int32_t block_idx = pto_block_idx();
  if (threadIdx.x == 0) out[(base_cl + block_idx) * FLOATS_PER_CACHE_LINE] = static_cast<float>(block_idx);
}
