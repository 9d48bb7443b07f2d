// External-kernel fixture with two tensors and an fp32 scalar: y[i] = alpha * x[i] + y[i], grid-stride.
// The product and the sum are rounded separately (no fused multiply-add) so that the result is
// bit-identical to the same expression evaluated by torch on the host.
//   args[0] = x (IN), args[1] = y (INOUT), args[2] = alpha (fp32 bits)
#include <cstdint>

#include "pypto_b200_device.h"

extern "C" __global__ void kernel_entry(const int64_t* args) {
  const float* x = pto_tensor_ptr<const float>(args, 0);
  float* y = pto_tensor_ptr<float>(args, 1);
  const float alpha = pto_scalar<float>(args, 2);
  const uint64_t n = pto_tensor_numel(args, 1);
  for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<uint64_t>(gridDim.x) * blockDim.x)
    y[i] = __fadd_rn(__fmul_rn(alpha, x[i]), y[i]);
}
