// External-kernel fixture for the failure path: block 0 waits, with a bound, for a flag that the test never sets.
// When the wait runs out the kernel records PTO_ERR_WAIT_TIMEOUT in the worker's error word and returns; it does
// not trap and does not spin on.  When the flag is already set it writes 1.0 to out[0].
//   args[0] = flag (IN, int32 [1]), args[1] = out (INOUT, fp32 [1]), args[2] = timeout in microseconds
#include <cstdint>

#include "pypto_b200_device.h"

extern "C" __global__ void kernel_entry(const int64_t* args) {
  const int32_t* flag = pto_tensor_ptr<const int32_t>(args, 0);
  float* out = pto_tensor_ptr<float>(args, 1);
  const uint64_t timeout_ns = static_cast<uint64_t>(pto_scalar<int64_t>(args, 2)) * 1000ull;
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  if (!pto_bounded_wait(flag, 1, timeout_ns)) {
    pto_report_error(args, PTO_ERR_WAIT_TIMEOUT, 900, *flag);
    return;
  }
  out[0] = 1.0f;
}
