/* Device-side view of the arguments of an external kernel launched by pto_run_kernel.
 *
 * An external kernel is the reference's way to attach hand-written device code to a program
 * (`@pl.function(type=AIV, external_source=...)`, `@pl.jit.extern`): the entry point receives
 * one array, tensors first as pointers to tensor descriptors, then the scalars bit-cast to
 * 64 bits (python/pypto/backend/pto_backend.py:541-629, 898-915; the reference's example
 * tests/st/runtime/external_kernel/kernels/aiv/spmd_write.cpp:59-69 reads
 * `ChipTensor::buffer.addr` and `start_offset` exactly like pto_tensor_ptr below).
 *
 *   #include "pypto_b200_device.h"
 *   extern "C" __global__ void kernel_entry(const int64_t* args) {
 *     float* out = pto_tensor_ptr<float>(args, 0);
 *     int base = pto_scalar<int>(args, 1);
 *     if (threadIdx.x == 0) out[(base + pto_block_idx()) * 16] = float(pto_block_idx());
 *   }
 *
 * One SPMD block of the reference is one CTA: pto_block_idx() / pto_block_num().
 */
#ifndef PYPTO_B200_DEVICE_H_
#define PYPTO_B200_DEVICE_H_

#include <stdint.h>

#include "pypto_b200.h"

#if defined(__CUDACC__)

__device__ __forceinline__ const pto_chip_tensor* pto_tensor(const int64_t* args, int i) {
  return reinterpret_cast<const pto_chip_tensor*>(static_cast<uintptr_t>(args[i]));
}

/* First element of tensor argument i (base address advanced by start_offset elements). */
template <typename T>
__device__ __forceinline__ T* pto_tensor_ptr(const int64_t* args, int i) {
  const pto_chip_tensor* t = pto_tensor(args, i);
  return reinterpret_cast<T*>(static_cast<uintptr_t>(t->addr)) + t->start_offset;
}

/* Number of elements of tensor argument i. */
__device__ __forceinline__ uint64_t pto_tensor_numel(const int64_t* args, int i) {
  const pto_chip_tensor* t = pto_tensor(args, i);
  uint64_t n = 1;
  for (uint32_t d = 0; d < t->ndims; ++d) n *= t->shapes[d];
  return n;
}

/* Scalar argument i (its position in the whole argument list): integers are passed sign-extended
 * to 64 bits, fp32 as its bit pattern in the low 32 bits, fp64 as its bit pattern. */
template <typename T>
__device__ __forceinline__ T pto_scalar(const int64_t* args, int i) {
  return static_cast<T>(args[i]);
}
template <>
__device__ __forceinline__ float pto_scalar<float>(const int64_t* args, int i) {
  return __uint_as_float(static_cast<uint32_t>(args[i]));
}
template <>
__device__ __forceinline__ double pto_scalar<double>(const int64_t* args, int i) {
  return __longlong_as_double(args[i]);
}

__device__ __forceinline__ int32_t pto_block_idx() { return static_cast<int32_t>(blockIdx.x); }
__device__ __forceinline__ int32_t pto_block_num() { return static_cast<int32_t>(gridDim.x); }

/* ---- reporting instead of faulting ----
 * The worker's device error word (four int32: code, site, block, detail) is what pto_device_status /
 * ChipWorker.device_status() reads and clears after a call.  A kernel that meets a condition it cannot continue
 * from records it there and returns; it never traps and never spins without a bound.  The first report wins.
 * Codes: 1 = a bounded wait ran out (PTO_DEVICE_TIMEOUT on the host), 2 = a block id or row outside its pool,
 * 3 = an index or count outside its array (both PTO_INVALID_ARGUMENT on the host). */
#define PTO_ERR_WAIT_TIMEOUT 1
#define PTO_ERR_BAD_BLOCK 2
#define PTO_ERR_BAD_INDEX 3

__device__ __forceinline__ int32_t* pto_error_word(const int64_t* args) {
  return reinterpret_cast<int32_t*>(static_cast<uintptr_t>(args[-2]));   /* header slot in front of the arguments */
}

__device__ __forceinline__ void pto_report_error(const int64_t* args, int32_t code, int32_t site, int32_t detail) {
  int32_t* w = pto_error_word(args);
  if (atomicCAS(w, 0, code) == 0) {
    w[1] = site;
    w[2] = static_cast<int32_t>(blockIdx.x);
    w[3] = detail;
    __threadfence();
  }
}

/* Spins until *flag == expected or `timeout_ns` of wall time have passed (%globaltimer).  Returns false on timeout;
 * the caller reports and returns.  The waiter and whoever sets the flag must be able to run at the same time:
 * blocks of one cooperative launch, or another device or the host -- never a later launch on the same GPU. */
__device__ __forceinline__ bool pto_bounded_wait(const volatile int32_t* flag, int32_t expected, uint64_t timeout_ns) {
  uint64_t t0, t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (*flag == expected) return true;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > timeout_ns) return false;
  }
}

#endif /* __CUDACC__ */
#endif /* PYPTO_B200_DEVICE_H_ */
