// Block-table row gather: the integer, bit-exact contract of `pl.paged_gather`
// (src/ir/op/tensor_ops/paged_gather.cpp:63-169;
//  tests/st/runtime/ops/test_paged_gather.py:14-17):
//   phys = block_table[idx / block_size] * block_size + idx % block_size
//   out[i, :] = src[phys, col_off : col_off + size]
// One warp per gathered row, 16-byte copies when the row slice allows it.
#include "common.cuh"
#include "kernels.h"

namespace pto {
namespace {

__global__ void __launch_bounds__(256)
paged_gather_kernel(const uint8_t* __restrict__ src, int64_t src_rows, int64_t row_bytes,
                    const int32_t* __restrict__ indices, int64_t n_indices,
                    const int32_t* __restrict__ block_table, int64_t table_len, int block_size,
                    int64_t off_bytes, int64_t copy_bytes, uint8_t* __restrict__ out, int32_t* err) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
       i < n_indices; i += warps_total) {
    const int64_t idx = indices[i];
    const int64_t lb = idx / block_size;
    int64_t phys = -1;
    if (idx >= 0 && lb < table_len)
      phys = static_cast<int64_t>(block_table[lb]) * block_size + (idx - lb * block_size);
    uint8_t* dst = out + i * copy_bytes;
    if (phys < 0 || phys >= src_rows) {
      if (lane == 0) report_error(err, kErrBadBlockId, 3, static_cast<int>(i));
      for (int64_t c = lane; c < copy_bytes; c += 32) dst[c] = 0;
      continue;
    }
    const uint8_t* s = src + phys * row_bytes + off_bytes;
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(dst) | copy_bytes) & 15) == 0) {
      const uint4* s4 = reinterpret_cast<const uint4*>(s);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (int64_t c = lane; c < copy_bytes / 16; c += 32) d4[c] = s4[c];
    } else {
      for (int64_t c = lane; c < copy_bytes; c += 32) dst[c] = s[c];
    }
  }
}

}  // namespace

int paged_gather_launch(const void* src, int64_t src_rows, int64_t src_cols, int elem_bytes,
                        const int32_t* indices, int64_t n_indices, const int32_t* block_table,
                        int64_t table_len, int block_size, int64_t col_off, int64_t size, void* out,
                        int32_t* err, cudaStream_t stream) {
  PTO_REQUIRE(elem_bytes > 0 && block_size > 0, "paged_gather: bad element or block size");
  PTO_REQUIRE(col_off >= 0 && size >= 0 && col_off + size <= src_cols, "paged_gather: column slice out of range");
  PTO_REQUIRE(n_indices >= 0 && table_len >= 0 && src_rows >= 0, "paged_gather: negative size");
  if (n_indices == 0 || size == 0) return kOk;
  const int warps_per_cta = 8;
  int64_t ctas = (n_indices + warps_per_cta - 1) / warps_per_cta;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (ctas > cap) ctas = cap;
  launch_kernel(paged_gather_kernel, dim3(static_cast<unsigned>(ctas)), dim3(warps_per_cta * 32), 0, stream, 
      static_cast<const uint8_t*>(src), src_rows, src_cols * elem_bytes, indices, n_indices,
      block_table, table_len, block_size, col_off * elem_bytes, size * elem_bytes,
      static_cast<uint8_t*>(out), err);
  return check_cuda(cudaGetLastError(), "paged_gather_kernel launch");
}

}  // namespace pto
