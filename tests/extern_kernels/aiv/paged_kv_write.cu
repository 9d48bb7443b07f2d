// External-kernel fixture: write new K (or V) rows of every sequence into a paged cache through its
// block table -- the inverse of the block-table gather.  Logical token t of sequence b lives in pool row
//   block_table[b * max_blocks + t / block_size] * block_size + t % block_size      (one KV head).
//   args[0] rows   bf16 [sum(count), head_dim]  new rows, sequences back to back          (IN)
//   args[1] pool   bf16 [pool_rows, head_dim]                                              (INOUT)
//   args[2] block_table int32 [batch * max_blocks]   args[3] start int32 [batch] first position written
//   args[4] count int32 [batch] rows per sequence    args[5] offset int32 [batch] exclusive prefix of count
//   args[6] block_size, args[7] max_blocks, args[8] head_dim (scalars)
// One SPMD block takes sequences block_idx, block_idx + block_num, ...; its threads copy 4-byte words.
#include <cstdint>

#include "pypto_b200_device.h"

extern "C" __global__ void kernel_entry(const int64_t* args) {
  const uint32_t* rows = pto_tensor_ptr<const uint32_t>(args, 0);
  uint32_t* pool = pto_tensor_ptr<uint32_t>(args, 1);
  const int32_t* block_table = pto_tensor_ptr<const int32_t>(args, 2);
  const int32_t* start = pto_tensor_ptr<const int32_t>(args, 3);
  const int32_t* count = pto_tensor_ptr<const int32_t>(args, 4);
  const int32_t* offset = pto_tensor_ptr<const int32_t>(args, 5);
  const int batch = static_cast<int>(pto_tensor_numel(args, 3));
  const int block_size = pto_scalar<int>(args, 6);
  const int max_blocks = pto_scalar<int>(args, 7);
  const int words = pto_scalar<int>(args, 8) / 2;   // bf16 pairs per row
  for (int b = pto_block_idx(); b < batch; b += pto_block_num()) {
    for (int i = 0; i < count[b]; ++i) {
      const int t = start[b] + i;
      const int64_t dst = static_cast<int64_t>(block_table[b * max_blocks + t / block_size]) * block_size + t % block_size;
      const int64_t src = offset[b] + i;
      for (int w = threadIdx.x; w < words; w += blockDim.x) pool[dst * words + w] = rows[src * words + w];
    }
  }
}
