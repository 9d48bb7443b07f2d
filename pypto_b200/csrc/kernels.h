// Internal launcher declarations shared by the C API and the operator registry.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace pto {

// paged_attention.cu
bool pa_fast_path_ok(int head_dim, int block_size);
size_t pa_scratch_bytes(int batch, int num_heads, int kv_heads, int q_len);
int pa_launch(const void* q, const void* kc, const void* vc, const int32_t* block_table,
              const int32_t* context_lens, void* out, int out_fp32, int batch, int num_heads,
              int kv_heads, int head_dim, int block_size, int max_blocks, int64_t pool_blocks,
              int q_len, float scale, void* scratch, size_t scratch_bytes, cudaStream_t stream);

// paged_gather.cu
int paged_gather_launch(const void* src, int64_t src_rows, int64_t src_cols, int elem_bytes,
                        const int32_t* indices, int64_t n_indices, const int32_t* block_table,
                        int64_t table_len, int block_size, int64_t col_off, int64_t size, void* out,
                        int32_t* err, cudaStream_t stream);

}  // namespace pto
