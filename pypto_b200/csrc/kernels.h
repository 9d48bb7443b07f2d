// Internal launcher declarations shared by the C API and the operator registry.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "pypto_b200.h"

namespace pto {

// paged_attention.cu
bool pa_fast_path_ok(int head_dim, int block_size);
size_t pa_scratch_bytes(int batch, int num_heads, int kv_heads, int q_len);
int pa_launch(const void* q, const void* kc, const void* vc, const int32_t* block_table,
              const int32_t* context_lens, void* out, int out_fp32, int batch, int num_heads,
              int kv_heads, int head_dim, int block_size, int max_blocks, int64_t pool_blocks,
              int q_len, float scale, void* scratch, size_t scratch_bytes, cudaStream_t stream);

size_t pa_static_scratch_capacity();
int pa_launch_static(const void* q, const void* kc, const void* vc, const int32_t* block_table,
                     const int32_t* context_lens, void* out, int out_fp32, int batch, int num_heads,
                     int kv_heads, int head_dim, int block_size, int max_blocks, int64_t pool_blocks,
                     int q_len, float scale, int32_t* status_dev, cudaStream_t stream);

// paged_gather.cu
int paged_gather_launch(const void* src, int64_t src_rows, int64_t src_cols, int elem_bytes,
                        const int32_t* indices, int64_t n_indices, const int32_t* block_table,
                        int64_t table_len, int block_size, int64_t col_off, int64_t size, void* out,
                        int32_t* err, cudaStream_t stream);

// gemm.cu
enum GemmEpi : int { kGemmEpiStore = 0, kGemmEpiAtomic = 1, kGemmEpiSwiglu = 2 };
// D[a_row, b_row] = sum_k A[a_row, k] * B[b_row, k]; A [a_rows, k], B [b_rows_total, k] bf16 K-major.
// Only the first b_rows rows of B form output columns; with the SwiGLU epilogue the tile at
// row offset dual_off supplies the second operand.  swap: output written transposed.
int gemm_bf16_launch(const void* a, int a_rows, const void* b, int b_rows_total, int b_rows, int k, void* out,
                     long long ldo, int out_bf16, int swap, int epi, int dual_off, int bn, int k_chunks,
                     int* err, cudaStream_t stream);
// gemm2.cu: the same product on CTA pairs (tcgen05.mma.cta_group::2), whole 256 x 256 tiles, store or SwiGLU epilogue
bool gemm2_eligible(int a_rows, int b_rows, int k, int epi, int swap, int bn, int dual);
int gemm2_bf16_launch(const void* a, int a_rows, const void* b, int b_rows_total, int b_rows, int k, void* out, long long ldo,
                      int out_bf16, int epi, int dual_off, int* err, cudaStream_t stream);

// linear.cpp
int linear_launch(const void* x, const void* w_packed, float* out, int m, int n, int k, int accumulate, int* err,
                  cudaStream_t stream);
size_t ffn_workspace_bytes(int m, int inter);
size_t ffn_f32_workspace_bytes(int m, int k, int inter);
size_t ffn_act_workspace_bytes(int m, int inter);
int ffn_act_launch(const void* x, const void* w_in, const void* w_down, float* out, int m, int k, int inter, int n_out,
                   int kind, float alpha, void* workspace, size_t workspace_bytes, int accumulate, int* err,
                   cudaStream_t stream);
int ffn_swiglu_f32_launch(const float* x, const void* w_gate_up, const void* w_down, float* out, int m, int k, int inter,
                          int n_out, void* workspace, size_t workspace_bytes, int accumulate, int* err,
                          cudaStream_t stream);
int ffn_swiglu_launch(const void* x, const void* w_gate_up, const void* w_down, float* out, int m, int k, int inter,
                      int n_out, void* workspace, size_t workspace_bytes, int accumulate, int* err,
                      cudaStream_t stream);

// ffn_fused.cu
bool ffn_fused_ok(int m, int k, int inter, int n_out);
size_t ffn_fused_workspace_bytes(int inter);
int ffn_fused_launch(const void* x, const void* w_gate_up, const void* w_down, float* out, int m, int k, int inter,
                     int n_out, void* workspace, size_t workspace_bytes, int* err, cudaStream_t stream,
                     const float* x_f32 = nullptr, void* xb = nullptr, int zero_out = 0);

// glue.cu
int rms_norm_launch(const void* x, int x_dtype, const float* gamma, void* out, int out_dtype, long long rows,
                    int hidden, float eps, float* copy_f32, void* zero, size_t zero_bytes, cudaStream_t stream);
int rope_kv_append_launch(const float* qkv, const int32_t* seq_lens, const float* cos_t, const float* sin_t,
                          int table_rows, const int32_t* block_table, int max_blocks, void* k_cache, void* v_cache,
                          void* q_out, int batch, int num_heads, int kv_heads, int head_dim, int block_size,
                          long long pool_blocks, int* err, cudaStream_t stream);
int contiguous_cache_tables_launch(const int32_t* seq_lens, int batch, int kv_heads, int blocks_per_seq,
                                   int32_t* seq_table, int32_t* head_table, int32_t* head_lens, cudaStream_t stream);
int swiglu_act_launch(const float* gate_up, void* act, long long rows, int inter, cudaStream_t stream);
int llama_mini_launch(const float* hidden, const float* mask, const float* cos_emb, const float* sin_emb, const float* wq,
                      const float* wk, const float* wv, const float* w_dense, const float* w_gate, const float* w_up,
                      const float* w_down, const float* w_lm, float* logits, int seq_len, int head_dim, int vocab,
                      cudaStream_t stream);
int cast_launch(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t stream);
int act_rows_launch(const float* h, void* act, long long n, int kind, float alpha, cudaStream_t stream);
int cast_zero_launch(const void* in, int in_dtype, void* out, int out_dtype, long long n, void* zero,
                     size_t zero_bytes, cudaStream_t stream);
int pack_weight_launch(const void* src, int src_dtype, void* dst, int k, int n, cudaStream_t stream);

// moe_route.cu
int moe_topk_launch(const float* scores, const float* bias, int is_logits, int tokens, int experts, int topk,
                    int32_t* idx, float* weights, cudaStream_t stream);
int quantize_rows_launch(const void* x, int x_dtype, void* q, float* scale, long long rows, int cols,
                         cudaStream_t stream);
int moe_dispatch_plan_launch(const int32_t* expert_of, int routes, int buckets, int32_t* counts, int32_t* offsets,
                             int32_t* pos, int32_t* route_at, int32_t* work, int* err, cudaStream_t stream);
int moe_recv_plan_launch(const int32_t* recv_counts, int world, int local_experts, int slot_stride, int capacity,
                         int32_t* counts, int32_t* offsets, int32_t* arrival_of, int32_t* grouped_of, int* err,
                         cudaStream_t stream);
int moe_move_rows_launch(const void* const* src, const long long* src_stride, void* const* dst,
                         const long long* dst_stride, const int* row_bytes, int n_arrays, const int32_t* src_row_of,
                         int div, long long rows, long long src_rows, int* err, cudaStream_t stream);
int scale_rows_launch(const void* x, const float* w, int w_stride, const int32_t* count, int slot_stride,
                      long long rows, int cols, void* y, cudaStream_t stream);
int moe_gather_f32_launch(const float* src, const int32_t* index, long long n, long long n_src, float* dst, int* err,
                          cudaStream_t stream);
// Peer-memory return path of the expert-parallel layer (moe_route.cu): every rank's sorted result buffer and flag
// words, as mapped into this process.
constexpr int kMoeMaxPeers = 32;
struct MoePeerTable {
  uint8_t* back[kMoeMaxPeers];
  int32_t* flags[kMoeMaxPeers];
};
int moe_push_rows_launch(const void* rows, int row_bytes, const int32_t* recv_counts, int world, int local_experts,
                         const int32_t* dst_base, const MoePeerTable& peers, int my_rank, int step, long long dst_rows,
                         long long rows_hint, int* done_counter, int* err, cudaStream_t stream);
int moe_wait_flags_launch(const int32_t* flags, int world, int step, int* err, cudaStream_t stream);
int moe_recv_bases_launch(const int32_t* recv_counts, int world, int local_experts, int32_t* base, cudaStream_t stream);
int moe_combine_launch(const void* rows, const int32_t* pos, const void* shared, int tokens, int topk, int hidden,
                       long long n_rows, void* y_bf16, float* y_f32, cudaStream_t stream);

// moe_gemm.cu
int moe_gemm_fp8_launch(int swiglu, const void* w, const float* w_scale, int experts, int w_rows_per_expert,
                        int n_out, int k, const void* x, const float* x_scale, const int32_t* offsets,
                        int total_rows, const float* route_w, const int32_t* out_rows, void* out, int* err,
                        cudaStream_t stream);

// matmul_mx.cu
int matmul_mx_launch(const void* a, const void* a_scale, int a_scale_layout, const void* b_t, const void* b_scale,
                     int b_scale_layout, const float* acc_in, float* out, int m, int n, int k, int* err,
                     cudaStream_t stream);
int transpose_u8_launch(const void* src, void* dst, long long rows, long long cols, cudaStream_t stream);

}  // namespace pto
