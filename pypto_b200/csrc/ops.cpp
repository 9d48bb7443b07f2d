// Operator registry (name -> adapter from the tensors-first task-argument list to a
// kernel launcher) and the direct C launchers.  The adapters take what a
// registered callable receives through pto_run: device tensors in the order of
// the reference program's orchestration signature, then scalars as uint64.
#include <cstring>
#include <string>

#include "common.cuh"
#include "kernels.h"
#include "pypto_b200.h"
#include "runtime.h"

namespace pto {
namespace {

inline void* tptr(const pto_chip_tensor& t, size_t elem_bytes) {
  return reinterpret_cast<void*>(t.addr + t.start_offset * elem_bytes);
}

inline size_t dtype_bytes(uint32_t d) {
  switch (d) {
    case PTO_FP32: case PTO_INT32: return 4;
    case PTO_BF16: case PTO_FP16: return 2;
    case PTO_INT64: return 8;
    default: return 1;
  }
}

inline float f32_from_bits(uint64_t v) {
  uint32_t b = static_cast<uint32_t>(v & 0xffffffffu);
  float f;
  memcpy(&f, &b, 4);
  return f;
}

inline int64_t numel(const pto_chip_tensor& t) {
  int64_t n = 1;
  for (uint32_t i = 0; i < t.ndims && i < 5; ++i) n *= t.shapes[i];
  return n;
}

// tensors: query, key_cache, value_cache, block_table, context_lens, out
// scalars: batch, num_heads, kv_heads, head_dim, block_size, max_blocks, q_len, scale (fp32 bits)
// (the order of the reference's config tensor, examples/models/04_paged_attention.py:287)
int op_paged_attention(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 6 || a->n_scalars != 8)
    return fail(kInvalidArgument, "paged_attention: expects 6 tensors and 8 scalars");
  const pto_chip_tensor* t = a->tensors;
  const uint64_t* s = a->scalars;
  const int batch = (int)s[0], heads = (int)s[1], kvh = (int)s[2], hd = (int)s[3], bs = (int)s[4];
  const int max_blocks = (int)s[5], q_len = (int)s[6];
  if (t[0].dtype != PTO_BF16 || t[1].dtype != PTO_BF16 || t[2].dtype != PTO_BF16)
    return fail(kInvalidArgument, "paged_attention: query and caches must be bf16");
  if (t[3].dtype != PTO_INT32 || t[4].dtype != PTO_INT32)
    return fail(kInvalidArgument, "paged_attention: block_table and context_lens must be int32");
  if (t[5].dtype != PTO_BF16 && t[5].dtype != PTO_FP32)
    return fail(kInvalidArgument, "paged_attention: out must be bf16 or fp32");
  if (batch < 0 || heads <= 0 || kvh <= 0 || hd <= 0 || bs <= 0 || max_blocks <= 0 || q_len <= 0)
    return fail(kInvalidArgument, "paged_attention: bad geometry scalars");
  if (numel(t[0]) != (int64_t)batch * q_len * heads * hd || numel(t[5]) != numel(t[0]))
    return fail(kInvalidArgument, "paged_attention: query/out size does not match batch*q_len*heads*head_dim");
  if (numel(t[3]) < (int64_t)batch * max_blocks || numel(t[4]) < batch)
    return fail(kInvalidArgument, "paged_attention: block_table/context_lens too small");
  const int64_t rows = numel(t[1]) / hd;
  if (numel(t[2]) != numel(t[1]) || rows % ((int64_t)kvh * bs) != 0)
    return fail(kInvalidArgument, "paged_attention: cache rows must be a multiple of kv_heads*block_size");
  const int64_t pool_blocks = rows / ((int64_t)kvh * bs);
  const size_t need = pa_scratch_bytes(batch, heads, kvh, q_len);
  int st = w->ensure_scratch(need);
  if (st != kOk) return st;
  return pa_launch(tptr(t[0], 2), tptr(t[1], 2), tptr(t[2], 2), static_cast<const int32_t*>(tptr(t[3], 4)),
                   static_cast<const int32_t*>(tptr(t[4], 4)), tptr(t[5], dtype_bytes(t[5].dtype)),
                   t[5].dtype == PTO_FP32, batch, heads, kvh, hd, bs, max_blocks, pool_blocks, q_len,
                   f32_from_bits(s[7]), w->scratch, w->scratch_bytes, w->stream);
}

// tensors: src [rows, cols], indices int32 [n], block_table int32 [m], out [n, size]
// scalars: block_size, col_off, size
int op_paged_gather(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 4 || a->n_scalars != 3)
    return fail(kInvalidArgument, "paged_gather: expects 4 tensors and 3 scalars");
  const pto_chip_tensor* t = a->tensors;
  if (t[0].ndims != 2) return fail(kInvalidArgument, "paged_gather: src must be 2-D");
  if (t[1].dtype != PTO_INT32 || t[2].dtype != PTO_INT32)
    return fail(kInvalidArgument, "paged_gather: indices and block_table must be int32");
  const size_t eb = dtype_bytes(t[0].dtype);
  if (dtype_bytes(t[3].dtype) != eb) return fail(kInvalidArgument, "paged_gather: out dtype differs from src");
  const int64_t n = numel(t[1]), size = (int64_t)a->scalars[2];
  if (numel(t[3]) != n * size) return fail(kInvalidArgument, "paged_gather: out must hold n_indices*size elements");
  int st = w->ensure_scratch(256);
  if (st != kOk) return st;
  return paged_gather_launch(tptr(t[0], eb), t[0].shapes[0], t[0].shapes[1], (int)eb,
                             static_cast<const int32_t*>(tptr(t[1], 4)), n,
                             static_cast<const int32_t*>(tptr(t[2], 4)), numel(t[2]), (int)a->scalars[0],
                             (int64_t)a->scalars[1], size, tptr(t[3], eb), static_cast<int32_t*>(w->scratch),
                             w->stream);
}

// tensors: x [rows, hidden] (fp32 or bf16), gamma fp32 [hidden] (or [1, hidden]), out (fp32 or bf16)
// scalars: eps (fp32 bits)
int op_rms_norm(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 3 || a->n_scalars != 1) return fail(kInvalidArgument, "rms_norm: expects 3 tensors and 1 scalar");
  const pto_chip_tensor* t = a->tensors;
  if (t[0].ndims < 1 || t[1].dtype != PTO_FP32) return fail(kInvalidArgument, "rms_norm: gamma must be fp32");
  const int hidden = (int)t[0].shapes[t[0].ndims - 1];
  if (numel(t[1]) != hidden || numel(t[2]) != numel(t[0]))
    return fail(kInvalidArgument, "rms_norm: gamma/out sizes do not match x");
  return rms_norm_launch(tptr(t[0], dtype_bytes(t[0].dtype)), (int)t[0].dtype, static_cast<const float*>(tptr(t[1], 4)),
                         tptr(t[2], dtype_bytes(t[2].dtype)), (int)t[2].dtype, numel(t[0]) / hidden, hidden,
                         f32_from_bits(a->scalars[0]), nullptr, nullptr, 0, w->stream);
}

// The reference's ffn_swiglu signature (examples/models/01_ffn.py:112-131): all fp32,
// weights in the x @ W layout.  tensors: x [m, k], w_gate [k, i], w_up [k, i], w_down [i, n], out [m, n]
// The operands are cast / packed to bf16 in the worker's scratch arena on every call (a one-shot
// call has nowhere to keep packed weights; resident use goes through pto_pack_weight + pto_ffn_swiglu).
int op_ffn_swiglu(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 5 || a->n_scalars != 0) return fail(kInvalidArgument, "ffn_swiglu: expects 5 tensors");
  const pto_chip_tensor* t = a->tensors;
  for (int i = 0; i < 5; ++i)
    if (t[i].ndims != 2 || (t[i].dtype != PTO_FP32 && !(i < 4 && t[i].dtype == PTO_BF16)))
      return fail(kInvalidArgument, "ffn_swiglu: 2-D fp32 (or bf16 input) tensors expected, fp32 output");
  const int m = t[0].shapes[0], k = t[0].shapes[1], inter = t[1].shapes[1], n = t[3].shapes[1];
  if ((int)t[1].shapes[0] != k || (int)t[2].shapes[0] != k || (int)t[2].shapes[1] != inter ||
      (int)t[3].shapes[0] != inter || (int)t[4].shapes[0] != m || (int)t[4].shapes[1] != n)
    return fail(kInvalidArgument, "ffn_swiglu: operand shapes do not chain");
  auto al = [](size_t v) { return (v + 255) / 256 * 256; };
  const size_t x_b = al((size_t)m * k * 2), gu_b = al((size_t)2 * inter * k * 2), d_b = al((size_t)n * inter * 2);
  const size_t ws_b = ffn_workspace_bytes(m, inter);
  int st = w->ensure_scratch(4096 + x_b + gu_b + d_b + ws_b);
  if (st != kOk) return st;
  uint8_t* base = static_cast<uint8_t*>(w->scratch) + 4096;
  void* xb = base; void* gu = base + x_b; void* wd = base + x_b + gu_b; void* ws = base + x_b + gu_b + d_b;
  if (t[0].dtype == PTO_FP32) st = cast_launch(tptr(t[0], 4), PTO_FP32, xb, PTO_BF16, (long long)m * k, w->stream);
  else st = check_cuda(cudaMemcpyAsync(xb, tptr(t[0], 2), (size_t)m * k * 2, cudaMemcpyDeviceToDevice, w->stream), "copy x");
  if (st != kOk) return st;
  st = pack_weight_launch(tptr(t[1], dtype_bytes(t[1].dtype)), (int)t[1].dtype, gu, k, inter, w->stream);
  if (st != kOk) return st;
  st = pack_weight_launch(tptr(t[2], dtype_bytes(t[2].dtype)), (int)t[2].dtype,
                          static_cast<uint8_t*>(gu) + (size_t)inter * k * 2, k, inter, w->stream);
  if (st != kOk) return st;
  st = pack_weight_launch(tptr(t[3], dtype_bytes(t[3].dtype)), (int)t[3].dtype, wd, inter, n, w->stream);
  if (st != kOk) return st;
  // the arena is shared with other operators, so the FFN's call counter does not survive between calls: clear it
  st = check_cuda(cudaMemsetAsync(ws, 0, ws_b < 8192 ? ws_b : 8192, w->stream), "cudaMemsetAsync(ffn header)");
  if (st != kOk) return st;
  return ffn_swiglu_launch(xb, gu, wd, static_cast<float*>(tptr(t[4], 4)), m, k, inter, n, ws, ws_b, 0,
                           static_cast<int*>(w->scratch), w->stream);
}

struct OpEntry {
  const char* name;
  OpFn fn;
};

// The reference's ffn_gelu / ffn_relu signatures (examples/models/01_ffn.py:92-108, 134-150): fp32 (or bf16 x),
// weights in the x @ W layout.  tensors: x [m, k], w_in [k, i], w_down [i, n], out [m, n];
// scalars: kind (1: x * sigmoid(alpha x), 2: relu), alpha as fp32 bits.  Operands are cast / packed per call.
int op_ffn_act(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 4 || a->n_scalars != 2) return fail(kInvalidArgument, "ffn_act: expects 4 tensors and 2 scalars");
  const pto_chip_tensor* t = a->tensors;
  for (int i = 0; i < 4; ++i)
    if (t[i].ndims != 2 || (t[i].dtype != PTO_FP32 && !(i < 3 && t[i].dtype == PTO_BF16)))
      return fail(kInvalidArgument, "ffn_act: 2-D fp32 (or bf16 input) tensors expected, fp32 output");
  const int m = t[0].shapes[0], k = t[0].shapes[1], inter = t[1].shapes[1], n = t[2].shapes[1];
  if ((int)t[1].shapes[0] != k || (int)t[2].shapes[0] != inter || (int)t[3].shapes[0] != m || (int)t[3].shapes[1] != n)
    return fail(kInvalidArgument, "ffn_act: operand shapes do not chain");
  const int kind = static_cast<int>(a->scalars[0]);
  const uint32_t bits = static_cast<uint32_t>(a->scalars[1]);
  float alpha;
  memcpy(&alpha, &bits, 4);
  auto al = [](size_t v) { return (v + 255) / 256 * 256; };
  const size_t x_b = al((size_t)m * k * 2), in_b = al((size_t)inter * k * 2), d_b = al((size_t)n * inter * 2);
  const size_t ws_b = ffn_act_workspace_bytes(m, inter);
  int st = w->ensure_scratch(4096 + x_b + in_b + d_b + ws_b);
  if (st != kOk) return st;
  uint8_t* base = static_cast<uint8_t*>(w->scratch) + 4096;
  void* xb = base; void* wi = base + x_b; void* wd = base + x_b + in_b; void* ws = base + x_b + in_b + d_b;
  if (t[0].dtype == PTO_FP32) st = cast_launch(tptr(t[0], 4), PTO_FP32, xb, PTO_BF16, (long long)m * k, w->stream);
  else st = check_cuda(cudaMemcpyAsync(xb, tptr(t[0], 2), (size_t)m * k * 2, cudaMemcpyDeviceToDevice, w->stream), "copy x");
  if (st != kOk) return st;
  st = pack_weight_launch(tptr(t[1], dtype_bytes(t[1].dtype)), (int)t[1].dtype, wi, k, inter, w->stream);
  if (st != kOk) return st;
  st = pack_weight_launch(tptr(t[2], dtype_bytes(t[2].dtype)), (int)t[2].dtype, wd, inter, n, w->stream);
  if (st != kOk) return st;
  return ffn_act_launch(xb, wi, wd, static_cast<float*>(tptr(t[3], 4)), m, k, inter, n, kind, alpha, ws, ws_b, 0,
                        static_cast<int*>(w->scratch), w->stream);
}

const OpEntry kOps[] = {
    {"paged_attention", op_paged_attention},
    {"paged_gather", op_paged_gather},
    {"rms_norm", op_rms_norm},
    {"ffn_swiglu", op_ffn_swiglu},
    {"ffn_act", op_ffn_act},
    {"linear", op_linear},
    {"rope_kv_append", op_rope_kv_append},
    {"scope3", op_scope3},
    {"decoder_layer", op_decoder_layer},
    {"matmul_mx", op_matmul_mx},
    {"moe_layer", op_moe_layer},
    {"llama_mini", op_llama_mini},
};

}  // namespace

OpFn find_op(const char* name) {
  for (const OpEntry& e : kOps)
    if (strcmp(e.name, name) == 0) return e.fn;
  return nullptr;
}

}  // namespace pto

extern "C" {

const char* pto_op_list(void) {
  static std::string names;
  if (names.empty()) {
    for (const pto::OpEntry& e : pto::kOps) {
      names += e.name;
      names.push_back('\0');
    }
    names.push_back('\0');
  }
  return names.c_str();
}

size_t pto_paged_attention_scratch_bytes(int batch, int num_heads, int kv_heads, int q_len) {
  if (batch < 0 || num_heads <= 0 || kv_heads <= 0 || q_len <= 0) return 0;
  return pto::pa_scratch_bytes(batch, num_heads, kv_heads, q_len);
}

int pto_paged_attention(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                        const int32_t* context_lens, void* out, int out_dtype, int batch, int num_heads,
                        int kv_heads, int head_dim, int block_size, int max_blocks, int64_t pool_blocks,
                        int q_len, float scale, void* scratch, size_t scratch_bytes, void* stream) {
  if (out_dtype != PTO_BF16 && out_dtype != PTO_FP32)
    return pto::fail(pto::kInvalidArgument, "paged_attention: out_dtype must be PTO_BF16 or PTO_FP32");
  if (!q || !k_cache || !v_cache || !block_table || !context_lens || !out)
    return pto::fail(pto::kInvalidArgument, "paged_attention: NULL tensor");
  return pto::pa_launch(q, k_cache, v_cache, block_table, context_lens, out, out_dtype == PTO_FP32, batch,
                        num_heads, kv_heads, head_dim, block_size, max_blocks, pool_blocks, q_len, scale,
                        scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

int pto_paged_attention_static(const void* q, const void* k_cache, const void* v_cache,
                               const int32_t* block_table, const int32_t* context_lens, void* out, int out_dtype,
                               int batch, int num_heads, int kv_heads, int head_dim, int block_size,
                               int max_blocks, int64_t pool_blocks, int q_len, float scale, int32_t* status_dev,
                               void* stream) {
  if (out_dtype != PTO_BF16 && out_dtype != PTO_FP32)
    return pto::fail(pto::kInvalidArgument, "paged_attention_static: out_dtype must be PTO_BF16 or PTO_FP32");
  if (!q || !k_cache || !v_cache || !block_table || !context_lens || !out)
    return pto::fail(pto::kInvalidArgument, "paged_attention_static: NULL tensor");
  return pto::pa_launch_static(q, k_cache, v_cache, block_table, context_lens, out, out_dtype == PTO_FP32, batch,
                               num_heads, kv_heads, head_dim, block_size, max_blocks, pool_blocks, q_len, scale,
                               status_dev, static_cast<cudaStream_t>(stream));
}

int pto_paged_gather(const void* src, int64_t src_rows, int64_t src_cols, int elem_bytes, const int32_t* indices,
                     int64_t n_indices, const int32_t* block_table, int64_t table_len, int block_size,
                     int64_t col_off, int64_t size, void* out, int32_t* err, void* stream) {
  if (n_indices > 0 && (!src || !indices || !block_table || !out))
    return pto::fail(pto::kInvalidArgument, "paged_gather: NULL tensor");
  return pto::paged_gather_launch(src, src_rows, src_cols, elem_bytes, indices, n_indices, block_table,
                                  table_len, block_size, col_off, size, out, err,
                                  static_cast<cudaStream_t>(stream));
}

int pto_pack_weight(const void* w, int w_dtype, void* packed, int k, int n, void* stream) {
  return pto::pack_weight_launch(w, w_dtype, packed, k, n, static_cast<cudaStream_t>(stream));
}

int pto_cast(const void* in, int in_dtype, void* out, int out_dtype, int64_t n, void* stream) {
  return pto::cast_launch(in, in_dtype, out, out_dtype, n, static_cast<cudaStream_t>(stream));
}

int pto_cast_zero(const void* in, int in_dtype, void* out, int out_dtype, int64_t n, void* zero, size_t zero_bytes,
                  void* stream) {
  return pto::cast_zero_launch(in, in_dtype, out, out_dtype, n, zero, zero_bytes, static_cast<cudaStream_t>(stream));
}

int pto_linear(const void* x, const void* w_packed, void* out, int m, int n, int k, int accumulate, int32_t* err,
               void* stream) {
  return pto::linear_launch(x, w_packed, static_cast<float*>(out), m, n, k, accumulate, err,
                            static_cast<cudaStream_t>(stream));
}

size_t pto_ffn_swiglu_workspace_bytes(int m, int inter) {
  if (m <= 0 || inter <= 0) return 0;
  return pto::ffn_workspace_bytes(m, inter);
}

int pto_ffn_swiglu(const void* x, const void* w_gate_up, const void* w_down, void* out, int m, int k, int inter,
                   int n_out, void* workspace, size_t workspace_bytes, int accumulate, int32_t* err, void* stream) {
  return pto::ffn_swiglu_launch(x, w_gate_up, w_down, static_cast<float*>(out), m, k, inter, n_out, workspace,
                                workspace_bytes, accumulate, err, static_cast<cudaStream_t>(stream));
}

size_t pto_ffn_act_workspace_bytes(int m, int inter) {
  if (m <= 0 || inter <= 0) return 0;
  return pto::ffn_act_workspace_bytes(m, inter);
}

int pto_ffn_act(const void* x, const void* w_in, const void* w_down, void* out, int m, int k, int inter, int n_out, int kind,
                float alpha, void* workspace, size_t workspace_bytes, int accumulate, int32_t* err, void* stream) {
  return pto::ffn_act_launch(x, w_in, w_down, static_cast<float*>(out), m, k, inter, n_out, kind, alpha, workspace,
                             workspace_bytes, accumulate, err, static_cast<cudaStream_t>(stream));
}

size_t pto_ffn_swiglu_f32_workspace_bytes(int m, int k, int inter) {
  if (m <= 0 || k <= 0 || inter <= 0) return 0;
  return pto::ffn_f32_workspace_bytes(m, k, inter);
}

int pto_ffn_swiglu_f32(const float* x, const void* w_gate_up, const void* w_down, void* out, int m, int k, int inter,
                       int n_out, void* workspace, size_t workspace_bytes, int accumulate, int32_t* err, void* stream) {
  return pto::ffn_swiglu_f32_launch(x, w_gate_up, w_down, static_cast<float*>(out), m, k, inter, n_out, workspace,
                                    workspace_bytes, accumulate, err, static_cast<cudaStream_t>(stream));
}

int pto_rms_norm(const void* x, int x_dtype, const float* gamma, void* out, int out_dtype, int64_t rows, int hidden,
                 float eps, void* stream) {
  return pto::rms_norm_launch(x, x_dtype, gamma, out, out_dtype, rows, hidden, eps, nullptr, nullptr, 0,
                              static_cast<cudaStream_t>(stream));
}

int pto_rms_norm_ex(const void* x, int x_dtype, const float* gamma, void* out, int out_dtype, int64_t rows, int hidden,
                    float eps, float* copy_f32, void* zero, size_t zero_bytes, void* stream) {
  return pto::rms_norm_launch(x, x_dtype, gamma, out, out_dtype, rows, hidden, eps, copy_f32, zero, zero_bytes,
                              static_cast<cudaStream_t>(stream));
}

int pto_rope_kv_append(const float* qkv, const int32_t* seq_lens, const float* cos_table, const float* sin_table,
                       int table_rows, const int32_t* block_table, int max_blocks, void* k_cache, void* v_cache,
                       void* q_out, int batch, int num_heads, int kv_heads, int head_dim, int block_size,
                       int64_t pool_blocks, int32_t* err, void* stream) {
  return pto::rope_kv_append_launch(qkv, seq_lens, cos_table, sin_table, table_rows, block_table, max_blocks,
                                    k_cache, v_cache, q_out, batch, num_heads, kv_heads, head_dim, block_size,
                                    pool_blocks, err, static_cast<cudaStream_t>(stream));
}

int pto_llama_mini(const float* hidden, const float* causal_mask, const float* cos_emb, const float* sin_emb,
                   const float* wq, const float* wk, const float* wv, const float* w_dense, const float* w_gate,
                   const float* w_up, const float* w_down, const float* w_lm, float* logits, int seq_len, int head_dim,
                   int vocab, void* stream) {
  return pto::llama_mini_launch(hidden, causal_mask, cos_emb, sin_emb, wq, wk, wv, w_dense, w_gate, w_up, w_down, w_lm,
                                logits, seq_len, head_dim, vocab, static_cast<cudaStream_t>(stream));
}

int pto_swiglu_act(const float* gate_up, void* act, int64_t rows, int inter, void* stream) {
  return pto::swiglu_act_launch(gate_up, act, rows, inter, static_cast<cudaStream_t>(stream));
}

int pto_moe_topk(const float* scores, const float* bias, int is_logits, int tokens, int experts, int topk,
                 int32_t* idx, float* weights, void* stream) {
  return pto::moe_topk_launch(scores, bias, is_logits, tokens, experts, topk, idx, weights,
                              static_cast<cudaStream_t>(stream));
}

int pto_quantize_rows(const void* x, int x_dtype, void* q, float* scale, int64_t rows, int cols, void* stream) {
  return pto::quantize_rows_launch(x, x_dtype, q, scale, rows, cols, static_cast<cudaStream_t>(stream));
}

int pto_moe_dispatch_plan(const int32_t* expert_of, int routes, int buckets, int32_t* counts, int32_t* offsets,
                          int32_t* pos, int32_t* route_at, int32_t* work, int32_t* err, void* stream) {
  return pto::moe_dispatch_plan_launch(expert_of, routes, buckets, counts, offsets, pos, route_at, work, err,
                                       static_cast<cudaStream_t>(stream));
}

int pto_moe_recv_plan(const int32_t* recv_counts, int world, int local_experts, int slot_stride, int capacity,
                      int32_t* counts, int32_t* offsets, int32_t* arrival_of, int32_t* grouped_of, int32_t* err,
                      void* stream) {
  return pto::moe_recv_plan_launch(recv_counts, world, local_experts, slot_stride, capacity, counts, offsets,
                                   arrival_of, grouped_of, err, static_cast<cudaStream_t>(stream));
}

int pto_moe_gather_rows(const void* const* src, void* const* dst, const int* row_bytes, int n_arrays,
                        const int32_t* index, int div, int64_t rows, int64_t src_rows, int32_t* err, void* stream) {
  if (!src || !dst || !row_bytes) return pto::fail(pto::kInvalidArgument, "moe_gather_rows: NULL argument");
  return pto::moe_move_rows_launch(src, nullptr, dst, nullptr, row_bytes, n_arrays, index, div, rows, src_rows, err,
                                   static_cast<cudaStream_t>(stream));
}

int pto_moe_move_rows(const void* const* src, const int64_t* src_stride, void* const* dst, const int64_t* dst_stride,
                      const int* row_bytes, int n_arrays, const int32_t* index, int div, int64_t rows,
                      int64_t src_rows, int32_t* err, void* stream) {
  static_assert(sizeof(long long) == sizeof(int64_t), "stride arrays are passed through as 64-bit integers");
  return pto::moe_move_rows_launch(src, reinterpret_cast<const long long*>(src_stride), dst,
                                   reinterpret_cast<const long long*>(dst_stride), row_bytes, n_arrays, index, div,
                                   rows, src_rows, err, static_cast<cudaStream_t>(stream));
}

int pto_moe_gather_f32(const float* src, const int32_t* index, int64_t n, int64_t n_src, float* dst, int32_t* err,
                       void* stream) {
  return pto::moe_gather_f32_launch(src, index, n, n_src, dst, err, static_cast<cudaStream_t>(stream));
}

int pto_scale_rows(const void* x, const float* w, int w_stride, const int32_t* count, int slot_stride, int64_t rows,
                   int cols, void* y, void* stream) {
  return pto::scale_rows_launch(x, w, w_stride, count, slot_stride, rows, cols, y, static_cast<cudaStream_t>(stream));
}

int pto_moe_expert_gemm(int swiglu, const void* w, const float* w_scale, int experts, int w_rows, int n_out, int k,
                        const void* x, const float* x_scale, const int32_t* offsets, int rows, const float* route_w,
                        const int32_t* out_rows, void* out, int32_t* err, void* stream) {
  return pto::moe_gemm_fp8_launch(swiglu, w, w_scale, experts, w_rows, n_out, k, x, x_scale, offsets, rows, route_w,
                                  out_rows, out, err, static_cast<cudaStream_t>(stream));
}

int pto_moe_combine(const void* rows, const int32_t* pos, const void* shared, int tokens, int topk, int hidden,
                    int64_t n_rows, void* y_bf16, float* y_f32, void* stream) {
  return pto::moe_combine_launch(rows, pos, shared, tokens, topk, hidden, n_rows, y_bf16, y_f32,
                                 static_cast<cudaStream_t>(stream));
}

int pto_moe_push_rows(const void* rows, int row_bytes, const int32_t* recv_counts, int world, int local_experts,
                      const int32_t* dst_base, void* const* back, int32_t* const* flags, int my_rank, int step,
                      int64_t dst_rows, int64_t rows_hint, int32_t* done_counter, int32_t* err, void* stream) {
  if (!back || !flags) return pto::fail(pto::kInvalidArgument, "moe_push_rows: NULL pointer table");
  if (world < 1 || world > pto::kMoeMaxPeers) return pto::fail(pto::kInvalidArgument, "moe_push_rows: 1..32 ranks");
  pto::MoePeerTable t = {};
  for (int r = 0; r < world; ++r) {
    if (!back[r] || !flags[r]) return pto::fail(pto::kInvalidArgument, "moe_push_rows: NULL buffer or flag pointer");
    t.back[r] = static_cast<uint8_t*>(back[r]);
    t.flags[r] = flags[r];
  }
  return pto::moe_push_rows_launch(rows, row_bytes, recv_counts, world, local_experts, dst_base, t, my_rank, step, dst_rows,
                                   rows_hint, done_counter, err, static_cast<cudaStream_t>(stream));
}

int pto_moe_wait_flags(const int32_t* flags, int world, int step, int32_t* err, void* stream) {
  return pto::moe_wait_flags_launch(flags, world, step, err, static_cast<cudaStream_t>(stream));
}

int pto_matmul_mx(const void* a, const void* a_scale, int a_scale_layout, const void* b_t, const void* b_scale,
                  int b_scale_layout, const float* acc_in, float* out, int m, int n, int k, int32_t* err,
                  void* stream) {
  return pto::matmul_mx_launch(a, a_scale, a_scale_layout, b_t, b_scale, b_scale_layout, acc_in, out, m, n, k, err,
                               static_cast<cudaStream_t>(stream));
}

int pto_transpose_u8(const void* src, void* dst, int64_t rows, int64_t cols, void* stream) {
  return pto::transpose_u8_launch(src, dst, rows, cols, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
