// Registered callables that compose several kernels: the decoder layer of the reference's decode example
// and its third scope, a linear layer and the RoPE / cache append in the `x @ W` weight layout the reference
// programs use, and the MX matmul program.  Each adapter receives what pto_run hands a callable: device
// tensors in the order of the reference program's signature, then scalars as uint64.
//
// Weights arrive in the reference's [in, out] layout and are re-packed K-major into the worker's scratch
// arena on every call: a one-shot call has nowhere to keep packed weights (callers that keep weights
// resident use pto_pack_weight once and the direct launchers).
#include <cmath>
#include <cstring>

#include "common.cuh"
#include "kernels.h"
#include "pypto_b200.h"
#include "runtime.h"

namespace pto {
namespace {

inline void* tptr(const pto_chip_tensor& t, size_t elem_bytes) {
  return reinterpret_cast<void*>(t.addr + t.start_offset * elem_bytes);
}
inline size_t al256(size_t v) { return (v + 255) / 256 * 256; }
inline float f32_bits(uint64_t v) {
  const uint32_t b = static_cast<uint32_t>(v & 0xffffffffu);
  float f;
  memcpy(&f, &b, 4);
  return f;
}
inline bool is2d(const pto_chip_tensor& t, uint32_t r, uint32_t c, uint32_t dtype) {
  return t.ndims == 2 && t.shapes[0] == r && t.shapes[1] == c && t.dtype == dtype;
}
inline int64_t numel(const pto_chip_tensor& t) {
  int64_t n = 1;
  for (uint32_t i = 0; i < t.ndims && i < 5; ++i) n *= t.shapes[i];
  return n;
}

// Bump allocator over the worker's scratch arena (after the error word and `reserve` bytes).
struct Arena {
  uint8_t* base;
  size_t used;
  void* take(size_t bytes) {
    void* p = base + used;
    used += al256(bytes);
    return p;
  }
};

// o-proj + residual -> RMSNorm -> SwiGLU MLP -> down-proj + residual -> bf16: scope 3 of the decode layer
// (tests/st/runtime/framework_and_models/test_qwen3_decode_scope3_mixed.py:256-287).  resid (fp32 [b, hidden])
// holds fp32(hidden_states) on entry.
int scope3_body(Worker* w, Arena& a, const void* attn, int q_dim, float* resid, const pto_chip_tensor& wo,
                const pto_chip_tensor& gamma, const pto_chip_tensor& wg, const pto_chip_tensor& wu,
                const pto_chip_tensor& wd, void* out_bf16, int b, int hidden, int inter, float eps) {
  int* err = static_cast<int*>(w->scratch);
  void* wo_p = a.take(static_cast<size_t>(hidden) * q_dim * 2);
  void* wgu_p = a.take(static_cast<size_t>(2) * inter * hidden * 2);
  void* wd_p = a.take(static_cast<size_t>(hidden) * inter * 2);
  void* post = a.take(static_cast<size_t>(b) * hidden * 2);
  const size_t ws_b = ffn_workspace_bytes(b, inter);
  void* ws = a.take(ws_b);
  int st = pack_weight_launch(tptr(wo, 2), PTO_BF16, wo_p, q_dim, hidden, w->stream);
  if (st != kOk) return st;
  st = pack_weight_launch(tptr(wg, 2), PTO_BF16, wgu_p, hidden, inter, w->stream);
  if (st != kOk) return st;
  st = pack_weight_launch(tptr(wu, 2), PTO_BF16, static_cast<uint8_t*>(wgu_p) + static_cast<size_t>(inter) * hidden * 2,
                          hidden, inter, w->stream);
  if (st != kOk) return st;
  st = pack_weight_launch(tptr(wd, 2), PTO_BF16, wd_p, inter, hidden, w->stream);
  if (st != kOk) return st;
  st = linear_launch(attn, wo_p, resid, b, hidden, q_dim, 1, err, w->stream);
  if (st != kOk) return st;
  st = rms_norm_launch(resid, PTO_FP32, static_cast<const float*>(tptr(gamma, 4)), post, PTO_BF16, b, hidden, eps,
                       nullptr, nullptr, 0, w->stream);
  if (st != kOk) return st;
  // the arena is shared with other operators, so the FFN's call counter does not survive between calls: clear it
  st = check_cuda(cudaMemsetAsync(ws, 0, ws_b < 8192 ? ws_b : 8192, w->stream), "cudaMemsetAsync(ffn header)");
  if (st != kOk) return st;
  st = ffn_swiglu_launch(post, wgu_p, wd_p, resid, b, hidden, inter, hidden, ws, ws_b, 1, err, w->stream);
  if (st != kOk) return st;
  return cast_launch(resid, PTO_FP32, out_bf16, PTO_BF16, static_cast<long long>(b) * hidden, w->stream);
}

size_t scope3_bytes(int b, int hidden, int q_dim, int inter) {
  return al256(static_cast<size_t>(hidden) * q_dim * 2) + al256(static_cast<size_t>(2) * inter * hidden * 2) +
         al256(static_cast<size_t>(hidden) * inter * 2) + al256(static_cast<size_t>(b) * hidden * 2) +
         al256(ffn_workspace_bytes(b, inter));
}

}  // namespace

// tensors: attn_out [b, hidden] bf16, hidden_states [b, hidden] bf16, wo [hidden, hidden] bf16, post_rms_weight
// fp32 [1, hidden], w_gate / w_up [hidden, inter] bf16, w_down [inter, hidden] bf16, out [b, hidden] bf16
// scalars: eps (fp32 bits)
int op_scope3(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 8 || a->n_scalars != 1) return fail(kInvalidArgument, "scope3: expects 8 tensors and 1 scalar");
  const pto_chip_tensor* t = a->tensors;
  if (t[0].ndims != 2) return fail(kInvalidArgument, "scope3: attn_out must be 2-D");
  const int b = t[0].shapes[0], hidden = t[1].shapes[1], q_dim = t[0].shapes[1], inter = t[4].shapes[1];
  if (!is2d(t[0], b, q_dim, PTO_BF16) || !is2d(t[1], b, hidden, PTO_BF16) || !is2d(t[2], q_dim, hidden, PTO_BF16) ||
      t[3].dtype != PTO_FP32 || numel(t[3]) != hidden || !is2d(t[4], hidden, inter, PTO_BF16) ||
      !is2d(t[5], hidden, inter, PTO_BF16) || !is2d(t[6], inter, hidden, PTO_BF16) || !is2d(t[7], b, hidden, PTO_BF16))
    return fail(kInvalidArgument, "scope3: tensor shapes or dtypes do not match the program signature");
  if (hidden % 8 || q_dim % 8 || inter % 32) return fail(kInvalidArgument, "scope3: hidden % 8, inter % 32 required");
  const size_t need = 4096 + al256(static_cast<size_t>(b) * hidden * 4) + scope3_bytes(b, hidden, q_dim, inter);
  int st = w->ensure_scratch(need);
  if (st != kOk) return st;
  Arena ar{static_cast<uint8_t*>(w->scratch), 4096};
  float* resid = static_cast<float*>(ar.take(static_cast<size_t>(b) * hidden * 4));
  st = cast_launch(tptr(t[1], 2), PTO_BF16, resid, PTO_FP32, static_cast<long long>(b) * hidden, w->stream);
  if (st != kOk) return st;
  return scope3_body(w, ar, tptr(t[0], 2), q_dim, resid, t[2], t[3], t[4], t[5], t[6], tptr(t[7], 2), b, hidden, inter,
                     f32_bits(a->scalars[0]));
}

// The decode layer of examples/models/qwen3_jit/qwen3_decode.py:49-112 with grouped-query attention over the
// contiguous KV cache in the place the example leaves open (:95-99).
// tensors (the example's order): hidden_states [b, H] bf16, input_rms_weight fp32 [1, H], wq [H, Hq*D],
//   wk, wv [H, Hkv*D] bf16, seq_lens int32 [b], rope_cos, rope_sin fp32 [max_seq, D], k_cache, v_cache bf16
//   [b * Hkv * max_seq, D] (row = (b * Hkv + ki) * max_seq + pos, updated in place at pos = seq_len - 1),
//   wo [Hq*D, H], post_rms_weight fp32 [1, H], w_gate, w_up [H, I], w_down [I, H] bf16, out [b, H] bf16
// scalars: eps (fp32 bits), softmax scale (fp32 bits; 0 = 1 / sqrt(D))
int op_decoder_layer(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 16 || a->n_scalars != 2)
    return fail(kInvalidArgument, "decoder_layer: expects 16 tensors and 2 scalars");
  const pto_chip_tensor* t = a->tensors;
  if (t[0].ndims != 2 || t[6].ndims != 2 || t[2].ndims != 2 || t[3].ndims != 2 || t[12].ndims != 2)
    return fail(kInvalidArgument, "decoder_layer: 2-D tensors expected");
  const int b = t[0].shapes[0], hidden = t[0].shapes[1], q_dim = t[2].shapes[1], kv_dim = t[3].shapes[1];
  const int max_seq = t[6].shapes[0], hd = t[6].shapes[1], inter = t[12].shapes[1];
  if (hd <= 0 || q_dim % hd || kv_dim % hd) return fail(kInvalidArgument, "decoder_layer: projections must be whole heads");
  const int heads = q_dim / hd, kvh = kv_dim / hd;
  if (kvh <= 0 || heads % kvh) return fail(kInvalidArgument, "decoder_layer: query heads must be a multiple of KV heads");
  const int64_t cache_rows = static_cast<int64_t>(b) * kvh * max_seq;
  if (!is2d(t[0], b, hidden, PTO_BF16) || t[1].dtype != PTO_FP32 || numel(t[1]) != hidden ||
      !is2d(t[2], hidden, q_dim, PTO_BF16) || !is2d(t[3], hidden, kv_dim, PTO_BF16) || !is2d(t[4], hidden, kv_dim, PTO_BF16) ||
      t[5].dtype != PTO_INT32 || numel(t[5]) != b || !is2d(t[6], max_seq, hd, PTO_FP32) || !is2d(t[7], max_seq, hd, PTO_FP32) ||
      t[8].dtype != PTO_BF16 || numel(t[8]) != cache_rows * hd || t[9].dtype != PTO_BF16 || numel(t[9]) != cache_rows * hd ||
      !is2d(t[10], q_dim, hidden, PTO_BF16) || t[11].dtype != PTO_FP32 || numel(t[11]) != hidden ||
      !is2d(t[12], hidden, inter, PTO_BF16) || !is2d(t[13], hidden, inter, PTO_BF16) ||
      !is2d(t[14], inter, hidden, PTO_BF16) || !is2d(t[15], b, hidden, PTO_BF16))
    return fail(kInvalidArgument, "decoder_layer: tensor shapes or dtypes do not match the program signature");
  if (max_seq % 128) return fail(kInvalidArgument, "decoder_layer: the cache length per sequence must be a multiple of 128");
  if (hidden % 8 || inter % 32) return fail(kInvalidArgument, "decoder_layer: hidden % 8, inter % 32 required");
  const float eps = f32_bits(a->scalars[0]);
  float scale = f32_bits(a->scalars[1]);
  if (scale == 0.f) scale = 1.f / std::sqrt(static_cast<float>(hd));
  const int qkv_dim = q_dim + 2 * kv_dim, nblk = max_seq / 128, group = heads / kvh;
  const size_t pa_b = al256(pa_scratch_bytes(b * kvh, group, 1, 1));
  const size_t need = pa_b + al256(static_cast<size_t>(qkv_dim) * hidden * 2) + al256(static_cast<size_t>(b) * hidden * 2) +
                      al256(static_cast<size_t>(b) * hidden * 4) + al256(static_cast<size_t>(b) * qkv_dim * 4) +
                      2 * al256(static_cast<size_t>(b) * q_dim * 2) + al256(static_cast<size_t>(b) * 4) +
                      al256(static_cast<size_t>(b) * kvh * nblk * 4) + al256(static_cast<size_t>(b) * kvh * 4) +
                      scope3_bytes(b, hidden, q_dim, inter) + 4096;
  int st = w->ensure_scratch(need);
  if (st != kOk) return st;
  int* err = static_cast<int*>(w->scratch);
  Arena ar{static_cast<uint8_t*>(w->scratch), pa_b};      // the attention kernel's scratch starts at the arena base
  void* wqkv = ar.take(static_cast<size_t>(qkv_dim) * hidden * 2);
  void* normed = ar.take(static_cast<size_t>(b) * hidden * 2);
  float* resid = static_cast<float*>(ar.take(static_cast<size_t>(b) * hidden * 4));
  float* qkv = static_cast<float*>(ar.take(static_cast<size_t>(b) * qkv_dim * 4));
  void* q_rot = ar.take(static_cast<size_t>(b) * q_dim * 2);
  void* attn = ar.take(static_cast<size_t>(b) * q_dim * 2);
  int32_t* seq_table = static_cast<int32_t*>(ar.take(static_cast<size_t>(b) * 4));
  int32_t* head_table = static_cast<int32_t*>(ar.take(static_cast<size_t>(b) * kvh * nblk * 4));
  int32_t* head_lens = static_cast<int32_t*>(ar.take(static_cast<size_t>(b) * kvh * 4));
  const int32_t* seq_lens = static_cast<const int32_t*>(tptr(t[5], 4));
  uint8_t* wq_p = static_cast<uint8_t*>(wqkv);
  st = pack_weight_launch(tptr(t[2], 2), PTO_BF16, wq_p, hidden, q_dim, w->stream);
  if (st != kOk) return st;
  st = pack_weight_launch(tptr(t[3], 2), PTO_BF16, wq_p + static_cast<size_t>(q_dim) * hidden * 2, hidden, kv_dim, w->stream);
  if (st != kOk) return st;
  st = pack_weight_launch(tptr(t[4], 2), PTO_BF16, wq_p + static_cast<size_t>(q_dim + kv_dim) * hidden * 2, hidden, kv_dim,
                          w->stream);
  if (st != kOk) return st;
  st = contiguous_cache_tables_launch(seq_lens, b, kvh, nblk, seq_table, head_table, head_lens, w->stream);
  if (st != kOk) return st;
  // scope 1: input RMSNorm (also leaves fp32(hidden) as the residual and clears the QKV accumulator), Q/K/V
  st = rms_norm_launch(tptr(t[0], 2), PTO_BF16, static_cast<const float*>(tptr(t[1], 4)), normed, PTO_BF16, b, hidden, eps,
                       resid, qkv, static_cast<size_t>(b) * qkv_dim * 4, w->stream);
  if (st != kOk) return st;
  st = linear_launch(normed, wqkv, qkv, b, qkv_dim, hidden, 1, err, w->stream);
  if (st != kOk) return st;
  // scope 2: RoPE + cache append at pos = seq_len - 1 (one block of max_seq tokens per sequence)
  st = rope_kv_append_launch(qkv, seq_lens, static_cast<const float*>(tptr(t[6], 4)), static_cast<const float*>(tptr(t[7], 4)),
                             max_seq, seq_table, 1, tptr(t[8], 2), tptr(t[9], 2), q_rot, b, heads, kvh, hd, max_seq, b, err,
                             w->stream);
  if (st != kOk) return st;
  // attention: every (sequence, kv head) is a single-KV-head sequence of 128-token blocks of the contiguous cache
  st = pa_launch(q_rot, tptr(t[8], 2), tptr(t[9], 2), head_table, head_lens, attn, 0, b * kvh, group, 1, hd, 128, nblk,
                 static_cast<int64_t>(b) * kvh * nblk, 1, scale, w->scratch, pa_b, w->stream);
  if (st != kOk) return st;
  // scope 3
  return scope3_body(w, ar, attn, q_dim, resid, t[10], t[11], t[12], t[13], t[14], tptr(t[15], 2), b, hidden, inter, eps);
}

// tensors: x [m, k] bf16, w [k, n] bf16 or fp32 (the `x @ W` layout), out [m, n] fp32; scalars: accumulate
// (examples/models/qwen3_jit/kernels/projection.py:36-143)
// tensors: x bf16 or fp32 [m, k] (fp32 is rounded to bf16 operands), w bf16/fp32 [k, n], out fp32 [m, n], and
// optionally bias fp32 [m, n]: out = x w + bias (examples/intermediate/01_fused_linear.py:60-66).  scalar: accumulate
// onto what out holds (ignored with a bias).
int op_linear(Worker* w, const pto_task_args* a) {
  if ((a->n_tensors != 3 && a->n_tensors != 4) || a->n_scalars != 1)
    return fail(kInvalidArgument, "linear: expects 3 or 4 tensors and 1 scalar");
  const pto_chip_tensor* t = a->tensors;
  if (t[0].ndims != 2 || t[1].ndims != 2) return fail(kInvalidArgument, "linear: 2-D tensors expected");
  const int m = t[0].shapes[0], k = t[0].shapes[1], n = t[1].shapes[1];
  if ((t[0].dtype != PTO_BF16 && t[0].dtype != PTO_FP32) || (t[1].dtype != PTO_BF16 && t[1].dtype != PTO_FP32) ||
      (int)t[1].shapes[0] != k || !is2d(t[2], m, n, PTO_FP32) || (a->n_tensors == 4 && !is2d(t[3], m, n, PTO_FP32)))
    return fail(kInvalidArgument, "linear: x bf16/fp32 [m, k], w bf16/fp32 [k, n], out (and bias) fp32 [m, n] expected");
  const size_t w_b = al256(static_cast<size_t>(n) * k * 2), x_b = al256(static_cast<size_t>(m) * k * 2);
  int st = w->ensure_scratch(4096 + w_b + x_b);
  if (st != kOk) return st;
  void* wp = static_cast<uint8_t*>(w->scratch) + 4096;
  st = pack_weight_launch(tptr(t[1], t[1].dtype == PTO_FP32 ? 4 : 2), (int)t[1].dtype, wp, k, n, w->stream);
  if (st != kOk) return st;
  const void* xb = tptr(t[0], 2);
  if (t[0].dtype == PTO_FP32) {
    void* cast_to = static_cast<uint8_t*>(wp) + w_b;
    st = cast_launch(tptr(t[0], 4), PTO_FP32, cast_to, PTO_BF16, static_cast<long long>(m) * k, w->stream);
    if (st != kOk) return st;
    xb = cast_to;
  }
  int accumulate = a->scalars[0] != 0;
  if (a->n_tensors == 4) {
    PTO_CUDA(cudaMemcpyAsync(tptr(t[2], 4), tptr(t[3], 4), static_cast<size_t>(m) * n * 4, cudaMemcpyDeviceToDevice, w->stream));
    accumulate = 1;
  }
  return linear_launch(xb, wp, static_cast<float*>(tptr(t[2], 4)), m, n, k, accumulate, static_cast<int*>(w->scratch),
                       w->stream);
}

// tensors: qkv fp32 [b, (Hq + 2 Hkv) * D], seq_lens int32 [b], rope_cos, rope_sin fp32 [rows, D], block_table int32
// [b, max_blocks], k_cache, v_cache bf16 [(block, kv head, token), D], q_out bf16 [b * Hq, D]
// scalars: num_heads, kv_heads, block_size   (examples/models/qwen3_jit/kernels/attention.py:40-111)
int op_rope_kv_append(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 8 || a->n_scalars != 3) return fail(kInvalidArgument, "rope_kv_append: expects 8 tensors and 3 scalars");
  const pto_chip_tensor* t = a->tensors;
  const int heads = (int)a->scalars[0], kvh = (int)a->scalars[1], bs = (int)a->scalars[2];
  if (t[2].ndims != 2 || heads <= 0 || kvh <= 0 || bs <= 0) return fail(kInvalidArgument, "rope_kv_append: bad geometry");
  const int hd = t[2].shapes[1], rows = t[2].shapes[0];
  const int64_t b = numel(t[1]);
  if (t[0].dtype != PTO_FP32 || numel(t[0]) != b * (heads + 2 * kvh) * hd || t[1].dtype != PTO_INT32 ||
      t[2].dtype != PTO_FP32 || t[3].dtype != PTO_FP32 || numel(t[3]) != numel(t[2]) || t[4].dtype != PTO_INT32 ||
      (b > 0 && numel(t[4]) % b) || t[5].dtype != PTO_BF16 || t[6].dtype != PTO_BF16 || numel(t[5]) != numel(t[6]) ||
      numel(t[5]) % (static_cast<int64_t>(kvh) * bs * hd) || t[7].dtype != PTO_BF16 || numel(t[7]) != b * heads * hd)
    return fail(kInvalidArgument, "rope_kv_append: tensor shapes or dtypes do not match");
  int st = w->ensure_scratch(256);
  if (st != kOk) return st;
  return rope_kv_append_launch(static_cast<const float*>(tptr(t[0], 4)), static_cast<const int32_t*>(tptr(t[1], 4)),
                               static_cast<const float*>(tptr(t[2], 4)), static_cast<const float*>(tptr(t[3], 4)), rows,
                               static_cast<const int32_t*>(tptr(t[4], 4)), b ? static_cast<int>(numel(t[4]) / b) : 1,
                               tptr(t[5], 2), tptr(t[6], 2), tptr(t[7], 2), static_cast<int>(b), heads, kvh, hd, bs,
                               numel(t[5]) / (static_cast<int64_t>(kvh) * bs * hd), static_cast<int*>(w->scratch), w->stream);
}

// The reference's MX matmul program (tests/st/runtime/ops/test_matmul_mx.py:170-226):
// tensors: a e4m3 [m, k], a_scale E8M0 [m, k/32] (MX_A_ZZ order), b e4m3 [k, n], b_scale E8M0 [k/32, n] (MX_B_NN
// order), out fp32 [m, n] = matmul_mx(...), out_acc fp32 [m, n] = matmul_mx_acc(out, ...)
// scalars: a_scale layout, b_scale layout (PTO_MX_SCALE_*)
int op_matmul_mx(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 6 || a->n_scalars != 2) return fail(kInvalidArgument, "matmul_mx: expects 6 tensors and 2 scalars");
  const pto_chip_tensor* t = a->tensors;
  if (t[0].ndims != 2 || t[2].ndims != 2) return fail(kInvalidArgument, "matmul_mx: 2-D operands expected");
  const int m = t[0].shapes[0], k = t[0].shapes[1], n = t[2].shapes[1];
  if ((int)t[2].shapes[0] != k || k % 32 || numel(t[1]) != static_cast<int64_t>(m) * (k / 32) ||
      numel(t[3]) != static_cast<int64_t>(k / 32) * n || !is2d(t[4], m, n, PTO_FP32) || !is2d(t[5], m, n, PTO_FP32))
    return fail(kInvalidArgument, "matmul_mx: operand, scale or output shapes do not match");
  int st = w->ensure_scratch(4096 + al256(static_cast<size_t>(n) * k));
  if (st != kOk) return st;
  void* b_t = static_cast<uint8_t*>(w->scratch) + 4096;
  int* err = static_cast<int*>(w->scratch);
  st = transpose_u8_launch(tptr(t[2], 1), b_t, k, n, w->stream);
  if (st != kOk) return st;
  float* out = static_cast<float*>(tptr(t[4], 4));
  st = matmul_mx_launch(tptr(t[0], 1), tptr(t[1], 1), (int)a->scalars[0], b_t, tptr(t[3], 1), (int)a->scalars[1], nullptr,
                        out, m, n, k, err, w->stream);
  if (st != kOk) return st;
  return matmul_mx_launch(tptr(t[0], 1), tptr(t[1], 1), (int)a->scalars[0], b_t, tptr(t[3], 1), (int)a->scalars[1], out,
                          static_cast<float*>(tptr(t[5], 4)), m, n, k, err, w->stream);
}

// Mixture-of-experts layer on one GPU (all experts local): sigmoid gate + top-k routing, grouped FP8 expert FFN,
// shared expert, combine.  The data movement of the reference's expert-parallel program
// (tests/st/distributed/test_l3_ep_dispatch_combine.py:104-402) with the real expert in place of its stand-in.
// tensors: x bf16 [T, H], gate bf16 [E, H] (packed), bias fp32 [E],
//          w_gu e4m3 [E, 2I, H], s_gu fp32 [E, 2I/128, H/128], w_d e4m3 [E, H, I], s_d fp32 [E, H/128, I/128],
//          the same four for the shared expert ([1, ...]; a shared expert is not optional here),
//          y bf16 [T, H]
// scalars: top-k
int op_moe_layer(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 12 || a->n_scalars != 1) return fail(kInvalidArgument, "moe_layer: expects 12 tensors and 1 scalar");
  const pto_chip_tensor* t = a->tensors;
  if (t[0].ndims != 2 || t[1].ndims != 2 || t[3].ndims != 3 || t[5].ndims != 3)
    return fail(kInvalidArgument, "moe_layer: x [T, H], gate [E, H], w_gu [E, 2I, H], w_d [E, H, I] expected");
  const int tokens = t[0].shapes[0], hidden = t[0].shapes[1], experts = t[1].shapes[0], inter = t[5].shapes[2];
  if (t[0].dtype != PTO_BF16 || t[1].dtype != PTO_BF16 || (int)t[1].shapes[1] != hidden || !is2d(t[11], tokens, hidden, PTO_BF16) ||
      numel(t[2]) != experts || t[2].dtype != PTO_FP32 || (int)t[3].shapes[0] != experts || (int)t[3].shapes[1] != 2 * inter ||
      (int)t[3].shapes[2] != hidden || (int)t[5].shapes[0] != experts || (int)t[5].shapes[1] != hidden ||
      numel(t[7]) != static_cast<int64_t>(2) * inter * hidden || numel(t[9]) != static_cast<int64_t>(hidden) * inter)
    return fail(kInvalidArgument, "moe_layer: tensor shapes or dtypes do not match");
  pto_moe_layer_desc d = {};
  d.hidden = hidden; d.inter = inter; d.n_experts = experts; d.topk = static_cast<int>(a->scalars[0]); d.max_tokens = tokens;
  d.gate_packed = tptr(t[1], 2); d.bias = static_cast<const float*>(tptr(t[2], 4));
  d.w_gu = tptr(t[3], 1); d.s_gu = static_cast<const float*>(tptr(t[4], 4));
  d.w_d = tptr(t[5], 1); d.s_d = static_cast<const float*>(tptr(t[6], 4));
  d.sh_w_gu = tptr(t[7], 1); d.sh_s_gu = static_cast<const float*>(tptr(t[8], 4));
  d.sh_w_d = tptr(t[9], 1); d.sh_s_d = static_cast<const float*>(tptr(t[10], 4));
  d.comm = nullptr;
  pto_moe_layer_desc have = w->moe_desc;
  have.max_tokens = d.max_tokens;   // a layer built for more tokens serves a smaller call
  if (w->moe == nullptr || memcmp(&have, &d, sizeof d) != 0 || w->moe_desc.max_tokens < tokens) {
    if (w->moe) {
      PTO_CUDA(cudaStreamSynchronize(w->stream));
      pto_moe_layer_destroy(w->moe);
      w->moe = nullptr;
    }
    int st = pto_moe_layer_create(&d, &w->moe);
    if (st != kOk) return st;
    w->moe_desc = d;
  }
  int st = pto_moe_layer_forward(w->moe, tptr(t[0], 2), tokens, nullptr, nullptr, tptr(t[11], 2), nullptr, nullptr, nullptr,
                                 w->stream);
  if (st != kOk) return st;
  // the layer's kernels report into its own error word: fold it into the worker's, which pto_device_status reads
  int32_t words[4];
  st = pto_moe_layer_status(w->moe, words, w->stream);
  if (st != kOk) return st;
  if (words[0] != 0) {
    st = w->ensure_scratch(4096);
    if (st != kOk) return st;
    PTO_CUDA(cudaMemcpyAsync(w->scratch, words, sizeof words, cudaMemcpyHostToDevice, w->stream));
    PTO_CUDA(cudaStreamSynchronize(w->stream));
  }
  return kOk;
}

// tensors (all fp32): hidden [S, D], causal_mask [S, S], cos_emb, sin_emb [S, D/2], wq, wk, wv, w_dense, w_gate, w_up,
// w_down [D, D], w_lm [D, V], logits [S, V] -- the signature of llama_mini_orch (examples/models/08_llama_mini.py:385-408)
int op_llama_mini(Worker* w, const pto_task_args* a) {
  if (a->n_tensors != 13 || a->n_scalars != 0) return fail(kInvalidArgument, "llama_mini: expects 13 tensors and no scalars");
  const pto_chip_tensor* t = a->tensors;
  if (t[0].ndims != 2 || t[11].ndims != 2) return fail(kInvalidArgument, "llama_mini: hidden [S, D] and w_lm [D, V] expected");
  const int s = t[0].shapes[0], d = t[0].shapes[1], v = t[11].shapes[1];
  bool ok = is2d(t[0], s, d, PTO_FP32) && is2d(t[1], s, s, PTO_FP32) && is2d(t[2], s, d / 2, PTO_FP32) &&
            is2d(t[3], s, d / 2, PTO_FP32) && is2d(t[11], d, v, PTO_FP32) && is2d(t[12], s, v, PTO_FP32);
  for (int i = 4; i <= 10; ++i) ok = ok && is2d(t[i], d, d, PTO_FP32);
  if (!ok) return fail(kInvalidArgument, "llama_mini: tensor shapes or dtypes do not match the program's signature");
  const float* f[12];
  for (int i = 0; i < 12; ++i) f[i] = static_cast<const float*>(tptr(t[i], 4));
  return llama_mini_launch(f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7], f[8], f[9], f[10], f[11],
                           static_cast<float*>(tptr(t[12], 4)), s, d, v, w->stream);
}

}  // namespace pto
