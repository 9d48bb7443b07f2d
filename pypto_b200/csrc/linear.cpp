// Host-side composition of the tensor-core GEMM into the operators the model programs
// use: a linear layer over pre-packed weights (q/k/v/o projections,
// examples/models/qwen3_jit/kernels/projection.py:36-177) and the fused SwiGLU FFN
// (examples/models/01_ffn.py:112-131; qwen3_jit/kernels/mlp.py:23-61).
//
// Orientation and split-K are chosen from the shape: with at most 256 activation rows
// (decode) the weights take the 128 TMEM lanes and the output is written transposed;
// the (tile, K block) iterations are split evenly over the SMs (stream-K) and partial sums
// meet in the fp32 output through red.global.add.f32.
#include "common.cuh"
#include "kernels.h"

namespace pto {

namespace {

int pick_bn_tokens(int m) { return m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256)); }

}  // namespace

// out[m, n] (+)= x[m, k] . w_packed[n, k]^T, fp32 out.  accumulate = 0 overwrites.
int linear_launch(const void* x, const void* w_packed, float* out, int m, int n, int k, int accumulate, int* err,
                  cudaStream_t stream) {
  PTO_REQUIRE(x && w_packed && out, "linear: NULL tensor");
  PTO_REQUIRE(m > 0 && n > 0 && k > 0 && k % 8 == 0, "linear: m, n > 0 and k a positive multiple of 8 required");
  if (m <= 256) {
    // decode orientation: A = weights [n, k], B = activations [m, k]
    const int bn = pick_bn_tokens(m);
    if (!accumulate) PTO_CUDA(cudaMemsetAsync(out, 0, sizeof(float) * static_cast<size_t>(m) * n, stream));
    return gemm_bf16_launch(w_packed, n, x, m, m, k, out, n, 0, 1, kGemmEpiAtomic, 0, bn, 1, err, stream);
  }
  int bn = n >= 256 ? 256 : 128;
  const int tiles = ((m + 127) / 128) * ((n + bn - 1) / bn);
  // few tiles: stream-K over (tile, K block) with the atomic epilogue keeps every SM busy
  const int epi = (accumulate || tiles < sm_count()) ? kGemmEpiAtomic : kGemmEpiStore;
  // every CTA of a stream-K launch reduces one partial tile (or two) into the output: narrower tiles, fewer bytes of
  // reductions (the tiles are few here, so the operand re-reads they cost stay in L2)
  // (measured at n = 1024, K = 4096: 16 tiles 37 -> 33 us for the FFN it is part of, 64 tiles 60 -> 63 us)
  if (epi == kGemmEpiAtomic && 4 * tiles <= sm_count()) bn = 128;
  if (epi == kGemmEpiAtomic && !accumulate)
    PTO_CUDA(cudaMemsetAsync(out, 0, sizeof(float) * static_cast<size_t>(m) * n, stream));
  return gemm_bf16_launch(x, m, w_packed, n, n, k, out, n, 0, 0, epi, 0, bn, 1, err, stream);
}

namespace {
// Column tile for the SwiGLU-epilogue GEMM (whole tiles, no stream-K): the bn in {128, 64, 32}
// dividing `inter` whose tile count fills the SMs best.  Returns the fill fraction.
double pick_swiglu_bn(int m, int inter, int* bn_out) {
  const int sms = sm_count(), a_tiles = (m + 127) / 128;
  double best = 0.0;
  *bn_out = 0;
  for (int bn = 128; bn >= 32; bn >>= 1) {
    if (inter % bn) continue;
    const long long tiles = static_cast<long long>(a_tiles) * (inter / bn);
    const double eff = static_cast<double>(tiles) / static_cast<double>((tiles + sms - 1) / sms * sms);
    if (eff > best + 0.03) { best = eff; *bn_out = bn; }
  }
  return best;
}
bool use_swiglu_epilogue(int m, int inter, int* bn) {
  const double eff = pick_swiglu_bn(m, inter, bn);
  return *bn != 0 && (m > 256 || eff >= 0.85);   // decode sizes fall back to stream-K when tiles quantise badly
}
}  // namespace

// A workspace serves calls of any size; larger batches must not touch the header that the one-launch kernel of
// small batches keeps its call number and slab counters in.
constexpr size_t kFfnHeaderBytes = 8192;

size_t ffn_workspace_bytes(int m, int inter) {
  // the first kFfnHeaderBytes stay reserved for the one-launch kernel's counters whatever path a call takes; then
  // bf16 activation [m, inter]; plus fp32 gate|up [m, 2*inter] for the stream-K path
  const size_t act = (static_cast<size_t>(m) * inter * 2 + 255) / 256 * 256;
  int bn;
  const size_t chain = kFfnHeaderBytes + (use_swiglu_epilogue(m, inter, &bn) ? act : act + static_cast<size_t>(m) * 2 * inter * 4);
  // decode-sized batches: the one-launch kernel's activation has 128 rows
  const size_t fused = (m <= 128 && inter % 64 == 0 && inter >= 64) ? ffn_fused_workspace_bytes(inter) : 0;
  return chain > fused ? chain : fused;
}

// One-projection FFN with an elementwise activation: out (+)= bf16(f(x W_in)) W_down, f = x sigmoid(alpha x)
// (kind 1; alpha 1.702: `ffn_gelu`, examples/models/01_ffn.py:92-108) or relu (kind 2; `ffn_relu`, :134-150).
// x bf16 [m, k], w_in packed [inter, k], w_down packed [n_out, inter].  Three launches: GEMM, activation, GEMM.
// Workspace: fp32 [m, inter] and bf16 [m, inter].
size_t ffn_act_workspace_bytes(int m, int inter) {
  const size_t n = static_cast<size_t>(m) * inter;
  return (n * 4 + 255) / 256 * 256 + (n * 2 + 255) / 256 * 256;
}

int ffn_act_launch(const void* x, const void* w_in, const void* w_down, float* out, int m, int k, int inter, int n_out,
                   int kind, float alpha, void* workspace, size_t workspace_bytes, int accumulate, int* err,
                   cudaStream_t stream) {
  PTO_REQUIRE(x && w_in && w_down && out && workspace, "ffn_act: NULL tensor");
  PTO_REQUIRE(m > 0 && k > 0 && inter > 0 && n_out > 0 && k % 8 == 0 && inter % 8 == 0,
              "ffn_act: sizes must be positive, k and inter multiples of 8");
  PTO_REQUIRE(workspace_bytes >= ffn_act_workspace_bytes(m, inter), "ffn_act: workspace too small");
  PTO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "ffn_act: workspace must be 256-byte aligned");
  const size_t n = static_cast<size_t>(m) * inter;
  float* h = static_cast<float*>(workspace);
  void* act = static_cast<uint8_t*>(workspace) + (n * 4 + 255) / 256 * 256;
  int st = linear_launch(x, w_in, h, m, inter, k, 0, err, stream);
  if (st != kOk) return st;
  st = act_rows_launch(h, act, static_cast<long long>(n), kind, alpha, stream);
  if (st != kOk) return st;
  return linear_launch(act, w_down, out, m, n_out, inter, accumulate, err, stream);
}

// The same for fp32 x: the workspace of the bf16 form followed by a bf16 copy of x.
size_t ffn_f32_workspace_bytes(int m, int k, int inter) {
  return (ffn_workspace_bytes(m, inter) + 255) / 256 * 256 + (static_cast<size_t>(m) * k * 2 + 255) / 256 * 256;
}

// fp32 x [m, k]: rounded to bf16 operands as the reference's bf16 kernels do.  With at most 128 rows the one-launch
// kernel casts x itself and clears the output (accumulate = 0) before its first GEMM: one launch in all.  Otherwise a
// cast kernel (which also clears the output) goes ahead of the bf16 form.
int ffn_swiglu_f32_launch(const float* x, const void* w_gate_up, const void* w_down, float* out, int m, int k, int inter,
                          int n_out, void* workspace, size_t workspace_bytes, int accumulate, int* err,
                          cudaStream_t stream) {
  PTO_REQUIRE(x && w_gate_up && w_down && out && workspace, "ffn_swiglu_f32: NULL tensor");
  PTO_REQUIRE(m > 0 && k > 0 && inter > 0 && n_out > 0 && k % 8 == 0 && inter % 8 == 0,
              "ffn_swiglu_f32: sizes must be positive, k and inter multiples of 8");
  PTO_REQUIRE(workspace_bytes >= ffn_f32_workspace_bytes(m, k, inter), "ffn_swiglu_f32: workspace too small");
  PTO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "ffn_swiglu_f32: workspace must be 256-byte aligned");
  const size_t base_bytes = (ffn_workspace_bytes(m, inter) + 255) / 256 * 256;
  void* xb = static_cast<uint8_t*>(workspace) + base_bytes;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (ffn_fused_ok(m, k, inter, n_out) && aligned)
    return ffn_fused_launch(nullptr, w_gate_up, w_down, out, m, k, inter, n_out, workspace, base_bytes, err, stream, x, xb,
                            accumulate ? 0 : 1);
  const size_t out_bytes = static_cast<size_t>(m) * n_out * 4;
  int st;
  if (!accumulate && aligned && out_bytes % 16 == 0) {
    st = cast_zero_launch(x, PTO_FP32, xb, PTO_BF16, static_cast<long long>(m) * k, out, out_bytes, stream);
  } else {
    st = cast_launch(x, PTO_FP32, xb, PTO_BF16, static_cast<long long>(m) * k, stream);
    if (st == kOk && !accumulate) st = check_cuda(cudaMemsetAsync(out, 0, out_bytes, stream), "cudaMemsetAsync(out)");
  }
  if (st != kOk) return st;
  return ffn_swiglu_launch(xb, w_gate_up, w_down, out, m, k, inter, n_out, workspace, base_bytes, 1, err, stream);
}

// out[m, n_out] (+)= (silu(x Wg) * (x Wu)) Wd with bf16 operands, fp32 accumulate, the
// activation rounded to bf16 before the down projection
// (tests/st/runtime/framework_and_models/test_qwen3_decode_scope3_mixed.py:282-285).
// w_gate_up packed [2*inter, k] (gate rows first), w_down packed [n_out, inter].
int ffn_swiglu_launch(const void* x, const void* w_gate_up, const void* w_down, float* out, int m, int k, int inter,
                      int n_out, void* workspace, size_t workspace_bytes, int accumulate, int* err,
                      cudaStream_t stream) {
  PTO_REQUIRE(x && w_gate_up && w_down && out && workspace, "ffn_swiglu: NULL tensor");
  PTO_REQUIRE(m > 0 && k > 0 && inter > 0 && n_out > 0 && k % 8 == 0 && inter % 8 == 0,
              "ffn_swiglu: sizes must be positive, k and inter multiples of 8");
  PTO_REQUIRE(workspace_bytes >= ffn_workspace_bytes(m, inter), "ffn_swiglu: workspace too small");
  PTO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "ffn_swiglu: workspace must be 256-byte aligned");
  if (ffn_fused_ok(m, k, inter, n_out)) {
    // at most 128 rows: both GEMMs in one persistent launch (the workspace header keeps its call counter)
    if (!accumulate) PTO_CUDA(cudaMemsetAsync(out, 0, sizeof(float) * static_cast<size_t>(m) * n_out, stream));
    return ffn_fused_launch(x, w_gate_up, w_down, out, m, k, inter, n_out, workspace, workspace_bytes, err, stream);
  }
  uint8_t* ws = static_cast<uint8_t*>(workspace) + kFfnHeaderBytes;
  __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(ws);
  int st;
  int bn = 0;
  if (use_swiglu_epilogue(m, inter, &bn)) {
    // 128 features per tile put the GEMM on SM pairs (256 x 256 tiles of [gate | up]) when the problem is large enough:
    // a pair moves two thirds of the bytes per FLOP of single CTAs, which outweighs a less even last wave
    if (inter % 128 == 0 && gemm2_eligible(m, inter, k, kGemmEpiSwiglu, 0, 128, 1)) bn = 128;
    // activations on the TMEM lanes (rows past m are zero filled by TMA), gate and up weight
    // tiles side by side as one MMA N; SiLU(gate) * up in the epilogue, no intermediate in HBM
    st = gemm_bf16_launch(x, m, w_gate_up, 2 * inter, inter, k, act, inter, 1, 0, kGemmEpiSwiglu, inter, bn, 1, err,
                          stream);
    if (st != kOk) return st;
  } else {
    float* gate_up = reinterpret_cast<float*>(ws + (static_cast<size_t>(m) * inter * 2 + 255) / 256 * 256);
    st = linear_launch(x, w_gate_up, gate_up, m, 2 * inter, k, 0, err, stream);
    if (st != kOk) return st;
    st = swiglu_act_launch(gate_up, act, m, inter, stream);
    if (st != kOk) return st;
  }
  return linear_launch(act, w_down, out, m, n_out, inter, accumulate, err, stream);
}

}  // namespace pto
