// The reference's minimal LLaMA forward pass (one decoder layer, one head, RoPE, LM head) as one kernel:
// examples/models/08_llama_mini.py:384-483 (orchestration `llama_mini_orch` over thirteen fp32 tensors), golden
// tests/st/examples/03_llm_models/test_llama_7b_mini_1h.py:118-199.
//
//   normed = rms_norm(hidden)                       x / sqrt(sum(x^2) / D + 1e-6), no gamma (:94-118)
//   q, k, v = normed @ wq, wk, wv ; q, k = rope(q), rope(k)       rotate-half with [S, D/2] tables (:324-352)
//   probs = softmax(q @ k^T * D^-0.5 + causal_mask) ; attn = probs @ v
//   attn_res = hidden + attn @ w_dense
//   h1 = attn_res + (silu(n2 @ w_gate) * (n2 @ w_up)) @ w_down,  n2 = rms_norm(attn_res)
//   logits = rms_norm(h1) @ w_lm
//
// Everything is fp32 as in the reference program, and the whole model is a few hundred kFLOP at its sizes
// (S = 16, D = 64, V = 64), so one CTA walks the stages with every intermediate in shared memory and plain FMAs:
// the tensor cores would need operands rounded to tf32 or bf16, which the fp32 golden does not allow.
#include "common.cuh"
#include "kernels.h"

namespace pto {
namespace {

constexpr int kLmThreads = 256;

struct LlamaMiniParams {
  const float *hidden, *mask, *cos_emb, *sin_emb, *wq, *wk, *wv, *w_dense, *w_gate, *w_up, *w_down, *w_lm;
  float* logits;
  int s, d, v;
};

// out[s, n] = sum_k in[s, k] * w[k, n] (+ add[s, n]); `in` in shared memory, `w` row-major (consecutive threads
// read consecutive columns) in global memory (W_GLOBAL: read through the read-only path) or in shared memory,
// `out` anywhere.
template <bool W_GLOBAL>
__device__ __forceinline__ void mm(float* out, const float* in, const float* w, const float* add, int rows, int kdim,
                                   int ndim) {
  for (int idx = threadIdx.x; idx < rows * ndim; idx += kLmThreads) {
    const int r = idx / ndim, n = idx - r * ndim;
    float acc = 0.f;
    for (int k = 0; k < kdim; ++k) {
      const float wv = W_GLOBAL ? __ldg(w + static_cast<size_t>(k) * ndim + n) : w[k * ndim + n];
      acc = fmaf(in[r * kdim + k], wv, acc);
    }
    out[idx] = add ? add[idx] + acc : acc;
  }
}

// out[r, :] = x[r, :] / sqrt(sum(x[r, :]^2) / d + eps); one warp per row
__device__ __forceinline__ void rms(float* out, const float* x, int rows, int d) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < rows; r += kLmThreads / 32) {
    float ss = 0.f;
    for (int c = lane; c < d; c += 32) ss = fmaf(x[r * d + c], x[r * d + c], ss);
    ss = warp_sum(ss);
    const float rms_v = sqrtf(ss / static_cast<float>(d) + 1e-6f);
    for (int c = lane; c < d; c += 32) out[r * d + c] = x[r * d + c] / rms_v;
  }
}

// rotate-half in place: lo' = lo cos - hi sin, hi' = hi cos + lo sin
__device__ __forceinline__ void rope(float* x, const float* __restrict__ c, const float* __restrict__ s, int rows, int d) {
  const int half = d >> 1;
  for (int idx = threadIdx.x; idx < rows * half; idx += kLmThreads) {
    const int r = idx / half, i = idx - r * half;
    const float lo = x[r * d + i], hi = x[r * d + half + i];
    const float cv = __ldg(c + idx), sv = __ldg(s + idx);
    x[r * d + i] = lo * cv - hi * sv;
    x[r * d + half + i] = hi * cv + lo * sv;
  }
}

__global__ void __launch_bounds__(kLmThreads, 1) llama_mini_kernel(const LlamaMiniParams p) {
  pdl_launch_dependents();
  extern __shared__ float lm_smem[];
  const int S = p.s, D = p.d, V = p.v;
  float* a = lm_smem;            // [S, D] normed activations / attention output
  float* q = a + S * D;          // [S, D] q, later the gate projection
  float* k = q + S * D;          // [S, D] k, later the up projection
  float* vv = k + S * D;         // [S, D] v, later silu(gate) * up
  float* res = vv + S * D;       // [S, D] residual stream
  float* pr = res + S * D;       // [S, S] scores / probabilities
  pdl_wait();
  for (int i = threadIdx.x; i < S * D; i += kLmThreads) res[i] = p.hidden[i];
  __syncthreads();
  rms(a, res, S, D);
  __syncthreads();
  mm<true>(q, a, p.wq, nullptr, S, D, D);
  mm<true>(k, a, p.wk, nullptr, S, D, D);
  mm<true>(vv, a, p.wv, nullptr, S, D, D);
  __syncthreads();
  rope(q, p.cos_emb, p.sin_emb, S, D);
  rope(k, p.cos_emb, p.sin_emb, S, D);
  __syncthreads();
  const float scale = rsqrtf(static_cast<float>(D));
  for (int idx = threadIdx.x; idx < S * S; idx += kLmThreads) {
    const int r = idx / S, t = idx - r * S;
    float acc = 0.f;
    for (int c = 0; c < D; ++c) acc = fmaf(q[r * D + c], k[t * D + c], acc);
    pr[idx] = acc * scale + __ldg(p.mask + idx);
  }
  __syncthreads();
  {   // softmax over each row, one warp per row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < S; r += kLmThreads / 32) {
      float m = -INFINITY;
      for (int c = lane; c < S; c += 32) m = fmaxf(m, pr[r * S + c]);
      m = warp_max(m);
      float sum = 0.f;
      for (int c = lane; c < S; c += 32) {
        const float e = expf(pr[r * S + c] - m);
        pr[r * S + c] = e;
        sum += e;
      }
      sum = warp_sum(sum);
      for (int c = lane; c < S; c += 32) pr[r * S + c] = pr[r * S + c] / sum;
    }
  }
  __syncthreads();
  mm<false>(a, pr, vv, nullptr, S, S, D);       // attention output: probabilities x v, both in shared memory
  __syncthreads();
  mm<true>(res, a, p.w_dense, res, S, D, D);           // first residual, element-wise in place
  __syncthreads();
  rms(a, res, S, D);
  __syncthreads();
  mm<true>(q, a, p.w_gate, nullptr, S, D, D);
  mm<true>(k, a, p.w_up, nullptr, S, D, D);
  __syncthreads();
  for (int i = threadIdx.x; i < S * D; i += kLmThreads) {
    const float g = q[i];
    vv[i] = g * (1.f / (1.f + expf(-g))) * k[i];
  }
  __syncthreads();
  mm<true>(res, vv, p.w_down, res, S, D, D);           // second residual
  __syncthreads();
  rms(a, res, S, D);
  __syncthreads();
  mm<true>(p.logits, a, p.w_lm, nullptr, S, D, V);
}

}  // namespace

int llama_mini_launch(const float* hidden, const float* mask, const float* cos_emb, const float* sin_emb, const float* wq,
                      const float* wk, const float* wv, const float* w_dense, const float* w_gate, const float* w_up,
                      const float* w_down, const float* w_lm, float* logits, int seq_len, int head_dim, int vocab,
                      cudaStream_t stream) {
  PTO_REQUIRE(hidden && mask && cos_emb && sin_emb && wq && wk && wv && w_dense && w_gate && w_up && w_down && w_lm && logits,
              "llama_mini: NULL tensor");
  PTO_REQUIRE(seq_len > 0 && head_dim > 0 && head_dim % 2 == 0 && vocab > 0, "llama_mini: bad sizes");
  const size_t smem = sizeof(float) * (static_cast<size_t>(5) * seq_len * head_dim + static_cast<size_t>(seq_len) * seq_len);
  PTO_REQUIRE(smem <= 200 * 1024, "llama_mini: the model's activations must fit in shared memory (5*S*D + S*S floats <= 200 KB)");
  if (first_use_on_device(4)) PTO_CUDA(cudaFuncSetAttribute(llama_mini_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  LlamaMiniParams p{hidden, mask, cos_emb, sin_emb, wq, wk, wv, w_dense, w_gate, w_up, w_down, w_lm, logits, seq_len, head_dim, vocab};
  launch_kernel(llama_mini_kernel, dim3(1), dim3(kLmThreads), smem, stream, p);
  return check_cuda(cudaGetLastError(), "llama_mini_kernel launch");
}

}  // namespace pto
