// Decoder-layer glue kernels: RMSNorm, RoPE + paged KV-cache append, SwiGLU activation,
// casts, and the one-time weight packing ([K, N] row-major -> [N, K] bf16, the K-major
// operand layout of the tensor-core GEMM).  All are bandwidth-bound elementwise / row
// kernels with 16-byte accesses where the shapes allow.
//
// Reference semantics:
//   RMSNorm   x * rsqrt(mean(x^2) + eps) * gamma, fp32 statistics, bf16 round at the end
//             (examples/models/qwen3_jit/kernels/rmsnorm.py:27-89;
//              tests/st/runtime/framework_and_models/test_qwen3_decode_scope3_mixed.py:278-280)
//   RoPE      rotate-half with cos/sin table rows at pos = seq_len - 1, rotated K and the V row
//             written to the cache as bf16, rotated Q as bf16
//             (examples/models/qwen3_jit/kernels/attention.py:40-111)
//   SwiGLU    bf16(gate * sigmoid(gate) * up) (examples/models/qwen3_jit/kernels/mlp.py:23-61)
#include "common.cuh"
#include "kernels.h"

namespace pto {
namespace {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) r += red[i];
  return r;
}

// One CTA (256 threads) per row.  Two optional side jobs let a decoder layer drop two launches: `copy`
// receives the row as fp32 (the residual that the next projection accumulates onto), and `zero`
// (16-byte vectors) is cleared by the whole grid (the accumulator of the next stream-K GEMM).
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
rms_norm_kernel(const TI* __restrict__ x, const float* __restrict__ gamma, TO* __restrict__ out, int hidden,
                float eps, float* __restrict__ copy, uint4* __restrict__ zero, long long zero_vecs) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[8];
  const TI* xr = x + static_cast<size_t>(blockIdx.x) * hidden;
  TO* orow = out + static_cast<size_t>(blockIdx.x) * hidden;
  float* crow = copy ? copy + static_cast<size_t>(blockIdx.x) * hidden : nullptr;
  for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < zero_vecs;
       i += static_cast<long long>(gridDim.x) * 256)
    zero[i] = make_uint4(0u, 0u, 0u, 0u);
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += 256) {
    const float v = to_f32(xr[i]);
    if (crow) crow[i] = v;
    ss += v * v;
  }
  const float mean = block_sum_256(ss, red) / static_cast<float>(hidden);
  const float inv = rsqrtf(mean + eps);
  for (int i = threadIdx.x; i < hidden; i += 256) {
    const float g = gamma ? gamma[i] : 1.f;
    orow[i] = from_f32<TO>(to_f32(xr[i]) * inv * g);
  }
}

// grid = (batch, num_heads + kv_heads); block = head_dim / 2 threads.
// qkv fp32 [batch, (num_heads + 2 kv_heads) * D]: q heads, then k heads, then v heads.
__global__ void rope_kv_append_kernel(const float* __restrict__ qkv, const int* __restrict__ seq_lens,
                                      const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                      int table_rows, const int* __restrict__ block_table, int max_blocks,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      __nv_bfloat16* __restrict__ q_out, int num_heads, int kv_heads, int head_dim,
                                      int block_size, int pool_blocks, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y, i = threadIdx.x, half = head_dim / 2;
  const int len = seq_lens[b];
  int pos = len - 1;
  if (pos < 0 || pos >= table_rows || pos / block_size >= max_blocks) {
    if (i == 0) report_error(err, kErrBadBlockId, 4, pos);
    return;
  }
  const size_t row_w = static_cast<size_t>(num_heads + 2 * kv_heads) * head_dim;
  const float* src = qkv + b * row_w + static_cast<size_t>(h) * head_dim;
  const float c_lo = cos_t[static_cast<size_t>(pos) * head_dim + i];
  const float c_hi = cos_t[static_cast<size_t>(pos) * head_dim + half + i];
  const float s_lo = sin_t[static_cast<size_t>(pos) * head_dim + i];
  const float s_hi = sin_t[static_cast<size_t>(pos) * head_dim + half + i];
  const float lo = src[i], hi = src[half + i];
  const float r_lo = lo * c_lo - hi * s_lo;
  const float r_hi = hi * c_hi + lo * s_hi;
  if (h < num_heads) {
    __nv_bfloat16* dst = q_out + (static_cast<size_t>(b) * num_heads + h) * head_dim;
    dst[i] = __float2bfloat16_rn(r_lo);
    dst[half + i] = __float2bfloat16_rn(r_hi);
    return;
  }
  const int ki = h - num_heads;
  const int blk = block_table[static_cast<size_t>(b) * max_blocks + pos / block_size];
  if (blk < 0 || blk >= pool_blocks) {
    if (i == 0) report_error(err, kErrBadBlockId, 5, blk);
    return;
  }
  const size_t row = (static_cast<size_t>(blk) * kv_heads + ki) * block_size + pos % block_size;
  k_cache[row * head_dim + i] = __float2bfloat16_rn(r_lo);
  k_cache[row * head_dim + half + i] = __float2bfloat16_rn(r_hi);
  const float* vsrc = qkv + b * row_w + static_cast<size_t>(num_heads + kv_heads + ki) * head_dim;
  v_cache[row * head_dim + i] = __float2bfloat16_rn(vsrc[i]);
  v_cache[row * head_dim + half + i] = __float2bfloat16_rn(vsrc[half + i]);
}

// Block tables that present a contiguous KV cache -- row = (b * kv_heads + ki) * max_seq + pos, the layout of
// examples/models/qwen3_jit/kernels/attention.py:72 -- to the paged kernels:
//   seq_table [batch]                          one block of max_seq tokens per sequence (for the cache append)
//   head_table [batch * kv_heads, blocks]      every (sequence, kv head) as its own single-head sequence of
//   head_lens [batch * kv_heads]               128-token blocks (for the attention kernel)
__global__ void contiguous_cache_tables_kernel(const int* __restrict__ seq_lens, int batch, int kv_heads,
                                               int blocks_per_seq, int* __restrict__ seq_table,
                                               int* __restrict__ head_table, int* __restrict__ head_lens) {
  pdl_launch_dependents();
  pdl_wait();
  const long long n = static_cast<long long>(batch) * kv_heads * blocks_per_seq;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    head_table[i] = static_cast<int>(i);
    if (i < batch) seq_table[i] = static_cast<int>(i);
    if (i < static_cast<long long>(batch) * kv_heads) head_lens[i] = seq_lens[i / kv_heads];
  }
}

// gate_up fp32 [rows, 2 * inter] (gate columns first) -> act bf16 [rows, inter]
__global__ void swiglu_act_kernel(const float* __restrict__ gate_up, __nv_bfloat16* __restrict__ act, long long rows,
                                  int inter) {
  pdl_launch_dependents();
  pdl_wait();
  const long long n = rows * inter;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / inter;
    const int c = static_cast<int>(idx - r * inter);
    const float g = gate_up[r * 2 * inter + c], u = gate_up[r * 2 * inter + inter + c];
    act[idx] = __float2bfloat16_rn(g * (1.f / (1.f + __expf(-g))) * u);
  }
}

// act[i] = bf16(f(h[i])) with f = x * sigmoid(alpha * x) (kind 1: alpha = 1.702 is the GELU of
// examples/models/01_ffn.py:51-62, alpha = 1 is SiLU; the sigmoid as recip(1 + exp(-alpha x)) like the reference's
// kernel) or f = max(x, 0) (kind 2, relu_kernel, :80-86).
__global__ void act_rows_kernel(const float* __restrict__ h, __nv_bfloat16* __restrict__ act, long long n, int kind,
                                float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float x = h[i];
    act[i] = __float2bfloat16_rn(kind == 2 ? fmaxf(x, 0.f) : x * (1.f / (1.f + __expf(-alpha * x))));
  }
}

// out = cast(in); optional side job of the same launch: `zero` (16-byte aligned, zero_vec uint4 words) is
// cleared, e.g. the fp32 accumulator of the GEMM that follows.
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n, uint4* __restrict__ zero,
                            long long zero_vec) {
  pdl_launch_dependents();
  pdl_wait();
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nth = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = tid; i < n; i += nth) out[i] = from_f32<TO>(to_f32(in[i]));
  for (long long i = tid; i < zero_vec; i += nth) zero[i] = make_uint4(0, 0, 0, 0);
}

// src [K, N] row-major -> dst [N, K] bf16; 32x32 tiles through shared memory.
template <typename TI>
__global__ void __launch_bounds__(256) pack_weight_kernel(const TI* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                          int k, int n) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float tile[32][33];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {
    const int kk = k0 + r, nn = n0 + tx;
    tile[r][tx] = (kk < k && nn < n) ? to_f32(src[static_cast<size_t>(kk) * n + nn]) : 0.f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int nn = n0 + r, kk = k0 + tx;
    if (nn < n && kk < k) dst[static_cast<size_t>(nn) * k + kk] = __float2bfloat16_rn(tile[tx][r]);
  }
}

int grid_for(long long n, int block) {
  long long g = (n + block - 1) / block;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

int rms_norm_launch(const void* x, int x_dtype, const float* gamma, void* out, int out_dtype, long long rows,
                    int hidden, float eps, float* copy_f32, void* zero, size_t zero_bytes, cudaStream_t stream) {
  PTO_REQUIRE(x && out && rows >= 0 && hidden > 0, "rms_norm: bad arguments");
  PTO_REQUIRE(zero_bytes == 0 || (zero && zero_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(zero) & 15) == 0),
              "rms_norm: the buffer to clear must be 16-byte aligned and a multiple of 16 bytes");
  if (rows == 0) {
    if (zero_bytes) PTO_CUDA(cudaMemsetAsync(zero, 0, zero_bytes, stream));
    return kOk;
  }
  const unsigned g = static_cast<unsigned>(rows);
  uint4* z = static_cast<uint4*>(zero);
  const long long zv = static_cast<long long>(zero_bytes / 16);
  if (x_dtype == PTO_BF16 && out_dtype == PTO_BF16)
    launch_kernel(rms_norm_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(g), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), gamma, static_cast<__nv_bfloat16*>(out), hidden, eps, copy_f32, z, zv);
  else if (x_dtype == PTO_FP32 && out_dtype == PTO_BF16)
    launch_kernel(rms_norm_kernel<float, __nv_bfloat16>, dim3(g), dim3(256), 0, stream, static_cast<const float*>(x), gamma, static_cast<__nv_bfloat16*>(out), hidden, eps, copy_f32, z, zv);
  else if (x_dtype == PTO_FP32 && out_dtype == PTO_FP32)
    launch_kernel(rms_norm_kernel<float, float>, dim3(g), dim3(256), 0, stream, static_cast<const float*>(x), gamma, static_cast<float*>(out), hidden, eps, copy_f32, z, zv);
  else if (x_dtype == PTO_BF16 && out_dtype == PTO_FP32)
    launch_kernel(rms_norm_kernel<__nv_bfloat16, float>, dim3(g), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), gamma, static_cast<float*>(out), hidden, eps, copy_f32, z, zv);
  else
    return fail(kInvalidArgument, "rms_norm: dtypes must be fp32 or bf16");
  return check_cuda(cudaGetLastError(), "rms_norm_kernel launch");
}

int contiguous_cache_tables_launch(const int32_t* seq_lens, int batch, int kv_heads, int blocks_per_seq,
                                   int32_t* seq_table, int32_t* head_table, int32_t* head_lens, cudaStream_t stream) {
  PTO_REQUIRE(seq_lens && seq_table && head_table && head_lens, "contiguous_cache_tables: NULL tensor");
  PTO_REQUIRE(batch > 0 && kv_heads > 0 && blocks_per_seq > 0, "contiguous_cache_tables: bad sizes");
  const long long n = static_cast<long long>(batch) * kv_heads * blocks_per_seq;
  launch_kernel(contiguous_cache_tables_kernel, dim3(grid_for(n, 256)), dim3(256), 0, stream, seq_lens, batch, kv_heads,
                blocks_per_seq, seq_table, head_table, head_lens);
  return check_cuda(cudaGetLastError(), "contiguous_cache_tables_kernel launch");
}

int rope_kv_append_launch(const float* qkv, const int32_t* seq_lens, const float* cos_t, const float* sin_t,
                          int table_rows, const int32_t* block_table, int max_blocks, void* k_cache, void* v_cache,
                          void* q_out, int batch, int num_heads, int kv_heads, int head_dim, int block_size,
                          long long pool_blocks, int* err, cudaStream_t stream) {
  PTO_REQUIRE(qkv && seq_lens && cos_t && sin_t && block_table && k_cache && v_cache && q_out, "rope: NULL tensor");
  PTO_REQUIRE(head_dim % 2 == 0 && head_dim <= 2048 && num_heads > 0 && kv_heads > 0, "rope: bad head geometry");
  if (batch == 0) return kOk;
  dim3 grid(batch, num_heads + kv_heads);
  launch_kernel(rope_kv_append_kernel, dim3(grid), dim3(head_dim / 2), 0, stream, 
      qkv, seq_lens, cos_t, sin_t, table_rows, block_table, max_blocks, static_cast<__nv_bfloat16*>(k_cache),
      static_cast<__nv_bfloat16*>(v_cache), static_cast<__nv_bfloat16*>(q_out), num_heads, kv_heads, head_dim,
      block_size, static_cast<int>(pool_blocks), err);
  return check_cuda(cudaGetLastError(), "rope_kv_append_kernel launch");
}

int swiglu_act_launch(const float* gate_up, void* act, long long rows, int inter, cudaStream_t stream) {
  PTO_REQUIRE(gate_up && act && rows >= 0 && inter > 0, "swiglu_act: bad arguments");
  if (rows == 0) return kOk;
  launch_kernel(swiglu_act_kernel, dim3(grid_for(rows * inter, 256)), dim3(256), 0, stream, gate_up, static_cast<__nv_bfloat16*>(act), rows, inter);
  return check_cuda(cudaGetLastError(), "swiglu_act_kernel launch");
}

int act_rows_launch(const float* h, void* act, long long n, int kind, float alpha, cudaStream_t stream) {
  PTO_REQUIRE(h && act && n >= 0 && (kind == 1 || kind == 2), "act_rows: bad arguments (kind 1 = x sigmoid(alpha x), 2 = relu)");
  if (n == 0) return kOk;
  launch_kernel(act_rows_kernel, dim3(grid_for(n, 256)), dim3(256), 0, stream, h, static_cast<__nv_bfloat16*>(act), n, kind, alpha);
  return check_cuda(cudaGetLastError(), "act_rows_kernel launch");
}

int cast_launch(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t stream) {
  return cast_zero_launch(in, in_dtype, out, out_dtype, n, nullptr, 0, stream);
}

int cast_zero_launch(const void* in, int in_dtype, void* out, int out_dtype, long long n, void* zero,
                     size_t zero_bytes, cudaStream_t stream) {
  PTO_REQUIRE(in && out && n >= 0, "cast: bad arguments");
  PTO_REQUIRE(zero_bytes == 0 || (zero && (reinterpret_cast<uintptr_t>(zero) & 15) == 0 && zero_bytes % 16 == 0),
              "cast: the region to clear must be 16-byte aligned and a multiple of 16 bytes");
  const long long zv = static_cast<long long>(zero_bytes / 16);
  if (n == 0 && zv == 0) return kOk;
  const int g = grid_for(n > zv * 4 ? n : zv * 4, 256);
  uint4* z = static_cast<uint4*>(zero);
  if (in_dtype == PTO_FP32 && out_dtype == PTO_BF16)
    launch_kernel(cast_kernel<float, __nv_bfloat16>, dim3(g), dim3(256), 0, stream, static_cast<const float*>(in), static_cast<__nv_bfloat16*>(out), n, z, zv);
  else if (in_dtype == PTO_BF16 && out_dtype == PTO_FP32)
    launch_kernel(cast_kernel<__nv_bfloat16, float>, dim3(g), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(in), static_cast<float*>(out), n, z, zv);
  else
    return fail(kInvalidArgument, "cast: only fp32 <-> bf16");
  return check_cuda(cudaGetLastError(), "cast_kernel launch");
}

int pack_weight_launch(const void* src, int src_dtype, void* dst, int k, int n, cudaStream_t stream) {
  PTO_REQUIRE(src && dst && k > 0 && n > 0, "pack_weight: bad arguments");
  dim3 grid((n + 31) / 32, (k + 31) / 32);
  if (src_dtype == PTO_FP32)
    launch_kernel(pack_weight_kernel<float>, dim3(grid), dim3(256), 0, stream, static_cast<const float*>(src), static_cast<__nv_bfloat16*>(dst), k, n);
  else if (src_dtype == PTO_BF16)
    launch_kernel(pack_weight_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), k, n);
  else
    return fail(kInvalidArgument, "pack_weight: source must be fp32 or bf16");
  return check_cuda(cudaGetLastError(), "pack_weight_kernel launch");
}

}  // namespace pto
