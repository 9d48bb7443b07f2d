// MoE routing and data movement: gate scores -> top-k, per-token FP8 quantisation, the
// dispatch permutation (counts, offsets, slots), row permutes, and the weighted combine.
//
// The integer parts follow the expert-parallel dispatch protocol of the reference
// (tests/st/distributed/test_l3_ep_dispatch_combine.py:104-299, golden :562-614):
// bucket = global expert id (destination rank = id / L, local expert = id % L); inside a
// bucket routes keep (t, k) lexicographic order; the route id carried with a row is
// t * TOPK + k.  Counts, offsets, slots and route ids are exact integers, rows are copied
// bit for bit.  The top-k is the descending selection with original indices that the
// reference builds from sort32 + mrgsort + gather (tests/st/runtime/ops/test_sort.py:602-632),
// ties going to the lower index.  The combine is combine_step (:337-402): y[t] = sum over k of
// fp32(row), in k order.
#include "common.cuh"
#include "kernels.h"

namespace pto {
namespace {

constexpr int kMaxExpertsPerLane = 32;  // up to 1024 experts per token row

// One warp per token.  scores_in holds logits (is_logits = 1: sigmoid applied here) or scores.  PER = experts a lane
// holds (ceil(experts / 32) rounded up to a power of two): the selection loops are unrolled over exactly those.
template <int PER>
__global__ void __launch_bounds__(256)
moe_topk_kernel(const float* __restrict__ scores_in, const float* __restrict__ bias, int is_logits, int tokens,
                int experts, int topk, int32_t* __restrict__ idx_out, float* __restrict__ w_out) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  float s[PER], sel[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    s[j] = 0.f;
    sel[j] = -INFINITY;
    const int e = j * 32 + lane;
    if (e < experts) {
      float v = scores_in[static_cast<size_t>(t) * experts + e];
      if (is_logits) v = 1.f / (1.f + expf(-v));
      s[j] = v;
      sel[j] = v + (bias ? bias[e] : 0.f);
    }
  }
  float picked_sum = 0.f, my_pick = 0.f;
  int my_idx = 0;
  for (int k = 0; k < topk; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = j * 32 + lane;
      if (sel[j] > best) { best = sel[j]; best_e = e; }  // ascending e per lane: ties keep the lower id
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    const int owner = best_e & 31, slot = best_e >> 5;
    float sc = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (j == slot && lane == owner) { sc = s[j]; sel[j] = -INFINITY; }
    sc = __shfl_sync(0xffffffffu, sc, owner);
    picked_sum += sc;
    if (lane == k) { my_pick = sc; my_idx = best_e; }
  }
  if (lane < topk) {
    idx_out[static_cast<size_t>(t) * topk + lane] = my_idx;
    w_out[static_cast<size_t>(t) * topk + lane] = my_pick / picked_sum;
  }
}

// scale = amax / 448 over a (row, 128-column group) (1 if the group is all zero), q = e4m3(x / scale), round to
// nearest even, saturating.  Sixteen lanes per group, eight elements per lane (16-byte loads of bf16), and four
// pairs of groups in flight per warp: with one group per warp and scalar loads the kernel had 16 KB in flight per
// SM and ran at a third of the HBM rate.
template <typename TI>
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const TI* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, long long rows,
                     int cols) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int kU = 4;                                    // group pairs per warp and pass
  const int lane = threadIdx.x & 31, half = lane >> 4, hl = lane & 15;
  const int groups = cols / 128;
  const long long total = rows * groups;
  const long long warp_id = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long base = warp_id * (2 * kU); base < total; base += warps * (2 * kU)) {
    float v[kU][8];
    long long off[kU];
    bool in[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const long long g = base + 2 * u + half;
      in[u] = g < total;
      const long long r = in[u] ? g / groups : 0;
      off[u] = in[u] ? r * cols + static_cast<long long>(g - r * groups) * 128 + hl * 8 : 0;
      if constexpr (sizeof(TI) == 2) {
        const uint4 w = in[u] ? __ldg(reinterpret_cast<const uint4*>(x + off[u])) : make_uint4(0, 0, 0, 0);
        v[u][0] = bf16_lo_to_float(w.x); v[u][1] = bf16_hi_to_float(w.x);
        v[u][2] = bf16_lo_to_float(w.y); v[u][3] = bf16_hi_to_float(w.y);
        v[u][4] = bf16_lo_to_float(w.z); v[u][5] = bf16_hi_to_float(w.z);
        v[u][6] = bf16_lo_to_float(w.w); v[u][7] = bf16_hi_to_float(w.w);
      } else {
        const float4 a = in[u] ? __ldg(reinterpret_cast<const float4*>(x + off[u])) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 b = in[u] ? __ldg(reinterpret_cast<const float4*>(x + off[u]) + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
        v[u][0] = a.x; v[u][1] = a.y; v[u][2] = a.z; v[u][3] = a.w;
        v[u][4] = b.x; v[u][5] = b.y; v[u][6] = b.z; v[u][7] = b.w;
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[u][i]));
#pragma unroll
      for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // within 16 lanes
      const float sc = amax > 0.f ? amax / 448.f : 1.f;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[u][i] / sc, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
        hi |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[u][4 + i] / sc, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
      }
      if (in[u]) {
        *reinterpret_cast<uint2*>(q + off[u]) = make_uint2(lo, hi);
        if (hl == 0) scale[base + 2 * u + half] = sc;
      }
    }
  }
}

// Dispatch plan = a stable counting sort of the routes by bucket (global expert id), in three small launches.
// Routes are cut into chunks of `chunk` consecutive routes, one warp per chunk.
//
//   moe_chunk_hist_kernel   every warp walks its chunk 32 routes at a time and counts, per bucket, the routes
//                           of the chunk: hist[chunk][bucket]
//   moe_offsets_kernel      per bucket an exclusive scan over the chunks (hist becomes "routes of this bucket in
//                           earlier chunks"), the bucket totals, and their exclusive scan: counts, offsets
//   moe_positions_kernel    every warp walks its chunk again: a route's slot = offsets[bucket] + routes of the
//                           bucket in earlier chunks + routes of the bucket earlier in this chunk
//
// The walk keeps (t, k) order: lanes holding the same bucket are found with a match, ranked by lane, and the
// running per-chunk count is advanced by the lowest of them.
__device__ __forceinline__ int chunk_walk_step(int e, bool valid, int lane, int* hist) {
  // returns the number of earlier routes of the chunk in bucket e (for valid lanes); advances hist
  const unsigned same = __match_any_sync(0xffffffffu, valid ? e : -1);
  int before = 0;
  if (valid) {
    before = hist[e] + __popc(same & ((1u << lane) - 1u));
  }
  __syncwarp();
  if (valid && (same & ((1u << lane) - 1u)) == 0) hist[e] += __popc(same);   // the lowest lane of each group
  __syncwarp();
  return before;
}

__global__ void __launch_bounds__(256)
moe_chunk_hist_kernel(const int32_t* __restrict__ expert_of, int routes, int buckets, int chunk, int n_chunks,
                      int32_t* __restrict__ hist_out) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int hist_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int c = blockIdx.x * warps + warp;
  int* hist = hist_smem + warp * buckets;
  for (int i = lane; i < buckets; i += 32) hist[i] = 0;
  __syncwarp();
  if (c >= n_chunks) return;
  const int r0 = c * chunk, r1 = min(routes, r0 + chunk);
  for (int base = r0; base < r1; base += 32) {
    const int r = base + lane;
    const int e = r < r1 ? expert_of[r] : -1;
    chunk_walk_step(e, r < r1 && e >= 0 && e < buckets, lane, hist);
  }
  for (int i = lane; i < buckets; i += 32) hist_out[static_cast<size_t>(c) * buckets + i] = hist[i];
}

// Single CTA.  hist [n_chunks][buckets] -> in place: routes of the bucket in earlier chunks; counts[b] = total;
// offsets[0..buckets] = exclusive scan of counts.
__global__ void __launch_bounds__(1024) moe_offsets_kernel(int32_t* __restrict__ hist, int n_chunks, int n,
                                                           int32_t* __restrict__ counts, int32_t* __restrict__ offsets) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int warp_sum_s[32];
  __shared__ int carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    const int i = base + threadIdx.x;
    int v = 0;
    if (i < n) {
      for (int c0 = 0; c0 < n_chunks; c0 += 8) {   // consecutive threads read consecutive buckets of a chunk;
        int h[8];                                  // eight loads in flight before the stores that follow them
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = c0 + j < n_chunks ? hist[static_cast<size_t>(c0 + j) * n + i] : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (c0 + j < n_chunks) hist[static_cast<size_t>(c0 + j) * n + i] = v;
          v += h[j];
        }
      }
      counts[i] = v;
    }
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += u;
    }
    if (lane == 31) warp_sum_s[warp] = inc;
    __syncthreads();
    int before = carry_s;
    for (int w = 0; w < warp; ++w) before += warp_sum_s[w];
    if (i < n) offsets[i] = before + inc - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = before + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[n] = carry_s;
}

// pos[r] = slot of route r in the bucket-sorted order; route_at[pos[r]] = r.
// A route whose expert id lies outside [0, buckets) belongs to no bucket: it is reported through the error
// word (kErrBadIndex), gets pos = -1 (the combine skips it) and nothing is read or written at an address
// derived from the id.  Such routes leave the last slots of route_at unused; those are set to -1.
__global__ void __launch_bounds__(256)
moe_positions_kernel(const int32_t* __restrict__ expert_of, const int32_t* __restrict__ chunk_before,
                     const int32_t* __restrict__ offsets, int routes, int buckets, int chunk, int n_chunks,
                     int32_t* __restrict__ pos, int32_t* __restrict__ route_at, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int hist_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int c = blockIdx.x * warps + warp;
  int* hist = hist_smem + warp * buckets;
  if (c >= n_chunks) return;
  // start the walk at "offset of the bucket + routes of the bucket in earlier chunks"
  for (int i = lane; i < buckets; i += 32) hist[i] = offsets[i] + chunk_before[static_cast<size_t>(c) * buckets + i];
  __syncwarp();
  const int total = offsets[buckets];
  const int r0 = c * chunk, r1 = min(routes, r0 + chunk);
  for (int base = r0; base < r1; base += 32) {
    const int r = base + lane;
    const int e = r < r1 ? expert_of[r] : -1;
    const bool valid = r < r1 && e >= 0 && e < buckets;
    const int p = chunk_walk_step(e, valid, lane, hist);
    if (r < r1) {
      if (r >= total) route_at[r] = -1;   // slots [total valid routes, routes) have no route
      if (valid) {
        pos[r] = p;
        route_at[p] = r;
      } else {
        report_error(err, kErrBadIndex, 60, r);
        pos[r] = -1;
      }
    }
  }
}

// Arrival plan of the expert-parallel receiver.  Rows arrive source-major, and inside a source ordered by
// local expert: recv_counts[s][e] rows from source s for local expert e.  The expert GEMM wants them grouped
// by expert, inside an expert by source and then arrival order (the bucket order of the reference's
// dispatch_step, tests/st/distributed/test_l3_ep_dispatch_combine.py:184-218).  One CTA:
//   counts[e]         rows of expert e
//   offsets[e]        first grouped row of expert e: dense (running sum, offsets[L] = number of rows) when
//                     slot_stride == 0, else e * slot_stride (the reference's padded [L, R] receive layout)
//   arrival_of[g]     arrival row that goes to grouped row g (-1 for a grouped row nothing arrives at)
//   grouped_of[a]     grouped row of arrival row a
// Rows that do not fit (more than `capacity` arrival or grouped rows, or more than slot_stride rows for one
// expert) are dropped and reported through the error word.
__global__ void __launch_bounds__(1024)
moe_recv_plan_kernel(const int32_t* __restrict__ recv_counts, int world, int local_experts, int slot_stride,
                     int capacity, int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                     int32_t* __restrict__ arrival_of, int32_t* __restrict__ grouped_of, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int plan_smem[];
  const int cells = world * local_experts;
  int* arr0 = plan_smem;             // [cells] first arrival row of cell (s, e)
  int* grp0 = plan_smem + cells;     // [cells] first grouped row of cell (s, e)
  int* eoff = grp0 + cells;          // [local_experts + 1]
  for (int g = threadIdx.x; g < capacity; g += blockDim.x) arrival_of[g] = -1;
  if (threadIdx.x == 0) {
    int run = 0;
    for (int c = 0; c < cells; ++c) {            // arrival order: s major, e minor
      arr0[c] = run;
      run += max(recv_counts[c], 0);
    }
    if (run > capacity) report_error(err, kErrBadIndex, 61, run);
    run = 0;
    for (int e = 0; e < local_experts; ++e) {    // grouped order: e major, s minor
      const int first = slot_stride > 0 ? e * slot_stride : run;
      eoff[e] = first;
      int in_e = 0;
      for (int s = 0; s < world; ++s) {
        grp0[s * local_experts + e] = first + in_e;
        in_e += max(recv_counts[s * local_experts + e], 0);
      }
      if (slot_stride > 0 && in_e > slot_stride) report_error(err, kErrBadIndex, 64, e);
      counts[e] = in_e;
      run = first + in_e;
    }
    eoff[local_experts] = slot_stride > 0 ? local_experts * slot_stride : run;
    if (eoff[local_experts] > capacity) report_error(err, kErrBadIndex, 61, eoff[local_experts]);
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= local_experts; e += blockDim.x) offsets[e] = min(eoff[e], capacity);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int c = warp; c < cells; c += warps) {
    const int e = c % local_experts;
    const int n = max(recv_counts[c], 0), a0 = arr0[c], g0 = grp0[c];
    const int g_end = slot_stride > 0 ? min((e + 1) * slot_stride, capacity) : capacity;
    for (int i = lane; i < n; i += 32) {
      if (a0 + i < capacity) {
        const bool fits = g0 + i < g_end;
        grouped_of[a0 + i] = fits ? g0 + i : -1;
        if (fits) arrival_of[g0 + i] = a0 + i;
      }
    }
  }
}

// dst row p = src row (src_row_of[p] / div) for each of `n` row-major byte arrays; each array has its own
// source and destination row stride, so that several arrays can be packed side by side into one payload row
// (and unpacked again).  One warp per destination row; 16-byte copies where both rows are 16-byte aligned.
// An index of -1 marks a destination row that nothing maps to (an unused slot of a padded layout, a route the
// plan refused): the row is cleared.  Any other source row outside [0, src_rows) is cleared too and reported
// through the error word (kErrBadIndex).
struct RowArrays {
  const uint8_t* src[3];
  uint8_t* dst[3];
  long long src_stride[3], dst_stride[3];
  int row_bytes[3];
  int n;
};

__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(RowArrays a, const int32_t* __restrict__ src_row_of, int div, long long rows,
                       long long src_rows, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  for (long long p = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); p < rows;
       p += static_cast<long long>(gridDim.x) * (blockDim.x >> 5)) {
    const long long raw = src_row_of ? src_row_of[p] : p;
    const long long s = raw >= 0 ? raw / div : -1;
    const bool ok = s >= 0 && s < src_rows;
    if (!ok && raw != -1 && lane == 0) report_error(err, kErrBadIndex, 62, static_cast<int>(p));
    for (int i = 0; i < a.n; ++i) {
      const int rb = a.row_bytes[i];
      const uint8_t* sp = a.src[i] + (ok ? s : 0) * a.src_stride[i];
      uint8_t* dp = a.dst[i] + p * a.dst_stride[i];
      if (!ok) {
        for (int c = lane; c < rb; c += 32) dp[c] = 0;
      } else if ((rb & 15) == 0 && ((reinterpret_cast<uintptr_t>(sp) | reinterpret_cast<uintptr_t>(dp)) & 15) == 0) {
        // four loads in flight per lane before the first store: source and destination are plain byte pointers, so
        // the compiler must keep every load behind the store before it
        const uint4* s16 = reinterpret_cast<const uint4*>(sp);
        uint4* d16 = reinterpret_cast<uint4*>(dp);
        const int n16 = rb / 16;
        int c = lane;
        for (; c + 96 < n16; c += 128) {
          const uint4 v0 = __ldg(s16 + c), v1 = __ldg(s16 + c + 32), v2 = __ldg(s16 + c + 64), v3 = __ldg(s16 + c + 96);
          d16[c] = v0; d16[c + 32] = v1; d16[c + 64] = v2; d16[c + 96] = v3;
        }
        for (; c < n16; c += 32) d16[c] = __ldg(s16 + c);
      } else if ((rb & 3) == 0 && ((reinterpret_cast<uintptr_t>(sp) | reinterpret_cast<uintptr_t>(dp)) & 3) == 0) {
        for (int c = lane; c < rb / 4; c += 32) reinterpret_cast<uint32_t*>(dp)[c] = reinterpret_cast<const uint32_t*>(sp)[c];
      } else {
        for (int c = lane; c < rb; c += 32) dp[c] = sp[c];
      }
    }
  }
}

// route_weight_sorted[p] = weights[route_at[p]]
__global__ void moe_gather_f32_kernel(const float* __restrict__ src, const int32_t* __restrict__ index, long long n,
                                      long long n_src, float* __restrict__ dst, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long j = index[i];
  if (j < 0 || j >= n_src) {
    if (j != -1) report_error(err, kErrBadIndex, 63, static_cast<int>(i));
    dst[i] = 0.f;
  } else {
    dst[i] = src[j];
  }
}

// y[t] = bf16( sum_k fp32(rows[pos[t*topk + k]]) + fp32(shared[t]) ), k ascending.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ rows, const int32_t* __restrict__ pos,
                   const __nv_bfloat16* __restrict__ shared, int topk, int hidden, long long n_rows,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ y32) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // eight routes at a time: their positions first, then their rows (all loads in flight together), then the sums in
    // k order.  A route that was refused by the plan, or a slot outside `rows`, contributes zeros.
    for (int k0 = 0; k0 < topk; k0 += 8) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int p = k0 + j < topk ? pos[static_cast<size_t>(t) * topk + k0 + j] : -1;
        v[j] = (p >= 0 && p < n_rows) ? __ldg(reinterpret_cast<const uint4*>(rows + static_cast<size_t>(p) * hidden + c))
                                      : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] += bf16_lo_to_float(w[i]);
          acc[2 * i + 1] += bf16_hi_to_float(w[i]);
        }
      }
    }
    if (shared) {
      const uint4 v = *reinterpret_cast<const uint4*>(shared + static_cast<size_t>(t) * hidden + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += bf16_lo_to_float(w[i]);
        acc[2 * i + 1] += bf16_hi_to_float(w[i]);
      }
    }
    if (y32) {
#pragma unroll
      for (int i = 0; i < 8; ++i) y32[static_cast<size_t>(t) * hidden + c + i] = acc[i];
    }
    if (y) {
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * hidden + c) = o;
    }
  }
}

// y[r, :] = bf16(fp32(x[r, :]) * w[r * w_stride]): the stand-in expert of the reference's expert-parallel test
// (local_expert_step, tests/st/distributed/test_l3_ep_dispatch_combine.py:309-327).  Rows r with
// r % slot_stride >= count[r / slot_stride] (unused slots of a padded [experts, slots] layout) are skipped when
// `count` is given.
__global__ void __launch_bounds__(256)
scale_rows_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, int w_stride,
                  const int32_t* __restrict__ count, int slot_stride, long long rows, int cols,
                  __nv_bfloat16* __restrict__ y) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    if (count != nullptr && static_cast<int>(r % slot_stride) >= count[r / slot_stride]) continue;
    const float wr = w[r * w_stride];
    for (int c = threadIdx.x; c < cols; c += blockDim.x)
      y[r * cols + c] = __float2bfloat16_rn(__bfloat162float(x[r * cols + c]) * wr);
  }
}

// ---- results on their way home through peer memory (expert parallel, every rank on the same NVSwitch) ----
//
// The expert GEMM leaves its result rows in the order the rows arrived: source rank after source rank, and inside a
// source in the order that rank sorted them.  A source's block therefore belongs, as it stands, at one offset of
// that source's own sorted result buffer -- the offset the source sent along with its counts.  This kernel copies
// every block straight into its source's buffer with plain stores to peer memory (one warp per row, 16-byte
// chunks, four loads in flight) instead of handing the rows to an all-to-all; the block for this rank itself takes the
// same path.  When the last CTA is done it raises this rank's flag on every peer to the step number: each CTA
// fences its stores system-wide before it counts itself in, the last one fences again and stores the flags with
// release semantics, so a peer that has seen the flag sees the rows.  No flag is ever reset: steps only count up.
__global__ void __launch_bounds__(256)
moe_push_rows_kernel(const uint8_t* __restrict__ rows, int row_bytes, const int32_t* __restrict__ recv_counts, int world,
                     int local_experts, const int32_t* __restrict__ dst_base, MoePeerTable peers, int my_rank, int step,
                     long long dst_rows, int* __restrict__ done_counter, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ long long first[kMoeMaxPeers + 1];   // arrival row at which the block of source s begins
  __shared__ int n_src[kMoeMaxPeers];
  if (static_cast<int>(threadIdx.x) < world) {
    int n = 0;
    for (int e = 0; e < local_experts; ++e) n += recv_counts[threadIdx.x * local_experts + e];
    n_src[threadIdx.x] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    long long run = 0;
    for (int r = 0; r < world; ++r) {
      first[r] = run;
      run += n_src[r];
    }
    first[world] = run;
  }
  __syncthreads();
  const long long total = first[world];
  const int lane = threadIdx.x & 31;
  const int n16 = row_bytes / 16;
  for (long long a = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); a < total;
       a += static_cast<long long>(gridDim.x) * (blockDim.x >> 5)) {
    int src = 0;
    while (src + 1 < world && a >= first[src + 1]) ++src;
    const long long slot = static_cast<long long>(dst_base[src]) + (a - first[src]);
    if (dst_base[src] < 0 || slot >= dst_rows) {          // a base that does not belong to a sorted buffer of this size
      if (lane == 0) report_error(err, kErrBadIndex, 65, src);
      continue;
    }
    const uint4* s16 = reinterpret_cast<const uint4*>(rows + a * row_bytes);
    uint4* d16 = reinterpret_cast<uint4*>(peers.back[src] + slot * row_bytes);
    int c = lane;
    for (; c + 96 < n16; c += 128) {
      const uint4 v0 = s16[c], v1 = s16[c + 32], v2 = s16[c + 64], v3 = s16[c + 96];
      d16[c] = v0; d16[c + 32] = v1; d16[c + 64] = v2; d16[c + 96] = v3;
    }
    for (; c < n16; c += 32) d16[c] = s16[c];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();                                // cumulative: the CTA's stores, ordered before it by the barrier
    if (atomicAdd(done_counter, 1) == static_cast<int>(gridDim.x) - 1) {
      *done_counter = 0;                                   // for the next launch (stream order)
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peers.flags[r] + my_rank), "r"(step) : "memory");
    }
  }
}

// base[s] = rows that arrive here from the ranks before s (recv_counts int32 [world][local_experts]): where the block
// of source s begins in this rank's receive buffer.
__global__ void __launch_bounds__(32)
moe_recv_bases_kernel(const int32_t* __restrict__ recv_counts, int world, int local_experts, int32_t* __restrict__ base) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x != 0) return;
  int run = 0;
  for (int s = 0; s < world; ++s) {
    base[s] = run;
    for (int e = 0; e < local_experts; ++e) run += recv_counts[s * local_experts + e];
  }
}

// One warp: lane r waits (bounded) until rank r has raised its flag here to `step`.
__global__ void __launch_bounds__(32)
moe_wait_flags_kernel(const int32_t* __restrict__ flags, int world, int step, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = threadIdx.x;
  if (r >= world) return;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
    if (v - step >= 0) return;
    if (global_timer_ns() - t0 > 2 * kWaitTimeoutNs) {
      report_error(err, kErrBarrierTimeout, 66, r);
      return;
    }
    __nanosleep(200);
  }
}

int grid_rows(long long rows, int warps_per_cta) {
  long long g = (rows + warps_per_cta - 1) / warps_per_cta;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

int moe_topk_launch(const float* scores, const float* bias, int is_logits, int tokens, int experts, int topk,
                    int32_t* idx, float* weights, cudaStream_t stream) {
  PTO_REQUIRE(scores && idx && weights, "moe_topk: NULL tensor");
  PTO_REQUIRE(experts > 0 && experts <= 32 * kMaxExpertsPerLane, "moe_topk: at most 1024 experts");
  PTO_REQUIRE(topk > 0 && topk <= 32 && topk <= experts, "moe_topk: 1 <= topk <= min(32, experts)");
  if (tokens <= 0) return kOk;
  const int per = (experts + 31) / 32;
  const dim3 grid((tokens + 7) / 8), block(256);
#define PTO_TOPK(P) launch_kernel(moe_topk_kernel<P>, grid, block, 0, stream, scores, bias, is_logits, tokens, experts, topk, idx, weights)
  if (per <= 1) PTO_TOPK(1);
  else if (per <= 2) PTO_TOPK(2);
  else if (per <= 4) PTO_TOPK(4);
  else if (per <= 8) PTO_TOPK(8);
  else if (per <= 16) PTO_TOPK(16);
  else PTO_TOPK(32);
#undef PTO_TOPK
  return check_cuda(cudaGetLastError(), "moe_topk_kernel launch");
}

int quantize_rows_launch(const void* x, int x_dtype, void* q, float* scale, long long rows, int cols,
                         cudaStream_t stream) {
  PTO_REQUIRE(x && q && scale, "quantize_rows: NULL tensor");
  PTO_REQUIRE(cols > 0 && cols % 128 == 0, "quantize_rows: columns must be a multiple of 128");
  PTO_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
              "quantize_rows: x must be 16-byte aligned, q 8-byte aligned");
  if (rows <= 0) return kOk;
  const int g = grid_rows((rows * (cols / 128) + 7) / 8, 8);     // a warp takes eight groups per pass
  if (x_dtype == PTO_BF16)
    launch_kernel(quantize_rows_kernel<__nv_bfloat16>, dim3(g), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scale, rows, cols);
  else if (x_dtype == PTO_FP32)
    launch_kernel(quantize_rows_kernel<float>, dim3(g), dim3(256), 0, stream, static_cast<const float*>(x), static_cast<uint8_t*>(q), scale, rows, cols);
  else
    return fail(kInvalidArgument, "quantize_rows: input must be bf16 or fp32");
  return check_cuda(cudaGetLastError(), "quantize_rows_kernel launch");
}

// expert_of int32 [routes] -> counts [buckets], offsets [buckets + 1], pos [routes], route_at [routes].
// `work` is an int32 [routes + buckets] work array (per-chunk bucket histograms).
int moe_dispatch_plan_launch(const int32_t* expert_of, int routes, int buckets, int32_t* counts, int32_t* offsets,
                             int32_t* pos, int32_t* route_at, int32_t* work, int* err, cudaStream_t stream) {
  PTO_REQUIRE(expert_of && counts && offsets && pos && route_at && work, "moe_dispatch_plan: NULL tensor");
  PTO_REQUIRE(buckets > 0 && buckets <= 8192 && routes >= 0, "moe_dispatch_plan: 1..8192 buckets, routes >= 0");
  // chunk >= buckets keeps the histograms (n_chunks x buckets ints) inside routes + buckets ints
  const int chunk = ((buckets > 512 ? buckets : 512) + 31) / 32 * 32;
  const int n_chunks = routes > 0 ? (routes + chunk - 1) / chunk : 0;
  int warps = 12288 / buckets;
  warps = warps > 8 ? 8 : (warps < 1 ? 1 : warps);
  const size_t smem = sizeof(int) * static_cast<size_t>(warps) * buckets;
  const int blocks = (n_chunks + warps - 1) / warps;
  if (n_chunks > 0) {
    launch_kernel(moe_chunk_hist_kernel, dim3(blocks), dim3(warps * 32), smem, stream, expert_of, routes, buckets, chunk,
                  n_chunks, work);
    PTO_CUDA(cudaGetLastError());
  }
  launch_kernel(moe_offsets_kernel, dim3(1), dim3(1024), 0, stream, work, n_chunks, buckets, counts, offsets);
  PTO_CUDA(cudaGetLastError());
  if (n_chunks > 0) {
    launch_kernel(moe_positions_kernel, dim3(blocks), dim3(warps * 32), smem, stream, expert_of,
                  static_cast<const int32_t*>(work), static_cast<const int32_t*>(offsets), routes, buckets, chunk,
                  n_chunks, pos, route_at, err);
    PTO_CUDA(cudaGetLastError());
  }
  return kOk;
}

int moe_recv_plan_launch(const int32_t* recv_counts, int world, int local_experts, int slot_stride, int capacity,
                         int32_t* counts, int32_t* offsets, int32_t* arrival_of, int32_t* grouped_of, int* err,
                         cudaStream_t stream) {
  PTO_REQUIRE(recv_counts && counts && offsets && arrival_of && grouped_of, "moe_recv_plan: NULL tensor");
  PTO_REQUIRE(world > 0 && local_experts > 0 && capacity >= 0 && slot_stride >= 0, "moe_recv_plan: bad sizes");
  const size_t smem = sizeof(int) * (2 * static_cast<size_t>(world) * local_experts + local_experts + 1);
  PTO_REQUIRE(smem <= 48 * 1024, "moe_recv_plan: world * local_experts too large");
  launch_kernel(moe_recv_plan_kernel, dim3(1), dim3(1024), smem, stream, recv_counts, world, local_experts,
                slot_stride, capacity, counts, offsets, arrival_of, grouped_of, err);
  return check_cuda(cudaGetLastError(), "moe_recv_plan_kernel launch");
}

int moe_move_rows_launch(const void* const* src, const long long* src_stride, void* const* dst,
                         const long long* dst_stride, const int* row_bytes, int n_arrays, const int32_t* src_row_of,
                         int div, long long rows, long long src_rows, int* err, cudaStream_t stream) {
  PTO_REQUIRE(n_arrays >= 1 && n_arrays <= 3 && div >= 1, "moe_move_rows: 1..3 arrays, div >= 1");
  PTO_REQUIRE(src && dst && row_bytes, "moe_move_rows: NULL argument");
  if (rows <= 0) return kOk;
  RowArrays a;
  a.n = n_arrays;
  for (int i = 0; i < n_arrays; ++i) {
    PTO_REQUIRE(src[i] && dst[i] && row_bytes[i] > 0, "moe_move_rows: NULL array or empty row");
    a.src[i] = static_cast<const uint8_t*>(src[i]);
    a.dst[i] = static_cast<uint8_t*>(dst[i]);
    a.row_bytes[i] = row_bytes[i];
    a.src_stride[i] = src_stride ? src_stride[i] : row_bytes[i];
    a.dst_stride[i] = dst_stride ? dst_stride[i] : row_bytes[i];
    PTO_REQUIRE(a.src_stride[i] >= row_bytes[i] && a.dst_stride[i] >= row_bytes[i], "moe_move_rows: stride below row size");
  }
  launch_kernel(moe_gather_rows_kernel, dim3(grid_rows(rows, 8)), dim3(256), 0, stream, a, src_row_of, div, rows,
                src_rows, err);
  return check_cuda(cudaGetLastError(), "moe_gather_rows_kernel launch");
}

int scale_rows_launch(const void* x, const float* w, int w_stride, const int32_t* count, int slot_stride,
                      long long rows, int cols, void* y, cudaStream_t stream) {
  PTO_REQUIRE(x && w && y, "scale_rows: NULL tensor");
  PTO_REQUIRE(cols > 0 && w_stride >= 1 && (count == nullptr || slot_stride > 0), "scale_rows: bad sizes");
  if (rows <= 0) return kOk;
  launch_kernel(scale_rows_kernel, dim3(grid_rows(rows, 1)), dim3(256), 0, stream,
                static_cast<const __nv_bfloat16*>(x), w, w_stride, count, slot_stride, rows, cols,
                static_cast<__nv_bfloat16*>(y));
  return check_cuda(cudaGetLastError(), "scale_rows_kernel launch");
}

int moe_gather_f32_launch(const float* src, const int32_t* index, long long n, long long n_src, float* dst, int* err,
                          cudaStream_t stream) {
  PTO_REQUIRE(src && index && dst, "moe_gather_f32: NULL tensor");
  if (n <= 0) return kOk;
  launch_kernel(moe_gather_f32_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, stream, src, index, n,
                n_src, dst, err);
  return check_cuda(cudaGetLastError(), "moe_gather_f32_kernel launch");
}

int moe_combine_launch(const void* rows, const int32_t* pos, const void* shared, int tokens, int topk, int hidden,
                       long long n_rows, void* y_bf16, float* y_f32, cudaStream_t stream) {
  PTO_REQUIRE(rows && pos && (y_bf16 || y_f32), "moe_combine: NULL tensor");
  PTO_REQUIRE(hidden > 0 && hidden % 8 == 0 && topk > 0, "moe_combine: hidden must be a multiple of 8");
  if (tokens <= 0) return kOk;
  launch_kernel(moe_combine_kernel, dim3(tokens), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(rows), pos,
                                                 static_cast<const __nv_bfloat16*>(shared), topk, hidden, n_rows,
                                                 static_cast<__nv_bfloat16*>(y_bf16), y_f32);
  return check_cuda(cudaGetLastError(), "moe_combine_kernel launch");
}

// Result rows (arrival order, `row_bytes` each, a multiple of 16) to the sorted result buffers of their source ranks
// through peer memory; then this rank's flag on every peer becomes `step`.  recv_counts int32 [world][local_experts]
// and dst_base int32 [world] (the offset each source asked for) are device arrays; `rows_hint` sizes the grid.
int moe_push_rows_launch(const void* rows, int row_bytes, const int32_t* recv_counts, int world, int local_experts,
                         const int32_t* dst_base, const MoePeerTable& peers, int my_rank, int step, long long dst_rows,
                         long long rows_hint, int* done_counter, int* err, cudaStream_t stream) {
  PTO_REQUIRE(rows && recv_counts && dst_base && done_counter, "moe_push_rows: NULL argument");
  PTO_REQUIRE(world >= 1 && world <= kMoeMaxPeers && local_experts >= 1 && row_bytes > 0 && row_bytes % 16 == 0,
              "moe_push_rows: 1..32 ranks, rows a multiple of 16 bytes");
  launch_kernel(moe_push_rows_kernel, dim3(grid_rows(rows_hint, 8)), dim3(256), 0, stream, static_cast<const uint8_t*>(rows),
                row_bytes, recv_counts, world, local_experts, dst_base, peers, my_rank, step, dst_rows, done_counter, err);
  return check_cuda(cudaGetLastError(), "moe_push_rows_kernel launch");
}

int moe_recv_bases_launch(const int32_t* recv_counts, int world, int local_experts, int32_t* base, cudaStream_t stream) {
  PTO_REQUIRE(recv_counts && base && world >= 1 && local_experts >= 1, "moe_recv_bases: bad argument");
  launch_kernel(moe_recv_bases_kernel, dim3(1), dim3(32), 0, stream, recv_counts, world, local_experts, base);
  return check_cuda(cudaGetLastError(), "moe_recv_bases_kernel launch");
}

int moe_wait_flags_launch(const int32_t* flags, int world, int step, int* err, cudaStream_t stream) {
  PTO_REQUIRE(flags && world >= 1 && world <= kMoeMaxPeers, "moe_wait_flags: 1..32 ranks");
  launch_kernel(moe_wait_flags_kernel, dim3(1), dim3(32), 0, stream, flags, world, step, err);
  return check_cuda(cudaGetLastError(), "moe_wait_flags_kernel launch");
}

}  // namespace pto
