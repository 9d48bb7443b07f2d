// Paged-attention decode over block tables for sm_100a.
//
// Replaces the reference's per-KV-block four-task pipeline (QK matmul, softmax
// prepare, PV matmul, online update: examples/models/04_paged_attention.py:62-227,
// orchestration :272-367) by one persistent, bandwidth-bound kernel plus a small
// merge kernel.
//
// Data layout in HBM
//   query        bf16 [batch * q_len * num_heads, 128], row = (sequence, draft j, head)
//   key/value    bf16 [pool_blocks * kv_heads * block_size, 128], row = (block, kv head, token)
//                (for kv_heads == 1 this is the reference's [(block, token), head_dim])
//   block_table  int32 [batch, max_blocks];  context_lens int32 [batch]
//
// Work decomposition
//   item  = (sequence, kv head, row group); its rows are the q_len * group query
//           rows that share the KV head (16 or 32 rows per item, zero padded).
//   tile  = 128 consecutive tokens of one item (128 / block_size physical blocks).
//   All tiles of all items form one global index space that is cut into equal
//   contiguous ranges, one per CTA (one CTA per SM).  A CTA therefore streams the
//   same number of KV bytes as every other CTA whatever the context lengths are.
//   Each maximal run of tiles of one item inside a CTA range is a "segment".
//
// CTA = 1 producer warp + 4 consumer warps
//   producer: walks the tile list, reads block ids, issues TMA loads
//             (cp.async.bulk.tensor, 128-byte swizzle) of K and V tiles into a ring
//             of 32 KB buffers guarded by full/empty mbarriers.
//   consumer warp w: owns tokens [32w, 32w+32) of every tile; S = Q K^T and O += P V
//             with mma.sync m16n8k16 (bf16 in, fp32 accumulate), online softmax with
//             quad shuffles, P rounded to bf16 and l summed from the rounded P as the
//             reference does (04_paged_attention.py:79-134).  Warps never synchronise
//             with one another on the data path; each keeps its own (m, l, O).
//   At the end of a segment every consumer warp writes its partial (m, l, O) to
//   scratch slot (item + cta); the merge kernel combines the partials of an item
//   (all warps of all covering CTAs) and writes O / l (0 where l == 0, the guard of
//   examples/models/09_paged_attention_spmd.py:647-651).
//
// Every mbarrier wait is bounded; on timeout the kernel records an error word and
// returns.
#include "common.cuh"

#include <math.h>
#include <stdio.h>

#include <mutex>

#include "kernels.h"

namespace pto {

namespace {

constexpr int kTile = 128;          // tokens per tile
constexpr int kD = 128;             // head_dim of the tensor-core path
constexpr int kConsumers = 4;       // consumer warps
constexpr int kThreads = 32 * (kConsumers + 1);
constexpr int kBuf = 32768;         // bytes of one K or V tile
constexpr int kNBuf = 6;            // ring depth (3 K + 3 V tiles in flight)
constexpr int kMaxBatch = 4096;     // sequences per launch (prefix array in smem)
constexpr float kLog2e = 1.4426950408889634f;

struct PAParams {
  const __nv_bfloat16* q;
  const int* block_table;
  const int* context_lens;
  float* part_o;    // [slot][warp][rows_per_item][128]
  float* part_ml;   // [slot][warp][rows_per_item][2]
  int* plan;        // [0]=total tiles, [1]=tiles per cta, [2..2+batch] prefix of tiles per sequence
  int* err;
  void* out;
  int out_fp32;
  int batch, num_heads, kv_heads, group, q_len;
  int block_size, max_blocks, blocks_per_tile;
  int rows_total;     // q_len * group
  int row_groups;     // ceil(rows_total / rows_per_item)
  int rows_per_item;  // 16 * MT
  int subs;           // kv_heads * row_groups (items per sequence)
  int pool_blocks;
  int grid_main;
  float scale_log2;   // softmax scale * log2(e)
};

__device__ __forceinline__ int tiles_of(int ctx, const PAParams& p) {
  int cap = p.max_blocks * p.block_size;
  if (ctx > cap) ctx = cap;
  if (ctx < 0) ctx = 0;
  return (ctx + kTile - 1) / kTile;
}

// first b with prefix[b + 1] > q
__device__ __forceinline__ int find_sequence(const int* prefix, int batch, int q) {
  int lo = 0, hi = batch - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (prefix[mid + 1] > q) hi = mid; else lo = mid + 1;
  }
  return lo;
}

struct Walk {
  int b, sub, t, g;
};

__device__ __forceinline__ Walk locate(const int* prefix, const PAParams& p, int g) {
  Walk w;
  w.g = g;
  w.b = find_sequence(prefix, p.batch, g / p.subs);
  int n = prefix[w.b + 1] - prefix[w.b];
  int rem = g - p.subs * prefix[w.b];
  w.sub = rem / n;
  w.t = rem - w.sub * n;
  return w;
}

__device__ __forceinline__ void advance(Walk& w, const int* prefix, const PAParams& p, int seg) {
  w.g += seg;
  w.t += seg;
  int n = prefix[w.b + 1] - prefix[w.b];
  if (w.t >= n) {
    w.t = 0;
    if (++w.sub >= p.subs) {
      w.sub = 0;
      do { ++w.b; } while (w.b < p.batch && prefix[w.b + 1] == prefix[w.b]);
    }
  }
}

template <int MT>
__global__ void __launch_bounds__(kThreads, 1)
pa_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const PAParams p) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* bufs = smem;
  uint8_t* q_s = bufs + kNBuf * kBuf;
  int* prefix = reinterpret_cast<int*>(q_s + 16 * MT * 256);
  uint64_t* full = reinterpret_cast<uint64_t*>(prefix + kMaxBatch + 2);
  uint64_t* empty = full + kNBuf;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    for (int i = 0; i < kNBuf; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kConsumers);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  // Ring buffers start as zeros so that rows a partial tile never loads hold
  // finite values (they are multiplied by P == 0).
  {
    uint4 z = make_uint4(0, 0, 0, 0);
    uint4* b4 = reinterpret_cast<uint4*>(bufs);
    for (int i = tid; i < kNBuf * kBuf / 16; i += kThreads) b4[i] = z;
    fence_proxy_async_smem();
  }
  pdl_wait();   // everything above is CTA-local; from here on global memory is read and written
  for (int b = tid; b < p.batch; b += kThreads) prefix[b + 1] = tiles_of(p.context_lens[b], p);
  if (tid == 0) prefix[0] = 0;
  __syncthreads();
  if (warp == 0) {  // inclusive scan of prefix[1..batch]
    int carry = 0;
    for (int base = 1; base <= p.batch; base += 32) {
      int i = base + lane;
      int v = (i <= p.batch) ? prefix[i] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      v += carry;
      if (i <= p.batch) prefix[i] = v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();

  const int total = p.subs * prefix[p.batch];
  const int per = (total + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  if (blockIdx.x == 0) {  // publish the plan for the merge kernel
    if (tid == 0) { p.plan[0] = total; p.plan[1] = per; }
    for (int b = tid; b <= p.batch; b += kThreads) p.plan[2 + b] = prefix[b];
  }
  const int g_lo = static_cast<int>(blockIdx.x) * per;
  const int g_hi = min(total, g_lo + per);
  if (g_lo >= g_hi) return;

  const int tpb = p.blocks_per_tile;

  if (warp == kConsumers) {
    // ------------------------------ producer ------------------------------
    Walk w = locate(prefix, p, g_lo);
    uint32_t q = 0;  // loads issued so far (K and V count separately)
    bool ok = true;
    while (w.g < g_hi && ok) {
      const int n = prefix[w.b + 1] - prefix[w.b];
      const int seg = min(n - w.t, g_hi - w.g);
      const int kvh = w.sub / p.row_groups;
      int ctx = p.context_lens[w.b];
      ctx = min(ctx, p.max_blocks * p.block_size);
      const int nblk_seq = (ctx + p.block_size - 1) / p.block_size;
      const int tiles_per_fetch = 32 / tpb;
      for (int i0 = 0; i0 < seg && ok; i0 += tiles_per_fetch) {
        const int e = (w.t + i0) * tpb + lane;
        int id = 0;
        if (e < nblk_seq) {
          id = p.block_table[static_cast<size_t>(w.b) * p.max_blocks + e];
          if (id < 0 || id >= p.pool_blocks) {
            report_error(p.err, kErrBadBlockId, 1, id);
            id = 0;
          }
        }
        const int ntl = min(seg - i0, tiles_per_fetch);
        for (int i = 0; i < ntl && ok; ++i) {
          const int tile = w.t + i0 + i;
          const int nb = min(tpb, nblk_seq - tile * tpb);
          for (int kv = 0; kv < 2; ++kv) {
            const uint32_t buf = q % kNBuf;
            const uint32_t round = q / kNBuf;
            int good = 1;
            if (lane == 0) good = mbar_wait(&empty[buf], (round & 1u) ^ 1u) ? 1 : 0;
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) {
              report_error(p.err, kErrBarrierTimeout, 10, static_cast<int>(q));
              ok = false;
              break;
            }
            if (lane == 0)
              mbar_arrive_expect_tx(&full[buf], static_cast<uint32_t>(nb * p.block_size * 256));
            for (int j = 0; j < nb; ++j) {
              const int bid = __shfl_sync(0xffffffffu, id, i * tpb + j);
              if (lane == 0) {
                const int y = (bid * p.kv_heads + kvh) * p.block_size;
                uint8_t* dst = bufs + buf * kBuf + j * p.block_size * 128;
                const CUtensorMap* tm = kv ? &tm_v : &tm_k;
                tma_load_2d(dst, tm, 0, y, &full[buf]);
                tma_load_2d(dst + 16384, tm, 64, y, &full[buf]);
              }
            }
            ++q;
          }
        }
      }
      advance(w, prefix, p, seg);
    }
    if (!ok && lane == 0) {
      // give the copies already issued a bounded chance to land before leaving
      uint32_t first = q > kNBuf ? q - kNBuf : 0;
      for (uint32_t i = first; i < q; ++i) mbar_wait(&full[i % kNBuf], (i / kNBuf) & 1u);
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int gid = lane >> 2;  // row within an 8-row group
  const int tig = lane & 3;
  const int mi = lane >> 3;   // ldmatrix: which 8x8 matrix this lane addresses
  const int r8 = lane & 7;
  const uint32_t q_base = smem_u32(q_s);
  const uint32_t bufs_base = smem_u32(bufs);

  Walk w = locate(prefix, p, g_lo);
  uint32_t nt_done = 0;  // tiles consumed so far
  bool dead = false;     // set after a barrier timeout; the warp then only walks
  while (w.g < g_hi) {
    const int n = prefix[w.b + 1] - prefix[w.b];
    const int seg = min(n - w.t, g_hi - w.g);
    const int kvh = w.sub / p.row_groups;
    const int rg = w.sub - kvh * p.row_groups;
    const int ctx = min(p.context_lens[w.b], p.max_blocks * p.block_size);

    // ---- stage the item's query rows (zero padded) in shared memory ----
    named_bar_sync(1, kConsumers * 32);
    for (int c = tid; c < 16 * MT * 16; c += kConsumers * 32) {
      const int r = c >> 4, ch = c & 15;
      const int rr = rg * 16 * MT + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (rr < p.rows_total) {
        const int j = rr / p.group, gh = rr - j * p.group;
        const size_t row = (static_cast<size_t>(w.b) * p.q_len + j) * p.num_heads + kvh * p.group + gh;
        v = *reinterpret_cast<const uint4*>(p.q + row * kD + ch * 8);
      }
      const int sw = (ch & 8) | ((ch ^ r) & 7);
      *reinterpret_cast<uint4*>(q_s + r * 256 + sw * 16) = v;
    }
    named_bar_sync(1, kConsumers * 32);

    int limit[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int rr = rg * 16 * MT + mt * 16 + h * 8 + gid;
        const int j = min(rr / p.group, p.q_len - 1);
        limit[mt][h] = max(0, ctx - p.q_len + j + 1);
      }
    const int min_limit = max(0, ctx - p.q_len + 1);

    float m_run[MT][2], l_run[MT][2];
    float o[MT][16][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      m_run[mt][0] = m_run[mt][1] = -INFINITY;
      l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
    }

    for (int i = 0; i < seg && !dead; ++i) {
      const int tile_base = (w.t + i) * kTile;
      const uint32_t qk = 2 * nt_done, qv = qk + 1;
      const uint32_t buf_k = qk % kNBuf, buf_v = qv % kNBuf;

      if (!mbar_wait_warp(&full[buf_k], (qk / kNBuf) & 1u)) {
        report_error(p.err, kErrBarrierTimeout, 20 + warp, static_cast<int>(nt_done));
        dead = true;
        break;
      }
      // ---- S = Q K^T for this warp's 32 tokens ----
      float s[MT][4][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) s[mt][nt][0] = s[mt][nt][1] = s[mt][nt][2] = s[mt][nt][3] = 0.f;
      const uint32_t kbuf = bufs_base + buf_k * kBuf;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const int row = mt * 16 + (mi & 1) * 8 + r8;
          const int ch = 2 * ks + (mi >> 1);
          ldmatrix_x4(a[mt], q_base + row * 256 + (((ch & 8) | ((ch ^ r8) & 7)) << 4));
        }
#pragma unroll
        for (int ntp = 0; ntp < 2; ++ntp) {
          const int tok = warp * 32 + ntp * 16 + (mi >> 1) * 8 + r8;
          const int ch = 2 * ks + (mi & 1);
          uint32_t kb[4];
          ldmatrix_x4(kb, kbuf + (ch >> 3) * 16384 + tok * 128 + (((ch & 7) ^ r8) << 4));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_bf16_16816(s[mt][2 * ntp], a[mt], kb[0], kb[1]);
            mma_bf16_16816(s[mt][2 * ntp + 1], a[mt], kb[2], kb[3]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[buf_k]);

      // ---- online softmax (per warp, per row) ----
      const bool need_mask = tile_base + kTile > min_limit;
      uint32_t pk[MT][4][2];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float mx = -INFINITY;
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            float x0 = s[mt][nt][2 * h] * p.scale_log2;
            float x1 = s[mt][nt][2 * h + 1] * p.scale_log2;
            if (need_mask) {
              const int tok = tile_base + warp * 32 + nt * 8 + tig * 2;
              if (tok >= limit[mt][h]) x0 = -INFINITY;
              if (tok + 1 >= limit[mt][h]) x1 = -INFINITY;
            }
            s[mt][nt][2 * h] = x0;
            s[mt][nt][2 * h + 1] = x1;
            mx = fmaxf(mx, fmaxf(x0, x1));
          }
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float m_new = fmaxf(m_run[mt][h], mx);
          const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
          const float alpha = fast_exp2(m_run[mt][h] - m_safe);
          m_run[mt][h] = m_new;
          float lsum = 0.f;
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            const float p0 = fast_exp2(s[mt][nt][2 * h] - m_safe);
            const float p1 = fast_exp2(s[mt][nt][2 * h + 1] - m_safe);
            const uint32_t pp = pack_bf16x2(p0, p1);
            pk[mt][nt][h] = pp;
            lsum += bf16_lo_to_float(pp) + bf16_hi_to_float(pp);
          }
          l_run[mt][h] = l_run[mt][h] * alpha + lsum;
#pragma unroll
          for (int i2 = 0; i2 < 16; ++i2) {
            o[mt][i2][2 * h] *= alpha;
            o[mt][i2][2 * h + 1] *= alpha;
          }
        }

      if (!mbar_wait_warp(&full[buf_v], (qv / kNBuf) & 1u)) {
        report_error(p.err, kErrBarrierTimeout, 30 + warp, static_cast<int>(nt_done));
        dead = true;
        break;
      }
      uint8_t* vbuf_g = bufs + buf_v * kBuf;
      const bool ragged = tile_base + kTile > ctx;
      if (ragged) {
        // Rows past the end of the sequence may hold anything (unwritten pool
        // memory); P is 0 there but 0 * NaN is NaN, so clear this warp's slice.
        const int first_bad = max(0, ctx - tile_base - warp * 32);
        for (int c = first_bad * 16 + lane; c < 32 * 16; c += 32) {
          const int tok = warp * 32 + (c >> 4), ch = c & 15;
          *reinterpret_cast<uint4*>(vbuf_g + (ch >> 3) * 16384 + tok * 128 + (ch & 7) * 16) =
              make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }
      // ---- O += P V ----
      const uint32_t vbuf = bufs_base + buf_v * kBuf;
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
        uint32_t a[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          a[mt][0] = pk[mt][2 * kt][0];
          a[mt][1] = pk[mt][2 * kt][1];
          a[mt][2] = pk[mt][2 * kt + 1][0];
          a[mt][3] = pk[mt][2 * kt + 1][1];
        }
        const int tok = warp * 32 + kt * 16 + (mi & 1) * 8 + r8;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int ch = 2 * j + (mi >> 1);
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, vbuf + (ch >> 3) * 16384 + tok * 128 + (((ch & 7) ^ r8) << 4));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_bf16_16816(o[mt][2 * j], a[mt], vb[0], vb[1]);
            mma_bf16_16816(o[mt][2 * j + 1], a[mt], vb[2], vb[3]);
          }
        }
      }
      if (ragged) fence_proxy_async_smem();  // generic writes above precede the next TMA write
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[buf_v]);
      ++nt_done;
    }
    if (dead) {  // keep walking so the named barriers above stay matched
      advance(w, prefix, p, seg);
      continue;
    }

    // ---- write this warp's partial (m, l, O) for the segment ----
    const int item = w.b * p.subs + w.sub;
    const size_t slot = static_cast<size_t>(item) + blockIdx.x;
    const size_t base = (slot * kConsumers + warp) * p.rows_per_item;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = mt * 16 + h * 8 + gid;
        float l = l_run[mt][h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (rg * 16 * MT + r >= p.rows_total) continue;
        if (tig == 0) {
          p.part_ml[(base + r) * 2] = m_run[mt][h];
          p.part_ml[(base + r) * 2 + 1] = l;
        }
        float* dst = p.part_o + (base + r) * kD + tig * 2;
#pragma unroll
        for (int i2 = 0; i2 < 16; ++i2)
          *reinterpret_cast<float2*>(dst + i2 * 8) = make_float2(o[mt][i2][2 * h], o[mt][i2][2 * h + 1]);
      }
    advance(w, prefix, p, seg);
  }
}

// One warp per (item, row): combine the partials of all covering CTAs and warps.
__global__ void __launch_bounds__(128) pa_merge_kernel(const PAParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int item = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.y * 4 + warp;
  const int b = item / p.subs, sub = item - b * p.subs;
  const int kvh = sub / p.row_groups, rg = sub - kvh * p.row_groups;
  const int rr = rg * p.rows_per_item + r;
  if (r >= p.rows_per_item || rr >= p.rows_total) return;
  const int per = p.plan[1];
  const int* prefix = p.plan + 2;
  const int n = prefix[b + 1] - prefix[b];
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l_tot = 0.f;
  if (n > 0) {
    const int t0 = p.subs * prefix[b] + sub * n;
    const int c_first = t0 / per, c_last = (t0 + n - 1) / per;
    float m_max = -INFINITY;
    for (int c = c_first; c <= c_last; ++c)
      for (int w = 0; w < kConsumers; ++w) {
        const size_t base = ((static_cast<size_t>(item) + c) * kConsumers + w) * p.rows_per_item + r;
        m_max = fmaxf(m_max, p.part_ml[base * 2]);
      }
    if (m_max > -INFINITY) {
      for (int c = c_first; c <= c_last; ++c)
        for (int w = 0; w < kConsumers; ++w) {
          const size_t base = ((static_cast<size_t>(item) + c) * kConsumers + w) * p.rows_per_item + r;
          const float mw = p.part_ml[base * 2];
          if (mw == -INFINITY) continue;
          const float wgt = fast_exp2(mw - m_max);
          l_tot += wgt * p.part_ml[base * 2 + 1];
          const float4 v = *reinterpret_cast<const float4*>(p.part_o + base * kD + lane * 4);
          acc.x += wgt * v.x; acc.y += wgt * v.y; acc.z += wgt * v.z; acc.w += wgt * v.w;
        }
    }
  }
  const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
  acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
  const int j = rr / p.group, gh = rr - j * p.group;
  const size_t row = (static_cast<size_t>(b) * p.q_len + j) * p.num_heads + kvh * p.group + gh;
  if (p.out_fp32) {
    *reinterpret_cast<float4*>(static_cast<float*>(p.out) + row * kD + lane * 4) = acc;
  } else {
    uint2 pk2 = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + row * kD + lane * 4) = pk2;
  }
}

// ---------------------------------------------------------------------------
// Generic kernel for geometries the tensor-core path does not take (head_dim
// other than 128, block sizes that do not divide 128).  One CTA per query row,
// one KV block at a time in exactly the reference's order: S * scale, mask,
// block max clamped at -1e30, P = exp(S - m) rounded to bf16, l = sum(P),
// O_blk = P V, fp32 merge (04_paged_attention.py:473-541).
// ---------------------------------------------------------------------------
constexpr int kGenThreads = 128;
constexpr int kGenMaxD = 256;
constexpr int kGenMaxBlock = 1024;

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
  for (int i = 1; i < kGenThreads / 32; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
  return r;
}

__global__ void __launch_bounds__(kGenThreads)
pa_generic_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                  const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table,
                  const int* __restrict__ context_lens, void* out, int out_fp32, int num_heads,
                  int kv_heads, int q_len, int head_dim, int block_size, int max_blocks,
                  int pool_blocks, float scale, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float q_f[kGenMaxD];
  __shared__ float s_f[kGenMaxBlock];
  __shared__ float red[kGenThreads / 32];
  const int row = blockIdx.x;
  const int h = row % num_heads;
  const int j = (row / num_heads) % q_len;
  const int b = row / (num_heads * q_len);
  const int kvh = h / (num_heads / kv_heads);
  int ctx = min(context_lens[b], max_blocks * block_size);
  const int limit = ctx > 0 ? max(0, ctx - q_len + j + 1) : 0;
  for (int d = threadIdx.x; d < head_dim; d += kGenThreads)
    q_f[d] = __bfloat162float(q[static_cast<size_t>(row) * head_dim + d]);
  float o_run[kGenMaxD / kGenThreads] = {0.f, 0.f};
  float m_run = 0.f, l_run = 0.f;
  __syncthreads();
  const int n_blk = (limit + block_size - 1) / block_size;
  for (int bn = 0; bn < n_blk; ++bn) {
    int id = block_table[static_cast<size_t>(b) * max_blocks + bn];
    if (id < 0 || id >= pool_blocks) {
      if (threadIdx.x == 0) report_error(err, kErrBadBlockId, 2, id);
      id = 0;
    }
    const int valid = min(block_size, limit - bn * block_size);
    const size_t base = (static_cast<size_t>(id) * kv_heads + kvh) * block_size;
    float mx = -INFINITY;
    for (int t = threadIdx.x; t < block_size; t += kGenThreads) {
      float sv = -INFINITY;
      if (t < valid) {
        const __nv_bfloat16* kr = kc + (base + t) * head_dim;
        float acc = 0.f;
        for (int d = 0; d < head_dim; ++d) acc += q_f[d] * __bfloat162float(kr[d]);
        sv = acc * scale;
      }
      s_f[t] = sv;
      mx = fmaxf(mx, sv);
    }
    const float m_blk = fmaxf(block_reduce(mx, red, true), -1e30f);
    float ls = 0.f;
    for (int t = threadIdx.x; t < block_size; t += kGenThreads) {
      float pv = 0.f;
      if (t < valid) pv = __bfloat162float(__float2bfloat16_rn(expf(s_f[t] - m_blk)));
      s_f[t] = pv;
      ls += pv;
    }
    const float l_blk = block_reduce(ls, red, false);  // also orders the s_f writes
    float alpha = 0.f, beta = 1.f, m_new = m_blk;
    if (bn > 0) {
      m_new = fmaxf(m_run, m_blk);
      alpha = expf(m_run - m_new);
      beta = expf(m_blk - m_new);
    }
#pragma unroll
    for (int k = 0; k < kGenMaxD / kGenThreads; ++k) {
      const int d = threadIdx.x + k * kGenThreads;
      if (d < head_dim) {
        float acc = 0.f;
        for (int t = 0; t < valid; ++t) acc += s_f[t] * __bfloat162float(vc[(base + t) * head_dim + d]);
        o_run[k] = bn == 0 ? acc : alpha * o_run[k] + beta * acc;
      }
    }
    l_run = bn == 0 ? l_blk : alpha * l_run + beta * l_blk;
    m_run = m_new;
    __syncthreads();
  }
#pragma unroll
  for (int k = 0; k < kGenMaxD / kGenThreads; ++k) {
    const int d = threadIdx.x + k * kGenThreads;
    if (d < head_dim) {
      const float v = l_run > 0.f ? o_run[k] / l_run : 0.f;
      if (out_fp32) static_cast<float*>(out)[static_cast<size_t>(row) * head_dim + d] = v;
      else static_cast<__nv_bfloat16*>(out)[static_cast<size_t>(row) * head_dim + d] = __float2bfloat16_rn(v);
    }
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct ScratchLayout {
  size_t err_off, plan_off, ml_off, o_off, total;
  int rows_per_item, row_groups, subs, slots;
};

ScratchLayout scratch_layout(int batch, int num_heads, int kv_heads, int q_len, int grid) {
  ScratchLayout s;
  const int group = num_heads / (kv_heads > 0 ? kv_heads : 1);
  const int rows_total = q_len * group;
  s.rows_per_item = rows_total <= 16 ? 16 : 32;
  s.row_groups = (rows_total + s.rows_per_item - 1) / s.rows_per_item;
  s.subs = kv_heads * s.row_groups;
  s.slots = batch * s.subs + grid;
  s.err_off = 0;
  s.plan_off = 256;
  s.ml_off = align_up(s.plan_off + sizeof(int) * (batch + 3), 256);
  s.o_off = align_up(s.ml_off + sizeof(float) * 2 * s.slots * kConsumers * s.rows_per_item, 256);
  s.total = s.o_off + sizeof(float) * kD * static_cast<size_t>(s.slots) * kConsumers * s.rows_per_item;
  return s;
}

constexpr size_t smem_bytes(int mt) {
  return 1024 + kNBuf * kBuf + 16 * mt * 256 + sizeof(int) * (kMaxBatch + 2) + 16 * kNBuf + 64;
}

}  // namespace

bool pa_fast_path_ok(int head_dim, int block_size) {
  return head_dim == kD && (block_size == 16 || block_size == 32 || block_size == 64 || block_size == 128);
}

size_t pa_scratch_bytes(int batch, int num_heads, int kv_heads, int q_len) {
  return scratch_layout(batch, num_heads, kv_heads, q_len, sm_count()).total;
}

int pa_launch(const void* q, const void* kc, const void* vc, const int32_t* block_table,
              const int32_t* context_lens, void* out, int out_fp32, int batch, int num_heads,
              int kv_heads, int head_dim, int block_size, int max_blocks, int64_t pool_blocks,
              int q_len, float scale, void* scratch, size_t scratch_bytes, cudaStream_t stream) {
  PTO_REQUIRE(batch >= 0 && num_heads > 0 && kv_heads > 0 && q_len > 0, "paged_attention: bad geometry");
  PTO_REQUIRE(num_heads % kv_heads == 0, "paged_attention: num_heads must be a multiple of kv_heads");
  PTO_REQUIRE(block_size > 0 && max_blocks > 0 && pool_blocks > 0, "paged_attention: bad block geometry");
  PTO_REQUIRE(scratch != nullptr && scratch_bytes >= 256, "paged_attention: scratch buffer required");
  if (batch == 0) return kOk;
  int* err = static_cast<int*>(scratch);
  const int64_t pool_rows = pool_blocks * kv_heads * block_size;
  PTO_REQUIRE(pool_rows < (1ll << 31), "paged_attention: pool has too many rows");

  if (!pa_fast_path_ok(head_dim, block_size)) {
    PTO_REQUIRE(head_dim <= kGenMaxD && block_size <= kGenMaxBlock,
                "paged_attention: head_dim <= 256 and block_size <= 1024 required");
    launch_kernel(pa_generic_kernel, dim3(batch * q_len * num_heads), dim3(kGenThreads), 0, stream, 
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(kc),
        static_cast<const __nv_bfloat16*>(vc), block_table, context_lens, out, out_fp32, num_heads,
        kv_heads, q_len, head_dim, block_size, max_blocks, static_cast<int>(pool_blocks), scale, err);
    return check_cuda(cudaGetLastError(), "pa_generic_kernel launch");
  }

  PTO_REQUIRE(batch <= kMaxBatch, "paged_attention: at most 4096 sequences per call");
  const int grid = sm_count();
  const ScratchLayout lay = scratch_layout(batch, num_heads, kv_heads, q_len, grid);
  PTO_REQUIRE(scratch_bytes >= lay.total, "paged_attention: scratch buffer too small");
  PTO_REQUIRE((reinterpret_cast<uintptr_t>(kc) & 15) == 0 && (reinterpret_cast<uintptr_t>(vc) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
              "paged_attention: tensors must be 16-byte aligned");

  CUtensorMap tm_k, tm_v;
  int st = make_tensor_map_2d(&tm_k, kc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, pool_rows, kD, kD * 2, 64,
                              block_size, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_v, vc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, pool_rows, kD, kD * 2, 64,
                          block_size, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;

  PAParams p;
  uint8_t* sb = static_cast<uint8_t*>(scratch);
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.block_table = block_table;
  p.context_lens = context_lens;
  p.err = err;
  p.plan = reinterpret_cast<int*>(sb + lay.plan_off);
  p.part_ml = reinterpret_cast<float*>(sb + lay.ml_off);
  p.part_o = reinterpret_cast<float*>(sb + lay.o_off);
  p.out = out;
  p.out_fp32 = out_fp32;
  p.batch = batch;
  p.num_heads = num_heads;
  p.kv_heads = kv_heads;
  p.group = num_heads / kv_heads;
  p.q_len = q_len;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.blocks_per_tile = kTile / block_size;
  p.rows_total = q_len * p.group;
  p.rows_per_item = lay.rows_per_item;
  p.row_groups = lay.row_groups;
  p.subs = lay.subs;
  p.pool_blocks = static_cast<int>(pool_blocks);
  p.grid_main = grid;
  p.scale_log2 = scale * kLog2e;

  const int mt = lay.rows_per_item / 16;
  const size_t smem = smem_bytes(mt);
  if (mt == 1) {
    PTO_CUDA(cudaFuncSetAttribute(pa_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_kernel(pa_decode_kernel<1>, dim3(grid), dim3(kThreads), smem, stream, tm_k, tm_v, p);
  } else {
    PTO_CUDA(cudaFuncSetAttribute(pa_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_kernel(pa_decode_kernel<2>, dim3(grid), dim3(kThreads), smem, stream, tm_k, tm_v, p);
  }
  PTO_CUDA(cudaGetLastError());
  dim3 mgrid(batch * lay.subs, (lay.rows_per_item + 3) / 4);
  launch_kernel(pa_merge_kernel, dim3(mgrid), dim3(128), 0, stream, p);
  return check_cuda(cudaGetLastError(), "pa_merge_kernel launch");
}

// ---------------------------------------------------------------------------
// Launch without any allocation.
//
// Some callers may not allocate device memory at the point where they launch: a serving
// loop that has handed the whole HBM budget to its KV-cache pool up front, a plugin
// running inside another framework's memory arena, a real-time control path where
// cudaMalloc's implicit device synchronisation is not acceptable.  For them the per-warp
// partial (m, l, O) rows and the plan live in the fixed array below instead of a buffer
// the caller or the worker allocates.  The array is part of the loaded module: every GPU
// that loads this library holds kStaticScratchBytes of it until the process exits.
//
// In host code the name `g_pa_static_scratch` is only a handle of the symbol, not a
// device address; the address is looked up once per device with cudaGetSymbolAddress
// (with that device current) and that pointer is what the kernels receive.
// ---------------------------------------------------------------------------
namespace {
constexpr size_t kStaticScratchBytes = 32u << 20;
static __device__ __align__(256) unsigned char g_pa_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_static_ptr[kMaxDevices] = {nullptr};
std::mutex g_static_mu;

int static_scratch_ptr(void** out) {
  int dev = -1;
  PTO_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(kInvalidArgument, "paged_attention_static: device index out of range");
  std::lock_guard<std::mutex> g(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    PTO_CUDA(cudaGetSymbolAddress(&ptr, g_pa_static_scratch));
    if (ptr == nullptr) return fail(kCudaError, "paged_attention_static: cudaGetSymbolAddress returned NULL");
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return kOk;
}
}  // namespace

size_t pa_static_scratch_capacity() { return kStaticScratchBytes; }

int pa_launch_static(const void* q, const void* kc, const void* vc, const int32_t* block_table,
                     const int32_t* context_lens, void* out, int out_fp32, int batch, int num_heads,
                     int kv_heads, int head_dim, int block_size, int max_blocks, int64_t pool_blocks,
                     int q_len, float scale, int32_t* status_dev, cudaStream_t stream) {
  PTO_REQUIRE(batch >= 0 && num_heads > 0 && kv_heads > 0 && q_len > 0 && num_heads % kv_heads == 0,
              "paged_attention_static: bad geometry");
  const size_t need = pa_scratch_bytes(batch, num_heads, kv_heads, q_len);
  if (need > kStaticScratchBytes) {
    char buf[200];
    snprintf(buf, sizeof buf,
             "paged_attention_static: this geometry needs %zu bytes of scratch, the built-in array holds %zu; "
             "use pto_paged_attention with a caller-provided buffer",
             need, kStaticScratchBytes);
    return fail(kInvalidArgument, buf);
  }
  void* scratch = nullptr;
  int st = static_scratch_ptr(&scratch);
  if (st != kOk) return st;
  // The array keeps whatever the previous call left.  Only the error word has to start
  // at zero; plan and partial rows are fully rewritten by every launch before they are read.
  PTO_CUDA(cudaMemsetAsync(scratch, 0, 64, stream));
  st = pa_launch(q, kc, vc, block_table, context_lens, out, out_fp32, batch, num_heads, kv_heads, head_dim,
                 block_size, max_blocks, pool_blocks, q_len, scale, scratch, kStaticScratchBytes, stream);
  if (st != kOk) return st;
  if (status_dev != nullptr)
    PTO_CUDA(cudaMemcpyAsync(status_dev, scratch, 4 * sizeof(int32_t), cudaMemcpyDeviceToDevice, stream));
  return kOk;
}


}  // namespace pto
