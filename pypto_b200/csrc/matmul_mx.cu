// MX block-scaled FP8 matmul on the hardware block-scaling path of the 5th-generation tensor cores.
//
//   out[m, n] = (acc_in[m, n] +) sum_k a[m, k] * 2^(sa[m, k/32] - 127) * b[k, n] * 2^(sb[k/32, n] - 127)
//
// It stands where the reference lowers tile.matmul_mx / tile.matmul_mx_acc to the MX cube
// instruction of its 950 target (src/ir/op/tile_ops/matmul_mx.cpp:321-345; numerics
// tests/st/runtime/ops/test_matmul_mx.py:119-131: dequantise per 32-wide K group, exact product).
// The same format is native here: `tcgen05.mma.kind::mxf8f6f4.block_scale` multiplies every 32-wide
// K group by one E8M0 scale per operand row, read from tensor memory, so no scale arithmetic runs on
// the CUDA cores.
//
// Operands: a e4m3 [m, k] and b_t e4m3 [n, k], both K-major, brought in by TMA with the 128-byte
// swizzle, 128 K bytes per pipeline stage (four MMAs of K = 32).  Scales: one byte per (row, K group).
// The tensor core wants the four scale bytes of a row for one stage in one 32-bit tensor-memory cell,
// rows 32 apart in neighbouring columns:
//     chunk byte offset of (row r, group g of the stage) = (r % 32) * 16 + (r / 32) * 4 + g
// for every 128 rows (512 bytes).  Scale-loader warps build those chunks in shared memory from the
// caller's layout (row-major, or the reference's MX_A_ZZ / MX_B_NN physical orders,
// test_matmul_mx.py:38-101); the MMA thread moves a chunk to tensor memory with
// `tcgen05.cp.32x128b.warpx4` and selects the byte with the scale-id field of the instruction.
//
// One CTA (small and medium problems) = warp 0 TMA producer, warp 1 MMA issuer (owns tensor memory), warps 2-5
// epilogue (one TMEM lane quarter each), warps 6-13 scale loaders (K blocks in turn, into a ring of scale blocks that
// runs ahead of the operand stages).  Tiles of 128 x bn outputs (bn = 128 with two accumulator buffers, or 256 with
// one) are taken by persistent CTAs in groups of tile rows, so that what the CTAs read at one time stays in L2.
//
// Large problems run on PAIRS of SMs (matmul_mx_pair_kernel: a cluster of two CTAs, tcgen05 .cta_group::2): a pair
// shares one 256 x 224 tile, each CTA brings its own 128 rows of a and its own half (112 rows) of the b_t tile, so a
// CTA's shared memory feeds the tensor core 30 KB per K block instead of 48 KB, and two accumulators (2 x 224
// columns) plus the scale columns still fit the 512 columns of tensor memory.  The pair has no loader warps: a small
// kernel first writes all scale blocks in the tensor core's order to scratch memory (1/32 of the operands' bytes) and
// the producer fetches them by TMA with the operands, each CTA the block of its own 128 rows and the blocks of ALL
// 224 columns.  (With loader warps in each CTA the pair ran at 1570-1800 TFLOP/s, with the blocks by TMA at 2230-2290:
// the loaders' global loads take about 2200 cycles under the operand traffic, and their stores and arrivals competed
// with the overlapped epilogue.)  The leader CTA issues the copies to tensor memory and the MMAs for both.
// Barriers: full[s] lives in the leader (its producer's expect_tx for both CTAs' bytes); empty[s] and tmem_full[b]
// are signalled in both CTAs by multicast commits; tmem_empty[b] lives in the leader (eight epilogue warps).
// No load is multicast.  Every wait is bounded.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "pair.cuh"

namespace pto {
namespace {

constexpr int kMxScaleWarps = 8;                      // a power of two
constexpr int kMxThreads = 192 + 32 * kMxScaleWarps;
constexpr int kMxPairThreads = 192;                   // a pair has no loader warps: its scale blocks come by TMA
constexpr int kMxMaxStages = 8;
constexpr int kMxBK = 128;           // K bytes per stage = 4 scale groups
constexpr int kMxSfSlots = 16;       // ring of scale blocks, one per K block; at least kMxScaleWarps

struct MxParams {
  int m, n, k;
  int m_tiles, n_tiles, kblocks, kgroups;
  int bn, nbuf, stages;
  int group_m;                     // tile rows per raster group
  const uint8_t* a_scale;
  const uint8_t* b_scale;
  int a_layout, b_layout;
  const float* acc_in;
  float* out;
  int* err;
};

// Address of the E8M0 code of (row, K group) of the left operand.  The loaders read every code with an
// unconditional load from a clamped position and replace codes outside the matrix by 127 (= 1.0) afterwards:
// a load behind a bounds branch cannot be issued ahead of the branch, and a K block needs 36 of them per lane.
__device__ __forceinline__ const uint8_t* a_scale_ptr(const MxParams& p, int row, int g) {
  row = min(row, p.m - 1);
  g = min(g, p.kgroups - 1);
  if (p.a_layout == PTO_MX_SCALE_A_ZZ)   // [m/16][kg/2][16][2]
    return p.a_scale + (static_cast<size_t>(row >> 4) * (p.kgroups >> 1) + (g >> 1)) * 32 + (row & 15) * 2 + (g & 1);
  return p.a_scale + static_cast<size_t>(row) * p.kgroups + g;
}
// Address of the E8M0 code of (K group, column) of the right operand.
__device__ __forceinline__ const uint8_t* b_scale_ptr(const MxParams& p, int col, int g) {
  col = min(col, p.n - 1);
  g = min(g, p.kgroups - 1);
  if (p.b_layout == PTO_MX_SCALE_B_NN)   // [n/16][kg/2][16][2]
    return p.b_scale + (static_cast<size_t>(col >> 4) * (p.kgroups >> 1) + (g >> 1)) * 32 + (col & 15) * 2 + (g & 1);
  return p.b_scale + static_cast<size_t>(g) * p.n + col;
}

// Shared-memory descriptor of one 512-byte scale chunk for tcgen05.cp: 32 rows of 16 bytes, no swizzle,
// 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;   // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;          // descriptor version (sm_100)
  return d;
}

template <bool PAIR>
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t desc) {
  if constexpr (PAIR)   // each CTA of the pair copies from its own shared memory to its own tensor memory
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
  else
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

// Block-scaled instruction descriptor: e4m3 x e4m3, K-major, E8M0 scales, M x N, scale byte ids.
__device__ __forceinline__ uint32_t mx_idesc(uint32_t m, uint32_t n, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (a_sf_id << 29);
}

template <bool PAIR>
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate, uint32_t tsfa, uint32_t tsfb) {
  if constexpr (PAIR)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
        : "memory");
}

// One CTA's part.  PAIR: the CTA is one of a cluster of two; `rank` 0 is the leader.
template <bool PAIR>
__device__ __forceinline__ void matmul_mx_body(const CUtensorMap* tm_a, const CUtensorMap* tm_b, const CUtensorMap* tm_sfa,
                                               const CUtensorMap* tm_sfb, const MxParams& p) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint32_t rank = 0;
  if constexpr (PAIR) rank = cluster_ctarank();
  const int unit0 = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);       // first tile of this CTA (pair)
  const int unit_step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  constexpr int kTileM = PAIR ? 256 : 128;
  const int my_row0 = static_cast<int>(rank) * 128;                  // this CTA's rows within the tile
  // b_t rows this CTA loads per K block: the whole tile width, or its half of it
  const uint32_t b_rows = PAIR ? static_cast<uint32_t>(p.bn) / 2 : static_cast<uint32_t>(p.bn);
  const uint32_t a_bytes = 128 * kMxBK, b_bytes = b_rows * kMxBK;
  const uint32_t sfb_chunks = (static_cast<uint32_t>(p.bn) + 127) / 128;
  const uint32_t sf_bytes = 512 * (1 + sfb_chunks);        // one K block's scale chunks
  // a multiple of 1024, so that stages stay aligned for the swizzle; a pair's stages end with the K block's scale block
  const uint32_t stage_bytes = a_bytes + b_bytes + (PAIR ? 1024 * ((sf_bytes + 1023) / 1024) : 0);
  // operand stages, then (one CTA) the ring of scale blocks, then the barriers
  uint8_t* sf_ring = smem + static_cast<size_t>(p.stages) * stage_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(sf_ring + (PAIR ? 0 : kMxSfSlots * sf_bytes));
  uint64_t* empty = full + kMxMaxStages;
  uint64_t* tmem_full = empty + kMxMaxStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* drain = tmem_empty + 2;
  uint64_t* sf_full = drain + 1;
  uint64_t* sf_empty = sf_full + kMxSfSlots;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_empty + kMxSfSlots);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t tmem_cols = 512;
  // accumulators in columns [0, nbuf * bn); two sets of scale columns after them (K blocks alternate)
  const uint32_t sf_col0 = static_cast<uint32_t>(p.nbuf * p.bn);
  const uint32_t sf_set = 4 + 4 * sfb_chunks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(&full[i], 1);    // the TMA producer's expect_tx arrival
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < kMxSfSlots; ++i) {
      mbar_init(&sf_full[i], PAIR ? 2 : 1);   // one scale-loader warp (of each CTA)
      mbar_init(&sf_empty[i], 1);             // the producer warp, once the K block's MMAs have completed
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], PAIR ? 8 : 4);
    }
    mbar_init(drain, 1);
    fence_barrier_init();
    tma_prefetch_desc(tm_a);
    tma_prefetch_desc(tm_b);
  }
  if (warp == 1) {
    if constexpr (PAIR) tmem_alloc_pair(tmem_slot, tmem_cols);   // the same warp in each CTA of the pair, together
    else tmem_alloc(tmem_slot, tmem_cols);
  }
  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all();   // both CTAs' barriers exist before anything is signalled across the pair
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  const int tiles = p.m_tiles * p.n_tiles;

  // Producer and issuer are one-thread jobs whose instruction streams sit on the critical path of every K block: the
  // whole warp walks the loop and waits (warp-uniform code keeps descriptors in uniform registers), one elected lane
  // issues, and stages and barrier phases are carried along instead of divided out.
  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    uint32_t it = 0, s = 0, ph = 0;
    bool ok = true;
    for (int tile = unit0; tile < tiles && ok; tile += unit_step) {
      int mt, nt;
      grouped_tile_coords(tile, p.group_m, p.m_tiles, p.n_tiles, mt, nt);
      for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
        if (!__all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u))) {
          if (lane == 0) report_error(p.err, kErrBarrierTimeout, 70, static_cast<int>(it));
          ok = false;
          break;
        }
        if (elect_one()) {
          // the K block that used this stage before has completed (its copies of the scales to tensor memory too):
          // its slot of the scale ring is free.  Completions are seen in order, one per K block.
          if (!PAIR && it >= static_cast<uint32_t>(p.stages)) mbar_arrive(&sf_empty[(it - p.stages) % kMxSfSlots]);
          uint8_t* st = smem + static_cast<size_t>(s) * stage_bytes;
          if constexpr (PAIR) {
            // both CTAs' bytes are counted by the leader's barrier, which its producer arms for the two of them
            const uint32_t leader_full = mapa_u32(smem_u32(&full[s]), 0);
            if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * (a_bytes + b_bytes + sf_bytes));
            tma_load_2d_pair(st, tm_a, kb * kMxBK, mt * kTileM + my_row0, leader_full);
            tma_load_2d_pair(st + a_bytes, tm_b, kb * kMxBK, nt * p.bn + static_cast<int>(rank * b_rows), leader_full);
            // the scale blocks, packed beforehand in the tensor core's order: this CTA's 128 rows, and all columns
            tma_load_2d_pair(st + a_bytes + b_bytes, tm_sfa, 0, (mt * 2 + static_cast<int>(rank)) * p.kblocks + kb, leader_full);
            tma_load_2d_pair(st + a_bytes + b_bytes + 512, tm_sfb, 0, nt * p.kblocks + kb, leader_full);
          } else {
            mbar_arrive_expect_tx(&full[s], a_bytes + b_bytes);
            tma_load_2d(st, tm_a, kb * kMxBK, mt * 128, &full[s]);          // past m or k the box is zero filled
            for (uint32_t c = 0; c < sfb_chunks; ++c)
              tma_load_2d(st + a_bytes + c * (128 * kMxBK), tm_b, kb * kMxBK, nt * p.bn + c * 128, &full[s]);
          }
        }
        __syncwarp();
        if (++s == static_cast<uint32_t>(p.stages)) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (the leader's, for a pair) -------------------------------
    uint32_t it = 0, s = 0, ph = 0;
    uint32_t ab = 0, ab_ph = 1;          // accumulator buffer and the phase of `tmem_empty` to wait for (first use: free)
    bool ok = true;
    const uint32_t idesc0 = mx_idesc(kTileM, static_cast<uint32_t>(p.bn), 0, 0), idesc1 = mx_idesc(kTileM, static_cast<uint32_t>(p.bn), 1, 1);
    const uint32_t idesc2 = mx_idesc(kTileM, static_cast<uint32_t>(p.bn), 2, 2), idesc3 = mx_idesc(kTileM, static_cast<uint32_t>(p.bn), 3, 3);
    const uint32_t smem0 = smem_u32(smem), sf_ring0 = smem_u32(sf_ring);
    uint32_t slot = 0, sph = 0;          // slot of the scale ring and its phase
    for (int tile = rank == 0 ? unit0 : tiles; tile < tiles && ok; tile += unit_step) {
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_empty[ab], ab_ph))) {
        if (lane == 0) report_error(p.err, kErrBarrierTimeout, 71, static_cast<int>(it));
        break;
      }
      tc_fence_after_sync();
      const uint32_t d0 = tmem_base + ab * p.bn;
      for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
        if (!__all_sync(0xffffffffu, mbar_wait(&full[s], ph))) {
          if (lane == 0) report_error(p.err, kErrBarrierTimeout, 72, static_cast<int>(it));
          ok = false;
          break;
        }
        if (!PAIR && !__all_sync(0xffffffffu, mbar_wait(&sf_full[slot], sph))) {
          if (lane == 0) report_error(p.err, kErrBarrierTimeout, 76, static_cast<int>(it));
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (elect_one()) {
          const uint32_t a_addr = smem0 + s * stage_bytes;
          const uint32_t b_addr = a_addr + a_bytes;
          const uint32_t sf_addr = PAIR ? b_addr + b_bytes : sf_ring0 + slot * sf_bytes;
          const uint32_t tsfa = tmem_base + sf_col0 + (it & 1u) * sf_set;
          const uint32_t tsfb = tsfa + 4;
          tmem_cp_32x128b_warpx4<PAIR>(tsfa, sf_desc(sf_addr));
          for (uint32_t c = 0; c < sfb_chunks; ++c) tmem_cp_32x128b_warpx4<PAIR>(tsfb + 4 * c, sf_desc(sf_addr + 512 * (1 + c)));
          const uint64_t ad = umma_desc_sw128(a_addr), bd = umma_desc_sw128(b_addr);   // + 2 per 32 bytes of K
          umma_mxf8<PAIR>(d0, ad, bd, idesc0, kb > 0 ? 1u : 0u, tsfa, tsfb);
          umma_mxf8<PAIR>(d0, ad + 2, bd + 2, idesc1, 1u, tsfa, tsfb);
          umma_mxf8<PAIR>(d0, ad + 4, bd + 4, idesc2, 1u, tsfa, tsfb);
          umma_mxf8<PAIR>(d0, ad + 6, bd + 6, idesc3, 1u, tsfa, tsfb);
          if constexpr (PAIR) umma_commit_pair(&empty[s]);   // frees the stage in both CTAs
          else umma_commit(&empty[s]);
        }
        __syncwarp();
        if (++s == static_cast<uint32_t>(p.stages)) {
          s = 0;
          ph ^= 1u;
        }
        if (++slot == kMxSfSlots) {
          slot = 0;
          sph ^= 1u;
        }
      }
      if (ok && elect_one()) {
        if constexpr (PAIR) umma_commit_pair(&tmem_full[ab]);
        else umma_commit(&tmem_full[ab]);
      }
      __syncwarp();
      if (p.nbuf == 2) {
        ab ^= 1u;
        if (ab == 0) ab_ph ^= 1u;
      } else {
        ab_ph ^= 1u;
      }
    }
    if (rank == 0 && elect_one()) {
      // tensor memory is released only after every MMA has completed
      if constexpr (PAIR)
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(drain)) : "memory");
      else
        umma_commit(drain);
      if (!mbar_wait(drain, 0)) report_error(p.err, kErrBarrierTimeout, 74, static_cast<int>(it));
    }
    __syncwarp();
  } else if (warp < 6) {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;   // TMEM lane quarter this warp may read
    uint32_t ui = 0;
    uint32_t leader_empty0 = 0, leader_empty1 = 0;
    if constexpr (PAIR) {
      leader_empty0 = mapa_u32(smem_u32(&tmem_empty[0]), 0);
      leader_empty1 = mapa_u32(smem_u32(&tmem_empty[1]), 0);
    }
    for (int tile = unit0; tile < tiles; tile += unit_step, ++ui) {
      int mt, nt;
      grouped_tile_coords(tile, p.group_m, p.m_tiles, p.n_tiles, mt, nt);
      const uint32_t ab = ui % p.nbuf;
      if (!mbar_wait_warp(&tmem_full[ab], (ui / p.nbuf) & 1u)) {
        report_error(p.err, kErrBarrierTimeout, 73, static_cast<int>(ui));
        break;
      }
      tc_fence_after_sync();
      const int row = mt * kTileM + my_row0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * p.bn;
      for (int c0 = 0; c0 < p.bn; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c0, v);
        tmem_ld_wait();
        const int col0 = nt * p.bn + c0;
        if (row < p.m && col0 < p.n) {
          const size_t o = static_cast<size_t>(row) * p.n + col0;
          const bool vec = col0 + 32 <= p.n && (p.n & 3) == 0;
          if (p.acc_in != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.n) v[j] = __float_as_uint(__uint_as_float(v[j]) + p.acc_in[o + j]);
          }
          if (vec) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<uint4*>(p.out + o + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.n) p.out[o + j] = __uint_as_float(v[j]);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(ab ? leader_empty1 : leader_empty0);   // the leader's barrier, from either CTA
        else mbar_arrive(&tmem_empty[ab]);
      }
    }
  } else if constexpr (!PAIR) {
    // ------------------------------ scale loaders (one CTA) ------------------------------
    // Per stage: 128 left-operand rows and bn right-operand columns, four scale bytes each, packed into one
    // 32-bit word at its place in the 512-byte chunk of its 128 rows.  The blocks go to a ring of their own, with more
    // slots than the operands have stages: the loader warps take K blocks in turn and run up to a ring ahead of the
    // MMAs, which hides the latency of their loads (about 2000 cycles under the operand traffic).  A warp's K blocks
    // lie kMxScaleWarps <= kMxSfSlots apart, so it is never more than one refill of a slot ahead and the slot's
    // phases stay distinguishable.
    static_assert(kMxScaleWarps <= kMxSfSlots && (kMxScaleWarps & (kMxScaleWarps - 1)) == 0, "loader warps");
    const uint32_t lw = static_cast<uint32_t>(warp - 6);   // 0 .. kMxScaleWarps - 1
    uint32_t it = 0;
    uint32_t s = lw, round = 0;          // slot of this warp's next K block, and how often that slot was refilled
    bool ok = true;
    for (int tile = unit0; tile < tiles && ok; tile += unit_step) {
      int mt, nt;
      grouped_tile_coords(tile, p.group_m, p.m_tiles, p.n_tiles, mt, nt);
      for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
        if ((it & static_cast<uint32_t>(kMxScaleWarps - 1)) != lw) continue;
        const int g0 = kb * 4;
        const int row0 = mt * kTileM + my_row0, col0 = nt * p.bn;
        // Loads first (they do not touch the stage), then the wait for the stage, then the stores.  A lane ends up
        // with up to four left-operand words (rows ar[i]) and eight right-operand words (columns bc[i]); word =
        // the four E8M0 codes of the K block, code g in byte g.
        //
        // Fast paths: when the tile lies inside the matrix and the scale arrays are aligned, a lane fetches the codes
        // of several neighbouring rows / columns with a few wide loads and sorts the bytes in registers.  One-byte
        // loads (the general path below) cost a memory round trip per 32 bytes and were 2.2x the time of the
        // whole kernel.
        uint32_t wa[4], wb[8];
        int ar[4], bc[8];
        int na = 4, nb = 0;
        const bool k_in = g0 + 4 <= p.kgroups && (p.kgroups & 3) == 0;
        const bool a_fast_log = p.a_layout == PTO_MX_SCALE_LOGICAL && k_in && (reinterpret_cast<uintptr_t>(p.a_scale) & 3) == 0;
        const bool a_fast_zz = p.a_layout == PTO_MX_SCALE_A_ZZ && k_in && row0 + 128 <= p.m &&
                               (reinterpret_cast<uintptr_t>(p.a_scale) & 7) == 0;
        const bool b_fast_log = p.b_layout == PTO_MX_SCALE_LOGICAL && k_in && col0 + p.bn <= p.n && (p.n & 7) == 0 &&
                                (reinterpret_cast<uintptr_t>(p.b_scale) & 7) == 0;
        const bool b_fast_nn = p.b_layout == PTO_MX_SCALE_B_NN && k_in && col0 + p.bn <= p.n &&
                               (reinterpret_cast<uintptr_t>(p.b_scale) & 15) == 0;
        // ---- left operand ----
        if (a_fast_zz) {
          // [m/16][kg/2][16 rows][2 codes]: a group of 16 rows keeps codes (g0, g0+1) of its rows in 32 contiguous bytes
          // and (g0+2, g0+3) in the next 32; lane = (group of 16 rows, quarter): four rows, two 8-byte loads
          const int grp = lane >> 2, qd = lane & 3;
          const uint8_t* base = p.a_scale + (static_cast<size_t>((row0 >> 4) + grp) * (p.kgroups >> 1) + (g0 >> 1)) * 32 + 8 * qd;
          const uint2 lo = __ldg(reinterpret_cast<const uint2*>(base)), hi = __ldg(reinterpret_cast<const uint2*>(base + 32));
          wa[0] = __byte_perm(lo.x, hi.x, 0x5410); wa[1] = __byte_perm(lo.x, hi.x, 0x7632);
          wa[2] = __byte_perm(lo.y, hi.y, 0x5410); wa[3] = __byte_perm(lo.y, hi.y, 0x7632);
#pragma unroll
          for (int i = 0; i < 4; ++i) ar[i] = grp * 16 + qd * 4 + i;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) ar[j] = j * 32 + lane;
          if (a_fast_log) {   // four codes of a row are one aligned word
#pragma unroll
            for (int j = 0; j < 4; ++j) wa[j] = __ldg(reinterpret_cast<const uint32_t*>(a_scale_ptr(p, row0 + ar[j], g0)));
          } else {
            uint32_t ca[16];
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
              for (int g = 0; g < 4; ++g) ca[j * 4 + g] = __ldg(a_scale_ptr(p, row0 + ar[j], g0 + g));
#pragma unroll
            for (int j = 0; j < 4; ++j) wa[j] = ca[j * 4] | (ca[j * 4 + 1] << 8) | (ca[j * 4 + 2] << 16) | (ca[j * 4 + 3] << 24);
          }
          // codes outside the matrix count as 1.0
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const bool row_in = row0 + ar[j] < p.m;
            uint32_t w = wa[j];
#pragma unroll
            for (int g = 0; g < 4; ++g)
              if (!row_in || g0 + g >= p.kgroups) w = (w & ~(0xFFu << (8 * g))) | (127u << (8 * g));
            wa[j] = w;
          }
        }
        // ---- right operand ----
        if (b_fast_log) {
          // [kg][n]: the codes of one K group are contiguous over the columns; lane = eight neighbouring columns, one
          // 8-byte load per K group, then a 4 x 8 byte transpose
          if (8 * lane < p.bn) {
            nb = 8;
            const uint8_t* base = p.b_scale + static_cast<size_t>(g0) * p.n + col0 + 8 * lane;
            const uint2 v0 = __ldg(reinterpret_cast<const uint2*>(base)), v1 = __ldg(reinterpret_cast<const uint2*>(base + p.n));
            const uint2 v2 = __ldg(reinterpret_cast<const uint2*>(base + 2 * static_cast<size_t>(p.n)));
            const uint2 v3 = __ldg(reinterpret_cast<const uint2*>(base + 3 * static_cast<size_t>(p.n)));
            uint32_t t0 = __byte_perm(v0.x, v1.x, 0x5140), t1 = __byte_perm(v2.x, v3.x, 0x5140);
            uint32_t t2 = __byte_perm(v0.x, v1.x, 0x7362), t3 = __byte_perm(v2.x, v3.x, 0x7362);
            wb[0] = __byte_perm(t0, t1, 0x5410); wb[1] = __byte_perm(t0, t1, 0x7632);
            wb[2] = __byte_perm(t2, t3, 0x5410); wb[3] = __byte_perm(t2, t3, 0x7632);
            t0 = __byte_perm(v0.y, v1.y, 0x5140); t1 = __byte_perm(v2.y, v3.y, 0x5140);
            t2 = __byte_perm(v0.y, v1.y, 0x7362); t3 = __byte_perm(v2.y, v3.y, 0x7362);
            wb[4] = __byte_perm(t0, t1, 0x5410); wb[5] = __byte_perm(t0, t1, 0x7632);
            wb[6] = __byte_perm(t2, t3, 0x5410); wb[7] = __byte_perm(t2, t3, 0x7632);
#pragma unroll
            for (int i = 0; i < 8; ++i) bc[i] = 8 * lane + i;
          }
        } else if (b_fast_nn) {
          // [n/16][kg/2][16 columns][2 codes]: as the left operand's physical layout; lane = (group of 16 columns,
          // half): eight columns, two 16-byte loads
          const int grp = lane >> 1, hf = lane & 1;
          if (grp * 16 < p.bn) {
            nb = 8;
            const uint8_t* base = p.b_scale + (static_cast<size_t>((col0 >> 4) + grp) * (p.kgroups >> 1) + (g0 >> 1)) * 32 + 16 * hf;
            const uint4 lo = __ldg(reinterpret_cast<const uint4*>(base)), hi = __ldg(reinterpret_cast<const uint4*>(base + 32));
            wb[0] = __byte_perm(lo.x, hi.x, 0x5410); wb[1] = __byte_perm(lo.x, hi.x, 0x7632);
            wb[2] = __byte_perm(lo.y, hi.y, 0x5410); wb[3] = __byte_perm(lo.y, hi.y, 0x7632);
            wb[4] = __byte_perm(lo.z, hi.z, 0x5410); wb[5] = __byte_perm(lo.z, hi.z, 0x7632);
            wb[6] = __byte_perm(lo.w, hi.w, 0x5410); wb[7] = __byte_perm(lo.w, hi.w, 0x7632);
#pragma unroll
            for (int i = 0; i < 8; ++i) bc[i] = grp * 16 + hf * 8 + i;
          }
        } else {
          nb = static_cast<int>(sfb_chunks) * 4;
          uint32_t cb[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            bc[j] = j * 32 + lane;
#pragma unroll
            for (int g = 0; g < 4; ++g)
              cb[j * 4 + g] = j < nb ? static_cast<uint32_t>(__ldg(b_scale_ptr(p, col0 + bc[j], g0 + g))) : 127u;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const bool col_in = col0 + bc[j] < p.n;
            uint32_t w = 0;
#pragma unroll
            for (int g = 0; g < 4; ++g) w |= ((col_in && g0 + g < p.kgroups) ? cb[j * 4 + g] : 127u) << (8 * g);
            wb[j] = w;
          }
        }
        if (!mbar_wait_warp(&sf_empty[s], (round & 1u) ^ 1u)) {
          report_error(p.err, kErrBarrierTimeout, 75, static_cast<int>(it));
          ok = false;
          break;
        }
        uint8_t* sf = sf_ring + s * sf_bytes;
        // row (or column) r of a 128-row chunk sits at byte (r % 32) * 16 + (r / 32) * 4 of the chunk; the left
        // operand's chunk comes first, the right operand's chunks (128 columns each) follow
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i < na) *reinterpret_cast<uint32_t*>(sf + (ar[i] & 31) * 16 + (ar[i] >> 5) * 4) = wa[i];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (i < nb) {
            const int r = bc[i] & 127;
            *reinterpret_cast<uint32_t*>(sf + 512 * (1 + (bc[i] >> 7)) + (r & 31) * 16 + (r >> 5) * 4) = wb[i];
          }
        fence_proxy_async_smem();   // the chunk is read by tcgen05.cp (async proxy)
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_peer(mapa_u32(smem_u32(&sf_full[s]), 0));
          else mbar_arrive(&sf_full[s]);
        }
        s += kMxScaleWarps;
        if (s >= kMxSfSlots) {
          s -= kMxSfSlots;
          ++round;
        }
      }
    }
  }
  tc_fence_before_sync();
  if constexpr (PAIR) {
    cluster_sync_all();   // neither CTA leaves, or frees tensor memory, while its partner may still signal or read it
    if (warp == 1) tmem_dealloc_pair(tmem_base, tmem_cols);
  } else {
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
  }
}

__global__ void __launch_bounds__(kMxThreads, 1)
matmul_mx_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const MxParams p) {
  matmul_mx_body<false>(&tm_a, &tm_b, nullptr, nullptr, p);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMxPairThreads, 1)
matmul_mx_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb,
                      const MxParams p) {
  matmul_mx_body<true>(&tm_a, &tm_b, &tm_sfa, &tm_sfb, p);
}

// Scale blocks for the pair kernel, in the order the tensor core reads them: word (r % 32) * 4 + r / 32 of a
// 512-byte chunk holds the four E8M0 codes of one K block for row (or column) r of the chunk's 128.
//   sfa: one chunk per (group of 128 rows of a, K block);   sfb: ceil(bn / 128) chunks per (tile column, K block),
// columns counted from the tile's first.  Codes outside the matrix, or past the tile's width, are 127 (= 1.0).
// One 512-byte chunk per group of 128 threads; thread t takes row (or column) t of the chunk, so the loads of the
// logical right-operand layout are contiguous over the threads.
__global__ void __launch_bounds__(256)
mx_pack_scales_kernel(const MxParams p, uint32_t* __restrict__ sfa, uint32_t* __restrict__ sfb, int a_groups) {
  pdl_launch_dependents();
  pdl_wait();
  const unsigned chunks = (p.bn + 127) / 128, kblocks = p.kblocks;
  const unsigned a_chunks = static_cast<unsigned>(a_groups) * kblocks;
  const unsigned all_chunks = a_chunks + static_cast<unsigned>(p.n_tiles) * kblocks * chunks;
  const unsigned r = threadIdx.x & 127;
  const bool k4 = (p.kgroups & 3) == 0;
  const bool a_words = p.a_layout == PTO_MX_SCALE_LOGICAL && k4 && (reinterpret_cast<uintptr_t>(p.a_scale) & 3) == 0;
  for (unsigned ch = blockIdx.x * 2 + (threadIdx.x >> 7); ch < all_chunks; ch += gridDim.x * 2) {
    uint32_t word = 0;
    if (ch < a_chunks) {
      const unsigned outer = ch / kblocks, kb = ch - outer * kblocks;
      const int row = static_cast<int>(outer * 128 + r), g0 = static_cast<int>(kb * 4);
      if (a_words && row < p.m && g0 + 4 <= p.kgroups) {   // the four codes of a row are one aligned word
        word = __ldg(reinterpret_cast<const uint32_t*>(p.a_scale + static_cast<size_t>(row) * p.kgroups + g0));
      } else {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t code = __ldg(a_scale_ptr(p, row, g0 + g));
          word |= ((row < p.m && g0 + g < p.kgroups) ? code : 127u) << (8 * g);
        }
      }
      sfa[static_cast<size_t>(ch) * 128 + (r & 31) * 4 + (r >> 5)] = word;
    } else {
      const unsigned j = ch - a_chunks;
      const unsigned blk = j / chunks, c = j - blk * chunks;
      const unsigned outer = blk / kblocks, kb = blk - outer * kblocks;
      const int cin = static_cast<int>(c * 128 + r), col = static_cast<int>(outer) * p.bn + cin, g0 = static_cast<int>(kb * 4);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint32_t code = __ldg(b_scale_ptr(p, col, g0 + g));
        word |= ((cin < p.bn && col < p.n && g0 + g < p.kgroups) ? code : 127u) << (8 * g);
      }
      sfb[static_cast<size_t>(j) * 128 + (r & 31) * 4 + (r >> 5)] = word;
    }
  }
}

// dst[c, r] = src[r, c], bytes; 32 x 32 tiles through shared memory.
__global__ void __launch_bounds__(256)
transpose_u8_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, long long rows, long long cols) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ uint8_t tile[32][33];
  const long long tiles_c = (cols + 31) / 32, tiles_r = (rows + 31) / 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  for (long long t = blockIdx.x; t < tiles_r * tiles_c; t += gridDim.x) {
    const long long r0 = (t / tiles_c) * 32, c0 = (t % tiles_c) * 32;
    for (int i = ty; i < 32; i += 8)
      if (r0 + i < rows && c0 + tx < cols) tile[i][tx] = src[(r0 + i) * cols + c0 + tx];
    __syncthreads();
    for (int i = ty; i < 32; i += 8)
      if (c0 + i < cols && r0 + tx < rows) dst[(c0 + i) * rows + r0 + tx] = tile[tx][i];
    __syncthreads();
  }
}

}  // namespace

int transpose_u8_launch(const void* src, void* dst, long long rows, long long cols, cudaStream_t stream) {
  PTO_REQUIRE(src && dst, "transpose_u8: NULL tensor");
  PTO_REQUIRE(rows >= 0 && cols >= 0, "transpose_u8: negative size");
  if (rows == 0 || cols == 0) return kOk;
  const long long tiles = ((rows + 31) / 32) * ((cols + 31) / 32);
  const long long cap = static_cast<long long>(sm_count()) * 16;
  launch_kernel(transpose_u8_kernel, dim3(static_cast<unsigned>(tiles < cap ? tiles : cap)), dim3(256), 0, stream,
                static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, cols);
  return check_cuda(cudaGetLastError(), "transpose_u8_kernel launch");
}

int matmul_mx_launch(const void* a, const void* a_scale, int a_scale_layout, const void* b_t, const void* b_scale,
                     int b_scale_layout, const float* acc_in, float* out, int m, int n, int k, int* err,
                     cudaStream_t stream) {
  PTO_REQUIRE(a && a_scale && b_t && b_scale && out, "matmul_mx: NULL tensor");
  PTO_REQUIRE(m > 0 && n > 0 && k > 0, "matmul_mx: empty problem");
  PTO_REQUIRE(k % 32 == 0, "matmul_mx: K must be a multiple of the 32-element scale group");
  PTO_REQUIRE(a_scale_layout == PTO_MX_SCALE_LOGICAL || a_scale_layout == PTO_MX_SCALE_A_ZZ,
              "matmul_mx: a_scale layout must be PTO_MX_SCALE_LOGICAL or PTO_MX_SCALE_A_ZZ");
  PTO_REQUIRE(b_scale_layout == PTO_MX_SCALE_LOGICAL || b_scale_layout == PTO_MX_SCALE_B_NN,
              "matmul_mx: b_scale layout must be PTO_MX_SCALE_LOGICAL or PTO_MX_SCALE_B_NN");
  const int kgroups = k / 32;
  PTO_REQUIRE(a_scale_layout == PTO_MX_SCALE_LOGICAL || (m % 16 == 0 && kgroups % 2 == 0),
              "matmul_mx: the MX_A_ZZ scale layout needs m a multiple of 16 and an even number of K groups");
  PTO_REQUIRE(b_scale_layout == PTO_MX_SCALE_LOGICAL || (n % 16 == 0 && kgroups % 2 == 0),
              "matmul_mx: the MX_B_NN scale layout needs n a multiple of 16 and an even number of K groups");
  MxParams p;
  p.m = m; p.n = n; p.k = k; p.kgroups = kgroups;
  p.kblocks = (k + kMxBK - 1) / kMxBK;
  // 256-column tiles halve the left-operand traffic per FLOP; they pay once the problem has many tiles
  const long long tiles128 = static_cast<long long>((m + 127) / 128) * ((n + 127) / 128);
  // SM pairs (256 x 224 tiles, two accumulators) once every pair has at least two tiles and K is long enough for the
  // kernel that packs the scale blocks to be small beside the matmul
  static const int pair_enabled = [] { const char* v = getenv("PTO_MX_PAIR"); return v ? atoi(v) : 1; }();
  const bool pair = pair_enabled && m >= 512 && n >= 448 && k >= 1024 &&
                    static_cast<long long>((m + 255) / 256) * ((n + 223) / 224) >= sm_count();
  if (pair) {
    p.bn = 224;
    p.nbuf = 2;
    p.m_tiles = (m + 255) / 256;
  } else {
    p.bn = (n >= 256 && tiles128 >= 4ll * sm_count()) ? 256 : 128;
    p.nbuf = p.bn == 128 ? 2 : 1;
    p.m_tiles = (m + 127) / 128;
  }
  p.n_tiles = (n + p.bn - 1) / p.bn;
  p.group_m = 16;   // 2048 (one CTA) or 4096 (pairs) rows of a per group; measured 4 / 8 / 16 / all rows
  p.a_scale = static_cast<const uint8_t*>(a_scale); p.b_scale = static_cast<const uint8_t*>(b_scale);
  p.a_layout = a_scale_layout; p.b_layout = b_scale_layout;
  p.acc_in = acc_in; p.out = out; p.err = err;
  const size_t sf_bytes = 512 * (1 + (p.bn + 127) / 128);
  const int b_box_rows = pair ? p.bn / 2 : 128;   // a CTA of a pair loads its half of the b_t tile with one box
  const size_t stage_bytes = static_cast<size_t>(128 + (pair ? p.bn / 2 : p.bn)) * kMxBK + (pair ? 1024 * ((sf_bytes + 1023) / 1024) : 0);
  const size_t fixed_bytes = 1024 + (pair ? 0 : kMxSfSlots * sf_bytes) + (2 * kMxMaxStages + 5 + 2 * kMxSfSlots) * 8 + 16;
  int stages = static_cast<int>((227 * 1024 - fixed_bytes) / stage_bytes);
  if (stages > kMxMaxStages) stages = kMxMaxStages;
  PTO_REQUIRE(stages >= 2, "matmul_mx: shared memory does not fit two pipeline stages");
  p.stages = stages;
  const size_t smem = fixed_bytes + stages * stage_bytes;
  const long long tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
  PTO_REQUIRE(tiles < (1ll << 31), "matmul_mx: problem too large");

  CUtensorMap tm_a, tm_b;
  int st = make_tensor_map_2d(&tm_a, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, m, k, k, kMxBK, 128,
                              CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_b, b_t, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, n, k, k, kMxBK, b_box_rows,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  if (pair) {
    // Scale blocks in the tensor core's order, built by a small kernel into stream-ordered scratch memory (1/32 of
    // the operands' bytes) and fetched by TMA like the operands.
    const int chunks = (p.bn + 127) / 128, a_groups = 2 * p.m_tiles;
    const size_t sfa_bytes = static_cast<size_t>(a_groups) * p.kblocks * 512;
    const size_t sfb_bytes = static_cast<size_t>(p.n_tiles) * p.kblocks * 512 * chunks;
    void* scratch = nullptr;
    st = scratch_alloc_async(&scratch, sfa_bytes + sfb_bytes, stream);
    if (st != kOk) return st;
    uint32_t* sfa = static_cast<uint32_t*>(scratch);
    uint32_t* sfb = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(scratch) + sfa_bytes);
    CUtensorMap tm_sfa, tm_sfb;
    st = make_tensor_map_2d(&tm_sfa, sfa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, static_cast<uint64_t>(a_groups) * p.kblocks, 128, 512,
                            128, 1, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st == kOk)
      st = make_tensor_map_2d(&tm_sfb, sfb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, static_cast<uint64_t>(p.n_tiles) * p.kblocks,
                              128 * chunks, 512 * chunks, 128 * chunks, 1, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != kOk) {
      scratch_free_async(scratch, stream);
      return st;
    }
    const long long pack_chunks = static_cast<long long>(sfa_bytes + sfb_bytes) / 512;
    PTO_REQUIRE(pack_chunks < (1ll << 31), "matmul_mx: problem too large");
    const long long pack_cap = static_cast<long long>(sm_count()) * 8;
    const long long pack_blocks = (pack_chunks + 1) / 2;
    launch_kernel(mx_pack_scales_kernel, dim3(static_cast<unsigned>(pack_blocks < pack_cap ? pack_blocks : pack_cap)), dim3(256), 0,
                  stream, p, sfa, sfb, a_groups);
    if (first_use_on_device(6))
      PTO_CUDA(cudaFuncSetAttribute(matmul_mx_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    int pairs = sm_count() / 2;
    if (pairs > tiles) pairs = static_cast<int>(tiles);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kMxPairThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = nullptr;      // the cluster shape is a compile-time attribute of the kernel
    cfg.numAttrs = 0;
    const cudaError_t launched = cudaLaunchKernelEx(&cfg, matmul_mx_pair_kernel, tm_a, tm_b, tm_sfa, tm_sfb, p);
    scratch_free_async(scratch, stream);   // in stream order: after the kernel
    PTO_CUDA(launched);
    return check_cuda(cudaGetLastError(), "matmul_mx_pair_kernel launch");
  }
  if (first_use_on_device(2))
    PTO_CUDA(cudaFuncSetAttribute(matmul_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  launch_kernel(matmul_mx_kernel, dim3(grid), dim3(kMxThreads), smem, stream, tm_a, tm_b, p);
  return check_cuda(cudaGetLastError(), "matmul_mx_kernel launch");
}

}  // namespace pto
