// Grouped expert GEMM in FP8 (e4m3) with 128x128 weight-block scales and per-(token, 128
// channel) activation scales, on tcgen05 tensor cores.
//
// It replaces the stand-in expert of the reference's expert-parallel test
// (local_expert_step, tests/st/distributed/test_l3_ep_dispatch_combine.py:309-327) by the real
// SwiGLU expert FFN of the workload.  The reference's nearest numerics are its MX-FP8 matmul
// golden, which dequantises per K group and accumulates exactly
// (tests/st/runtime/ops/test_matmul_mx.py:119-131); here the scale granularity is one fp32
// per 128x128 weight block and per (token, 128 channels):
//
//   out[t, n] = sum over 128-wide K blocks kb of
//               ( sum_k xq[t, k] * wq[n, k] ) * xs[t, kb] * ws[n / 128, kb]
//
// Tokens arrive sorted by expert (rows offsets[e] .. offsets[e+1]).  One work unit is
// (expert, 128-row weight tile, chunk of up to 128 tokens).  The token chunk fills the 128 TMEM
// lanes (A operand) and the weight tile is the MMA N dimension, so a promotion thread owns ONE
// token and the two scales of a K block collapse into one scalar per thread,
// xs[token, kb] * ws[tile, kb].  Every weight byte of an expert is streamed once per token chunk:
// the kernel is weight-bandwidth bound at ~128 tokens per expert.
//
// Per K block the raw fp8 products land in one of four TMEM partial buffers; eight promotion warps
// pull them into registers (64 fp32 accumulators per thread), scale and accumulate.  What bounds the
// kernel is the number of instructions an SM issues per K block around that handful of FMAs (waits,
// arrivals, address arithmetic, loop control), so the promotion loop is built to keep that number low --
//   * eight warps with 64 columns each instead of sixteen with 32: the per-warp cost of a K block (one wait
//     for the tensor core, one arrival, the loop) is paid half as often;
//   * a thread loads half of its columns at a time (two 16-column TMEM loads) into one of two register sets:
//     while the FMAs of one half run, the loads of the next half are in flight;
//   * the loop is unrolled over the four partial buffers, so barrier and TMEM addresses are constants;
//   * a thread reads the scales of its own token straight from global memory, four K blocks per 16-byte
//     load and one load ahead of their use; the producer brings in what a unit shares (two bulk copies of
//     weight-block scales, a record with the unit's rows) one unit ahead;
//   * promotion warps never decode units and share no barrier among themselves; a warp whose 32
//     tokens all lie past the end of a short chunk only hands the partial buffers back;
//   * the two producer threads and the two issuer threads carry stages, buffers and barrier phases along
//     instead of dividing, and the issuers advance the operand descriptors by additions.
//
//   SwiGLU mode: the tile is 64 gate rows + the 64 matching up rows; a thread holds 32 gate
//                columns and the 32 matching up columns, so silu(g) * u needs no exchange.
//                (The per-(token, 128) re-quantisation for the down projection is a
//                separate row pass.)
//   plain mode:  128 output features; epilogue = bf16(acc * route_weight[token]), written to
//                row out_rows[token] when a row map is given.
//
// CTA = 12 warps: two TMA producers and two MMA issuers (alternating K blocks), 8
// promotion/epilogue warps (2 per TMEM lane quarter).  Bounded waits.
#include "common.cuh"
#include "kernels.h"

namespace pto {
namespace {

constexpr int kTN = 128;          // tokens per chunk = MMA M (TMEM lanes)
constexpr int kPromoWarps = 8;
constexpr int kRoleWarps = 4;      // two TMA producers and two MMA issuers, alternating K blocks
constexpr int kMoeThreads = (kRoleWarps + kPromoWarps) * 32;
constexpr int kNumPartial = 4;    // TMEM partial buffers of 128 feature columns
constexpr int kNumTables = 3;     // unit tables: the unit in work, the next one, and one being released
constexpr int kMoeMaxStages = 8;
constexpr int kMoeMaxKBlocks = 64;   // K <= 8192
struct MoeGemmParams {
  const int32_t* offsets;   // [experts + 1]
  int experts, n_tiles, kblocks;
  int w_rows_per_expert, up_row_off;   // SwiGLU: up rows start up_row_off rows after the gate rows
  int n_out;                // output features per row
  const float* w_scale;     // [experts][w_rows_per_expert / 128][kblocks]
  const float* x_scale;     // [rows][kblocks]
  const float* route_w;     // [rows] or NULL
  const int32_t* out_rows;  // [rows] or NULL: output row of each input row (plain mode)
  __nv_bfloat16* out;       // [rows][n_out]
  int total_rows, stages;
  int* err;
};

// One unit table: ws[2][kbp] (weight-block scales of the gate or plain rows, of the up rows) and a 4-int
// record {first row, end row of the expert, tile, unused}; kbp = K blocks rounded up to 4.
__host__ __device__ inline int table_floats(int kblocks) {
  const int kbp = (kblocks + 3) & ~3;
  return (2 * kbp + 4 + 31) & ~31;   // whole 128-byte lines
}

__device__ __forceinline__ float lds_f32(uint32_t saddr) {
  float r;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(r) : "r"(saddr));
  return r;
}
__device__ __forceinline__ float4 ldg_f32x4(const float* p) {
  float4 r;
  asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ int4 lds_s32x4(uint32_t saddr) {
  int4 r;
  asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(saddr));
  return r;
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Waits for this thread's TMEM loads.  The loaded registers pass through the statement, so every use of them
// is ordered after the wait, also while another set of registers is still being loaded.
__device__ __forceinline__ void tmem_ld_wait_regs(uint32_t (&a)[16], uint32_t (&b)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]),
                 "+r"(a[8]), "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15])
               :
               : "memory");
  asm volatile(""
               : "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]),
                 "+r"(b[8]), "+r"(b[9]), "+r"(b[10]), "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15])
               :
               : "memory");
}

// A unit = (expert, weight tile, chunk of 128 tokens).
//   plain mode:  the tile is 128 consecutive output features (TMEM columns 0-127).
//   SwiGLU mode: the tile is 64 gate rows (columns 0-63) followed by the 64 matching up rows
//                (columns 64-127); the epilogue writes bf16(silu(g) * u) for 64 features.
// FAST: K blocks come in fours and the scale arrays are 16-byte aligned, so scales move in 16-byte units and the
// promotion loop runs with constant partial-buffer numbers.  Otherwise the first producer warp copies the
// weight-block scales with plain loads, token scales are read one by one and the loop computes buffer numbers
// as it goes.
template <bool SWIGLU, bool FAST>
__global__ void __launch_bounds__(kMoeThreads, 1)
moe_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                    const MoeGemmParams p) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t tile_bytes = 128 * 128;
  const uint32_t stage_bytes = 2 * tile_bytes;   // weight tile, token tile
  uint8_t* after = smem + static_cast<size_t>(p.stages) * stage_bytes;
  const int kbp = (p.kblocks + 3) & ~3;
  const int tab_floats = table_floats(p.kblocks);
  float* tables = reinterpret_cast<float*>(after);                     // [kNumTables][tab_floats]
  int* prefix = reinterpret_cast<int*>(tables + kNumTables * tab_floats);   // [experts + 1] chunk prefix
  int* offs = prefix + ((p.experts + 2) & ~1);                         // [experts + 1] copy of the row offsets
  uint64_t* full = reinterpret_cast<uint64_t*>(offs + ((p.experts + 2) & ~1));
  uint64_t* empty = full + kMoeMaxStages;
  uint64_t* pfull = empty + kMoeMaxStages;
  uint64_t* pempty = pfull + kNumPartial;
  uint64_t* sfull = pempty + kNumPartial;    // scale table written
  uint64_t* sempty = sfull + kNumTables;     // scale table no longer read (one arrival per promotion warp)
  uint64_t* drain = sempty + kNumTables;     // one per MMA issuer: all of its MMAs have completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t tmem_cols = kNumPartial * 128;  // 512

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < kNumPartial; ++i) {
      mbar_init(&pfull[i], 1);
      mbar_init(&pempty[i], kPromoWarps);
    }
    for (int i = 0; i < kNumTables; ++i) {
      mbar_init(&sfull[i], 1);
      mbar_init(&sempty[i], kPromoWarps);
    }
    mbar_init(&drain[0], 1);
    mbar_init(&drain[1], 1);
    fence_barrier_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 2) tmem_alloc(tmem_slot, tmem_cols);
  pdl_wait();   // barrier set-up and TMEM allocation overlap the previous kernel; offsets are read next
  // chunk prefix over experts: prefix[e] = number of token chunks of experts before e
  for (int e = threadIdx.x; e <= p.experts; e += kMoeThreads) {
    const int o = p.offsets[e];
    offs[e] = o;
    if (e < p.experts) {
      const int n = p.offsets[e + 1] - o;
      prefix[e + 1] = n > 0 ? (n + kTN - 1) / kTN : 0;
    }
  }
  if (threadIdx.x == 0) prefix[0] = 0;
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 1; base <= p.experts; base += 32) {
      const int i = base + lane;
      int v = i <= p.experts ? prefix[i] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      v += carry;
      if (i <= p.experts) prefix[i] = v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int units = prefix[p.experts] * p.n_tiles;
  const int grid = static_cast<int>(gridDim.x);

  // unit -> (expert, tile, chunk); units of one (expert, tile) are adjacent
  auto decode = [&](int u, int& e, int& tile, int& chunk) {
    int lo = 0, hi = p.experts - 1;
    const int target = u / p.n_tiles;  // first e with prefix[e + 1] > target
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid + 1] > target) hi = mid; else lo = mid + 1;
    }
    e = lo;
    const int chunks = prefix[e + 1] - prefix[e];
    const int rem = u - prefix[e] * p.n_tiles;
    tile = rem / chunks;
    chunk = rem - tile * chunks;
  };

  if (warp < kRoleWarps) {
    // A single thread needs several hundred cycles per K block for its barrier waits, TMA or MMA
    // issues and commits; two producers and two issuers take alternate K blocks to keep up.
    if (warp < 2) {
      // ------------------------------ TMA producers ------------------------------
      // The first producer warp also brings in the scale table of every unit, one unit ahead of the operands.
      // n-th unit of this CTA -> table n % kNumTables; the table of unit n + 1 reuses the one of unit n - 2,
      // which the promotion warps have long released, so that wait does not hold the operand stream up.
      auto stage_table = [&](int n, int e, int tile, int chunk) -> bool {
        const int tb = n % kNumTables, use = n / kNumTables;
        int ok = 1;
        if (use > 0 && lane == 0) ok = mbar_wait(&sempty[tb], (static_cast<uint32_t>(use) - 1u) & 1u) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0) report_error(p.err, kErrBarrierTimeout, 54, n);
          return false;
        }
        float* tab = tables + tb * tab_floats;
        const int row0 = offs[e] + chunk * kTN;
        const int wrow = e * p.w_rows_per_expert + (SWIGLU ? tile * 64 : tile * 128);
        const float* w0 = p.w_scale + static_cast<size_t>(wrow / 128) * p.kblocks;
        const float* w1 = p.w_scale + static_cast<size_t>((wrow + p.up_row_off) / 128) * p.kblocks;
        if (lane == 0) {
          int* rec = reinterpret_cast<int*>(tab + 2 * kbp);
          rec[0] = row0;
          rec[1] = min(offs[e + 1], p.total_rows);
          rec[2] = tile;
          rec[3] = 0;
        }
        if (FAST) {
          if (lane == 0) {
            const uint32_t ws_bytes = static_cast<uint32_t>(p.kblocks * 4);
            mbar_arrive_expect_tx(&sfull[tb], 2 * ws_bytes);   // releases the record written above
            bulk_load(tab, w0, ws_bytes, &sfull[tb]);
            bulk_load(tab + kbp, w1, ws_bytes, &sfull[tb]);
          }
        } else {
          for (int kb = lane; kb < p.kblocks; kb += 32) {
            tab[kb] = __ldg(w0 + kb);
            tab[kbp + kb] = __ldg(w1 + kb);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&sfull[tb]);
        }
        return true;
      };

      // K blocks are numbered through all units of this CTA; producer `me` takes the blocks i with i % 2 == me and
      // block i lives in stage i % stages.  The stage and the phase of its barriers are carried along, not
      // recomputed: a division per K block is most of what such a one-thread loop would cost.
      const uint32_t me = static_cast<uint32_t>(warp);
      uint32_t it = 0;                  // index of the unit's first K block
      uint32_t st_i = me, st_ph = 0;    // stage of this producer's next block and how often it has been refilled (mod 2)
      uint32_t next_i = me;             // this producer's next block
      bool ok = true;
      int e = 0, tile = 0, chunk = 0, n = 0;
      if (static_cast<int>(blockIdx.x) < units) {
        decode(blockIdx.x, e, tile, chunk);
        if (me == 0) ok = stage_table(0, e, tile, chunk);
      }
      for (int u = blockIdx.x; u < units && ok; u += grid, ++n) {
        int e2 = 0, tile2 = 0, chunk2 = 0;
        if (u + grid < units) {
          decode(u + grid, e2, tile2, chunk2);
          if (me == 0) ok = stage_table(n + 1, e2, tile2, chunk2);
        }
        if (ok) {   // the whole warp walks the K blocks and waits; one elected lane issues the copies
          const int row0 = offs[e] + chunk * kTN;
          const int wrow = e * p.w_rows_per_expert + tile * (SWIGLU ? 64 : 128);
          const uint32_t end_i = it + static_cast<uint32_t>(p.kblocks);
          for (; next_i < end_i; next_i += 2) {
            const int kb = static_cast<int>(next_i - it);
            if (!__all_sync(0xffffffffu, mbar_wait(&empty[st_i], st_ph ^ 1u))) {
              if (lane == 0) report_error(p.err, kErrBarrierTimeout, 50, static_cast<int>(next_i));
              ok = false;
              break;
            }
            if (elect_one()) {
              uint8_t* st = smem + st_i * stage_bytes;
              mbar_arrive_expect_tx(&full[st_i], stage_bytes);
              if (SWIGLU) {   // two 64-row boxes: gate rows, then the matching up rows
                tma_load_2d(st, &tm_w, kb * 128, wrow, &full[st_i]);
                tma_load_2d(st + 64 * 128, &tm_w, kb * 128, wrow + p.up_row_off, &full[st_i]);
              } else {
                tma_load_2d(st, &tm_w, kb * 128, wrow, &full[st_i]);
              }
              tma_load_2d(st + tile_bytes, &tm_x, kb * 128, row0, &full[st_i]);
            }
            __syncwarp();
            st_i += 2;                  // the stage count is even: a producer keeps to the stages of its parity
            if (st_i >= static_cast<uint32_t>(p.stages)) {
              st_i -= static_cast<uint32_t>(p.stages);
              st_ph ^= 1u;
            }
          }
        }
        it += static_cast<uint32_t>(p.kblocks);
        e = e2; tile = tile2; chunk = chunk2;
      }
    } else {
      // ------------------------------- MMA issuers -------------------------------
      // The whole warp walks the loop and waits; one elected lane issues.  Warp-uniform code keeps descriptors and
      // barrier addresses in uniform registers, which is what the MMA and commit instructions take.
      const uint32_t me = static_cast<uint32_t>(warp - 2);
      const uint32_t idesc = umma_idesc(kTN, 128, 0, 0);  // e4m3 x e4m3 -> fp32; M = tokens, N = features
      // The issuer does not need the units, only the number of K blocks of this CTA.  Issuer `me` takes the
      // blocks i with i % 2 == me: stage i % stages, partial buffer i % 4 (me or me + 2).  Stage, buffer and
      // barrier phases are carried along, and the operand descriptors advance by additions.
      const int my_units = static_cast<int>(blockIdx.x) < units ? (units - 1 - static_cast<int>(blockIdx.x)) / grid + 1 : 0;
      const uint32_t total = static_cast<uint32_t>(my_units) * static_cast<uint32_t>(p.kblocks);
      const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);   // stride byte offset, version, 128-byte swizzle
      const uint32_t lo0 = ((smem_u32(smem) & 0x3FFFFu) >> 4) | (1u << 16);
      uint32_t st_i = me, st_ph = 0;       // stage and phase of its `full` barrier
      uint32_t pb = me, pb_ph = 1;         // partial buffer and the phase of `pempty` to wait for (first use: free)
      uint32_t i = me;
      for (; i < total; i += 2) {
        const bool ok = mbar_wait(&full[st_i], st_ph) && mbar_wait(&pempty[pb], pb_ph);
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0) report_error(p.err, kErrBarrierTimeout, 51, static_cast<int>(i));
          break;
        }
        tc_fence_after_sync();
        if (elect_one()) {
          const uint32_t w_lo = lo0 + st_i * (stage_bytes >> 4);
          const uint32_t x_lo = w_lo + (tile_bytes >> 4);
          const uint32_t d0 = tmem_base + pb * 128;
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) {
            const uint64_t xd = (static_cast<uint64_t>(desc_hi) << 32) | (x_lo + 2 * k);   // 32 bytes of K per step
            const uint64_t wd = (static_cast<uint64_t>(desc_hi) << 32) | (w_lo + 2 * k);
            umma_fp8(d0, xd, wd, idesc, k > 0 ? 1u : 0u);
          }
          umma_commit(&empty[st_i]);
          umma_commit(&pfull[pb]);
        }
        __syncwarp();
        st_i += 2;
        if (st_i >= static_cast<uint32_t>(p.stages)) {
          st_i -= static_cast<uint32_t>(p.stages);
          st_ph ^= 1u;
        }
        pb ^= 2u;
        if (pb == me) pb_ph ^= 1u;
      }
      // TMEM is released only after every MMA of this warp has completed, also when a wait gave up:
      // a CTA that exits with tensor-core work in flight ends the whole launch with an error.
      if (elect_one()) {
        umma_commit(&drain[me]);
        if (!mbar_wait(&drain[me], 0)) report_error(p.err, kErrBarrierTimeout, 53, static_cast<int>(i));
      }
    }
    __syncwarp();
  } else {
    // -------------------------- promotion + epilogue --------------------------
    const int pw = warp - kRoleWarps; // 0..7
    const int q = warp & 3;          // TMEM lane quarter of this warp
    const int tok = q * 32 + lane;   // this thread's token within the chunk = its TMEM lane
    // Columns of this thread, in two halves of 32 (each loaded as 2 x 16):
    //   SwiGLU: gate features c0 .. c0+31, then the matching up features 64 + c0 ..; plain: features c0 .. c0+63.
    const int c0 = (pw >> 2) * (SWIGLU ? 32 : 64);
    const int cb = SWIGLU ? 64 + c0 : c0 + 32;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);

    uint32_t it = 0;   // K blocks done by this CTA; a multiple of four at the start of every unit when FAST
    int n = 0;
    for (int u = blockIdx.x; u < units; u += grid, ++n) {
      const int tb = n % kNumTables;
      if (!mbar_wait_warp(&sfull[tb], static_cast<uint32_t>(n / kNumTables) & 1u)) {
        report_error(p.err, kErrBarrierTimeout, 55, n);
        break;   // a promotion warp shares no barrier with the others: it may leave
      }
      const uint32_t tab_a = smem_u32(tables + tb * tab_floats);
      const int4 rec = lds_s32x4(tab_a + 2 * kbp * 4);   // {first row, end row, tile, -}
      const int row = rec.x + tok;
      const bool active = rec.x + q * 32 < rec.y;   // warp-uniform: some token of this warp exists
      bool dead = false;

      if (!active) {
        // Nothing to promote: only hand every partial buffer back as the tensor core fills it.
        for (int kb = 0; kb < p.kblocks; ++kb) {
          const uint32_t i = it + static_cast<uint32_t>(kb);
          if (!mbar_wait_warp(&pfull[i & 3u], (i >> 2) & 1u)) {
            report_error(p.err, kErrBarrierTimeout, 52, static_cast<int>(i));
            dead = true;
            break;
          }
          if (lane == 0) mbar_arrive(&pempty[i & 3u]);
        }
        if (dead) break;
        it += static_cast<uint32_t>(p.kblocks);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sempty[tb]);
        continue;
      }

      // this token's scales, one per K block (a token past the end of the array reads the last row: never stored)
      const float* xs_p = p.x_scale + static_cast<size_t>(min(row, p.total_rows - 1)) * p.kblocks;
      float4 x4n = make_float4(0.f, 0.f, 0.f, 0.f);
      if (FAST) x4n = ldg_f32x4(xs_p);
      const uint32_t ws_a = tab_a;                  // weight-block scales: [kb] gate or plain rows, [kbp + kb] up rows
      // per-row words of the plain epilogue, fetched before the K loop
      float wgt = 1.f;
      int orow = row;
      if (!SWIGLU && row < rec.y) {
        if (p.route_w) wgt = __ldg(p.route_w + row);
        if (p.out_rows) orow = __ldg(p.out_rows + row);
      }

      unsigned long long acc_a[16], acc_b[16];   // 2 x 32 fp32 accumulators as packed pairs (FFMA2)
#pragma unroll
      for (int j = 0; j < 16; ++j) acc_a[j] = acc_b[j] = 0ull;
      // Raw products of a K block, one half of this thread's columns per register set: while the FMAs of one
      // half run, the TMEM loads of the next half (of this K block or of the next) are in flight into the other.
      uint32_t ra0[16], ra1[16], rb0[16], rb1[16];
      uint32_t par = (it >> 2) & 1u;             // FAST: phase of the partial buffers for the current four K blocks

      // Waits for the tensor core to finish K block kb (buffer s of the current four when FAST) and starts the
      // TMEM loads of the first half of this thread's columns.
      auto open_block = [&](int kb, int s, uint32_t ph) {
        const uint32_t i = it + static_cast<uint32_t>(kb);
        const uint32_t pb = FAST ? static_cast<uint32_t>(s) : (i & 3u);
        if (!FAST) ph = (i >> 2) & 1u;
        if (!mbar_wait_warp(&pfull[pb], ph)) {
          report_error(p.err, kErrBarrierTimeout, 52, static_cast<int>(i));
          dead = true;
          return;
        }
        tc_fence_after_sync();
        tmem_ld_32x16(lane_base + pb * 128 + c0, ra0);
        tmem_ld_32x16(lane_base + pb * 128 + c0 + 16, ra1);
      };
      // One K block: first half (ra) while the second half loads, then the second half (rb) while the first half
      // of the next K block loads; the partial buffer goes back to the tensor core as soon as both halves have
      // landed.
      auto block = [&](float xsv, int kb, int s, bool has_next, int s_next, uint32_t ph_next) {
        const uint32_t pb = FAST ? static_cast<uint32_t>(s) : ((it + static_cast<uint32_t>(kb)) & 3u);
        const float sa = xsv * lds_f32(ws_a + kb * 4);
        const float sb = SWIGLU ? xsv * lds_f32(ws_a + (kbp + kb) * 4) : sa;
        const unsigned long long sa2 = pack_f32x2(sa, sa), sb2 = pack_f32x2(sb, sb);
        // the second half joins the first in flight; once both have landed the buffer goes back
        tmem_ld_32x16(lane_base + pb * 128 + cb, rb0);
        tmem_ld_32x16(lane_base + pb * 128 + cb + 16, rb1);
        tmem_ld_wait_regs(ra0, ra1);
        tmem_ld_wait_regs(rb0, rb1);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[pb]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          fma_f32x2(acc_a[j], pack_f32x2(__uint_as_float(ra0[2 * j]), __uint_as_float(ra0[2 * j + 1])), sa2);
          fma_f32x2(acc_a[8 + j], pack_f32x2(__uint_as_float(ra1[2 * j]), __uint_as_float(ra1[2 * j + 1])), sa2);
        }
        if (has_next) open_block(kb + 1, s_next, ph_next);   // the first half of the next K block loads during the FMAs below
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          fma_f32x2(acc_b[j], pack_f32x2(__uint_as_float(rb0[2 * j]), __uint_as_float(rb0[2 * j + 1])), sb2);
          fma_f32x2(acc_b[8 + j], pack_f32x2(__uint_as_float(rb1[2 * j]), __uint_as_float(rb1[2 * j + 1])), sb2);
        }
      };

      open_block(0, 0, par);
      for (int kb4 = 0; kb4 < p.kblocks && !dead; kb4 += 4) {
        float4 x4 = x4n;   // this token's scales of the four K blocks; the next four are fetched now
        if (FAST) {
          if (kb4 + 4 < p.kblocks) x4n = ldg_f32x4(xs_p + kb4 + 4);
        } else {
          x4.x = __ldg(xs_p + kb4);
          if (kb4 + 1 < p.kblocks) x4.y = __ldg(xs_p + kb4 + 1);
          if (kb4 + 2 < p.kblocks) x4.z = __ldg(xs_p + kb4 + 2);
          if (kb4 + 3 < p.kblocks) x4.w = __ldg(xs_p + kb4 + 3);
        }
        block(x4.x, kb4, 0, FAST || kb4 + 1 < p.kblocks, 1, par);
        if ((!FAST && kb4 + 1 >= p.kblocks) || dead) break;
        block(x4.y, kb4 + 1, 1, FAST || kb4 + 2 < p.kblocks, 2, par);
        if ((!FAST && kb4 + 2 >= p.kblocks) || dead) break;
        block(x4.z, kb4 + 2, 2, FAST || kb4 + 3 < p.kblocks, 3, par);
        if ((!FAST && kb4 + 3 >= p.kblocks) || dead) break;
        par ^= 1u;   // the next four K blocks run in the other phase of the partial buffers
        block(x4.w, kb4 + 3, 3, kb4 + 4 < p.kblocks, 0, par);
      }
      if (dead) break;   // nothing of this warp is in flight: a failed wait comes before the loads it guards
      it += static_cast<uint32_t>(p.kblocks);
      __syncwarp();
      if (lane == 0) mbar_arrive(&sempty[tb]);   // this warp is done with the unit's table

      const bool store = row < rec.y;
      const int tile = rec.z;
      if constexpr (SWIGLU) {
        if (store) {
          uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(row) * p.n_out + tile * 64 + c0);
#pragma unroll
          for (int v = 0; v < 4; ++v) {   // 8 features per 16-byte store
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float g0, g1, u0, u1;
              unpack_f32x2(acc_a[4 * v + j], g0, g1);
              unpack_f32x2(acc_b[4 * v + j], u0, u1);
              o[j] = pack_bf16x2(__fdividef(g0, 1.f + __expf(-g0)) * u0, __fdividef(g1, 1.f + __expf(-g1)) * u1);
            }
            dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      } else {
        if (store && orow >= 0 && orow < p.total_rows) {   // e.g. back to the order the rows arrived in
          uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(orow) * p.n_out + tile * 128 + c0);
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float f0, f1;
              unpack_f32x2(v < 4 ? acc_a[4 * v + j] : acc_b[4 * (v - 4) + j], f0, f1);
              o[j] = pack_bf16x2(f0 * wgt, f1 * wgt);
            }
            dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, tmem_cols);
}

}  // namespace

// swiglu = 1: w rows per expert = 2 * n_out (gate rows then up rows), out = bf16(silu(g) * u) [rows, n_out];
// swiglu = 0: w rows per expert = n_out, out[out_rows ? out_rows[row] : row] = bf16(acc * route_w[row]).
// w: fp8 [experts * w_rows_per_expert, k] K-major; w_scale [experts][w_rows_per_expert/128][k/128];
// x: fp8 [rows, k]; x_scale [rows][k/128]; offsets int32 [experts + 1] (device).
int moe_gemm_fp8_launch(int swiglu, const void* w, const float* w_scale, int experts, int w_rows_per_expert,
                        int n_out, int k, const void* x, const float* x_scale, const int32_t* offsets,
                        int total_rows, const float* route_w, const int32_t* out_rows, void* out, int* err,
                        cudaStream_t stream) {
  PTO_REQUIRE(w && w_scale && x && x_scale && offsets && out, "moe_gemm: NULL tensor");
  PTO_REQUIRE(experts > 0 && experts <= 4096, "moe_gemm: 1..4096 experts");
  PTO_REQUIRE(k > 0 && k % 128 == 0 && k <= kMoeMaxKBlocks * 128, "moe_gemm: K must be a multiple of 128, at most 8192");
  PTO_REQUIRE(n_out > 0 && n_out % 128 == 0, "moe_gemm: output features must be a multiple of 128");
  PTO_REQUIRE(w_rows_per_expert == (swiglu ? 2 * n_out : n_out), "moe_gemm: weight rows per expert mismatch");
  PTO_REQUIRE(!(swiglu && out_rows), "moe_gemm: an output row map applies to the plain mode only");
  PTO_REQUIRE(reinterpret_cast<uintptr_t>(out) % 16 == 0, "moe_gemm: out must be 16-byte aligned");
  if (total_rows <= 0) return kOk;
  MoeGemmParams p;
  p.offsets = offsets; p.experts = experts; p.kblocks = k / 128; p.n_out = n_out;
  p.n_tiles = swiglu ? n_out / 64 : n_out / 128;
  p.w_rows_per_expert = w_rows_per_expert; p.up_row_off = swiglu ? n_out : 0;
  p.w_scale = w_scale; p.x_scale = x_scale; p.route_w = route_w; p.out_rows = out_rows;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.total_rows = total_rows; p.err = err;
  const size_t stage_bytes = static_cast<size_t>(2) * 128 * 128;
  const size_t fixed = 1024 + sizeof(float) * static_cast<size_t>(kNumTables) * table_floats(p.kblocks) +
                       sizeof(int) * 2 * (experts + 2) +
                       8 * (2 * kMoeMaxStages + 2 * kNumPartial + 2 * kNumTables + 2) + 16;
  int stages = static_cast<int>((227 * 1024 - fixed) / stage_bytes);
  if (stages > kMoeMaxStages) stages = kMoeMaxStages;
  // The two producers (and the two issuers) take alternate K blocks.  With an even number of stages every stage
  // belongs to one producer and one issuer, so each stage is an ordinary in-order ring.  With an odd number a
  // stage alternates between the two producers, and a producer that is ten K blocks ahead of a lagging issuer
  // would find the stage's `empty` barrier in a phase of the parity it waits for (zero completed phases look
  // like two) and overwrite operands that have not been consumed.
  stages &= ~1;
  PTO_REQUIRE(stages >= 2, "moe_gemm: shared memory does not fit two pipeline stages");
  p.stages = stages;
  const size_t smem = fixed + stages * stage_bytes;

  CUtensorMap tm_w, tm_x;
  int st = make_tensor_map_2d(&tm_w, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1,
                              static_cast<uint64_t>(experts) * w_rows_per_expert, k, k, 128, swiglu ? 64 : 128,
                              CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_x, x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, total_rows, k, k, 128, kTN,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  // Scales move in 16-byte units when K blocks come in fours and the arrays are aligned.
  const bool fast = p.kblocks % 4 == 0 && reinterpret_cast<uintptr_t>(x_scale) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(w_scale) % 16 == 0;
  if (first_use_on_device(1)) {
    PTO_CUDA(cudaFuncSetAttribute(moe_gemm_fp8_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    PTO_CUDA(cudaFuncSetAttribute(moe_gemm_fp8_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    PTO_CUDA(cudaFuncSetAttribute(moe_gemm_fp8_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    PTO_CUDA(cudaFuncSetAttribute(moe_gemm_fp8_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  }
  const dim3 g(sm_count()), b(kMoeThreads);
  if (swiglu && fast) launch_kernel(moe_gemm_fp8_kernel<true, true>, g, b, smem, stream, tm_w, tm_x, p);
  else if (swiglu) launch_kernel(moe_gemm_fp8_kernel<true, false>, g, b, smem, stream, tm_w, tm_x, p);
  else if (fast) launch_kernel(moe_gemm_fp8_kernel<false, true>, g, b, smem, stream, tm_w, tm_x, p);
  else launch_kernel(moe_gemm_fp8_kernel<false, false>, g, b, smem, stream, tm_w, tm_x, p);
  return check_cuda(cudaGetLastError(), "moe_gemm_fp8_kernel launch");
}

}  // namespace pto
