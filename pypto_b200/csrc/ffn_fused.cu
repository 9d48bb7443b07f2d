// SwiGLU FFN for a decode-sized batch (at most 128 rows) and weights of a few tens of MB in ONE launch:
//
//   out[m, n_out] += bf16(silu(x Wg) * (x Wu)) Wd          (out holds zeros or the residual on entry)
//
// It replaces the chain gate/up GEMM -> SwiGLU -> down GEMM of examples/models/01_ffn.py:112-131 and of
// mlp_block + down_projection_residual (examples/models/qwen3_jit/kernels/mlp.py:23-61,
// kernels/projection.py:146-177), where every intermediate goes through global memory between task launches.
// At this size the step is bound by streaming 3 * k * inter weight elements once; a chain of launches pays a
// prologue, a pipeline fill and a tail per GEMM, several times the streaming time.  Here one persistent grid
// (one CTA per SM, launched cooperatively so that all CTAs are resident) runs both GEMMs:
//
//   phase 1  tile = 32 gate + 32 up features: tokens on the 128 TMEM lanes, the two weight tiles side by side as
//            one MMA of N = 64 (the finest tile the tensor core takes at M = 128: 4096 features give 128 CTAs
//            work).  The epilogue writes bf16(silu(g) * u) to the activation buffer (it stays in L2) and
//            publishes it: barrier, one fence, one release-increment of the counter of its 64-feature slab.
//   phase 2  stream-K over (128 output features, 64-wide K block of the activation), an equal run per CTA, weights
//            on the TMEM lanes, tokens as MMA N.  A CTA first streams the down-projection weights of its run into
//            the pipeline (they do not depend on phase 1), then waits (bounded) for the counters of the slabs it
//            needs, then loads activation blocks; partial sums meet in `out` through red.global.add.f32, every CTA
//            walking the tokens from a different start so that the reductions do not queue on one line.
//
// What bounds phase 1 at 128 tokens is not DRAM: every CTA needs all of x (k * 256 bytes, from L2) next to its own
// weight tile, and an SM takes in about 55 GB/s through TMA, so the phase costs (weights / CTAs + x) / 55 GB/s.
//
// The slab counters live in the first 8 KB of the workspace and start every call at zero: the last CTA to leave
// clears the ones the call used, so no launch is needed to reset anything.
#include "common.cuh"
#include "kernels.h"

namespace pto {
namespace {

constexpr int kFfThreads = 192;          // warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue
constexpr int kFfMaxStages = 12;
constexpr int kFfTile1 = 32;             // phase 1: features per tile (gate 32 | up 32 -> MMA N = 64)
constexpr int kTilesPerSlab = 64 / kFfTile1;   // phase-1 tiles that make one 64-feature slab (= one phase-2 K block)
constexpr int kFfHeaderInts = 64;        // workspace header: [1] CTAs that have left, [8..23] cast counters; slab counters follow
constexpr int kFfCastCounter0 = 8, kFfCastCounters = 16;   // header[8 .. 23]: CTAs done with their share of the cast
constexpr size_t kFfHeaderBytes = 8192;  // header + counters; the activation starts here

struct FfnParams {
  int m, k, inter, n_out, ntok;          // ntok: MMA N (tokens rounded up to 32 / 64 / 128)
  int tiles1, kblocks1;                  // phase 1: inter / 32 tiles, ceil(k / 64) K blocks each
  int tiles2, kblocks2, iters2;          // phase 2: ceil(n_out / 128) tiles x inter / 64 K blocks
  int n2_base, n2_rem;                   // phase-2 run of CTA b: n2_base (+1 for b < n2_rem) iterations
  int stages;
  uint32_t stage_bytes;
  __nv_bfloat16* act;                    // [128, inter]
  int* header;                           // kFfHeaderInts ints, then inter / 64 slab counters
  float* out;                            // [m, n_out]
  int* err;
  // fp32 input: the CTAs first cast x to bf16 (into `xb`, which the x tensor map points at) and, if asked, clear the
  // output, each its share; header[8..23] count the CTAs that are done with it
  const float* x_f32;                    // [m, k], or NULL when x is given as bf16
  __nv_bfloat16* xb;                     // [m, k] in the workspace
  int zero_out;
};

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void red_release_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  // sigmoid as recip(1 + exp(-g)), the form of examples/models/01_ffn.py:66-77 (hardware reciprocal)
  return __fdividef(g, 1.f + __expf(-g)) * u;
}

__global__ void __launch_bounds__(kFfThreads, 1)
ffn_fused_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gu,
                 const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_d,
                 const FfnParams p) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(p.stages) * p.stage_bytes);
  uint64_t* empty = full + kFfMaxStages;
  uint64_t* tmem_full = empty + kFfMaxStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* drain = tmem_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
  int* last_to_leave = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t tmem_cols = 256;   // two accumulator buffers of 128 columns (phase 1 uses 64 of them)

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);
    }
    mbar_init(drain, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_gu);
    tma_prefetch_desc(&tm_act);
    tma_prefetch_desc(&tm_d);
  }
  if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  int* counters = p.header + kFfHeaderInts;

  // this CTA's phase-1 tiles are blockIdx.x, + gridDim.x, ...; its phase-2 run of (tile, K block) iterations:
  const int b = blockIdx.x;
  const int n2 = p.n2_base + (b < p.n2_rem ? 1 : 0);
  const int it2_lo = b * p.n2_base + min(b, p.n2_rem);
  const int it2_hi = min(p.iters2, it2_lo + n2);
  const uint32_t lane_bytes = 128 * 128;                                 // operand on the lanes: x tile / Wd tile of a K block
  const uint32_t w1_bytes = 2 * kFfTile1 * 128;                          // phase 1: gate | up weight tiles of a K block
  const uint32_t t2_bytes = static_cast<uint32_t>(p.ntok) * 128;         // phase 2: activation tile of a K block
  int n1 = 0;
  for (int tile = b; tile < p.tiles1; tile += gridDim.x) n1 += p.kblocks1;   // phase-1 iterations of this CTA
  const uint32_t S = static_cast<uint32_t>(p.stages);
  auto stage_ptr = [&](uint32_t j) { return smem + static_cast<size_t>(j % S) * p.stage_bytes; };
  auto issue_w1 = [&](uint32_t j, int i1) {      // i1: phase-1 iteration of this CTA
    const int tile = b + (i1 / p.kblocks1) * static_cast<int>(gridDim.x), kb = i1 % p.kblocks1;
    uint8_t* st = stage_ptr(j) + lane_bytes;
    mbar_arrive_expect_tx(&full[j % S], lane_bytes + w1_bytes);
    tma_load_2d(st, &tm_gu, kb * 64, tile * kFfTile1, &full[j % S]);                               // gate rows
    tma_load_2d(st + kFfTile1 * 128, &tm_gu, kb * 64, p.inter + tile * kFfTile1, &full[j % S]);    // up rows
  };
  // The weights of the first stages do not depend on the kernel before this one: they are requested before the wait
  // on it (programmatic dependent launch) and before the cast of x, the activations after.
  const int first = min(n1, p.stages);
  if (threadIdx.x == 0)
    for (int i1 = 0; i1 < first; ++i1) issue_w1(static_cast<uint32_t>(i1), i1);

  if (p.x_f32 != nullptr) {
    // ---- phase 0: this CTA's share of x -> bf16 and of clearing the output ----
    pdl_wait();   // x and the output belong to the kernels before this one until here; so do the header's counters
    const long long stride = static_cast<long long>(gridDim.x) * kFfThreads;
    const long long i0 = static_cast<long long>(b) * kFfThreads + threadIdx.x;
    const long long n_x4 = static_cast<long long>(p.m) * p.k / 4;
    for (long long i = i0; i < n_x4; i += stride) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(p.x_f32) + i);
      reinterpret_cast<uint2*>(p.xb)[i] = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    }
    if (p.zero_out) {
      const long long n_o4 = static_cast<long long>(p.m) * p.n_out / 4;
      for (long long i = i0; i < n_o4; i += stride) reinterpret_cast<uint4*>(p.out)[i] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();                       // cumulative: covers the stores the barrier ordered before it
      red_release_add(p.header + kFfCastCounter0 + (b % kFfCastCounters), 1);   // spread: increments of one word queue up
    }
  }

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    uint32_t it = 0;
    bool ok = true;
    auto wait_stage = [&](uint32_t j, int site) {
      if (!mbar_spin_wait(&empty[j % S], ((j / S) & 1u) ^ 1u)) {
        report_error(p.err, kErrBarrierTimeout, site, static_cast<int>(j));
        ok = false;
      }
      return ok;
    };
    auto issue_x1 = [&](uint32_t j, int i1) {
      tma_load_2d(stage_ptr(j), &tm_x, (i1 % p.kblocks1) * 64, 0, &full[j % S]);                     // rows past m: zeros
    };
    pdl_wait();
    if (p.x_f32 != nullptr && n1 > 0) {
      // every CTA's share of the cast: x is whole once all of them have counted themselves in (lane l watches
      // counter l, which CTAs l, l + 16, ... increment)
      bool mine = true;
      if (lane < kFfCastCounters) {
        const int want = (static_cast<int>(gridDim.x) - lane + kFfCastCounters - 1) / kFfCastCounters;
        const unsigned long long t0 = global_timer_ns();
        while (ld_acquire(p.header + kFfCastCounter0 + lane) < want) {
          if (global_timer_ns() - t0 > kWaitTimeoutNs) {
            mine = false;
            break;
          }
        }
      }
      if (!__all_sync(0xffffffffu, mine)) {
        if (lane == 0) report_error(p.err, kErrBarrierTimeout, 88, 0);
        ok = false;
      }
    }
    if (lane == 0) {
      // x was written with ordinary stores by other CTAs: order the bulk (async-proxy) reads after the acquires
      if (p.x_f32 != nullptr) asm volatile("fence.proxy.async.global;" ::: "memory");
      for (int i1 = 0; i1 < first && ok; ++i1) issue_x1(it + i1, i1);
      it += first;
      for (int i1 = first; i1 < n1 && ok; ++i1, ++it) {
        if (!wait_stage(it, 80)) break;
        issue_w1(it, i1);
        issue_x1(it, i1);
      }
    }
    // Phase 2.  First window: down-projection weights into every stage that frees up, then the wait for the slabs.
    const int win = min(it2_hi - it2_lo, p.stages);
    if (lane == 0 && ok) {
      for (int i = 0; i < win && ok; ++i) {
        const int i2 = it2_lo + i, tile = i2 / p.kblocks2, kb = i2 - tile * p.kblocks2;
        if (!wait_stage(it + i, 81)) break;
        mbar_arrive_expect_tx(&full[(it + i) % S], lane_bytes + t2_bytes);
        tma_load_2d(stage_ptr(it + i), &tm_d, kb * 64, tile * 128, &full[(it + i) % S]);
      }
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    // All lanes: wait until every slab of the run has been published (lane l polls the run's iterations l, l+32, ...).
    // Not before the kernel ahead of this one has finished: it may be a call of this operator on the same
    // workspace, whose last CTA clears the counters.
    pdl_wait();
    if (ok) {
      bool mine = true;
      const unsigned long long t0 = global_timer_ns();
      for (int i2 = it2_lo + lane; i2 < it2_hi && mine; i2 += 32) {
        const int* c = &counters[i2 % p.kblocks2];
        while (ld_acquire(c) < kTilesPerSlab) {
          if (global_timer_ns() - t0 > kWaitTimeoutNs) {
            mine = false;
            break;
          }
        }
      }
      if (!__all_sync(0xffffffffu, mine)) {
        if (lane == 0) report_error(p.err, kErrBarrierTimeout, 82, it2_lo);
        ok = false;
      }
    }
    if (lane == 0 && ok) {
      // the slabs were written with ordinary stores by other CTAs: order the bulk (async-proxy) reads after the acquires
      asm volatile("fence.proxy.async.global;" ::: "memory");
      for (int i = 0; i < win; ++i)
        tma_load_2d(stage_ptr(it + i) + lane_bytes, &tm_act, ((it2_lo + i) % p.kblocks2) * 64, 0, &full[(it + i) % S]);
      it += win;
      for (int i2 = it2_lo + win; i2 < it2_hi && ok; ++i2, ++it) {
        const int tile = i2 / p.kblocks2, kb = i2 - tile * p.kblocks2;
        if (!wait_stage(it, 81)) break;
        mbar_arrive_expect_tx(&full[it % S], lane_bytes + t2_bytes);
        tma_load_2d(stage_ptr(it), &tm_d, kb * 64, tile * 128, &full[it % S]);
        tma_load_2d(stage_ptr(it) + lane_bytes, &tm_act, kb * 64, 0, &full[it % S]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      const uint32_t idesc1 = umma_idesc(128, 2 * kFfTile1, 1, 1);
      const uint32_t idesc2 = umma_idesc(128, static_cast<uint32_t>(p.ntok), 1, 1);
      const uint32_t S = static_cast<uint32_t>(p.stages);
      uint32_t it = 0, ui = 0;
      bool ok = true;
      auto unit = [&](int kblocks, uint32_t idesc) {
        const uint32_t ab = ui & 1u;
        if (!mbar_spin_wait(&tmem_empty[ab], ((ui >> 1) & 1u) ^ 1u)) {
          report_error(p.err, kErrBarrierTimeout, 83, static_cast<int>(ui));
          ok = false;
          return;
        }
        tc_fence_after_sync();
        const uint32_t d0 = tmem_base + ab * 128;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % S, round = it / S;
          if (!mbar_spin_wait(&full[s], round & 1u)) {
            report_error(p.err, kErrBarrierTimeout, 84, static_cast<int>(it));
            ok = false;
            return;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + static_cast<size_t>(s) * p.stage_bytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(d0, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(a_addr + lane_bytes + k * 32), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        umma_commit(&tmem_full[ab]);
        ++ui;
      };
      for (int tile = b; tile < p.tiles1 && ok; tile += gridDim.x) unit(p.kblocks1, idesc1);
      for (int i2 = it2_lo; i2 < it2_hi && ok;) {          // segments of the run, cut at tile boundaries
        const int seg_end = min(it2_hi, (i2 / p.kblocks2 + 1) * p.kblocks2);
        unit(seg_end - i2, idesc2);
        i2 = seg_end;
      }
      umma_commit(drain);   // tensor memory is released only after every MMA has completed
      if (!mbar_wait(drain, 0)) report_error(p.err, kErrBarrierTimeout, 85, static_cast<int>(it));
    }
    __syncwarp();
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;               // phase 1: token; phase 2: output feature within the tile
    uint32_t ui = 0;
    bool ok = true;
    pdl_wait();                                  // before the first global write
    for (int tile = b; tile < p.tiles1; tile += gridDim.x, ++ui) {
      const uint32_t ab = ui & 1u;
      if (ok && !mbar_wait_warp(&tmem_full[ab], (ui >> 1) & 1u)) {
        report_error(p.err, kErrBarrierTimeout, 86, static_cast<int>(ui));
        ok = false;
      }
      if (ok) {
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * 128;
        uint32_t g[32], u[32];
        tmem_ld_32x32(taddr, g);
        tmem_ld_32x32(taddr + kFfTile1, u);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[ab]);
        // every one of the 128 rows is written (rows past m hold silu(0) * 0 = 0): phase 2 reads whole tiles
        __nv_bfloat16* dst = p.act + static_cast<size_t>(row) * p.inter + tile * kFfTile1;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 pk;
          pk.x = pack_bf16x2(silu_mul(__uint_as_float(g[j]), __uint_as_float(u[j])),
                             silu_mul(__uint_as_float(g[j + 1]), __uint_as_float(u[j + 1])));
          pk.y = pack_bf16x2(silu_mul(__uint_as_float(g[j + 2]), __uint_as_float(u[j + 2])),
                             silu_mul(__uint_as_float(g[j + 3]), __uint_as_float(u[j + 3])));
          pk.z = pack_bf16x2(silu_mul(__uint_as_float(g[j + 4]), __uint_as_float(u[j + 4])),
                             silu_mul(__uint_as_float(g[j + 5]), __uint_as_float(u[j + 5])));
          pk.w = pack_bf16x2(silu_mul(__uint_as_float(g[j + 6]), __uint_as_float(u[j + 6])),
                             silu_mul(__uint_as_float(g[j + 7]), __uint_as_float(u[j + 7])));
          *reinterpret_cast<uint4*>(dst + j) = pk;
        }
      }
      named_bar_sync(1, 128);                      // the tile is written by all four epilogue warps
      if (ok && warp == 2 && lane == 0) {
        __threadfence();                           // cumulative: covers the stores the barrier ordered before it
        red_release_add(&counters[tile / kTilesPerSlab], 1);
      }
    }
    const int tok0 = (b * 32) % p.ntok;          // every CTA starts its walk over the tokens elsewhere
    for (int i2 = it2_lo; i2 < it2_hi && ok; ++ui) {
      const int tile = i2 / p.kblocks2;
      i2 = min(it2_hi, (tile + 1) * p.kblocks2);
      const uint32_t ab = ui & 1u;
      if (!mbar_wait_warp(&tmem_full[ab], (ui >> 1) & 1u)) {
        report_error(p.err, kErrBarrierTimeout, 87, static_cast<int>(ui));
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * 128;
      const int feat = tile * 128 + row;
      for (int cc = 0; cc < p.ntok; cc += 32) {
        const int c0 = (tok0 + cc) % p.ntok;
        uint32_t v[32];
        tmem_ld_32x32(taddr + c0, v);
        tmem_ld_wait();
        if (feat < p.n_out) {
          // lanes are consecutive features: coalesced reductions.  The CTAs that share an output tile start at
          // different tokens (tok0 above, and the group of eight below), so they do not queue on one line.
          auto reduce8 = [&](int j0) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (c0 + j0 + j < p.m)
                red_add_f32(p.out + static_cast<size_t>(c0 + j0 + j) * p.n_out + feat, __uint_as_float(v[j0 + j]));
          };
          const int rot = (b >> 2) & 3;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            switch ((g + rot) & 3) {
              case 0: reduce8(0); break;
              case 1: reduce8(8); break;
              case 2: reduce8(16); break;
              default: reduce8(24); break;
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[ab]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
  // The last CTA to leave clears the counters for the next call: by then every CTA is past its last wait.
  if (threadIdx.x == 0) {
    __threadfence();
    *last_to_leave = atomicAdd(p.header + 1, 1) == static_cast<int>(gridDim.x) - 1;
  }
  __syncthreads();
  if (*last_to_leave) {
    for (int i = threadIdx.x; i < p.kblocks2; i += kFfThreads) counters[i] = 0;
    if (threadIdx.x == 0) p.header[1] = 0;
    if (threadIdx.x < kFfCastCounters) p.header[kFfCastCounter0 + threadIdx.x] = 0;
  }
}

}  // namespace

size_t ffn_fused_workspace_bytes(int inter) {
  // header + slab counters, then the activation [128, inter] bf16
  return kFfHeaderBytes + static_cast<size_t>(128) * inter * 2;
}

bool ffn_fused_ok(int m, int k, int inter, int n_out) {
  // Worth it while prologues and pipeline fills of a launch chain weigh more than this kernel's re-reading of x
  // by every CTA: weights of a few tens of MB.  Larger FFNs keep the chain of stream-K GEMMs.
  const size_t weight_bytes = (static_cast<size_t>(2) * inter * k + static_cast<size_t>(n_out) * inter) * 2;
  return m > 0 && m <= 128 && k % 8 == 0 && inter % 64 == 0 && inter >= 64 && n_out % 4 == 0 &&
         weight_bytes <= (static_cast<size_t>(64) << 20) &&
         sizeof(int) * (kFfHeaderInts + static_cast<size_t>(inter) / 64) <= kFfHeaderBytes;
}

// x bf16 [m, k] (m <= 128), w_gate_up packed [2 * inter, k] (gate rows first), w_down packed [n_out, inter],
// out fp32 [m, n_out] holding zeros or the residual.  `workspace`: ffn_fused_workspace_bytes(inter) bytes,
// 256-byte aligned, zeroed once when it is allocated and then owned by this operator (one call at a time).
// x_f32 (fp32 [m, k], 16-byte aligned) instead of x: the kernel casts it itself into `xb` (bf16 [m, k], 16-byte
// aligned, not part of the workspace above) and clears `out` first when zero_out is set.
int ffn_fused_launch(const void* x, const void* w_gate_up, const void* w_down, float* out, int m, int k, int inter,
                     int n_out, void* workspace, size_t workspace_bytes, int* err, cudaStream_t stream,
                     const float* x_f32, void* xb, int zero_out) {
  PTO_REQUIRE((x || (x_f32 && xb)) && w_gate_up && w_down && out && workspace, "ffn_fused: NULL tensor");
  if (x_f32) {
    PTO_REQUIRE(((reinterpret_cast<uintptr_t>(x_f32) | reinterpret_cast<uintptr_t>(xb) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
                "ffn_fused: fp32 x, its bf16 copy and the output must be 16-byte aligned");
    x = xb;
  }
  PTO_REQUIRE(ffn_fused_ok(m, k, inter, n_out), "ffn_fused: m <= 128, k % 8 == 0, inter % 64 == 0, n_out % 4 == 0 required");
  PTO_REQUIRE(workspace_bytes >= ffn_fused_workspace_bytes(inter), "ffn_fused: workspace too small");
  PTO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "ffn_fused: workspace must be 256-byte aligned");
  const int grid = sm_count();
  FfnParams p;
  p.m = m; p.k = k; p.inter = inter; p.n_out = n_out;
  p.ntok = m <= 32 ? 32 : (m <= 64 ? 64 : 128);
  p.tiles1 = inter / kFfTile1;
  p.kblocks1 = (k + 63) / 64;
  p.tiles2 = (n_out + 127) / 128;
  p.kblocks2 = inter / 64;
  p.iters2 = p.tiles2 * p.kblocks2;
  p.n2_base = p.iters2 / grid;
  p.n2_rem = p.iters2 % grid;
  // a stage holds a phase-1 K block (x tile 16 KB + gate | up tiles 8 KB) or a phase-2 one (Wd tile 16 KB + activation)
  p.stage_bytes = 128 * 128 + (p.ntok * 128 > 2 * kFfTile1 * 128 ? static_cast<uint32_t>(p.ntok) * 128 : 2 * kFfTile1 * 128);
  const size_t fixed = 1024 + (2 * kFfMaxStages + 5) * 8 + 16;
  int stages = static_cast<int>((227 * 1024 - fixed) / p.stage_bytes);
  if (stages > kFfMaxStages) stages = kFfMaxStages;
  p.stages = stages;
  p.header = static_cast<int*>(workspace);
  p.act = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(workspace) + kFfHeaderBytes);
  p.out = out; p.err = err;
  p.x_f32 = x_f32; p.xb = static_cast<__nv_bfloat16*>(xb); p.zero_out = zero_out;

  CUtensorMap tm_x, tm_gu, tm_act, tm_d;
  int st = make_tensor_map_2d(&tm_x, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, m, k, static_cast<uint64_t>(k) * 2, 64,
                              128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_gu, w_gate_up, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(2) * inter, k,
                          static_cast<uint64_t>(k) * 2, 64, kFfTile1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_act, p.act, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 128, inter,
                          static_cast<uint64_t>(inter) * 2, 64, p.ntok, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_d, w_down, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, n_out, inter,
                          static_cast<uint64_t>(inter) * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  const size_t smem = fixed + static_cast<size_t>(stages) * p.stage_bytes;
  if (first_use_on_device(3))
    PTO_CUDA(cudaFuncSetAttribute(ffn_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  // CTAs wait on one another (phase 2 on phase 1): a cooperative launch guarantees that all of them are resident.
  // Programmatic dependent launch lets the prologue and the first weight requests overlap the kernel before.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kFfThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static bool pdl_with_cooperative = pdl_enabled();
  cfg.numAttrs = pdl_with_cooperative ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, ffn_fused_kernel, tm_x, tm_gu, tm_act, tm_d, p);
  if (e != cudaSuccess && pdl_with_cooperative) {
    // a driver that does not take both attributes together: cooperative alone (the kernel's waits on the previous
    // kernel then return at once)
    (void)cudaGetLastError();
    pdl_with_cooperative = false;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, ffn_fused_kernel, tm_x, tm_gu, tm_act, tm_d, p);
  }
  return check_cuda(e, "ffn_fused_kernel launch");
}

}  // namespace pto
