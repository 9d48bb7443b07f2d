// SwiGLU FFN for a decode-sized batch (at most 128 rows) in ONE launch:
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
//            one MMA of N = 64; the epilogue writes bf16(silu(g) * u) to the activation buffer (stays in L2) and
//            publishes it: fence, then one atomic increment of the counter of its 64-feature slab.
//   phase 2  stream-K over (128 output features, 64-wide K block of the activation): every CTA takes an equal
//            run of K blocks, weights on the TMEM lanes, tokens as MMA N; before it loads an activation block it
//            waits (bounded) for the slab's counter; partial sums meet in `out` through red.global.add.f32.
//
// The producer warp runs ahead: the down-projection weights of a CTA's run are already in shared memory while
// the grid finishes phase 1.  The slab counters live in the first 8 KB of the workspace and start every call at
// zero: the last CTA to leave clears the ones the call used, so no launch is needed to reset anything.
#include "common.cuh"
#include "kernels.h"

namespace pto {
namespace {

constexpr int kFfThreads = 192;          // warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue
constexpr int kFfStages = 6;
constexpr int kFfStageBytes = 32 * 1024; // one 64-wide K atom: 16 KB of the lane operand + up to 16 KB of the other
constexpr int kFfBn1 = 32;               // phase 1: features per tile (gate 32 | up 32 -> MMA N = 64)
constexpr int kFfHeaderInts = 64;        // workspace header: [1] CTAs that have left; slab counters follow
constexpr size_t kFfHeaderBytes = 8192;  // header + counters; the activation starts here

struct FfnParams {
  int m, k, inter, n_out, ntok;          // ntok: MMA N of phase 2 (tokens rounded up to 32 / 64 / 128)
  int tiles1, kblocks1;                  // phase 1: inter / 32 tiles, ceil(k / 64) K blocks each
  int tiles2, kblocks2, iters2, iters2_per_cta;   // phase 2: ceil(n_out / 128) tiles x inter / 64 K blocks
  __nv_bfloat16* act;                    // [128, inter]
  int* header;                           // kFfHeaderInts ints, then inter / 64 slab counters
  float* out;                            // [m, n_out]
  int* err;
};

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until *p - target >= 0 (counters wrap; the difference does not).
__device__ __forceinline__ bool wait_counter(const int* p, int target) {
  if (ld_acquire(p) - target >= 0) return true;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (ld_acquire(p) - target >= 0) return true;
    if (global_timer_ns() - t0 > kWaitTimeoutNs) return false;
  }
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  // sigmoid as recip(1 + exp(-g)), the form of examples/models/01_ffn.py:66-77
  return g * (1.f / (1.f + __expf(-g))) * u;
}

__global__ void __launch_bounds__(kFfThreads, 1)
ffn_fused_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gu,
                 const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_d,
                 const FfnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kFfStages * kFfStageBytes);
  uint64_t* empty = full + kFfStages;
  uint64_t* tmem_full = empty + kFfStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* drain = tmem_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t tmem_cols = 256;   // two accumulator buffers of 128 columns (phase 1 uses 64 of them)

  if (threadIdx.x == 0) {
    for (int i = 0; i < kFfStages; ++i) {
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
  constexpr int kTilesPerSlab = 64 / kFfBn1;      // phase-1 tiles that make one 64-feature slab
  constexpr int slab_target = kTilesPerSlab;

  // this CTA's phase-2 run of (tile, K block) iterations
  const int it2_lo = min(p.iters2, static_cast<int>(blockIdx.x) * p.iters2_per_cta);
  const int it2_hi = min(p.iters2, it2_lo + p.iters2_per_cta);
  const uint32_t a1_bytes = 128 * 128, b1_bytes = 2 * kFfBn1 * 128;            // x tile, gate | up tiles
  const uint32_t a2_bytes = 128 * 128, b2_bytes = static_cast<uint32_t>(p.ntok) * 128;   // Wd tile, activation tile

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.tiles1 && ok; tile += gridDim.x) {
        for (int kb = 0; kb < p.kblocks1; ++kb, ++it) {
          const uint32_t s = it % kFfStages, round = it / kFfStages;
          if (!mbar_spin_wait(&empty[s], (round & 1u) ^ 1u)) {
            report_error(p.err, kErrBarrierTimeout, 80, static_cast<int>(it));
            ok = false;
            break;
          }
          uint8_t* st = smem + static_cast<size_t>(s) * kFfStageBytes;
          mbar_arrive_expect_tx(&full[s], a1_bytes + b1_bytes);
          tma_load_2d(st, &tm_x, kb * 64, 0, &full[s]);                                   // rows past m: zeros
          tma_load_2d(st + a1_bytes, &tm_gu, kb * 64, tile * kFfBn1, &full[s]);            // gate rows
          tma_load_2d(st + a1_bytes + kFfBn1 * 128, &tm_gu, kb * 64, p.inter + tile * kFfBn1, &full[s]);   // up rows
        }
      }
      // Phase 2 in windows of kFfStages iterations: first every weight tile of the window (they do not depend on
      // phase 1, so they stream in while the grid finishes it), then, slab by slab, the activation tiles.
      for (int w0 = it2_lo; w0 < it2_hi && ok; w0 += kFfStages) {
        const int w1 = min(it2_hi, w0 + kFfStages);
        for (int i2 = w0; i2 < w1; ++i2) {
          const int tile = i2 / p.kblocks2, kb = i2 - tile * p.kblocks2;
          const uint32_t j = it + static_cast<uint32_t>(i2 - w0);
          const uint32_t s = j % kFfStages, round = j / kFfStages;
          if (!mbar_spin_wait(&empty[s], (round & 1u) ^ 1u)) {
            report_error(p.err, kErrBarrierTimeout, 81, static_cast<int>(j));
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[s], a2_bytes + b2_bytes);
          tma_load_2d(smem + static_cast<size_t>(s) * kFfStageBytes, &tm_d, kb * 64, tile * 128, &full[s]);
        }
        for (int i2 = w0; i2 < w1 && ok; ++i2) {
          const int kb = i2 % p.kblocks2;
          const uint32_t s = (it + static_cast<uint32_t>(i2 - w0)) % kFfStages;
          if (!wait_counter(&counters[kb], slab_target)) {
            report_error(p.err, kErrBarrierTimeout, 82, kb);
            ok = false;
            break;
          }
          // the slab was written with ordinary stores by other CTAs: order the bulk (async-proxy) read after the acquire
          asm volatile("fence.proxy.async.global;" ::: "memory");
          tma_load_2d(smem + static_cast<size_t>(s) * kFfStageBytes + a2_bytes, &tm_act, kb * 64, 0, &full[s]);
        }
        it += static_cast<uint32_t>(w1 - w0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      const uint32_t idesc1 = umma_idesc(128, 2 * kFfBn1, 1, 1);
      const uint32_t idesc2 = umma_idesc(128, static_cast<uint32_t>(p.ntok), 1, 1);
      uint32_t it = 0, ui = 0;
      bool ok = true;
      auto unit = [&](int kblocks, uint32_t b_off, uint32_t idesc) {
        const uint32_t ab = ui & 1u;
        if (!mbar_spin_wait(&tmem_empty[ab], ((ui >> 1) & 1u) ^ 1u)) {
          report_error(p.err, kErrBarrierTimeout, 83, static_cast<int>(ui));
          ok = false;
          return;
        }
        tc_fence_after_sync();
        const uint32_t d0 = tmem_base + ab * 128;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % kFfStages, round = it / kFfStages;
          if (!mbar_spin_wait(&full[s], round & 1u)) {
            report_error(p.err, kErrBarrierTimeout, 84, static_cast<int>(it));
            ok = false;
            return;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + static_cast<size_t>(s) * kFfStageBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(d0, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(a_addr + b_off + k * 32), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        umma_commit(&tmem_full[ab]);
        ++ui;
      };
      for (int tile = blockIdx.x; tile < p.tiles1 && ok; tile += gridDim.x) unit(p.kblocks1, a1_bytes, idesc1);
      for (int i2 = it2_lo; i2 < it2_hi && ok;) {          // segments of the run, cut at tile boundaries
        const int tile = i2 / p.kblocks2;
        const int seg_end = min(it2_hi, (tile + 1) * p.kblocks2);
        unit(seg_end - i2, a2_bytes, idesc2);
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
    for (int tile = blockIdx.x; tile < p.tiles1; tile += gridDim.x, ++ui) {
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
        tmem_ld_32x32(taddr + kFfBn1, u);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[ab]);
        // every one of the 128 rows is written (rows past m hold silu(0) * 0 = 0): phase 2 reads whole tiles
        __nv_bfloat16* dst = p.act + static_cast<size_t>(row) * p.inter + tile * kFfBn1;
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
        __threadfence();                           // this thread's stores are visible device-wide ...
      }
      named_bar_sync(1, 128);                      // ... for all four epilogue warps ...
      if (ok && warp == 2 && lane == 0)            // ... before the tile is counted
        atomicAdd(&counters[tile / kTilesPerSlab], 1);
    }
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
      for (int c0 = 0; c0 < p.ntok; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c0, v);
        tmem_ld_wait();
        if (feat < p.n_out) {
#pragma unroll
          for (int j = 0; j < 32; ++j)              // lanes are consecutive features: coalesced reductions
            if (c0 + j < p.m) red_add_f32(p.out + static_cast<size_t>(c0 + j) * p.n_out + feat, __uint_as_float(v[j]));
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
  __shared__ int last_to_leave;
  if (threadIdx.x == 0) {
    __threadfence();
    last_to_leave = atomicAdd(p.header + 1, 1) == static_cast<int>(gridDim.x) - 1;
  }
  __syncthreads();
  if (last_to_leave) {
    for (int i = threadIdx.x; i < p.kblocks2; i += kFfThreads) counters[i] = 0;
    if (threadIdx.x == 0) p.header[1] = 0;
  }
}

}  // namespace

size_t ffn_fused_workspace_bytes(int inter) {
  // header + slab counters, then the activation [128, inter] bf16
  return kFfHeaderBytes + static_cast<size_t>(128) * inter * 2;
}

bool ffn_fused_ok(int m, int k, int inter, int n_out) {
  return m > 0 && m <= 128 && k % 8 == 0 && inter % 64 == 0 && inter >= 64 && n_out % 4 == 0 &&
         sizeof(int) * (kFfHeaderInts + static_cast<size_t>(inter) / 64) <= kFfHeaderBytes;
}

// x bf16 [m, k] (m <= 128), w_gate_up packed [2 * inter, k] (gate rows first), w_down packed [n_out, inter],
// out fp32 [m, n_out] holding zeros or the residual.  `workspace`: ffn_fused_workspace_bytes(inter) bytes,
// 256-byte aligned, zeroed once when it is allocated and then owned by this operator (one call at a time).
int ffn_fused_launch(const void* x, const void* w_gate_up, const void* w_down, float* out, int m, int k, int inter,
                     int n_out, void* workspace, size_t workspace_bytes, int* err, cudaStream_t stream) {
  PTO_REQUIRE(x && w_gate_up && w_down && out && workspace, "ffn_fused: NULL tensor");
  PTO_REQUIRE(ffn_fused_ok(m, k, inter, n_out), "ffn_fused: m <= 128, k % 8 == 0, inter % 64 == 0, n_out % 4 == 0 required");
  PTO_REQUIRE(workspace_bytes >= ffn_fused_workspace_bytes(inter), "ffn_fused: workspace too small");
  PTO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "ffn_fused: workspace must be 256-byte aligned");
  FfnParams p;
  p.m = m; p.k = k; p.inter = inter; p.n_out = n_out;
  p.ntok = m <= 32 ? 32 : (m <= 64 ? 64 : 128);
  p.tiles1 = inter / kFfBn1;
  p.kblocks1 = (k + 63) / 64;
  p.tiles2 = (n_out + 127) / 128;
  p.kblocks2 = inter / 64;
  p.iters2 = p.tiles2 * p.kblocks2;
  const int grid = sm_count();                     // CTAs without a phase-1 tile go straight to their phase-2 run
  p.iters2_per_cta = (p.iters2 + grid - 1) / grid;
  p.header = static_cast<int*>(workspace);
  p.act = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(workspace) + kFfHeaderBytes);
  p.out = out; p.err = err;

  CUtensorMap tm_x, tm_gu, tm_act, tm_d;
  int st = make_tensor_map_2d(&tm_x, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, m, k, static_cast<uint64_t>(k) * 2, 64, 128,
                              CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_gu, w_gate_up, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(2) * inter, k,
                          static_cast<uint64_t>(k) * 2, 64, kFfBn1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_act, p.act, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 128, inter,
                          static_cast<uint64_t>(inter) * 2, 64, p.ntok, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_d, w_down, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, n_out, inter,
                          static_cast<uint64_t>(inter) * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  const size_t smem = 1024 + static_cast<size_t>(kFfStages) * kFfStageBytes + (2 * kFfStages + 5) * 8 + 16;
  if (first_use_on_device(3))
    PTO_CUDA(cudaFuncSetAttribute(ffn_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  // CTAs wait on one another (phase 2 on phase 1): a cooperative launch guarantees that all of them are resident
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kFfThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, ffn_fused_kernel, tm_x, tm_gu, tm_act, tm_d, p), "ffn_fused_kernel launch");
}

}  // namespace pto
