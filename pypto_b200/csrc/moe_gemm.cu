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
// (expert, 128-row weight tile, chunk of up to 128 tokens).  The weight tile fills the 128
// TMEM lanes (A operand), tokens are the MMA N dimension, so every weight byte of an expert
// is streamed once per token chunk -- the kernel is weight-bandwidth bound at ~128 tokens per
// expert.  Per K block the raw fp8 products land in one of four TMEM partial buffers; sixteen
// promotion warps pull them into registers (32 fp32 accumulators per thread), multiply by the
// two scales and accumulate while the tensor core fills the other buffers.
//
//   SwiGLU mode: the tile is 64 gate rows + the 64 matching up rows; the epilogue pairs them
//                through shared memory and writes bf16(silu(g) * u).  (The per-(token, 128)
//                re-quantisation for the down projection is a separate row pass.)
//   plain mode:  128 output features; epilogue = bf16(acc * route_weight[token]).
//
// CTA = 20 warps: two TMA producers and two MMA issuers (alternating K blocks), 16
// promotion/epilogue warps (4 per TMEM lane quarter, 32 token columns each).  Bounded waits.
#include "common.cuh"
#include "kernels.h"

#include <type_traits>

namespace pto {
namespace {

constexpr int kTN = 128;          // tokens per chunk = MMA N
constexpr int kPromoWarps = 16;
constexpr int kRoleWarps = 4;      // two TMA producers and two MMA issuers, alternating K blocks
constexpr int kMoeThreads = (kRoleWarps + kPromoWarps) * 32;
constexpr int kNumPartial = 4;    // TMEM partial buffers of 128 token columns
constexpr int kTabStride = kTN + 4;   // padded row of the scale table: the fill hits 8 banks, reads stay 16-byte aligned
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

__host__ __device__ inline int scale_region_floats(bool swiglu, int kblocks) {
  const int comb = (swiglu ? 2 : 1) * kblocks * kTabStride;
  const int exch = swiglu ? 64 * kTN : 0;
  return comb > exch ? comb : exch;
}

// A unit = (expert, weight tile, chunk of 128 tokens).
//   plain mode:  the tile is 128 consecutive output features.
//   SwiGLU mode: the tile is 64 gate rows (TMEM lanes 0-63) followed by the 64 matching up
//                rows (lanes 64-127); the epilogue pairs them through shared memory and
//                writes bf16(silu(g) * u) for 64 features.
template <bool SWIGLU>
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
  // comb[a][kb][kTabStride]: weight-block scale x token scale, a = 0 gate (or plain) rows, 1 up rows.
  // SwiGLU overlays the [kTN][64] exchange buffer of the epilogue on the same bytes.
  float* comb = reinterpret_cast<float*>(after);
  float* exch = comb;
  int* prefix = reinterpret_cast<int*>(comb + scale_region_floats(SWIGLU, p.kblocks)); // [experts + 1] chunk prefix
  uint64_t* full = reinterpret_cast<uint64_t*>(prefix + ((p.experts + 2) & ~1));
  uint64_t* empty = full + kMoeMaxStages;
  uint64_t* pfull = empty + kMoeMaxStages;
  uint64_t* pempty = pfull + kNumPartial;
  uint64_t* drain = pempty + kNumPartial;   // one per MMA issuer: all of its MMAs have completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t tmem_cols = kNumPartial * kTN;  // 512

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < kNumPartial; ++i) {
      mbar_init(&pfull[i], 1);
      mbar_init(&pempty[i], kPromoWarps);
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
  for (int e = threadIdx.x; e < p.experts; e += kMoeThreads) {
    const int n = p.offsets[e + 1] - p.offsets[e];
    prefix[e + 1] = n > 0 ? (n + kTN - 1) / kTN : 0;
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

  // A single thread needs several hundred cycles per K block for its barrier waits, TMA or MMA
  // issues and commits; two producers and two issuers take alternate K blocks to keep up.
  if (warp < 2) {
    // ------------------------------ TMA producers ------------------------------
    if (lane == 0) {
      const uint32_t me = static_cast<uint32_t>(warp);
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        int e, tile, chunk;
        decode(u, e, tile, chunk);
        const int row0 = p.offsets[e] + chunk * kTN;
        const int wrow = e * p.w_rows_per_expert + tile * (SWIGLU ? 64 : 128);
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          if ((it & 1u) != me) continue;
          const uint32_t s = it % p.stages, round = it / p.stages;
          if (!mbar_wait(&empty[s], (round & 1u) ^ 1u)) {
            report_error(p.err, kErrBarrierTimeout, 50, static_cast<int>(it));
            ok = false;
            break;
          }
          uint8_t* st = smem + static_cast<size_t>(s) * stage_bytes;
          mbar_arrive_expect_tx(&full[s], stage_bytes);
          if (SWIGLU) {   // two 64-row boxes: gate rows, then the matching up rows
            tma_load_2d(st, &tm_w, kb * 128, wrow, &full[s]);
            tma_load_2d(st + 64 * 128, &tm_w, kb * 128, wrow + p.up_row_off, &full[s]);
          } else {
            tma_load_2d(st, &tm_w, kb * 128, wrow, &full[s]);
          }
          tma_load_2d(st + tile_bytes, &tm_x, kb * 128, row0, &full[s]);
        }
      }
    }
  } else if (warp < kRoleWarps) {
    // ------------------------------- MMA issuers -------------------------------
    if (lane == 0) {
      const uint32_t me = static_cast<uint32_t>(warp - 2);
      const uint32_t idesc = umma_idesc(128, kTN, 0, 0);  // e4m3 x e4m3 -> fp32
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          if ((it & 1u) != me) continue;
          const uint32_t s = it % p.stages, round = it / p.stages;
          const uint32_t pb = it % kNumPartial;
          if (!mbar_wait(&full[s], round & 1u) || !mbar_wait(&pempty[pb], ((it / kNumPartial) & 1u) ^ 1u)) {
            report_error(p.err, kErrBarrierTimeout, 51, static_cast<int>(it));
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + static_cast<size_t>(s) * stage_bytes);
          const uint32_t x_addr = a_addr + tile_bytes;
          const uint32_t d0 = tmem_base + pb * kTN;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_fp8(d0, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(x_addr + k * 32), idesc, k > 0 ? 1u : 0u);
          umma_commit(&empty[s]);
          umma_commit(&pfull[pb]);
        }
      }
      // TMEM is released only after every MMA of this thread has completed, also when a wait gave up:
      // a CTA that exits with tensor-core work in flight ends the whole launch with an error.
      umma_commit(&drain[me]);
      if (!mbar_wait(&drain[me], 0)) report_error(p.err, kErrBarrierTimeout, 53, static_cast<int>(it));
    }
    __syncwarp();
  } else {
    // -------------------------- promotion + epilogue --------------------------
    const int pw = warp - kRoleWarps; // 0..15
    const int q = warp & 3;          // TMEM lane quarter of this warp
    const int col0 = (pw >> 2) * 32; // first of this warp's 32 token columns
    const int ptid = threadIdx.x - kRoleWarps * 32;
    uint32_t it = 0;
    bool dead = false;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      int e, tile, chunk;
      decode(u, e, tile, chunk);
      const int row0 = p.offsets[e] + chunk * kTN;
      const int row_end = min(p.offsets[e + 1], p.total_rows);
      named_bar_sync(1, kPromoWarps * 32);  // previous unit's scales / exchange buffer no longer in use
      {
        // the chunk's token scales are one contiguous run of x_scale: row-major [token][kb]
        const int valid = max(0, min(row_end - row0, kTN)) * p.kblocks;
        const float* xsrc = p.x_scale + static_cast<size_t>(row0) * p.kblocks;
        const int wrow = e * p.w_rows_per_expert + (SWIGLU ? tile * 64 : tile * 128);
        const float* w0 = p.w_scale + static_cast<size_t>(wrow / 128) * p.kblocks;
        const float* w1 = p.w_scale + static_cast<size_t>((wrow + p.up_row_off) / 128) * p.kblocks;
        // Loads of a batch are all issued before their first use, so a batch costs one memory latency.
        const int total = kTN * p.kblocks;
        const int step_col = (kPromoWarps * 32) / p.kblocks, step_kb = (kPromoWarps * 32) % p.kblocks;
        int col = ptid / p.kblocks, kb = ptid % p.kblocks;
        auto fill = [&](auto batch_tag) {
          constexpr int kBatch = decltype(batch_tag)::value;
          for (int base = ptid; base < total; base += kBatch * kPromoWarps * 32) {
            float xv[kBatch];
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
              const int i = base + r * kPromoWarps * 32;
              xv[r] = i < valid ? __ldg(xsrc + i) : 0.f;
            }
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
              if (base + r * kPromoWarps * 32 < total) {
                const int at = kb * kTabStride + col;
                comb[at] = xv[r] * __ldg(w0 + kb);
                if (SWIGLU) comb[p.kblocks * kTabStride + at] = xv[r] * __ldg(w1 + kb);
              }
              col += step_col;
              kb += step_kb;
              if (kb >= p.kblocks) {
                kb -= p.kblocks;
                ++col;
              }
            }
          }
        };
        if (p.kblocks > 32) fill(std::integral_constant<int, 8>{});
        else fill(std::integral_constant<int, 4>{});
      }
      named_bar_sync(1, kPromoWarps * 32);
      // lanes 64-127 hold up rows; shared-space address of this warp's 32 token columns
      uint32_t xs = smem_u32(comb + ((SWIGLU && q >= 2) ? p.kblocks * kTabStride : 0) + col0);

      unsigned long long acc2[16];   // 32 fp32 accumulators as packed pairs (FFMA2)
#pragma unroll
      for (int j = 0; j < 16; ++j) acc2[j] = 0ull;

      for (int kb = 0; kb < p.kblocks && !dead; ++kb, ++it) {
        const uint32_t pb = it % kNumPartial;
        if (!mbar_wait_warp(&pfull[pb], (it / kNumPartial) & 1u)) {
          report_error(p.err, kErrBarrierTimeout, 52, static_cast<int>(it));
          dead = true;
          break;
        }
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + pb * kTN + col0;
        uint32_t v[32];
        tmem_ld_32x32(taddr, v);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[pb]);
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const ulonglong2 x4 = lds_u64x2(xs + j * 4);   // four combined scales
          fma_f32x2(acc2[j / 2], pack_f32x2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), x4.x);
          fma_f32x2(acc2[j / 2 + 1], pack_f32x2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])), x4.y);
        }
        xs += kTabStride * 4;
      }
      float acc[32];
#pragma unroll
      for (int j = 0; j < 16; ++j) unpack_f32x2(acc2[j], acc[2 * j], acc[2 * j + 1]);
      // a warp that timed out keeps walking the units so that the named barriers stay matched

      if constexpr (SWIGLU) {
        // Gate rows sit in lanes 0-63, the matching up rows in lanes 64-127.  The two threads of a feature
        // swap half of their 32 token columns through shared memory and each finishes 16 outputs.
        named_bar_sync(2, kPromoWarps * 32);   // every warp is done with the scale table under exch
        const bool is_up = q >= 2;
        const int f = (q & 1) * 32 + lane;     // feature within the tile
        float* mine = exch + col0 * 64 + f;
        if (!dead) {
          if (is_up) {
#pragma unroll
            for (int j = 0; j < 16; ++j) mine[j * 64] = acc[j];
          } else {
#pragma unroll
            for (int j = 16; j < 32; ++j) mine[j * 64] = acc[j];
          }
        }
        named_bar_sync(3 + (pw >> 2) * 2 + (q & 1), 64);   // the gate warp and the up warp of these features
        if (!dead) {
          const int feat = tile * 64 + f;
          if (is_up) {
#pragma unroll
            for (int j = 16; j < 32; ++j) {
              const int row = row0 + col0 + j;
              if (row < row_end) {
                const float g = mine[j * 64];
                p.out[static_cast<size_t>(row) * p.n_out + feat] =
                    __float2bfloat16_rn(g * (1.f / (1.f + __expf(-g))) * acc[j]);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int row = row0 + col0 + j;
              if (row < row_end) {
                const float g = acc[j];
                p.out[static_cast<size_t>(row) * p.n_out + feat] =
                    __float2bfloat16_rn(g * (1.f / (1.f + __expf(-g))) * mine[j * 64]);
              }
            }
          }
        }
      } else if (!dead) {
        const int feat = tile * 128 + q * 32 + lane;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int row = row0 + col0 + j;
          if (row < row_end) {
            const float wgt = p.route_w ? p.route_w[row] : 1.f;
            const int orow = p.out_rows ? p.out_rows[row] : row;     // e.g. back to the order the rows arrived in
            if (orow >= 0 && orow < p.total_rows)
              p.out[static_cast<size_t>(orow) * p.n_out + feat] = __float2bfloat16_rn(acc[j] * wgt);
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
  if (total_rows <= 0) return kOk;
  MoeGemmParams p;
  p.offsets = offsets; p.experts = experts; p.kblocks = k / 128; p.n_out = n_out;
  p.n_tiles = swiglu ? n_out / 64 : n_out / 128;
  p.w_rows_per_expert = w_rows_per_expert; p.up_row_off = swiglu ? n_out : 0;
  p.w_scale = w_scale; p.x_scale = x_scale; p.route_w = route_w; p.out_rows = out_rows;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.total_rows = total_rows; p.err = err;
  const size_t stage_bytes = static_cast<size_t>(2) * 128 * 128;
  const size_t fixed = 1024 + sizeof(float) * static_cast<size_t>(scale_region_floats(swiglu != 0, p.kblocks)) +
                       sizeof(int) * (experts + 2) + 8 * (2 * kMoeMaxStages + 2 * kNumPartial + 2) + 16;
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
  if (first_use_on_device(1)) {
    PTO_CUDA(cudaFuncSetAttribute(moe_gemm_fp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    PTO_CUDA(cudaFuncSetAttribute(moe_gemm_fp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  }
  if (swiglu) launch_kernel(moe_gemm_fp8_kernel<true>, dim3(sm_count()), dim3(kMoeThreads), smem, stream, tm_w, tm_x, p);
  else launch_kernel(moe_gemm_fp8_kernel<false>, dim3(sm_count()), dim3(kMoeThreads), smem, stream, tm_w, tm_x, p);
  return check_cuda(cudaGetLastError(), "moe_gemm_fp8_kernel launch");
}

}  // namespace pto
