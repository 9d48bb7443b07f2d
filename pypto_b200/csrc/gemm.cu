// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM,
// operands staged by TMA), with the epilogues the fused operators need.
//
//   D[a_row, b_row] = sum_k A[a_row, k] * B[b_row, k]        (both operands K-major bf16)
//
// It stands where the reference runs `matmul_kernel` / `pl.matmul` tiles with every
// intermediate written back to global memory (examples/models/01_ffn.py:37-45, 112-131;
// examples/models/qwen3_jit/kernels/projection.py:36-177, kernels/mlp.py:23-61): fp32
// accumulation of bf16 operands, the rule of python/pypto/debug/torch_codegen.py:1078-1086.
//
// Orientation.  TMEM lanes hold A rows (128 per tile), TMEM columns hold B rows (bn per
// tile).  For a prefill-sized activation matrix A = activations, B = weights [N, K].
// For decode (a few dozen tokens) the operands are swapped: A = weights, so that the 128
// lanes are filled by output features and the token count becomes the small N of the
// MMA; the output is then written transposed (`swap`).
//
// Work split.  The (tile, K block) iterations of the whole problem form one index space
// that is cut into equal contiguous ranges, one per persistent CTA (stream-K): every CTA
// streams the same number of operand bytes.  A maximal run of K blocks of one tile inside
// a range is a segment; with the atomic epilogue a segment adds its partial sums to the
// output with red.global.add.f32 (the output is initialised by the caller: zeros, or the
// residual that the reference adds after the projection).  The other epilogues need whole
// tiles, so ranges are then rounded to tile boundaries.
//
// CTA = 6 warps: warp 0 TMA producer, warp 1 MMA issuer (owns the TMEM allocation),
// warps 2-5 epilogue (TMEM -> registers -> global).  smem ring of (A, B[, B2]) stages with
// full/empty mbarriers; two TMEM accumulator buffers so that the epilogue of unit i
// overlaps the main loop of unit i+1.  All waits are bounded.
#include "common.cuh"
#include "kernels.h"

namespace pto {
namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;  // bf16 elements per stage row = 128 bytes = one swizzle atom
constexpr int kGemmThreads = 192;
constexpr int kMaxStages = 12;

struct GemmParams {
  int a_rows, b_rows, k;
  int a_tiles, b_tiles, kblocks_total;
  int iters_total, iters_per_cta;  // (tile, K block) iterations; per CTA a multiple of kblocks_total unless atomic
  int bn;
  int dual, dual_off;  // SwiGLU: second B tile (up weights) at row offset dual_off
  int swap;            // out[b_row * ldo + a_row] instead of out[a_row * ldo + b_row]
  int epi;             // GemmEpi
  int out_bf16;
  int stages;
  int katoms;          // 64-wide K atoms per pipeline stage (2 amortises the per-stage barrier traffic)
  int mt;              // 128-row A tiles per CTA tile (2: a 256-row tile halves the B traffic per FLOP)
  int nbuf;            // TMEM accumulator buffers (2 = epilogue overlaps the next main loop)
  void* out;
  long long ldo;
  int* err;
};

__device__ __forceinline__ float silu_mul(float g, float u) {
  // sigmoid as recip(1 + exp(-g)), the form of examples/models/01_ffn.py:66-77
  // (approximate quotient, 2 ulp: an IEEE division costs a dozen instructions per element and made the epilogue of
  // short-K tiles longer than their MMAs)
  return __fdividef(g, 1.f + __expf(-g)) * u;
}

// Segment walk shared by the three roles: iterations [lo, hi) of this CTA, cut at tile
// boundaries.
struct Seg {
  int tile, kb0, kb1;
};
// stride == 0: contiguous iteration range [it, hi) (stream-K).  stride > 0: whole tiles
// it, it + stride, ... below hi, so that CTAs running at the same time work on
// neighbouring tiles and share operand tiles in L2.
__device__ __forceinline__ bool next_seg(int& it, int hi, int kblocks, int stride, Seg& s) {
  if (it >= hi) return false;
  if (stride > 0) {
    s.tile = it;
    s.kb0 = 0;
    s.kb1 = kblocks;
    it += stride;
    return true;
  }
  s.tile = it / kblocks;
  s.kb0 = it - s.tile * kblocks;
  const int len = min(kblocks - s.kb0, hi - it);
  s.kb1 = s.kb0 + len;
  it += len;
  return true;
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const GemmParams p) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int nacc = p.dual ? 2 : 1;
  const uint32_t a_atom = p.mt * kBM * 128, b_atom = nacc * p.bn * 128;   // one 64-wide K atom of A / of B (gate|up)
  const uint32_t a_bytes = p.katoms * a_atom;
  const uint32_t b_bytes = p.bn * 128;
  const uint32_t stage_bytes = a_bytes + p.katoms * b_atom;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(p.stages) * stage_bytes);
  uint64_t* empty = full + kMaxStages;
  uint64_t* tmem_full = empty + kMaxStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* drain = tmem_empty + 2;   // every MMA of the issuer has completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t acc_cols = nacc * p.bn;                // columns of one 128-row accumulator
  const uint32_t buf_cols = p.mt * acc_cols;            // columns of one accumulator buffer
  uint32_t tmem_cols = 32;
  while (tmem_cols < p.nbuf * buf_cols) tmem_cols <<= 1;

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
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // the prologue above overlaps the previous kernel; operands and outputs are touched below
  const bool stream_k = p.epi == kGemmEpiAtomic;
  const int stride = stream_k ? 0 : static_cast<int>(gridDim.x);
  const int it_lo = stream_k ? min(p.iters_total, static_cast<int>(blockIdx.x) * p.iters_per_cta)
                             : static_cast<int>(blockIdx.x);
  const int it_hi = stream_k ? min(p.iters_total, it_lo + p.iters_per_cta) : p.a_tiles * p.b_tiles;

  // The producer and the issuer are one-thread jobs whose instruction streams bound the K loop of small problems:
  // the whole warp walks the loop and waits (warp-uniform code keeps descriptors and barrier addresses in uniform
  // registers), one elected lane issues, stages and barrier phases are carried along instead of divided out, and the
  // operand descriptors advance by additions.
  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    uint32_t it = 0, s = 0, ph = 0;   // K blocks issued, stage of the next one, how often that stage was refilled (mod 2)
    bool ok = true;
    int cur = it_lo;
    Seg sg;
    while (ok && next_seg(cur, it_hi, p.kblocks_total, stride, sg)) {
      const int at = sg.tile / p.b_tiles, bt = sg.tile - at * p.b_tiles;
      for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
        if (!__all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u))) {
          if (lane == 0) report_error(p.err, kErrBarrierTimeout, 40, static_cast<int>(it));
          ok = false;
          break;
        }
        if (elect_one()) {
          uint8_t* st = smem + static_cast<size_t>(s) * stage_bytes;
          mbar_arrive_expect_tx(&full[s], stage_bytes);
          for (int a = 0; a < p.katoms; ++a) {
            const int kx = (kb * p.katoms + a) * kBK;   // past K the box is zero filled
            tma_load_2d(st + a * a_atom, &tm_a, kx, at * p.mt * kBM, &full[s]);
            tma_load_2d(st + a_bytes + a * b_atom, &tm_b, kx, bt * p.bn, &full[s]);
            if (p.dual) tma_load_2d(st + a_bytes + a * b_atom + b_bytes, &tm_b, kx, p.dual_off + bt * p.bn, &full[s]);
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
    // ------------------------------- MMA issuer -------------------------------
    const uint32_t idesc = p.dual ? umma_idesc(kBM, 2 * p.bn, 1, 1)   // gate and up tiles are adjacent in smem
                                  : umma_idesc(kBM, p.bn, 1, 1);
    const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);   // stride byte offset, version, 128-byte swizzle
    const uint32_t lo0 = ((smem_u32(smem) & 0x3FFFFu) >> 4) | (1u << 16);
    uint32_t it = 0, s = 0, ph = 0;      // K blocks issued, stage, phase of its `full` barrier
    uint32_t ab = 0, ab_ph = 1;          // accumulator buffer and the phase of `tmem_empty` to wait for (first use: free)
    bool ok = true;
    int cur = it_lo;
    Seg sg;
    while (ok && next_seg(cur, it_hi, p.kblocks_total, stride, sg)) {
      const int kb0 = sg.kb0, kb1 = sg.kb1;
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_empty[ab], ab_ph))) {
        if (lane == 0) report_error(p.err, kErrBarrierTimeout, 41, static_cast<int>(it));
        break;
      }
      tc_fence_after_sync();
      const uint32_t d0 = tmem_base + ab * buf_cols;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        if (!__all_sync(0xffffffffu, mbar_wait(&full[s], ph))) {
          if (lane == 0) report_error(p.err, kErrBarrierTimeout, 42, static_cast<int>(it));
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (elect_one()) {
          const uint32_t a_lo = lo0 + s * (stage_bytes >> 4);
          const uint32_t b_lo = a_lo + (a_bytes >> 4);
          for (int a = 0; a < p.katoms; ++a) {
#pragma unroll
            for (uint32_t k = 0; k < kBK / 16; ++k) {   // 16 bf16 = 32 bytes of K per step: the address field moves by 2
              const uint32_t acc = (kb > kb0 || a > 0 || k > 0) ? 1u : 0u;
              const uint64_t bd = (static_cast<uint64_t>(desc_hi) << 32) | (b_lo + a * (b_atom >> 4) + 2 * k);
              for (int mi = 0; mi < p.mt; ++mi) {
                const uint64_t ad = (static_cast<uint64_t>(desc_hi) << 32) |
                                    (a_lo + a * (a_atom >> 4) + mi * ((kBM * 128) >> 4) + 2 * k);
                umma_bf16(d0 + mi * acc_cols, ad, bd, idesc, acc);
              }
            }
          }
          umma_commit(&empty[s]);
        }
        __syncwarp();
        if (++s == static_cast<uint32_t>(p.stages)) {
          s = 0;
          ph ^= 1u;
        }
      }
      if (ok && elect_one()) umma_commit(&tmem_full[ab]);
      __syncwarp();
      if (p.nbuf == 2) {
        ab ^= 1u;
        if (ab == 0) ab_ph ^= 1u;
      } else {
        ab_ph ^= 1u;
      }
    }
    // TMEM is released only after every MMA has completed, also when a wait gave up
    if (elect_one()) {
      umma_commit(drain);
      if (!mbar_wait(drain, 0)) report_error(p.err, kErrBarrierTimeout, 44, static_cast<int>(it));
    }
    __syncwarp();
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t ui = 0;
    int cur = it_lo;
    Seg sg;
    for (; next_seg(cur, it_hi, p.kblocks_total, stride, sg); ++ui) {
      const int at = sg.tile / p.b_tiles, bt = sg.tile - at * p.b_tiles;
      const uint32_t ab = ui % p.nbuf;
      if (!mbar_wait_warp(&tmem_full[ab], (ui / p.nbuf) & 1u)) {
        report_error(p.err, kErrBarrierTimeout, 43, static_cast<int>(ui));
        break;
      }
      tc_fence_after_sync();
      for (int mi = 0; mi < p.mt; ++mi) {
      const int a_row = (at * p.mt + mi) * kBM + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * buf_cols + mi * acc_cols;
      for (int c0 = 0; c0 < p.bn; c0 += 32) {
        uint32_t v[32], w[32];
        tmem_ld_32x32(taddr + c0, v);
        if (p.dual) tmem_ld_32x32(taddr + p.bn + c0, w);
        tmem_ld_wait();
        const int b_row0 = bt * p.bn + c0;
        if (p.epi == kGemmEpiSwiglu) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(silu_mul(__uint_as_float(v[j]), __uint_as_float(w[j])));
        }
        if (a_row < p.a_rows) {
          if (p.swap) {
            // out[(b_row0 + j) * ldo + a_row]: the warp's lanes are consecutive a_row
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (b_row0 + j >= p.b_rows) break;
              const long long o = static_cast<long long>(b_row0 + j) * p.ldo + a_row;
              const float x = __uint_as_float(v[j]);
              if (p.epi == kGemmEpiAtomic) red_add_f32(static_cast<float*>(p.out) + o, x);
              else if (p.out_bf16) static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(x);
              else static_cast<float*>(p.out)[o] = x;
            }
          } else {
            const long long o = static_cast<long long>(a_row) * p.ldo + b_row0;
            const bool full_row = b_row0 + 32 <= p.b_rows;
            if (p.epi == kGemmEpiAtomic) {
              // a lane owns 32 neighbouring outputs of its row: vector reductions where the row segment is whole and
              // aligned (scalar ones from 32 lanes hit 32 different lines per instruction)
              float* dst = static_cast<float*>(p.out) + o;
              if (full_row && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  red_add_f32x4(dst + j, __uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                __uint_as_float(v[j + 3]));
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (b_row0 + j < p.b_rows) red_add_f32(dst + j, __uint_as_float(v[j]));
              }
            } else if (p.out_bf16) {
              __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + o;
              if (full_row && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 pk;
                  pk.x = pack_bf16x2(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                  pk.y = pack_bf16x2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                  pk.z = pack_bf16x2(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                  pk.w = pack_bf16x2(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                  *reinterpret_cast<uint4*>(dst + j) = pk;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (b_row0 + j < p.b_rows) dst[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
              }
            } else {
              float* dst = static_cast<float*>(p.out) + o;
              if (full_row && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  *reinterpret_cast<uint4*>(dst + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (b_row0 + j < p.b_rows) dst[j] = __uint_as_float(v[j]);
              }
            }
          }
        }
      }
      }  // mi
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[ab]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

}  // namespace

int gemm_bf16_launch(const void* a, int a_rows, const void* b, int b_rows_total, int b_rows, int k, void* out,
                     long long ldo, int out_bf16, int swap, int epi, int dual_off, int bn, int k_chunks,
                     int* err, cudaStream_t stream) {
  PTO_REQUIRE(a && b && out, "gemm: NULL operand");
  PTO_REQUIRE(a_rows > 0 && b_rows > 0 && k > 0, "gemm: empty problem");
  PTO_REQUIRE(k % 8 == 0, "gemm: K must be a multiple of 8 (16-byte rows)");
  PTO_REQUIRE(bn == 32 || bn == 64 || bn == 128 || bn == 256, "gemm: bn must be 32, 64, 128 or 256");
  const int dual = epi == kGemmEpiSwiglu ? 1 : 0;
  PTO_REQUIRE(!dual || (bn <= 128 && !swap), "gemm: SwiGLU epilogue needs bn <= 128 and the normal orientation");
  PTO_REQUIRE(epi != kGemmEpiAtomic || !out_bf16, "gemm: atomic epilogue accumulates in fp32");
  (void)k_chunks;
  // large whole-tile problems run on CTA pairs (256 x 256 tiles, half the B tile per CTA)
  if (gemm2_eligible(a_rows, b_rows, k, epi, swap, bn, dual))
    return gemm2_bf16_launch(a, a_rows, b, b_rows_total, b_rows, k, out, ldo, out_bf16, epi, dual_off, err, stream);

  GemmParams p;
  p.a_rows = a_rows; p.b_rows = b_rows; p.k = k;
  // 256-row CTA tiles when the problem is large enough to be L2->SM bound (whole-tile epilogues only):
  // the B tile is then shared by two A tiles and the accumulators take all 512 TMEM columns
  const int acc_cols = (dual ? 2 : 1) * bn;
  const long long tiles128 = static_cast<long long>((a_rows + kBM - 1) / kBM) * ((b_rows + bn - 1) / bn);
  // (with a short K the single-buffered accumulators cost more than the halved B traffic gains)
  p.mt = (epi != kGemmEpiAtomic && !swap && acc_cols == 256 && a_rows >= 512 && k >= 2048 &&
          tiles128 >= 4ll * sm_count()) ? 2 : 1;
  p.nbuf = (p.mt * acc_cols * 2 <= 512) ? 2 : 1;
  p.a_tiles = (a_rows + p.mt * kBM - 1) / (p.mt * kBM);
  p.b_tiles = (b_rows + bn - 1) / bn;
  const int stage_atom_bytes = p.mt * kBM * 128 + (dual ? 2 : 1) * bn * 128;
  p.katoms = (stage_atom_bytes <= 24 * 1024 && k > kBK) ? 2 : 1;   // small stages: two K atoms per barrier round
  const int tiles = p.a_tiles * p.b_tiles;
  // Decode-shaped problems (weights as A, a few dozen tokens as the MMA N) with a long stream per CTA: four atoms
  // per round.  Each round costs a fixed ~0.3 us of barrier hand-offs next to 0.4 us per atom of loading and
  // MMA issue, so longer rounds pay as long as every CTA still gets ten or more of them.
  if (swap && epi == kGemmEpiAtomic && p.katoms == 2 &&
      static_cast<long long>(tiles) * ((k + 4 * kBK - 1) / (4 * kBK)) >= 10ll * sm_count())
    p.katoms = 4;
  p.kblocks_total = (k + kBK * p.katoms - 1) / (kBK * p.katoms);
  PTO_REQUIRE(static_cast<long long>(tiles) * p.kblocks_total < (1ll << 31), "gemm: problem too large");
  p.iters_total = tiles * p.kblocks_total;
  int grid = sm_count();
  if (epi == kGemmEpiAtomic) {
    // stream-K; keep segments at least 4 K blocks long on average
    const int max_ctas = (p.iters_total + 3) / 4;
    if (grid > max_ctas) grid = max_ctas;
    p.iters_per_cta = (p.iters_total + grid - 1) / grid;
  } else {
    if (grid > tiles) grid = tiles;
    p.iters_per_cta = 0;  // whole tiles, taken round-robin
  }
  if (epi == kGemmEpiAtomic) grid = (p.iters_total + p.iters_per_cta - 1) / p.iters_per_cta;
  p.bn = bn; p.dual = dual; p.dual_off = dual_off; p.swap = swap; p.epi = epi; p.out_bf16 = out_bf16;
  p.out = out; p.ldo = ldo; p.err = err;
  const int stage_bytes = p.katoms * stage_atom_bytes;
  int stages = (200 * 1024) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) stages = 2;
  p.stages = stages;
  const size_t smem = 1024 + static_cast<size_t>(stages) * stage_bytes + (2 * kMaxStages + 5) * 8 + 16;

  CUtensorMap tm_a, tm_b;
  int st = make_tensor_map_2d(&tm_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_rows, k, static_cast<uint64_t>(k) * 2,
                              kBK, p.mt * kBM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_rows_total, k,
                          static_cast<uint64_t>(k) * 2, kBK, bn, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  if (first_use_on_device(0))
    PTO_CUDA(cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  launch_kernel(gemm_bf16_kernel, dim3(grid), dim3(kGemmThreads), smem, stream, tm_a, tm_b, p);
  return check_cuda(cudaGetLastError(), "gemm_bf16_kernel launch");
}

}  // namespace pto
