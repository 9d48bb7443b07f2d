// bf16 GEMM for large problems on a PAIR of SMs: tcgen05.mma.cta_group::2.
//
//   D[a_row, b_row] = sum_k A[a_row, k] * B[b_row, k]        (both operands K-major bf16, fp32 accumulation:
//   python/pypto/debug/torch_codegen.py:1078-1086; it stands where the reference runs `matmul_kernel` tiles,
//   examples/models/01_ffn.py:37-45, 112-131)
//
// Two CTAs of a cluster share one 256 x 256 output tile.  Each loads its own 128 rows of A and its own HALF of the
// B tile (128 rows), so a CTA pulls 32 KB per 64-wide K block for 128 x 256 x 64 MMA work of its own -- two thirds of
// the bytes per FLOP of a single CTA's 128 x 256 tile, which is what bounds large GEMMs on this part (L2 -> SM).  One
// elected thread of the even ("leader") CTA issues every MMA for both; each CTA keeps the 128 x 256 accumulator of
// its own rows in its own TMEM, double buffered, and its own four epilogue warps write it out.
// With the SwiGLU epilogue the B tile is [128 gate rows | 128 up rows]: the leader loads the gate half, its peer
// the up half, and a thread finds silu(g) * u in columns j and 128 + j of its own accumulator row.
//
// Hand-offs across the pair:
//   full[s]       lives in the leader: it expects the bytes of BOTH CTAs' loads (the peer's TMA signals the
//                 leader's barrier: cp.async.bulk.tensor ... .cta_group::2)
//   empty[s]      one in each CTA, released by tcgen05.commit ... .multicast::cluster to both
//   tmem_full[b]  one in each CTA, same multicast commit after the last K block of a tile
//   tmem_empty[b] lives in the leader: eight arrivals, one per epilogue warp of the pair (the peer's arrive remotely)
// No TMA load is multicast.  Every mbarrier wait is bounded; the two cluster-wide barriers (after set-up, before
// tear-down) are reached by every thread on every path.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "pair.cuh"

namespace pto {
namespace {

constexpr int kG2Threads = 192;
constexpr int kG2Stages = 6;
constexpr int kG2BK = 64;                                   // bf16 per K block = one 128-byte swizzle atom
constexpr uint32_t kG2TileBytes = 128 * kG2BK * 2;          // 16 KB: 128 rows x 64 bf16
constexpr uint32_t kG2StageBytes = 2 * kG2TileBytes;        // A rows of this CTA, B half of this CTA

struct Gemm2Params {
  int a_rows, b_rows, k;
  int a_tiles, b_tiles, kblocks;    // tiles of 256 A rows x 256 accumulator columns
  int group;                        // tile rows per group of the tile order
  int dual, dual_off;               // SwiGLU: the second half of the B tile is the up weights at row offset dual_off
  int out_bf16;
  void* out;
  long long ldo;
  int* err;
};

// silu(g) * u with the sigmoid as recip(1 + exp(-g)) (examples/models/01_ffn.py:66-77); the quotient is the approximate
// one (2 ulp): an IEEE division costs a dozen instructions per element and the epilogue of a short-K tile is as long as
// the tile's MMAs
__device__ __forceinline__ float silu_mul2(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kG2Threads, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kG2Stages) * kG2StageBytes);
  uint64_t* empty = full + kG2Stages;
  uint64_t* tmem_full = empty + kG2Stages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* drain = tmem_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs), 1 = peer
  const int pair = static_cast<int>(blockIdx.x >> 1), npairs = static_cast<int>(gridDim.x >> 1);
  constexpr uint32_t tmem_cols = 512;               // two accumulators of 256 columns

  if (threadIdx.x == 0) {
    for (int i = 0; i < kG2Stages; ++i) {
      mbar_init(&full[i], 1);      // the leader's arrive.expect_tx (bytes of both CTAs)
      mbar_init(&empty[i], 1);     // one multicast commit
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 8);   // four epilogue warps in each CTA of the pair
    }
    mbar_init(drain, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, tmem_cols);   // the same warp in each CTA of the pair, together
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();              // both CTAs' barriers are initialised before anything is signalled across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles = p.a_tiles * p.b_tiles;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    uint32_t it = 0, s = 0, ph = 0;
    bool ok = true;
    for (int tile = pair; tile < tiles && ok; tile += npairs) {
      int at, bt;
      grouped_tile_coords(tile, p.group, p.a_tiles, p.b_tiles, at, bt);
      const int a_row = at * 256 + static_cast<int>(rank) * 128;
      // this CTA's half of the B tile: rows of the second half are the up weights when the epilogue is SwiGLU
      const int b_row = p.dual ? (rank ? p.dual_off + bt * 128 : bt * 128) : bt * 256 + static_cast<int>(rank) * 128;
      for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
        if (!__all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u))) {
          if (lane == 0) report_error(p.err, kErrBarrierTimeout, 90, static_cast<int>(it));
          ok = false;
          break;
        }
        if (elect_one()) {
          uint8_t* st = smem + static_cast<size_t>(s) * kG2StageBytes;
          const uint32_t leader_full = mapa_u32(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * kG2StageBytes);
          tma_load_2d_pair(st, &tm_a, kb * kG2BK, a_row, leader_full);              // past the matrix: zero filled
          tma_load_2d_pair(st + kG2TileBytes, &tm_b, kb * kG2BK, b_row, leader_full);
        }
        __syncwarp();
        if (++s == kG2Stages) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader only) -------------------------------
    if (rank == 0) {
      const uint32_t idesc = umma_idesc(256, 256, 1, 1);
      const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);   // stride byte offset, version, 128-byte swizzle
      const uint32_t lo0 = ((smem_u32(smem) & 0x3FFFFu) >> 4) | (1u << 16);
      uint32_t it = 0, s = 0, ph = 0, ab = 0, ab_ph = 1;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += npairs) {
        if (!__all_sync(0xffffffffu, mbar_wait(&tmem_empty[ab], ab_ph))) {
          if (lane == 0) report_error(p.err, kErrBarrierTimeout, 91, static_cast<int>(it));
          break;
        }
        tc_fence_after_sync();
        const uint32_t d0 = tmem_base + ab * 256;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          if (!__all_sync(0xffffffffu, mbar_wait(&full[s], ph))) {
            if (lane == 0) report_error(p.err, kErrBarrierTimeout, 92, static_cast<int>(it));
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (elect_one()) {
            const uint32_t a_lo = lo0 + s * (kG2StageBytes >> 4);
            const uint32_t b_lo = a_lo + (kG2TileBytes >> 4);
#pragma unroll
            for (uint32_t k = 0; k < kG2BK / 16; ++k) {   // 16 bf16 = 32 bytes of K per MMA: the address field moves by 2
              const uint64_t ad = (static_cast<uint64_t>(desc_hi) << 32) | (a_lo + 2 * k);
              const uint64_t bd = (static_cast<uint64_t>(desc_hi) << 32) | (b_lo + 2 * k);
              umma_bf16_pair(d0, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit_pair(&empty[s]);
          }
          __syncwarp();
          if (++s == kG2Stages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok && elect_one()) umma_commit_pair(&tmem_full[ab]);
        __syncwarp();
        ab ^= 1u;
        if (ab == 0) ab_ph ^= 1u;
      }
      // no CTA of the pair releases tensor memory before every MMA has completed, also when a wait gave up
      if (elect_one()) {
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(drain)) : "memory");
        if (!mbar_wait(drain, 0)) report_error(p.err, kErrBarrierTimeout, 94, static_cast<int>(it));
      }
      __syncwarp();
    }
  } else {
    // -------------------------------- epilogue (both CTAs) --------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t ui = 0;
    const uint32_t leader_empty0 = mapa_u32(smem_u32(&tmem_empty[0]), 0), leader_empty1 = mapa_u32(smem_u32(&tmem_empty[1]), 0);
    for (int tile = pair; tile < tiles; tile += npairs, ++ui) {
      int at, bt;
      grouped_tile_coords(tile, p.group, p.a_tiles, p.b_tiles, at, bt);
      const uint32_t ab = ui & 1u;
      if (!mbar_wait_warp(&tmem_full[ab], (ui >> 1) & 1u)) {
        report_error(p.err, kErrBarrierTimeout, 93, static_cast<int>(ui));
        break;
      }
      tc_fence_after_sync();
      const int a_row = at * 256 + static_cast<int>(rank) * 128 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * 256;
      const int ncol = p.dual ? 128 : 256;          // output columns of this tile
      for (int c0 = 0; c0 < ncol; c0 += 32) {
        uint32_t v[32], w[32];
        tmem_ld_32x32(taddr + c0, v);
        if (p.dual) tmem_ld_32x32(taddr + 128 + c0, w);
        tmem_ld_wait();
        if (p.dual) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(silu_mul2(__uint_as_float(v[j]), __uint_as_float(w[j])));
        }
        const int b_row0 = bt * ncol + c0;
        if (a_row < p.a_rows && b_row0 < p.b_rows) {
          const long long o = static_cast<long long>(a_row) * p.ldo + b_row0;
          const bool full_row = b_row0 + 32 <= p.b_rows;
          if (p.out_bf16) {
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
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(dst + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (b_row0 + j < p.b_rows) dst[j] = __uint_as_float(v[j]);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(ab ? leader_empty1 : leader_empty0);   // the leader's barrier, from either CTA
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves, or frees tensor memory, while its partner may still signal or read it
  if (warp == 1) tmem_dealloc_pair(tmem_base, tmem_cols);
}

}  // namespace

bool gemm2_eligible(int a_rows, int b_rows, int k, int epi, int swap, int bn, int dual) {
  static const int enabled = [] { const char* v = getenv("PTO_GEMM_PAIR"); return v ? atoi(v) : 1; }();
  if (!enabled || swap || epi == kGemmEpiAtomic) return false;
  if ((dual ? 2 : 1) * bn != 256) return false;
  const long long tiles = static_cast<long long>((a_rows + 255) / 256) * ((b_rows + (dual ? 127 : 255)) / (dual ? 128 : 256));
  return a_rows >= 1024 && k >= 256 && tiles >= sm_count() / 2;
}

// Whole 256 x 256 tiles, taken round-robin by CTA pairs.  epi: store or SwiGLU (dual_off = row offset of the up weights).
int gemm2_bf16_launch(const void* a, int a_rows, const void* b, int b_rows_total, int b_rows, int k, void* out, long long ldo,
                      int out_bf16, int epi, int dual_off, int* err, cudaStream_t stream) {
  PTO_REQUIRE(a && b && out, "gemm: NULL operand");
  PTO_REQUIRE(a_rows > 0 && b_rows > 0 && k > 0 && k % 8 == 0, "gemm: empty problem or K not a multiple of 8");
  Gemm2Params p;
  p.a_rows = a_rows; p.b_rows = b_rows; p.k = k;
  p.dual = epi == kGemmEpiSwiglu ? 1 : 0;
  p.dual_off = dual_off;
  p.a_tiles = (a_rows + 255) / 256;
  p.b_tiles = p.dual ? (b_rows + 127) / 128 : (b_rows + 255) / 256;
  p.kblocks = (k + kG2BK - 1) / kG2BK;
  p.group = 16;                     // measured 4 / 8 / 16 / all rows at M = 8192, K 4096 -> 2 x 14336: 1452 / 1499 / 1522 / 1455 TFLOP/s
  p.out_bf16 = out_bf16; p.out = out; p.ldo = ldo; p.err = err;
  const long long tiles = static_cast<long long>(p.a_tiles) * p.b_tiles;
  PTO_REQUIRE(tiles * p.kblocks < (1ll << 31), "gemm: problem too large");
  int pairs = sm_count() / 2;
  if (pairs > tiles) pairs = static_cast<int>(tiles);
  const size_t smem = 1024 + static_cast<size_t>(kG2Stages) * kG2StageBytes + (2 * kG2Stages + 5) * 8 + 16;
  CUtensorMap tm_a, tm_b;
  int st = make_tensor_map_2d(&tm_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_rows, k, static_cast<uint64_t>(k) * 2, kG2BK, 128,
                              CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  st = make_tensor_map_2d(&tm_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_rows_total, k, static_cast<uint64_t>(k) * 2, kG2BK, 128,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != kOk) return st;
  if (first_use_on_device(5))
    PTO_CUDA(cudaFuncSetAttribute(gemm2_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kG2Threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = nullptr;      // the cluster shape is a compile-time attribute of the kernel
  cfg.numAttrs = 0;
  PTO_CUDA(cudaLaunchKernelEx(&cfg, gemm2_bf16_kernel, tm_a, tm_b, p));
  return check_cuda(cudaGetLastError(), "gemm2_bf16_kernel launch");
}

}  // namespace pto
