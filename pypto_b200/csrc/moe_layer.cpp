// The mixture-of-experts layer as one object of the C++ runtime: gate + top-k routing, dispatch, grouped FP8
// expert FFN, combine -- on one GPU, or expert-parallel over the ranks of a communicator.
//
// Data movement follows the reference's expert-parallel pattern (dispatch_step -> local_expert_step ->
// combine_step, tests/st/distributed/test_l3_ep_dispatch_combine.py:104-402): destination rank = expert id / L,
// rows of a (rank, local expert) bucket ordered by source rank then (t, k), combine = fp32 sum over k of the
// returned bf16 rows.  One forward call issues every kernel and both exchanges of a step:
//
//   route (gate GEMM, top-k) -> quantise tokens -> [side stream: shared expert] -> dispatch plan ->
//   counts all-to-all -> pack payload rows (fp8 row | scales | weight) -> ONE all-to-all-v ->
//   receive plan -> unpack -> gate/up GEMM -> quantise -> down GEMM (rows written in arrival order) ->
//   ONE all-to-all-v back -> combine
//
// When every rank can map every other rank's buffers (one node, CUDA IPC, checked and agreed on when the layer is
// created; PTO_EP_PEER=0 turns it off), the way back is no collective at all: a kernel stores each source's block
// of result rows straight into that source's sorted result buffer through peer memory and raises a flag there, and
// the source's combine waits (bounded) for the flags of all ranks (moe_push_rows_kernel, moe_wait_flags_kernel).
// The offset of a block in its source's buffer travels with the counts.  With PTO_EP_PEER=2 on every rank the way
// out works the same way (each destination tells its sources where their blocks begin in its receive buffer, the
// same kernel stores the packed rows there, a second set of flags); by default it stays an all-to-all-v.  What orders
// a rank's next step behind the combine of the ranks it writes to are the small all-to-alls of every step (counts,
// offsets): every pair of ranks exchanges a word in them, and a rank enqueues them after its previous combine.
//
// The host waits once per step, for the row counts of the exchange (a pinned buffer and an event); everything
// before that wait is already queued, so the GPU packs the payload and runs the shared expert meanwhile.
// All buffers are allocated when the layer is created, sized for `max_tokens` and the worst-case arrival count.
#include <nvtx3/nvToolsExt.h>

#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#include "pypto_b200.h"
#include "runtime.h"

extern "C" int pto_comm_rank(const pto_comm* c);
extern "C" int pto_comm_size(const pto_comm* c);

namespace pto {
namespace {

inline size_t al256(size_t v) { return (v + 255) / 256 * 256; }

constexpr int kPhases = 10;   // route_quantize, plan, pack, exchange_out, unpack, experts, exchange_back, combine

}  // namespace
}  // namespace pto

struct pto_moe_layer {
  pto_moe_layer_desc d;
  int world = 1, rank = 0, local_experts = 0, device = 0;
  size_t payload = 0;            // bytes of one dispatched row: fp8 tokens | fp32 scales | fp32 weight, padded to 16
  size_t off_scale = 0, off_weight = 0;
  long long capacity = 0;        // rows that can arrive at this rank
  uint8_t* arena = nullptr;
  // buffers inside the arena
  float* logits; int32_t* idx; float* w; uint8_t* xq; float* xs;
  int32_t *counts, *offsets, *pos, *route_at, *work, *recv_counts, *counts2, *offsets2, *arrival_of, *grouped_of, *whole;
  uint8_t *send_buf, *recv_buf, *xq_g; float *xs_g, *w_g;
  uint8_t *act, *act_q; float* act_s; uint8_t *y_g, *back;
  uint8_t *sh_act, *sh_act_q; float* sh_act_s; uint8_t* sh_out;
  int32_t* err;
  int32_t* host_counts = nullptr;   // pinned
  int32_t* host_whole = nullptr;    // pinned {0, tokens}: offsets of the one-expert group the shared expert runs as
  int whole_tokens = -1;            // the token count `whole` holds on the device (uploaded again only when it changes)
  cudaStream_t side = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_counts = nullptr, ev_whole = nullptr;
  cudaEvent_t ev_phase[pto::kPhases + 1] = {};
  // peer-memory paths: 1 = the way back, 2 = the way out as well
  bool peer = false;
  int peer_level = 0;
  int step = 0;                     // forward calls so far: the value this rank's flags are raised to
  int32_t *flags = nullptr, *done_counter = nullptr, *base_send = nullptr, *base_recv = nullptr;   // in the arena
  int32_t *flags_out = nullptr, *done_counter_out = nullptr, *obase_send = nullptr, *obase_recv = nullptr;
  void* peer_arena[pto::kMoeMaxPeers] = {};   // other ranks' arenas as mapped here (NULL for this rank)
  pto::MoePeerTable peers = {};       // result buffers and return flags of every rank
  pto::MoePeerTable peers_out = {};   // receive buffers and arrival flags of every rank
};

namespace pto {
namespace {

int experts_ffn(pto_moe_layer* L, const void* w_gu, const float* s_gu, const void* w_d, const float* s_d, int experts,
                const void* xq, const float* xs, const int32_t* offsets, int rows, const float* route_w,
                const int32_t* out_rows, void* act, void* act_q, float* act_s, void* out, cudaStream_t s) {
  const int H = L->d.hidden, I = L->d.inter;
  int st = moe_gemm_fp8_launch(1, w_gu, s_gu, experts, 2 * I, I, H, xq, xs, offsets, rows, nullptr, nullptr, act, L->err, s);
  if (st != kOk) return st;
  st = quantize_rows_launch(act, PTO_BF16, act_q, act_s, rows, I, s);
  if (st != kOk) return st;
  return moe_gemm_fp8_launch(0, w_d, s_d, experts, H, H, I, act_q, act_s, offsets, rows, route_w, out_rows, out, L->err, s);
}

// Collective over the layer's communicator: every rank exports its arena (CUDA IPC), the handles and the offsets of
// the result buffer and the flag words go round in an all-to-all, every rank maps the others, and a second
// all-to-all of one word tells whether ALL of them could.  Only then is the peer path used; any refusal (another
// node, no peer access, PTO_EP_PEER=0 on some rank) leaves every rank on the collective, all alike.
struct PeerHello {
  cudaIpcMemHandle_t handle;
  unsigned long long arena_bytes, back_off, flags_off, recv_off, flags_out_off;
  int want;                         // 0: the collectives; 1: results return through peer memory; 2: rows go out that way too
  char pad[128 - sizeof(cudaIpcMemHandle_t) - 5 * sizeof(unsigned long long) - sizeof(int)];
};
static_assert(sizeof(PeerHello) == 128, "one hello per rank, 128 bytes");

int peer_setup(pto_moe_layer* L, size_t arena_bytes) {
  const int W = L->world;
  const char* env = getenv("PTO_EP_PEER");
  int want = env == nullptr ? 1 : atoi(env);
  want = W > kMoeMaxPeers || want < 0 ? 0 : (want > 2 ? 2 : want);
  PeerHello mine = {};
  if (want && cudaIpcGetMemHandle(&mine.handle, L->arena) != cudaSuccess) {
    (void)cudaGetLastError();
    want = 0;
  }
  mine.arena_bytes = arena_bytes;
  mine.back_off = static_cast<unsigned long long>(L->back - L->arena);
  mine.flags_off = static_cast<unsigned long long>(reinterpret_cast<uint8_t*>(L->flags) - L->arena);
  mine.recv_off = static_cast<unsigned long long>(L->recv_buf - L->arena);
  mine.flags_out_off = static_cast<unsigned long long>(reinterpret_cast<uint8_t*>(L->flags_out) - L->arena);
  mine.want = want;
  std::vector<PeerHello> out(W, mine), in(W);
  uint8_t* dev = nullptr;
  PTO_CUDA(cudaMalloc(reinterpret_cast<void**>(&dev), 2 * sizeof(PeerHello) * W));
  struct FreeAtExit { uint8_t* p; ~FreeAtExit() { cudaFree(p); } } free_at_exit{dev};
  PTO_CUDA(cudaMemcpy(dev, out.data(), sizeof(PeerHello) * W, cudaMemcpyHostToDevice));
  int st = pto_all_to_all(L->d.comm, dev, dev + sizeof(PeerHello) * W, sizeof(PeerHello), nullptr);
  if (st != kOk) return st;
  PTO_CUDA(cudaStreamSynchronize(nullptr));
  PTO_CUDA(cudaMemcpy(in.data(), dev + sizeof(PeerHello) * W, sizeof(PeerHello) * W, cudaMemcpyDeviceToHost));
  int ok = want > 0, level = want;
  for (int r = 0; r < W && ok; ++r) {
    if (in[r].want < level) level = in[r].want;   // the most cautious rank decides
    if (!in[r].want || in[r].arena_bytes != arena_bytes || in[r].back_off != mine.back_off || in[r].flags_off != mine.flags_off ||
        in[r].recv_off != mine.recv_off || in[r].flags_out_off != mine.flags_out_off) {
      ok = 0;                                   // a rank that refuses, or a layer of another shape
      break;
    }
    if (r == L->rank) continue;
    void* base = nullptr;
    if (cudaIpcOpenMemHandle(&base, in[r].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      (void)cudaGetLastError();
      ok = 0;
      break;
    }
    L->peer_arena[r] = base;
  }
  // agreement: the peer path only if every rank mapped every other
  std::vector<int> mine_ok(W * 32, ok), all_ok(W * 32, 0);   // 128 bytes per rank: the all-to-all's granule is not tested below that
  PTO_CUDA(cudaMemcpy(dev, mine_ok.data(), 128 * W, cudaMemcpyHostToDevice));
  st = pto_all_to_all(L->d.comm, dev, dev + sizeof(PeerHello) * W, 128, nullptr);
  if (st != kOk) return st;
  PTO_CUDA(cudaStreamSynchronize(nullptr));
  PTO_CUDA(cudaMemcpy(all_ok.data(), dev + sizeof(PeerHello) * W, 128 * W, cudaMemcpyDeviceToHost));
  for (int r = 0; r < W; ++r) ok = ok && all_ok[r * 32];
  if (!ok) {
    for (void*& p : L->peer_arena) {
      if (p) cudaIpcCloseMemHandle(p);
      p = nullptr;
    }
    return kOk;
  }
  for (int r = 0; r < W; ++r) {
    uint8_t* base = r == L->rank ? L->arena : static_cast<uint8_t*>(L->peer_arena[r]);
    L->peers.back[r] = base + mine.back_off;
    L->peers.flags[r] = reinterpret_cast<int32_t*>(base + mine.flags_off);
    L->peers_out.back[r] = base + mine.recv_off;
    L->peers_out.flags[r] = reinterpret_cast<int32_t*>(base + mine.flags_out_off);
  }
  L->peer = true;
  L->peer_level = level;
  return kOk;
}

}  // namespace
}  // namespace pto

extern "C" {

int pto_moe_layer_destroy(pto_moe_layer* L) {
  if (!L) return pto::kOk;
  cudaSetDevice(L->device);
  cudaDeviceSynchronize();   // nothing of this rank is still writing into a peer's buffers
  for (void* p : L->peer_arena) if (p) cudaIpcCloseMemHandle(p);
  for (cudaEvent_t e : L->ev_phase) if (e) cudaEventDestroy(e);
  if (L->ev_fork) cudaEventDestroy(L->ev_fork);
  if (L->ev_join) cudaEventDestroy(L->ev_join);
  if (L->ev_counts) cudaEventDestroy(L->ev_counts);
  if (L->ev_whole) cudaEventDestroy(L->ev_whole);
  if (L->side) cudaStreamDestroy(L->side);
  if (L->host_counts) cudaFreeHost(L->host_counts);
  if (L->host_whole) cudaFreeHost(L->host_whole);
  if (L->arena) cudaFree(L->arena);
  delete L;
  return pto::kOk;
}

int pto_moe_layer_create(const pto_moe_layer_desc* desc, pto_moe_layer** out) {
  using namespace pto;
  if (!desc || !out) return fail(kInvalidArgument, "moe_layer_create: NULL argument");
  *out = nullptr;
  const pto_moe_layer_desc& d = *desc;
  PTO_REQUIRE(d.hidden > 0 && d.hidden % 128 == 0 && d.inter > 0 && d.inter % 128 == 0,
              "moe_layer: hidden and intermediate sizes must be multiples of 128");
  PTO_REQUIRE(d.n_experts > 0 && d.topk > 0 && d.topk <= 32 && d.topk <= d.n_experts && d.max_tokens > 0,
              "moe_layer: bad expert / top-k / token counts");
  PTO_REQUIRE(d.gate_packed && d.bias && d.w_gu && d.s_gu && d.w_d && d.s_d, "moe_layer: NULL weight");
  const int world = d.comm ? pto_comm_size(d.comm) : 1;
  PTO_REQUIRE(d.n_experts % world == 0, "moe_layer: experts must split evenly over the ranks");
  pto_moe_layer* L = new pto_moe_layer;
  L->d = d;
  L->world = world;
  L->rank = d.comm ? pto_comm_rank(d.comm) : 0;
  L->local_experts = d.n_experts / world;
  if (cudaGetDevice(&L->device) != cudaSuccess) { delete L; return fail(kCudaError, "moe_layer: no current device"); }
  const long long T = d.max_tokens, K = d.topk, H = d.hidden, I = d.inter, E = d.n_experts;
  const long long routes = T * K;
  L->capacity = world > 1 ? routes * world : routes;
  PTO_REQUIRE(L->capacity < (1ll << 31), "moe_layer: too many routes");
  L->off_scale = (static_cast<size_t>(H) + 15) / 16 * 16;
  L->off_weight = L->off_scale + (static_cast<size_t>(H) / 128 * 4 + 15) / 16 * 16;
  L->payload = L->off_weight + 16;
  const long long C = L->capacity;
  struct Slot { void** p; size_t bytes; };
  std::vector<Slot> slots = {
      {(void**)&L->err, 256}, {(void**)&L->logits, (size_t)(T * E * 4)}, {(void**)&L->idx, (size_t)(routes * 4)},
      {(void**)&L->w, (size_t)(routes * 4)}, {(void**)&L->xq, (size_t)(T * H)}, {(void**)&L->xs, (size_t)(T * (H / 128) * 4)},
      {(void**)&L->counts, (size_t)(E * 4)}, {(void**)&L->offsets, (size_t)((E + 1) * 4)}, {(void**)&L->pos, (size_t)(routes * 4)},
      {(void**)&L->route_at, (size_t)(routes * 4)}, {(void**)&L->work, (size_t)((routes + E) * 4)},
      {(void**)&L->recv_counts, (size_t)(E * 4)}, {(void**)&L->counts2, (size_t)(L->local_experts * 4)},
      {(void**)&L->offsets2, (size_t)((L->local_experts + 1) * 4)}, {(void**)&L->arrival_of, (size_t)(C * 4)},
      {(void**)&L->grouped_of, (size_t)(C * 4)}, {(void**)&L->whole, 16},
      {(void**)&L->send_buf, world > 1 ? (size_t)routes * L->payload : 0}, {(void**)&L->recv_buf, world > 1 ? (size_t)C * L->payload : 0},
      {(void**)&L->xq_g, (size_t)(C * H)}, {(void**)&L->xs_g, (size_t)(C * (H / 128) * 4)}, {(void**)&L->w_g, (size_t)(C * 4)},
      {(void**)&L->act, (size_t)(C * I * 2)}, {(void**)&L->act_q, (size_t)(C * I)}, {(void**)&L->act_s, (size_t)(C * (I / 128) * 4)},
      {(void**)&L->y_g, (size_t)(C * H * 2)}, {(void**)&L->back, world > 1 ? (size_t)(routes * H * 2) : 0},
      {(void**)&L->sh_act, d.sh_w_gu ? (size_t)(T * I * 2) : 0}, {(void**)&L->sh_act_q, d.sh_w_gu ? (size_t)(T * I) : 0},
      {(void**)&L->sh_act_s, d.sh_w_gu ? (size_t)(T * (I / 128) * 4) : 0}, {(void**)&L->sh_out, d.sh_w_gu ? (size_t)(T * H * 2) : 0},
      {(void**)&L->flags, 256}, {(void**)&L->done_counter, 256}, {(void**)&L->flags_out, 256}, {(void**)&L->done_counter_out, 256},
      {(void**)&L->base_send, (size_t)(world * 4)}, {(void**)&L->base_recv, (size_t)(world * 4)},
      {(void**)&L->obase_send, (size_t)(world * 4)}, {(void**)&L->obase_recv, (size_t)(world * 4)}};
  size_t total = 0;
  for (auto& s : slots) total += al256(s.bytes ? s.bytes : 1);
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&L->arena), total);
  if (e != cudaSuccess) { delete L; return check_cuda(e, "moe_layer: cudaMalloc of the layer's buffers"); }
  size_t off = 0;
  for (auto& s : slots) {
    *s.p = L->arena + off;
    off += al256(s.bytes ? s.bytes : 1);
  }
  int st = check_cuda(cudaMemset(L->err, 0, 256), "cudaMemset");
  if (st == kOk) st = check_cuda(cudaMemset(L->flags, 0, 1024), "cudaMemset");   // both flag arrays and the push kernels' counters
  if (st == kOk) st = check_cuda(cudaMallocHost(reinterpret_cast<void**>(&L->host_counts), (2 * E + 2) * 4), "cudaMallocHost");
  if (st == kOk) st = check_cuda(cudaMallocHost(reinterpret_cast<void**>(&L->host_whole), 16), "cudaMallocHost");
  if (st == kOk) st = check_cuda(cudaStreamCreateWithFlags(&L->side, cudaStreamNonBlocking), "cudaStreamCreate");
  if (st == kOk) st = check_cuda(cudaEventCreateWithFlags(&L->ev_fork, cudaEventDisableTiming), "cudaEventCreate");
  if (st == kOk) st = check_cuda(cudaEventCreateWithFlags(&L->ev_join, cudaEventDisableTiming), "cudaEventCreate");
  if (st == kOk) st = check_cuda(cudaEventCreateWithFlags(&L->ev_counts, cudaEventDisableTiming), "cudaEventCreate");
  if (st == kOk) st = check_cuda(cudaEventCreateWithFlags(&L->ev_whole, cudaEventDisableTiming), "cudaEventCreate");
  for (int i = 0; st == kOk && i <= kPhases; ++i) st = check_cuda(cudaEventCreate(&L->ev_phase[i]), "cudaEventCreate");
  if (st == kOk && world > 1) st = peer_setup(L, total);
  if (st != kOk) { pto_moe_layer_destroy(L); return st; }
  *out = L;
  return kOk;
}

int pto_moe_layer_peer_exchange(const pto_moe_layer* L) { return L && L->peer ? L->peer_level : 0; }

int pto_moe_layer_status(pto_moe_layer* L, int32_t out4[4], void* stream) {
  using namespace pto;
  if (!L || !out4) return fail(kInvalidArgument, "moe_layer_status: NULL argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PTO_CUDA(cudaMemcpyAsync(out4, L->err, 16, cudaMemcpyDeviceToHost, s));
  PTO_CUDA(cudaStreamSynchronize(s));
  if (out4[0] != 0) PTO_CUDA(cudaMemsetAsync(L->err, 0, 64, s));
  return kOk;
}

int pto_moe_layer_forward(pto_moe_layer* L, const void* x, int tokens, const int32_t* idx_in, const float* w_in, void* y,
                          int32_t* idx_out, float* w_out, float* phase_ms, void* stream) {
  using namespace pto;
  if (!L || !x || !y) return fail(kInvalidArgument, "moe_layer_forward: NULL argument");
  PTO_REQUIRE(tokens > 0 && tokens <= L->d.max_tokens, "moe_layer_forward: token count outside 1..max_tokens");
  PTO_REQUIRE((idx_in == nullptr) == (w_in == nullptr), "moe_layer_forward: routing needs both indices and weights");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const pto_moe_layer_desc& d = L->d;
  const int T = tokens, K = d.topk, H = d.hidden, E = d.n_experts, W = L->world, Le = L->local_experts;
  const long long routes = static_cast<long long>(T) * K;
  int ph = 0;
  // trace level 1: one NVTX range per phase (host-side issue ranges; the kernels inside carry their own names)
  static const char* const kPhaseNames[] = {"moe.route_quantize", "moe.plan", "moe.pack", "moe.exchange_out", "moe.unpack",
                                            "moe.experts", "moe.exchange_back", "moe.combine"};
  const bool nvtx = trace_level() >= 1;
  int nv = 0;
  bool nv_open = false;
  auto mark = [&]() -> int {
    if (nvtx) {
      if (nv_open) nvtxRangePop();
      nv_open = nv < 8;
      if (nv_open) nvtxRangePushA(kPhaseNames[nv++]);
    }
    if (!phase_ms) return kOk;
    return check_cuda(cudaEventRecord(L->ev_phase[ph++], s), "cudaEventRecord");
  };
  struct PopAtExit { bool* open; ~PopAtExit() { if (*open) nvtxRangePop(); } } pop_at_exit{&nv_open};
  TraceRange whole("moe_layer.forward");
  int st = mark();
  if (st != kOk) return st;
  // ---- route + quantise ----
  const int32_t* idx = idx_in;
  const float* w = w_in;
  if (!idx_in) {
    st = linear_launch(x, d.gate_packed, L->logits, T, E, H, 0, L->err, s);
    if (st != kOk) return st;
    st = moe_topk_launch(L->logits, d.bias, 1, T, E, K, L->idx, L->w, s);
    if (st != kOk) return st;
    idx = L->idx;
    w = L->w;
  }
  st = quantize_rows_launch(x, PTO_BF16, L->xq, L->xs, T, H, s);
  if (st != kOk) return st;
  if ((st = mark()) != kOk) return st;
  // ---- the shared expert runs beside the rest on its own stream ----
  if (d.sh_w_gu) {
    if (L->whole_tokens != T) {
      if (L->whole_tokens >= 0) PTO_CUDA(cudaEventSynchronize(L->ev_whole));   // the last upload has left the pinned words
      L->host_whole[0] = 0;
      L->host_whole[1] = T;
      PTO_CUDA(cudaMemcpyAsync(L->whole, L->host_whole, 8, cudaMemcpyHostToDevice, s));
      PTO_CUDA(cudaEventRecord(L->ev_whole, s));
      L->whole_tokens = T;
    }
    PTO_CUDA(cudaEventRecord(L->ev_fork, s));
    PTO_CUDA(cudaStreamWaitEvent(L->side, L->ev_fork, 0));
    st = experts_ffn(L, d.sh_w_gu, d.sh_s_gu, d.sh_w_d, d.sh_s_d, 1, L->xq, L->xs, L->whole, T, nullptr, nullptr, L->sh_act,
                     L->sh_act_q, L->sh_act_s, L->sh_out, L->side);
    if (st != kOk) return st;
    PTO_CUDA(cudaEventRecord(L->ev_join, L->side));
  }
  // ---- dispatch plan ----
  st = moe_dispatch_plan_launch(idx, static_cast<int>(routes), E, L->counts, L->offsets, L->pos, L->route_at, L->work,
                                L->err, s);
  if (st != kOk) return st;
  if ((st = mark()) != kOk) return st;
  const void* src3[3];
  void* dst3[3];
  long long ss[3], ds[3];
  int rb[3];
  long long rows_in = routes;                 // rows the experts of this rank work on
  const int32_t* offsets_g = L->offsets;      // their offsets by local expert
  const int32_t* out_rows = nullptr;
  if (W == 1) {
    // all experts are local: the sorted rows are the grouped rows
    src3[0] = L->xq; dst3[0] = L->xq_g; ss[0] = ds[0] = H; rb[0] = H;
    src3[1] = L->xs; dst3[1] = L->xs_g; ss[1] = ds[1] = H / 128 * 4; rb[1] = H / 128 * 4;
    st = moe_move_rows_launch(src3, ss, dst3, ds, rb, 2, L->route_at, K, routes, T, L->err, s);
    if (st != kOk) return st;
    st = moe_gather_f32_launch(w, L->route_at, routes, routes, L->w_g, L->err, s);
    if (st != kOk) return st;
    if ((st = mark()) != kOk) return st;   // pack
    if ((st = mark()) != kOk) return st;   // exchange_out (none)
    if ((st = mark()) != kOk) return st;   // unpack (none)
  } else {
    // counts exchange, and their way to the host
    st = pto_all_to_all(d.comm, L->counts, L->recv_counts, static_cast<size_t>(Le) * 4, s);
    if (st != kOk) return st;
    if (L->peer) {
      ++L->step;
      // where, in MY sorted result buffer, the block of each destination rank begins: offsets[r * Le]
      PTO_CUDA(cudaMemcpy2DAsync(L->base_send, 4, L->offsets, static_cast<size_t>(Le) * 4, 4, W, cudaMemcpyDeviceToDevice, s));
      st = pto_all_to_all(d.comm, L->base_send, L->base_recv, 4, s);
      if (st != kOk) return st;
      if (L->peer_level >= 2) {
        // and where, in each destination's receive buffer, MY block begins: the destination knows (rows of the
        // ranks before me) and tells
        st = moe_recv_bases_launch(L->recv_counts, W, Le, L->obase_send, s);
        if (st != kOk) return st;
        st = pto_all_to_all(d.comm, L->obase_send, L->obase_recv, 4, s);
        if (st != kOk) return st;
      }
    }
    PTO_CUDA(cudaMemcpyAsync(L->host_counts, L->offsets, (E + 1) * 4, cudaMemcpyDeviceToHost, s));
    PTO_CUDA(cudaMemcpyAsync(L->host_counts + E + 1, L->recv_counts, E * 4, cudaMemcpyDeviceToHost, s));
    PTO_CUDA(cudaEventRecord(L->ev_counts, s));
    // pack: [fp8 row | scales] by token, weight by route -- queued before the host waits
    src3[0] = L->xq; dst3[0] = L->send_buf; ss[0] = H; ds[0] = static_cast<long long>(L->payload); rb[0] = H;
    src3[1] = L->xs; dst3[1] = L->send_buf + L->off_scale; ss[1] = H / 128 * 4; ds[1] = static_cast<long long>(L->payload);
    rb[1] = H / 128 * 4;
    st = moe_move_rows_launch(src3, ss, dst3, ds, rb, 2, L->route_at, K, routes, T, L->err, s);
    if (st != kOk) return st;
    src3[0] = w; dst3[0] = L->send_buf + L->off_weight; ss[0] = 4; ds[0] = static_cast<long long>(L->payload); rb[0] = 4;
    st = moe_move_rows_launch(src3, ss, dst3, ds, rb, 1, L->route_at, 1, routes, routes, L->err, s);
    if (st != kOk) return st;
    if ((st = mark()) != kOk) return st;   // pack
    PTO_CUDA(cudaEventSynchronize(L->ev_counts));          // the one host wait of a step
    std::vector<int64_t> send_rows(W), recv_rows(W);
    long long arrived = 0;
    for (int r = 0; r < W; ++r) {
      send_rows[r] = L->host_counts[(r + 1) * Le] - L->host_counts[r * Le];
      long long n = 0;
      for (int e = 0; e < Le; ++e) n += L->host_counts[E + 1 + r * Le + e];
      recv_rows[r] = n;
      arrived += n;
    }
    if (arrived > L->capacity) return fail(kInvalidArgument, "moe_layer_forward: more rows arrive than the layer was sized for");
    if (L->peer && L->peer_level >= 2) {
      // the packed rows of every destination straight into that destination's receive buffer, then the flags; the
      // unpack below starts once every rank's flag here shows this step
      st = moe_push_rows_launch(L->send_buf, static_cast<int>(L->payload), L->counts, W, Le, L->obase_recv, L->peers_out, L->rank,
                                L->step, L->capacity, routes, L->done_counter_out, L->err, s);
      if (st != kOk) return st;
      st = moe_wait_flags_launch(L->flags_out, W, L->step, L->err, s);
      if (st != kOk) return st;
    } else {
      st = pto_all_to_all_v(d.comm, L->send_buf, send_rows.data(), L->recv_buf, recv_rows.data(), L->payload, s);
      if (st != kOk) return st;
    }
    if ((st = mark()) != kOk) return st;   // exchange_out
    st = moe_recv_plan_launch(L->recv_counts, W, Le, 0, static_cast<int>(arrived > 0 ? arrived : 1), L->counts2, L->offsets2,
                              L->arrival_of, L->grouped_of, L->err, s);
    if (st != kOk) return st;
    src3[0] = L->recv_buf; dst3[0] = L->xq_g; ss[0] = static_cast<long long>(L->payload); ds[0] = H; rb[0] = H;
    src3[1] = L->recv_buf + L->off_scale; dst3[1] = L->xs_g; ss[1] = static_cast<long long>(L->payload); ds[1] = H / 128 * 4;
    rb[1] = H / 128 * 4;
    src3[2] = L->recv_buf + L->off_weight; dst3[2] = L->w_g; ss[2] = static_cast<long long>(L->payload); ds[2] = 4; rb[2] = 4;
    st = moe_move_rows_launch(src3, ss, dst3, ds, rb, 3, L->arrival_of, 1, arrived, arrived, L->err, s);
    if (st != kOk) return st;
    if ((st = mark()) != kOk) return st;   // unpack
    rows_in = arrived;
    offsets_g = L->offsets2;
    out_rows = L->arrival_of;              // results leave in the order the rows arrived in
    // ---- experts, exchange back ----
    if (rows_in > 0) {
      st = experts_ffn(L, d.w_gu, d.s_gu, d.w_d, d.s_d, Le, L->xq_g, L->xs_g, offsets_g, static_cast<int>(rows_in), L->w_g,
                       out_rows, L->act, L->act_q, L->act_s, L->y_g, s);
      if (st != kOk) return st;
    }
    if ((st = mark()) != kOk) return st;   // experts
    if (L->peer) {
      // every source's block of result rows straight into that source's sorted buffer, then the flags; the combine
      // below starts once every rank's flag here shows this step
      st = moe_push_rows_launch(L->y_g, H * 2, L->recv_counts, W, Le, L->base_recv, L->peers, L->rank, L->step,
                                static_cast<long long>(d.max_tokens) * K, arrived, L->done_counter, L->err, s);
      if (st != kOk) return st;
      st = moe_wait_flags_launch(L->flags, W, L->step, L->err, s);
      if (st != kOk) return st;
    } else {
      st = pto_all_to_all_v(d.comm, L->y_g, recv_rows.data(), L->back, send_rows.data(), static_cast<size_t>(H) * 2, s);
      if (st != kOk) return st;
    }
    if ((st = mark()) != kOk) return st;   // exchange_back
  }
  if (W == 1) {
    st = experts_ffn(L, d.w_gu, d.s_gu, d.w_d, d.s_d, Le, L->xq_g, L->xs_g, offsets_g, static_cast<int>(rows_in), L->w_g,
                     nullptr, L->act, L->act_q, L->act_s, L->y_g, s);
    if (st != kOk) return st;
    if ((st = mark()) != kOk) return st;   // experts
    if ((st = mark()) != kOk) return st;   // exchange_back (none)
  }
  // ---- combine ----
  if (d.sh_w_gu) PTO_CUDA(cudaStreamWaitEvent(s, L->ev_join, 0));
  st = moe_combine_launch(W == 1 ? L->y_g : L->back, L->pos, d.sh_w_gu ? L->sh_out : nullptr, T, K, H, routes, y, nullptr, s);
  if (st != kOk) return st;
  if (idx_out && idx != idx_out) PTO_CUDA(cudaMemcpyAsync(idx_out, idx, routes * 4, cudaMemcpyDeviceToDevice, s));
  if (w_out && w != w_out) PTO_CUDA(cudaMemcpyAsync(w_out, w, routes * 4, cudaMemcpyDeviceToDevice, s));
  if ((st = mark()) != kOk) return st;     // combine
  if (phase_ms) {
    PTO_CUDA(cudaEventSynchronize(L->ev_phase[ph - 1]));
    for (int i = 0; i + 1 < ph && i < kPhases; ++i) {
      float ms = 0.f;
      PTO_CUDA(cudaEventElapsedTime(&ms, L->ev_phase[i], L->ev_phase[i + 1]));
      phase_ms[i] = ms;
    }
  }
  return kOk;
}

}  // extern "C"
