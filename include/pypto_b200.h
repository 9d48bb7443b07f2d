/* C ABI of the B200 (sm_100a) backend for pypto's fused model operators.
 *
 * Two groups of entry points:
 *   1. the runtime object the reference obtains from its external device runtime
 *      (`simpler.Worker`: init / malloc / free / copy_to / copy_from / register /
 *      run / close, used at python/pypto/runtime/device_runner.py:821-842 and
 *      python/pypto/runtime/worker.py:222-423), and
 *   2. one direct launcher per fused operator, taking plain device pointers and
 *      sizes, for callers that manage memory themselves.
 *
 * Conventions: every function returns 0 on success or a pto_status code; no C++
 * exception crosses this boundary; `pto_last_error()` gives the message of the
 * last failure on the calling thread.  All `*_dev` / device pointers are CUDA
 * device addresses on the worker's (or the current) device.  `stream` is a
 * `cudaStream_t` passed as `void*` (NULL = the legacy default stream).  Kernels
 * are asynchronous; `pto_synchronize` / `pto_device_status` wait for them.
 */
#ifndef PYPTO_B200_H_
#define PYPTO_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define PTO_API __attribute__((visibility("default")))
#else
#define PTO_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pto_status {
  PTO_OK = 0,
  PTO_INVALID_ARGUMENT = 1,
  PTO_CUDA_ERROR = 2,
  PTO_UNSUPPORTED = 3,
  PTO_DEVICE_TIMEOUT = 4, /* a bounded device-side wait ran out; see pto_device_status */
  PTO_OUT_OF_MEMORY = 5,
  PTO_NOT_FOUND = 6
} pto_status;

/* Element types, numbered like the subset of pypto's DataType that the fused
 * operators use (python/pypto/__init__.py:53-56 lists the fp8 members). */
typedef enum pto_dtype {
  PTO_FP32 = 0,
  PTO_BF16 = 1,
  PTO_FP16 = 2,
  PTO_INT32 = 3,
  PTO_INT64 = 4,
  PTO_FP8E4M3 = 5,
  PTO_UINT8 = 6
} pto_dtype;

/* Tensor descriptor handed to a registered callable.  Mirrors the fields of the
 * reference's ChipTensor that generated kernels read (buffer.addr, start_offset
 * in elements, shapes[], ndims: python/pypto/runtime/builtins/collectives/
 * all_to_all_v/templates/kernel.cpp.in:45-94). */
typedef struct pto_chip_tensor {
  uint64_t addr;
  uint64_t start_offset;
  uint32_t shapes[5];
  uint32_t ndims;
  uint32_t dtype; /* pto_dtype */
  uint32_t reserved;
} pto_chip_tensor;

/* Arguments of one launch: tensors first, then scalars bit-cast to uint64, the
 * order of the reference's `kernel_entry(int64_t* args)` convention
 * (python/pypto/backend/pto_backend.py:541-629, 898-915). */
typedef struct pto_task_args {
  const pto_chip_tensor* tensors;
  uint32_t n_tensors;
  const uint64_t* scalars;
  uint32_t n_scalars;
} pto_task_args;

typedef struct pto_worker pto_worker;

PTO_API const char* pto_last_error(void);
PTO_API const char* pto_version(void);

/* ---- runtime object (replaces simpler.Worker: device_runner.py:821-842) ---- */
PTO_API int pto_worker_create(int device_id, pto_worker** out);
PTO_API int pto_worker_destroy(pto_worker* w); /* idempotent on NULL; frees what the worker still owns */
PTO_API int pto_malloc(pto_worker* w, size_t nbytes, uint64_t* dev_ptr);      /* worker.py:349-366 */
PTO_API int pto_free(pto_worker* w, uint64_t dev_ptr);                        /* worker.py:368-379; unknown or already freed pointers are an error */
PTO_API int pto_copy_to(pto_worker* w, uint64_t dst_dev, const void* src_host, size_t nbytes);   /* worker.py:381-400 */
PTO_API int pto_copy_from(pto_worker* w, void* dst_host, uint64_t src_dev, size_t nbytes);       /* worker.py:402-423 */
/* The same copies enqueued on the worker's stream without waiting for them (a one-shot call stages every
 * argument, launches, reads back and waits once at the end: runner.py:1459-1462 copies before and after a
 * run).  The host buffer must stay valid until pto_synchronize / pto_device_status returns; with pageable
 * host memory the CUDA runtime itself makes the call wait as far as that needs. */
PTO_API int pto_copy_to_async(pto_worker* w, uint64_t dst_dev, const void* src_host, size_t nbytes);
PTO_API int pto_copy_from_async(pto_worker* w, void* dst_host, uint64_t src_dev, size_t nbytes);
PTO_API int pto_synchronize(pto_worker* w);
PTO_API void* pto_worker_stream(pto_worker* w);
/* Reads and clears the device error word of the worker's scratch arena:
 * out[0] code (0 none, 1 a bounded wait ran out, 2 block id outside the pool, 3 an index or row count
 * outside its array: the kernel skipped the access), out[1] site, out[2] CTA, out[3] detail.
 * Synchronises the worker's stream.  Returns PTO_DEVICE_TIMEOUT for code 1 and PTO_INVALID_ARGUMENT
 * for codes 2 and 3 (out is filled either way). */
PTO_API int pto_device_status(pto_worker* w, int32_t out[4]);
/* The worker's scratch arena (grown on demand, never shrunk). */
PTO_API int pto_worker_scratch(pto_worker* w, size_t min_bytes, uint64_t* dev_ptr, size_t* nbytes);

/* Registered callables (replaces Worker.register / Worker.run with a ChipCallable:
 * device_runner.py:651-656, worker.py:532-626).  `op_name` names a fused operator:
 * "paged_attention", "paged_gather", "rms_norm", "ffn_swiglu", "linear", "rope_kv_append", "scope3",
 * "decoder_layer", "matmul_mx" (pto_op_list; tensor and scalar order beside each adapter in csrc/ops.cpp and
 * csrc/layer_ops.cpp). */
PTO_API int pto_register_callable(pto_worker* w, const char* op_name, int32_t* cid);
PTO_API int pto_unregister_callable(pto_worker* w, int32_t cid);
PTO_API int pto_run(pto_worker* w, int32_t cid, const pto_task_args* args);
/* NUL-separated, double-NUL-terminated list of operator names. */
PTO_API const char* pto_op_list(void);

/* External kernels: the reference's plugin hook for hand-written device code,
 * `@pl.function(type=AIV, external_source=...)` / `@pl.jit.extern(source=...)`
 * (python/pypto/jit/decorator.py:2669-2738; the backend references the file instead of
 * generating code, python/pypto/backend/pto_backend.py:1181-1191, 1884-1897; example kernel
 * tests/st/runtime/external_kernel/kernels/aiv/spmd_write.cpp:59-69).
 *   image   a cubin or PTX image for sm_100a (copied; need not outlive the call) that defines
 *           `extern "C" __global__ void <entry>(const int64_t* args)`
 *   launch  `block_num` CTAs (the reference's SPMD blocks: blockIdx.x is the block index) of
 *           `threads_per_block` threads on the worker's stream
 *   args    in device memory, the reference's kernel_entry order: args[0..T-1] are pointers to
 *           one pto_chip_tensor per tensor, args[T..] the scalars bit-cast to 64 bits
 *           (include/pypto_b200_device.h has the accessors).
 * Ids share the space of pto_register_callable and are released by pto_unregister_callable. */
PTO_API int pto_register_kernel_image(pto_worker* w, const void* image, size_t nbytes, const char* entry,
                                      int32_t* cid);
PTO_API int pto_run_kernel(pto_worker* w, int32_t cid, const pto_task_args* args, uint32_t block_num,
                           uint32_t threads_per_block);

/* ---- direct launchers ---- */

/* Paged-attention decode.  Replaces the orchestration `paged_attention` and its four
 * kernels (examples/models/04_paged_attention.py:62-227, 272-367) and the SPMD variant
 * (examples/models/09_paged_attention_spmd.py:503-572).
 *   q            bf16 [batch * q_len * num_heads, head_dim], row = (sequence, draft, head)
 *   k_cache, v_cache  bf16 [pool_blocks * kv_heads * block_size, head_dim],
 *                row = (block, kv head, token)
 *   block_table  int32 [batch, max_blocks]; context_lens int32 [batch]
 *   out          bf16 (out_dtype PTO_BF16) or fp32 (PTO_FP32), same rows as q
 *   q_len > 1    draft token j of a sequence sees its first ctx - q_len + j + 1 keys
 *   scratch      device buffer of at least pto_paged_attention_scratch_bytes() bytes whose
 *                first 64 bytes were zeroed once (error word); reused across calls on
 *                one stream, not shared between concurrent launches. */
PTO_API size_t pto_paged_attention_scratch_bytes(int batch, int num_heads, int kv_heads, int q_len);
PTO_API int pto_paged_attention(const void* q, const void* k_cache, const void* v_cache,
                        const int32_t* block_table, const int32_t* context_lens, void* out,
                        int out_dtype, int batch, int num_heads, int kv_heads, int head_dim,
                        int block_size, int max_blocks, int64_t pool_blocks, int q_len, float scale,
                        void* scratch, size_t scratch_bytes, void* stream);

/* Paged-attention decode for callers that must not allocate.  No counterpart in the
 * reference: it exists for hosts that cannot call cudaMalloc where they launch -- an engine
 * that has already given all free HBM to its KV pool, a plugin living inside another
 * framework's arena, a latency-critical loop that cannot take cudaMalloc's device-wide
 * synchronisation.  Same arguments and results as pto_paged_attention, minus the scratch
 * buffer: the partial softmax rows and the plan go to a fixed 32 MiB array inside the
 * library (present on every GPU that loads it, until the process exits).
 *   - Geometries whose scratch need (pto_paged_attention_scratch_bytes) exceeds 32 MiB are
 *     rejected with PTO_INVALID_ARGUMENT; the benchmark geometry (batch 64, 32/8 heads,
 *     q_len 1: about 22 MiB) fits.
 *   - The first call on a device looks up the array's device address; make that call
 *     before starting any stream capture.  No call allocates or frees device memory.
 *   - All calls on one GPU share the array: launches that overlap on the GPU (different
 *     streams, or two host threads) race and corrupt each other.  Serialise them.
 *   - status_dev (optional, device int32[4]) receives the error word of this call
 *     (0 = none; see pto_device_status for the codes), copied on `stream` after the kernels. */
PTO_API int pto_paged_attention_static(const void* q, const void* k_cache, const void* v_cache,
                               const int32_t* block_table, const int32_t* context_lens, void* out,
                               int out_dtype, int batch, int num_heads, int kv_heads, int head_dim,
                               int block_size, int max_blocks, int64_t pool_blocks, int q_len, float scale,
                               int32_t* status_dev, void* stream);

/* Block-table row gather.  Replaces `pl.paged_gather`
 * (src/ir/op/tensor_ops/paged_gather.cpp:63-169; semantics
 * tests/st/runtime/ops/test_paged_gather.py:14-17):
 *   phys = block_table[idx / block_size] * block_size + idx % block_size
 *   out[i, 0:size] = src[phys, col_off : col_off + size]
 * `elem_bytes` is the element size; rows are copied bit-exactly.  `err` (may be NULL)
 * points at a zeroed int32[4] that receives code 2 if a row falls outside `src_rows`. */
PTO_API int pto_paged_gather(const void* src, int64_t src_rows, int64_t src_cols, int elem_bytes,
                     const int32_t* indices, int64_t n_indices, const int32_t* block_table,
                     int64_t table_len, int block_size, int64_t col_off, int64_t size, void* out,
                     int32_t* err, void* stream);

/* ---- tensor-core linear algebra (weights pre-packed) ---- */

/* One-time weight packing: w [k, n] row-major (fp32 or bf16), the layout of the reference's
 * `x @ W` weights (examples/models/01_ffn.py:157-160) -> packed [n, k] bf16, the K-major
 * operand layout of the tcgen05 GEMM. */
PTO_API int pto_pack_weight(const void* w, int w_dtype, void* packed, int k, int n, void* stream);
/* fp32 <-> bf16 element cast. */
PTO_API int pto_cast(const void* in, int in_dtype, void* out, int out_dtype, int64_t n, void* stream);
/* The same with a side job of the same launch: `zero` (16-byte aligned, zero_bytes a multiple of 16) is
 * cleared -- e.g. the fp32 output that pto_ffn_swiglu then accumulates into. */
PTO_API int pto_cast_zero(const void* in, int in_dtype, void* out, int out_dtype, int64_t n, void* zero,
                          size_t zero_bytes, void* stream);

/* out[m, n] = x[m, k] @ W (accumulate = 0) or out += x @ W (accumulate = 1; out then holds
 * e.g. the residual), x bf16, W packed [n, k] bf16, out fp32, fp32 accumulation.  Replaces the
 * projection kernels of examples/models/qwen3_jit/kernels/projection.py:36-177 and
 * `matmul_kernel` of examples/models/01_ffn.py:37-45.  `err` (may be NULL): device int32[4]
 * error word. */
PTO_API int pto_linear(const void* x, const void* w_packed, void* out, int m, int n, int k, int accumulate,
                       int32_t* err, void* stream);

/* Fused SwiGLU FFN: out[m, n_out] (+)= bf16(silu(x Wg) * (x Wu)) Wd.  Replaces `ffn_swiglu`
 * (examples/models/01_ffn.py:112-131) and `mlp_block` + `down_projection_residual`
 * (examples/models/qwen3_jit/kernels/mlp.py:23-61, kernels/projection.py:146-177).
 *   x bf16 [m, k]; w_gate_up packed [2*inter, k] (gate rows, then up rows);
 *   w_down packed [n_out, inter]; out fp32 [m, n_out];
 *   workspace: device buffer of pto_ffn_swiglu_workspace_bytes(m, inter), 256-byte aligned.  With at most
 *   128 rows both GEMMs run in ONE cooperative launch whose CTAs hand the activation over through counters
 *   in the first 8 KB of the workspace: zero those bytes once after allocating it and leave them to the
 *   operator afterwards (or clear them before every call); one call at a time per workspace. */
PTO_API size_t pto_ffn_swiglu_workspace_bytes(int m, int inter);
PTO_API int pto_ffn_swiglu(const void* x, const void* w_gate_up, const void* w_down, void* out, int m, int k,
                           int inter, int n_out, void* workspace, size_t workspace_bytes, int accumulate,
                           int32_t* err, void* stream);
/* The same with x in fp32 [m, k], the dtype of `ffn_swiglu`'s own inputs (examples/models/01_ffn.py:155-160): x is
 * rounded to bf16 operands.  With at most 128 rows the one-launch kernel does that cast itself, each CTA its share,
 * and clears the output when accumulate = 0: ONE launch for the whole operator.  The workspace
 * (pto_ffn_swiglu_f32_workspace_bytes, 256-byte aligned, same rules as above) also holds the bf16 copy of x. */
PTO_API size_t pto_ffn_swiglu_f32_workspace_bytes(int m, int k, int inter);
PTO_API int pto_ffn_swiglu_f32(const float* x, const void* w_gate_up, const void* w_down, void* out, int m, int k,
                               int inter, int n_out, void* workspace, size_t workspace_bytes, int accumulate,
                               int32_t* err, void* stream);

/* One-projection FFN with an elementwise activation: out[m, n_out] (+)= bf16(f(x W_in)) W_down, with
 * kind 1: f(h) = h * sigmoid(alpha h) (alpha = 1.702 is `ffn_gelu`, examples/models/01_ffn.py:51-62, 92-108), or
 * kind 2: f(h) = max(h, 0) (`ffn_relu`, :80-86, 134-150).  x bf16 [m, k]; w_in packed [inter, k]; w_down packed
 * [n_out, inter]; out fp32.  Workspace: pto_ffn_act_workspace_bytes(m, inter), 256-byte aligned. */
PTO_API size_t pto_ffn_act_workspace_bytes(int m, int inter);
PTO_API int pto_ffn_act(const void* x, const void* w_in, const void* w_down, void* out, int m, int k, int inter,
                        int n_out, int kind, float alpha, void* workspace, size_t workspace_bytes, int accumulate,
                        int32_t* err, void* stream);

/* ---- decoder-layer glue ---- */

/* out = x * rsqrt(mean(x^2) + eps) * gamma, fp32 statistics; x and out fp32 or bf16, gamma
 * fp32 [hidden] or NULL (examples/models/qwen3_jit/kernels/rmsnorm.py:27-89;
 * examples/models/08_llama_mini.py:94-118 is the gamma-free form). */
PTO_API int pto_rms_norm(const void* x, int x_dtype, const float* gamma, void* out, int out_dtype, int64_t rows,
                         int hidden, float eps, void* stream);
/* The same with two optional side jobs that save a decoder layer two launches
 * (examples/models/qwen3_jit/qwen3_decode.py:50-112 runs the norm right before the QKV projection and keeps
 * the un-normalised rows as the residual): copy_f32 (or NULL) receives x as fp32 [rows, hidden];
 * zero (or NULL; 16-byte aligned, zero_bytes a multiple of 16) is cleared, e.g. the fp32 accumulator of the
 * projection that follows. */
PTO_API int pto_rms_norm_ex(const void* x, int x_dtype, const float* gamma, void* out, int out_dtype, int64_t rows,
                            int hidden, float eps, float* copy_f32, void* zero, size_t zero_bytes, void* stream);

/* RoPE (rotate-half) on Q and K at pos = seq_len - 1 and append of the rotated K row and the
 * V row to the paged cache (examples/models/qwen3_jit/kernels/attention.py:40-111).
 *   qkv fp32 [batch, (num_heads + 2*kv_heads) * head_dim]: q heads, k heads, v heads;
 *   cos/sin fp32 [table_rows, head_dim]; caches bf16 [(block, kv head, token), head_dim];
 *   q_out bf16 [batch * num_heads, head_dim]. */
PTO_API int pto_rope_kv_append(const float* qkv, const int32_t* seq_lens, const float* cos_table,
                               const float* sin_table, int table_rows, const int32_t* block_table,
                               int max_blocks, void* k_cache, void* v_cache, void* q_out, int batch,
                               int num_heads, int kv_heads, int head_dim, int block_size, int64_t pool_blocks,
                               int32_t* err, void* stream);

/* act[r, c] = bf16(silu(gate_up[r, c]) * gate_up[r, inter + c]), gate_up fp32 [rows, 2*inter]. */
PTO_API int pto_swiglu_act(const float* gate_up, void* act, int64_t rows, int inter, void* stream);

/* ---- tracing (the reference's run-time diagnostics: RunConfig.enable_chip_swimlane and friends,
 * python/pypto/runtime/runner.py:344-348, docs/en/dev/03-runtime-dfx.md:10-18) ----
 * level 0: off (default; the environment variable PTO_TRACE sets the initial level);
 * level 1: an NVTX range around every registered callable (named after the operator) and around every phase of the
 *          MoE layer's forward call, for timeline tools;
 * level 2: also CUDA events around every pto_run; pto_last_run_ms waits for the last one and returns its device time. */
PTO_API int pto_set_trace(int level);
PTO_API int pto_get_trace(void);
PTO_API int pto_last_run_ms(pto_worker* worker, float* ms);

/* The minimal LLaMA forward pass of examples/models/08_llama_mini.py:384-483 (orchestration `llama_mini_orch`;
 * golden tests/st/examples/03_llm_models/test_llama_7b_mini_1h.py:118-199), all tensors fp32 row-major:
 * hidden [S, D], causal_mask [S, S] (added to the scaled scores), cos_emb / sin_emb [S, D/2], wq wk wv w_dense
 * w_gate w_up w_down [D, D], w_lm [D, V], logits [S, V].  5*S*D + S*S floats must fit in 200 KB. */
PTO_API int pto_llama_mini(const float* hidden, const float* causal_mask, const float* cos_emb, const float* sin_emb,
                           const float* wq, const float* wk, const float* wv, const float* w_dense,
                           const float* w_gate, const float* w_up, const float* w_down, const float* w_lm,
                           float* logits, int seq_len, int head_dim, int vocab, void* stream);

/* ---- mixture of experts ---- */

/* Top-k routing.  `scores` fp32 [tokens, experts] holds gate logits (is_logits = 1: sigmoid is
 * applied) or ready scores (0).  Experts are chosen by the top-k of score + bias (bias may be
 * NULL), listed in descending order, ties to the lower expert id; weight = score / sum of the
 * chosen scores.  The index contract is that of the reference's descending sort with original
 * indices (sort32 + mrgsort + gather, tests/st/runtime/ops/test_sort.py:602-632): exact integers. */
PTO_API int pto_moe_topk(const float* scores, const float* bias, int is_logits, int tokens, int experts,
                         int topk, int32_t* idx, float* weights, void* stream);

/* Per-(row, 128 columns) e4m3 quantisation: scale = amax / 448 (1 for an all-zero group),
 * q = e4m3(x / scale) round-to-nearest-even.  x bf16 or fp32 [rows, cols], cols % 128 == 0. */
PTO_API int pto_quantize_rows(const void* x, int x_dtype, void* q, float* scale, int64_t rows, int cols,
                              void* stream);

/* Dispatch plan (dispatch_step, tests/st/distributed/test_l3_ep_dispatch_combine.py:104-299):
 * bucket of route r is expert_of[r]; inside a bucket routes keep ascending r = t * TOPK + k.
 * Outputs: counts [buckets], offsets [buckets + 1], pos [routes] (slot of each route in the
 * bucket-sorted order), route_at [routes] (inverse).  work: int32 [routes + buckets] work array.
 * An expert id outside [0, buckets) is not dereferenced: the route gets pos = -1, the unused
 * tail of route_at is set to -1 and `err` (device int32[4], may be NULL) receives code 3. */
PTO_API int pto_moe_dispatch_plan(const int32_t* expert_of, int routes, int buckets, int32_t* counts,
                                  int32_t* offsets, int32_t* pos, int32_t* route_at, int32_t* work,
                                  int32_t* err, void* stream);

/* Receiver side of dispatch_step (:184-218): rows arrive source-major and, inside a source, ordered
 * by local expert; recv_counts int32 [world, local_experts] says how many.  Outputs: counts
 * [local_experts]; offsets [local_experts + 1] (dense when slot_stride = 0, e * slot_stride for the
 * reference's padded [L, R] receive layout); arrival_of [capacity] (grouped row -> arrival row, -1
 * where nothing arrives); grouped_of [capacity] (arrival row -> grouped row).  Inside an expert rows
 * are ordered by source rank, then arrival order -- the reference's slot order. */
PTO_API int pto_moe_recv_plan(const int32_t* recv_counts, int world, int local_experts, int slot_stride,
                              int capacity, int32_t* counts, int32_t* offsets, int32_t* arrival_of,
                              int32_t* grouped_of, int32_t* err, void* stream);

/* dst_i[p, :] = src_i[index[p] / div, :] for up to 3 byte arrays with row sizes row_bytes[i]
 * (index NULL: identity).  Bit-exact row copies (the payload move of dispatch_step).  index -1 clears
 * the destination row; any other source row outside [0, src_rows) clears it and sets code 3 in `err`.
 * pto_moe_move_rows is the same with a row stride per source and destination array (NULL = packed),
 * which packs several arrays side by side into one payload row and takes them apart again. */
PTO_API int pto_moe_gather_rows(const void* const* src, void* const* dst, const int* row_bytes, int n_arrays,
                                const int32_t* index, int div, int64_t rows, int64_t src_rows, int32_t* err,
                                void* stream);
PTO_API int pto_moe_move_rows(const void* const* src, const int64_t* src_stride, void* const* dst,
                              const int64_t* dst_stride, const int* row_bytes, int n_arrays, const int32_t* index,
                              int div, int64_t rows, int64_t src_rows, int32_t* err, void* stream);
PTO_API int pto_moe_gather_f32(const float* src, const int32_t* index, int64_t n, int64_t n_src, float* dst,
                               int32_t* err, void* stream);

/* y[r, :] = bf16(fp32(x[r, :]) * w[r * w_stride]) over bf16 rows: the stand-in expert of the reference's
 * expert-parallel test (local_expert_step, test_l3_ep_dispatch_combine.py:309-327).  With `count`
 * (int32 [rows / slot_stride]) only the first count[e] rows of each block of slot_stride rows are written. */
PTO_API int pto_scale_rows(const void* x, const float* w, int w_stride, const int32_t* count, int slot_stride,
                           int64_t rows, int cols, void* y, void* stream);

/* Grouped FP8 expert GEMM over tokens sorted by expert (replaces local_expert_step,
 * test_l3_ep_dispatch_combine.py:309-327, by the SwiGLU expert FFN).
 *   w fp8 [experts * w_rows, k] K-major, w_scale fp32 [experts][w_rows / 128][k / 128]
 *   x fp8 [rows, k], x_scale fp32 [rows][k / 128], offsets int32 [experts + 1]
 * swiglu = 1: w_rows = 2 * n_out (gate rows then up rows); out bf16 [rows, n_out] =
 *             bf16(silu(gate) * up) (re-quantise it with pto_quantize_rows for the down projection).
 * swiglu = 0: w_rows = n_out; out bf16 [rows, n_out]: row (out_rows ? out_rows[r] : r) = acc[r] * route_w[r]
 *             (route_w may be NULL; out_rows, int32 [rows] or NULL, lets the expert-parallel receiver get its
 *             results back in the order the rows arrived in, ready to be sent home; a mapped row outside
 *             [0, rows) is not written). */
PTO_API int pto_moe_expert_gemm(int swiglu, const void* w, const float* w_scale, int experts, int w_rows,
                                int n_out, int k, const void* x, const float* x_scale, const int32_t* offsets,
                                int rows, const float* route_w, const int32_t* out_rows, void* out, int32_t* err,
                                void* stream);

/* Combine (combine_step, test_l3_ep_dispatch_combine.py:337-402): y[t] = sum_k fp32(rows[pos[t*topk+k]])
 * (+ fp32(shared[t]) if given), k ascending; written as bf16 (y_bf16) and/or fp32 (y_f32).  `rows` holds
 * n_rows bf16 rows; a pos outside [0, n_rows) contributes nothing. */
PTO_API int pto_moe_combine(const void* rows, const int32_t* pos, const void* shared, int tokens, int topk,
                            int hidden, int64_t n_rows, void* y_bf16, float* y_f32, void* stream);

/* The return path of the expert-parallel layer as two calls (pto_moe_layer_forward issues them itself): result
 * rows in arrival order -- source rank after source rank, recv_counts int32 [world][local_experts] rows from each --
 * are stored block by block into the sorted result buffers of their sources, back[r] + dst_base[r] * row_bytes
 * (device pointers of this process; another rank's buffer is one mapped from its CUDA IPC handle), and then
 * flags[r][my_rank] = step on every rank r.  row_bytes a multiple of 16; dst_rows = rows a result buffer holds
 * (a block that would not fit is refused through the error word); done_counter: one zeroed int32 on the device,
 * left at zero; rows_hint sizes the grid.  pto_moe_wait_flags: one warp waits, for at most two seconds, until
 * flags[r] >= step for every r < world, then the error word says which rank did not show (PTO_DEVICE_TIMEOUT). */
PTO_API int pto_moe_push_rows(const void* rows, int row_bytes, const int32_t* recv_counts, int world, int local_experts,
                              const int32_t* dst_base, void* const* back, int32_t* const* flags, int my_rank, int step,
                              int64_t dst_rows, int64_t rows_hint, int32_t* done_counter, int32_t* err, void* stream);
PTO_API int pto_moe_wait_flags(const int32_t* flags, int world, int step, int32_t* err, void* stream);

/* ---- MX block-scaled FP8 matmul ---- */

/* out[m, n] = (acc_in[m, n] +) sum_k a[m, k] * 2^(sa[m, k/32] - 127) * b[k, n] * 2^(sb[k/32, n] - 127).
 * Replaces tile.matmul_mx / tile.matmul_mx_acc (src/ir/op/tile_ops/matmul_mx.cpp:321-345; golden
 * tests/st/runtime/ops/test_matmul_mx.py:119-131) on the hardware block-scaled path
 * (tcgen05.mma kind::mxf8f6f4.block_scale, E8M0 scales staged in tensor memory).
 *   a          e4m3 [m, k] row-major; k a multiple of 32
 *   b_t        e4m3 [n, k]: the right operand with K contiguous (pto_transpose_u8 of the
 *              reference's [k, n] tensor, done once for a resident weight)
 *   a_scale    E8M0 codes, uint8 [m, k/32]; b_scale uint8 [k/32, n]
 *   *_layout   PTO_MX_SCALE_LOGICAL (row-major as written above), PTO_MX_SCALE_A_ZZ / PTO_MX_SCALE_B_NN:
 *              the physical orders the reference hands its kernel (test_matmul_mx.py:38-101;
 *              these need m, n multiples of 16 and k/32 even)
 *   acc_in     fp32 [m, n] added to the product (matmul_mx_acc), or NULL; may alias out
 *   out        fp32 [m, n]
 * Large problems (m >= 512, n >= 448, k >= 1024, at least two 256 x 224 tiles per pair of SMs) run on SM pairs;
 * that path first rewrites the scale codes in the tensor core's order into scratch memory of (m + n) * k / 32 bytes
 * (rounded up to whole tiles) taken in stream order from a memory pool of the library's own (cudaMallocFromPoolAsync /
 * cudaFreeAsync on `stream`, no synchronisation; capturable in a graph; the pool keeps its memory between calls).  Environment: PTO_MX_PAIR=0 keeps every problem on the
 * one-CTA kernel, which allocates nothing. */
enum { PTO_MX_SCALE_LOGICAL = 0, PTO_MX_SCALE_A_ZZ = 1, PTO_MX_SCALE_B_NN = 2 };
PTO_API int pto_matmul_mx(const void* a, const void* a_scale, int a_scale_layout, const void* b_t,
                          const void* b_scale, int b_scale_layout, const float* acc_in, float* out, int m, int n,
                          int k, int32_t* err, void* stream);
/* dst[c, r] = src[r, c] for a byte matrix src [rows, cols] (operand re-layout for pto_matmul_mx). */
PTO_API int pto_transpose_u8(const void* src, void* dst, int64_t rows, int64_t cols, void* stream);

/* ---- communicator: one rank per GPU, NCCL over NVLink ---- */

/* Replaces the communication-domain set-up of the reference's level-3 runtime and its all_to_all /
 * all_to_all_v builtins (python/pypto/runtime/builtins/collectives/all_to_all_v/templates/
 * kernel.cpp.in:96-160; DistributedWorker, python/pypto/runtime/distributed_runner.py:1442).
 * One process (or thread) per GPU creates one communicator; rank 0 makes the 128-byte id with
 * pto_comm_unique_id and hands it to the others by any host channel.  pto_comm_init is collective:
 * every rank must call it.  NCCL is looked up at run time; without it these return PTO_UNSUPPORTED. */
#define PTO_UNIQUE_ID_BYTES 128
typedef struct pto_comm pto_comm;
PTO_API int pto_comm_unique_id(void* id_out);
PTO_API int pto_comm_init(int rank, int nranks, const void* unique_id, int device_id, pto_comm** out);
PTO_API int pto_comm_destroy(pto_comm* c); /* idempotent on NULL */
PTO_API int pto_comm_rank(const pto_comm* c);
PTO_API int pto_comm_size(const pto_comm* c);
PTO_API int pto_comm_nccl_version(void);   /* 0 when NCCL could not be loaded */
/* Rank r's block p of `send` (bytes_per_rank each) lands in rank p's block r of `recv`. */
PTO_API int pto_all_to_all(pto_comm* c, const void* send, void* recv, size_t bytes_per_rank, void* stream);
/* This rank sends send_rows[p] consecutive rows of `send` to rank p and receives recv_rows[p] rows from
 * rank p, stored in source-rank order in `recv`; exact counts (host arrays of nranks entries, typically
 * from a pto_all_to_all of the counts).  Rows for this rank itself are a device copy. */
PTO_API int pto_all_to_all_v(pto_comm* c, const void* send, const int64_t* send_rows, void* recv,
                             const int64_t* recv_rows, size_t row_bytes, void* stream);

/* ---- the mixture-of-experts layer as one runtime object ---- */

/* Gate + top-k routing, dispatch, grouped FP8 expert FFN and combine behind one call; with a communicator the
 * experts are split over its ranks (global expert e on rank e / (n_experts / nranks)) and a forward call performs
 * the reference's dispatch_step / local_expert_step / combine_step protocol
 * (tests/st/distributed/test_l3_ep_dispatch_combine.py:104-402) with one payload exchange each way.
 * Weights stay owned by the caller and must outlive the layer:
 *   gate_packed  bf16 [n_experts, hidden] (pto_pack_weight of the [hidden, n_experts] gate); bias fp32 [n_experts]
 *   w_gu e4m3 [local, 2*inter, hidden] (gate rows, then up rows), s_gu fp32 [local, 2*inter/128, hidden/128]
 *   w_d  e4m3 [local, hidden, inter],   s_d  fp32 [local, hidden/128, inter/128]
 *   sh_* the same for one shared expert, or all NULL
 * pto_moe_layer_create allocates every buffer a step needs, sized for max_tokens tokens per call and the worst
 * case of rows arriving at this rank; with a communicator it and every forward call are collective.
 * Return path through peer memory: when every rank of the communicator can map every other rank's buffers (one
 * node; CUDA IPC handles go round inside pto_moe_layer_create and all ranks agree on the outcome; the environment
 * variable PTO_EP_PEER=0 on any rank turns it off for all), the result rows do not travel through a collective:
 * each rank stores them into their source's buffer with its own kernel and raises a flag there
 * (pto_moe_layer_peer_exchange tells).  Destroy such layers on all ranks only after all of them have finished their
 * last forward call (every rank's buffers are mapped by the others until each has destroyed its layer). */
typedef struct pto_moe_layer_desc {
  int hidden, inter, n_experts, topk, max_tokens;
  const void* gate_packed;
  const float* bias;
  const void* w_gu; const float* s_gu; const void* w_d; const float* s_d;
  const void* sh_w_gu; const float* sh_s_gu; const void* sh_w_d; const float* sh_s_d;
  pto_comm* comm; /* NULL: one GPU, all experts local */
} pto_moe_layer_desc;
typedef struct pto_moe_layer pto_moe_layer;
PTO_API int pto_moe_layer_create(const pto_moe_layer_desc* desc, pto_moe_layer** out);
PTO_API int pto_moe_layer_destroy(pto_moe_layer* layer); /* idempotent on NULL */
PTO_API int pto_moe_layer_peer_exchange(const pto_moe_layer* layer); /* 0: collectives; 1: results return through peer
                                                                       * memory; 2 (PTO_EP_PEER=2 on every rank): the
                                                                       * dispatched rows go out through it as well */
/* x bf16 [tokens, hidden] -> y bf16 [tokens, hidden].  idx_in / w_in (int32 / fp32 [tokens, topk], both or
 * neither) replace the layer's own routing; idx_out / w_out (may be NULL) receive the routing used.  phase_ms
 * (host float[8] or NULL) receives the device time of route+quantise, plan, pack, exchange out, unpack, experts,
 * exchange back, combine; asking for it makes the call wait for the step.  The host waits once per call for the
 * row counts of the exchange (not at all on one GPU). */
PTO_API int pto_moe_layer_forward(pto_moe_layer* layer, const void* x, int tokens, const int32_t* idx_in,
                                  const float* w_in, void* y, int32_t* idx_out, float* w_out, float* phase_ms,
                                  void* stream);
/* Reads (and clears) the layer's device error word, see pto_device_status; synchronises `stream`. */
PTO_API int pto_moe_layer_status(pto_moe_layer* layer, int32_t out[4], void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PYPTO_B200_H_ */
