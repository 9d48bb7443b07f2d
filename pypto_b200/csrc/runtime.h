// Worker object and operator registry (host side, internal).
#pragma once

#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <string>

#include "pypto_b200.h"

namespace pto {

struct Worker;
using OpFn = int (*)(Worker*, const pto_task_args*);

// A user kernel loaded from a cubin / PTX image (pto_register_kernel_image).
struct ExternKernel {
  cudaLibrary_t library = nullptr;
  cudaKernel_t kernel = nullptr;
  void* args_dev = nullptr;   // ring of argument blocks: the launch reads its block from device memory
  uint32_t next_slot = 0;
};
constexpr uint32_t kExternArgSlots = 32;
constexpr size_t kExternArgSlotBytes = 4096;

struct Worker {
  int device = 0;
  cudaStream_t stream = nullptr;
  std::mutex mu;
  std::map<uint64_t, size_t> allocs;  // device pointers handed out by pto_malloc
  std::map<int32_t, OpFn> callables;
  std::map<int32_t, std::string> callable_names;   // for trace ranges
  cudaEvent_t trace_ev[2] = {nullptr, nullptr};    // device time of the last traced pto_run
  bool trace_valid = false;
  std::map<int32_t, ExternKernel> kernels;   // share the id space of `callables`
  int32_t next_cid = 1;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  // the mixture-of-experts layer object behind the "moe_layer" callable: built on first use, rebuilt when the
  // weights or sizes of a call differ from the ones it was built for
  pto_moe_layer* moe = nullptr;
  pto_moe_layer_desc moe_desc = {};
  ~Worker();
  int ensure_scratch(size_t nbytes);
};

OpFn find_op(const char* name);

// Tracing (pto_set_trace): 0 off; 1 = an NVTX range around every registered callable and every phase of the MoE layer;
// 2 = also CUDA events around every callable, read back with pto_last_run_ms.
int trace_level();
struct TraceRange {   // NVTX push / pop when tracing is on
  explicit TraceRange(const char* name);
  ~TraceRange();
  bool on;
};

// layer_ops.cpp: callables composed of several kernels
int op_scope3(Worker* w, const pto_task_args* a);
int op_decoder_layer(Worker* w, const pto_task_args* a);
int op_linear(Worker* w, const pto_task_args* a);
int op_rope_kv_append(Worker* w, const pto_task_args* a);
int op_matmul_mx(Worker* w, const pto_task_args* a);
int op_moe_layer(Worker* w, const pto_task_args* a);
int op_llama_mini(Worker* w, const pto_task_args* a);

}  // namespace pto
