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

struct Worker {
  int device = 0;
  cudaStream_t stream = nullptr;
  std::mutex mu;
  std::map<uint64_t, size_t> allocs;  // device pointers handed out by pto_malloc
  std::map<int32_t, OpFn> callables;
  int32_t next_cid = 1;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  ~Worker();
  int ensure_scratch(size_t nbytes);
};

OpFn find_op(const char* name);

}  // namespace pto
