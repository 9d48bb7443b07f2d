// Host runtime behind the C ABI: worker object (device, stream, allocations,
// scratch arena), registered callables, error plumbing, tensor-map encoding.
// It stands where the reference loads its external device runtime
// (python/pypto/runtime/device_runner.py:821-842).
#include <nvtx3/nvToolsExt.h>

#include <atomic>
#include "runtime.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "pypto_b200.h"

namespace pto {

namespace {
thread_local std::string g_last_error;
}

void set_last_error(const std::string& msg) { g_last_error = msg; }

int fail(int status, const std::string& msg) {
  g_last_error = msg;
  return status;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return kOk;
  g_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
  return e == cudaErrorMemoryAllocation ? kOutOfMemory : kCudaError;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("PTO_PDL");
    return v == nullptr || v[0] != '0';
  }();
  return on;
}

namespace {
std::atomic<int> g_trace_level{-1};
}

int trace_level() {
  int v = g_trace_level.load(std::memory_order_relaxed);
  if (v < 0) {   // first use: the environment decides until pto_set_trace is called
    const char* e = getenv("PTO_TRACE");
    v = e ? atoi(e) : 0;
    if (v < 0) v = 0;
    g_trace_level.store(v, std::memory_order_relaxed);
  }
  return v;
}

TraceRange::TraceRange(const char* name) : on(trace_level() >= 1) {
  if (on) nvtxRangePushA(name);
}
TraceRange::~TraceRange() {
  if (on) nvtxRangePop();
}

bool first_use_on_device(int key) {
  static std::mutex mu;
  static bool seen[32][64] = {};
  int dev = 0;
  if (key < 0 || key >= 32 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
  std::lock_guard<std::mutex> g(mu);
  const bool first = !seen[key][dev];
  seen[key][dev] = true;
  return first;
}

// Stream-ordered scratch memory from a pool of the library's own (one per device).  The pool keeps what it has
// been given (release threshold = everything): with the default threshold a pool hands its memory back to the driver
// at every synchronisation, and the next call pays for mapping it again.
int scratch_alloc_async(void** out, size_t bytes, cudaStream_t stream) {
  static std::mutex mu;
  static cudaMemPool_t pools[64] = {};
  int dev = 0;
  PTO_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(kInvalidArgument, "scratch_alloc_async: device ordinal out of range");
  cudaMemPool_t pool;
  {
    std::lock_guard<std::mutex> g(mu);
    if (pools[dev] == nullptr) {
      cudaMemPoolProps props = {};
      props.allocType = cudaMemAllocationTypePinned;
      props.handleTypes = cudaMemHandleTypeNone;
      props.location.type = cudaMemLocationTypeDevice;
      props.location.id = dev;
      PTO_CUDA(cudaMemPoolCreate(&pools[dev], &props));
      unsigned long long keep = ~0ull;
      PTO_CUDA(cudaMemPoolSetAttribute(pools[dev], cudaMemPoolAttrReleaseThreshold, &keep));
    }
    pool = pools[dev];
  }
  PTO_CUDA(cudaMallocFromPoolAsync(out, bytes, pool, stream));
  return kOk;
}

int scratch_free_async(void* p, cudaStream_t stream) {
  PTO_CUDA(cudaFreeAsync(p, stream));
  return kOk;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

int make_tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                       uint64_t rows, uint64_t cols, uint64_t row_stride_bytes, uint32_t box_cols,
                       uint32_t box_rows, CUtensorMapSwizzle swizzle) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return fail(kCudaError, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride_bytes & 15) != 0)
    return fail(kInvalidArgument, "tensor map: base and row stride must be multiples of 16 bytes");
  if (box_cols * static_cast<uint64_t>(elem_bytes) % 16 != 0 || box_rows == 0 || box_rows > 256 || box_cols > 256)
    return fail(kInvalidArgument, "tensor map: bad box");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu cols=%llu box=%ux%u)",
             static_cast<int>(r), (unsigned long long)rows, (unsigned long long)cols, box_cols, box_rows);
    return fail(kCudaError, buf);
  }
  return kOk;
}

// ------------------------------- Worker -----------------------------------

Worker::~Worker() {
  cudaSetDevice(device);
  for (auto& kv : allocs) cudaFree(reinterpret_cast<void*>(kv.first));
  allocs.clear();
  for (auto& kv : kernels) {
    if (kv.second.args_dev) cudaFree(kv.second.args_dev);
    if (kv.second.library) cudaLibraryUnload(kv.second.library);
  }
  kernels.clear();
  for (cudaEvent_t e : trace_ev) if (e) cudaEventDestroy(e);
  if (moe) pto_moe_layer_destroy(moe);
  if (scratch) cudaFree(scratch);
  if (stream) cudaStreamDestroy(stream);
}

int Worker::ensure_scratch(size_t nbytes) {
  if (nbytes <= scratch_bytes) return kOk;
  PTO_CUDA(cudaSetDevice(device));
  PTO_CUDA(cudaStreamSynchronize(stream));
  size_t want = nbytes < (size_t(1) << 20) ? (size_t(1) << 20) : nbytes;
  void* p = nullptr;
  PTO_CUDA(cudaMalloc(&p, want));
  cudaError_t e = cudaMemsetAsync(p, 0, 256, stream);
  if (e != cudaSuccess) { cudaFree(p); return check_cuda(e, "cudaMemsetAsync(scratch)"); }
  if (scratch) cudaFree(scratch);
  scratch = p;
  scratch_bytes = want;
  return kOk;
}

}  // namespace pto

using pto::Worker;

extern "C" {

const char* pto_last_error(void) { return pto::g_last_error.c_str(); }
const char* pto_version(void) { return "pypto-b200 0.1 (sm_100a)"; }

int pto_worker_create(int device_id, pto_worker** out) {
  if (out == nullptr) return pto::fail(pto::kInvalidArgument, "worker_create: out is NULL");
  *out = nullptr;
  int n = 0;
  PTO_CUDA(cudaGetDeviceCount(&n));
  if (device_id < 0 || device_id >= n) return pto::fail(pto::kInvalidArgument, "worker_create: no such device");
  PTO_CUDA(cudaSetDevice(device_id));
  Worker* w = new (std::nothrow) Worker();
  if (w == nullptr) return pto::fail(pto::kOutOfMemory, "worker_create: host allocation failed");
  w->device = device_id;
  cudaError_t e = cudaStreamCreateWithFlags(&w->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) { delete w; return pto::check_cuda(e, "cudaStreamCreate"); }
  *out = reinterpret_cast<pto_worker*>(w);
  return pto::kOk;
}

int pto_worker_destroy(pto_worker* h) {
  if (h == nullptr) return pto::kOk;
  Worker* w = reinterpret_cast<Worker*>(h);
  cudaSetDevice(w->device);
  cudaStreamSynchronize(w->stream);
  delete w;
  return pto::kOk;
}

#define PTO_WORKER(h)                                                              \
  Worker* w = reinterpret_cast<Worker*>(h);                                        \
  if (w == nullptr) return pto::fail(pto::kInvalidArgument, "worker handle is NULL"); \
  PTO_CUDA(cudaSetDevice(w->device))

int pto_malloc(pto_worker* h, size_t nbytes, uint64_t* dev_ptr) {
  PTO_WORKER(h);
  if (dev_ptr == nullptr) return pto::fail(pto::kInvalidArgument, "malloc: dev_ptr is NULL");
  void* p = nullptr;
  PTO_CUDA(cudaMalloc(&p, nbytes == 0 ? 1 : nbytes));
  std::lock_guard<std::mutex> g(w->mu);
  w->allocs[reinterpret_cast<uint64_t>(p)] = nbytes;
  *dev_ptr = reinterpret_cast<uint64_t>(p);
  return pto::kOk;
}

int pto_free(pto_worker* h, uint64_t dev_ptr) {
  PTO_WORKER(h);
  {
    std::lock_guard<std::mutex> g(w->mu);
    auto it = w->allocs.find(dev_ptr);
    if (it == w->allocs.end()) return pto::fail(pto::kNotFound, "free: pointer is not owned by this worker (double free?)");
    w->allocs.erase(it);
  }
  PTO_CUDA(cudaStreamSynchronize(w->stream));
  PTO_CUDA(cudaFree(reinterpret_cast<void*>(dev_ptr)));
  return pto::kOk;
}

int pto_copy_to(pto_worker* h, uint64_t dst_dev, const void* src_host, size_t nbytes) {
  PTO_WORKER(h);
  if (nbytes == 0) return pto::kOk;
  if (src_host == nullptr || dst_dev == 0) return pto::fail(pto::kInvalidArgument, "copy_to: NULL pointer");
  PTO_CUDA(cudaMemcpyAsync(reinterpret_cast<void*>(dst_dev), src_host, nbytes, cudaMemcpyHostToDevice, w->stream));
  PTO_CUDA(cudaStreamSynchronize(w->stream));
  return pto::kOk;
}

int pto_copy_from(pto_worker* h, void* dst_host, uint64_t src_dev, size_t nbytes) {
  PTO_WORKER(h);
  if (nbytes == 0) return pto::kOk;
  if (dst_host == nullptr || src_dev == 0) return pto::fail(pto::kInvalidArgument, "copy_from: NULL pointer");
  PTO_CUDA(cudaMemcpyAsync(dst_host, reinterpret_cast<const void*>(src_dev), nbytes, cudaMemcpyDeviceToHost, w->stream));
  PTO_CUDA(cudaStreamSynchronize(w->stream));
  return pto::kOk;
}

int pto_copy_to_async(pto_worker* h, uint64_t dst_dev, const void* src_host, size_t nbytes) {
  PTO_WORKER(h);
  if (nbytes == 0) return pto::kOk;
  if (src_host == nullptr || dst_dev == 0) return pto::fail(pto::kInvalidArgument, "copy_to_async: NULL pointer");
  PTO_CUDA(cudaMemcpyAsync(reinterpret_cast<void*>(dst_dev), src_host, nbytes, cudaMemcpyHostToDevice, w->stream));
  return pto::kOk;
}

int pto_copy_from_async(pto_worker* h, void* dst_host, uint64_t src_dev, size_t nbytes) {
  PTO_WORKER(h);
  if (nbytes == 0) return pto::kOk;
  if (dst_host == nullptr || src_dev == 0) return pto::fail(pto::kInvalidArgument, "copy_from_async: NULL pointer");
  PTO_CUDA(cudaMemcpyAsync(dst_host, reinterpret_cast<const void*>(src_dev), nbytes, cudaMemcpyDeviceToHost, w->stream));
  return pto::kOk;
}

int pto_synchronize(pto_worker* h) {
  PTO_WORKER(h);
  PTO_CUDA(cudaStreamSynchronize(w->stream));
  return pto::kOk;
}

void* pto_worker_stream(pto_worker* h) {
  return h ? reinterpret_cast<Worker*>(h)->stream : nullptr;
}

int pto_worker_scratch(pto_worker* h, size_t min_bytes, uint64_t* dev_ptr, size_t* nbytes) {
  PTO_WORKER(h);
  int st = w->ensure_scratch(min_bytes < 256 ? 256 : min_bytes);
  if (st != pto::kOk) return st;
  if (dev_ptr) *dev_ptr = reinterpret_cast<uint64_t>(w->scratch);
  if (nbytes) *nbytes = w->scratch_bytes;
  return pto::kOk;
}

int pto_device_status(pto_worker* h, int32_t out[4]) {
  PTO_WORKER(h);
  int32_t words[4] = {0, 0, 0, 0};
  PTO_CUDA(cudaStreamSynchronize(w->stream));
  if (w->scratch) {
    PTO_CUDA(cudaMemcpyAsync(words, w->scratch, sizeof words, cudaMemcpyDeviceToHost, w->stream));
    PTO_CUDA(cudaStreamSynchronize(w->stream));
    if (words[0] != 0) {
      PTO_CUDA(cudaMemsetAsync(w->scratch, 0, 64, w->stream));
      PTO_CUDA(cudaStreamSynchronize(w->stream));
    }
  }
  if (out) memcpy(out, words, sizeof words);
  if (words[0] == pto::kErrBarrierTimeout) {
    char buf[128];
    snprintf(buf, sizeof buf, "device wait timed out (site %d, CTA %d, detail %d)", words[1], words[2], words[3]);
    return pto::fail(pto::kDeviceTimeout, buf);
  }
  if (words[0] == pto::kErrBadBlockId) {
    char buf[128];
    snprintf(buf, sizeof buf, "block id or row outside the pool (site %d, CTA %d, value %d)", words[1], words[2], words[3]);
    return pto::fail(pto::kInvalidArgument, buf);
  }
  if (words[0] == pto::kErrBadIndex) {
    char buf[128];
    snprintf(buf, sizeof buf, "index or row count outside its array, access skipped (site %d, CTA %d, value %d)",
             words[1], words[2], words[3]);
    return pto::fail(pto::kInvalidArgument, buf);
  }
  return pto::kOk;
}

int pto_register_callable(pto_worker* h, const char* op_name, int32_t* cid) {
  PTO_WORKER(h);
  if (op_name == nullptr || cid == nullptr) return pto::fail(pto::kInvalidArgument, "register: NULL argument");
  pto::OpFn fn = pto::find_op(op_name);
  if (fn == nullptr) return pto::fail(pto::kNotFound, std::string("no fused kernel registered for '") + op_name + "'");
  std::lock_guard<std::mutex> g(w->mu);
  int32_t id = w->next_cid++;
  w->callables[id] = fn;
  w->callable_names[id] = op_name;
  *cid = id;
  return pto::kOk;
}

int pto_unregister_callable(pto_worker* h, int32_t cid) {
  PTO_WORKER(h);
  std::lock_guard<std::mutex> g(w->mu);
  auto k = w->kernels.find(cid);
  if (k != w->kernels.end()) {
    PTO_CUDA(cudaStreamSynchronize(w->stream));   // a launch may still read its argument block
    if (k->second.args_dev) cudaFree(k->second.args_dev);
    if (k->second.library) cudaLibraryUnload(k->second.library);
    w->kernels.erase(k);
    return pto::kOk;
  }
  if (w->callables.erase(cid) == 0) return pto::fail(pto::kNotFound, "unregister: unknown callable id");
  return pto::kOk;
}

int pto_register_kernel_image(pto_worker* h, const void* image, size_t nbytes, const char* entry, int32_t* cid) {
  PTO_WORKER(h);
  if (image == nullptr || nbytes == 0 || entry == nullptr || cid == nullptr)
    return pto::fail(pto::kInvalidArgument, "register_kernel_image: NULL or empty argument");
  pto::ExternKernel k;
  // The image is copied by the loader; it need not outlive this call.
  cudaError_t e = cudaLibraryLoadData(&k.library, image, nullptr, nullptr, 0, nullptr, nullptr, 0);
  if (e != cudaSuccess) return pto::check_cuda(e, "cudaLibraryLoadData (is the image built for sm_100a?)");
  e = cudaLibraryGetKernel(&k.kernel, k.library, entry);
  if (e != cudaSuccess) {
    cudaLibraryUnload(k.library);
    cudaGetLastError();
    return pto::fail(pto::kNotFound, std::string("kernel image has no extern \"C\" __global__ entry '") + entry + "'");
  }
  e = cudaMalloc(&k.args_dev, pto::kExternArgSlots * pto::kExternArgSlotBytes);
  if (e != cudaSuccess) {
    cudaLibraryUnload(k.library);
    return pto::check_cuda(e, "cudaMalloc(kernel argument ring)");
  }
  std::lock_guard<std::mutex> g(w->mu);
  int32_t id = w->next_cid++;
  w->kernels[id] = k;
  *cid = id;
  return pto::kOk;
}

int pto_run_kernel(pto_worker* h, int32_t cid, const pto_task_args* args, uint32_t block_num,
                   uint32_t threads_per_block) {
  PTO_WORKER(h);
  if (args == nullptr) return pto::fail(pto::kInvalidArgument, "run_kernel: args is NULL");
  if (block_num == 0 || threads_per_block == 0 || threads_per_block > 1024)
    return pto::fail(pto::kInvalidArgument, "run_kernel: block_num >= 1 and 1 <= threads_per_block <= 1024");
  if ((args->n_tensors && !args->tensors) || (args->n_scalars && !args->scalars))
    return pto::fail(pto::kInvalidArgument, "run_kernel: NULL tensor or scalar array");
  // block layout: a 16-byte header {address of the worker's device error word, reserved}, then what the kernel
  // receives: int64 args[n_tensors + n_scalars], padded to 16 bytes, then the tensor descriptors
  constexpr size_t kHeader = 16;
  const size_t n = static_cast<size_t>(args->n_tensors) + args->n_scalars;
  const size_t desc_off = kHeader + ((n * sizeof(int64_t) + 15) & ~static_cast<size_t>(15));
  const size_t total = desc_off + args->n_tensors * sizeof(pto_chip_tensor);
  if (total > pto::kExternArgSlotBytes) return pto::fail(pto::kInvalidArgument, "run_kernel: too many arguments");
  cudaKernel_t kernel = nullptr;
  uint8_t* slot = nullptr;
  {
    std::lock_guard<std::mutex> g(w->mu);
    auto it = w->kernels.find(cid);
    if (it == w->kernels.end()) return pto::fail(pto::kNotFound, "run_kernel: unknown kernel id");
    kernel = it->second.kernel;
    slot = static_cast<uint8_t*>(it->second.args_dev) +
           (it->second.next_slot++ % pto::kExternArgSlots) * pto::kExternArgSlotBytes;
  }
  {
    const int st = w->ensure_scratch(4096);   // the error word lives at the start of the worker's scratch arena
    if (st != pto::kOk) return st;
  }
  alignas(16) uint8_t block[pto::kExternArgSlotBytes];
  reinterpret_cast<int64_t*>(block)[0] = static_cast<int64_t>(reinterpret_cast<uintptr_t>(w->scratch));
  reinterpret_cast<int64_t*>(block)[1] = 0;
  int64_t* a = reinterpret_cast<int64_t*>(block + kHeader);
  for (uint32_t i = 0; i < args->n_tensors; ++i)
    a[i] = static_cast<int64_t>(reinterpret_cast<uintptr_t>(slot + desc_off + i * sizeof(pto_chip_tensor)));
  for (uint32_t i = 0; i < args->n_scalars; ++i) a[args->n_tensors + i] = static_cast<int64_t>(args->scalars[i]);
  if (args->n_tensors) memcpy(block + desc_off, args->tensors, args->n_tensors * sizeof(pto_chip_tensor));
  // Pageable source: the runtime stages it before returning, so `block` may go out of scope.  The ring slot is
  // reused only after kExternArgSlots later launches on the same stream, i.e. after this launch has finished.
  PTO_CUDA(cudaMemcpyAsync(slot, block, total, cudaMemcpyHostToDevice, w->stream));
  void* dev_args = slot + kHeader;
  void* params[] = {&dev_args};
  PTO_CUDA(cudaLaunchKernel(reinterpret_cast<const void*>(kernel), dim3(block_num), dim3(threads_per_block), params, 0,
                            w->stream));
  return pto::kOk;
}

int pto_run(pto_worker* h, int32_t cid, const pto_task_args* args) {
  PTO_WORKER(h);
  if (args == nullptr) return pto::fail(pto::kInvalidArgument, "run: args is NULL");
  pto::OpFn fn = nullptr;
  const char* name = "callable";
  {
    std::lock_guard<std::mutex> g(w->mu);
    auto it = w->callables.find(cid);
    if (it == w->callables.end()) return pto::fail(pto::kNotFound, "run: unknown callable id");
    fn = it->second;
    auto nm = w->callable_names.find(cid);
    if (nm != w->callable_names.end()) name = nm->second.c_str();   // map nodes are stable while the id is registered
  }
  const int level = pto::trace_level();
  if (level < 1) return fn(w, args);
  pto::TraceRange range(name);
  if (level >= 2) {
    for (cudaEvent_t& e : w->trace_ev)
      if (e == nullptr) PTO_CUDA(cudaEventCreate(&e));
    PTO_CUDA(cudaEventRecord(w->trace_ev[0], w->stream));
  }
  const int st = fn(w, args);
  if (level >= 2 && st == pto::kOk) {
    PTO_CUDA(cudaEventRecord(w->trace_ev[1], w->stream));
    w->trace_valid = true;
  }
  return st;
}

int pto_set_trace(int level) {
  if (level < 0 || level > 2) return pto::fail(pto::kInvalidArgument, "set_trace: level must be 0, 1 or 2");
  pto::g_trace_level.store(level, std::memory_order_relaxed);
  return pto::kOk;
}

int pto_get_trace(void) { return pto::trace_level(); }

int pto_last_run_ms(pto_worker* h, float* ms) {
  PTO_WORKER(h);
  if (ms == nullptr) return pto::fail(pto::kInvalidArgument, "last_run_ms: ms is NULL");
  if (!w->trace_valid) return pto::fail(pto::kNotFound, "last_run_ms: no callable has run with trace level 2 on this worker");
  PTO_CUDA(cudaEventSynchronize(w->trace_ev[1]));
  PTO_CUDA(cudaEventElapsedTime(ms, w->trace_ev[0], w->trace_ev[1]));
  return pto::kOk;
}

}  // extern "C"
