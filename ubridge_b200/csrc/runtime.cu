// Host runtime of the shim: status bookkeeping, the device/stream/memory surface that
// mirrors GcuDevice (src/gcu_device.rs:61-635) and GcuSlice (src/gcu_slice.rs:49-101), and
// the per-device error word kernels write instead of trapping.
#include <atomic>
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"

namespace {
thread_local int t_status = UB_OK;
thread_local int t_cuda_error = 0;

// One error word per device; lives in the module's device image.
__device__ int g_ub_device_error = 0;

struct ErrWordCache {
  std::mutex mu;
  int* ptr[64] = {nullptr};
};
ErrWordCache g_err_cache;

// Streams on which this library has just launched a kernel that writes GGUF weight bytes (quantise, repack).
// The decode kernels request weight tiles before their dependency wait, which is only safe while no kernel
// in front of them on the stream produces those bytes; the next quantized matmul on a marked stream is
// launched without that early request and clears the mark.
std::mutex g_fresh_mu;
std::vector<cudaStream_t> g_fresh_streams;
std::atomic<int> g_fresh_count{0};
}  // namespace

namespace ub {
void set_status(int st) { t_status = st; }
void set_cuda_error(cudaError_t e) { t_cuda_error = static_cast<int>(e); }
int fail(int st) {
  t_status = st;
  return st;
}
int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_cuda_error(e);
    return fail(UB_ERR_CUDA);
  }
  t_status = UB_OK;
  return UB_OK;
}

void mark_weights_written(cudaStream_t s) {
  std::lock_guard<std::mutex> lk(g_fresh_mu);
  for (cudaStream_t t : g_fresh_streams)
    if (t == s) return;
  g_fresh_streams.push_back(s);
  g_fresh_count.store(static_cast<int>(g_fresh_streams.size()), std::memory_order_release);
}
bool take_weights_written(cudaStream_t s) {
  if (g_fresh_count.load(std::memory_order_acquire) == 0) return false;
  std::lock_guard<std::mutex> lk(g_fresh_mu);
  for (size_t i = 0; i < g_fresh_streams.size(); i++)
    if (g_fresh_streams[i] == s) {
      g_fresh_streams.erase(g_fresh_streams.begin() + i);
      g_fresh_count.store(static_cast<int>(g_fresh_streams.size()), std::memory_order_release);
      return true;
    }
  return false;
}

int* device_error_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_err_cache.mu);
  if (!g_err_cache.ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_ub_device_error);
    if (e != cudaSuccess) {
      set_cuda_error(e);
      return nullptr;
    }
    g_err_cache.ptr[dev] = static_cast<int*>(p);
  }
  return g_err_cache.ptr[dev];
}
}  // namespace ub

struct ub_device {
  int ordinal;
  cudaStream_t stream;
};

#define UB_CUDA_TRY(expr)                   \
  do {                                      \
    cudaError_t e__ = (expr);               \
    if (e__ != cudaSuccess) {               \
      ub::set_cuda_error(e__);              \
      return ub::fail(UB_ERR_CUDA);         \
    }                                       \
  } while (0)

extern "C" {

int ub_version(void) { return 100; }

const char* ub_status_string(int status) {
  switch (status) {
    case UB_OK: return "ok";
    case UB_ERR_INVALID_ARG: return "invalid argument";
    case UB_ERR_UNSUPPORTED: return "unsupported function or path";
    case UB_ERR_WORKSPACE: return "workspace missing or too small";
    case UB_ERR_CUDA: return "CUDA runtime error";
    case UB_ERR_BAD_INDEX: return "index out of range seen on device";
    case UB_ERR_TIMEOUT: return "bounded device wait ran out";
    case UB_ERR_NCCL: return "NCCL unavailable or failed";
    case UB_ERR_TOO_LARGE: return "size beyond the entry point's fixed limit";
    default: return "unknown status";
  }
}

int ub_last_status(void) { return t_status; }
int ub_last_cuda_error(void) { return t_cuda_error; }

int ub_device_status(void* stream) {
  int* w = ub::device_error_word();
  if (!w) return ub::fail(UB_ERR_CUDA);
  int host = 0;
  cudaStream_t s = ub::as_stream(stream);
  UB_CUDA_TRY(cudaMemcpyAsync(&host, w, sizeof(int), cudaMemcpyDeviceToHost, s));
  UB_CUDA_TRY(cudaMemsetAsync(w, 0, sizeof(int), s));
  UB_CUDA_TRY(cudaStreamSynchronize(s));
  return host;
}

int ub_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}

int ub_device_new(int ordinal, ub_device** out) {
  if (!out) return ub::fail(UB_ERR_INVALID_ARG);
  *out = nullptr;
  int n = ub_device_count();
  if (ordinal < 0 || ordinal >= n) return ub::fail(UB_ERR_INVALID_ARG);
  UB_CUDA_TRY(cudaSetDevice(ordinal));
  cudaStream_t s = nullptr;
  UB_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  ub_device* d = new (std::nothrow) ub_device{ordinal, s};
  if (!d) {
    cudaStreamDestroy(s);
    return ub::fail(UB_ERR_CUDA);
  }
  *out = d;
  return ub::fail(UB_OK);
}

void ub_device_free(ub_device* dev) {
  if (!dev) return;
  cudaSetDevice(dev->ordinal);
  cudaStreamSynchronize(dev->stream);
  cudaStreamDestroy(dev->stream);
  delete dev;
}

int ub_device_ordinal(const ub_device* dev) { return dev ? dev->ordinal : -1; }
void* ub_device_stream(const ub_device* dev) { return dev ? reinterpret_cast<void*>(dev->stream) : nullptr; }

int ub_device_bind(const ub_device* dev) {
  if (!dev) return ub::fail(UB_ERR_INVALID_ARG);
  UB_CUDA_TRY(cudaSetDevice(dev->ordinal));
  return ub::fail(UB_OK);
}

int ub_alloc(ub_device* dev, size_t bytes, void** out) {
  if (!dev || !out) return ub::fail(UB_ERR_INVALID_ARG);
  *out = nullptr;
  if (bytes == 0) return ub::fail(UB_OK);
  UB_CUDA_TRY(cudaSetDevice(dev->ordinal));
  UB_CUDA_TRY(cudaMallocAsync(out, bytes, dev->stream));
  return ub::fail(UB_OK);
}

int ub_alloc_zeros(ub_device* dev, size_t bytes, void** out) {
  int st = ub_alloc(dev, bytes, out);
  if (st != UB_OK || bytes == 0) return st;
  UB_CUDA_TRY(cudaMemsetAsync(*out, 0, bytes, dev->stream));
  return ub::fail(UB_OK);
}

int ub_free(ub_device* dev, void* ptr) {
  if (!dev) return ub::fail(UB_ERR_INVALID_ARG);
  if (!ptr) return ub::fail(UB_OK);
  UB_CUDA_TRY(cudaSetDevice(dev->ordinal));
  UB_CUDA_TRY(cudaFreeAsync(ptr, dev->stream));
  return ub::fail(UB_OK);
}

int ub_memcpy_htod(ub_device* dev, void* dst, const void* host_src, size_t bytes) {
  if (!dev || (bytes && (!dst || !host_src))) return ub::fail(UB_ERR_INVALID_ARG);
  UB_CUDA_TRY(cudaMemcpyAsync(dst, host_src, bytes, cudaMemcpyHostToDevice, dev->stream));
  return ub::fail(UB_OK);
}

int ub_memcpy_dtoh(ub_device* dev, void* host_dst, const void* src, size_t bytes) {
  if (!dev || (bytes && (!host_dst || !src))) return ub::fail(UB_ERR_INVALID_ARG);
  UB_CUDA_TRY(cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, dev->stream));
  return ub::fail(UB_OK);
}

int ub_memcpy_dtod(ub_device* dev, void* dst, const void* src, size_t bytes) {
  if (!dev || (bytes && (!dst || !src))) return ub::fail(UB_ERR_INVALID_ARG);
  UB_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, dev->stream));
  return ub::fail(UB_OK);
}

int ub_memcpy_dtod_2d(ub_device* dev, void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                      size_t width_bytes, size_t height) {
  if (!dev || ((width_bytes && height) && (!dst || !src))) return ub::fail(UB_ERR_INVALID_ARG);
  if (width_bytes == 0 || height == 0) return ub::fail(UB_OK);
  UB_CUDA_TRY(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, height, cudaMemcpyDeviceToDevice,
                                dev->stream));
  return ub::fail(UB_OK);
}

int ub_synchronize(ub_device* dev) {
  if (!dev) return ub::fail(UB_ERR_INVALID_ARG);
  UB_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  return ub::fail(UB_OK);
}

int ub_mem_info(ub_device* dev, size_t* free_bytes, size_t* total_bytes) {
  if (!dev || !free_bytes || !total_bytes) return ub::fail(UB_ERR_INVALID_ARG);
  UB_CUDA_TRY(cudaSetDevice(dev->ordinal));
  UB_CUDA_TRY(cudaMemGetInfo(free_bytes, total_bytes));
  return ub::fail(UB_OK);
}

int ub_stream_query(void* stream) {
  const cudaError_t e = cudaStreamQuery(ub::as_stream(stream));
  if (e == cudaSuccess) return ub::fail(UB_OK);
  if (e == cudaErrorNotReady) {
    cudaGetLastError();  // not an error: clear it
    return ub::fail(UB_ERR_NOT_READY);
  }
  ub::set_cuda_error(e);
  return ub::fail(UB_ERR_CUDA);
}

}  // extern "C"
