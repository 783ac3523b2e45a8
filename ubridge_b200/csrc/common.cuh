// Shared helpers for the sm_100a kernels: status bookkeeping, storage-type load/store,
// GGUF block layouts and the Q4_K 6-bit scale decoding.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/ubridge_b200.h"

#define UB_QK8_0 32
#define UB_QK_K 256
#define UB_Q8_0_BYTES 34
#define UB_Q4K_BYTES 144

namespace ub {

// ---- per-thread host status (void exports cannot return one) ----
void set_status(int st);
void set_cuda_error(cudaError_t e);
int fail(int st);                 // records and returns st
int check_launch();               // cudaGetLastError -> UB_OK / UB_ERR_CUDA (recorded)

// ---- weight bytes produced on a stream by this library's own kernels (quantise, repack) ----
// mark: called by those entry points; take: true once for the next quantized matmul on that stream, which then
// requests no weight tile ahead of its dependency wait.
void mark_weights_written(cudaStream_t s);
bool take_weights_written(cudaStream_t s);

// ---- per-device error word written by kernels instead of trapping ----
// Address of the device's error word (resolved once per device with cudaGetSymbolAddress).
int* device_error_word();

__device__ __forceinline__ void report_device_error(int* err_word, int code) {
  if (err_word) atomicMax(err_word, code);
}

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline int num_sms() {
  static std::atomic<int> cached[64];  // zero-initialised; threads of different ranks fill it concurrently
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// ---- storage types ----
template <typename T> struct dtype_code;
template <> struct dtype_code<float> { static constexpr int value = UB_DTYPE_F32; };
template <> struct dtype_code<__half> { static constexpr int value = UB_DTYPE_F16; };
template <> struct dtype_code<__nv_bfloat16> { static constexpr int value = UB_DTYPE_BF16; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Dispatch a callable templated on the storage type from a runtime dtype code.
#define UB_DISPATCH_FLOAT(code, T, ...)                                  \
  switch (code) {                                                        \
    case UB_DTYPE_F32: { using T = float; __VA_ARGS__; break; }          \
    case UB_DTYPE_F16: { using T = __half; __VA_ARGS__; break; }         \
    case UB_DTYPE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    default: return ub::fail(UB_ERR_INVALID_ARG);                        \
  }

// ---- Q4_K scale decoding ----
// The 12 scale bytes as three little-endian words s0 (bytes 0-3), s1 (4-7), s2 (8-11).
// Pair j < 4:  sc = b[j] & 63,                      m = b[j+4] & 63
// Pair j >= 4: sc = (b[j+4] & 15) | (b[j-4] >> 6) << 4,  m = (b[j+4] >> 4) | (b[j] >> 6) << 4
// Returns the 8 scales as two words of 4 bytes each (pairs 0-3, pairs 4-7); same for mins.
__device__ __forceinline__ void q4k_unpack_scales(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t& sc_lo,
                                                  uint32_t& sc_hi, uint32_t& mn_lo, uint32_t& mn_hi) {
  sc_lo = s0 & 0x3F3F3F3Fu;
  mn_lo = s1 & 0x3F3F3F3Fu;
  sc_hi = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
  mn_hi = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
}

__device__ __forceinline__ float half_bits_to_f32(uint32_t h16) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h16 & 0xFFFFu)));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

}  // namespace ub
