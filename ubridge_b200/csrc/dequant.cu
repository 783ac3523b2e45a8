// GGUF block (de)quantisation kernels: Q8_0 and Q4_K -> f32/f16/bf16 (bit-exact), f32/f16/bf16 ->
// Q8_0, and the repack between interleaved GGUF bytes and the reference's split device layout.
//
// Replaces kernels/quant.cpp:188-268 (Q8_0 dequant), :270-353 (Q8_0 quant), :372-488 (Q4_K
// dequant).  Formats: kernels/quant.cpp:98-104 (block_q8_0), :145-150 (block_q4_K), :356-363
// (get_scale_min_k4).  The Q4_K arithmetic follows the format ((d*sc)*q - dmin*m per 32-value
// sub-block with its own min), not the vector code at :411-412 which reuses the first sub-block's
// min for the second.
//
// These kernels are HBM-bound on their OUTPUT (4 B written per 0.56-1.06 B read for f32), so the
// layout is chosen for coalesced 16-byte stores: one warp per Q4_K super-block (lane w owns qs word
// w: four low-nibble and four high-nibble values), eight lanes per Q8_0 block.
#include "common.cuh"

namespace {

using namespace ub;

template <typename T> struct Vec4;
template <> struct Vec4<float> { using type = float4; };
template <> struct Vec4<__half> { using type = uint2; };
template <> struct Vec4<__nv_bfloat16> { using type = uint2; };

template <typename T>
__device__ __forceinline__ void store4(T* dst, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<__half>(__half* dst, float a, float b, float c, float d) {
  __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = v;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = v;
}

// One warp per super-block.  SPLIT selects the reference's de-interleaved layout
// ([nb x 16-byte header][nb x 128-byte qs]) instead of interleaved 144-byte blocks.
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(256) dequant_q4k_kernel(const uint8_t* __restrict__ in, T* __restrict__ out,
                                                           size_t nblocks) {
  const int lane = threadIdx.x & 31;
  const size_t warp = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
  for (size_t b = warp; b < nblocks; b += nwarps) {
    const uint8_t* hdr = SPLIT ? in + b * 16 : in + b * UB_Q4K_BYTES;
    const uint8_t* qs = SPLIT ? in + nblocks * 16 + b * 128 : hdr + 16;
    const uint4 h = __ldg(reinterpret_cast<const uint4*>(hdr));
    const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(qs) + lane);
    const float d = half_bits_to_f32(h.x), dmin = half_bits_to_f32(h.x >> 16);
    uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
    q4k_unpack_scales(h.y, h.z, h.w, sc_lo, sc_hi, mn_lo, mn_hi);
    const int g = lane >> 3;  // 64-value group; pairs 2g (low nibbles) and 2g+1 (high nibbles)
    const uint32_t scw = (g < 2) ? sc_lo : sc_hi, mnw = (g < 2) ? mn_lo : mn_hi;
    const int sh = (g & 1) * 16;
    const float d1 = d * static_cast<float>((scw >> sh) & 0xFF), m1 = dmin * static_cast<float>((mnw >> sh) & 0xFF);
    const float d2 = d * static_cast<float>((scw >> (sh + 8)) & 0xFF),
                m2 = dmin * static_cast<float>((mnw >> (sh + 8)) & 0xFF);
    T* y = out + b * UB_QK_K + 64 * g + 4 * (lane & 7);
    // products are exact in f32 (11+6+4 significant bits); the subtraction rounds once
    store4<T>(y, __fsub_rn(__fmul_rn(d1, static_cast<float>(w & 0xF)), m1),
              __fsub_rn(__fmul_rn(d1, static_cast<float>((w >> 8) & 0xF)), m1),
              __fsub_rn(__fmul_rn(d1, static_cast<float>((w >> 16) & 0xF)), m1),
              __fsub_rn(__fmul_rn(d1, static_cast<float>((w >> 24) & 0xF)), m1));
    store4<T>(y + 32, __fsub_rn(__fmul_rn(d2, static_cast<float>((w >> 4) & 0xF)), m2),
              __fsub_rn(__fmul_rn(d2, static_cast<float>((w >> 12) & 0xF)), m2),
              __fsub_rn(__fmul_rn(d2, static_cast<float>((w >> 20) & 0xF)), m2),
              __fsub_rn(__fmul_rn(d2, static_cast<float>((w >> 28) & 0xF)), m2));
  }
}

// Eight lanes per 32-value block, four values per lane.  Blocks are only 2-byte aligned in the
// interleaved layout, so quants are fetched as two 16-bit loads.
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(256) dequant_q8_0_kernel(const uint8_t* __restrict__ in, T* __restrict__ out,
                                                            size_t nblocks) {
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = tid; i < nblocks * 8; i += nthreads) {
    const size_t b = i >> 3;
    const int part = static_cast<int>(i & 7);
    const uint8_t* dptr = SPLIT ? in + b * 2 : in + b * UB_Q8_0_BYTES;
    const uint8_t* qptr = (SPLIT ? in + nblocks * 2 + b * 32 : dptr + 2) + part * 4;
    const float d = half_bits_to_f32(__ldg(reinterpret_cast<const unsigned short*>(dptr)));
    const uint32_t lo = __ldg(reinterpret_cast<const unsigned short*>(qptr));
    const uint32_t hi = __ldg(reinterpret_cast<const unsigned short*>(qptr + 2));
    const uint32_t w = lo | (hi << 16);
    store4<T>(out + b * UB_QK8_0 + part * 4, d * static_cast<float>(static_cast<int8_t>(w & 0xFF)),
              d * static_cast<float>(static_cast<int8_t>((w >> 8) & 0xFF)),
              d * static_cast<float>(static_cast<int8_t>((w >> 16) & 0xFF)),
              d * static_cast<float>(static_cast<int8_t>((w >> 24) & 0xFF)));
  }
}

// One warp per block: lane i owns value i.  d = amax/127, id = 1/d (0 when d == 0),
// q = roundf(x*id) (half away from zero), stored scale = f16(d).
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const T* __restrict__ x, uint8_t* __restrict__ out,
                                                             size_t nblocks) {
  const int lane = threadIdx.x & 31;
  const size_t warp = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
  for (size_t b = warp; b < nblocks; b += nwarps) {
    const float v = to_f32(x[b * UB_QK8_0 + lane]);
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const float d = __fdiv_rn(amax, 127.f);
    const float id = (d != 0.f) ? __fdiv_rn(1.f, d) : 0.f;
    const int q = static_cast<int>(roundf(__fmul_rn(v, id)));
    uint8_t* dptr = SPLIT ? out + b * 2 : out + b * UB_Q8_0_BYTES;
    uint8_t* qptr = SPLIT ? out + nblocks * 2 + b * 32 : dptr + 2;
    qptr[lane] = static_cast<uint8_t>(static_cast<int8_t>(q));
    if (lane == 0) *reinterpret_cast<unsigned short*>(dptr) = __half_as_ushort(__float2half_rn(d));
  }
}

// interleaved <-> split, 2 bytes per thread (both layouts are at least 2-byte aligned)
template <bool TO_SPLIT>
__global__ void __launch_bounds__(256) repack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                      size_t nblocks, int hb, int qb) {
  const size_t per = static_cast<size_t>(hb + qb) / 2;
  const size_t total = nblocks * per;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t b = i / per;
    const size_t o = (i % per) * 2;  // byte offset inside the interleaved block
    const size_t inter = b * (hb + qb) + o;
    const size_t split = (o < static_cast<size_t>(hb)) ? b * hb + o : nblocks * hb + b * qb + (o - hb);
    const unsigned short v = *reinterpret_cast<const unsigned short*>(src + (TO_SPLIT ? inter : split));
    *reinterpret_cast<unsigned short*>(dst + (TO_SPLIT ? split : inter)) = v;
  }
}

inline int grid_for(size_t work_items, int per_block) {
  size_t blocks = (work_items + per_block - 1) / per_block;
  const size_t cap = static_cast<size_t>(ub::num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  return static_cast<int>(blocks);
}

template <bool SPLIT>
int dequant_q4k_launch(void* out, const void* in, size_t numel, int out_dtype, cudaStream_t s) {
  if (numel == 0) return ub::fail(UB_OK);
  if (!out || !in || numel % UB_QK_K) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t nb = numel / UB_QK_K;
  UB_DISPATCH_FLOAT(out_dtype, T, (dequant_q4k_kernel<T, SPLIT><<<grid_for(nb, 8), 256, 0, s>>>(
                                      static_cast<const uint8_t*>(in), static_cast<T*>(out), nb)));
  return ub::check_launch();
}

template <bool SPLIT>
int dequant_q8_0_launch(void* out, const void* in, size_t numel, int out_dtype, cudaStream_t s) {
  if (numel == 0) return ub::fail(UB_OK);
  if (!out || !in || numel % UB_QK8_0) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t nb = numel / UB_QK8_0;
  UB_DISPATCH_FLOAT(out_dtype, T, (dequant_q8_0_kernel<T, SPLIT><<<grid_for(nb * 8, 256), 256, 0, s>>>(
                                      static_cast<const uint8_t*>(in), static_cast<T*>(out), nb)));
  return ub::check_launch();
}

template <bool SPLIT>
int quantize_q8_0_launch(void* out, const void* x, size_t numel, int in_dtype, cudaStream_t s) {
  if (numel == 0) return ub::fail(UB_OK);
  if (!out || !x || numel % UB_QK8_0) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t nb = numel / UB_QK8_0;
  UB_DISPATCH_FLOAT(in_dtype, T, (quantize_q8_0_kernel<T, SPLIT><<<grid_for(nb, 8), 256, 0, s>>>(
                                     static_cast<const T*>(x), static_cast<uint8_t*>(out), nb)));
  return ub::check_launch();
}

}  // namespace

namespace ub {
// Split-layout launchers used by the name registry (module "quant").
int dequant_q8_0_split(void* out, const void* in, size_t numel, int dt, cudaStream_t s) {
  return dequant_q8_0_launch<true>(out, in, numel, dt, s);
}
int dequant_q4k_split(void* out, const void* in, size_t numel, int dt, cudaStream_t s) {
  return dequant_q4k_launch<true>(out, in, numel, dt, s);
}
int quantize_q8_0_split(void* out, const void* x, size_t numel, int dt, cudaStream_t s) {
  return quantize_q8_0_launch<true>(out, x, numel, dt, s);
}
}  // namespace ub

extern "C" {

int ub_dequant_q8_0(void* out, const void* blocks, size_t numel, int out_dtype, void* stream) {
  return dequant_q8_0_launch<false>(out, blocks, numel, out_dtype, ub::as_stream(stream));
}
int ub_dequant_q4k(void* out, const void* blocks, size_t numel, int out_dtype, void* stream) {
  return dequant_q4k_launch<false>(out, blocks, numel, out_dtype, ub::as_stream(stream));
}
int ub_quantize_q8_0(void* blocks, const void* x, size_t numel, int in_dtype, void* stream) {
  const int st = quantize_q8_0_launch<false>(blocks, x, numel, in_dtype, ub::as_stream(stream));
  if (st == UB_OK && numel) ub::mark_weights_written(ub::as_stream(stream));
  return st;
}

int ub_repack_to_split(void* split, const void* interleaved, size_t nblocks, int is_q4k, void* stream) {
  if (nblocks == 0) return ub::fail(UB_OK);
  if (!split || !interleaved) return ub::fail(UB_ERR_INVALID_ARG);
  const int hb = is_q4k ? 16 : 2, qb = is_q4k ? 128 : 32;
  repack_kernel<true><<<grid_for(nblocks * (hb + qb) / 2, 256), 256, 0, ub::as_stream(stream)>>>(
      static_cast<const uint8_t*>(interleaved), static_cast<uint8_t*>(split), nblocks, hb, qb);
  return ub::check_launch();
}

int ub_repack_to_interleaved(void* interleaved, const void* split, size_t nblocks, int is_q4k, void* stream) {
  if (nblocks == 0) return ub::fail(UB_OK);
  if (!split || !interleaved) return ub::fail(UB_ERR_INVALID_ARG);
  const int hb = is_q4k ? 16 : 2, qb = is_q4k ? 128 : 32;
  repack_kernel<false><<<grid_for(nblocks * (hb + qb) / 2, 256), 256, 0, ub::as_stream(stream)>>>(
      static_cast<const uint8_t*>(split), static_cast<uint8_t*>(interleaved), nblocks, hb, qb);
  ub::mark_weights_written(ub::as_stream(stream));
  return ub::check_launch();
}

}  // extern "C"
