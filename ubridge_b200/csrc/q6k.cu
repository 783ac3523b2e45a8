// GGUF Q6_K: dequantisation and the decode matmul (weights streamed once, f32 accumulation).
//
// The reference declares the block (kernels/quant.cpp:170-177: ql[128] low nibbles, qh[64] upper two bits,
// int8 scales[16], f16 d; 210 bytes per 256 values) but ships no kernel for it; in Q4_K_M model files the
// output and embedding matrices come in this format.  The arithmetic is the published GGML one:
// element i of a super-block (h = i / 128, j = (i % 128) / 32, l = i % 32) has its low nibble in
// ql[64h + 32(j & 1) + l] (upper half of the byte for j >= 2) and its top two bits at bit 2j of qh[32h + l];
// y = (d * scales[i / 16]) * (q - 32).
//
// A block is 210 bytes, so nothing in it is better than 2-byte aligned: all weight loads are 16-bit ones, and
// consecutive lanes read consecutive bytes.  The dequantisation kernel gives a lane two neighbouring l of one
// half (eight weights), the matmul kernel four (sixteen weights).
#include "common.cuh"

#define UB_Q6K_BYTES 210

namespace {

using namespace ub;

__device__ __forceinline__ uint32_t ldg_u16(const uint8_t* p) {
  return __ldg(reinterpret_cast<const unsigned short*>(p));
}

// One warp per super-block.
template <typename T>
__global__ void __launch_bounds__(256) dequant_q6k_kernel(const uint8_t* __restrict__ in, T* __restrict__ out,
                                                          size_t nb) {
  const int lane = threadIdx.x & 31;
  const int h = lane >> 4, l0 = (lane & 15) * 2;
  const size_t warps = static_cast<size_t>(gridDim.x) * (blockDim.x >> 5);
  for (size_t b = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); b < nb; b += warps) {
    const uint8_t* blk = in + b * UB_Q6K_BYTES;
    const float d = half_bits_to_f32(ldg_u16(blk + 208));
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192) + 8 * h + (l0 >> 4);
    const uint32_t qa = ldg_u16(blk + 64 * h + l0), qb = ldg_u16(blk + 64 * h + 32 + l0);
    const uint32_t qh = ldg_u16(blk + 128 + 32 * h + l0);
    T* o = out + b * UB_QK_K + 128 * h + l0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float ds = d * static_cast<float>(__ldg(sc + 2 * j));  // (d * scale) first, as the format defines it
      const uint32_t src = (j & 1) ? qb : qa;
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const uint32_t lo = (src >> (8 * e + (j >= 2 ? 4 : 0))) & 0xF;
        const uint32_t hi = (qh >> (8 * e + 2 * j)) & 3;
        o[32 * j + e] = from_f32<T>(ds * static_cast<float>(static_cast<int>(lo | (hi << 4)) - 32));
      }
    }
  }
}

// Four neighbouring activations with one load (index a multiple of 4 in a 16-byte aligned row).
__device__ __forceinline__ void load_quad(const float* p, float (&v)[4]) {
  const float4 q = __ldg(reinterpret_cast<const float4*>(p));
  v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
}
__device__ __forceinline__ void load_quad(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 q = __ldg(reinterpret_cast<const uint2*>(p));
  v[0] = __uint_as_float(q.x << 16), v[1] = __uint_as_float(q.x & 0xFFFF0000u);
  v[2] = __uint_as_float(q.y << 16), v[3] = __uint_as_float(q.y & 0xFFFF0000u);
}
__device__ __forceinline__ uint32_t ldg_2x16(const uint8_t* p) {  // four bytes from a 2-byte aligned address
  return ldg_u16(p) | (ldg_u16(p + 2) << 16);
}

constexpr int kQ6kRowsPerWarp = 2;  // the activations a lane loads serve this many weight rows

// Decode matmul: one warp per pair of weight rows, MT tokens per pass; x is re-read through L1/L2 (it is K * MT values).
// A warp takes two super-blocks per step (lanes 0-15 the even one, 16-31 the odd one); inside a super-block a
// lane owns four neighbouring positions l of one 128-value half, i.e. 16 weights: their four 6-bit values per j
// are assembled with byte-parallel masks (four values per instruction), turned into floats by placing each byte
// in the mantissa of 2^23 (one byte permute) and subtracting 2^23 + 32, and multiplied with the activations at
// the same positions; the int8 scale is applied once per j, d once per super-block.  The row's partial sums are
// added across the warp by shuffles, in a fixed order.
template <typename XT, int MT>
__global__ void __launch_bounds__(256) qgemv_q6k_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x,
                                                        void* __restrict__ y, int y_dtype, int N, int K, int ldy) {
  constexpr int RW = kQ6kRowsPerWarp;
  const int lane = threadIdx.x & 31;
  const int sub = lane >> 4, h = (lane >> 3) & 1, l0 = (lane & 7) * 4;
  const int nsb = K / UB_QK_K;
  const size_t row_bytes = static_cast<size_t>(nsb) * UB_Q6K_BYTES;
  const int warps = gridDim.x * (blockDim.x >> 5);
  for (int n0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RW; n0 < N; n0 += warps * RW) {
    const uint8_t* row[RW];
#pragma unroll
    for (int r = 0; r < RW; r++)  // rows beyond N repeat the last one; their sums are not written
      row[r] = wq + static_cast<size_t>(n0 + r < N ? n0 + r : N - 1) * row_bytes;
    float acc[RW][MT];
#pragma unroll
    for (int r = 0; r < RW; r++)
#pragma unroll
      for (int t = 0; t < MT; t++) acc[r][t] = 0.f;
    for (int sb = sub; sb < nsb; sb += 2) {
      uint32_t q[RW][4];
      float s[RW][4], d[RW];
#pragma unroll
      for (int r = 0; r < RW; r++) {
        const uint8_t* blk = row[r] + static_cast<size_t>(sb) * UB_Q6K_BYTES;
        const uint32_t qa = ldg_2x16(blk + 64 * h + l0);       // low nibbles: j = 0, high: j = 2
        const uint32_t qb = ldg_2x16(blk + 64 * h + 32 + l0);  // low nibbles: j = 1, high: j = 3
        const uint32_t qh = ldg_2x16(blk + 128 + 32 * h + l0);
        const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192) + 8 * h + (l0 >> 4);
#pragma unroll
        for (int j = 0; j < 4; j++) s[r][j] = static_cast<float>(__ldg(sc + 2 * j));
        d[r] = half_bits_to_f32(ldg_u16(blk + 208));
        q[r][0] = (qa & 0x0F0F0F0Fu) | ((qh << 4) & 0x30303030u);
        q[r][1] = (qb & 0x0F0F0F0Fu) | ((qh << 2) & 0x30303030u);
        q[r][2] = ((qa >> 4) & 0x0F0F0F0Fu) | (qh & 0x30303030u);
        q[r][3] = ((qb >> 4) & 0x0F0F0F0Fu) | ((qh >> 2) & 0x30303030u);
      }
      float part[RW][MT];
#pragma unroll
      for (int r = 0; r < RW; r++)
#pragma unroll
        for (int t = 0; t < MT; t++) part[r][t] = 0.f;
      const int k0 = sb * UB_QK_K + 128 * h + l0;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float xv[MT][4];
#pragma unroll
        for (int t = 0; t < MT; t++) load_quad(x + static_cast<size_t>(t) * K + k0 + 32 * j, xv[t]);
#pragma unroll
        for (int r = 0; r < RW; r++) {
          float w[4];
#pragma unroll
          for (int e = 0; e < 4; e++)  // 0x4B000000 | byte e of q = 2^23 + q as a float
            w[e] = __uint_as_float(__byte_perm(q[r][j], 0x4B000000u, 0x7440u | e)) - 8388640.f;
#pragma unroll
          for (int t = 0; t < MT; t++) {
            float pj = w[0] * xv[t][0];
            pj = fmaf(w[1], xv[t][1], pj);
            pj = fmaf(w[2], xv[t][2], pj);
            pj = fmaf(w[3], xv[t][3], pj);
            part[r][t] = fmaf(s[r][j], pj, part[r][t]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RW; r++)
#pragma unroll
        for (int t = 0; t < MT; t++) acc[r][t] = fmaf(d[r], part[r][t], acc[r][t]);
    }
#pragma unroll
    for (int r = 0; r < RW; r++)
#pragma unroll
      for (int t = 0; t < MT; t++) {
        float v = acc[r][t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && n0 + r < N) {
          const size_t at = static_cast<size_t>(t) * ldy + n0 + r;
          if (y_dtype == UB_DTYPE_F32) static_cast<float*>(y)[at] = v;
          else if (y_dtype == UB_DTYPE_BF16) static_cast<__nv_bfloat16*>(y)[at] = __float2bfloat16_rn(v);
          else static_cast<__half*>(y)[at] = __float2half_rn(v);
        }
      }
  }
}

template <typename XT>
int q6k_matmul(void* y, const XT* x, const void* wq, int M, int N, int K, int out_dtype, cudaStream_t s) {
  if (M == 0 || N == 0) return ub::fail(UB_OK);
  if (!y || !x || !wq || M < 0 || N < 0 || K <= 0 || K % UB_QK_K) return ub::fail(UB_ERR_INVALID_ARG);
  if (out_dtype != UB_DTYPE_F32 && out_dtype != UB_DTYPE_BF16 && out_dtype != UB_DTYPE_F16)
    return ub::fail(UB_ERR_INVALID_ARG);
  if ((reinterpret_cast<uintptr_t>(wq) & 1) || (reinterpret_cast<uintptr_t>(x) & 15))  // x rows: paired loads
    return ub::fail(UB_ERR_INVALID_ARG);
  const int esz = out_dtype == UB_DTYPE_F32 ? 4 : 2;
  const int grid = (N + 8 * kQ6kRowsPerWarp - 1) / (8 * kQ6kRowsPerWarp);  // the CTA scheduler evens out the load
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  for (int m0 = 0; m0 < M;) {  // passes of up to four tokens: the weights are read once per pass
    const int left = M - m0;
    const XT* xp = x + static_cast<size_t>(m0) * K;
    void* yp = static_cast<char*>(y) + static_cast<size_t>(m0) * N * esz;
    if (left >= 4) {
      qgemv_q6k_kernel<XT, 4><<<grid, 256, 0, s>>>(w, xp, yp, out_dtype, N, K, N);
      m0 += 4;
    } else if (left >= 2) {
      qgemv_q6k_kernel<XT, 2><<<grid, 256, 0, s>>>(w, xp, yp, out_dtype, N, K, N);
      m0 += 2;
    } else {
      qgemv_q6k_kernel<XT, 1><<<grid, 256, 0, s>>>(w, xp, yp, out_dtype, N, K, N);
      m0 += 1;
    }
  }
  return ub::check_launch();
}

}  // namespace

extern "C" {

int ub_dequant_q6k(void* out, const void* blocks, size_t numel, int out_dtype, void* stream) {
  if (numel == 0) return ub::fail(UB_OK);
  if (!out || !blocks || numel % UB_QK_K || (reinterpret_cast<uintptr_t>(blocks) & 1))
    return ub::fail(UB_ERR_INVALID_ARG);
  const size_t nb = numel / UB_QK_K;
  const size_t want = (nb + 7) / 8, cap = static_cast<size_t>(ub::num_sms()) * 16;
  const int grid = static_cast<int>(want < cap ? want : cap);
  cudaStream_t s = ub::as_stream(stream);
  UB_DISPATCH_FLOAT(out_dtype, T, (dequant_q6k_kernel<T><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(blocks),
                                                                               static_cast<T*>(out), nb)));
  return ub::check_launch();
}

int ub_qmatmul_q6k_f32(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* stream) {
  return q6k_matmul<float>(y, static_cast<const float*>(x), wq, M, N, K, out_dtype, ub::as_stream(stream));
}
int ub_qmatmul_q6k_bf16(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* stream) {
  return q6k_matmul<__nv_bfloat16>(y, static_cast<const __nv_bfloat16*>(x), wq, M, N, K, out_dtype,
                                   ub::as_stream(stream));
}

}  // extern "C"
