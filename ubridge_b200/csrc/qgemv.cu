// Fused dequantise + GEMV for GGUF Q8_0 / Q4_K weights (decode shapes, small M), CUDA-core path.
//
// y[M,N] = x[M,K] . W^T, W = N rows of interleaved blocks.  The reference computes this with two
// kernels and a dense temporary (kernels/quant.cpp:257-268,477-488 then kernels/matmul.cpp:1143-1184;
// its small-M streaming shape is kernels/third_party/matmul_decoding.h:12-570).  Here the packed
// weights are streamed once with 128-bit loads and dequantised in registers.
//
// Work split: one warp per weight row; lanes stride over 64-value Q4_K groups (32 B of nibbles +
// the super-block's 16-byte header) or over runs of eight Q8_0 blocks (272 B = 17 x 16 B, which is
// what makes 128-bit loads legal on the 34-byte blocks).  Nibbles/bytes are turned into floats with a
// byte-permute into the mantissa of a constant (128 + q resp. 2^23 + q), so no integer->float
// conversion instruction is issued.  For Q4_K the per-32-value sums of x are computed once per CTA
// into shared memory; the row result is
//     sum_g  (d*sc_g) * sum_k (128 + q_k) x_k  -  (128*d*sc_g + dmin*m_g) * sum_k x_k .
// Accumulation is f32; a warp-shuffle reduction finishes each row.
#include "common.cuh"

namespace {

using namespace ub;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// float(128 + nibble) for byte `i` of a word already masked with 0x0F0F0F0F
template <int I>
__device__ __forceinline__ float nib_biased(uint32_t w4) {
  return __uint_as_float(__byte_perm(w4, 0x43000000u, 0x7044u | (I << 8)));
}
// exact float(int8) for byte `i` of a word already XOR-ed with 0x80808080
template <int I>
__device__ __forceinline__ float s8_exact(uint32_t wx) {
  return __uint_as_float(__byte_perm(wx, 0x4B000000u, 0x7440u | I)) - 8388736.0f;  // 2^23 + 128
}

template <typename XT>
__device__ __forceinline__ void load_x8(const XT* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load_x8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load_x8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xFFFF0000u);
  v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xFFFF0000u);
  v[4] = __uint_as_float(a.z << 16); v[5] = __uint_as_float(a.z & 0xFFFF0000u);
  v[6] = __uint_as_float(a.w << 16); v[7] = __uint_as_float(a.w & 0xFFFF0000u);
}

__device__ __forceinline__ void store_y(void* y, size_t idx, int dtype, float v) {
  if (dtype == UB_DTYPE_F32)
    static_cast<float*>(y)[idx] = v;
  else if (dtype == UB_DTYPE_BF16)
    static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
  else
    static_cast<__half*>(y)[idx] = __float2half_rn(v);
}

// ------------------------------------------------------------------ Q4_K
// sx[m][K/32]: sums of 32 consecutive activations, in dynamic shared memory.
template <typename XT, int MT>
__global__ void __launch_bounds__(kThreads) qgemv_q4k_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x,
                                                              void* __restrict__ y, int N, int K, int y_dtype) {
  extern __shared__ float sx[];
  const int ng32 = K >> 5;
  for (int i = threadIdx.x; i < MT * ng32; i += kThreads) {
    const int m = i / ng32, g = i - m * ng32;
    const XT* xp = x + static_cast<size_t>(m) * K + static_cast<size_t>(g) * 32;
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float v[8];
      load_x8<XT>(xp + 8 * j, v);
#pragma unroll
      for (int t = 0; t < 8; t++) s += v[t];
    }
    sx[i] = s;
  }
  __syncthreads();

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nsb = K >> 8;
  const int nitems = nsb * 4;  // 64-value groups per row
  const size_t row_bytes = static_cast<size_t>(nsb) * UB_Q4K_BYTES;

  for (int n = blockIdx.x * kWarps + warp; n < N; n += gridDim.x * kWarps) {
    const uint8_t* row = wq + static_cast<size_t>(n) * row_bytes;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.f;

    for (int it = lane; it < nitems; it += 32) {
      const int sb = it >> 2, g = it & 3;
      const uint8_t* blk = row + static_cast<size_t>(sb) * UB_Q4K_BYTES;
      const uint4 h = __ldg(reinterpret_cast<const uint4*>(blk));
      const uint4 qa = __ldg(reinterpret_cast<const uint4*>(blk + 16 + g * 32));
      const uint4 qb = __ldg(reinterpret_cast<const uint4*>(blk + 16 + g * 32) + 1);
      const float d = half_bits_to_f32(h.x), dmin = half_bits_to_f32(h.x >> 16);
      uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
      q4k_unpack_scales(h.y, h.z, h.w, sc_lo, sc_hi, mn_lo, mn_hi);
      const uint32_t scw = (g < 2) ? sc_lo : sc_hi, mnw = (g < 2) ? mn_lo : mn_hi;
      const int sh = (g & 1) * 16;
      const float d1 = d * static_cast<float>((scw >> sh) & 0xFF), m1 = dmin * static_cast<float>((mnw >> sh) & 0xFF);
      const float d2 = d * static_cast<float>((scw >> (sh + 8)) & 0xFF),
                  m2 = dmin * static_cast<float>((mnw >> (sh + 8)) & 0xFF);
      const float c1 = fmaf(128.f, d1, m1), c2 = fmaf(128.f, d2, m2);
      const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
      const int kbase = sb * 256 + g * 64;
#pragma unroll
      for (int m = 0; m < MT; m++) {
        const XT* xr = x + static_cast<size_t>(m) * K + kbase;
        float slo = 0.f, shi = 0.f;
#pragma unroll
        for (int c = 0; c < 4; c++) {  // 8 bytes of qs -> 8 low values and 8 high values
          float xl[8], xh[8];
          load_x8<XT>(xr + 8 * c, xl);
          load_x8<XT>(xr + 32 + 8 * c, xh);
          const uint32_t w0 = qw[2 * c], w1 = qw[2 * c + 1];
          const uint32_t l0 = w0 & 0x0F0F0F0Fu, h0 = (w0 >> 4) & 0x0F0F0F0Fu;
          const uint32_t l1 = w1 & 0x0F0F0F0Fu, h1 = (w1 >> 4) & 0x0F0F0F0Fu;
          slo = fmaf(nib_biased<0>(l0), xl[0], slo); slo = fmaf(nib_biased<1>(l0), xl[1], slo);
          slo = fmaf(nib_biased<2>(l0), xl[2], slo); slo = fmaf(nib_biased<3>(l0), xl[3], slo);
          slo = fmaf(nib_biased<0>(l1), xl[4], slo); slo = fmaf(nib_biased<1>(l1), xl[5], slo);
          slo = fmaf(nib_biased<2>(l1), xl[6], slo); slo = fmaf(nib_biased<3>(l1), xl[7], slo);
          shi = fmaf(nib_biased<0>(h0), xh[0], shi); shi = fmaf(nib_biased<1>(h0), xh[1], shi);
          shi = fmaf(nib_biased<2>(h0), xh[2], shi); shi = fmaf(nib_biased<3>(h0), xh[3], shi);
          shi = fmaf(nib_biased<0>(h1), xh[4], shi); shi = fmaf(nib_biased<1>(h1), xh[5], shi);
          shi = fmaf(nib_biased<2>(h1), xh[6], shi); shi = fmaf(nib_biased<3>(h1), xh[7], shi);
        }
        const float sxl = sx[m * ng32 + (kbase >> 5)], sxh = sx[m * ng32 + (kbase >> 5) + 1];
        acc[m] += (d1 * slo - c1 * sxl) + (d2 * shi - c2 * sxh);
      }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
      const float r = warp_sum(acc[m]);
      if (lane == 0) store_y(y, static_cast<size_t>(m) * N + n, y_dtype, r);
    }
  }
}

// ------------------------------------------------------------------ Q8_0
// FAST: K % 256 == 0, lanes take runs of 8 blocks with 17 aligned 16-byte loads.
// Otherwise one block per lane step with 2-byte loads.
template <typename XT, int MT, bool FAST>
__global__ void __launch_bounds__(kThreads) qgemv_q8_0_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x,
                                                               void* __restrict__ y, int N, int K, int y_dtype) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nblk = K >> 5;
  const size_t row_bytes = static_cast<size_t>(nblk) * UB_Q8_0_BYTES;

  for (int n = blockIdx.x * kWarps + warp; n < N; n += gridDim.x * kWarps) {
    const uint8_t* row = wq + static_cast<size_t>(n) * row_bytes;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.f;

    if (FAST) {
      const int nruns = nblk >> 3;
      for (int run = lane; run < nruns; run += 32) {
        uint32_t r[69];
        const uint4* p = reinterpret_cast<const uint4*>(row + static_cast<size_t>(run) * 272);
#pragma unroll
        for (int i = 0; i < 17; i++) {
          const uint4 v = __ldg(p + i);
          r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
        }
        r[68] = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int off = 34 * j;  // compile-time after unrolling
          const uint32_t dw = __funnelshift_r(r[off >> 2], r[(off >> 2) + 1], (off & 3) * 8);
          const float d = half_bits_to_f32(dw);
          uint32_t q[8];
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int qo = off + 2 + 4 * i;
            q[i] = __funnelshift_r(r[qo >> 2], r[(qo >> 2) + 1], (qo & 3) * 8) ^ 0x80808080u;
          }
#pragma unroll
          for (int m = 0; m < MT; m++) {
            const XT* xr = x + static_cast<size_t>(m) * K + (static_cast<size_t>(run) * 8 + j) * 32;
            float s = 0.f;
#pragma unroll
            for (int c = 0; c < 4; c++) {
              float xv[8];
              load_x8<XT>(xr + 8 * c, xv);
              s = fmaf(s8_exact<0>(q[2 * c]), xv[0], s); s = fmaf(s8_exact<1>(q[2 * c]), xv[1], s);
              s = fmaf(s8_exact<2>(q[2 * c]), xv[2], s); s = fmaf(s8_exact<3>(q[2 * c]), xv[3], s);
              s = fmaf(s8_exact<0>(q[2 * c + 1]), xv[4], s); s = fmaf(s8_exact<1>(q[2 * c + 1]), xv[5], s);
              s = fmaf(s8_exact<2>(q[2 * c + 1]), xv[6], s); s = fmaf(s8_exact<3>(q[2 * c + 1]), xv[7], s);
            }
            acc[m] = fmaf(d, s, acc[m]);
          }
        }
      }
    } else {
      for (int b = lane; b < nblk; b += 32) {
        const unsigned short* p = reinterpret_cast<const unsigned short*>(row + static_cast<size_t>(b) * UB_Q8_0_BYTES);
        const float d = half_bits_to_f32(__ldg(p));
        uint32_t q[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
          q[i] = (static_cast<uint32_t>(__ldg(p + 1 + 2 * i)) | (static_cast<uint32_t>(__ldg(p + 2 + 2 * i)) << 16)) ^
                 0x80808080u;
#pragma unroll
        for (int m = 0; m < MT; m++) {
          const XT* xr = x + static_cast<size_t>(m) * K + static_cast<size_t>(b) * 32;
          float s = 0.f;
#pragma unroll
          for (int c = 0; c < 4; c++) {
            float xv[8];
            load_x8<XT>(xr + 8 * c, xv);
            s = fmaf(s8_exact<0>(q[2 * c]), xv[0], s); s = fmaf(s8_exact<1>(q[2 * c]), xv[1], s);
            s = fmaf(s8_exact<2>(q[2 * c]), xv[2], s); s = fmaf(s8_exact<3>(q[2 * c]), xv[3], s);
            s = fmaf(s8_exact<0>(q[2 * c + 1]), xv[4], s); s = fmaf(s8_exact<1>(q[2 * c + 1]), xv[5], s);
            s = fmaf(s8_exact<2>(q[2 * c + 1]), xv[6], s); s = fmaf(s8_exact<3>(q[2 * c + 1]), xv[7], s);
          }
          acc[m] = fmaf(d, s, acc[m]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
      const float rsum = warp_sum(acc[m]);
      if (lane == 0) store_y(y, static_cast<size_t>(m) * N + n, y_dtype, rsum);
    }
  }
}

inline int gemv_grid(int N) {
  const int want = (N + kWarps - 1) / kWarps;
  const int cap = ub::num_sms() * 8;
  return want < cap ? (want > 0 ? want : 1) : cap;
}

template <typename XT, int MT>
int launch_q4k(const uint8_t* wq, const XT* x, void* y, int N, int K, int y_dtype, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(MT) * (K / 32) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(qgemv_q4k_kernel<XT, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) {
      ub::set_cuda_error(e);
      return ub::fail(UB_ERR_CUDA);
    }
  }
  qgemv_q4k_kernel<XT, MT><<<gemv_grid(N), kThreads, smem, s>>>(wq, x, y, N, K, y_dtype);
  return ub::check_launch();
}

template <typename XT, int MT>
int launch_q8_0(const uint8_t* wq, const XT* x, void* y, int N, int K, int y_dtype, cudaStream_t s) {
  const bool fast = (K % 256 == 0) && ((reinterpret_cast<uintptr_t>(wq) & 15) == 0);
  if (fast)
    qgemv_q8_0_kernel<XT, MT, true><<<gemv_grid(N), kThreads, 0, s>>>(wq, x, y, N, K, y_dtype);
  else
    qgemv_q8_0_kernel<XT, MT, false><<<gemv_grid(N), kThreads, 0, s>>>(wq, x, y, N, K, y_dtype);
  return ub::check_launch();
}

inline size_t dtype_size(int dt) { return dt == UB_DTYPE_F32 ? 4 : 2; }

}  // namespace

namespace ub {

// Rows of x are processed four (then two, then one) at a time; each pass streams W once.
template <typename XT>
int qgemv(bool is_q4k, void* y, const XT* x, const void* wq, int M, int N, int K, int y_dtype, cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  int m0 = 0;
  while (m0 < M) {
    const int left = M - m0;
    const int mt = left >= 4 ? 4 : (left >= 2 ? 2 : 1);
    const XT* xp = x + static_cast<size_t>(m0) * K;
    void* yp = static_cast<char*>(y) + static_cast<size_t>(m0) * N * dtype_size(y_dtype);
    int st;
    if (is_q4k) {
      st = mt == 4 ? launch_q4k<XT, 4>(w, xp, yp, N, K, y_dtype, s)
                   : (mt == 2 ? launch_q4k<XT, 2>(w, xp, yp, N, K, y_dtype, s)
                              : launch_q4k<XT, 1>(w, xp, yp, N, K, y_dtype, s));
    } else {
      st = mt == 4 ? launch_q8_0<XT, 4>(w, xp, yp, N, K, y_dtype, s)
                   : (mt == 2 ? launch_q8_0<XT, 2>(w, xp, yp, N, K, y_dtype, s)
                              : launch_q8_0<XT, 1>(w, xp, yp, N, K, y_dtype, s));
    }
    if (st != UB_OK) return st;
    m0 += mt;
  }
  return ub::fail(UB_OK);
}

template int qgemv<float>(bool, void*, const float*, const void*, int, int, int, int, cudaStream_t);
template int qgemv<__nv_bfloat16>(bool, void*, const __nv_bfloat16*, const void*, int, int, int, int, cudaStream_t);

}  // namespace ub
