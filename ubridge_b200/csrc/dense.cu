// Dense matmul and Enflame-style groupwise W4A16 / W8A16 matmul behind the reference's names, plus the
// standalone W4A16 dequantiser.
//
//   matmul_{f32,f16,bf16}           out[B,M,N] = lhs[B,M,K] . rhs[B or 1,K,N]       kernels/matmul.cpp:36-514,1143-1184
//   matmul_{f16,bf16}_{4bit,8bit}   rhs given as packed nibbles / int8 + scales (+ zeros) kernels/matmul.cpp:516-1140,1186-1215
//   dequant_{f16,bf16}              packed nibbles -> dense T                        kernels/dequant_host.cpp:19-306
//
// These are the compatibility entries of the path: a caller that dequantises and then multiplies by name finds
// the names it binds to.  The GGUF formats go through the fused kernels instead (qmatmul.cu), which is where
// the time is spent; this file is a plain shared-memory tiled kernel with f32 accumulation on the CUDA cores,
// correct for every flag combination and not tuned.
//
// Semantics taken from the reference: operands row-major, `lhs_transpose` means lhs is stored [K,M],
// `rhs_transpose` means rhs is stored [N,K] (kernels/matmul.cpp:96-110); `broadcasted_weight` shares one rhs
// across the batch (:102); alpha / beta / addmm_beta are carried in the parameter list but the reference kernel
// only zero-fills its accumulator (:280-286), so out = lhs . rhs; the multicore and sip_* tiling hints are
// accepted and ignored.
//
// W4A16 / W8A16 convention (ASSUMED: the reference unpacks inside a vendor routine whose code is not part of
// its source tree, so parity with it is unpinned):
//   4 bit: rhs is u8 [K/2, N] (rhs_transpose: [N, K/2]); the byte at packed row r holds reduction index 2r in
//          its low nibble and 2r+1 in its high nibble; w[k,n] = (q - zeros[k/g, n]) * scales[k/g, n];
//   8 bit: rhs is i8 [K, N] (rhs_transpose: [N, K]);     w[k,n] = q * scales[k/g, n];
//   scales / zeros are T [K/g, N]; group_size <= 0 means one group over all of K.
#include "common.cuh"

namespace {

using namespace ub;

constexpr int kTM = 64, kTN = 64, kTK = 32;

struct DenseArgs {
  const void* a;
  const void* b;
  void* out;
  const void* scales;
  const void* zeros;
  int B, M, K, N;
  int lhs_t, rhs_t, bcast_w, group;
};

// QUANT: 0 dense, 1 packed nibbles, 2 int8
template <typename T, int QUANT>
__global__ void __launch_bounds__(256) dense_matmul_kernel(DenseArgs p) {
  __shared__ float As[kTK][kTM + 1];
  __shared__ float Bs[kTK][kTN + 1];
  const int bz = blockIdx.z;
  const int m0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // thread computes rows ty*4.., cols tx*4..
  const T* A = static_cast<const T*>(p.a) + static_cast<size_t>(bz) * p.M * p.K;
  const size_t b_elems = QUANT == 1 ? static_cast<size_t>(p.K / 2) * p.N : static_cast<size_t>(p.K) * p.N;
  const size_t b_off = p.bcast_w ? 0 : static_cast<size_t>(bz) * b_elems;
  const int group = p.group > 0 ? p.group : p.K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < p.K; k0 += kTK) {
    for (int e = threadIdx.x; e < kTK * kTM; e += 256) {
      // consecutive threads walk the contiguous dimension of the operand
      const int kk = p.lhs_t ? e / kTM : e % kTK, mm = p.lhs_t ? e % kTM : e / kTK;
      const int k = k0 + kk, m = m0 + mm;
      float v = 0.f;
      if (k < p.K && m < p.M) v = to_f32(p.lhs_t ? A[static_cast<size_t>(k) * p.M + m] : A[static_cast<size_t>(m) * p.K + k]);
      As[kk][mm] = v;
    }
    for (int e = threadIdx.x; e < kTK * kTN; e += 256) {
      const int kk = p.rhs_t ? e % kTK : e / kTN, nn = p.rhs_t ? e / kTK : e % kTN;
      const int k = k0 + kk, n = n0 + nn;
      float v = 0.f;
      if (k < p.K && n < p.N) {
        if (QUANT == 0) {
          const T* Bp = static_cast<const T*>(p.b) + b_off;
          v = to_f32(p.rhs_t ? Bp[static_cast<size_t>(n) * p.K + k] : Bp[static_cast<size_t>(k) * p.N + n]);
        } else {
          const size_t sidx = static_cast<size_t>(k / group) * p.N + n;
          const float sc = to_f32(static_cast<const T*>(p.scales)[sidx]);
          if (QUANT == 1) {
            const uint8_t* Bp = static_cast<const uint8_t*>(p.b) + b_off;
            const uint8_t byte = p.rhs_t ? Bp[static_cast<size_t>(n) * (p.K / 2) + (k >> 1)]
                                         : Bp[static_cast<size_t>(k >> 1) * p.N + n];
            const float q = static_cast<float>((k & 1) ? (byte >> 4) : (byte & 15));
            const float z = p.zeros ? to_f32(static_cast<const T*>(p.zeros)[sidx]) : 0.f;
            v = (q - z) * sc;
          } else {
            const int8_t* Bp = static_cast<const int8_t*>(p.b) + b_off;
            const int8_t q = p.rhs_t ? Bp[static_cast<size_t>(n) * p.K + k] : Bp[static_cast<size_t>(k) * p.N + n];
            v = static_cast<float>(q) * sc;
          }
          // the reference dequantises into the activation type before its matrix engine sees the tile
          v = to_f32(from_f32<T>(v));
        }
      }
      Bs[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTK; kk++) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i], bv[i] = Bs[kk][tx * 4 + i];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  T* O = static_cast<T*>(p.out) + static_cast<size_t>(bz) * p.M * p.N;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < p.N) O[static_cast<size_t>(m) * p.N + n] = from_f32<T>(acc[i][j]);
    }
  }
}

template <typename T, int QUANT>
int dense_launch(const DenseArgs& p, cudaStream_t s) {
  if (p.B == 0 || p.M == 0 || p.N == 0) return ub::fail(UB_OK);
  if (!p.a || !p.b || !p.out || p.B < 0 || p.M < 0 || p.N < 0 || p.K <= 0) return ub::fail(UB_ERR_INVALID_ARG);
  if (QUANT != 0 && !p.scales) return ub::fail(UB_ERR_INVALID_ARG);
  if (QUANT == 1 && (p.K & 1)) return ub::fail(UB_ERR_INVALID_ARG);
  if (p.group > 0 && p.K % p.group) return ub::fail(UB_ERR_INVALID_ARG);
  if (p.B > 65535) return ub::fail(UB_ERR_TOO_LARGE);
  dim3 grid((p.N + kTN - 1) / kTN, (p.M + kTM - 1) / kTM, p.B);
  dense_matmul_kernel<T, QUANT><<<grid, 256, 0, s>>>(p);
  return ub::check_launch();
}

// out[k, n] = (q - zeros[k/g, n]) * scale[k/g, n]; packed as documented at the top of the file
template <typename T>
__global__ void dequant_w4_kernel(T* __restrict__ out, const uint8_t* __restrict__ rhs, const T* __restrict__ scale,
                                  const T* __restrict__ zeros, int K, int N, int weight_transpose, int group) {
  const size_t total = static_cast<size_t>(K) * N;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int k = static_cast<int>(i / N), n = static_cast<int>(i - static_cast<size_t>(k) * N);
    const uint8_t byte = weight_transpose ? rhs[static_cast<size_t>(n) * (K / 2) + (k >> 1)]
                                          : rhs[static_cast<size_t>(k >> 1) * N + n];
    const float q = static_cast<float>((k & 1) ? (byte >> 4) : (byte & 15));
    const size_t sidx = static_cast<size_t>(k / group) * N + n;
    const float z = zeros ? to_f32(zeros[sidx]) : 0.f;
    out[i] = from_f32<T>((q - z) * to_f32(scale[sidx]));
  }
}

template <typename T>
void dequant_w4_launch(void* out, const uint8_t* rhs, const void* scale, const void* zeros, int K, int N,
                       int weight_transpose, int group_size, cudaStream_t s) {
  if (K == 0 || N == 0) {
    ub::set_status(UB_OK);
    return;
  }
  const int group = group_size > 0 ? group_size : K;
  if (!out || !rhs || !scale || K < 0 || N < 0 || (K & 1) || K % group) {
    ub::set_status(UB_ERR_INVALID_ARG);
    return;
  }
  const size_t total = static_cast<size_t>(K) * N;
  size_t blocks = (total + 255) / 256;
  const size_t cap = static_cast<size_t>(ub::num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  dequant_w4_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<T*>(out), rhs,
                                                                      static_cast<const T*>(scale),
                                                                      static_cast<const T*>(zeros), K, N,
                                                                      weight_transpose, group);
  ub::check_launch();
}

}  // namespace

namespace ub {

// quant: 0 dense, 1 packed nibbles, 2 int8.  dtype: UB_DTYPE_F32 (dense only) / F16 / BF16.
int dense_matmul(int dtype, int quant, const void* a, const void* b, void* out, const void* scales, const void* zeros,
                 int B, int M, int K, int N, int lhs_t, int rhs_t, int bcast_w, int group, cudaStream_t s) {
  DenseArgs p{a, b, out, scales, zeros, B, M, K, N, lhs_t != 0, rhs_t != 0, bcast_w != 0, group};
  if (quant == 0) {
    UB_DISPATCH_FLOAT(dtype, T, return (dense_launch<T, 0>(p, s)));
  }
  if (dtype == UB_DTYPE_F16) return quant == 1 ? dense_launch<__half, 1>(p, s) : dense_launch<__half, 2>(p, s);
  if (dtype == UB_DTYPE_BF16)
    return quant == 1 ? dense_launch<__nv_bfloat16, 1>(p, s) : dense_launch<__nv_bfloat16, 2>(p, s);
  return ub::fail(UB_ERR_INVALID_ARG);
}

}  // namespace ub

extern "C" {

void dequant_f16(void* out, uint8_t* rhs, void* scale, void* zeros, int K, int N, int weight_transpose,
                 int group_size, void* stream) {
  dequant_w4_launch<__half>(out, rhs, scale, zeros, K, N, weight_transpose, group_size, ub::as_stream(stream));
}
void dequant_bf16(void* out, uint8_t* rhs, void* scale, void* zeros, int K, int N, int weight_transpose,
                  int group_size, void* stream) {
  dequant_w4_launch<__nv_bfloat16>(out, rhs, scale, zeros, K, N, weight_transpose, group_size,
                                   ub::as_stream(stream));
}

}  // extern "C"
