// GGUF tensor entry points: dispatch on the GGML type tag, plus two more block formats.
//
// A GGUF file stores a tensor as (type tag, dims, raw bytes of interleaved blocks).  These entries take exactly
// that: the blob's bytes as they lie in the file (no repack: the kernels of this library consume interleaved
// blocks), the type tag, and the logical shape.  The reference declares the block structs of the whole family
// (kernels/quant.cpp:64-185: block_q4_0 .. block_q8_K) and ships kernels for Q8_0 and Q4_K only
// (dequantize_block_* :257-268,477-488); Q6_K lives in q6k.cu, and this file adds
//   Q4_0 (kernels/quant.cpp:64-69:   18 bytes = f16 d + 16 bytes; y = d * (nibble - 8), low nibbles are values
//         0..15 of the block, high nibbles values 16..31)
//   Q5_K (kernels/quant.cpp:154-161: 176 bytes = f16 d, f16 dmin, 12 bytes of 6-bit scales/mins packed as in
//         Q4_K, qh[32] fifth bits, qs[128] low nibbles; for 64-value group g: values 0..31 take the low nibbles
//         of qs[32g..], bit 2g of qh[l] and pair 2g, values 32..63 the high nibbles, bit 2g+1 and pair 2g+1;
//         y = d * sc * q - dmin * m)
// with the published GGML arithmetic.  Their matmul is a plain bandwidth kernel (a warp per weight row,
// activations staged in shared memory as f32, f32 FMA, fixed reduction order), for up to eight tokens per pass.
#include "common.cuh"

#define UB_Q4_0_BYTES 18
#define UB_Q5K_BYTES 176

// GGML type tags (the values GGUF files carry)
enum { GGML_Q4_0 = 2, GGML_Q8_0 = 8, GGML_Q4_K = 12, GGML_Q5_K = 13, GGML_Q6_K = 14 };

namespace ub {
template <typename XT>
int q5k_gemv_staged(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s);
template <typename XT>
int q4_0_gemv_staged(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s);
}

namespace {

using namespace ub;

__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) { return __ldg(reinterpret_cast<const unsigned short*>(p)); }

// ---- Q4_0: a thread per (block, nibble byte) ----
template <typename T>
__global__ void __launch_bounds__(256) dequant_q4_0_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, size_t nb) {
  const size_t total = nb * 16;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t b = i >> 4;
    const int l = static_cast<int>(i & 15);
    const uint8_t* blk = in + b * UB_Q4_0_BYTES;
    const float d = half_bits_to_f32(ld_u16(blk));
    const uint32_t q = __ldg(blk + 2 + l);
    out[b * 32 + l] = from_f32<T>(d * static_cast<float>(static_cast<int>(q & 15) - 8));
    out[b * 32 + 16 + l] = from_f32<T>(d * static_cast<float>(static_cast<int>(q >> 4) - 8));
  }
}

// ---- Q5_K: a warp per super-block; lane = position l of every 32-value sub-block ----
template <typename T>
__global__ void __launch_bounds__(256) dequant_q5k_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, size_t nb) {
  const int lane = threadIdx.x & 31;
  const size_t warps = static_cast<size_t>(gridDim.x) * (blockDim.x >> 5);
  for (size_t b = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); b < nb; b += warps) {
    const uint8_t* blk = in + b * UB_Q5K_BYTES;
    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));  // blocks are 16-byte aligned (176 = 11 * 16)
    const float d = half_bits_to_f32(hdr.x), dmin = half_bits_to_f32(hdr.x >> 16);
    uint32_t scw[2], mnw[2];
    q4k_unpack_scales(hdr.y, hdr.z, hdr.w, scw[0], scw[1], mnw[0], mnw[1]);
    const uint32_t qh = __ldg(blk + 16 + lane);
    T* o = out + b * UB_QK_K;
#pragma unroll
    for (int g = 0; g < 4; g++) {
      const uint32_t q = __ldg(blk + 48 + 32 * g + lane);
      const int j0 = 2 * g, j1 = 2 * g + 1;
      const float d0 = __fmul_rn(d, static_cast<float>((scw[j0 >> 2] >> (8 * (j0 & 3))) & 0xFF));
      const float m0 = __fmul_rn(dmin, static_cast<float>((mnw[j0 >> 2] >> (8 * (j0 & 3))) & 0xFF));
      const float d1 = __fmul_rn(d, static_cast<float>((scw[j1 >> 2] >> (8 * (j1 & 3))) & 0xFF));
      const float m1 = __fmul_rn(dmin, static_cast<float>((mnw[j1 >> 2] >> (8 * (j1 & 3))) & 0xFF));
      const int q0 = static_cast<int>(q & 15) + (((qh >> j0) & 1) << 4);
      const int q1 = static_cast<int>(q >> 4) + (((qh >> j1) & 1) << 4);
      // product and difference rounded separately (no fused multiply-add): the bits of the format's definition
      o[64 * g + lane] = from_f32<T>(__fsub_rn(__fmul_rn(d0, static_cast<float>(q0)), m0));
      o[64 * g + 32 + lane] = from_f32<T>(__fsub_rn(__fmul_rn(d1, static_cast<float>(q1)), m1));
    }
  }
}

// ---- matmul for the two formats: a warp per weight row, up to MT tokens per pass ----
// FMT 0: Q4_0, FMT 1: Q5_K.  xs: [MT][K] f32 in shared memory.
template <int FMT, int MT>
__device__ __forceinline__ void row_dot(const uint8_t* __restrict__ row, const float* __restrict__ xs, int K, int lane,
                                        float (&acc)[MT]) {
  if (FMT == 0) {
    // a lane takes nibble byte l = lane & 15 of every other block: the lower and the upper half-warp interleave blocks
    const int l = lane & 15, half = lane >> 4;
    for (int b = half; b < K / 32; b += 2) {
      const uint8_t* blk = row + static_cast<size_t>(b) * UB_Q4_0_BYTES;
      const float d = half_bits_to_f32(ld_u16(blk));
      const uint32_t q = __ldg(blk + 2 + l);
      const float w0 = d * static_cast<float>(static_cast<int>(q & 15) - 8);
      const float w1 = d * static_cast<float>(static_cast<int>(q >> 4) - 8);
#pragma unroll
      for (int m = 0; m < MT; m++) {
        const float* x = xs + static_cast<size_t>(m) * K + b * 32;
        acc[m] = fmaf(w0, x[l], fmaf(w1, x[16 + l], acc[m]));
      }
    }
  } else {
    for (int sb = 0; sb < K / 256; sb++) {
      const uint8_t* blk = row + static_cast<size_t>(sb) * UB_Q5K_BYTES;
      const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));
      const float d = half_bits_to_f32(hdr.x), dmin = half_bits_to_f32(hdr.x >> 16);
      uint32_t scw[2], mnw[2];
      q4k_unpack_scales(hdr.y, hdr.z, hdr.w, scw[0], scw[1], mnw[0], mnw[1]);
      const uint32_t qh = __ldg(blk + 16 + lane);
#pragma unroll
      for (int g = 0; g < 4; g++) {
        const uint32_t q = __ldg(blk + 48 + 32 * g + lane);
        const int j0 = 2 * g, j1 = 2 * g + 1;
        const float w0 = d * static_cast<float>((scw[j0 >> 2] >> (8 * (j0 & 3))) & 0xFF) *
                             static_cast<float>(static_cast<int>(q & 15) + (((qh >> j0) & 1) << 4)) -
                         dmin * static_cast<float>((mnw[j0 >> 2] >> (8 * (j0 & 3))) & 0xFF);
        const float w1 = d * static_cast<float>((scw[j1 >> 2] >> (8 * (j1 & 3))) & 0xFF) *
                             static_cast<float>(static_cast<int>(q >> 4) + (((qh >> j1) & 1) << 4)) -
                         dmin * static_cast<float>((mnw[j1 >> 2] >> (8 * (j1 & 3))) & 0xFF);
#pragma unroll
        for (int m = 0; m < MT; m++) {
          const float* x = xs + static_cast<size_t>(m) * K + sb * 256 + 64 * g;
          acc[m] = fmaf(w0, x[lane], fmaf(w1, x[32 + lane], acc[m]));
        }
      }
    }
  }
}

template <typename XT, int FMT, int MT>
__global__ void __launch_bounds__(256) qgemv_gguf_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x,
                                                         void* __restrict__ y, int M, int N, int K, int y_dtype) {
  extern __shared__ float xs[];  // [MT][K]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < MT * K; i += blockDim.x) {
    const int m = i / K;
    xs[i] = m < M ? to_f32(x[i]) : 0.f;
  }
  __syncthreads();
  const size_t row_bytes = FMT == 0 ? static_cast<size_t>(K / 32) * UB_Q4_0_BYTES : static_cast<size_t>(K / 256) * UB_Q5K_BYTES;
  for (int n = blockIdx.x * 8 + warp; n < N; n += gridDim.x * 8) {
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.f;
    row_dot<FMT, MT>(wq + static_cast<size_t>(n) * row_bytes, xs, K, lane, acc);
#pragma unroll
    for (int m = 0; m < MT; m++) {
      const float v = warp_sum(acc[m]);
      if (lane == 0 && m < M) {
        const size_t idx = static_cast<size_t>(m) * N + n;
        if (y_dtype == UB_DTYPE_F32)
          static_cast<float*>(y)[idx] = v;
        else if (y_dtype == UB_DTYPE_BF16)
          static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
        else
          static_cast<__half*>(y)[idx] = __float2half_rn(v);
      }
    }
  }
}

template <typename XT, int FMT, int MT>
int launch_gguf_gemv(const uint8_t* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(MT) * K * sizeof(float);
  if (smem > 200 * 1024) return ub::fail(UB_ERR_TOO_LARGE);
  auto kernel = qgemv_gguf_kernel<XT, FMT, MT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) {
      ub::set_cuda_error(e);
      return ub::fail(UB_ERR_CUDA);
    }
  }
  int grid = (N + 7) / 8;
  const int cap = ub::num_sms() * 4;
  if (grid > cap) grid = cap;
  kernel<<<grid, 256, smem, s>>>(wq, x, y, M, N, K, y_dtype);
  return ub::check_launch();
}

template <typename XT, int FMT>
int gguf_matmul(void* y, const XT* x, const void* wq, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  const size_t esz = y_dtype == UB_DTYPE_F32 ? 4 : 2;
  for (int m0 = 0; m0 < M;) {
    const int left = M - m0;
    const XT* xp = x + static_cast<size_t>(m0) * K;
    void* yp = static_cast<char*>(y) + static_cast<size_t>(m0) * N * esz;
    int st, step;
    {  // rows of whole 2048 values: staged by bulk copies, dp4a on fixed-point activations
      step = left < 4 ? left : 4;
      st = FMT == 1 ? ub::q5k_gemv_staged<XT>(w, xp, yp, step, N, K, y_dtype, fresh, s)
                    : ub::q4_0_gemv_staged<XT>(w, xp, yp, step, N, K, y_dtype, fresh, s);
      if (st == UB_OK) {
        m0 += step;
        continue;
      }
      if (st != UB_ERR_UNSUPPORTED) return st;
    }
    // tokens per pass: as many as the activations' f32 copy leaves room for in shared memory
    if (left >= 4 && static_cast<size_t>(4) * K * 4 <= 200 * 1024) {
      step = left < 4 ? left : 4;
      st = launch_gguf_gemv<XT, FMT, 4>(w, xp, yp, step, N, K, y_dtype, s);
    } else if (left >= 2 && static_cast<size_t>(2) * K * 4 <= 200 * 1024) {
      step = 2;
      st = launch_gguf_gemv<XT, FMT, 2>(w, xp, yp, step, N, K, y_dtype, s);
    } else {
      step = 1;
      st = launch_gguf_gemv<XT, FMT, 1>(w, xp, yp, step, N, K, y_dtype, s);
    }
    if (st != UB_OK) return st;
    m0 += step;
  }
  return ub::fail(UB_OK);
}

inline int grid_blocks(size_t items, int per_block) {
  size_t b = (items + per_block - 1) / per_block;
  const size_t cap = static_cast<size_t>(ub::num_sms()) * 16;
  return static_cast<int>(b > cap ? cap : (b ? b : 1));
}

}  // namespace

extern "C" {

int ub_dequant_q8_0(void* out, const void* blocks, size_t numel, int out_dtype, void* stream);
int ub_dequant_q4k(void* out, const void* blocks, size_t numel, int out_dtype, void* stream);
int ub_dequant_q6k(void* out, const void* blocks, size_t numel, int out_dtype, void* stream);

// values per block and bytes per block of a GGML type this library takes; 0 for the others
int ub_gguf_block_values(int ggml_type) {
  switch (ggml_type) {
    case GGML_Q4_0: case GGML_Q8_0: return 32;
    case GGML_Q4_K: case GGML_Q5_K: case GGML_Q6_K: return 256;
    default: return 0;
  }
}
int ub_gguf_block_bytes(int ggml_type) {
  switch (ggml_type) {
    case GGML_Q4_0: return UB_Q4_0_BYTES;
    case GGML_Q8_0: return UB_Q8_0_BYTES;
    case GGML_Q4_K: return UB_Q4K_BYTES;
    case GGML_Q5_K: return UB_Q5K_BYTES;
    case GGML_Q6_K: return 210;
    default: return 0;
  }
}

// Bytes of a GGUF tensor blob with `numel` values of that type (0 when the type is not taken or numel is not a
// whole number of blocks).
size_t ub_gguf_tensor_bytes(int ggml_type, size_t numel) {
  const int per = ub_gguf_block_values(ggml_type);
  if (!per || numel % per) return 0;
  return numel / per * ub_gguf_block_bytes(ggml_type);
}

int ub_dequant_gguf(void* out, const void* blob, int ggml_type, size_t numel, int out_dtype, void* stream) {
  switch (ggml_type) {
    case GGML_Q8_0: return ub_dequant_q8_0(out, blob, numel, out_dtype, stream);
    case GGML_Q4_K: return ub_dequant_q4k(out, blob, numel, out_dtype, stream);
    case GGML_Q6_K: return ub_dequant_q6k(out, blob, numel, out_dtype, stream);
    default: break;
  }
  if (ggml_type != GGML_Q4_0 && ggml_type != GGML_Q5_K) return ub::fail(UB_ERR_UNSUPPORTED);
  if (numel == 0) return ub::fail(UB_OK);
  const int per = ub_gguf_block_values(ggml_type);
  if (!out || !blob || numel % per) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t nb = numel / per;
  cudaStream_t s = ub::as_stream(stream);
  const uint8_t* in = static_cast<const uint8_t*>(blob);
  if (ggml_type == GGML_Q4_0) {
    if (reinterpret_cast<uintptr_t>(blob) & 1) return ub::fail(UB_ERR_INVALID_ARG);
    UB_DISPATCH_FLOAT(out_dtype, T, (dequant_q4_0_kernel<T><<<grid_blocks(nb * 16, 256), 256, 0, s>>>(
                                        in, static_cast<T*>(out), nb)));
  } else {
    if (reinterpret_cast<uintptr_t>(blob) & 15) return ub::fail(UB_ERR_INVALID_ARG);
    UB_DISPATCH_FLOAT(out_dtype, T, (dequant_q5k_kernel<T><<<grid_blocks(nb, 8), 256, 0, s>>>(in, static_cast<T*>(out), nb)));
  }
  return ub::check_launch();
}

int ub_qmatmul_q8_0_f32(void*, const void*, const void*, int, int, int, int, void*, size_t, void*);
int ub_qmatmul_q8_0_bf16(void*, const void*, const void*, int, int, int, int, void*, size_t, void*);
int ub_qmatmul_q4k_f32(void*, const void*, const void*, int, int, int, int, void*, size_t, void*);
int ub_qmatmul_q4k_bf16(void*, const void*, const void*, int, int, int, int, void*, size_t, void*);
int ub_qmatmul_q6k_f32(void*, const void*, const void*, int, int, int, int, void*);
int ub_qmatmul_q6k_bf16(void*, const void*, const void*, int, int, int, int, void*);
size_t ub_qmatmul_workspace_bytes(int M, int N, int K, int is_q4k);

size_t ub_qmatmul_gguf_workspace_bytes(int ggml_type, int M, int N, int K) {
  return ggml_type == GGML_Q4_K ? ub_qmatmul_workspace_bytes(M, N, K, 1) : 0;
}

// y[M,N] = x[M,K] . W^T for a GGUF tensor blob W of N rows x K values; x_dtype f32 / bf16.
int ub_qmatmul_gguf(void* y, const void* x, const void* blob, int ggml_type, int M, int N, int K, int x_dtype,
                    int out_dtype, void* workspace, size_t ws_bytes, void* stream) {
  if (x_dtype != UB_DTYPE_F32 && x_dtype != UB_DTYPE_BF16) return ub::fail(UB_ERR_INVALID_ARG);
  const bool f32 = x_dtype == UB_DTYPE_F32;
  switch (ggml_type) {
    case GGML_Q8_0:
      return (f32 ? ub_qmatmul_q8_0_f32 : ub_qmatmul_q8_0_bf16)(y, x, blob, M, N, K, out_dtype, workspace, ws_bytes, stream);
    case GGML_Q4_K:
      return (f32 ? ub_qmatmul_q4k_f32 : ub_qmatmul_q4k_bf16)(y, x, blob, M, N, K, out_dtype, workspace, ws_bytes, stream);
    case GGML_Q6_K:
      return (f32 ? ub_qmatmul_q6k_f32 : ub_qmatmul_q6k_bf16)(y, x, blob, M, N, K, out_dtype, stream);
    default: break;
  }
  if (ggml_type != GGML_Q4_0 && ggml_type != GGML_Q5_K) return ub::fail(UB_ERR_UNSUPPORTED);
  // UB_QMATMUL_WEIGHTS_FRESH rides in the upper bits of out_dtype, as in ub_qmatmul_*
  bool fresh = (out_dtype & UB_QMATMUL_WEIGHTS_FRESH) != 0;
  out_dtype &= ~UB_QMATMUL_WEIGHTS_FRESH;
  if (M == 0 || N == 0) return ub::fail(UB_OK);
  const int per = ub_gguf_block_values(ggml_type);
  if (!y || !x || !blob || M < 0 || N < 0 || K <= 0 || K % per) return ub::fail(UB_ERR_INVALID_ARG);
  if (out_dtype != UB_DTYPE_F32 && out_dtype != UB_DTYPE_BF16 && out_dtype != UB_DTYPE_F16)
    return ub::fail(UB_ERR_INVALID_ARG);
  if (reinterpret_cast<uintptr_t>(blob) & (ggml_type == GGML_Q5_K ? 15 : 1)) return ub::fail(UB_ERR_INVALID_ARG);
  cudaStream_t s = ub::as_stream(stream);
  if (ub::take_weights_written(s)) fresh = true;
  if (ggml_type == GGML_Q4_0)
    return f32 ? gguf_matmul<float, 0>(y, static_cast<const float*>(x), blob, M, N, K, out_dtype, fresh, s)
               : gguf_matmul<__nv_bfloat16, 0>(y, static_cast<const __nv_bfloat16*>(x), blob, M, N, K, out_dtype, fresh, s);
  return f32 ? gguf_matmul<float, 1>(y, static_cast<const float*>(x), blob, M, N, K, out_dtype, fresh, s)
             : gguf_matmul<__nv_bfloat16, 1>(y, static_cast<const __nv_bfloat16*>(x), blob, M, N, K, out_dtype, fresh, s);
}

}  // extern "C"
