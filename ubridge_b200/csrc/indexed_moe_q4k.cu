// indexed_moe on Q4_K expert weights: the decode-time sibling of the grouped expert GEMM.
//
//   out[b, t, :] = in[b, (M == 1 ? 0 : t), :] . dequant(Wq[indices[b, t]])^T
//
// in [batch, M, K] (M = 1 or topk), Wq [num_experts][N rows of K/256 Q4_K super-blocks], indices [batch, topk],
// out [batch, topk, N]: the contract of the reference's indexed_moe_{f16,bf16} (kernels/moe_host.cpp:100-109,
// 278-293, CPU statement :325-353) with the expert matrices kept in GGUF blocks (kernels/quant.cpp:145-150,
// scales :356-363) instead of dense T.  The reference runs this for small batches (its decode variant is chosen
// for batch <= 12, :285-289): every (token, slot) pair is a matrix-vector product against ITS expert, so the
// work is a set of independent weight streams and the kernel is bandwidth bound.
//
// One CTA = one (token, slot) pair and 64 output rows; the activation row is staged once in shared memory as
// f32; a warp owns one weight row at a time, a lane one 4-byte piece of every 32-byte nibble group (consecutive
// lanes read consecutive words: coalesced), f32 FMA against the activations, the 6-bit scales and mins applied
// once per sub-block and lane, a fixed shuffle order (deterministic).  An expert index outside
// [0, num_experts) writes zeros and records UB_ERR_BAD_INDEX in the device error word instead of trapping.
#include "common.cuh"

namespace {

using namespace ub;

constexpr int kRowsPerCta = 64;

template <typename T>
__global__ void __launch_bounds__(256) indexed_moe_q4k_kernel(const T* __restrict__ in, const uint8_t* __restrict__ wq,
                                                              T* __restrict__ out, const uint32_t* __restrict__ indices,
                                                              int N, int K, int M, int topk, int num_experts,
                                                              int* err_word) {
  extern __shared__ float xs[];  // [K]
  const int bt = blockIdx.y;     // flat (token, slot)
  const int b = bt / topk, t = bt - b * topk;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = blockIdx.x * kRowsPerCta;
  const uint32_t e = indices[bt];
  T* const orow = out + static_cast<size_t>(bt) * N;
  if (e >= static_cast<uint32_t>(num_experts)) {
    if (threadIdx.x == 0) report_device_error(err_word, UB_ERR_BAD_INDEX);
    for (int r = threadIdx.x; r < kRowsPerCta; r += blockDim.x)
      if (n0 + r < N) orow[n0 + r] = from_f32<T>(0.f);
    return;
  }
  const T* xr = in + (static_cast<size_t>(b) * M + (M == 1 ? 0 : t)) * K;
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_f32(xr[k]);
  __syncthreads();
  const int nsb = K >> 8;
  const size_t row_bytes = static_cast<size_t>(nsb) * UB_Q4K_BYTES;
  const uint8_t* const wbase = wq + static_cast<size_t>(e) * N * row_bytes;
  const int G = lane >> 3, pos = 4 * (lane & 7);  // nibble group and first byte of this lane's word inside it
  for (int r = warp; r < kRowsPerCta; r += 8) {
    const int n = n0 + r;
    if (n >= N) break;
    const uint8_t* row = wbase + static_cast<size_t>(n) * row_bytes;
    float acc = 0.f;
    for (int sb = 0; sb < nsb; sb++) {
      const uint8_t* blk = row + static_cast<size_t>(sb) * UB_Q4K_BYTES;
      const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));  // d, dmin, 12 scale bytes (same for all lanes)
      const uint32_t qw = __ldg(reinterpret_cast<const uint32_t*>(blk + 16) + lane);  // bytes 32 G + pos .. + 3
      uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
      q4k_unpack_scales(hdr.y, hdr.z, hdr.w, sc_lo, sc_hi, mn_lo, mn_hi);
      // sub-blocks 2G (low nibbles) and 2G+1 (high nibbles)
      const int j0 = 2 * G, j1 = 2 * G + 1;
      const uint32_t scw0 = j0 < 4 ? sc_lo : sc_hi, scw1 = j1 < 4 ? sc_lo : sc_hi;
      const uint32_t mnw0 = j0 < 4 ? mn_lo : mn_hi, mnw1 = j1 < 4 ? mn_lo : mn_hi;
      const float s0 = static_cast<float>((scw0 >> (8 * (j0 & 3))) & 0xFF), s1 = static_cast<float>((scw1 >> (8 * (j1 & 3))) & 0xFF);
      const float m0 = static_cast<float>((mnw0 >> (8 * (j0 & 3))) & 0xFF), m1 = static_cast<float>((mnw1 >> (8 * (j1 & 3))) & 0xFF);
      const float d = half_bits_to_f32(hdr.x), dmin = half_bits_to_f32(hdr.x >> 16);
      const float* x0 = xs + sb * 256 + 64 * G + pos;  // activations under the low nibbles
      const float* x1 = x0 + 32;                       // ... under the high nibbles
      float dot0 = 0.f, dot1 = 0.f, sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint32_t byte = (qw >> (8 * i)) & 0xFF;
        dot0 = fmaf(static_cast<float>(byte & 15), x0[i], dot0);
        dot1 = fmaf(static_cast<float>(byte >> 4), x1[i], dot1);
        sum0 += x0[i];
        sum1 += x1[i];
      }
      acc += d * (s0 * dot0 + s1 * dot1) - dmin * (m0 * sum0 + m1 * sum1);
    }
    acc = warp_sum(acc);
    if (lane == 0) orow[n] = from_f32<T>(acc);
  }
}

template <typename T>
int indexed_moe_q4k_launch(const void* in, const void* wq, void* out, const uint32_t* indices, int N, int K, int M,
                           int batch, int topk, int num_experts, cudaStream_t s) {
  if (batch == 0 || topk == 0 || N == 0) return ub::fail(UB_OK);
  if (!in || !wq || !out || !indices || N < 0 || K <= 0 || K % UB_QK_K || batch < 0 || topk < 0 || num_experts <= 0 ||
      (M != 1 && M != topk))
    return ub::fail(UB_ERR_INVALID_ARG);
  if (reinterpret_cast<uintptr_t>(wq) & 15) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t slots = static_cast<size_t>(batch) * topk;
  if (slots > 65535) return ub::fail(UB_ERR_TOO_LARGE);
  const size_t smem = static_cast<size_t>(K) * sizeof(float);
  if (smem > 200 * 1024) return ub::fail(UB_ERR_TOO_LARGE);
  auto kernel = indexed_moe_q4k_kernel<T>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) {
      ub::set_cuda_error(e);
      return ub::fail(UB_ERR_CUDA);
    }
  }
  dim3 grid((N + kRowsPerCta - 1) / kRowsPerCta, static_cast<unsigned>(slots));
  kernel<<<grid, 256, smem, s>>>(static_cast<const T*>(in), static_cast<const uint8_t*>(wq), static_cast<T*>(out),
                                 indices, N, K, M, topk, num_experts, ub::device_error_word());
  return ub::check_launch();
}

}  // namespace

extern "C" {

int ub_indexed_moe_q4k(void* out, const void* in, const void* wq, const uint32_t* indices, int N, int K, int M,
                       int batch, int topk, int num_experts, int dtype, void* stream) {
  if (dtype == UB_DTYPE_BF16)
    return indexed_moe_q4k_launch<__nv_bfloat16>(in, wq, out, indices, N, K, M, batch, topk, num_experts,
                                                 ub::as_stream(stream));
  if (dtype == UB_DTYPE_F16)
    return indexed_moe_q4k_launch<__half>(in, wq, out, indices, N, K, M, batch, topk, num_experts,
                                          ub::as_stream(stream));
  return ub::fail(UB_ERR_INVALID_ARG);
}

}  // extern "C"
