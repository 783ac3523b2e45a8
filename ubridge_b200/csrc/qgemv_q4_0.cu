// Decode matmul for GGUF Q4_0 weights, one to four tokens, rows of a multiple of 2048 values:
//
//   y[M,N] = x[M,K] . dequant(Wq)[N,K]^T        (f32 accumulation of exact integer dots)
//
// The reference declares the block (kernels/quant.cpp:64-70: f16 d and sixteen bytes of nibbles, 18 bytes per 32
// values; value i in the low half of byte i, value 16 + i in the high half; w = d * (q - 8)) and ships no kernel for
// it.  Same structure as the Q5_K and Q6_K kernels (qgemv_q5k.cu, q6k.cu): a CTA (two per SM, eight warps) owns a
// contiguous, balanced range of rows and walks it in stages of up to sixteen rows = ONE bulk copy (cp.async.bulk,
// mbarrier ring, programmatic dependent launch with the first stage requested ahead of the dependency wait); warp
// w takes rows w and w + 8 of a stage of sixteen (the two rows share every read of the activation limbs, which at 2
// bytes per value against 0.56 of the weights are most of what the shared-memory pipe moves), a lane one block of
// each per step.  Blocks are 18 bytes apart, so the even ones start on a
// 4-byte boundary and the odd ones two bytes later: a step takes blocks of one parity in all lanes (2 lane + p),
// five aligned words each, and the nibble words are a funnel shift (even) or the words themselves (odd).  The
// nibbles are unsigned bytes and meet 15-bit block-fixed-point activations (q = 254 hi + lo, one scale per 256
// values, quantised once per CTA into shared memory) in dp4a.u32.s32; the -8 goes against the sum of the block's
// activations, stored beside their limbs; one float conversion per block.
#include <string.h>

#include "common.cuh"

#define UB_Q4_0_BYTES 18

namespace {

using namespace ub;

constexpr int kW = 8;          // warps per CTA
constexpr int kR = 2;          // rows per warp and stage: the two rows share every read of the activation limbs
constexpr int kRows = kW * kR; // rows per stage
constexpr int kMaxStages = 4;
constexpr uint32_t kSpin = 400000;
constexpr float kXQMax = 32258.f;                // 127 * 254
constexpr size_t kDynBudget = 104 * 1024;        // two CTAs per SM
constexpr size_t kDynBudgetOne = 222 * 1024;     // one CTA per SM

__device__ __forceinline__ bool mb_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mb_wait(uint32_t bar, uint32_t parity) {
  if (mb_try(bar, parity)) return true;
  for (uint32_t i = 0; i < kSpin; i++) {
    if (mb_try(bar, parity)) return true;
    if (i >= 2) __nanosleep(40);
  }
  return false;
}
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
__device__ __forceinline__ int dp4a_us(uint32_t a_u8x4, uint32_t b_s8x4, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
  return d;
}
// eight values from x + k (k a multiple of 8)
__device__ __forceinline__ void load8(const float* x, int k, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(x + k)), b = __ldg(reinterpret_cast<const float4*>(x + k) + 1);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* x, int k, float (&v)[8]) {
  const uint4 q = __ldg(reinterpret_cast<const uint4*>(x + k));
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; i++) v[2 * i] = __uint_as_float(w[i] << 16), v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
}

// Activations of one block of 32 values: limb words 0-3 = values 0-15 (the low nibbles' partners), 4-7 = 16-31.
struct XSlot {
  uint4 hi[2], lo[2];  // the limbs
  int sum;             // sum of q over the block
  int pad[3];
};

// MT: token slots (1, 2 or 4; only the fourth can be empty).
template <typename XT, int MT>
__global__ void __launch_bounds__(kW * 32, 2)
qgemv_q4_0_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x, void* __restrict__ y, int y_dtype, int M, int N,
                 int K, int S, int early, int* err_word) {
  extern __shared__ __align__(128) unsigned char q40_smem[];
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages];  // full[S], empty[S]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nsb = K / UB_QK_K, nb = K / 32;
  const uint32_t row_bytes = static_cast<uint32_t>(nb) * UB_Q4_0_BYTES, stage_bytes = kRows * row_bytes;
  unsigned char* const ring = q40_smem;
  XSlot* const xq = reinterpret_cast<XSlot*>(q40_smem + static_cast<size_t>(S) * stage_bytes);  // [MT][K / 32]
  float* const xsc = reinterpret_cast<float*>(xq + MT * nb);                                     // [MT][nsb]
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  // rows of this CTA
  const int base = N / static_cast<int>(gridDim.x), extra = N % static_cast<int>(gridDim.x);
  const int bx = static_cast<int>(blockIdx.x);
  const int r0 = bx * base + (bx < extra ? bx : extra), nrows = base + (bx < extra ? 1 : 0);
  const int nst = (nrows + kRows - 1) / kRows;

  // The next kernel in the stream may start as soon as every CTA of this grid has passed this point.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars_s + 8 * s), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars_s + 8 * (kMaxStages + s)), "r"(kW) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // stage n of this CTA = rows r0 + 8 n .. of the range -> ring slot n % S, one bulk copy
  auto issue = [&](int n) {
    const int rows = min(kRows, nrows - kRows * n);
    const uint32_t bytes = static_cast<uint32_t>(rows) * row_bytes, full = bars_s + 8 * (n % S);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     ring_s + (n % S) * stage_bytes),
                 "l"(wq + static_cast<size_t>(r0 + kRows * n) * row_bytes), "r"(bytes), "r"(full)
                 : "memory");
  };
  const int n_early = min(min(early, S), nst);
  if (threadIdx.x == 0)
    for (int n = 0; n < n_early; n++) issue(n);

  // everything below reads what the previous kernel may have written (x) or writes what it may still read (y)
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- activations -> 15-bit block fixed point in shared memory: a thread quantises one block of 32 values, the
  // eight threads of a 256-value run share its scale ----
  for (int b0 = 0; b0 < M * nb; b0 += kW * 32) {
    // whole warps are inside or outside (K / 32 is a multiple of 64); tok: the token, b: the block of its row
    const int gb = b0 + threadIdx.x, tok = gb / nb, b = gb - tok * nb;
    float v[4][8];
    if (gb < M * nb) {
#pragma unroll
      for (int u = 0; u < 4; u++) load8(x + static_cast<size_t>(tok) * K, 32 * b + 8 * u, v[u]);
    }
    if (b0 == 0 && threadIdx.x == 0)  // the rest of the ring goes out right behind the activation loads
      for (int n = n_early; n < min(S, nst); n++) issue(n);
    if (gb < M * nb) {
      float amax = 0.f;
#pragma unroll
      for (int u = 0; u < 4; u++)
#pragma unroll
        for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[u][e]));
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));  // 256 values
      const float inv = amax > 0.f ? kXQMax / amax : 0.f, inv254 = inv * (1.f / 254.f);
      uint32_t wh[8], wl[8];
      int sum = 0;
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int hi[8], lo[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {  // rounding through the mantissa of 1.5 * 2^23; |lo| <= 127 either way
          const int q = __float_as_int(fmaf(v[u][e], inv, 12582912.f)) - 0x4B400000;
          hi[e] = __float_as_int(fmaf(v[u][e], inv254, 12582912.f)) - 0x4B400000;
          lo[e] = q - 254 * hi[e];
          sum += q;
        }
        wh[2 * u] = pack4(hi[0], hi[1], hi[2], hi[3]), wh[2 * u + 1] = pack4(hi[4], hi[5], hi[6], hi[7]);
        wl[2 * u] = pack4(lo[0], lo[1], lo[2], lo[3]), wl[2 * u + 1] = pack4(lo[4], lo[5], lo[6], lo[7]);
      }
      XSlot s;
      s.hi[0] = make_uint4(wh[0], wh[1], wh[2], wh[3]), s.hi[1] = make_uint4(wh[4], wh[5], wh[6], wh[7]);
      s.lo[0] = make_uint4(wl[0], wl[1], wl[2], wl[3]), s.lo[1] = make_uint4(wl[4], wl[5], wl[6], wl[7]);
      s.sum = sum, s.pad[0] = s.pad[1] = s.pad[2] = 0;
      xq[gb] = s;
      if ((b & 7) == 0) xsc[tok * nsb + (b >> 3)] = amax * (1.f / kXQMax);
    }
  }
  __syncthreads();

  bool ok = true;
  int slot = 0, round = 0;
#pragma unroll 1
  for (int n = 0; n < nst; n++) {
    if (ok) ok = mb_wait(bars_s + 8 * slot, round & 1);
    const int rows = min(kRows, nrows - kRows * n);
    float acc[kR][MT];
#pragma unroll
    for (int r = 0; r < kR; r++)
#pragma unroll
      for (int m = 0; m < MT; m++) acc[r][m] = 0.f;
    if (warp < rows) {
      const bool two = warp + kW < rows;  // the warp's second row (row warp + 8 of the stage) exists
      const unsigned char* rowp = ring + static_cast<size_t>(slot) * stage_bytes + static_cast<size_t>(warp) * row_bytes;
#pragma unroll
      for (int par = 0; par < 2; par++)
#pragma unroll 2
        for (int b = 2 * lane + par; b < nb; b += 64) {
          // even block: starts on a word, d in its low half, the nibbles from its high half on; odd block: starts two
          // bytes into a word, d in that word's high half, the nibbles in the four words that follow
          uint32_t lo4[kR][4], hi4[kR][4];
          float d[kR];
#pragma unroll
          for (int r = 0; r < kR; r++) {
            if (r == 0 || two) {
              const uint32_t* al = reinterpret_cast<const uint32_t*>(rowp + static_cast<size_t>(r) * kW * row_bytes +
                                                                     b * UB_Q4_0_BYTES - 2 * par);
              const uint32_t w0 = al[0], w1 = al[1], w2 = al[2], w3 = al[3], w4 = al[4];
              d[r] = half_bits_to_f32(par ? w0 >> 16 : w0);
              const uint32_t q0 = par ? w1 : __funnelshift_r(w0, w1, 16), q1 = par ? w2 : __funnelshift_r(w1, w2, 16);
              const uint32_t q2 = par ? w3 : __funnelshift_r(w2, w3, 16), q3 = par ? w4 : __funnelshift_r(w3, w4, 16);
              lo4[r][0] = q0 & 0x0F0F0F0Fu, lo4[r][1] = q1 & 0x0F0F0F0Fu, lo4[r][2] = q2 & 0x0F0F0F0Fu, lo4[r][3] = q3 & 0x0F0F0F0Fu;
              hi4[r][0] = (q0 >> 4) & 0x0F0F0F0Fu, hi4[r][1] = (q1 >> 4) & 0x0F0F0F0Fu;
              hi4[r][2] = (q2 >> 4) & 0x0F0F0F0Fu, hi4[r][3] = (q3 >> 4) & 0x0F0F0F0Fu;
            } else {
              d[r] = 0.f;
#pragma unroll
              for (int i = 0; i < 4; i++) lo4[r][i] = hi4[r][i] = 0;
            }
          }
#pragma unroll
          for (int m = 0; m < MT; m++) {
            if (m < 3 || M > 3) {  // only the fourth slot can be empty (one, two or four slots for M = 1, 2, 3-4)
              const XSlot& xs = xq[m * nb + b];
              const uint4 xa = xs.hi[0], xb = xs.hi[1], ya = xs.lo[0], yb = xs.lo[1];
              const int s8 = 8 * xs.sum;
              const float xsv = xsc[m * nsb + (b >> 3)];
#pragma unroll
              for (int r = 0; r < kR; r++) {
                const int H = dp4a_us(hi4[r][3], xb.w, dp4a_us(hi4[r][2], xb.z, dp4a_us(hi4[r][1], xb.y, dp4a_us(hi4[r][0], xb.x,
                              dp4a_us(lo4[r][3], xa.w, dp4a_us(lo4[r][2], xa.z, dp4a_us(lo4[r][1], xa.y, dp4a_us(lo4[r][0], xa.x, 0))))))));
                const int L = dp4a_us(hi4[r][3], yb.w, dp4a_us(hi4[r][2], yb.z, dp4a_us(hi4[r][1], yb.y, dp4a_us(hi4[r][0], yb.x,
                              dp4a_us(lo4[r][3], ya.w, dp4a_us(lo4[r][2], ya.z, dp4a_us(lo4[r][1], ya.y, dp4a_us(lo4[r][0], ya.x, 0))))))));
                // sum (q - 8) xq = 254 H + L - 8 sum(xq): < 2^25
                const int t = 254 * H + L - s8;
                acc[r][m] = fmaf(static_cast<float>(t), d[r] * xsv, acc[r][m]);
              }
            }
          }
        }
    }
    // everything this warp needs from the stage has been read: hand the slot back
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bars_s + 8 * (kMaxStages + slot)) : "memory");
    if ((n & (kW - 1)) == warp && n + S < nst) {
      if (ok) ok = mb_wait(bars_s + 8 * (kMaxStages + slot), round & 1);
      if (ok && lane == 0) issue(n + S);
    }
#pragma unroll
    for (int r = 0; r < kR; r++) {
      if (warp + kW * r < rows) {
#pragma unroll
        for (int m = 0; m < MT; m++) {
          float v = acc[r][m];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
          if (lane == 0 && (m < 3 || M > 3)) {
            const size_t at = static_cast<size_t>(m) * N + static_cast<size_t>(r0 + kRows * n + warp + kW * r);
            if (y_dtype == UB_DTYPE_F32) static_cast<float*>(y)[at] = v;
            else if (y_dtype == UB_DTYPE_BF16) static_cast<__nv_bfloat16*>(y)[at] = __float2bfloat16_rn(v);
            else static_cast<__half*>(y)[at] = __float2half_rn(v);
          }
        }
      }
    }
    if (++slot == S) slot = 0, round++;
  }
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

template <typename XT, int MT>
int launch_q4_0(const uint8_t* w, const XT* x, void* y, int M, int N, int K, int out_dtype, bool fresh, cudaStream_t s) {
  const size_t row_bytes = static_cast<size_t>(K / 32) * UB_Q4_0_BYTES, stage_bytes = kRows * row_bytes;
  const size_t xbytes = MT * (static_cast<size_t>(K / 32) * sizeof(XSlot) + static_cast<size_t>(K / UB_QK_K) * 4);
  int ctas = 2;
  int S = xbytes + 2 * stage_bytes <= kDynBudget ? static_cast<int>((kDynBudget - xbytes) / stage_bytes) : 0;
  if (S < 2) {
    ctas = 1;
    S = xbytes + 2 * stage_bytes <= kDynBudgetOne ? static_cast<int>((kDynBudgetOne - xbytes) / stage_bytes) : 0;
  }
  if (S > kMaxStages) S = kMaxStages;
  if (S < 2) return UB_ERR_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(S) * stage_bytes + xbytes;
  auto kernel = qgemv_q4_0_kernel<XT, MT>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  const int slots = ctas * ub::num_sms(), want = (N + kRows - 1) / kRows;
  const int grid = want < slots ? want : slots;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kW * 32), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, w, x, y, out_dtype, M, N, K, S, fresh ? 0 : 1, ub::device_error_word());
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::check_launch();
}

}  // namespace

namespace ub {

// y[M,N] = x[M,K] . dequant(Wq)^T for one to four tokens of Q4_0; UB_ERR_UNSUPPORTED (without touching the thread's
// status) for what this kernel does not take: other M, K not a multiple of 2048 or too long for two stages beside
// the tokens' limbs, weights or activations that are not 16-byte aligned.
// fresh: the weight bytes may have been written by the kernel launched just before on the same stream.
template <typename XT>
int q4_0_gemv_staged(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  if (M < 1 || M > 4 || K % 2048 || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15))
    return UB_ERR_UNSUPPORTED;
  if (M == 1) return launch_q4_0<XT, 1>(w, x, y, M, N, K, y_dtype, fresh, s);
  if (M == 2) return launch_q4_0<XT, 2>(w, x, y, M, N, K, y_dtype, fresh, s);
  return launch_q4_0<XT, 4>(w, x, y, M, N, K, y_dtype, fresh, s);
}

template int q4_0_gemv_staged<float>(const void*, const float*, void*, int, int, int, int, bool, cudaStream_t);
template int q4_0_gemv_staged<__nv_bfloat16>(const void*, const __nv_bfloat16*, void*, int, int, int, int, bool,
                                            cudaStream_t);

}  // namespace ub
