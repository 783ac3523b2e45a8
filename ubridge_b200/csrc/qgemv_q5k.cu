// Decode matmul for GGUF Q5_K weights, one to four tokens, rows of a multiple of 2048 values:
//
//   y[M,N] = x[M,K] . dequant(Wq)[N,K]^T        (f32 accumulation of exact integer dots)
//
// The reference declares the block (kernels/quant.cpp:152-160: f16 d, f16 dmin, twelve bytes of 6-bit scales and
// mins as in Q4_K, qh[32] with the fifth bit of every value, qs[128] with the nibbles; 176 bytes per 256 values) and
// ships no kernel for it.  Element l of sub-block j: q = nibble (low half of qs[32 (j / 2) + l] for even j, high
// half for odd j) + 16 * bit j of qh[l];  w = d * sc[j] * q - dmin * m[j].
//
// Same structure as the Q6_K kernel of q6k.cu: a CTA (two per SM, eight warps) owns a contiguous, balanced range of
// rows and walks it in stages of up to eight rows = ONE bulk copy (cp.async.bulk, mbarrier ring, programmatic
// dependent launch with the first stage requested ahead of the dependency wait); warp w takes row w of the stage,
// two super-blocks per step (16 lanes each).  A lane owns the 64-value group g = lane / 4 % 4 and there eight
// neighbouring l: eight bytes of qs, eight of qh (blocks are 16-byte aligned: every load is an aligned one), i.e.
// eight values of sub-block 2g and eight of 2g + 1.  The values are unsigned bytes (nibble | bit << 4) and meet
// 15-bit block-fixed-point activations (q = 254 hi + lo, quantised once per CTA into shared memory) in
// dp4a.u32.s32; 6-bit scales and mins in integer arithmetic (the mins against the sums of the lane's activations,
// stored beside their limbs), one float conversion per limb and super-block.  (Measured on B200, 14336 x 4096, one
// token: 13.1 us.  Two rows per warp sharing the activation reads, which took the Q4_0 kernel from 13.4 to 9.7 us,
// make this one slower, 13.5 us: its stages are then 45 KB and only two fit.)
#include <string.h>

#include "common.cuh"

#define UB_Q5K_BYTES 176

namespace {

using namespace ub;

constexpr int kW = 8;  // warps per CTA = rows per stage
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

// Activation slot of a lane: 16 values = eight of sub-block 2g (words 0, 1) and eight of 2g + 1 (words 2, 3).
struct XSlot {
  uint4 hi, lo;   // the limbs
  int sum[2];     // sums of q over the eight values of either sub-block
  int pad[2];
};

// MT: token slots (1, 2 or 4; only the fourth can be empty).
template <typename XT, int MT>
__global__ void __launch_bounds__(kW * 32, 2)
qgemv_q5k_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x, void* __restrict__ y, int y_dtype, int M, int N,
                 int K, int S, int early, int* err_word) {
  extern __shared__ __align__(128) unsigned char q5_smem[];
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages];  // full[S], empty[S]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nsb = K / UB_QK_K;
  const uint32_t row_bytes = static_cast<uint32_t>(nsb) * UB_Q5K_BYTES, stage_bytes = kW * row_bytes;
  unsigned char* const ring = q5_smem;
  XSlot* const xq = reinterpret_cast<XSlot*>(q5_smem + static_cast<size_t>(S) * stage_bytes);  // [MT][K / 16]
  float* const xsc = reinterpret_cast<float*>(xq + MT * (K / 16));                              // [MT][nsb]
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  // rows of this CTA
  const int base = N / static_cast<int>(gridDim.x), extra = N % static_cast<int>(gridDim.x);
  const int bx = static_cast<int>(blockIdx.x);
  const int r0 = bx * base + (bx < extra ? bx : extra), nrows = base + (bx < extra ? 1 : 0);
  const int nst = (nrows + kW - 1) / kW;

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
    const int rows = min(kW, nrows - kW * n);
    const uint32_t bytes = static_cast<uint32_t>(rows) * row_bytes, full = bars_s + 8 * (n % S);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     ring_s + (n % S) * stage_bytes),
                 "l"(wq + static_cast<size_t>(r0 + kW * n) * row_bytes), "r"(bytes), "r"(full)
                 : "memory");
  };
  const int n_early = min(min(early, S), nst);
  if (threadIdx.x == 0)
    for (int n = 0; n < n_early; n++) issue(n);

  // everything below reads what the previous kernel may have written (x) or writes what it may still read (y)
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- activations -> 15-bit block fixed point in shared memory.  A thread quantises the slot of one lane:
  // slot = 16 sb + 4 g + l / 8 holds values 256 sb + 64 g + l .. l + 7 and 256 sb + 64 g + 32 + l .. l + 7 ----
  for (int slot0 = 0; slot0 < M * (K / 16); slot0 += kW * 32) {
    // whole warps are inside or outside (K / 16 is a multiple of 128); tok: the token, slot: inside its row
    const int gslot = slot0 + threadIdx.x, tok = gslot / (K / 16), slot = gslot - tok * (K / 16);
    float v[2][8];
    if (gslot < M * (K / 16)) {
      const int k0 = (slot >> 4) * UB_QK_K + ((slot >> 2) & 3) * 64 + (slot & 3) * 8;
      load8(x + static_cast<size_t>(tok) * K, k0, v[0]);
      load8(x + static_cast<size_t>(tok) * K, k0 + 32, v[1]);
    }
    if (slot0 == 0 && threadIdx.x == 0)  // the rest of the ring goes out right behind the activation loads
      for (int n = n_early; n < min(S, nst); n++) issue(n);
    if (gslot < M * (K / 16)) {
      float amax = 0.f;
#pragma unroll
      for (int u = 0; u < 2; u++)
#pragma unroll
        for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[u][e]));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));  // the super-block
      const float inv = amax > 0.f ? kXQMax / amax : 0.f, inv254 = inv * (1.f / 254.f);
      uint32_t wh[4], wl[4];
      int sum[2];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        int hi[8], lo[8];
        sum[u] = 0;
#pragma unroll
        for (int e = 0; e < 8; e++) {  // rounding through the mantissa of 1.5 * 2^23; |lo| <= 127 either way
          const int q = __float_as_int(fmaf(v[u][e], inv, 12582912.f)) - 0x4B400000;
          hi[e] = __float_as_int(fmaf(v[u][e], inv254, 12582912.f)) - 0x4B400000;
          lo[e] = q - 254 * hi[e];
          sum[u] += q;
        }
        wh[2 * u] = pack4(hi[0], hi[1], hi[2], hi[3]), wh[2 * u + 1] = pack4(hi[4], hi[5], hi[6], hi[7]);
        wl[2 * u] = pack4(lo[0], lo[1], lo[2], lo[3]), wl[2 * u + 1] = pack4(lo[4], lo[5], lo[6], lo[7]);
      }
      XSlot s;
      s.hi = make_uint4(wh[0], wh[1], wh[2], wh[3]);
      s.lo = make_uint4(wl[0], wl[1], wl[2], wl[3]);
      s.sum[0] = sum[0], s.sum[1] = sum[1], s.pad[0] = s.pad[1] = 0;
      xq[gslot] = s;
      if ((slot & 15) == 0) xsc[tok * nsb + (slot >> 4)] = amax * (1.f / kXQMax);
    }
  }
  __syncthreads();

  const int sub = lane >> 4, g = (lane >> 2) & 3, lq = lane & 3;
  bool ok = true;
  int slot = 0, round = 0;
#pragma unroll 1
  for (int n = 0; n < nst; n++) {
    if (ok) ok = mb_wait(bars_s + 8 * slot, round & 1);
    const int rows = min(kW, nrows - kW * n);
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.f;
    if (warp < rows) {
      const unsigned char* rowp = ring + static_cast<size_t>(slot) * stage_bytes + static_cast<size_t>(warp) * row_bytes;
#pragma unroll 2
      for (int sb = sub; sb < nsb; sb += 2) {
        const unsigned char* blk = rowp + sb * UB_Q5K_BYTES;
        const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
        const uint2 qh = *reinterpret_cast<const uint2*>(blk + 16 + 8 * lq);
        const uint2 qs = *reinterpret_cast<const uint2*>(blk + 48 + 32 * g + 8 * lq);
        // unsigned bytes nibble | fifth bit << 4 of sub-blocks 2g (a) and 2g + 1 (b)
        const uint32_t h0 = qh.x >> (2 * g), h1 = qh.y >> (2 * g);
        const uint32_t a0 = (qs.x & 0x0F0F0F0Fu) | ((h0 << 4) & 0x10101010u), a1 = (qs.y & 0x0F0F0F0Fu) | ((h1 << 4) & 0x10101010u);
        const uint32_t b0 = ((qs.x >> 4) & 0x0F0F0F0Fu) | ((h0 << 3) & 0x10101010u),
                       b1 = ((qs.y >> 4) & 0x0F0F0F0Fu) | ((h1 << 3) & 0x10101010u);
        // 6-bit scales and mins of sub-blocks 2g, 2g + 1: bytes 2 (g & 1), 2 (g & 1) + 1 of word g / 2
        uint32_t scw[2], mnw[2];
        q4k_unpack_scales(hdr.y, hdr.z, hdr.w, scw[0], scw[1], mnw[0], mnw[1]);
        const uint32_t sp = (g >> 1 ? scw[1] : scw[0]) >> (16 * (g & 1)), mp = (g >> 1 ? mnw[1] : mnw[0]) >> (16 * (g & 1));
        const int sa = sp & 0xFF, sb_ = (sp >> 8) & 0xFF, ma = mp & 0xFF, mb = (mp >> 8) & 0xFF;
        const float d = half_bits_to_f32(hdr.x), dmin = half_bits_to_f32(hdr.x >> 16);
#pragma unroll
        for (int m = 0; m < MT; m++) {
          if (m < 3 || M > 3) {  // only the fourth slot can be empty (one, two or four slots for M = 1, 2, 3-4)
            const XSlot& xs = xq[m * (K / 16) + 16 * sb + 4 * g + lq];
            const uint4 xh = xs.hi, xl = xs.lo;
            const int2 sm = *reinterpret_cast<const int2*>(xs.sum);
            // scales meet the limb dots in integers (|scale * dot| < 2^25), one conversion per limb
            const int H = sa * dp4a_us(a1, xh.y, dp4a_us(a0, xh.x, 0)) + sb_ * dp4a_us(b1, xh.w, dp4a_us(b0, xh.z, 0));
            const int L = sa * dp4a_us(a1, xl.y, dp4a_us(a0, xl.x, 0)) + sb_ * dp4a_us(b1, xl.w, dp4a_us(b0, xl.z, 0));
            const int T = ma * sm.x + mb * sm.y;
            const float xsv = xsc[m * nsb + sb];
            const float f = fmaf(static_cast<float>(H), 254.f, static_cast<float>(L));
            acc[m] = fmaf(f, d * xsv, acc[m]);
            acc[m] = fmaf(-static_cast<float>(T), dmin * xsv, acc[m]);
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
    if (warp < rows) {
#pragma unroll
      for (int m = 0; m < MT; m++) {
        float v = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if (lane == 0 && (m < 3 || M > 3)) {
          const size_t at = static_cast<size_t>(m) * N + static_cast<size_t>(r0 + kW * n + warp);
          if (y_dtype == UB_DTYPE_F32) static_cast<float*>(y)[at] = v;
          else if (y_dtype == UB_DTYPE_BF16) static_cast<__nv_bfloat16*>(y)[at] = __float2bfloat16_rn(v);
          else static_cast<__half*>(y)[at] = __float2half_rn(v);
        }
      }
    }
    if (++slot == S) slot = 0, round++;
  }
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

template <typename XT, int MT>
int launch_q5k(const uint8_t* w, const XT* x, void* y, int M, int N, int K, int out_dtype, bool fresh, cudaStream_t s) {
  const size_t row_bytes = static_cast<size_t>(K / UB_QK_K) * UB_Q5K_BYTES, stage_bytes = kW * row_bytes;
  const size_t xbytes = MT * (static_cast<size_t>(K / 16) * sizeof(XSlot) + static_cast<size_t>(K / UB_QK_K) * 4);
  int ctas = 2;
  int S = xbytes + 2 * stage_bytes <= kDynBudget ? static_cast<int>((kDynBudget - xbytes) / stage_bytes) : 0;
  if (S < 2) {
    ctas = 1;
    S = xbytes + 2 * stage_bytes <= kDynBudgetOne ? static_cast<int>((kDynBudgetOne - xbytes) / stage_bytes) : 0;
  }
  if (S > kMaxStages) S = kMaxStages;
  if (S < 2) return UB_ERR_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(S) * stage_bytes + xbytes;
  auto kernel = qgemv_q5k_kernel<XT, MT>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  const int slots = ctas * ub::num_sms(), want = (N + kW - 1) / kW;
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

// y[M,N] = x[M,K] . dequant(Wq)^T for one to four tokens of Q5_K; UB_ERR_UNSUPPORTED (without touching the thread's
// status) for what this kernel does not take: other M, K not a multiple of 2048 or too long for two stages beside
// the tokens' limbs, weights or activations that are not 16-byte aligned.
// fresh: the weight bytes may have been written by the kernel launched just before on the same stream.
template <typename XT>
int q5k_gemv_staged(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  if (M < 1 || M > 4 || K % 2048 || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15))
    return UB_ERR_UNSUPPORTED;
  if (M == 1) return launch_q5k<XT, 1>(w, x, y, M, N, K, y_dtype, fresh, s);
  if (M == 2) return launch_q5k<XT, 2>(w, x, y, M, N, K, y_dtype, fresh, s);
  return launch_q5k<XT, 4>(w, x, y, M, N, K, y_dtype, fresh, s);
}

template int q5k_gemv_staged<float>(const void*, const float*, void*, int, int, int, int, bool, cudaStream_t);
template int q5k_gemv_staged<__nv_bfloat16>(const void*, const __nv_bfloat16*, void*, int, int, int, int, bool,
                                            cudaStream_t);

}  // namespace ub
