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


// ------------------------------------------------------------------ streaming decode kernels
// Second generation of the decode kernels, used whenever the activations fit in shared memory.
//
// A warp owns 8 consecutive weight rows; lane (g,t) = (lane>>2, lane&3) owns row g and every fourth
// super-block (Q4_K) / run of eight Q8_0 blocks of that row, so the four lanes of a row read
// consecutive 144-byte (272-byte) pieces.  Each lane copies its pieces global -> shared memory with
// 16-byte asynchronous copies into a private slot of a per-warp ring (two pieces in flight ahead of the
// one being consumed), so the depth of the memory pipeline does not depend on registers or on how the
// compiler schedules loads.  A lane's slot is 144 bytes: slot stride 36 words makes the 128-bit reads of
// eight neighbouring lanes fall into disjoint banks.  Activations sit in shared memory as f32 with four
// floats of padding per 256, so the four super-blocks a warp touches at once are in different banks and
// every activation load is a conflict-free four-address broadcast.  Products use the packed f32x2 FMA of
// sm_100 (two weights per issue slot).  One CTA per SM; its warps take 8-row tiles round-robin over the
// whole grid, which spreads the N/8 tiles over the SMs to within one tile.
constexpr int kStreamMaxWarps = 16;
constexpr int kStages = 3;
constexpr int kXPad = 260;  // floats per super-block of activations in shared memory

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

// float(2048 + nibble) for byte I of a word masked with 0xF0F0F0F0 (the nibble sits in the byte's high half)
template <int I>
__device__ __forceinline__ float nib_hi_biased(uint32_t w4) {
  return __uint_as_float(__byte_perm(w4, 0x45000000u, 0x7404u | (I << 4)));
}

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory");
}

// x[MT][K] -> shared f32 [MT][K/256][kXPad]
template <typename XT, int MT>
__device__ __forceinline__ void stage_x_padded(float* xs, const XT* __restrict__ x, int K, int kpad) {
  for (int i = threadIdx.x * 8; i < MT * K; i += blockDim.x * 8) {
    const int m = i / K, k = i - m * K;
    float v[8];
    load_x8<XT>(x + i, v);
    float* dst = xs + m * kpad + (k >> 8) * kXPad + (k & 255);
    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

// One super-block (nine 16-byte words at `blk` in shared memory) against MT activation rows.
// xs: this super-block's activations of row 0 (row stride kpad); sx: its eight 32-value sums (row stride nsx).
template <int MT>
__device__ __forceinline__ void dot_q4k_smem(const uint4* blk, const float* xs, const float* sx, int kpad, int nsx,
                                             float (&acc)[MT]) {
  const uint4 h = blk[0];
  const float d = half_bits_to_f32(h.x), dmin = half_bits_to_f32(h.x >> 16);
  uint32_t scw[2], mnw[2];
  q4k_unpack_scales(h.y, h.z, h.w, scw[0], scw[1], mnw[0], mnw[1]);
#pragma unroll
  for (int G = 0; G < 4; G++) {
    const int sh = (G & 1) * 16;
    const float d1 = d * static_cast<float>((scw[G >> 1] >> sh) & 0xFF);
    const float m1 = dmin * static_cast<float>((mnw[G >> 1] >> sh) & 0xFF);
    const float d2 = d * static_cast<float>((scw[G >> 1] >> (sh + 8)) & 0xFF);
    const float m2 = dmin * static_cast<float>((mnw[G >> 1] >> (sh + 8)) & 0xFF);
    const float c1 = fmaf(128.f, d1, m1), c2 = fmaf(2048.f, d2, m2);
    const uint4 qa = blk[1 + 2 * G], qb = blk[2 + 2 * G];
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    float2 alo[MT], ahi[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) alo[m] = ahi[m] = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t lo = w[i] & 0x0F0F0F0Fu, hi = w[i] & 0xF0F0F0F0u;
      const float2 l01 = make_float2(nib_biased<0>(lo), nib_biased<1>(lo));
      const float2 l23 = make_float2(nib_biased<2>(lo), nib_biased<3>(lo));
      const float2 h01 = make_float2(nib_hi_biased<0>(hi), nib_hi_biased<1>(hi));
      const float2 h23 = make_float2(nib_hi_biased<2>(hi), nib_hi_biased<3>(hi));
#pragma unroll
      for (int m = 0; m < MT; m++) {
        const float4 xl = *reinterpret_cast<const float4*>(xs + m * kpad + 64 * G + 4 * i);
        const float4 xh = *reinterpret_cast<const float4*>(xs + m * kpad + 64 * G + 32 + 4 * i);
        alo[m] = ffma2(l01, make_float2(xl.x, xl.y), alo[m]);
        alo[m] = ffma2(l23, make_float2(xl.z, xl.w), alo[m]);
        ahi[m] = ffma2(h01, make_float2(xh.x, xh.y), ahi[m]);
        ahi[m] = ffma2(h23, make_float2(xh.z, xh.w), ahi[m]);
      }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
      const float sl = sx[m * nsx + 2 * G], sh2 = sx[m * nsx + 2 * G + 1];
      acc[m] += fmaf(d1, alo[m].x + alo[m].y, -c1 * sl) + fmaf(d2, ahi[m].x + ahi[m].y, -c2 * sh2);
    }
  }
}

template <typename XT, int MT>
__global__ void __launch_bounds__(kStreamMaxWarps * 32, 1)
qgemv_q4k_stream_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x, void* __restrict__ y, int N, int K,
                        int y_dtype) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int nsb = K >> 8;
  const int kpad = nsb * kXPad, nsx = K >> 5;
  float* xs = reinterpret_cast<float*>(smem_raw);          // [MT][kpad]
  float* sx = xs + MT * kpad;                               // [MT][K/32]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  unsigned char* ring = smem_raw + ((static_cast<size_t>(MT) * (kpad + nsx) * 4 + 15) & ~static_cast<size_t>(15));
  unsigned char* my_ring = ring + (static_cast<size_t>(warp) * kStages * 32 + lane) * UB_Q4K_BYTES;  // + stage*32*144
  const uint32_t my_ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(my_ring));
  const size_t row_bytes = static_cast<size_t>(nsb) * UB_Q4K_BYTES;
  const int ntiles = (N + 7) >> 3;
  const int P = (nsb + 3) >> 2;                       // pieces per tile per lane (some may be empty)
  const int tile0 = blockIdx.x + gridDim.x * warp, tile_step = gridDim.x * nwarps;
  const int my_tiles = tile0 < ntiles ? (ntiles - tile0 + tile_step - 1) / tile_step : 0;
  const int Q = my_tiles * P;                         // pieces this lane walks through

  auto issue = [&](int q) {
    if (q < Q) {
      const int ti = q / P, p = q - ti * P;
      const int n = (tile0 + ti * tile_step) * 8 + g, sb = t + 4 * p;
      if (n < N && sb < nsb) {
        const uint8_t* src = wq + static_cast<size_t>(n) * row_bytes + static_cast<size_t>(sb) * UB_Q4K_BYTES;
        const uint32_t dst = my_ring_s + (q % kStages) * (32 * UB_Q4K_BYTES);
#pragma unroll
        for (int i = 0; i < 9; i++) cp_async16(dst + 16 * i, src + 16 * i);
      }
    }
    cp_async_commit();
  };

  // weights first, so that they are in flight while the activations are staged
#pragma unroll
  for (int q = 0; q < kStages - 1; q++) issue(q);
  stage_x_padded<XT, MT>(xs, x, K, kpad);
  __syncthreads();
  for (int i = threadIdx.x; i < MT * nsx; i += blockDim.x) {
    const int m = i / nsx, gi = i - m * nsx;
    const float4* p4 = reinterpret_cast<const float4*>(xs + m * kpad + (gi >> 3) * kXPad + (gi & 7) * 32);
    float sacc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float4 v = p4[j];
      sacc += (v.x + v.y) + (v.z + v.w);
    }
    sx[i] = sacc;
  }
  __syncthreads();

  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m] = 0.f;
  int p = 0, ti = 0;
  for (int q = 0; q < Q; q++) {
    issue(q + kStages - 1);
    cp_async_wait<kStages - 1>();
    const int n = (tile0 + ti * tile_step) * 8 + g, sb = t + 4 * p;
    if (n < N && sb < nsb) {
      const uint4* blk = reinterpret_cast<const uint4*>(my_ring + (q % kStages) * (32 * UB_Q4K_BYTES));
      dot_q4k_smem<MT>(blk, xs + sb * kXPad, sx + sb * 8, kpad, nsx, acc);
    }
    if (++p == P) {
#pragma unroll
      for (int m = 0; m < MT; m++) {
        float v = acc[m];
        v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
        v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
        if (t == 0 && n < N) store_y(y, static_cast<size_t>(m) * N + n, y_dtype, v);
        acc[m] = 0.f;
      }
      p = 0;
      ti++;
    }
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------ M = 1: activations in registers
// The single-row decode kernel.  Measured on B200: the logic pipe (byte permutes, masks, shifts) issues
// at half the FMA rate and a 128-bit shared-memory broadcast costs two wavefronts, so both "nibble ->
// float + FMA" and "activations in shared memory" cost more issue time per weight than HBM needs to
// deliver it (0.5625 B/weight at 22 B/clk/SM).  Hence:
//
// * Activations never leave registers.  A lane owns ONE 64-value group position (k-slice) for the whole
//   kernel.  Its 64 activations are converted once to 16-bit block fixed point (per 32 values an f32
//   scale amax/32767 and integers split into a signed high and an unsigned low byte, four per register).
// * The inner product is integer: nibbles are masked to bytes (one logic op per four weights) and
//   multiplied with dp4a, two per four weights (high and low activation byte).  A 32-value sub-block sum
//   is below 2^24, exact in int32 and in its f32 conversion; the sub-block scale and min are applied once
//   per 32 weights.  The 16-bit activation grid costs about 3e-5 relative L2 error on the output.
// * K/64 lanes (K/2048 warps, a "team") cover a row; `teams` rows are in progress per CTA.
// * Weights reach the SM as bulk asynchronous copies (cp.async.bulk, the 1-D TMA path): one CTA per SM
//   owns a contiguous range of rows, i.e. one contiguous byte range, which a producer warp streams into a
//   ring of shared-memory stages (one stage = one row per team, a single copy of `teams * row_bytes`
//   bytes), completion signalled on an mbarrier per stage.  Per-lane 16-byte loads could not keep enough
//   bytes in flight (each occupies a miss slot for half a sector); bulk copies are fully coalesced, need
//   no registers and run up to the ring depth ahead of the arithmetic.  A lane reads its 48 bytes (header
//   + 32 bytes of nibbles) from the stage with three conflict-free 128-bit loads.
// * Rows are reduced eight at a time with a transposing butterfly (about four instructions per row
//   instead of ten), then across the team's warps through shared memory.
// Every mbarrier wait is bounded: on expiry the kernel records UB_ERR_TIMEOUT in the device error word,
// stops reading and runs out its loops without further waits.
template <typename K_>
inline int set_smem(K_ kernel, size_t smem);

constexpr int kTmaMaxStages = 10;
constexpr uint32_t kWaitLimit = 400000;

struct KslRaw {
  uint4 h, qa, qb;
};

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the phase did not complete within kWaitLimit polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitLimit; i++)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Transposing butterfly: 8 per-lane partials -> the total of row `jrow(lane)` in every lane.
__device__ __forceinline__ float ksl_reduce8(const float (&part)[8], int lane) {
  float v4[4], v2[2], v1;
  {
    const bool up = lane & 16;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float send = up ? part[i] : part[i + 4], keep = up ? part[i + 4] : part[i];
      v4[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 16);
    }
  }
  {
    const bool up = lane & 8;
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const float send = up ? v4[i] : v4[i + 2], keep = up ? v4[i + 2] : v4[i];
      v2[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 8);
    }
  }
  {
    const bool up = lane & 4;
    const float send = up ? v2[0] : v2[1], keep = up ? v2[1] : v2[0];
    v1 = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 4);
  }
  v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 2);
  v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 1);
  return v1;
}
__device__ __forceinline__ int ksl_jrow(int lane) {
  return ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
}

// dp4a with an unsigned first and a signed second operand (weights are unsigned nibbles, the high limb
// of an activation is signed); the all-unsigned flavour is the __dp4a intrinsic.
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// The activations of a lane as 16-bit block fixed point: per 32 values one f32 scale (amax / 32767) and
// integers n in [-32767, 32767] split into a signed high byte and an unsigned low byte, four values per
// register, in k order.  Against 4-bit weights the integer dot of a 32-value sub-block is at most
// 32 * 15 * 32767 < 2^24, so it is exact in int32 and converts exactly to f32.
struct XLimbs {
  uint32_t hi[8], lo[8];  // 32 values
  float scale;            // amax / 32767
  float sumx;             // scale * sum(n): the quantised activations' sum, for the min term
};

template <typename XT>
__device__ __forceinline__ void quantize_x32(const XT* __restrict__ xp, XLimbs& q) {
  float v[32];
#pragma unroll
  for (int c = 0; c < 4; c++) {
    float t8[8];
    load_x8<XT>(xp + 8 * c, t8);
#pragma unroll
    for (int j = 0; j < 8; j++) v[8 * c + j] = t8[j];
  }
  // amax as a tree (the chain of 32 dependent max operations would sit on the kernel's critical path)
  float m8[8];
#pragma unroll
  for (int i = 0; i < 8; i++)
    m8[i] = fmaxf(fmaxf(fabsf(v[4 * i]), fabsf(v[4 * i + 1])), fmaxf(fabsf(v[4 * i + 2]), fabsf(v[4 * i + 3])));
  const float amax = fmaxf(fmaxf(fmaxf(m8[0], m8[1]), fmaxf(m8[2], m8[3])), fmaxf(fmaxf(m8[4], m8[5]), fmaxf(m8[6], m8[7])));
  const float inv = amax > 0.f ? 32767.f / amax : 0.f;
  q.scale = amax * (1.f / 32767.f);
  int total = 0;
#pragma unroll
  for (int w = 0; w < 8; w++) {
    // round-to-nearest-even through the mantissa of 1.5 * 2^23: no float->int conversion instruction;
    // bytes are gathered with byte permutes (three per word) rather than shift/mask/or chains
    int n[4];
#pragma unroll
    for (int b = 0; b < 4; b++) {
      n[b] = __float_as_int(fmaf(v[4 * w + b], inv, 12582912.f)) - 0x4B400000;
      total += n[b];
    }
    q.hi[w] = __byte_perm(__byte_perm(n[0], n[1], 0x0051), __byte_perm(n[2], n[3], 0x0051), 0x5410);
    q.lo[w] = __byte_perm(__byte_perm(n[0], n[1], 0x0040), __byte_perm(n[2], n[3], 0x0040), 0x5410);
  }
  q.sumx = q.scale * static_cast<float>(total);
}

template <int I>
__device__ __forceinline__ float byte_to_f32(uint32_t w) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440u | I)) - 8388608.0f;
}

// One lane's 64 weights of one row (header + 32 bytes of nibbles) against its activation limbs.
__device__ __forceinline__ float dp4a_row_dot(const KslRaw& r, const XLimbs& xl, const XLimbs& xh, int sh, bool upper) {
  const float d = half_bits_to_f32(r.h.x), dmin = half_bits_to_f32(r.h.x >> 16);
  uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
  q4k_unpack_scales(r.h.y, r.h.z, r.h.w, sc_lo, sc_hi, mn_lo, mn_hi);
  const uint32_t scw = (upper ? sc_hi : sc_lo) >> sh, mnw = (upper ? mn_hi : mn_lo) >> sh;
  // 6-bit integers -> float through the mantissa of 2^23 (exact, no conversion instruction)
  const float d1 = d * byte_to_f32<0>(scw), m1 = dmin * byte_to_f32<0>(mnw);
  const float d2 = d * byte_to_f32<1>(scw), m2 = dmin * byte_to_f32<1>(mnw);
  const uint32_t w[8] = {r.qa.x, r.qa.y, r.qa.z, r.qa.w, r.qb.x, r.qb.y, r.qb.z, r.qb.w};
  int lh = 0, hh = 0;
  uint32_t ll = 0, hl = 0;
#pragma unroll
  for (int q = 0; q < 8; q++) {
    const uint32_t lo4 = w[q] & 0x0F0F0F0Fu, hi4 = (w[q] >> 4) & 0x0F0F0F0Fu;
    lh = dp4a_us(lo4, xl.hi[q], lh);
    ll = __dp4a(lo4, xl.lo[q], ll);
    hh = dp4a_us(hi4, xh.hi[q], hh);
    hl = __dp4a(hi4, xh.lo[q], hl);
  }
  const float sl = static_cast<float>(lh * 256 + static_cast<int>(ll));
  const float shv = static_cast<float>(hh * 256 + static_cast<int>(hl));
  return fmaf(d1 * xl.scale, sl, -m1 * xl.sumx) + fmaf(d2 * xh.scale, shv, -m2 * xh.sumx);
}

// MAXW = compute warps + 1 producer warp.
template <typename XT, int MAXW>
__global__ void __launch_bounds__(MAXW * 32, 1)
qgemv_q4k_tma_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x, void* __restrict__ y, int N, int K,
                     int y_dtype, int wpr, int teams, int S, int* err_word) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ float red[2][MAXW][8];
  __shared__ __align__(8) unsigned long long bars[2 * kTmaMaxStages];  // full[S], empty[S]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cw = wpr * teams;  // compute warps; warp `cw` is the producer
  const size_t row_bytes = static_cast<size_t>(K >> 8) * UB_Q4K_BYTES;
  const uint32_t stage_bytes = static_cast<uint32_t>(teams * row_bytes);
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(dyn_smem));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));

  // rows of this CTA: contiguous, near-even split of N over the grid
  const int base = N / gridDim.x, rem = N % gridDim.x;
  const int r0 = blockIdx.x * base + min(static_cast<int>(blockIdx.x), rem);
  const int nrows = base + (static_cast<int>(blockIdx.x) < rem ? 1 : 0);
  const int nst = (nrows + teams - 1) / teams;  // stages this CTA walks through

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      mbar_init(bars_s + 8 * s, 1);
      mbar_init(bars_s + 8 * (kTmaMaxStages + s), cw);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == cw) {
    // ---- producer: one lane streams the CTA's byte range, stage by stage ----
    if (lane == 0) {
      bool ok = true;
      for (int st = 0; st < nst && ok; st++) {
        const int slot = st % S, round = st / S;
        if (round > 0) ok = mbar_wait(bars_s + 8 * (kTmaMaxStages + slot), (round - 1) & 1);
        if (!ok) {
          report_device_error(err_word, UB_ERR_TIMEOUT);
          break;
        }
        const int rows_here = min(teams, nrows - st * teams);
        const uint32_t bytes = static_cast<uint32_t>(rows_here * row_bytes);
        const uint32_t full = bars_s + 8 * slot;
        mbar_expect_tx(full, bytes);
        bulk_copy_g2s(ring_s + slot * stage_bytes, wq + static_cast<size_t>(r0 + st * teams) * row_bytes, bytes, full);
      }
    }
    return;
  }

  // ---- consumers ----
  const int team = warp / wpr, wit = warp - team * wpr;
  const int slot_k = wit * 32 + lane;  // 64-value group index inside the row
  const bool active = slot_k < (K >> 6);
  const int sb = slot_k >> 2, G = slot_k & 3;
  const int my_rows = team < nrows ? (nrows - team + teams - 1) / teams : 0;
  // byte offsets of this lane's header and nibbles inside a stage
  const uint32_t hdr_off = static_cast<uint32_t>(team * row_bytes + (active ? sb * UB_Q4K_BYTES : 0));
  const uint32_t q_off = hdr_off + 16 + (active ? 32 * G : 0);

  XLimbs xl, xh;  // values [64*slot_k, +32) pair with the low nibbles, [+32, +64) with the high ones
  quantize_x32<XT>(x + (active ? 64 * slot_k : 0), xl);
  quantize_x32<XT>(x + (active ? 64 * slot_k + 32 : 0), xh);
  const int sh = (G & 1) * 16;
  const bool upper = G >= 2;

  bool ok = true;
  const int nbatches = (nst + 7) >> 3;
  for (int b = 0; b < nbatches; b++) {
    float part[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int st = b * 8 + j;
      float res = 0.f;
      if (st < nst) {
        const int slot = st % S, round = st / S;
        if (ok) ok = mbar_wait(bars_s + 8 * slot, round & 1);
        KslRaw r;
        if (ok) {
          const unsigned char* stage = dyn_smem + static_cast<size_t>(slot) * stage_bytes;
          r.h = *reinterpret_cast<const uint4*>(stage + hdr_off);
          r.qa = *reinterpret_cast<const uint4*>(stage + q_off);
          r.qb = *reinterpret_cast<const uint4*>(stage + q_off + 16);
        } else {
          r.h = r.qa = r.qb = make_uint4(0, 0, 0, 0);
        }
        if (active && st < my_rows) res = dp4a_row_dot(r, xl, xh, sh, upper);
        // release the stage only after the loaded words have been consumed by the arithmetic above
        __syncwarp();
        if (lane == 0) mbar_arrive(bars_s + 8 * (kTmaMaxStages + slot));
      }
      part[j] = res;
    }
    const float v1 = ksl_reduce8(part, lane);
    const int par = b & 1;
    if ((lane & 3) == 0) red[par][warp][ksl_jrow(lane)] = v1;
    asm volatile("bar.sync 1, %0;" ::"r"(cw * 32) : "memory");  // compute warps only
    if (wit == 0 && lane < 8) {
      const int i = b * 8 + lane;
      if (i < my_rows) {
        float tot = 0.f;
        for (int w2 = 0; w2 < wpr; w2++) tot += red[par][warp + w2][lane];
        store_y(y, static_cast<size_t>(r0 + team + i * teams), y_dtype, tot);
      }
    }
  }
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

template <typename XT, int MT>
__device__ __forceinline__ void stage_x(float* xs, const XT* __restrict__ x, int K, int nthreads) {
  for (int i = threadIdx.x * 8; i < MT * K; i += nthreads * 8) {
    float v[8];
    load_x8<XT>(x + i, v);
    *reinterpret_cast<float4*>(xs + i) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(xs + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

// Q8_0: a piece is a run of eight blocks (272 bytes, 256 weights).  Bytes become exact floats
// (2^23 + 128 + q, minus the constant, as a packed f32x2 add) before the packed FMA.
struct Q80Raw {
  uint4 v[17];
};

__device__ __forceinline__ void load_q80(Q80Raw& r, const uint8_t* run) {
  const uint4* p = reinterpret_cast<const uint4*>(run);
#pragma unroll
  for (int i = 0; i < 17; i++) r.v[i] = __ldg(p + i);
}

template <int MT>
__device__ __forceinline__ void dot_q80_run(const Q80Raw& raw, const float* xs, int K, float (&acc)[MT]) {
  uint32_t r[69];
#pragma unroll
  for (int i = 0; i < 17; i++) {
    r[4 * i] = raw.v[i].x; r[4 * i + 1] = raw.v[i].y; r[4 * i + 2] = raw.v[i].z; r[4 * i + 3] = raw.v[i].w;
  }
  r[68] = 0;
  const float2 kBias = make_float2(-8388736.0f, -8388736.0f);  // -(2^23 + 128)
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const int off = 34 * j;
    const float d = half_bits_to_f32(__funnelshift_r(r[off >> 2], r[(off >> 2) + 1], (off & 3) * 8));
    float2 a[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) a[m] = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int qo = off + 2 + 4 * i;
      const uint32_t w = __funnelshift_r(r[qo >> 2], r[(qo >> 2) + 1], (qo & 3) * 8) ^ 0x80808080u;
      const float2 f01 = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440)),
                                                __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7441))), kBias);
      const float2 f23 = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7442)),
                                                __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7443))), kBias);
#pragma unroll
      for (int m = 0; m < MT; m++) {
        const float4 xv = *reinterpret_cast<const float4*>(xs + m * K + 32 * j + 4 * i);
        a[m] = ffma2(f01, make_float2(xv.x, xv.y), a[m]);
        a[m] = ffma2(f23, make_float2(xv.z, xv.w), a[m]);
      }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = fmaf(d, a[m].x + a[m].y, acc[m]);
  }
}

constexpr int kStreamMaxWarpsQ8 = 8;  // two 68-register pieces per lane are live: keep 255 registers available

template <typename XT, int MT>
__global__ void __launch_bounds__(kStreamMaxWarpsQ8 * 32, 1)
qgemv_q8_0_stream_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x, void* __restrict__ y, int N, int K,
                         int y_dtype) {
  extern __shared__ __align__(16) float smem[];
  float* xs = smem;  // [MT][K]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int nruns = K >> 8;
  const size_t row_bytes = static_cast<size_t>(nruns) * 272;
  const int ntiles = (N + 7) >> 3;

  int tile = blockIdx.x + gridDim.x * warp;
  Q80Raw cur;
  bool have = false;
  {
    const int n = tile * 8 + g;
    if (tile < ntiles && n < N && t < nruns) {
      load_q80(cur, wq + static_cast<size_t>(n) * row_bytes + static_cast<size_t>(t) * 272);
      have = true;
    }
  }
  stage_x<XT, MT>(xs, x, K, blockDim.x);
  __syncthreads();

  for (; tile < ntiles; tile += gridDim.x * nwarps) {
    const int n = tile * 8 + g;
    const bool row_ok = n < N;
    const uint8_t* row = wq + static_cast<size_t>(row_ok ? n : 0) * row_bytes;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.f;
    for (int run = t; run < nruns; run += 4) {
      Q80Raw nxt;
      bool have_next = false;
      if (run + 4 < nruns) {
        if (row_ok) {
          load_q80(nxt, row + static_cast<size_t>(run + 4) * 272);
          have_next = true;
        }
      } else {
        const int tile2 = tile + gridDim.x * nwarps;
        const int n2 = tile2 * 8 + g;
        if (tile2 < ntiles && n2 < N && t < nruns) {
          load_q80(nxt, wq + static_cast<size_t>(n2) * row_bytes + static_cast<size_t>(t) * 272);
          have_next = true;
        }
      }
      if (have) dot_q80_run<MT>(cur, xs + run * 256, K, acc);
      if (have_next) cur = nxt;
      have = have_next;
    }
    if (nruns <= t) have = false;
#pragma unroll
    for (int m = 0; m < MT; m++) {
      float v = acc[m];
      v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
      v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
      if (t == 0 && row_ok) store_y(y, static_cast<size_t>(m) * N + n, y_dtype, v);
    }
  }
}

constexpr size_t kStreamMaxSmem = 220 * 1024;

inline void stream_geometry(int N, int max_warps, int& grid, int& warps) {
  const int ntiles = (N + 7) / 8;
  const int sms = ub::num_sms();
  grid = ntiles < sms ? ntiles : sms;
  warps = (ntiles + grid - 1) / grid;
  if (warps > max_warps) warps = max_warps;
  if (warps < 1) warps = 1;
}

template <typename K_>
inline int set_smem(K_ kernel, size_t smem) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) {
      ub::set_cuda_error(e);
      return ub::fail(UB_ERR_CUDA);
    }
  }
  return UB_OK;
}

inline int gemv_grid(int N) {
  const int want = (N + kWarps - 1) / kWarps;
  const int cap = ub::num_sms() * 8;
  return want < cap ? (want > 0 ? want : 1) : cap;
}

template <typename XT, int MT>
int launch_q4k(const uint8_t* wq, const XT* x, void* y, int N, int K, int y_dtype, cudaStream_t s) {
  if (MT == 1) {
    const int wpr = (K / 64 + 31) / 32;
    if (wpr <= 16) {
      const int sms = ub::num_sms();
      const int grid = N < sms ? N : sms;
      const int teams = 16 / wpr;
      const int cw = wpr * teams;
      const size_t stage_bytes = static_cast<size_t>(teams) * (K / 256) * UB_Q4K_BYTES;
      int S = static_cast<int>((200 * 1024) / stage_bytes);
      if (S > kTmaMaxStages) S = kTmaMaxStages;
      if (S >= 2) {
        const size_t ring = stage_bytes * S;
        int* err = ub::device_error_word();
        if (set_smem(qgemv_q4k_tma_kernel<XT, 17>, ring) != UB_OK) return UB_ERR_CUDA;
        qgemv_q4k_tma_kernel<XT, 17><<<grid, (cw + 1) * 32, ring, s>>>(wq, x, y, N, K, y_dtype, wpr, teams, S, err);
        return ub::check_launch();
      }
    }
  }
  const size_t x_smem = ((static_cast<size_t>(MT) * ((K / 256) * kXPad + K / 32) * sizeof(float)) + 15) & ~size_t(15);
  const size_t ring_per_warp = static_cast<size_t>(kStages) * 32 * UB_Q4K_BYTES;
  if (x_smem + ring_per_warp <= kStreamMaxSmem) {
    int grid, warps;
    stream_geometry(N, kStreamMaxWarps, grid, warps);
    const int fit = static_cast<int>((kStreamMaxSmem - x_smem) / ring_per_warp);
    if (warps > fit) warps = fit;
    const size_t stream_smem = x_smem + warps * ring_per_warp;
    if (set_smem(qgemv_q4k_stream_kernel<XT, MT>, stream_smem) != UB_OK) return UB_ERR_CUDA;
    qgemv_q4k_stream_kernel<XT, MT><<<grid, warps * 32, stream_smem, s>>>(wq, x, y, N, K, y_dtype);
    return ub::check_launch();
  }
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
  const size_t stream_smem = static_cast<size_t>(MT) * K * sizeof(float);
  if (fast && stream_smem <= kStreamMaxSmem) {
    int grid, warps;
    stream_geometry(N, kStreamMaxWarpsQ8, grid, warps);
    if (set_smem(qgemv_q8_0_stream_kernel<XT, MT>, stream_smem) != UB_OK) return UB_ERR_CUDA;
    qgemv_q8_0_stream_kernel<XT, MT><<<grid, warps * 32, stream_smem, s>>>(wq, x, y, N, K, y_dtype);
    return ub::check_launch();
  }
  if (fast)
    qgemv_q8_0_kernel<XT, MT, true><<<gemv_grid(N), kThreads, 0, s>>>(wq, x, y, N, K, y_dtype);
  else
    qgemv_q8_0_kernel<XT, MT, false><<<gemv_grid(N), kThreads, 0, s>>>(wq, x, y, N, K, y_dtype);
  return ub::check_launch();
}

inline size_t dtype_size(int dt) { return dt == UB_DTYPE_F32 ? 4 : 2; }

}  // namespace

namespace ub {

struct ArParams;
template <typename XT>
int q4k_gemv_imma(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, const ArParams* ar,
                  cudaStream_t s);
template <typename XT>
int q8_0_gemv_imma(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s);
template <typename XT>
int q4k_gemv_m1(const void* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, const ArParams* ar,
                cudaStream_t s);

template <typename XT>
int q4k_gemv_mt(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s);
template <typename XT>
int q8_0_gemv_m1(const void* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, cudaStream_t s);
template <typename XT>
int q4k_gemv_mc(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s);
template <typename XT>
int qgemv_ar(bool is_q4k, void* y, const XT* x, const void* wq, int M, int N, int K, int y_dtype, bool fresh,
             const ArParams* ar, cudaStream_t s);

// Q4_K: up to eight rows of x per pass on the integer tensor-core kernel when its shared-memory plan fits.
// Otherwise rows of x are processed four (then two, then one) at a time; each pass streams W once.
template <typename XT>
int qgemv(bool is_q4k, void* y, const XT* x, const void* wq, int M, int N, int K, int y_dtype, bool fresh,
          cudaStream_t s) {
  return qgemv_ar<XT>(is_q4k, y, x, wq, M, N, K, y_dtype, fresh, nullptr, s);
}

// ar != nullptr: one token of Q4_K whose launch ends with the all-reduce over the ranks (see ar_epilogue.cuh);
// UB_ERR_UNSUPPORTED when no kernel with that epilogue takes the shape (the caller then runs matmul and exchange
// as two launches).
template <typename XT>
int qgemv_ar(bool is_q4k, void* y, const XT* x, const void* wq, int M, int N, int K, int y_dtype, bool fresh,
             const ArParams* ar, cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  int m0 = 0;
  while (m0 < M) {
    const int left = M - m0;
    const int mt = left >= 4 ? 4 : (left >= 2 ? 2 : 1);
    const XT* xp = x + static_cast<size_t>(m0) * K;
    void* yp = static_cast<char*>(y) + static_cast<size_t>(m0) * N * dtype_size(y_dtype);
    int st;
    if ((reinterpret_cast<uintptr_t>(wq) & 15) == 0) {
      // five to eight tokens at K = 2048 / 4096 / 8192: tokens in the MMA columns, one pass
      if (is_q4k && !ar && left >= 5) {
        const int mc = left >= 8 ? 8 : left;
        st = q4k_gemv_mc<XT>(wq, xp, yp, mc, N, K, y_dtype, fresh, s);
        if (st == UB_OK) {
          m0 += mc;
          continue;
        }
        if (st != UB_ERR_UNSUPPORTED) return st;
      }
      const int mi = left >= 8 ? 8 : left;
      // one token, or two to four at K = 2048 / 4096: the two-CTAs-per-SM kernels; everything else: the
      // one-CTA-per-SM kernels with token pairs / quads
      st = UB_ERR_UNSUPPORTED;
      if (is_q4k && mi == 1) st = q4k_gemv_m1<XT>(wq, xp, yp, N, K, y_dtype, fresh, ar, s);
      if (is_q4k && mi >= 2 && mi <= 4 && !ar) st = q4k_gemv_mt<XT>(wq, xp, yp, mi, N, K, y_dtype, fresh, s);
      if (!is_q4k && mi == 1) st = q8_0_gemv_m1<XT>(wq, xp, yp, N, K, y_dtype, fresh, s);
      if (st == UB_ERR_UNSUPPORTED)
        st = is_q4k ? q4k_gemv_imma<XT>(wq, xp, yp, mi, N, K, y_dtype, fresh, ar, s)
                    : q8_0_gemv_imma<XT>(wq, xp, yp, mi, N, K, y_dtype, fresh, s);
      if (st == UB_OK) {
        m0 += mi;
        continue;
      }
      if (st != UB_ERR_UNSUPPORTED) return st;
    }
    if (ar) return UB_ERR_UNSUPPORTED;  // the streaming fallbacks below have no exchange epilogue
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

template int qgemv_ar<float>(bool, void*, const float*, const void*, int, int, int, int, bool, const ArParams*,
                             cudaStream_t);
template int qgemv_ar<__nv_bfloat16>(bool, void*, const __nv_bfloat16*, const void*, int, int, int, int, bool,
                                     const ArParams*, cudaStream_t);
template int qgemv<float>(bool, void*, const float*, const void*, int, int, int, int, bool, cudaStream_t);
template int qgemv<__nv_bfloat16>(bool, void*, const __nv_bfloat16*, const void*, int, int, int, int, bool, cudaStream_t);

}  // namespace ub
