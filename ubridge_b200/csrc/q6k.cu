// GGUF Q6_K: dequantisation and the decode matmul (weights streamed once, f32 accumulation).
//
// The reference declares the block (kernels/quant.cpp:170-177: ql[128] low nibbles, qh[64] upper two bits,
// int8 scales[16], f16 d; 210 bytes per 256 values) but ships no kernel for it; in Q4_K_M model files the
// output and embedding matrices come in this format.  The arithmetic is the published GGML one:
// element i of a super-block (h = i / 128, j = (i % 128) / 32, l = i % 32) has its low nibble in
// ql[64h + 32(j & 1) + l] (upper half of the byte for j >= 2) and its top two bits at bit 2j of qh[32h + l];
// y = (d * scales[i / 16]) * (q - 32).
//
// A block is 210 bytes, so nothing in it is better than 2-byte aligned: all weight loads from global memory are
// 16-bit ones, and consecutive lanes read consecutive bytes.  The dequantisation kernel gives a lane two
// neighbouring l of one half (eight weights), the matmul kernels four (sixteen weights).
//
// One to four tokens with rows of a multiple of 2048 values up to 14336 (qgemv_q6k_m1_kernel) do not load weights
// through the load-store unit at all: a row of K / 256 blocks is a multiple of 16 bytes there, so up to eight consecutive rows come into
// shared memory as ONE bulk copy (cp.async.bulk, mbarrier ring, two CTAs per SM, programmatic dependent launch as
// in the Q4_K one-token kernel), are read with aligned 32-bit shared loads (plus a funnel shift in the odd
// blocks) and meet 15-bit block-fixed-point activations in dp4a.
#include <string.h>

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

// ----------------------------------------------------------------------------------------------------------------
// One token, K a multiple of 2048.  A CTA owns a contiguous range of rows (ranges differ by at most one row) and walks
// it in stages of up to eight rows = one bulk copy; warp w takes row w of the stage, all its super-blocks, two per
// step (lanes 0-15 the even one, 16-31 the odd one; inside a super-block a lane owns four neighbouring l of one
// 128-value half and all four j, i.e. 16 weights).  The four 6-bit values of a word become signed bytes 4 (q - 32)
// without a subtraction: ql nibble << 2 | qh bits << 6, top bit flipped.  Activations are quantised once per CTA to
// 15-bit block fixed point per 256 values (q = 254 hi + lo, two signed bytes) and stored so that a lane's sixteen
// values are one 16-byte read per limb.  Per (row, super-block, j): two dp4a, each multiplied by the int8 scale and
// added up in integers; one conversion per limb, d and the activation scale once per super-block.  (Measured on
// B200, 14336 x 4096: 13.8 us; with 32 weights per lane, eight lanes per super-block, 14.7 us; with three CTAs per
// SM 13.9 us.  The shared-memory pipe is the busiest, 42 %, at 59 % issue utilisation.)  A row's sum is added across the warp by
// shuffles in a fixed order.
constexpr int kQ6W = 8;            // warps per CTA = rows per stage
constexpr int kQ6MaxStages = 4;
constexpr uint32_t kQ6Spin = 400000;
constexpr float kQ6XQMax = 32258.f;  // 127 * 254
constexpr size_t kQ6DynBudget = 104 * 1024;     // two CTAs per SM
constexpr size_t kQ6DynBudgetOne = 222 * 1024;  // one CTA per SM

__device__ __forceinline__ bool q6_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool q6_wait(uint32_t bar, uint32_t parity) {
  if (q6_try(bar, parity)) return true;
  for (uint32_t i = 0; i < kQ6Spin; i++) {
    if (q6_try(bar, parity)) return true;
    if (i >= 2) __nanosleep(40);
  }
  return false;
}
__device__ __forceinline__ uint32_t q6_pack4(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
// four values from x + k (k a multiple of 4)
__device__ __forceinline__ void q6_load4(const float* x, int k, float (&v)[4]) {
  const float4 q = __ldg(reinterpret_cast<const float4*>(x + k));
  v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
}
__device__ __forceinline__ void q6_load4(const __nv_bfloat16* x, int k, float (&v)[4]) {
  const uint2 q = __ldg(reinterpret_cast<const uint2*>(x + k));
  v[0] = __uint_as_float(q.x << 16), v[1] = __uint_as_float(q.x & 0xFFFF0000u);
  v[2] = __uint_as_float(q.y << 16), v[3] = __uint_as_float(q.y & 0xFFFF0000u);
}

// MT: token slots (1, 2 or 4; M <= MT tokens are real, the others are not computed).  The weights of a step are
// unpacked once and meet every token's limbs.
template <typename XT, int MT>
__global__ void __launch_bounds__(kQ6W * 32, 2)
qgemv_q6k_m1_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x, void* __restrict__ y, int y_dtype, int M,
                    int N, int K, int S, int early, int* err_word) {
  extern __shared__ __align__(128) unsigned char q6_smem[];
  __shared__ __align__(8) unsigned long long bars[2 * kQ6MaxStages];  // full[S], empty[S]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nsb = K / UB_QK_K;
  const uint32_t row_bytes = static_cast<uint32_t>(nsb) * UB_Q6K_BYTES, stage_bytes = kQ6W * row_bytes;
  unsigned char* const ring = q6_smem;
  uint4* const xhi = reinterpret_cast<uint4*>(q6_smem + static_cast<size_t>(S) * stage_bytes);  // [MT][K / 16]
  uint4* const xlo = xhi + MT * (K / 16);
  float* const xsc = reinterpret_cast<float*>(xlo + MT * (K / 16));  // [MT][nsb]
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  // rows of this CTA
  const int base = N / static_cast<int>(gridDim.x), extra = N % static_cast<int>(gridDim.x);
  const int bx = static_cast<int>(blockIdx.x);
  const int r0 = bx * base + (bx < extra ? bx : extra), nrows = base + (bx < extra ? 1 : 0);
  const int nst = (nrows + kQ6W - 1) / kQ6W;

  // The next kernel in the stream may start as soon as every CTA of this grid has passed this point.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars_s + 8 * s), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars_s + 8 * (kQ6MaxStages + s)), "r"(kQ6W) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // stage n of this CTA = rows r0 + 8 n .. of the range -> ring slot n % S, one bulk copy
  auto issue = [&](int n) {
    const int rows = min(kQ6W, nrows - kQ6W * n);
    const uint32_t bytes = static_cast<uint32_t>(rows) * row_bytes, full = bars_s + 8 * (n % S);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     ring_s + (n % S) * stage_bytes),
                 "l"(wq + static_cast<size_t>(r0 + kQ6W * n) * row_bytes), "r"(bytes), "r"(full)
                 : "memory");
  };
  const int n_early = min(min(early, S), nst);
  if (threadIdx.x == 0)
    for (int n = 0; n < n_early; n++) issue(n);

  // everything below reads what the previous kernel may have written (x) or writes what it may still read (y)
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- activations -> 15-bit block fixed point in shared memory; slot = 16 sb + 8 h + l / 4 holds the sixteen
  // values 256 sb + 128 h + 32 j + l .. l + 3 (j = 0..3), one word per j and limb ----
  for (int slot0 = 0; slot0 < M * (K / 16); slot0 += kQ6W * 32) {
    // whole half-warps are inside or outside (K / 16 is a multiple of 16); tok: the token, slot: inside its row
    const int gslot = slot0 + threadIdx.x, tok = gslot / (K / 16), slot = gslot - tok * (K / 16);
    float v[4][4];
    if (gslot < M * (K / 16)) {
      const int k0 = (slot >> 4) * UB_QK_K + ((slot >> 3) & 1) * 128 + (slot & 7) * 4;
#pragma unroll
      for (int j = 0; j < 4; j++) q6_load4(x + static_cast<size_t>(tok) * K, k0 + 32 * j, v[j]);
    }
    if (slot0 == 0 && threadIdx.x == 0)  // the rest of the ring goes out right behind the activation loads
      for (int n = n_early; n < min(S, nst); n++) issue(n);
    if (gslot < M * (K / 16)) {
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 4; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) amax = fmaxf(amax, fabsf(v[j][e]));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));  // the super-block
      const float inv = amax > 0.f ? kQ6XQMax / amax : 0.f, inv254 = inv * (1.f / 254.f);
      uint32_t wh[4], wl[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        int hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {  // rounding through the mantissa of 1.5 * 2^23; |lo| <= 127 either way
          const int q = __float_as_int(fmaf(v[j][e], inv, 12582912.f)) - 0x4B400000;
          hi[e] = __float_as_int(fmaf(v[j][e], inv254, 12582912.f)) - 0x4B400000;
          lo[e] = q - 254 * hi[e];
        }
        wh[j] = q6_pack4(hi[0], hi[1], hi[2], hi[3]);
        wl[j] = q6_pack4(lo[0], lo[1], lo[2], lo[3]);
      }
      xhi[gslot] = make_uint4(wh[0], wh[1], wh[2], wh[3]);
      xlo[gslot] = make_uint4(wl[0], wl[1], wl[2], wl[3]);
      if ((slot & 15) == 0) xsc[tok * nsb + (slot >> 4)] = amax * (1.f / kQ6XQMax);
    }
  }
  __syncthreads();

  const int sub = lane >> 4, h = (lane >> 3) & 1, lg = lane & 7;
  bool ok = true;
  int slot = 0, round = 0;
#pragma unroll 1
  for (int n = 0; n < nst; n++) {
    if (ok) ok = q6_wait(bars_s + 8 * slot, round & 1);
    const int rows = min(kQ6W, nrows - kQ6W * n);
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.f;
    if (warp < rows) {
      const unsigned char* rowp = ring + static_cast<size_t>(slot) * stage_bytes + static_cast<size_t>(warp) * row_bytes;
      // even super-blocks first, then the odd ones: a block starts 2 (sb & 1) bytes past a 4-byte boundary, and with
      // the parity the same in all lanes the even ones need one aligned word per field, the odd ones two and a
      // funnel shift
#pragma unroll
      for (int par = 0; par < 2; par++)
#pragma unroll 2
      for (int sb = par + 2 * sub; sb < nsb; sb += 4) {
        const unsigned char* blk = rowp + sb * UB_Q6K_BYTES;
        const uint32_t* al = reinterpret_cast<const uint32_t*>(blk - 2 * par);
        const int ia = 16 * h + lg, ib = ia + 8, ih = 32 + 8 * h + lg;
        uint32_t qa = al[ia], qb = al[ib], qh = al[ih];  // qa: low nibbles j = 0, high j = 2; qb: j = 1, j = 3
        if (par) {
          qa = __funnelshift_r(qa, al[ia + 1], 16);
          qb = __funnelshift_r(qb, al[ib + 1], 16);
          qh = __funnelshift_r(qh, al[ih + 1], 16);
        }
        const signed char* sc = reinterpret_cast<const signed char*>(blk + 192) + 8 * h + (lg >> 2);
        const float d = half_bits_to_f32(*reinterpret_cast<const unsigned short*>(blk + 208));
        // signed bytes 4 (q - 32): six bits in bits 2-7, top bit flipped
        const uint32_t w0 = (((qa << 2) & 0x3C3C3C3Cu) | ((qh << 6) & 0xC0C0C0C0u)) ^ 0x80808080u;
        const uint32_t w1 = (((qb << 2) & 0x3C3C3C3Cu) | ((qh << 4) & 0xC0C0C0C0u)) ^ 0x80808080u;
        const uint32_t w2 = (((qa >> 2) & 0x3C3C3C3Cu) | ((qh << 2) & 0xC0C0C0C0u)) ^ 0x80808080u;
        const uint32_t w3 = (((qb >> 2) & 0x3C3C3C3Cu) | (qh & 0xC0C0C0C0u)) ^ 0x80808080u;
        // the int8 scales meet the limb dots in integers (|scale * dot| < 2^23 each), one conversion per limb
        const int s0 = sc[0], s1 = sc[2], s2 = sc[4], s3 = sc[6];
#pragma unroll
        for (int m = 0; m < MT; m++) {
          if (m < 3 || M > 3) {  // only the fourth slot can be empty (one, two or four slots for M = 1, 2, 3-4)
            const uint4 xh = xhi[m * (K / 16) + 16 * sb + 8 * h + lg], xl = xlo[m * (K / 16) + 16 * sb + 8 * h + lg];
            const int H = s0 * __dp4a(static_cast<int>(w0), static_cast<int>(xh.x), 0) +
                          s1 * __dp4a(static_cast<int>(w1), static_cast<int>(xh.y), 0) +
                          s2 * __dp4a(static_cast<int>(w2), static_cast<int>(xh.z), 0) +
                          s3 * __dp4a(static_cast<int>(w3), static_cast<int>(xh.w), 0);
            const int L = s0 * __dp4a(static_cast<int>(w0), static_cast<int>(xl.x), 0) +
                          s1 * __dp4a(static_cast<int>(w1), static_cast<int>(xl.y), 0) +
                          s2 * __dp4a(static_cast<int>(w2), static_cast<int>(xl.z), 0) +
                          s3 * __dp4a(static_cast<int>(w3), static_cast<int>(xl.w), 0);
            const float f = fmaf(static_cast<float>(H), 254.f, static_cast<float>(L));
            acc[m] = fmaf(f, d * (0.25f * xsc[m * nsb + sb]), acc[m]);
          }
        }
      }
    }
    // everything this warp needs from the stage has been read: hand the slot back
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bars_s + 8 * (kQ6MaxStages + slot)) : "memory");
    if ((n & (kQ6W - 1)) == warp && n + S < nst) {
      if (ok) ok = q6_wait(bars_s + 8 * (kQ6MaxStages + slot), round & 1);
      if (ok && lane == 0) issue(n + S);
    }
    if (warp < rows) {
#pragma unroll
      for (int m = 0; m < MT; m++) {
        float v = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if (lane == 0 && (m < 3 || M > 3)) {
          const size_t at = static_cast<size_t>(m) * N + static_cast<size_t>(r0 + kQ6W * n + warp);
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

// One to four tokens, K a multiple of 2048 (rows are then whole 16-byte pieces) while two stages fit beside the
// tokens' limbs (one token: up to 14336), 16-byte aligned weights; UB_ERR_UNSUPPORTED for everything else.  Two CTAs per SM while two stages of eight rows fit beside the activation
// limbs in half an SM's shared memory (K <= 4096), one CTA per SM with the whole of it beyond.
template <typename XT, int MT>
int launch_q6k_m1(const uint8_t* w, const XT* x, void* y, int M, int N, int K, int out_dtype, bool fresh,
                  cudaStream_t s) {
  if (K % 2048 || (reinterpret_cast<uintptr_t>(w) & 15)) return UB_ERR_UNSUPPORTED;
  const size_t row_bytes = static_cast<size_t>(K / UB_QK_K) * UB_Q6K_BYTES, stage_bytes = kQ6W * row_bytes;
  const size_t xbytes = MT * (static_cast<size_t>(K / 16) * 32 + static_cast<size_t>(K / UB_QK_K) * 4);
  int ctas = 2;
  int S = xbytes + 2 * stage_bytes <= kQ6DynBudget ? static_cast<int>((kQ6DynBudget - xbytes) / stage_bytes) : 0;
  if (S < 2) {
    ctas = 1;
    S = xbytes + 2 * stage_bytes <= kQ6DynBudgetOne ? static_cast<int>((kQ6DynBudgetOne - xbytes) / stage_bytes) : 0;
  }
  if (S > kQ6MaxStages) S = kQ6MaxStages;
  if (S < 2) return UB_ERR_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(S) * stage_bytes + xbytes;
  auto kernel = qgemv_q6k_m1_kernel<XT, MT>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  const int slots = ctas * ub::num_sms(), want = (N + kQ6W - 1) / kQ6W;
  const int grid = want < slots ? want : slots;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kQ6W * 32), cfg.dynamicSmemBytes = smem, cfg.stream = s;
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

template <typename XT>
int q6k_matmul(void* y, const XT* x, const void* wq, int M, int N, int K, int out_dtype, cudaStream_t s) {
  // UB_QMATMUL_WEIGHTS_FRESH rides in the upper bits of out_dtype, as in ub_qmatmul_*
  bool fresh = (out_dtype & UB_QMATMUL_WEIGHTS_FRESH) != 0;
  out_dtype &= ~UB_QMATMUL_WEIGHTS_FRESH;
  if (M == 0 || N == 0) return ub::fail(UB_OK);
  if (!y || !x || !wq || M < 0 || N < 0 || K <= 0 || K % UB_QK_K) return ub::fail(UB_ERR_INVALID_ARG);
  if (out_dtype != UB_DTYPE_F32 && out_dtype != UB_DTYPE_BF16 && out_dtype != UB_DTYPE_F16)
    return ub::fail(UB_ERR_INVALID_ARG);
  if ((reinterpret_cast<uintptr_t>(wq) & 1) || (reinterpret_cast<uintptr_t>(x) & 15))  // x rows: paired loads
    return ub::fail(UB_ERR_INVALID_ARG);
  const int esz = out_dtype == UB_DTYPE_F32 ? 4 : 2;
  const int grid = (N + 8 * kQ6kRowsPerWarp - 1) / (8 * kQ6kRowsPerWarp);  // the CTA scheduler evens out the load
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  if (ub::take_weights_written(s)) fresh = true;
  for (int m0 = 0; m0 < M;) {  // passes of up to four tokens: the weights are read once per pass
    const int left = M - m0;
    const XT* xp = x + static_cast<size_t>(m0) * K;
    void* yp = static_cast<char*>(y) + static_cast<size_t>(m0) * N * esz;
    {  // rows staged by bulk copies where the shape allows (the output rows of a pass are N apart there as well)
      const int mt = left >= 4 ? 4 : left;
      const int st = mt == 1   ? launch_q6k_m1<XT, 1>(w, xp, yp, mt, N, K, out_dtype, fresh, s)
                     : mt == 2 ? launch_q6k_m1<XT, 2>(w, xp, yp, mt, N, K, out_dtype, fresh, s)
                               : launch_q6k_m1<XT, 4>(w, xp, yp, mt, N, K, out_dtype, fresh, s);
      if (st == UB_OK) {
        m0 += mt;
        continue;
      }
      if (st != UB_ERR_UNSUPPORTED) return st;
    }
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
