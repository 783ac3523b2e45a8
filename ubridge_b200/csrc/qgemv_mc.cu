// Decode matmul for FIVE TO EIGHT tokens on Q4_K weights with rows of 2048, 4096 or 8192 values, with the tokens in
// the columns of the integer tensor-core instruction:
//
//   y[M,N] = x[M,K] . dequant(Wq)[N,K]^T        (f32 accumulation of exact integer dots)
//
// Replaces the reference's LHS-resident decode matmul (kernels/matmul.cpp:1197-1208,
// kernels/third_party/matmul_decoding.h:381-552) for GGUF Q4_K weights (kernels/quant.cpp:145-150, :356-363) at
// small batch.
//
// Arithmetic.  mma.sync.m16n8k32 (u8 x s8 -> s32) takes 16 weight rows x 32 bytes as A and 32 values of eight
// tokens as B.  The 32 bytes of a 64-value group hold sub-block 2G in the low nibbles and 2G+1 in the high ones:
// A = raw & 0x0F gives the first exactly, A = raw & 0xF0 sixteen times the second, so nibbles are never shifted.
// Activations are 15-bit block fixed point per 256 values, q = 254 hi + lo with hi, lo signed bytes: four
// instructions per group and eight tokens.  Their s32 results are multiplied by the row's 6-bit sub-block scales
// and added up over the super-block in integers (even and odd sub-blocks apart, the odd ones carry the factor 16),
// one conversion to float per super-block.  The min term  sum_j m[row][j] * (sum of q over sub-block j of the token)
// is itself a small matrix product and runs as ONE mma.sync.m16n8k16 (f16 x f16 -> f32) per super-block: the
// sub-block sums (< 2^20) go in as two exact f16 limbs of ten bits, the mins as m * 1024 and m (exact in f16).
//
// Layout.  One CTA of sixteen warps per SM; a stage is 16 rows x 8 super-blocks (18 KB, one swizzled tensor-map
// copy), warp w takes super-block w % 8 of every stage and there the 64-value groups 2 (w / 8), 2 (w / 8) + 1.
// The activation fragments of all tokens (2 bytes per value, 64 KB for eight tokens of 4096 values) stay in shared
// memory for the whole launch.
// Quantising them in every CTA would cost several microseconds, so the CTAs of a cluster of two share the work:
// each quantises the super-blocks of one half of K into its own shared memory and sends that contiguous piece to
// the other with one bulk copy (cp.async.bulk shared::cta -> shared::cluster, counted on a barrier of the
// receiver); then every CTA runs on its own.  (Scattered st.shared::cluster stores into four memories took 2.7 us.)
// Partial sums of the warps meet in shared memory once per tile; the addition (fixed order) is deferred until the
// first stage of the next tile has been consumed, so nobody waits for the slowest warp.  Programmatic dependent
// launch with the first stages requested ahead of the dependency wait, every mbarrier wait bounded, as in the
// one-token kernel.
//
// Measured on B200, 14336 x 4096: 16.4 us for five to eight tokens (the tcgen05 kernel with its K split: 20.8 us; the
// token-pair kernel 11.5 us at four tokens, which is why this one starts at five).  Clusters of four (a quarter of
// K each) fit only 33 at a time, 132 of 148 SMs, and took 17.6 us; with a release / acquire cluster barrier
// between quantisation and exchange 18.9 us.  The launch is bound by instruction issue (597 warp instructions per
// 16 rows x 256 weights, tensor pipe 11 % busy); the same layout with two token groups took 25.5 us for nine to
// sixteen tokens, no better than tcgen05, and was not kept.
#include <cuda.h>  // CUtensorMap type and enums only; the encoder is resolved at run time

#include <string.h>

#include <atomic>

#include "common.cuh"

namespace ub {
void* tensor_map_encoder();
}

namespace {

using namespace ub;

constexpr int kW = 16;  // warps per CTA, all of them compute
constexpr int kThreads = kW * 32;
constexpr int kMaxStages = 8;
constexpr int kCluster = 2;  // CTAs that share the quantisation of the activations
constexpr uint32_t kSpin = 400000;
constexpr float kXQMax = 32258.f;  // 127 * 254
constexpr int kRowStride = 8 * UB_Q4K_BYTES;  // 1152 = 9 lines of 128 bytes
constexpr int kStageBytes = 16 * kRowStride;  // 18 KB
// fragments of one super-block (eight token slots): [8 sub-blocks][hi, lo][32 lanes] uint2, then the min term's B
// operand [32 lanes] uint2, then the eight block scales
constexpr int kFragLimbs = 8 * 2 * 256;
constexpr int kFragMin = 256;
constexpr int kFragSB = kFragLimbs + kFragMin + 32;
constexpr size_t kDynMax = 227 * 1024 - 8 * 1024 - 1024;  // beside 8 KB of partial sums and the barriers

__device__ __forceinline__ void mb_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mb_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mb_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
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
// d = A(16x32 u8, row) . B(32x8 s8, col)
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "r"(0));
}
// d = A(16x16 f16, row) . B(16x8 f16, col), f32
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "f"(0.f));
}
__device__ __forceinline__ uint32_t pack4b(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
__device__ __forceinline__ uint32_t peer_addr(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

// Eight activations of a lane: load and conversion are separate steps, so that all loads of a warp are in flight
// before the first conversion waits.
template <typename XT>
struct Raw8;
template <>
struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void zero() { a = b = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ void unpack(float (&v)[8]) const {
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  }
};
template <>
struct Raw8<__nv_bfloat16> {
  uint4 r;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { r = __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void zero() { r = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void unpack(float (&v)[8]) const {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
};

__device__ __forceinline__ void st_out(void* y, size_t idx, int dtype, float v) {
  if (dtype == UB_DTYPE_F32)
    static_cast<float*>(y)[idx] = v;
  else if (dtype == UB_DTYPE_BF16)
    static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
  else
    static_cast<__half*>(y)[idx] = __float2half_rn(v);
}

// two 6-bit values (bytes lo, lo + 1 of w) as packed f16
__device__ __forceinline__ uint32_t two_bytes_f16(uint32_t w, int sh) {
  const uint32_t biased = __byte_perm(w >> sh, 0x64646464u, 0x4140);  // f16 (1024 + m) in each half
  const uint32_t c1024 = 0x64006400u;
  const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&biased), *reinterpret_cast<const __half2*>(&c1024));
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t times_1024(uint32_t h2) {
  const uint32_t c1024 = 0x64006400u;
  const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&h2), *reinterpret_cast<const __half2*>(&c1024));
  return *reinterpret_cast<const uint32_t*>(&v);
}

// NCH: stages per tile = K / 2048.  M <= 8; token slots the launch does not fill multiply by zero.
template <typename XT, int NCH>
__global__ void __launch_bounds__(kThreads, 1)
qgemv_q4k_mc_kernel(const XT* __restrict__ x, void* __restrict__ y, int M, int N, int y_dtype, int S, int early,
                    int* err_word, const __grid_constant__ CUtensorMap w_map) {
  constexpr int K = 2048 * NCH;
  constexpr int MT = 8;     // token slots
  constexpr int CPW = 4 * NCH / kCluster;  // (token, super-block) chunks of 256 values a warp quantises
  constexpr int NG = 2;     // 64-value groups of its super-block a warp multiplies
  static_assert(MT * 8 * NCH == kCluster * kW * CPW, "every chunk has a warp");
  extern __shared__ __align__(128) unsigned char mc_smem_raw[];
  // swizzled stages need 1024-byte alignment; the launch reserves 1 KB of slack for rounding the base up
  unsigned char* const sm =
      mc_smem_raw + ((1024u - (static_cast<uint32_t>(__cvta_generic_to_shared(mc_smem_raw)) & 1023u)) & 1023u);
  // full[S], empty[S], partial sums full / read, fragments of the other CTAs arrived
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages + 3];
  __shared__ float red[kW][128];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int sbw = warp & 7, part = warp >> 3;
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(sm));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  const uint32_t redfull_s = bars_s + 8 * (2 * kMaxStages), redread_s = redfull_s + 8, fragfull_s = redfull_s + 16;
  unsigned char* const frag = sm + static_cast<size_t>(S) * kStageBytes;  // [8 NCH super-blocks][kFragSB]
  const uint32_t frag_s = ring_s + static_cast<uint32_t>(S) * kStageBytes;
  uint32_t crank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
  const int total_tiles = (N + 15) >> 4;
  const int my_tiles =
      static_cast<int>(blockIdx.x) < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int my_items = my_tiles * NCH;

  // The next kernel in the stream may start as soon as every CTA of this grid has passed this point.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      mb_init(bars_s + 8 * s, 1);
      mb_init(bars_s + 8 * (kMaxStages + s), kW);
    }
    mb_init(redfull_s, kW);
    mb_init(redread_s, kW);
    mb_init(fragfull_s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // "this CTA runs and its barriers exist": the others wait for it before they send their fragments here
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

  // item n of this CTA = (tile n / NCH, stage n % NCH) -> ring slot n % S; rows past N arrive as zeros
  auto issue_item = [&](int n) {
    const int tile = n / NCH, c = n - tile * NCH;
    const uint32_t full = bars_s + 8 * (n % S);
    mb_expect_tx(full, kStageBytes);
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::
            "r"(ring_s + (n % S) * kStageBytes),
        "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(full), "r"(0), "r"(c * (kRowStride >> 7)),
        "r"(16 * (static_cast<int>(blockIdx.x) + tile * static_cast<int>(gridDim.x)))
        : "memory");
  };
  const int n_early = min(min(early, S), my_items);
  if (threadIdx.x == 0)
    for (int n = 0; n < n_early; n++) issue_item(n);

  // everything below reads what the previous kernel may have written (x) or writes what it may still read (y)
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- this warp's share of this CTA's quarter of K, all tokens -> fragments in shared memory ----
  {
    Raw8<XT> raw[CPW];
#pragma unroll
    for (int i = 0; i < CPW; i++) {
      const int id = (static_cast<int>(crank) * kW + warp) * CPW + i, m = id % MT, sbi = id / MT;
      if (m < M)
        raw[i].load(x + static_cast<size_t>(m) * K + static_cast<size_t>(sbi) * 256 + 8 * lane);
      else
        raw[i].zero();  // a token this launch does not have: its columns multiply by zero
    }
    // the rest of the ring goes out right behind the activation loads
    if (threadIdx.x == 0)
      for (int n = n_early; n < min(S, my_items); n++) issue_item(n);
    const int j = lane >> 2;  // this lane holds values 8t .. 8t+7 of sub-block j
#pragma unroll
    for (int i = 0; i < CPW; i++) {
      const int id = (static_cast<int>(crank) * kW + warp) * CPW + i, m = id % MT, sbi = id / MT;
      float v[8];
      raw[i].unpack(v);
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      const float inv = amax > 0.f ? kXQMax / amax : 0.f;
      // Round through the mantissa of 1.5 * 2^23.  q = rint(v inv); hi = rint(v inv / 254) differs from
      // rint(q / 254) only where q / 254 is within 0.002 of a half, and there both choices leave |lo| <= 127.
      const float inv254 = inv * (1.f / 254.f);
      int hi[8], lo[8], sum = 0;
#pragma unroll
      for (int e = 0; e < 8; e++) {
        const int q = __float_as_int(fmaf(v[e], inv, 12582912.f)) - 0x4B400000;
        hi[e] = __float_as_int(fmaf(v[e], inv254, 12582912.f)) - 0x4B400000;
        lo[e] = q - 254 * hi[e];
        sum += q;
      }
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);  // sum of q over this lane's 32-value sub-block, |sum| < 2^20
      const uint32_t h0 = pack4b(hi[0], hi[1], hi[2], hi[3]), h1 = pack4b(hi[4], hi[5], hi[6], hi[7]);
      const uint32_t l0 = pack4b(lo[0], lo[1], lo[2], lo[3]), l1 = pack4b(lo[4], lo[5], lo[6], lo[7]);
      const int col = m & 7;
      const uint32_t sb_off = static_cast<uint32_t>(sbi * kFragSB);
      // B fragment of sub-block j: lane (column = token, t) holds k rows 4t..4t+3 and 16+4t.. = its values 8t..8t+7
      const uint32_t off_hi = sb_off + static_cast<uint32_t>(((2 * j) * 32 + col * 4 + t) * 8), off_lo = off_hi + 256;
      // the min term's B operand: lane (column, t') holds (S_hi[2t'], S_hi[2t'+1]) and (S_lo[2t'], S_lo[2t'+1])
      const int s_hi = sum >> 10, s_lo = sum & 1023;
      const uint32_t off_s = sb_off + kFragLimbs + static_cast<uint32_t>((col * 4 + (j >> 1)) * 8 + (j & 1) * 2);
      const unsigned short sh16 = __half_as_ushort(__int2half_rn(s_hi)), sl16 = __half_as_ushort(__int2half_rn(s_lo));
      const float xs = amax * (1.f / kXQMax);
      *reinterpret_cast<uint2*>(frag + off_hi) = make_uint2(h0, h1);
      *reinterpret_cast<uint2*>(frag + off_lo) = make_uint2(l0, l1);
      if (t == 0) {
        *reinterpret_cast<unsigned short*>(frag + off_s) = sh16;
        *reinterpret_cast<unsigned short*>(frag + off_s + 4) = sl16;
      }
      if (lane == 0) *reinterpret_cast<float*>(frag + sb_off + kFragLimbs + kFragMin + col * 4) = xs;
    }
  }
  // This CTA's piece (its 8 NCH / kCluster super-blocks: contiguous) is complete; the bulk copies below read it
  // through the asynchronous proxy.  The cluster barrier only says that every CTA of the cluster runs and has
  // initialised its barriers (they arrived long ago); a piece arrives wherever it is sent whenever it is ready.
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
  constexpr uint32_t kPiece = 8 * NCH / kCluster * kFragSB;
  static_assert(kPiece % 16 == 0, "bulk copy size");
  if (threadIdx.x == 0) {
    mb_expect_tx(fragfull_s, (kCluster - 1) * kPiece);
    const uint32_t src = frag_s + crank * kPiece;
    for (uint32_t r = 0; r < kCluster; r++)
      if (r != crank)
        asm volatile(
            "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                peer_addr(src, r)),
            "r"(src), "r"(kPiece), "r"(peer_addr(fragfull_s, r))
            : "memory");
  }
  bool ok = mb_wait(fragfull_s, 0);  // the other three pieces have arrived here
  // "this CTA has all it was sent"; the matching wait at the end keeps every CTA (the source of three copies)
  // alive until all of them have said so
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

  // byte offsets of this lane's header and nibble pieces inside a stage (row g, super-block sbw); the 16-byte
  // unit index is XORed with the 128-byte line index modulo 8 (the copy's swizzle).  Row g + 8 lies a multiple
  // of 8 lines further and shares the offsets.
  uint32_t off_h, off_q[NG];
  {
    auto swz = [](uint32_t L) { return L ^ (((L >> 7) & 7u) << 4); };
    const uint32_t L0 = static_cast<uint32_t>(g * kRowStride + sbw * UB_Q4K_BYTES);
    off_h = swz(L0);
#pragma unroll
    for (int G = 0; G < NG; G++) off_q[G] = swz(L0 + 16 + 32 * (2 * part + G) + 8 * t);
  }

  // partial sums of tile `tile_i` (all warps have published them) -> y; each output is added up by the threads
  // 4 o .. 4 o + 3 (four warps each) in a fixed order
  auto reduce = [&](int tile_i) {
    if (ok) ok = mb_wait(redfull_s, tile_i & 1);
    const int o = threadIdx.x >> 2, sub = threadIdx.x & 3;
    const int r = o & 15, c = o >> 4;  // row of the tile, token
    const int idx = ((r >> 3) * 2 + (c & 1)) * 32 + (r & 7) * 4 + (c >> 1);
    const int w0 = 4 * sub;
    float v = (red[w0][idx] + red[w0 + 1][idx]) + (red[w0 + 2][idx] + red[w0 + 3][idx]);
    v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
    v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
    __syncwarp();
    if (lane == 0) mb_arrive(redread_s);
    const int row = 16 * (static_cast<int>(blockIdx.x) + tile_i * static_cast<int>(gridDim.x)) + r;
    if (sub == 0 && row < N && c < M) st_out(y, static_cast<size_t>(c) * N + row, y_dtype, v);
  };

  int slot = 0, round = 0, item = 0;
#pragma unroll 1
  for (int tile_i = 0; tile_i < my_tiles; tile_i++) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int c = 0; c < NCH; c++, item++) {
      if (ok) ok = mb_wait(bars_s + 8 * slot, round & 1);
      const unsigned char* rowA = sm + static_cast<size_t>(slot) * kStageBytes;
      const unsigned char* rowB = rowA + 8 * kRowStride;
      const uint4 hA = *reinterpret_cast<const uint4*>(rowA + off_h);
      const uint4 hB = *reinterpret_cast<const uint4*>(rowB + off_h);
      uint2 wA[NG], wB[NG];
#pragma unroll
      for (int G = 0; G < NG; G++) {
        wA[G] = *reinterpret_cast<const uint2*>(rowA + off_q[G]);
        wB[G] = *reinterpret_cast<const uint2*>(rowB + off_q[G]);
      }
      // everything this warp needs from the stage is in registers: hand the slot back (the arrive is a
      // release, so the loads above are performed before the re-arming warp sees it)
      __syncwarp();
      if (lane == 0) mb_arrive(bars_s + 8 * (kMaxStages + slot));
      if ((item & (kW - 1)) == warp && item + S < my_items) {
        if (ok) ok = mb_wait(bars_s + 8 * (kMaxStages + slot), round & 1);
        if (ok && lane == 0) issue_item(item + S);
      }
      // 6-bit scales and mins (kernels/quant.cpp:356-363), four per word, rows g (A) and g + 8 (B)
      uint32_t scA[2], mnA[2], scB[2], mnB[2];
      q4k_unpack_scales(hA.y, hA.z, hA.w, scA[0], scA[1], mnA[0], mnA[1]);
      q4k_unpack_scales(hB.y, hB.z, hB.w, scB[0], scB[1], mnB[0], mnB[1]);
      const unsigned char* const fsb = frag + static_cast<size_t>(8 * c + sbw) * kFragSB;
      const uint2* const F = reinterpret_cast<const uint2*>(fsb);
      // integer sums over the sub-blocks: [0..3] high limb, [4..7] low limb of (row g: tokens 2t, 2t+1; row g + 8)
      int ev[8] = {0, 0, 0, 0, 0, 0, 0, 0}, od[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int G = 0; G < NG; G++) {
        const int Gs = 2 * part + G;  // group of the super-block: sub-blocks 2 Gs, 2 Gs + 1
        const uint2 bh0 = F[(4 * Gs) * 32 + lane], bl0 = F[(4 * Gs + 1) * 32 + lane];
        const uint2 bh1 = F[(4 * Gs + 2) * 32 + lane], bl1 = F[(4 * Gs + 3) * 32 + lane];
        const uint32_t a0 = wA[G].x & 0x0F0F0F0Fu, a1 = wB[G].x & 0x0F0F0F0Fu, a2 = wA[G].y & 0x0F0F0F0Fu,
                       a3 = wB[G].y & 0x0F0F0F0Fu;
        const uint32_t c0 = wA[G].x & 0xF0F0F0F0u, c1 = wB[G].x & 0xF0F0F0F0u, c2 = wA[G].y & 0xF0F0F0F0u,
                       c3 = wB[G].y & 0xF0F0F0F0u;
        int dh0[4], dl0[4], dh1[4], dl1[4];
        mma_u8s8(dh0, a0, a1, a2, a3, bh0);
        mma_u8s8(dl0, a0, a1, a2, a3, bl0);
        mma_u8s8(dh1, c0, c1, c2, c3, bh1);
        mma_u8s8(dl1, c0, c1, c2, c3, bl1);
        // scales of sub-blocks 2 Gs (even) and 2 Gs + 1 (odd): word `part`, bytes 2 G and 2 G + 1
        const int sh = 16 * G;
        const uint32_t wa = part ? scA[1] : scA[0], wb = part ? scB[1] : scB[0];
        const int sAe = (wa >> sh) & 0xFF, sAo = (wa >> (sh + 8)) & 0xFF;
        const int sBe = (wb >> sh) & 0xFF, sBo = (wb >> (sh + 8)) & 0xFF;
        ev[0] += dh0[0] * sAe, ev[1] += dh0[1] * sAe, ev[2] += dh0[2] * sBe, ev[3] += dh0[3] * sBe;
        ev[4] += dl0[0] * sAe, ev[5] += dl0[1] * sAe, ev[6] += dl0[2] * sBe, ev[7] += dl0[3] * sBe;
        od[0] += dh1[0] * sAo, od[1] += dh1[1] * sAo, od[2] += dh1[2] * sBo, od[3] += dh1[3] * sBo;
        od[4] += dl1[0] * sAo, od[5] += dl1[1] * sAo, od[6] += dl1[2] * sBo, od[7] += dl1[3] * sBo;
      }
      // min term (one of the two warps of a super-block does it)
      float dm[4] = {0.f, 0.f, 0.f, 0.f};
      if (part == 0) {
        const int sh = 16 * (t & 1);
        const uint32_t pa = two_bytes_f16(t >> 1 ? mnA[1] : mnA[0], sh), pb = two_bytes_f16(t >> 1 ? mnB[1] : mnB[0], sh);
        const uint2 bm = *reinterpret_cast<const uint2*>(fsb + kFragLimbs + lane * 8);
        mma_f16(dm, times_1024(pa), times_1024(pb), pa, pb, bm);
      }
      const float2 xs2 = *reinterpret_cast<const float2*>(fsb + kFragLimbs + kFragMin + t * 8);
      const float dA = half_bits_to_f32(hA.x), dminA = half_bits_to_f32(hA.x >> 16);
      const float dB = half_bits_to_f32(hB.x), dminB = half_bits_to_f32(hB.x >> 16);
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float fe = fmaf(static_cast<float>(ev[e]), 254.f, static_cast<float>(ev[4 + e]));
        const float fo = fmaf(static_cast<float>(od[e]), 254.f, static_cast<float>(od[4 + e]));
        const float f = fmaf(fo, 0.0625f, fe);  // the odd sub-blocks carry 16 x their nibbles
        const float xs = (e & 1) ? xs2.y : xs2.x;
        const float d = e < 2 ? dA : dB, dmin = e < 2 ? dminA : dminB;
        acc[e] = fmaf(d * xs, f, acc[e]);
        acc[e] = fmaf(-(dmin * xs), dm[e], acc[e]);
      }
      if (++slot == S) slot = 0, round++;
      // the previous tile's partial sums: every warp has had a stage's time to publish them
      if (c == 0 && tile_i > 0) reduce(tile_i - 1);
    }
    // publish this tile's partial sums once everybody has read the previous tile's
    if (tile_i > 0 && ok) ok = mb_wait(redread_s, (tile_i - 1) & 1);
#pragma unroll
    for (int e = 0; e < 4; e++) red[warp][e * 32 + lane] = acc[e];
    __syncwarp();
    if (lane == 0) mb_arrive(redfull_s);
  }
  if (my_tiles > 0) reduce(my_tiles - 1);
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

template <typename XT, int NCH>
int launch_mc(const uint8_t* wq, const XT* x, void* y, int M, int N, int y_dtype, bool fresh, cudaStream_t s) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ub::tensor_map_encoder());
  if (!enc) return UB_ERR_UNSUPPORTED;
  constexpr int K = 2048 * NCH;
  constexpr size_t frag_bytes = static_cast<size_t>(8) * NCH * kFragSB;
  static_assert(frag_bytes + 3 * static_cast<size_t>(kStageBytes) + 1024 <= kDynMax, "shared-memory plan");
  int S = static_cast<int>((kDynMax - 1024 - frag_bytes) / kStageBytes);
  if (S > kMaxStages) S = kMaxStages;
  CUtensorMap wmap;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(K / UB_QK_K) * UB_Q4K_BYTES;
  const cuuint64_t dims[3] = {128, row_bytes / 128, static_cast<cuuint64_t>(N)};
  const cuuint64_t strides[2] = {128, row_bytes};
  const cuuint32_t box[3] = {128, static_cast<cuuint32_t>(kRowStride / 128), 16u};
  const cuuint32_t estr[3] = {1, 1, 1};
  if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(wq), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return UB_ERR_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(S) * kStageBytes + frag_bytes + 1024;
  auto kernel = qgemv_q4k_mc_kernel<XT, NCH>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(kCluster), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCluster, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  // Clusters that run at once: a cluster lives inside one processor cluster of the chip, so fewer CTAs than SMs
  // may fit (132 of 148 with clusters of four on B200); a grid larger than that would run its last clusters after
  // all the others.
  static std::atomic<int> cached_clusters{0};  // per instantiation; the same on every device of a node
  int max_clusters = cached_clusters.load(std::memory_order_relaxed);
  if (max_clusters == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      return UB_ERR_UNSUPPORTED;
    }
    max_clusters = n;
    cached_clusters.store(n, std::memory_order_relaxed);
  }
  // whole clusters: CTAs without a tile still quantise their share of the activations
  const int tiles = (N + 15) / 16;
  const int slots = max_clusters * kCluster;
  const int grid = tiles < slots ? (tiles + kCluster - 1) / kCluster * kCluster : slots;
  const int early = fresh ? 0 : 2;  // 36 KB per CTA ahead of the dependency wait, as in the one-token kernel
  cfg.gridDim = dim3(grid), cfg.numAttrs = 2;
  e = cudaLaunchKernelEx(&cfg, kernel, x, y, M, N, y_dtype, S, early, ub::device_error_word(), wmap);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::check_launch();
}

}  // namespace

namespace ub {

// Shapes the kernel below takes.
bool q4k_gemv_mc_supported(int M, int K) {
  if (!tensor_map_encoder()) return false;
  return M >= 5 && M <= 8 && (K == 2048 || K == 4096 || K == 8192);
}

// y[M,N] = x[M,K] . dequant(Wq)^T for five to eight tokens; UB_ERR_UNSUPPORTED (without touching the thread's
// status) for what this kernel does not take (other M or K, unaligned weights, no tensor-map encoder).
// fresh: the weight bytes may have been written by the kernel launched just before on the same stream.
template <typename XT>
int q4k_gemv_mc(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  if (!q4k_gemv_mc_supported(M, K) || (reinterpret_cast<uintptr_t>(w) & 15)) return UB_ERR_UNSUPPORTED;
  if (K == 8192) return launch_mc<XT, 4>(w, x, y, M, N, y_dtype, fresh, s);
  if (K == 4096) return launch_mc<XT, 2>(w, x, y, M, N, y_dtype, fresh, s);
  return launch_mc<XT, 1>(w, x, y, M, N, y_dtype, fresh, s);
}

template int q4k_gemv_mc<float>(const void*, const float*, void*, int, int, int, int, bool, cudaStream_t);
template int q4k_gemv_mc<__nv_bfloat16>(const void*, const __nv_bfloat16*, void*, int, int, int, int, bool,
                                        cudaStream_t);

}  // namespace ub
