// Decode GEMV for ONE token (M = 1) on Q4_K weights with K = 2048 or 4096: the launch-to-launch pipeline.
//
//   y[N] = dequant(Wq)[N,K] . x[K]        (f32 accumulation of exact integer dots)
//
// Replaces the reference's LHS-resident decode matmul (kernels/matmul.cpp:1197-1208,
// kernels/third_party/matmul_decoding.h:12-570) for GGUF Q4_K weights (block layout kernels/quant.cpp:145-150,
// scale unpacking :356-363) at the shape the decode path spends its time on.
//
// A 14336 x 4096 Q4_K matrix is 33 MB: at HBM speed it streams in 5 us, so what one launch costs is decided
// by everything that is NOT streaming: the hand-over between consecutive launches, the wait for the
// activations, the arithmetic behind the last tile.  The design follows from that:
//
// * Two CTAs of 8 warps per SM (<= 113 KB of shared memory, 128 registers), grid = 2 x SMs.  A CTA takes the
//   16-row tiles blockIdx.x, blockIdx.x + gridDim.x, ... (three of the 896 at 14336 rows) and its ring of
//   three 36 KB stages holds all of them.  With programmatic dependent launch the CTAs of the NEXT launch
//   move in as the CTAs of this one retire, request their first stage at once (the weights are not
//   written by any kernel; see `fresh`) and only then wait for the previous launch: the first third of the
//   next matrix crosses HBM while the tail of this launch computes, the rest is requested right behind
//   the activation loads.  More than one stage ahead of the wait costs more than it gains: the activation
//   loads then queue behind the weight traffic of their own SM.
// * No producer warp: the warp that is (item mod 8) re-arms a stage once all eight have read it.
// * One-token MMA arrangement.  mma.sync.m16n8k32 (u8 x s8 -> s32) takes the nibble bytes as they lie in
//   memory.  The k range of one instruction is split in two: k 0..15 carries 16 bytes of group Ga = 2q,
//   k 16..31 carries 16 bytes of group Gb = 2q+1 of the same 16 rows; columns 0-3 of B are non-zero only
//   for k < 16, columns 4-7 only for k >= 16.  Per group the four columns are
//       raw bytes  x [ xh(2G) | xl(2G) |    0     |    0     ]
//       raw & 0xF0 x [-xh(2G) |-xl(2G) | xh(2G+1) | xl(2G+1) ]      (accumulated on top)
//   which leaves sum(lo . x(2G)) and 16 sum(hi . x(2G+1)) for both limbs of the activation: all eight columns
//   and all 32 lanes carry results of the one token (lane t owns sub-blocks t and 4+t of rows g, g+8).
//   Activations are quantised once per launch to 15-bit block fixed point per 256 values
//   (q = 254 hi + lo, both limbs signed bytes); each warp quantises only the two super-blocks it owns and
//   keeps their B fragments in registers: no shared memory, no CTA-wide barrier in front of the main loop.
// * Every mbarrier wait is bounded; on expiry the kernel records UB_ERR_TIMEOUT in the device error word and
//   runs out its loops without waiting again.
#include <cuda.h>  // CUtensorMap type and enums only; the encoder is resolved at run time

#include <string.h>

#include "ar_epilogue.cuh"
#include "common.cuh"

namespace ub {
void* tensor_map_encoder();
}

namespace {

using namespace ub;

constexpr int kW = 8;                 // warps per CTA, all of them compute
constexpr int kThreadsM1 = kW * 32;
constexpr int kMaxStagesM1 = 8;
constexpr int kBatchTiles = 4;        // tiles whose row sums are added across warps at once
constexpr uint32_t kSpinM1 = 400000;
constexpr float kXQMaxM1 = 32258.f;   // 127 * 254
constexpr size_t kRingBudget = 110 * 1024 + 512;  // two CTAs per SM: 2 x (ring + 1 KB slack + static + 1 KB reserved) <= 228 KB

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
  for (uint32_t i = 0; i < kSpinM1; i++) {
    if (mb_try(bar, parity)) return true;
    if (i >= 2) __nanosleep(40);
  }
  return false;
}
// d = A(16x32 u8, row) . B(32x8 s8, col)
__device__ __forceinline__ void mma_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "r"(0));
}
// d += A . B
__device__ __forceinline__ void mma_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
}
__device__ __forceinline__ uint32_t pack4_m1(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// Eight activations of a lane: the load and the conversion are separate steps, so that nothing between them
// (the requests for the rest of the ring) waits for the data to arrive.
template <typename XT>
struct Raw8;
template <>
struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void unpack(float (&v)[8]) const {
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  }
};
template <>
struct Raw8<__nv_bfloat16> {
  uint4 r;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { r = __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void unpack(float (&v)[8]) const {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
};

// a normalised activation as a stand-alone RMSNorm kernel would have stored it (rounded to the activation type)
__device__ __forceinline__ float round_as(float v, const float*) { return v; }
__device__ __forceinline__ float round_as(float v, const __nv_bfloat16*) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// RMSNorm scale of the row from the per-warp sums of squares: every warp adds the kW partials in the same order
__device__ __forceinline__ float rms_scale(float my_ss, float* ssq, int warp, int lane, int K, float eps) {
  my_ss = warp_sum(my_ss);
  if (lane == 0) ssq[warp] = my_ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kW; w++) tot += ssq[w];
  return rsqrtf(tot / static_cast<float>(K) + eps);
}

__device__ __forceinline__ void st_out(void* y, size_t idx, int dtype, float v) {
  if (dtype == UB_DTYPE_F32)
    static_cast<float*>(y)[idx] = v;
  else if (dtype == UB_DTYPE_BF16)
    static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
  else
    static_cast<__half*>(y)[idx] = __float2half_rn(v);
}

// SBW: super-blocks per warp = K / 2048.  A stage is one 16-row tile: 16 rows x 8*SBW super-blocks.
// early: stages requested before the wait for the previous kernel (0 when the weights may be fresh).
template <typename XT, int SBW>
__global__ void __launch_bounds__(kThreadsM1, 2)
qgemv_q4k_m1_kernel(const XT* __restrict__ x, void* __restrict__ y, int N, int y_dtype, int S, int early, int split,
                    int* err_word, const XT* __restrict__ gamma, float eps, const ArParams ar,
                    const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap w_map8) {
  constexpr int kRowStride = 8 * SBW * UB_Q4K_BYTES;  // 1152 or 2304: whole 128-byte lines
  constexpr int kStageBytes = 16 * kRowStride;
  extern __shared__ __align__(128) unsigned char m1_smem_raw[];
  // swizzled stages need 1024-byte alignment; the launch reserves 1 KB of slack for rounding the base up
  unsigned char* const sm =
      m1_smem_raw + ((1024u - (static_cast<uint32_t>(__cvta_generic_to_shared(m1_smem_raw)) & 1023u)) & 1023u);
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStagesM1];  // full[S], empty[S]
  __shared__ float red[kW][kBatchTiles][16];
  __shared__ float ssq[kW];  // per-warp sums of squares of the activations (RMSNorm prologue)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(sm));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  const int total_tiles = (N + 15) >> 4;
  // split > 0: the `split` tiles left over after the full rounds are not dealt as a last tile to `split` CTAs, which
  // would then finish a whole tile later than everybody else and hold back the next launch; they are cut in halves
  // of eight rows, one for each of the first 2 * split CTAs (the last tile of such a CTA, rows 0-7 of its stage).
  const int rounds = total_tiles / static_cast<int>(gridDim.x);
  const bool has_half = split > 0 && static_cast<int>(blockIdx.x) < 2 * split;
  const int my_tiles =
      split > 0 ? rounds + (has_half ? 1 : 0)
                : (static_cast<int>(blockIdx.x) < total_tiles
                       ? (total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                             static_cast<int>(gridDim.x)
                       : 0);
  const int nbatches = (my_tiles + kBatchTiles - 1) / kBatchTiles;
  // first row of this CTA's tile n
  auto tile_row0 = [&](int n) {
    if (has_half && n == my_tiles - 1)
      return 16 * (rounds * static_cast<int>(gridDim.x) + (static_cast<int>(blockIdx.x) >> 1)) +
             8 * (static_cast<int>(blockIdx.x) & 1);
    return 16 * (static_cast<int>(blockIdx.x) + n * static_cast<int>(gridDim.x));
  };

  // The next kernel in the stream may start as soon as every CTA of this grid has passed this point: its
  // CTAs take over SMs as ours retire.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      mb_init(bars_s + 8 * s, 1);
      mb_init(bars_s + 8 * (kMaxStagesM1 + s), kW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // tile n of this CTA -> ring slot n % S: one tensor-map copy of 16 rows x (kRowStride / 128) lines, 128-byte
  // swizzle; rows past N arrive as zeros
  auto issue_tile = [&](int n) {
    const uint32_t full = bars_s + 8 * (n % S);
    const bool half = has_half && n == my_tiles - 1;  // eight rows through the map with the eight-row box
    mb_expect_tx(full, half ? kStageBytes / 2 : kStageBytes);
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::
            "r"(ring_s + (n % S) * kStageBytes),
        "l"(reinterpret_cast<uint64_t>(half ? &w_map8 : &w_map)), "r"(full), "r"(0), "r"(0), "r"(tile_row0(n))
        : "memory");
  };
  const int n_early = min(min(early, S), my_tiles);
  if (threadIdx.x == 0)
    for (int n = 0; n < n_early; n++) issue_tile(n);

  // everything below reads what the previous kernel may have written (x) or writes what it may still read (y)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t epoch = ar.world > 1 ? ar_epoch(ar) : 0;  // of the fused all-reduce, read after the wait

  // ---- activations of this warp's super-blocks -> B fragments in registers ----
  uint2 bf[SBW][2][4];  // [super-block][q][MMA 1 first/second half, MMA 2 first/second half] = (k < 16, k >= 16)
  int Sa[SBW], Sb[SBW];  // sums of q over sub-blocks t and 4 + t (for the min term)
  float xs[SBW];
  {
    Raw8<XT> raw[SBW];
#pragma unroll
    for (int k = 0; k < SBW; k++) raw[k].load(x + static_cast<size_t>(warp + 8 * k) * 256 + 8 * lane);
    // the rest of the ring goes out right behind the activation loads
    Raw8<XT> graw[SBW];
    if (gamma)
#pragma unroll
      for (int k = 0; k < SBW; k++) graw[k].load(gamma + static_cast<size_t>(warp + 8 * k) * 256 + 8 * lane);
    if (threadIdx.x == 0)
      for (int n = n_early; n < min(S, my_tiles); n++) issue_tile(n);
    float v[SBW][8];
#pragma unroll
    for (int k = 0; k < SBW; k++) raw[k].unpack(v[k]);
    if (gamma) {  // RMSNorm in front of the matmul: x * rsqrt(mean(x^2) + eps) * gamma, rounded to the activation type
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < SBW; k++)
#pragma unroll
        for (int e = 0; e < 8; e++) ss = fmaf(v[k][e], v[k][e], ss);
      const float scale = rms_scale(ss, ssq, warp, lane, 2048 * SBW, eps);
#pragma unroll
      for (int k = 0; k < SBW; k++) {
        float gv[8];
        graw[k].unpack(gv);
#pragma unroll
        for (int e = 0; e < 8; e++) v[k][e] = round_as(round_as(v[k][e] * scale, x) * gv[e], x);
      }
    }
#pragma unroll
    for (int k = 0; k < SBW; k++) {
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[k][e]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      const float inv = amax > 0.f ? kXQMaxM1 / amax : 0.f;
      xs[k] = amax * (1.f / kXQMaxM1);
      // Round through the mantissa of 1.5 * 2^23.  q = rint(v inv); hi = rint(v inv / 254) differs from
      // rint(q / 254) only where q / 254 is within 0.002 of a half, and there both choices leave |lo| <= 127.
      const float inv254 = inv * (1.f / 254.f);
      int hi[8], lo[8], sum = 0;
#pragma unroll
      for (int e = 0; e < 8; e++) {
        const int q = __float_as_int(fmaf(v[k][e], inv, 12582912.f)) - 0x4B400000;
        hi[e] = __float_as_int(fmaf(v[k][e], inv254, 12582912.f)) - 0x4B400000;
        lo[e] = q - 254 * hi[e];
        sum += q;
      }
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);  // sum of q over this lane's 32-value sub-block (lane / 4)
      const uint32_t hvx = pack4_m1(hi[0], hi[1], hi[2], hi[3]), hvy = pack4_m1(hi[4], hi[5], hi[6], hi[7]);
      const uint32_t lvx = pack4_m1(lo[0], lo[1], lo[2], lo[3]), lvy = pack4_m1(lo[4], lo[5], lo[6], lo[7]);
      // B fragment of lane (column g, k rows 4t..4t+3): column g of group pair q belongs to sub-block
      // 4q + g/2, even columns carry the high limb, odd ones the low limb; elements 8t..8t+7 of that
      // sub-block sit in lane 4 (4q + g/2) + t
#pragma unroll
      for (int q = 0; q < 2; q++) {
        const int src = 4 * (4 * q + (g >> 1)) + t;
        const uint32_t hx = __shfl_sync(0xFFFFFFFFu, hvx, src), hy = __shfl_sync(0xFFFFFFFFu, hvy, src);
        const uint32_t lx = __shfl_sync(0xFFFFFFFFu, lvx, src), ly = __shfl_sync(0xFFFFFFFFu, lvy, src);
        const uint32_t wx = (g & 1) ? lx : hx, wy = (g & 1) ? ly : hy;
        // MMA 1 (raw bytes): columns 0, 1, 4, 5 only.  MMA 2 (raw & 0xF0): those negated, columns 2, 3, 6, 7 plain
        // (no limb is -128, so the per-byte negation cannot overflow)
        const uint32_t m1x = (g & 2) ? 0u : wx, m1y = (g & 2) ? 0u : wy;
        const uint32_t m2x = (g & 2) ? wx : __vneg4(wx), m2y = (g & 2) ? wy : __vneg4(wy);
        const bool lowk = g < 4;  // columns 0-3 live in k 0..15, columns 4-7 in k 16..31
        bf[k][q][0] = lowk ? make_uint2(m1x, 0) : make_uint2(0, m1x);
        bf[k][q][1] = lowk ? make_uint2(m1y, 0) : make_uint2(0, m1y);
        bf[k][q][2] = lowk ? make_uint2(m2x, 0) : make_uint2(0, m2x);
        bf[k][q][3] = lowk ? make_uint2(m2y, 0) : make_uint2(0, m2y);
      }
      Sa[k] = __shfl_sync(0xFFFFFFFFu, sum, 4 * t);
      Sb[k] = __shfl_sync(0xFFFFFFFFu, sum, 16 + 4 * t);
    }
  }

  // byte offsets of this lane's header and nibble pieces inside a stage (row g, super-blocks warp + 8 i); the
  // 16-byte unit index is XORed with the 128-byte line index modulo 8 (the copy's swizzle).  Row g + 8 lies a
  // multiple of 8 lines further and shares the offsets.
  uint32_t off_h[SBW], off_q[SBW][4];
#pragma unroll
  for (int i = 0; i < SBW; i++) {
    auto swz = [](uint32_t L) { return L ^ (((L >> 7) & 7u) << 4); };
    const uint32_t L0 = static_cast<uint32_t>(g * kRowStride + (warp + 8 * i) * UB_Q4K_BYTES);
    off_h[i] = swz(L0);
#pragma unroll
    for (int G = 0; G < 4; G++) off_q[i][G] = swz(L0 + 16 + 32 * G + 8 * t);
  }
  const uint32_t selb = 0x4440u | static_cast<uint32_t>(t);  // byte t of a word
  const float odd16 = (t & 1) ? 0.0625f : 1.f;               // odd lanes carry 16 x the high nibbles

  bool ok = true;
  int slot = 0, round = 0, tile = 0;
  for (int b = 0; b < nbatches; b++) {
    const int n_mt = min(kBatchTiles, my_tiles - b * kBatchTiles);
#pragma unroll 1
    for (int mt = 0; mt < n_mt; mt++, tile++) {
      if (ok) ok = mb_wait(bars_s + 8 * slot, round & 1);
      const unsigned char* rowA = sm + static_cast<size_t>(slot) * kStageBytes;
      const unsigned char* rowB = rowA + 8 * kRowStride;
      const bool half = has_half && tile == my_tiles - 1;  // rows 8-15 of the stage hold nothing of this tile
      uint4 hA[SBW], hB[SBW];
      uint2 wA[SBW][4], wB[SBW][4];
#pragma unroll
      for (int i = 0; i < SBW; i++) {
        hA[i] = *reinterpret_cast<const uint4*>(rowA + off_h[i]);
#pragma unroll
        for (int G = 0; G < 4; G++) wA[i][G] = *reinterpret_cast<const uint2*>(rowA + off_q[i][G]);
        if (!half) {
          hB[i] = *reinterpret_cast<const uint4*>(rowB + off_h[i]);
#pragma unroll
          for (int G = 0; G < 4; G++) wB[i][G] = *reinterpret_cast<const uint2*>(rowB + off_q[i][G]);
        } else {
          hB[i] = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int G = 0; G < 4; G++) wB[i][G] = make_uint2(0, 0);
        }
      }
      // everything this warp needs from the stage is in registers: hand the slot back (the arrive is a
      // release, so the loads above are performed before the re-arming warp sees it)
      __syncwarp();
      if (lane == 0) mb_arrive(bars_s + 8 * (kMaxStagesM1 + slot));
      if ((tile & (kW - 1)) == warp && tile + S < my_tiles) {
        if (ok) ok = mb_wait(bars_s + 8 * (kMaxStagesM1 + slot), round & 1);
        if (ok && lane == 0) issue_tile(tile + S);
      }
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int i = 0; i < SBW; i++) {
        int d[2][4];
#pragma unroll
        for (int q = 0; q < 2; q++) {
          const int Ga = 2 * q, Gb = 2 * q + 1;
          mma_first(d[q], wA[i][Ga].x, wB[i][Ga].x, wA[i][Gb].x, wB[i][Gb].x, bf[i][q][0]);
          mma_acc(d[q], wA[i][Ga].y, wB[i][Ga].y, wA[i][Gb].y, wB[i][Gb].y, bf[i][q][1]);
          mma_acc(d[q], wA[i][Ga].x & 0xF0F0F0F0u, wB[i][Ga].x & 0xF0F0F0F0u, wA[i][Gb].x & 0xF0F0F0F0u,
                  wB[i][Gb].x & 0xF0F0F0F0u, bf[i][q][2]);
          mma_acc(d[q], wA[i][Ga].y & 0xF0F0F0F0u, wB[i][Ga].y & 0xF0F0F0F0u, wA[i][Gb].y & 0xF0F0F0F0u,
                  wB[i][Gb].y & 0xF0F0F0F0u, bf[i][q][3]);
        }
        // 6-bit scales and mins of sub-blocks t and 4 + t (kernels/quant.cpp:356-363), rows g (A) and g + 8 (B)
        const uint32_t a0 = __byte_perm(hA[i].y, 0, selb), a1 = __byte_perm(hA[i].z, 0, selb),
                       a2 = __byte_perm(hA[i].w, 0, selb);
        const int scA0 = a0 & 63, mnA0 = a1 & 63, scA1 = (a2 & 15) | ((a0 >> 2) & 0x30),
                  mnA1 = (a2 >> 4) | ((a1 >> 2) & 0x30);
        // columns 2t, 2t+1 of d: high- and low-limb dots of sub-block 4q + t
        const int hiA = d[0][0] * scA0 + d[1][0] * scA1, loA = d[0][1] * scA0 + d[1][1] * scA1;
        const int tA = mnA0 * Sa[i] + mnA1 * Sb[i];
        const float dA = half_bits_to_f32(hA[i].x), dminA = half_bits_to_f32(hA[i].x >> 16);
        const float fA = fmaf(static_cast<float>(hiA), 254.f, static_cast<float>(loA));
        const float xsm = xs[i] * odd16;
        acc0 = fmaf(fA, dA * xsm, acc0);
        acc0 = fmaf(-static_cast<float>(tA), dminA * xs[i], acc0);
        if (!half) {  // rows 8-15
          const uint32_t b0 = __byte_perm(hB[i].y, 0, selb), b1 = __byte_perm(hB[i].z, 0, selb),
                         b2 = __byte_perm(hB[i].w, 0, selb);
          const int scB0 = b0 & 63, mnB0 = b1 & 63, scB1 = (b2 & 15) | ((b0 >> 2) & 0x30),
                    mnB1 = (b2 >> 4) | ((b1 >> 2) & 0x30);
          const int hiB = d[0][2] * scB0 + d[1][2] * scB1, loB = d[0][3] * scB0 + d[1][3] * scB1;
          const int tB = mnB0 * Sa[i] + mnB1 * Sb[i];
          const float dB = half_bits_to_f32(hB[i].x), dminB = half_bits_to_f32(hB[i].x >> 16);
          const float fB = fmaf(static_cast<float>(hiB), 254.f, static_cast<float>(loB));
          acc1 = fmaf(fB, dB * xsm, acc1);
          acc1 = fmaf(-static_cast<float>(tB), dminB * xs[i], acc1);
        }
      }
      // rows g and g + 8 of this tile: add the four lanes of a row (fixed order), park the warp's partial sums
      acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 1);
      acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 1);
      acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 2);
      acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 2);
      if (t == 0) red[warp][mt][g] = acc0, red[warp][mt][8 + g] = acc1;
      if (++slot == S) slot = 0, round++;
    }
    __syncthreads();  // partial sums of the batch are complete
    if (static_cast<int>(threadIdx.x) < n_mt * 16) {
      const int mt = threadIdx.x >> 4, r = threadIdx.x & 15;
      const int n = b * kBatchTiles + mt;
      const int row = tile_row0(n) + r;
      if (row < N && !(has_half && n == my_tiles - 1 && r >= 8)) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kW; w++) tot += red[w][mt][r];  // fixed order: deterministic
        if (ar.world > 1)
          ar_push(ar, epoch, row, tot);
        else
          st_out(y, row, y_dtype, ar.residual ? tot + __bfloat162float(ar.residual[row]) : tot);
      }
    }
    if (b + 1 < nbatches) __syncthreads();  // before the next batch overwrites the partial sums
  }
  if (ar.world > 1) ar_finish(ar, epoch, y, N, err_word);
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

template <typename XT, int SBW>
int launch_m1(const uint8_t* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, const XT* gamma,
              float eps, const ArParams& ar, cudaStream_t s) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ub::tensor_map_encoder());
  if (!enc) return UB_ERR_UNSUPPORTED;
  constexpr int kRowStride = 8 * SBW * UB_Q4K_BYTES;
  constexpr int kStageBytes = 16 * kRowStride;
  // A decode step calls this once per weight matrix and token, and the host side of a call costs about as much
  // as the launch runs on the GPU (5-7 us against 6.6 us at 14336 x 4096): the two tensor maps of a matrix depend
  // on its address and shape only and are kept per thread, and the kernel's shared-memory attribute is set once
  // per device.
  struct MapEntry {
    const uint8_t* wq;
    int N, K;
    CUtensorMap m16, m8;
  };
  static thread_local MapEntry cache[8];
  static thread_local int cache_next = 0;
  const MapEntry* hit = nullptr;
  for (int i = 0; i < 8; i++)
    if (cache[i].wq == wq && cache[i].N == N && cache[i].K == K) hit = &cache[i];
  if (!hit) {
    MapEntry ent;
    ent.wq = wq, ent.N = N, ent.K = K;
    // rows as lines of 128 bytes: {128 bytes, lines per row, N rows}; box = one 16-row tile
    const cuuint64_t row_bytes = static_cast<cuuint64_t>(K / UB_QK_K) * UB_Q4K_BYTES;
    const cuuint64_t dims[3] = {128, row_bytes / 128, static_cast<cuuint64_t>(N)};
    const cuuint64_t strides[2] = {128, row_bytes};
    const cuuint32_t box[3] = {128, static_cast<cuuint32_t>(kRowStride / 128), 16};
    const cuuint32_t estr[3] = {1, 1, 1};
    if (enc(&ent.m16, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(wq), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return UB_ERR_UNSUPPORTED;
    // the same rows through a box of eight: the halves of the tiles left over after the full rounds
    const cuuint32_t box8[3] = {128, static_cast<cuuint32_t>(kRowStride / 128), 8};
    if (enc(&ent.m8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(wq), dims, strides, box8, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return UB_ERR_UNSUPPORTED;
    cache[cache_next] = ent;
    hit = &cache[cache_next];
    cache_next = (cache_next + 1) & 7;
  }
  const CUtensorMap& wmap = hit->m16;
  const CUtensorMap& wmap8 = hit->m8;
  int S = static_cast<int>(kRingBudget / kStageBytes);
  if (S > kMaxStagesM1) S = kMaxStagesM1;
  const size_t smem = static_cast<size_t>(S) * kStageBytes + 1024;
  auto kernel = qgemv_q4k_m1_kernel<XT, SBW>;
  cudaError_t e;
  {
    static std::atomic<unsigned long long> attr_set{0};  // bit d: done on device d (this instantiation)
    int dev = 0;
    cudaGetDevice(&dev);
    const unsigned long long bit = (dev >= 0 && dev < 64) ? 1ull << dev : 0;
    if (!(attr_set.load(std::memory_order_relaxed) & bit) || !bit) {
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) {
        ub::set_cuda_error(e);
        return ub::fail(UB_ERR_CUDA);
      }
      attr_set.fetch_or(bit, std::memory_order_relaxed);
    }
  }
  const int tiles = (N + 15) / 16;
  const int slots = 2 * ub::num_sms();
  const int grid = tiles < slots ? tiles : slots;
  // one 36 KB stage (two 18 KB ones) ahead of the dependency wait; none when the weights may still be
  // in flight from the previous kernel
  const int early = fresh ? 0 : (SBW == 2 ? 1 : 2);
  // A few tiles left over after the full rounds (8 of 896 on 296 CTAs at 14336 rows) would make as many CTAs
  // finish a tile later than the rest, and the next launch waits for the last CTA: cut them in halves instead.
  // Only for a few: with 88 of 384 left over (6144 rows) halves measured 1 % slower than whole tiles.
  const int rem = tiles % grid;
  const int split = (tiles > grid && rem > 0 && 8 * rem <= grid) ? rem : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kThreadsM1), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, x, y, N, y_dtype, S, early, split, ub::device_error_word(), gamma, eps, ar, wmap,
                         wmap8);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::check_launch();
}


// =====================================================================================================
// The same kernel for longer rows (K a multiple of 2048: the 8192-wide projections of a 70B-shaped stack in one
// pass, its 28672-wide down projection in four).  A stage is 16 rows x 8 super-blocks (18 KB), a tile takes K / 2048 stages and warp w owns
// super-block 8c + w of every stage c.  The activation fragments no longer fit the register file: each warp
// writes those of its own super-blocks to shared memory once per launch (one word per MMA and lane: the
// half of the B operand that is zero by construction is not stored, the main loop puts the word into the
// k < 16 or the k >= 16 register by lane) and reads them back per stage; only the owning warp ever touches
// them, so there is still no CTA-wide barrier in front of the main loop.
constexpr int kFragBytesPerSb = 1024 + 48;  // 8 words x 32 lanes, then {S_t, S_4+t} x 4 and the block scale
constexpr int kMaxChunks = 6;

// GU: the matrix is [gate rows; up rows] (2 N rows) and y[r] = silu(gate_r . x) * (up_r . x): a stage holds gate
// rows 8T..8T+7 in its rows 0-7 and the matching up rows in its rows 8-15 (two 8-row copies), so that the two
// halves of every MMA row pair meet in one thread of the epilogue.  Gate and up are rounded to the output type
// before the activation, which gives the bits of the two-kernel sequence (matmul, then ub_silu_and_mul).
// MULTI: K is consumed in `npass` passes (rows too long for all activation fragments to be resident at once).
template <typename XT, bool GU, bool MULTI>
__global__ void __launch_bounds__(kThreadsM1, 2)
qgemv_q4k_m1_long_kernel(const XT* __restrict__ x, void* __restrict__ y, int N, int nch, int npass, int y_dtype, int S,
                         int early, int* err_word, const XT* __restrict__ gamma, float eps, const ArParams ar,
                         const __grid_constant__ CUtensorMap w_map) {
  constexpr int kRowStride = 8 * UB_Q4K_BYTES;  // 1152 = 9 lines
  constexpr int kStageBytes = 16 * kRowStride;
  extern __shared__ __align__(128) unsigned char m1_smem_raw[];
  unsigned char* const sm =
      m1_smem_raw + ((1024u - (static_cast<uint32_t>(__cvta_generic_to_shared(m1_smem_raw)) & 1023u)) & 1023u);
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStagesM1];
  __shared__ float red[kW][kBatchTiles][16];
  __shared__ float ssq[kW];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(sm));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  unsigned char* const frag = sm + static_cast<size_t>(S) * kStageBytes;  // [nch * 8][kFragBytesPerSb]
  constexpr int kTileRows = GU ? 8 : 16;  // output rows per tile
  const int total_tiles = (N + kTileRows - 1) / kTileRows;
  const int my_tiles =
      static_cast<int>(blockIdx.x) < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int my_items = my_tiles * nch;
  const int nbatches = (my_tiles + kBatchTiles - 1) / kBatchTiles;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      mb_init(bars_s + 8 * s, 1);
      mb_init(bars_s + 8 * (kMaxStagesM1 + s), kW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // K in passes of cpp stages (npass > 1: rows too long for all activation fragments to be resident at once; the
  // launcher then guarantees a single batch of tiles): items run pass by pass, inside a pass tile by tile.
  const int cpp = (nch + npass - 1) / npass;
  // item n of this CTA -> (tile, stage) -> ring slot n % S
  auto issue_item = [&](int n) {
    int tile, c;
    if (!MULTI) {
      tile = n / nch, c = n - tile * nch;
    } else {
      int p = 0, r = n;
      while (r >= my_tiles * min(cpp, nch - p * cpp)) r -= my_tiles * min(cpp, nch - p * cpp), p++;
      const int cn = min(cpp, nch - p * cpp);
      tile = r / cn, c = p * cpp + (r - tile * cn);
    }
    const uint32_t full = bars_s + 8 * (n % S);
    const int row0 = kTileRows * (static_cast<int>(blockIdx.x) + tile * static_cast<int>(gridDim.x));
    mb_expect_tx(full, kStageBytes);
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::
            "r"(ring_s + (n % S) * kStageBytes),
        "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(full), "r"(0), "r"(c * (kRowStride >> 7)), "r"(row0)
        : "memory");
    if (GU)  // the tensor map's box is 8 rows tall: the up rows follow N rows further down
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::
              "r"(ring_s + (n % S) * kStageBytes + 8 * kRowStride),
          "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(full), "r"(0), "r"(c * (kRowStride >> 7)), "r"(N + row0)
          : "memory");
  };
  const int n_early = min(min(early, S), my_items);
  if (threadIdx.x == 0)
    for (int n = 0; n < n_early; n++) issue_item(n);

  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t epoch = ar.world > 1 ? ar_epoch(ar) : 0;  // of the fused all-reduce, read after the wait

  // ---- activations of this warp's super-blocks of one pass (stages c0 .. c0 + cn - 1, super-block 8c + warp) ->
  // fragments in shared memory, slot c - c0.  Only this warp reads them back, so a pass may overwrite them
  // behind a warp-level barrier.
  // (Fetching the next pass's activations into shared memory with asynchronous copies while the current pass
  // computes was measured and is no faster: 37.0 against 35.7 us at 8192 x 28672; it costs a ring stage.)
  auto quantise = [&](int c0, int cn, bool first) {
    Raw8<XT> raw[kMaxChunks];
#pragma unroll
    for (int c = 0; c < kMaxChunks; c++)
      if (c < cn) raw[c].load(x + static_cast<size_t>(8 * (c0 + c) + warp) * 256 + 8 * lane);
    Raw8<XT> graw[kMaxChunks];
    if (gamma)
#pragma unroll
      for (int c = 0; c < kMaxChunks; c++)
        if (c < cn) graw[c].load(gamma + static_cast<size_t>(8 * (c0 + c) + warp) * 256 + 8 * lane);
    if (first && threadIdx.x == 0)
      for (int n = n_early; n < min(S, my_items); n++) issue_item(n);
    float scale = 1.f;
    if (gamma) {  // RMSNorm in front of the matmul
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < kMaxChunks; c++) {
        if (c >= cn) break;
        float v[8];
        raw[c].unpack(v);
#pragma unroll
        for (int e = 0; e < 8; e++) ss = fmaf(v[e], v[e], ss);
      }
      scale = rms_scale(ss, ssq, warp, lane, 2048 * nch, eps);
    }
#pragma unroll
    for (int c = 0; c < kMaxChunks; c++) {
      if (c >= cn) break;
      float v[8];
      raw[c].unpack(v);
      if (gamma) {
        float gv[8];
        graw[c].unpack(gv);
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = round_as(round_as(v[e] * scale, x) * gv[e], x);
      }
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      const float inv = amax > 0.f ? kXQMaxM1 / amax : 0.f;
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
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
      const uint32_t hvx = pack4_m1(hi[0], hi[1], hi[2], hi[3]), hvy = pack4_m1(hi[4], hi[5], hi[6], hi[7]);
      const uint32_t lvx = pack4_m1(lo[0], lo[1], lo[2], lo[3]), lvy = pack4_m1(lo[4], lo[5], lo[6], lo[7]);
      unsigned char* const f = frag + static_cast<size_t>(8 * c + warp) * kFragBytesPerSb;
#pragma unroll
      for (int q = 0; q < 2; q++) {
        const int src = 4 * (4 * q + (g >> 1)) + t;
        const uint32_t hx = __shfl_sync(0xFFFFFFFFu, hvx, src), hy = __shfl_sync(0xFFFFFFFFu, hvy, src);
        const uint32_t lx = __shfl_sync(0xFFFFFFFFu, lvx, src), ly = __shfl_sync(0xFFFFFFFFu, lvy, src);
        const uint32_t wx = (g & 1) ? lx : hx, wy = (g & 1) ? ly : hy;
        uint4 w4;
        w4.x = (g & 2) ? 0u : wx;            // MMA 1, first half of the group bytes
        w4.y = (g & 2) ? 0u : wy;            // MMA 1, second half
        w4.z = (g & 2) ? wx : __vneg4(wx);   // MMA 2, first half
        w4.w = (g & 2) ? wy : __vneg4(wy);   // MMA 2, second half
        reinterpret_cast<uint4*>(f + q * 512)[lane] = w4;
      }
      const int s_lo = __shfl_sync(0xFFFFFFFFu, sum, 4 * t), s_hi = __shfl_sync(0xFFFFFFFFu, sum, 16 + 4 * t);
      if (g == 0) reinterpret_cast<int2*>(f + 1024)[t] = make_int2(s_lo, s_hi);
      if (lane == 0) *reinterpret_cast<float*>(f + 1024 + 32) = amax * (1.f / kXQMaxM1);
    }
    __syncwarp();
  };
  if (!MULTI) quantise(0, nch, true);

  uint32_t off_h, off_q[4];
  {
    auto swz = [](uint32_t L) { return L ^ (((L >> 7) & 7u) << 4); };
    const uint32_t L0 = static_cast<uint32_t>(g * kRowStride + warp * UB_Q4K_BYTES);
    off_h = swz(L0);
#pragma unroll
    for (int G = 0; G < 4; G++) off_q[G] = swz(L0 + 16 + 32 * G + 8 * t);
  }
  const uint32_t selb = 0x4440u | static_cast<uint32_t>(t);
  const float odd16 = (t & 1) ? 0.0625f : 1.f;
  const uint32_t mlo = g < 4 ? 0xFFFFFFFFu : 0u, mhi = ~mlo;  // which half of the k range this lane's columns use

  bool ok = true;
  int slot = 0, round = 0, item = 0;
  for (int b = 0; b < nbatches; b++) {
    const int n_mt = min(kBatchTiles, my_tiles - b * kBatchTiles);
#pragma unroll 1
    for (int pass = 0; pass < (MULTI ? npass : 1); pass++) {
    const int c_lo = MULTI ? pass * cpp : 0, c_n = MULTI ? min(cpp, nch - c_lo) : nch;
    if (MULTI) quantise(c_lo, c_n, pass == 0);
#pragma unroll 1
    for (int mt = 0; mt < n_mt; mt++) {
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 1
      for (int c = 0; c < c_n; c++, item++) {
        if (ok) ok = mb_wait(bars_s + 8 * slot, round & 1);
        const unsigned char* rowA = sm + static_cast<size_t>(slot) * kStageBytes;
        const unsigned char* rowB = rowA + 8 * kRowStride;
        const uint4 hA = *reinterpret_cast<const uint4*>(rowA + off_h);
        const uint4 hB = *reinterpret_cast<const uint4*>(rowB + off_h);
        uint2 wA[4], wB[4];
#pragma unroll
        for (int G = 0; G < 4; G++) {
          wA[G] = *reinterpret_cast<const uint2*>(rowA + off_q[G]);
          wB[G] = *reinterpret_cast<const uint2*>(rowB + off_q[G]);
        }
        __syncwarp();
        if (lane == 0) mb_arrive(bars_s + 8 * (kMaxStagesM1 + slot));
        if ((item & (kW - 1)) == warp && item + S < my_items) {
          if (ok) ok = mb_wait(bars_s + 8 * (kMaxStagesM1 + slot), round & 1);
          if (ok && lane == 0) issue_item(item + S);
        }
        const unsigned char* f = frag + static_cast<size_t>(8 * c + warp) * kFragBytesPerSb;
        const uint4 f0 = reinterpret_cast<const uint4*>(f)[lane], f1 = reinterpret_cast<const uint4*>(f + 512)[lane];
        const int2 ss = reinterpret_cast<const int2*>(f + 1024)[t];
        const float xs = *reinterpret_cast<const float*>(f + 1024 + 32);
        int d0[4], d1[4];
        mma_first(d0, wA[0].x, wB[0].x, wA[1].x, wB[1].x, make_uint2(f0.x & mlo, f0.x & mhi));
        mma_first(d1, wA[2].x, wB[2].x, wA[3].x, wB[3].x, make_uint2(f1.x & mlo, f1.x & mhi));
        mma_acc(d0, wA[0].y, wB[0].y, wA[1].y, wB[1].y, make_uint2(f0.y & mlo, f0.y & mhi));
        mma_acc(d1, wA[2].y, wB[2].y, wA[3].y, wB[3].y, make_uint2(f1.y & mlo, f1.y & mhi));
        mma_acc(d0, wA[0].x & 0xF0F0F0F0u, wB[0].x & 0xF0F0F0F0u, wA[1].x & 0xF0F0F0F0u, wB[1].x & 0xF0F0F0F0u,
                make_uint2(f0.z & mlo, f0.z & mhi));
        mma_acc(d1, wA[2].x & 0xF0F0F0F0u, wB[2].x & 0xF0F0F0F0u, wA[3].x & 0xF0F0F0F0u, wB[3].x & 0xF0F0F0F0u,
                make_uint2(f1.z & mlo, f1.z & mhi));
        mma_acc(d0, wA[0].y & 0xF0F0F0F0u, wB[0].y & 0xF0F0F0F0u, wA[1].y & 0xF0F0F0F0u, wB[1].y & 0xF0F0F0F0u,
                make_uint2(f0.w & mlo, f0.w & mhi));
        mma_acc(d1, wA[2].y & 0xF0F0F0F0u, wB[2].y & 0xF0F0F0F0u, wA[3].y & 0xF0F0F0F0u, wB[3].y & 0xF0F0F0F0u,
                make_uint2(f1.w & mlo, f1.w & mhi));
        const uint32_t a0 = __byte_perm(hA.y, 0, selb), a1 = __byte_perm(hA.z, 0, selb), a2 = __byte_perm(hA.w, 0, selb);
        const uint32_t b0 = __byte_perm(hB.y, 0, selb), b1 = __byte_perm(hB.z, 0, selb), b2 = __byte_perm(hB.w, 0, selb);
        const int scA0 = a0 & 63, mnA0 = a1 & 63, scA1 = (a2 & 15) | ((a0 >> 2) & 0x30),
                  mnA1 = (a2 >> 4) | ((a1 >> 2) & 0x30);
        const int scB0 = b0 & 63, mnB0 = b1 & 63, scB1 = (b2 & 15) | ((b0 >> 2) & 0x30),
                  mnB1 = (b2 >> 4) | ((b1 >> 2) & 0x30);
        const int hiA = d0[0] * scA0 + d1[0] * scA1, loA = d0[1] * scA0 + d1[1] * scA1;
        const int hiB = d0[2] * scB0 + d1[2] * scB1, loB = d0[3] * scB0 + d1[3] * scB1;
        const int tA = mnA0 * ss.x + mnA1 * ss.y, tB = mnB0 * ss.x + mnB1 * ss.y;
        const float dA = half_bits_to_f32(hA.x), dminA = half_bits_to_f32(hA.x >> 16);
        const float dB = half_bits_to_f32(hB.x), dminB = half_bits_to_f32(hB.x >> 16);
        const float fA = fmaf(static_cast<float>(hiA), 254.f, static_cast<float>(loA));
        const float fB = fmaf(static_cast<float>(hiB), 254.f, static_cast<float>(loB));
        const float xsm = xs * odd16;
        acc0 = fmaf(fA, dA * xsm, acc0);
        acc0 = fmaf(-static_cast<float>(tA), dminA * xs, acc0);
        acc1 = fmaf(fB, dB * xsm, acc1);
        acc1 = fmaf(-static_cast<float>(tB), dminB * xs, acc1);
        if (++slot == S) slot = 0, round++;
      }
      acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 1);
      acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 1);
      acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 2);
      acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 2);
      if (t == 0) {  // later passes add to what this same thread stored in the first
        if (!MULTI || pass == 0)
          red[warp][mt][g] = acc0, red[warp][mt][8 + g] = acc1;
        else
          red[warp][mt][g] += acc0, red[warp][mt][8 + g] += acc1;
      }
    }
    }
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < n_mt * kTileRows) {
      const int mt = threadIdx.x / kTileRows, r = threadIdx.x % kTileRows;
      const int row =
          kTileRows * (static_cast<int>(blockIdx.x) + (b * kBatchTiles + mt) * static_cast<int>(gridDim.x)) + r;
      if (row < N) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kW; w++) tot += red[w][mt][r];
        if (GU) {
          float up = 0.f;
#pragma unroll
          for (int w = 0; w < kW; w++) up += red[w][mt][8 + r];
          if (y_dtype == UB_DTYPE_BF16)
            tot = __bfloat162float(__float2bfloat16_rn(tot)), up = __bfloat162float(__float2bfloat16_rn(up));
          else if (y_dtype == UB_DTYPE_F16)
            tot = __half2float(__float2half_rn(tot)), up = __half2float(__float2half_rn(up));
          tot = __fmul_rn(__fdiv_rn(tot, 1.f + expf(-tot)), up);  // as ub_silu_and_mul computes it
        }
        if (ar.world > 1)
          ar_push(ar, epoch, row, tot);
        else
          st_out(y, row, y_dtype, ar.residual ? tot + __bfloat162float(ar.residual[row]) : tot);
      }
    }
    if (b + 1 < nbatches) __syncthreads();
  }
  if (ar.world > 1) ar_finish(ar, epoch, y, N, err_word);
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

// =====================================================================================================
// Rows beyond 12288 values in ONE pass: one CTA of SIXTEEN warps per SM (up to 224 KB of shared memory), so that
// the fragments of a whole 28672-value row (120 KB) fit beside the ring and every SM quantises the row once
// instead of once per pass and per CTA.  The two halves of the CTA (warps 0-7, 8-15) take the even and the odd
// stages of every tile: half h owns stage c of a tile when c % 2 == h, warp w of it the super-block 8c + w.  A
// stage is consumed by one half only (its empty barrier counts eight arrivals), both halves keep partial sums of
// every tile, the final sum runs over all sixteen warps.  The number of stages per tile and the ring depth are
// both EVEN, so that a ring slot always serves the same half: a half that skipped a round of a slot could not
// tell, from the barrier's phase parity alone, the round it waits for from the one before the skipped one.
// No launch-to-launch overlap on an SM (one CTA fills it); at 130 MB per matrix the hand-over is a few percent.
constexpr int kWideWarps = 16;
constexpr int kWideMaxUnits = 7;  // stages per half: rows up to 28672 values

template <typename XT>
__global__ void __launch_bounds__(kWideWarps * 32, 1)
qgemv_q4k_m1_wide_kernel(const XT* __restrict__ x, void* __restrict__ y, int N, int nch, int y_dtype, int S, int early,
                         int* err_word, const __grid_constant__ CUtensorMap w_map) {
  constexpr int kRowStride = 8 * UB_Q4K_BYTES;  // 1152 = 9 lines
  constexpr int kStageBytes = 16 * kRowStride;
  extern __shared__ __align__(128) unsigned char m1_smem_raw[];
  unsigned char* const sm =
      m1_smem_raw + ((1024u - (static_cast<uint32_t>(__cvta_generic_to_shared(m1_smem_raw)) & 1023u)) & 1023u);
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStagesM1];
  __shared__ float red[kWideWarps][kBatchTiles][16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = warp >> 3, w8 = warp & 7;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(sm));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  unsigned char* const frag = sm + static_cast<size_t>(S) * kStageBytes;  // [nch * 8][kFragBytesPerSb]
  const int total_tiles = (N + 15) / 16;
  const int my_tiles =
      static_cast<int>(blockIdx.x) < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int my_items = my_tiles * nch;
  const int nbatches = (my_tiles + kBatchTiles - 1) / kBatchTiles;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      mb_init(bars_s + 8 * s, 1);
      mb_init(bars_s + 8 * (kMaxStagesM1 + s), 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // item n of this CTA = (tile n / nch, stage n % nch) -> ring slot n % S
  auto issue_item = [&](int n) {
    const int tile = n / nch, c = n - tile * nch;
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

  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- activations of this warp's super-blocks (stages c = half, half + 2, ...; super-block 8c + w8) ----
  {
    Raw8<XT> raw[kWideMaxUnits];
#pragma unroll
    for (int u = 0; u < kWideMaxUnits; u++) {
      const int c = 2 * u + half;
      if (c < nch) raw[u].load(x + static_cast<size_t>(8 * c + w8) * 256 + 8 * lane);
    }
    if (threadIdx.x == 0)
      for (int n = n_early; n < min(S, my_items); n++) issue_item(n);
#pragma unroll
    for (int u = 0; u < kWideMaxUnits; u++) {
      const int c = 2 * u + half;
      if (c >= nch) break;
      float v[8];
      raw[u].unpack(v);
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      const float inv = amax > 0.f ? kXQMaxM1 / amax : 0.f;
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
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
      const uint32_t hvx = pack4_m1(hi[0], hi[1], hi[2], hi[3]), hvy = pack4_m1(hi[4], hi[5], hi[6], hi[7]);
      const uint32_t lvx = pack4_m1(lo[0], lo[1], lo[2], lo[3]), lvy = pack4_m1(lo[4], lo[5], lo[6], lo[7]);
      unsigned char* const f = frag + static_cast<size_t>(8 * c + w8) * kFragBytesPerSb;
#pragma unroll
      for (int q = 0; q < 2; q++) {
        const int src = 4 * (4 * q + (g >> 1)) + t;
        const uint32_t hx = __shfl_sync(0xFFFFFFFFu, hvx, src), hy = __shfl_sync(0xFFFFFFFFu, hvy, src);
        const uint32_t lx = __shfl_sync(0xFFFFFFFFu, lvx, src), ly = __shfl_sync(0xFFFFFFFFu, lvy, src);
        const uint32_t wx = (g & 1) ? lx : hx, wy = (g & 1) ? ly : hy;
        uint4 w4;
        w4.x = (g & 2) ? 0u : wx;
        w4.y = (g & 2) ? 0u : wy;
        w4.z = (g & 2) ? wx : __vneg4(wx);
        w4.w = (g & 2) ? wy : __vneg4(wy);
        reinterpret_cast<uint4*>(f + q * 512)[lane] = w4;
      }
      const int s_lo = __shfl_sync(0xFFFFFFFFu, sum, 4 * t), s_hi = __shfl_sync(0xFFFFFFFFu, sum, 16 + 4 * t);
      if (g == 0) reinterpret_cast<int2*>(f + 1024)[t] = make_int2(s_lo, s_hi);
      if (lane == 0) *reinterpret_cast<float*>(f + 1024 + 32) = amax * (1.f / kXQMaxM1);
    }
    __syncwarp();
  }

  uint32_t off_h, off_q[4];
  {
    auto swz = [](uint32_t L) { return L ^ (((L >> 7) & 7u) << 4); };
    const uint32_t L0 = static_cast<uint32_t>(g * kRowStride + w8 * UB_Q4K_BYTES);
    off_h = swz(L0);
#pragma unroll
    for (int G = 0; G < 4; G++) off_q[G] = swz(L0 + 16 + 32 * G + 8 * t);
  }
  const uint32_t selb = 0x4440u | static_cast<uint32_t>(t);
  const float odd16 = (t & 1) ? 0.0625f : 1.f;
  const uint32_t mlo = g < 4 ? 0xFFFFFFFFu : 0u, mhi = ~mlo;

  bool ok = true;
  for (int b = 0; b < nbatches; b++) {
    const int n_mt = min(kBatchTiles, my_tiles - b * kBatchTiles);
#pragma unroll 1
    for (int mt = 0; mt < n_mt; mt++) {
      float acc0 = 0.f, acc1 = 0.f;
      const int tile = b * kBatchTiles + mt;
#pragma unroll 1
      for (int c = half; c < nch; c += 2) {
        const int item = tile * nch + c, slot = item % S;
        const uint32_t par = static_cast<uint32_t>(item / S) & 1u;
        if (ok) ok = mb_wait(bars_s + 8 * slot, par);
        const unsigned char* rowA = sm + static_cast<size_t>(slot) * kStageBytes;
        const unsigned char* rowB = rowA + 8 * kRowStride;
        const uint4 hA = *reinterpret_cast<const uint4*>(rowA + off_h);
        const uint4 hB = *reinterpret_cast<const uint4*>(rowB + off_h);
        uint2 wA[4], wB[4];
#pragma unroll
        for (int G = 0; G < 4; G++) {
          wA[G] = *reinterpret_cast<const uint2*>(rowA + off_q[G]);
          wB[G] = *reinterpret_cast<const uint2*>(rowB + off_q[G]);
        }
        __syncwarp();
        if (lane == 0) mb_arrive(bars_s + 8 * (kMaxStagesM1 + slot));
        // the warp (item / 2) % 8 of the consuming half re-arms the slot once its eight warps have read it
        if (((item >> 1) & 7) == w8 && item + S < my_items) {
          if (ok) ok = mb_wait(bars_s + 8 * (kMaxStagesM1 + slot), par);
          if (ok && lane == 0) issue_item(item + S);
        }
        const unsigned char* f = frag + static_cast<size_t>(8 * c + w8) * kFragBytesPerSb;
        const uint4 f0 = reinterpret_cast<const uint4*>(f)[lane], f1 = reinterpret_cast<const uint4*>(f + 512)[lane];
        const int2 ss = reinterpret_cast<const int2*>(f + 1024)[t];
        const float xs = *reinterpret_cast<const float*>(f + 1024 + 32);
        int d0[4], d1[4];
        mma_first(d0, wA[0].x, wB[0].x, wA[1].x, wB[1].x, make_uint2(f0.x & mlo, f0.x & mhi));
        mma_first(d1, wA[2].x, wB[2].x, wA[3].x, wB[3].x, make_uint2(f1.x & mlo, f1.x & mhi));
        mma_acc(d0, wA[0].y, wB[0].y, wA[1].y, wB[1].y, make_uint2(f0.y & mlo, f0.y & mhi));
        mma_acc(d1, wA[2].y, wB[2].y, wA[3].y, wB[3].y, make_uint2(f1.y & mlo, f1.y & mhi));
        mma_acc(d0, wA[0].x & 0xF0F0F0F0u, wB[0].x & 0xF0F0F0F0u, wA[1].x & 0xF0F0F0F0u, wB[1].x & 0xF0F0F0F0u,
                make_uint2(f0.z & mlo, f0.z & mhi));
        mma_acc(d1, wA[2].x & 0xF0F0F0F0u, wB[2].x & 0xF0F0F0F0u, wA[3].x & 0xF0F0F0F0u, wB[3].x & 0xF0F0F0F0u,
                make_uint2(f1.z & mlo, f1.z & mhi));
        mma_acc(d0, wA[0].y & 0xF0F0F0F0u, wB[0].y & 0xF0F0F0F0u, wA[1].y & 0xF0F0F0F0u, wB[1].y & 0xF0F0F0F0u,
                make_uint2(f0.w & mlo, f0.w & mhi));
        mma_acc(d1, wA[2].y & 0xF0F0F0F0u, wB[2].y & 0xF0F0F0F0u, wA[3].y & 0xF0F0F0F0u, wB[3].y & 0xF0F0F0F0u,
                make_uint2(f1.w & mlo, f1.w & mhi));
        const uint32_t a0 = __byte_perm(hA.y, 0, selb), a1 = __byte_perm(hA.z, 0, selb), a2 = __byte_perm(hA.w, 0, selb);
        const uint32_t b0 = __byte_perm(hB.y, 0, selb), b1 = __byte_perm(hB.z, 0, selb), b2 = __byte_perm(hB.w, 0, selb);
        const int scA0 = a0 & 63, mnA0 = a1 & 63, scA1 = (a2 & 15) | ((a0 >> 2) & 0x30),
                  mnA1 = (a2 >> 4) | ((a1 >> 2) & 0x30);
        const int scB0 = b0 & 63, mnB0 = b1 & 63, scB1 = (b2 & 15) | ((b0 >> 2) & 0x30),
                  mnB1 = (b2 >> 4) | ((b1 >> 2) & 0x30);
        const int hiA = d0[0] * scA0 + d1[0] * scA1, loA = d0[1] * scA0 + d1[1] * scA1;
        const int hiB = d0[2] * scB0 + d1[2] * scB1, loB = d0[3] * scB0 + d1[3] * scB1;
        const int tA = mnA0 * ss.x + mnA1 * ss.y, tB = mnB0 * ss.x + mnB1 * ss.y;
        const float dA = half_bits_to_f32(hA.x), dminA = half_bits_to_f32(hA.x >> 16);
        const float dB = half_bits_to_f32(hB.x), dminB = half_bits_to_f32(hB.x >> 16);
        const float fA = fmaf(static_cast<float>(hiA), 254.f, static_cast<float>(loA));
        const float fB = fmaf(static_cast<float>(hiB), 254.f, static_cast<float>(loB));
        const float xsm = xs * odd16;
        acc0 = fmaf(fA, dA * xsm, acc0);
        acc0 = fmaf(-static_cast<float>(tA), dminA * xs, acc0);
        acc1 = fmaf(fB, dB * xsm, acc1);
        acc1 = fmaf(-static_cast<float>(tB), dminB * xs, acc1);
      }
      acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 1);
      acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 1);
      acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, 2);
      acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, 2);
      if (t == 0) red[warp][mt][g] = acc0, red[warp][mt][8 + g] = acc1;
    }
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < n_mt * 16) {
      const int mt = threadIdx.x >> 4, r = threadIdx.x & 15;
      const int row = 16 * (static_cast<int>(blockIdx.x) + (b * kBatchTiles + mt) * static_cast<int>(gridDim.x)) + r;
      if (row < N) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kWideWarps; w++) tot += red[w][mt][r];  // fixed order: deterministic
        st_out(y, row, y_dtype, tot);
      }
    }
    if (b + 1 < nbatches) __syncthreads();
  }
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

template <typename XT>
int launch_m1_wide(const uint8_t* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, cudaStream_t s) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ub::tensor_map_encoder());
  if (!enc) return UB_ERR_UNSUPPORTED;
  constexpr int kRowStride = 8 * UB_Q4K_BYTES;
  constexpr int kStageBytes = 16 * kRowStride;
  constexpr size_t kBudget = 222 * 1024;  // one CTA per SM: ring + fragments + 1 KB slack + ~4.5 KB static <= 227 KB
  const int nch = K / 2048;
  if (nch > 2 * kWideMaxUnits || (nch & 1)) return UB_ERR_UNSUPPORTED;
  const size_t frag_bytes = static_cast<size_t>(nch) * 8 * kFragBytesPerSb;
  if (frag_bytes + 4 * static_cast<size_t>(kStageBytes) + 1024 > kBudget) return UB_ERR_UNSUPPORTED;
  int S = static_cast<int>((kBudget - 1024 - frag_bytes) / kStageBytes);
  if (S > kMaxStagesM1) S = kMaxStagesM1;
  S &= ~1;  // even: a slot always serves the same half of the CTA
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
  auto kernel = qgemv_q4k_m1_wide_kernel<XT>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  const int tiles = (N + 15) / 16;
  const int sms = ub::num_sms();
  const int grid = tiles < sms ? tiles : sms;
  const int early = fresh ? 0 : 2;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kWideWarps * 32), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, x, y, N, nch, y_dtype, S, early, ub::device_error_word(), wmap);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::check_launch();
}

template <typename XT, bool GU>
int launch_m1_long(const uint8_t* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, const XT* gamma,
                   float eps, const ArParams& ar, cudaStream_t s) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ub::tensor_map_encoder());
  if (!enc) return UB_ERR_UNSUPPORTED;
  constexpr int kRowStride = 8 * UB_Q4K_BYTES;
  constexpr int kStageBytes = 16 * kRowStride;
  const int nch = K / 2048;
  const int tiles = GU ? (N + 7) / 8 : (N + 15) / 16;
  const int slots = 2 * ub::num_sms();
  const int grid = tiles < slots ? tiles : slots;
  // Rows beyond 12288 values: the activation fragments of a whole row no longer fit beside the ring, so K is
  // consumed in passes of at most four stages whose fragments replace one another (the 28672-wide down
  // projection of a 70B-shaped stack: four passes).  Needs every CTA's tiles to fit one batch, and the
  // whole-row RMSNorm prologue is not available.
  int npass = 1;
  if (nch > kMaxChunks) {
    if (GU || gamma || tiles > kBatchTiles * grid) return UB_ERR_UNSUPPORTED;
    npass = (nch + 3) / 4;
  }
  const int cpp = (nch + npass - 1) / npass;
  const size_t frag_bytes = static_cast<size_t>(cpp) * 8 * kFragBytesPerSb;
  if (frag_bytes + 3 * static_cast<size_t>(kStageBytes) > kRingBudget) return UB_ERR_UNSUPPORTED;
  int S = static_cast<int>((kRingBudget - frag_bytes) / kStageBytes);
  if (S > kMaxStagesM1) S = kMaxStagesM1;
  CUtensorMap wmap;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(K / UB_QK_K) * UB_Q4K_BYTES;
  const cuuint64_t dims[3] = {128, row_bytes / 128, static_cast<cuuint64_t>(GU ? 2 * N : N)};
  const cuuint64_t strides[2] = {128, row_bytes};
  const cuuint32_t box[3] = {128, static_cast<cuuint32_t>(kRowStride / 128), GU ? 8u : 16u};
  const cuuint32_t estr[3] = {1, 1, 1};
  if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(wq), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return UB_ERR_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(S) * kStageBytes + frag_bytes + 1024;
  auto kernel = npass > 1 ? qgemv_q4k_m1_long_kernel<XT, false, true> : qgemv_q4k_m1_long_kernel<XT, GU, false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  const int early = fresh ? 0 : 2;  // 36 KB per CTA ahead of the dependency wait, as in the short-row kernel
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kThreadsM1), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, x, y, N, nch, npass, y_dtype, S, early, ub::device_error_word(), gamma, eps, ar,
                         wmap);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::check_launch();
}

}  // namespace

namespace ub {

// y[N] = dequant(Wq) . x for one token; UB_ERR_UNSUPPORTED (without touching the thread's status) for shapes
// these kernels do not take (K not a multiple of 2048; beyond 12288: more rows than one batch of tiles per CTA, or
// with the RMSNorm prologue; unaligned weights; no tensor-map encoder).
// fresh: the weight bytes may have been written by the kernel launched just before on the same stream.
template <typename XT>
int q4k_gemv_m1x(const void* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, const M1Extras& ex,
                 cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  if (reinterpret_cast<uintptr_t>(w) & 15) return UB_ERR_UNSUPPORTED;
  ArParams none;
  memset(&none, 0, sizeof(none));
  const ArParams& a = ex.ar ? *ex.ar : none;
  const XT* gamma = static_cast<const XT*>(ex.gamma);
  if (K == 4096) return launch_m1<XT, 2>(w, x, y, N, K, y_dtype, fresh, gamma, ex.eps, a, s);
  if (K == 2048) return launch_m1<XT, 1>(w, x, y, N, K, y_dtype, fresh, gamma, ex.eps, a, s);
  if (K % 2048 == 0 && K >= 12288 && !gamma && a.world <= 1 && !a.residual) {
    // one pass, one CTA of sixteen warps per SM (an even number of stages per row); measured on B200 at 8192 rows:
    // 12288 values 13.1 us against 14.1 with two CTAs per SM, 28672 values 30.0 against 35.7 in four passes;
    // at 8192 values the two-CTA kernel is the faster one (11.0 against 12.1 us at 10240 rows)
    const int st = launch_m1_wide<XT>(w, x, y, N, K, y_dtype, fresh, s);
    if (st != UB_ERR_UNSUPPORTED) return st;
  }
  if (K % 2048 == 0) return launch_m1_long<XT, false>(w, x, y, N, K, y_dtype, fresh, gamma, ex.eps, a, s);
  return UB_ERR_UNSUPPORTED;
}

template <typename XT>
int q4k_gemv_m1(const void* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, const ArParams* ar,
                cudaStream_t s) {
  const M1Extras ex = {nullptr, 0.f, ar};
  return q4k_gemv_m1x<XT>(wq, x, y, N, K, y_dtype, fresh, ex, s);
}

// y[N] = silu(Wgate . x) * (Wup . x) for one token, wq = [gate rows; up rows] (2 N rows of K); same contract;
// gamma != null: on rmsnorm(x).
template <typename XT>
int q4k_gemv_m1_gate_up(const void* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, const void* gamma,
                        float eps, cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  if ((reinterpret_cast<uintptr_t>(w) & 15) || K % 2048) return UB_ERR_UNSUPPORTED;
  ArParams none;
  memset(&none, 0, sizeof(none));
  return launch_m1_long<XT, true>(w, x, y, N, K, y_dtype, fresh, static_cast<const XT*>(gamma), eps, none, s);
}

template int q4k_gemv_m1x<float>(const void*, const float*, void*, int, int, int, bool, const M1Extras&, cudaStream_t);
template int q4k_gemv_m1x<__nv_bfloat16>(const void*, const __nv_bfloat16*, void*, int, int, int, bool, const M1Extras&,
                                         cudaStream_t);
template int q4k_gemv_m1<float>(const void*, const float*, void*, int, int, int, bool, const ArParams*, cudaStream_t);
template int q4k_gemv_m1<__nv_bfloat16>(const void*, const __nv_bfloat16*, void*, int, int, int, bool, const ArParams*,
                                        cudaStream_t);
template int q4k_gemv_m1_gate_up<float>(const void*, const float*, void*, int, int, int, bool, const void*, float,
                                        cudaStream_t);
template int q4k_gemv_m1_gate_up<__nv_bfloat16>(const void*, const __nv_bfloat16*, void*, int, int, int, bool, const void*,
                                                float, cudaStream_t);

}  // namespace ub
