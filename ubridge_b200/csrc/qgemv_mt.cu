// Decode matmul for TWO TO FOUR tokens on Q4_K weights with K = 2048 or 4096, in the launch-to-launch pipeline
// of the one-token kernel (qgemv_m1.cu):
//
//   y[M,N] = x[M,K] . dequant(Wq)[N,K]^T        (f32 accumulation of exact integer dots)
//
// Replaces the reference's LHS-resident decode matmul (kernels/matmul.cpp:1197-1208,
// kernels/third_party/matmul_decoding.h:381-552) for GGUF Q4_K weights (kernels/quant.cpp:145-150, :356-363) at
// small batch.
//
// Structure as in the one-token kernel: two CTAs of eight warps per SM, 16-row tiles dealt round robin, a ring of
// 18 KB stages (16 rows x 8 super-blocks, one swizzled tensor-map copy each) that the warp `item mod 8` re-arms,
// programmatic dependent launch with the first two stages requested ahead of the dependency wait, every wait
// bounded.  Warp w owns super-block 8c + w of every stage c.
//
// Token arrangement.  Tokens ride in the MMA columns in pairs: a token takes four of the eight columns of
// mma.sync.m16n8k32 (u8 x s8 -> s32), {x(2G) high limb, x(2G) low limb, x(2G+1) high limb, x(2G+1) low limb} for
// the 64-value group G whose 32 bytes are the A operand.  Two products per group share that B operand:
//       d1 = raw bytes  . B        d2 = (raw & 0xF0) . B
// Columns 0, 1 of a token then give sum(lo . x(2G)) = d1 - d2, columns 2, 3 give 16 sum(hi . x(2G+1)) = d2 (what
// d1 holds there is not used).  The sign and the choice are folded into the integer multiply with the 6-bit
// scales that follows anyway (two multiply-adds per accumulator with scale factors {s, -s} or {0, s} by lane), so
// one fragment set per token pair serves both products: 1 KB per (pair, super-block) in shared memory, written
// once per launch by the warp that owns the super-block and read back only by it (no CTA-wide barrier before the
// main loop).  Activations are quantised to 15-bit block fixed point per 256 values (q = 254 hi + lo).
#include <cuda.h>  // CUtensorMap type and enums only; the encoder is resolved at run time

#include <string.h>

#include "common.cuh"

namespace ub {
void* tensor_map_encoder();
}

namespace {

using namespace ub;

constexpr int kW = 8;  // warps per CTA, all of them compute
constexpr int kThreads = kW * 32;
constexpr int kMaxStages = 8;
constexpr int kBatchTiles = 4;  // tiles whose row sums are added across warps at once
constexpr uint32_t kSpin = 400000;
constexpr float kXQMax = 32258.f;  // 127 * 254
// two CTAs per SM: 2 x (ring + fragments + 1 KB slack + ~9 KB static + 1 KB reserved) <= 228 KB
constexpr size_t kDynBudget = 103 * 1024;
constexpr int kRowStride = 8 * UB_Q4K_BYTES;  // 1152 = 9 lines of 128 bytes
constexpr int kStageBytes = 16 * kRowStride;  // 18 KB
constexpr int kFragPair = 1024 + 64;          // per (pair, super-block): uint2 P[4 groups][32 lanes], uint4 meta[4]

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
__device__ __forceinline__ uint32_t pack4b(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
__device__ __forceinline__ int dp4a_us(uint32_t a_u8x4, uint32_t b_s8x4, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
  return d;
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

__device__ __forceinline__ void st_out(void* y, size_t idx, int dtype, float v) {
  if (dtype == UB_DTYPE_F32)
    static_cast<float*>(y)[idx] = v;
  else if (dtype == UB_DTYPE_BF16)
    static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
  else
    static_cast<__half*>(y)[idx] = __float2half_rn(v);
}

// MP: token pairs per launch (M <= 2 MP; tokens the launch does not have multiply by zero).
// NCH: stages per tile = K / 2048.
template <typename XT, int MP, int NCH>
__global__ void __launch_bounds__(kThreads, 2)
qgemv_q4k_mt_kernel(const XT* __restrict__ x, void* __restrict__ y, int M, int N, int y_dtype, int S, int early,
                    int* err_word, const __grid_constant__ CUtensorMap w_map) {
  constexpr int K = 2048 * NCH;
  extern __shared__ __align__(128) unsigned char mt_smem_raw[];
  // swizzled stages need 1024-byte alignment; the launch reserves 1 KB of slack for rounding the base up
  unsigned char* const sm =
      mt_smem_raw + ((1024u - (static_cast<uint32_t>(__cvta_generic_to_shared(mt_smem_raw)) & 1023u)) & 1023u);
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages];  // full[S], empty[S]
  __shared__ float red[kW][kBatchTiles][2 * MP][16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3, par = t & 1;
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(sm));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  unsigned char* const frag = sm + static_cast<size_t>(S) * kStageBytes;  // [MP][8 NCH][kFragPair]
  const int total_tiles = (N + 15) >> 4;
  const int my_tiles =
      static_cast<int>(blockIdx.x) < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int my_items = my_tiles * NCH;
  const int nbatches = (my_tiles + kBatchTiles - 1) / kBatchTiles;

  // The next kernel in the stream may start as soon as every CTA of this grid has passed this point.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      mb_init(bars_s + 8 * s, 1);
      mb_init(bars_s + 8 * (kMaxStages + s), kW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

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

  // ---- activations of this warp's super-blocks (8c + warp), every token -> fragments in shared memory ----
  {
    Raw8<XT> raw[2 * MP][NCH];
#pragma unroll
    for (int m = 0; m < 2 * MP; m++)
#pragma unroll
      for (int c = 0; c < NCH; c++) {
        if (m < M)
          raw[m][c].load(x + static_cast<size_t>(m) * K + static_cast<size_t>(8 * c + warp) * 256 + 8 * lane);
      }
    // the rest of the ring goes out right behind the activation loads
    if (threadIdx.x == 0)
      for (int n = n_early; n < min(S, my_items); n++) issue_item(n);
    const int j = lane >> 2, G = j >> 1;  // this lane holds values 8t .. 8t+7 of sub-block j
#pragma unroll
    for (int m = 0; m < 2 * MP; m++)
#pragma unroll
      for (int c = 0; c < NCH; c++) {
        unsigned char* const f = frag + (static_cast<size_t>(m >> 1) * (8 * NCH) + 8 * c + warp) * kFragPair;
        // B fragment of group G: lane (column, t) holds k rows 4t..4t+3 and 16+4t..; this token's columns are
        // 4 (m & 1) + {0, 1} for its even sub-block (high, low limb) and + {2, 3} for the odd one
        uint2* const P = reinterpret_cast<uint2*>(f) + G * 32 + (4 * (m & 1) + 2 * (j & 1)) * 4 + t;
        // sub-block sums for the min term: three byte limbs (top one signed) of sub-block j in byte j % 4 of
        // the words x, y, z of entry 2 (m & 1) + j / 4; w = the block scale
        unsigned char* const meta = f + 1024 + (2 * (m & 1) + (j >> 2)) * 16;
        if (m >= M) {  // a token this launch does not have: its columns multiply by zero
          P[0] = P[4] = make_uint2(0, 0);
          if (t == 0) meta[j & 3] = meta[4 + (j & 3)] = meta[8 + (j & 3)] = 0;
          if ((lane & 15) == 0) *reinterpret_cast<float*>(meta + 12) = 0.f;
          continue;
        }
        float v[8];
        raw[m][c].unpack(v);
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
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);  // sum of q over this lane's 32-value sub-block
        P[0] = make_uint2(pack4b(hi[0], hi[1], hi[2], hi[3]), pack4b(hi[4], hi[5], hi[6], hi[7]));
        P[4] = make_uint2(pack4b(lo[0], lo[1], lo[2], lo[3]), pack4b(lo[4], lo[5], lo[6], lo[7]));
        if (t == 0) {
          meta[j & 3] = static_cast<unsigned char>(sum);
          meta[4 + (j & 3)] = static_cast<unsigned char>(sum >> 8);
          meta[8 + (j & 3)] = static_cast<unsigned char>(sum >> 16);
        }
        if ((lane & 15) == 0) *reinterpret_cast<float*>(meta + 12) = amax * (1.f / kXQMax);
      }
    __syncwarp();
  }

  // byte offsets of this lane's header and nibble pieces inside a stage (row g, super-block `warp`); the 16-byte
  // unit index is XORed with the 128-byte line index modulo 8 (the copy's swizzle).  Row g + 8 lies a multiple
  // of 8 lines further and shares the offsets.
  uint32_t off_h, off_q[4];
  {
    auto swz = [](uint32_t L) { return L ^ (((L >> 7) & 7u) << 4); };
    const uint32_t L0 = static_cast<uint32_t>(g * kRowStride + warp * UB_Q4K_BYTES);
    off_h = swz(L0);
#pragma unroll
    for (int G = 0; G < 4; G++) off_q[G] = swz(L0 + 16 + 32 * G + 8 * t);
  }

  bool ok = true;
  int slot = 0, round = 0, item = 0;
  for (int b = 0; b < nbatches; b++) {
    const int n_mt = min(kBatchTiles, my_tiles - b * kBatchTiles);
#pragma unroll 1
    for (int mt = 0; mt < n_mt; mt++) {
      float acc[MP][2];
#pragma unroll
      for (int p = 0; p < MP; p++) acc[p][0] = acc[p][1] = 0.f;
#pragma unroll 1
      for (int c = 0; c < NCH; c++, item++) {
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
        // everything this warp needs from the stage is in registers: hand the slot back (the arrive is a
        // release, so the loads above are performed before the re-arming warp sees it)
        __syncwarp();
        if (lane == 0) mb_arrive(bars_s + 8 * (kMaxStages + slot));
        if ((item & (kW - 1)) == warp && item + S < my_items) {
          if (ok) ok = mb_wait(bars_s + 8 * (kMaxStages + slot), round & 1);
          if (ok && lane == 0) issue_item(item + S);
        }
        // 6-bit scales and mins (kernels/quant.cpp:356-363): four per word; this lane's columns belong to
        // sub-blocks 2G + par (scales brought to bytes 0 and 2) and to sub-blocks 4 par .. 4 par + 3 for the mins
        uint32_t scA[2], mnA[2], scB[2], mnB[2];
        q4k_unpack_scales(hA.y, hA.z, hA.w, scA[0], scA[1], mnA[0], mnA[1]);
        q4k_unpack_scales(hB.y, hB.z, hB.w, scB[0], scB[1], mnB[0], mnB[1]);
        scA[0] >>= 8 * par, scA[1] >>= 8 * par, scB[0] >>= 8 * par, scB[1] >>= 8 * par;
        const uint32_t mA = par ? mnA[1] : mnA[0], mB = par ? mnB[1] : mnB[0];
        const float dA = half_bits_to_f32(hA.x), dminA = half_bits_to_f32(hA.x >> 16);
        const float dB = half_bits_to_f32(hB.x), dminB = half_bits_to_f32(hB.x >> 16);
        // factors of d1 and d2 per group: even sub-blocks take d1 - d2, odd ones d2
        int s1A[4], s2A[4], s1B[4], s2B[4];
#pragma unroll
        for (int G = 0; G < 4; G++) {
          const int sa = (G & 1) ? __byte_perm(scA[G >> 1], 0, 0x4442) : (scA[G >> 1] & 0xFF);
          const int sb = (G & 1) ? __byte_perm(scB[G >> 1], 0, 0x4442) : (scB[G >> 1] & 0xFF);
          s1A[G] = par ? 0 : sa, s2A[G] = par ? sa : -sa;
          s1B[G] = par ? 0 : sb, s2B[G] = par ? sb : -sb;
        }
        const unsigned char* fbase = frag + static_cast<size_t>(8 * c + warp) * kFragPair;
#pragma unroll
        for (int p = 0; p < MP; p++) {
          const unsigned char* f = fbase + static_cast<size_t>(p) * (8 * NCH) * kFragPair;
          uint2 bq[4];
#pragma unroll
          for (int G = 0; G < 4; G++) bq[G] = reinterpret_cast<const uint2*>(f)[G * 32 + lane];
          const uint4 mt4 = reinterpret_cast<const uint4*>(f + 1024)[t];
          int d1[4][4], d2[4][4];
#pragma unroll
          for (int G = 0; G < 4; G++) mma_u8s8(d1[G], wA[G].x, wB[G].x, wA[G].y, wB[G].y, bq[G]);
#pragma unroll
          for (int G = 0; G < 4; G++)
            mma_u8s8(d2[G], wA[G].x & 0xF0F0F0F0u, wB[G].x & 0xF0F0F0F0u, wA[G].y & 0xF0F0F0F0u,
                     wB[G].y & 0xF0F0F0F0u, bq[G]);
          // columns 2t, 2t+1 of rows g (d[0], d[1]) and g + 8 (d[2], d[3]): high and low limb
          int hiA = 0, loA = 0, hiB = 0, loB = 0;
#pragma unroll
          for (int G = 0; G < 4; G++) {
            hiA += d1[G][0] * s1A[G] + d2[G][0] * s2A[G];
            loA += d1[G][1] * s1A[G] + d2[G][1] * s2A[G];
            hiB += d1[G][2] * s1B[G] + d2[G][2] * s2B[G];
            loB += d1[G][3] * s1B[G] + d2[G][3] * s2B[G];
          }
          const float xs = __uint_as_float(mt4.w);
          const float xsm = par ? xs * 0.0625f : xs;  // odd lanes carry 16 x the high nibbles
          const int tA = (dp4a_us(mA, mt4.z, 0) * 256 + static_cast<int>(__dp4a(mA, mt4.y, 0u))) * 256 +
                         static_cast<int>(__dp4a(mA, mt4.x, 0u));
          const int tB = (dp4a_us(mB, mt4.z, 0) * 256 + static_cast<int>(__dp4a(mB, mt4.y, 0u))) * 256 +
                         static_cast<int>(__dp4a(mB, mt4.x, 0u));
          const float fA = fmaf(static_cast<float>(hiA), 254.f, static_cast<float>(loA));
          const float fB = fmaf(static_cast<float>(hiB), 254.f, static_cast<float>(loB));
          acc[p][0] += fmaf(dA * xsm, fA, -(dminA * xs) * static_cast<float>(tA));
          acc[p][1] += fmaf(dB * xsm, fB, -(dminB * xs) * static_cast<float>(tB));
        }
        if (++slot == S) slot = 0, round++;
      }
      // the two lanes of a (row, token) pair hold its even and odd sub-blocks
#pragma unroll
      for (int p = 0; p < MP; p++)
#pragma unroll
        for (int rs = 0; rs < 2; rs++) {
          const float v = acc[p][rs] + __shfl_xor_sync(0xFFFFFFFFu, acc[p][rs], 1);
          if (par == 0) red[warp][mt][2 * p + (t >> 1)][8 * rs + g] = v;
        }
    }
    __syncthreads();  // partial sums of the batch are complete
    for (int o = threadIdx.x; o < n_mt * 16 * 2 * MP; o += kThreads) {
      const int mt = o / (32 * MP), rem = o - mt * (32 * MP), tok = rem >> 4, r = rem & 15;
      const int row = 16 * (static_cast<int>(blockIdx.x) + (b * kBatchTiles + mt) * static_cast<int>(gridDim.x)) + r;
      if (row < N && tok < M) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kW; w++) tot += red[w][mt][tok][r];  // fixed order: deterministic
        st_out(y, static_cast<size_t>(tok) * N + row, y_dtype, tot);
      }
    }
    if (b + 1 < nbatches) __syncthreads();  // before the next batch overwrites the partial sums
  }
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

template <typename XT, int MP, int NCH>
int launch_mt(const uint8_t* wq, const XT* x, void* y, int M, int N, int y_dtype, bool fresh, cudaStream_t s) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ub::tensor_map_encoder());
  if (!enc) return UB_ERR_UNSUPPORTED;
  constexpr int K = 2048 * NCH;
  constexpr size_t frag_bytes = static_cast<size_t>(MP) * 8 * NCH * kFragPair;
  static_assert(frag_bytes + 3 * static_cast<size_t>(kStageBytes) + 1024 <= kDynBudget, "shared-memory plan");
  int S = static_cast<int>((kDynBudget - 1024 - frag_bytes) / kStageBytes);
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
  auto kernel = qgemv_q4k_mt_kernel<XT, MP, NCH>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  const int tiles = (N + 15) / 16;
  const int slots = 2 * ub::num_sms();
  const int grid = tiles < slots ? tiles : slots;
  const int early = fresh ? 0 : 2;  // 36 KB per CTA ahead of the dependency wait, as in the one-token kernel
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, x, y, M, N, y_dtype, S, early, ub::device_error_word(), wmap);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::check_launch();
}

}  // namespace

namespace ub {

// y[M,N] = x[M,K] . dequant(Wq)^T for two to four tokens; UB_ERR_UNSUPPORTED (without touching the thread's
// status) for what this kernel does not take (other M, K other than 2048 / 4096, unaligned weights, no tensor-map
// encoder).  fresh: the weight bytes may have been written by the kernel launched just before on the same stream.
template <typename XT>
int q4k_gemv_mt(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  if (M < 2 || M > 4 || (reinterpret_cast<uintptr_t>(w) & 15)) return UB_ERR_UNSUPPORTED;
  if (K == 4096)
    return M <= 2 ? launch_mt<XT, 1, 2>(w, x, y, M, N, y_dtype, fresh, s)
                  : launch_mt<XT, 2, 2>(w, x, y, M, N, y_dtype, fresh, s);
  if (K == 2048)
    return M <= 2 ? launch_mt<XT, 1, 1>(w, x, y, M, N, y_dtype, fresh, s)
                  : launch_mt<XT, 2, 1>(w, x, y, M, N, y_dtype, fresh, s);
  return UB_ERR_UNSUPPORTED;
}

template int q4k_gemv_mt<float>(const void*, const float*, void*, int, int, int, int, bool, cudaStream_t);
template int q4k_gemv_mt<__nv_bfloat16>(const void*, const __nv_bfloat16*, void*, int, int, int, int, bool,
                                        cudaStream_t);

}  // namespace ub
