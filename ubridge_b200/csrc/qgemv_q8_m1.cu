// Decode matmul for ONE token on Q8_0 weights with K = 2048 or 4096, in the launch-to-launch pipeline of the
// one-token Q4_K kernel (qgemv_m1.cu):
//
//   y[N] = dequant(Wq)[N,K] . x[K]        (f32 accumulation of exact integer dots)
//
// Replaces the reference's dequantise + decode matmul for block_q8_0 weights (kernels/quant.cpp:98-104,
// :188-268; kernels/third_party/matmul_decoding.h:381-552 is its weight-streaming shape).
//
// Structure: two CTAs of eight warps per SM, tiles of EIGHT rows dealt round robin, a ring of three stages (one
// tile each, 34 KB at K = 4096) that the warp `tile mod 8` re-arms, programmatic dependent launch with the first
// stage requested ahead of the dependency wait, every wait bounded.
//
// MMA arrangement.  A block's 32 signed bytes are the A operand of mma.sync.m16n8k32 (s8 x s8 -> s32) as they
// lie in memory.  With one token only two of the eight B columns would carry data (the two limbs of the
// activations, q = 254 hi + lo per 32-value block), so the sixteen A rows are not sixteen weight rows but eight
// weight rows TWICE: rows 0-7 hold a block of the first half of K, rows 8-15 the block 1/2 K further of the same
// weight rows, and columns 0, 1 carry the activations of the first block, columns 2, 3 those of the second.
// Lane t = 0 of a quad then holds the first block's dots of row g (accumulators 0, 1), lane t = 1 the second
// block's (accumulators 2, 3); the cross products are not used.  One instruction covers 8 rows x 64 weights.
// A stage is stored as boxes of [8 rows][17 lines of 128 bytes] (64 blocks of a row each), so that the eight rows
// a quarter-warp reads fall into distinct 128-byte swizzle phases.  In every other block the weight bytes start
// two bytes after a word boundary: those are read as three aligned words and funnel shifted.
#include <cuda.h>  // CUtensorMap type and enums only; the encoder is resolved at run time

#include <string.h>

#include "common.cuh"

namespace ub {
void* tensor_map_encoder();
}

namespace {

using namespace ub;

constexpr int kW = 8;
constexpr int kThreads = kW * 32;
constexpr int kStages = 3;
constexpr int kBatchTiles = 4;
constexpr uint32_t kSpin = 400000;
constexpr float kXQMax = 32258.f;         // 127 * 254
constexpr int kBoxRowBytes = 64 * UB_Q8_0_BYTES;  // 2176 = 17 lines
constexpr int kBoxBytes = 8 * kBoxRowBytes;       // 17408

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
// d = A(16x32 s8, row) . B(32x8 s8, col)
__device__ __forceinline__ void mma_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "r"(0));
}
__device__ __forceinline__ uint32_t pack4b(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
__device__ __forceinline__ uint32_t swz128(uint32_t L) { return L ^ (((L >> 7) & 7u) << 4); }

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

// NBOX: 64-block boxes per row = K / 2048 (1 or 2).  Blocks per row NB = 64 NBOX, the two halves of K are
// blocks [0, NB/2) and [NB/2, NB); warp w owns BPW = NB / 16 blocks of each half: w BPW + i and NB/2 + w BPW + i.
template <typename XT, int NBOX, int NB = 64 * NBOX, int BPW = NB / 16, int U = BPW / 4>  // U: 256-value units per warp
__global__ void __launch_bounds__(kThreads, 2)
qgemv_q8_0_m1_kernel(const XT* __restrict__ x, void* __restrict__ y, int N, int y_dtype, int early, int* err_word,
                     const __grid_constant__ CUtensorMap w_map) {
  constexpr int kStageBytes = NBOX * kBoxBytes;
  extern __shared__ __align__(128) unsigned char q8_smem_raw[];
  // swizzled stages need 1024-byte alignment; the launch reserves 1 KB of slack for rounding the base up
  unsigned char* const sm =
      q8_smem_raw + ((1024u - (static_cast<uint32_t>(__cvta_generic_to_shared(q8_smem_raw)) & 1023u)) & 1023u);
  __shared__ __align__(8) unsigned long long bars[2 * kStages];  // full[S], empty[S]
  __shared__ float red[kW][kBatchTiles][8];
  __shared__ __align__(16) uint4 xlimbs[kW][U][32];  // per warp: packed activation limbs of its own blocks
  __shared__ float xscale[kW][2 * BPW];              // and their block scales, in list order
  __shared__ __align__(8) uint2 xzero[kW];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(sm));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  const int total_tiles = (N + 7) >> 3;
  const int my_tiles =
      static_cast<int>(blockIdx.x) < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int nbatches = (my_tiles + kBatchTiles - 1) / kBatchTiles;

  // The next kernel in the stream may start as soon as every CTA of this grid has passed this point.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      mb_init(bars_s + 8 * s, 1);
      mb_init(bars_s + 8 * (kStages + s), kW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // tile n of this CTA -> ring slot n % kStages: NBOX copies of 8 rows x 17 lines; rows past N arrive as zeros
  auto issue_tile = [&](int n) {
    const uint32_t full = bars_s + 8 * (n % kStages);
    const int row0 = 8 * (static_cast<int>(blockIdx.x) + n * static_cast<int>(gridDim.x));
    mb_expect_tx(full, kStageBytes);
#pragma unroll
    for (int bx = 0; bx < NBOX; bx++)
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::
              "r"(ring_s + (n % kStages) * kStageBytes + bx * kBoxBytes),
          "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(full), "r"(0), "r"(bx * (kBoxRowBytes >> 7)), "r"(row0)
          : "memory");
  };
  const int n_early = min(min(early, kStages), my_tiles);
  if (threadIdx.x == 0)
    for (int n = 0; n < n_early; n++) issue_tile(n);

  // everything below reads what the previous kernel may have written (x) or writes what it may still read (y)
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- activations of this warp's 2 BPW blocks -> B fragments and block scales in registers ----
  // The warp's blocks as a list: entries 0 .. BPW-1 = first-half blocks w BPW + i, entries BPW .. = second-half
  // blocks NB/2 + w BPW + i.  Unit u, lane l holds values 8 (l % 4) .. + 7 of list entry 8u + l / 4.
  uint2 bf[BPW];   // B fragment of MMA i
  float xsc[BPW];  // activation block scale this lane needs for MMA i (t = 0: first block, t = 1: second block)
  {
    Raw8<XT> raw[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int e = 8 * u + (lane >> 2);
      const int blk = e < BPW ? warp * BPW + e : NB / 2 + warp * BPW + (e - BPW);
      raw[u].load(x + static_cast<size_t>(blk) * 32 + 8 * (lane & 3));
    }
    // the rest of the ring goes out right behind the activation loads
    if (threadIdx.x == 0)
      for (int n = n_early; n < min(kStages, my_tiles); n++) issue_tile(n);
    // Each warp parks the packed limbs of its own units in shared memory (nobody else reads them, so a warp-level
    // barrier is all it takes) and every lane then picks up its B fragments with one load per MMA: shuffling them
    // into place cost ten shuffles and as many selects per MMA, and sixteen warps per SM do this at once while
    // the whole launch waits for it.
#pragma unroll
    for (int u = 0; u < U; u++) {
      float v[8];
      raw[u].unpack(v);
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));  // over the block's four lanes
      const float inv = amax > 0.f ? kXQMax / amax : 0.f;
      // Round through the mantissa of 1.5 * 2^23.  q = rint(v inv); hi = rint(v inv / 254) differs from
      // rint(q / 254) only where q / 254 is within 0.002 of a half, and there both choices leave |lo| <= 127.
      const float inv254 = inv * (1.f / 254.f);
      int hi[8], lo[8];
#pragma unroll
      for (int e = 0; e < 8; e++) {
        const int q = __float_as_int(fmaf(v[e], inv, 12582912.f)) - 0x4B400000;
        hi[e] = __float_as_int(fmaf(v[e], inv254, 12582912.f)) - 0x4B400000;
        lo[e] = q - 254 * hi[e];
      }
      // [unit][lane] = {high limbs 0-3, high 4-7, low 0-3, low 4-7} of values 8 (lane % 4) .. of entry 8u + lane / 4
      xlimbs[warp][u][lane] = make_uint4(pack4b(hi[0], hi[1], hi[2], hi[3]), pack4b(hi[4], hi[5], hi[6], hi[7]),
                                         pack4b(lo[0], lo[1], lo[2], lo[3]), pack4b(lo[4], lo[5], lo[6], lo[7]));
      if ((lane & 3) == 0) xscale[warp][8 * u + (lane >> 2)] = amax * (1.f / kXQMax);
    }
    if (lane == 0) xzero[warp] = make_uint2(0, 0);
    __syncwarp();
    // B fragment of MMA i, lane (column g, t): column 0 / 1 = high / low limb of list entry i, column 2 / 3 of
    // entry BPW + i, columns 4-7 zero; values 8t .. 8t+7 of entry e sit in lane 4 (e % 8) + t of unit e / 8.
    // Entries i and BPW + i are 64 bytes times i apart from entries 0 and BPW: one base address per lane.
    {
      const int e0 = (g & 2) ? BPW : 0;
      const unsigned char* fb = g < 4 ? reinterpret_cast<const unsigned char*>(&xlimbs[warp][e0 >> 3][4 * (e0 & 7) + t]) +
                                            8 * (g & 1)
                                      : reinterpret_cast<const unsigned char*>(&xzero[warp]);
      const int fstep = g < 4 ? 64 : 0;
      const float* sb = &xscale[warp][t == 0 ? 0 : BPW];
#pragma unroll
      for (int i = 0; i < BPW; i++) {
        bf[i] = *reinterpret_cast<const uint2*>(fb + i * fstep);
        xsc[i] = sb[i];
      }
    }
  }

  // Byte offsets inside a stage of what this lane reads for MMA i: row g, first-half block (accumulator rows 0-7)
  // and second-half block (rows 8-15); lanes t >= 2 read too (their k slices of the A operand) but hold no useful
  // accumulators, they take the first block's scale.
  auto block_off = [&](int blk) {  // byte offset of block `blk` of row g inside the stage (before the swizzle)
    return static_cast<uint32_t>((blk >> 6) * kBoxBytes + g * kBoxRowBytes + (blk & 63) * UB_Q8_0_BYTES);
  };
  const int b1_0 = warp * BPW, b2_0 = NB / 2 + warp * BPW;

  bool ok = true;
  int slot = 0, round = 0, tile = 0;
  for (int b = 0; b < nbatches; b++) {
    const int n_mt = min(kBatchTiles, my_tiles - b * kBatchTiles);
#pragma unroll 1
    for (int mt = 0; mt < n_mt; mt++, tile++) {
      if (ok) ok = mb_wait(bars_s + 8 * slot, round & 1);
      const unsigned char* st = sm + static_cast<size_t>(slot) * kStageBytes;
      uint32_t a[BPW][4];
      float dw[BPW];
#pragma unroll
      for (int i = 0; i < BPW; i++) {
        const uint32_t L1 = block_off(b1_0 + i), L2 = block_off(b2_0 + i);
        dw[i] = half_bits_to_f32(*reinterpret_cast<const unsigned short*>(st + swz128(t == 1 ? L2 : L1)));
        // the 32 weight bytes of a block start at L + 2; this lane takes bytes 8t .. 8t+7 of them.
        // (b1_0 + i) and (b2_0 + i) have the parity of i: BPW and NB/2 are even.
        if (i & 1) {  // 34 blk + 2 is a multiple of 4 for odd blocks: aligned words
          a[i][0] = *reinterpret_cast<const uint32_t*>(st + swz128(L1 + 2 + 8 * t));
          a[i][2] = *reinterpret_cast<const uint32_t*>(st + swz128(L1 + 6 + 8 * t));
          a[i][1] = *reinterpret_cast<const uint32_t*>(st + swz128(L2 + 2 + 8 * t));
          a[i][3] = *reinterpret_cast<const uint32_t*>(st + swz128(L2 + 6 + 8 * t));
        } else {  // two bytes past a word boundary: three words, funnel shifted by 16 bits
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(st + swz128(L1 + 8 * t));
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(st + swz128(L1 + 4 + 8 * t));
          const uint32_t w2 = *reinterpret_cast<const uint32_t*>(st + swz128(L1 + 8 + 8 * t));
          a[i][0] = __funnelshift_r(w0, w1, 16), a[i][2] = __funnelshift_r(w1, w2, 16);
          const uint32_t v0 = *reinterpret_cast<const uint32_t*>(st + swz128(L2 + 8 * t));
          const uint32_t v1 = *reinterpret_cast<const uint32_t*>(st + swz128(L2 + 4 + 8 * t));
          const uint32_t v2 = *reinterpret_cast<const uint32_t*>(st + swz128(L2 + 8 + 8 * t));
          a[i][1] = __funnelshift_r(v0, v1, 16), a[i][3] = __funnelshift_r(v1, v2, 16);
        }
      }
      // everything this warp needs from the stage is in registers: hand the slot back (the arrive is a
      // release, so the loads above are performed before the re-arming warp sees it)
      __syncwarp();
      if (lane == 0) mb_arrive(bars_s + 8 * (kStages + slot));
      if ((tile & (kW - 1)) == warp && tile + kStages < my_tiles) {
        if (ok) ok = mb_wait(bars_s + 8 * (kStages + slot), round & 1);
        if (ok && lane == 0) issue_tile(tile + kStages);
      }
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < BPW; i++) {
        int d[4];
        mma_s8s8(d, a[i][0], a[i][1], a[i][2], a[i][3], bf[i]);
        // t = 0: row g x first block = columns 0, 1 of accumulator rows 0-7; t = 1: second block = columns 2, 3
        // of rows 8-15 (this lane's columns 2t, 2t+1)
        const int hi = t == 1 ? d[2] : d[0], lo = t == 1 ? d[3] : d[1];
        acc = fmaf(static_cast<float>(hi * 254 + lo), dw[i] * xsc[i], acc);
      }
      if (t >= 2) acc = 0.f;  // cross products and zero columns
      acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
      if (t == 0) red[warp][mt][g] = acc;
      if (++slot == kStages) slot = 0, round++;
    }
    __syncthreads();  // partial sums of the batch are complete
    if (static_cast<int>(threadIdx.x) < n_mt * 8) {
      const int mt = threadIdx.x >> 3, r = threadIdx.x & 7;
      const int row = 8 * (static_cast<int>(blockIdx.x) + (b * kBatchTiles + mt) * static_cast<int>(gridDim.x)) + r;
      if (row < N) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kW; w++) tot += red[w][mt][r];  // fixed order: deterministic
        st_out(y, row, y_dtype, tot);
      }
    }
    if (b + 1 < nbatches) __syncthreads();  // before the next batch overwrites the partial sums
  }
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

template <typename XT, int NBOX>
int launch_q8_m1(const uint8_t* wq, const XT* x, void* y, int N, int y_dtype, bool fresh, cudaStream_t s) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ub::tensor_map_encoder());
  if (!enc) return UB_ERR_UNSUPPORTED;
  constexpr int kStageBytes = NBOX * kBoxBytes;
  CUtensorMap wmap;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(NBOX) * kBoxRowBytes;
  const cuuint64_t dims[3] = {128, row_bytes / 128, static_cast<cuuint64_t>(N)};
  const cuuint64_t strides[2] = {128, row_bytes};
  const cuuint32_t box[3] = {128, static_cast<cuuint32_t>(kBoxRowBytes / 128), 8u};
  const cuuint32_t estr[3] = {1, 1, 1};
  if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(wq), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return UB_ERR_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(kStages) * kStageBytes + 1024;
  auto kernel = qgemv_q8_0_m1_kernel<XT, NBOX>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  const int tiles = (N + 7) / 8;
  const int slots = 2 * ub::num_sms();
  const int grid = tiles < slots ? tiles : slots;
  // Stages requested ahead of the dependency wait.  Measured on B200 at K = 4096 with one / two: 4096 rows (1.7 tiles
  // per CTA) 4.81 / 5.69 us, 8192 rows (3.5) 7.03 / 7.54 us, 10240 rows (4.3) 8.45 / 8.04 us, 14336 rows (6.1)
  // 10.86 / 9.97 us (0.96 of the measured copy bandwidth): a second one pays from four tiles per CTA on.
  const int early = fresh ? 0 : (tiles >= 4 * grid ? 2 : 1);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, x, y, N, y_dtype, early, ub::device_error_word(), wmap);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::check_launch();
}

}  // namespace

namespace ub {

// y[N] = dequant(Wq) . x for one token of Q8_0; UB_ERR_UNSUPPORTED (without touching the thread's status) for
// what this kernel does not take (K other than 2048 / 4096, weights not 16-byte aligned, no tensor-map encoder).
// fresh: the weight bytes may have been written by the kernel launched just before on the same stream.
template <typename XT>
int q8_0_gemv_m1(const void* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  if (reinterpret_cast<uintptr_t>(w) & 15) return UB_ERR_UNSUPPORTED;
  if (K == 4096) return launch_q8_m1<XT, 2>(w, x, y, N, y_dtype, fresh, s);
  if (K == 2048) return launch_q8_m1<XT, 1>(w, x, y, N, y_dtype, fresh, s);
  return UB_ERR_UNSUPPORTED;
}

template int q8_0_gemv_m1<float>(const void*, const float*, void*, int, int, int, bool, cudaStream_t);
template int q8_0_gemv_m1<__nv_bfloat16>(const void*, const __nv_bfloat16*, void*, int, int, int, bool, cudaStream_t);

}  // namespace ub
