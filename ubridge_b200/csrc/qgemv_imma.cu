// Decode GEMV / small-batch matmul for Q4_K weights on the integer tensor-core path.
//
//   y[M,N] = x[M,K] . dequant(Wq)^T   for M <= 8 tokens per launch, f32 accumulation of exact integer dots.
//
// Replaces the reference's LHS-resident decode matmul (kernels/matmul.cpp:1197-1208,
// kernels/third_party/matmul_decoding.h:12-570) for GGUF Q4_K weights (block layout kernels/quant.cpp:145-150,
// scale unpacking :356-363).
//
// Idea.  A Q4_K byte holds two weights of two different 32-value sub-blocks (low nibble: sub-block 2G, high
// nibble: 2G+1).  mma.sync.m16n8k32 (u8 x s8 -> s32) multiplies 16 weight rows x 32 bytes by 8 columns, so one
// instruction covers one sub-block pair of 16 rows, and the bytes are used AS THEY LIE IN MEMORY:
//     MMA 1:  A = raw bytes (lo + 16 hi),   B = [ x(2G) | 0 ]          -> sum(lo x(2G)) + 16 sum(hi x(2G)) | 0
//     MMA 2:  A = raw & 0xF0 (16 hi),       B = [ -x(2G) | x(2G+1) ]   accumulated on top
//                                                                       -> sum(lo x(2G)) | 16 sum(hi x(2G+1))
// One mask per word is all the unpacking there is.  Activations are quantised once per launch to 15-bit
// block fixed point per 256 values (q = 254 hi + lo, |hi|,|lo| <= 127, scale amax / 32258), the two limbs are
// two B columns, so a token occupies four of the eight columns and a launch carries token PAIRS.  The integer
// dots are exact; they meet the 6-bit scales in integer arithmetic, the mins through dp4a against the
// sub-block sums of q, and turn into f32 once per (row, super-block).
//
// Data movement.  One persistent CTA per SM takes the 16-row tiles blockIdx.x, blockIdx.x + gridDim.x, ...
// (the grid as a whole sweeps the matrix linearly).  A producer warp streams the tiles into an mbarrier
// ring; 16 compute warps each own one super-block column of the tile.  A tile is ONE
// tensor-map copy (rows viewed as lines of 128 bytes, 128-byte swizzle, so that the reads of eight rows fall
// into distinct banks); issuing a bulk copy costs about 70 ns, so one copy per row would take longer to
// issue than the data takes to arrive.  Rows that are not a multiple of 128 bytes fall back to per-row
// copies into a padded layout.  Per-row partial sums stay in registers for up to seven
// tiles and are added across warps once at the end, in a fixed order.
// Every mbarrier wait is bounded: on expiry the kernel records UB_ERR_TIMEOUT in the device error word,
// stops waiting and runs out its loops.
#include <cuda.h>  // CUtensorMap type and enums only; the encoder is resolved at run time

#include <string.h>

#include "ar_epilogue.cuh"
#include "common.cuh"

namespace ub {
void* tensor_map_encoder();
}

namespace {

using namespace ub;

constexpr int kCW = 16;                     // compute warps; warp kCW is the producer
constexpr int kImmaThreads = (kCW + 1) * 32;
// 16-row tiles whose partial sums a lane keeps in registers between two cross-warp reductions: seven cover the
// 97 rows per SM of a 14336-row matrix in one batch; with four token pairs that many accumulators spill
constexpr int imma_mt(int mp) { return mp >= 4 ? 4 : 7; }
constexpr int kChunkSb = 16;                // super-blocks of K per ring stage (one per compute warp)
constexpr int kMaxStages = 8;
constexpr int kEarlySlots = 2;              // ring slots filled before the dependency wait
constexpr uint32_t kSpinLimit = 400000;
constexpr float kXQMax = 32258.f;           // 127 * 254
constexpr size_t kSmemBudget = 219 * 1024;  // ring + fragments; 1 KB more goes to the alignment slack

__device__ __forceinline__ void ib_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void ib_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ib_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool ib_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool ib_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (ib_try(bar, parity)) return true;
    if (i >= 2) __nanosleep(40);  // waiting warps would otherwise take issue slots from the working ones
  }
  return false;
}
__device__ __forceinline__ void ib_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// d += A(16x32 u8, row) . B(32x8 s8, col)
__device__ __forceinline__ void imma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
}
// d = A . B (no accumulator to clear beforehand)
__device__ __forceinline__ void imma_u8s8_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint2 b) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "r"(0));
}
__device__ __forceinline__ int dp4a_u_s(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

template <typename XT>
__device__ __forceinline__ void ld_x8(const XT* p, float (&v)[8]);
template <>
__device__ __forceinline__ void ld_x8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
template <>
__device__ __forceinline__ void ld_x8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

__device__ __forceinline__ void st_y(void* y, size_t idx, int dtype, float v) {
  if (dtype == UB_DTYPE_F32)
    static_cast<float*>(y)[idx] = v;
  else if (dtype == UB_DTYPE_BF16)
    static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
  else
    static_cast<__half*>(y)[idx] = __float2half_rn(v);
}

// low bytes of four integers -> one word (three byte permutes)
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// Shared-memory geometry shared by host and device.
struct ImmaGeom {
  int nsb, nchunks, row_stride, stage_bytes;
};
// use_tm: tiles arrive by tensor-map copies (dense rows of whole 128-byte lines, swizzled)
__host__ __device__ inline bool imma_tm_ok(int K) { return ((K >> 8) % 8) == 0; }
__host__ __device__ inline ImmaGeom imma_geom(int K, bool use_tm) {
  ImmaGeom g;
  g.nsb = K >> 8;
  g.nchunks = (g.nsb + kChunkSb - 1) / kChunkSb;
  const int cs = g.nsb < kChunkSb ? g.nsb : kChunkSb;
  if (use_tm) {
    g.row_stride = cs * UB_Q4K_BYTES;  // a multiple of 128 bytes (cs is a multiple of 8)
    g.stage_bytes = 16 * g.row_stride;
    return g;
  }
  // 16-byte loads of eight rows must fall into distinct banks: stride = 32 bytes modulo 128
  g.row_stride = (cs * UB_Q4K_BYTES + 127) / 128 * 128 + 32;
  g.stage_bytes = 16 * g.row_stride;
  return g;
}

// MP: token pairs per launch (tokens 2p and 2p+1 share an MMA; M <= 2 MP, missing tokens are zeros).
template <typename XT, int MP>
__global__ void __launch_bounds__(kImmaThreads, 1)
qgemv_q4k_imma_kernel(const uint8_t* __restrict__ wq, const XT* __restrict__ x, void* __restrict__ y, int M, int N,
                      int K, int y_dtype, int S, int early, int* err_word, int use_tm, const ArParams ar,
                      const __grid_constant__ CUtensorMap w_map) {
  constexpr int kMT = imma_mt(MP);
  extern __shared__ __align__(128) unsigned char ismem_raw[];
  // swizzled tiles need 1024-byte alignment; the launch reserves 1 KB of slack for rounding the base up
  unsigned char* const ismem =
      ismem_raw + ((1024u - (static_cast<uint32_t>(__cvta_generic_to_shared(ismem_raw)) & 1023u)) & 1023u);
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages];  // full[S], empty[S]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const ImmaGeom geo = imma_geom(K, use_tm != 0);
  const int nsb = geo.nsb, nchunks = geo.nchunks;
  const size_t row_bytes = static_cast<size_t>(nsb) * UB_Q4K_BYTES;
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ismem));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  unsigned char* const bfrag = ismem + static_cast<size_t>(S) * geo.stage_bytes;  // [MP][nsb][4 G][2][32 lanes] uint2
  unsigned char* const meta = bfrag + static_cast<size_t>(MP) * nsb * 2048;        // [MP][nsb][4 t] uint4
  float* const red = reinterpret_cast<float*>(ismem);  // aliases the ring between batches

  // 16-row tiles of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
  const int total_tiles = (N + 15) >> 4;
  const int my_tiles =
      static_cast<int>(blockIdx.x) < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int nbatches = (my_tiles + kMT - 1) / kMT;

  // Programmatic dependent launch: the next kernel in the stream may start as soon as every CTA of this
  // grid has passed this point (its CTAs take over SMs as ours retire, instead of waiting for the whole grid
  // to drain), and this kernel may itself have been started early: everything up to the wait below touches
  // only shared memory; the weights, which no kernel writes, are requested by the producer warp right away.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // The ring's barriers come first, and with them the only CTA-wide barrier before the main loop: the
  // producer warp must not be held back by the compute warps' wait for the previous kernel.
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      ib_init(bars_s + 8 * s, 1);
      ib_init(bars_s + 8 * (kMaxStages + s), kCW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp < kCW) asm volatile("griddepcontrol.wait;" ::: "memory");  // activations may come from the previous kernel
  // the first activation piece of this warp is requested before anything else: its latency is on the
  // critical path of the whole launch
  float v_first[8];
  const bool first_live = warp < kCW && warp < 2 * MP * nsb && warp / nsb < M;
  if (first_live) {
    ld_x8<XT>(x + static_cast<size_t>(warp / nsb) * K + (warp % nsb) * 256 + 8 * lane, v_first);
  } else {
#pragma unroll
    for (int e = 0; e < 8; e++) v_first[e] = 0.f;
  }


  bool ok = true;
  // ring position of the next item (same sequence on the producer and the consumer side), kept as counters:
  // a division by the run-time ring depth per item would cost more than the item's address arithmetic
  int slot = 0, round = 0;
  auto ring_next = [&]() {
    if (++slot == S) {
      slot = 0;
      round++;
    }
  };

  if (warp < kCW) {
    // ---- activations -> fragments of the B operand, once per launch ----
    for (int u = warp; u < 2 * MP * nsb; u += kCW) {
      const int m = u / nsb, sb = u - m * nsb;
      const int p = m >> 1, cb = 4 * (m & 1);
      const int j = lane >> 2, tt = lane & 3, G = j >> 1;
      uint2* f1 = reinterpret_cast<uint2*>(bfrag) + ((static_cast<size_t>(p) * nsb + sb) * 4 + G) * 64;  // MMA 1
      uint2* f2 = f1 + 32;                                                                                // MMA 2
      if (m >= M) {
        // a token this launch does not have: its columns multiply by zero
        const int c0 = cb + 2 * (j & 1);
        f1[c0 * 4 + tt] = f1[(c0 + 1) * 4 + tt] = f2[c0 * 4 + tt] = f2[(c0 + 1) * 4 + tt] = make_uint2(0, 0);
        if (lane < 2)
          reinterpret_cast<uint4*>(meta)[(static_cast<size_t>(p) * nsb + sb) * 4 + 2 * (m & 1) + lane] =
              make_uint4(0, 0, 0, 0);
        continue;
      }
      float v[8];
      if (u == warp) {
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = v_first[e];
      } else {
        ld_x8<XT>(x + static_cast<size_t>(m) * K + sb * 256 + 8 * lane, v);
      }
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      const float inv = amax > 0.f ? kXQMax / amax : 0.f;
      const float xs = amax * (1.f / kXQMax);
      // Round through the mantissa of 1.5 * 2^23 (no conversion instructions: their pipe is narrow and all
      // sixteen warps are here at once).  q = rint(v inv); hi = rint(v inv / 254) differs from rint(q / 254)
      // only where q / 254 is within 0.002 of a half, and there both choices leave |lo| <= 127.
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
      const uint2 hv = make_uint2(pack4(hi[0], hi[1], hi[2], hi[3]), pack4(hi[4], hi[5], hi[6], hi[7]));
      const uint2 lv = make_uint2(pack4(lo[0], lo[1], lo[2], lo[3]), pack4(lo[4], lo[5], lo[6], lo[7]));
      // per-byte negation (no limb is -128, so nothing overflows)
      const uint2 nhv = make_uint2(__vneg4(hv.x), __vneg4(hv.y)), nlv = make_uint2(__vneg4(lv.x), __vneg4(lv.y));
      if ((j & 1) == 0) {
        f1[(cb + 0) * 4 + tt] = hv;
        f1[(cb + 1) * 4 + tt] = lv;
        f2[(cb + 0) * 4 + tt] = nhv;
        f2[(cb + 1) * 4 + tt] = nlv;
      } else {
        f1[(cb + 2) * 4 + tt] = make_uint2(0, 0);
        f1[(cb + 3) * 4 + tt] = make_uint2(0, 0);
        f2[(cb + 2) * 4 + tt] = hv;
        f2[(cb + 3) * 4 + tt] = lv;
      }
      // sub-block sums as three byte limbs (top one signed), four sub-blocks per word, for the min term
      int sj[8];
#pragma unroll
      for (int q = 0; q < 8; q++) sj[q] = __shfl_sync(0xFFFFFFFFu, sum, 4 * q);
      if (lane < 2) {
        const int s4[4] = {lane ? sj[4] : sj[0], lane ? sj[5] : sj[1], lane ? sj[6] : sj[2], lane ? sj[7] : sj[3]};
        uint4 mt;
        mt.x = pack4(s4[0], s4[1], s4[2], s4[3]);
        mt.y = pack4(s4[0] >> 8, s4[1] >> 8, s4[2] >> 8, s4[3] >> 8);
        mt.z = pack4(s4[0] >> 16, s4[1] >> 16, s4[2] >> 16, s4[3] >> 16);
        mt.w = __float_as_uint(xs);
        reinterpret_cast<uint4*>(meta)[(static_cast<size_t>(p) * nsb + sb) * 4 + 2 * (m & 1) + lane] = mt;
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory");  // compute warps: fragments complete
  }

  const int par = t & 1;
  // byte offsets of this lane's header and nibble pieces inside a stage (row g, super-block `warp` of the
  // chunk); with tensor-map tiles the 16-byte unit index is XORed with the 128-byte line index modulo 8
  uint32_t off_h, off_q[4];
  {
    auto swz = [&](uint32_t L) { return use_tm ? (L ^ (((L >> 7) & 7u) << 4)) : L; };
    const uint32_t L0 = static_cast<uint32_t>(g * geo.row_stride + warp * UB_Q4K_BYTES);
    off_h = swz(L0);
#pragma unroll
    for (int G = 0; G < 4; G++) off_q[G] = swz(L0 + 16 + 32 * G + 8 * t);
  }
  // B fragments and activation metadata of this warp's super-block: constant over the launch when K fits one
  // chunk and there is one token pair, then kept in registers
  const bool hoist = MP == 1 && nchunks == 1;
  uint2 bq1[4], bq2[4];
  uint4 mt4 = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int G = 0; G < 4; G++) bq1[G] = bq2[G] = make_uint2(0, 0);
  if (hoist && warp < nsb) {
    const uint2* f1 = reinterpret_cast<const uint2*>(bfrag) + static_cast<size_t>(warp) * 256 + lane;
#pragma unroll
    for (int G = 0; G < 4; G++) bq1[G] = f1[G * 64], bq2[G] = f1[G * 64 + 32];
    mt4 = reinterpret_cast<const uint4*>(meta)[static_cast<size_t>(warp) * 4 + t];
  }
  for (int b = 0; b < nbatches; b++) {
    const int n_mt = min(kMT, my_tiles - b * kMT);
    // first row of this batch's tile `mt`: tiles are dealt round robin, so that at any moment the grid as a
    // whole reads one contiguous window of the matrix
    auto tile_row0 = [&](int mt) { return 16 * (static_cast<int>(blockIdx.x) + (b * kMT + mt) * static_cast<int>(gridDim.x)); };

    float acc[kMT][MP][2];  // consumers: partial sums of rows (g, g + 8) of each tile, per token pair
    if (warp == kCW) {
      // ---- producer: 16-row tiles, one bulk copy per row ----
      for (int mt = 0; mt < n_mt; mt++) {
        const int rows_here = min(16, N - tile_row0(mt));
        for (int c = 0; c < nchunks; c++, ring_next()) {
          if (round == 0 && slot == early) {
            // Two tiles are requested before the previous kernel has finished; the rest of the ring waits
            // until the compute warps have sent their activation loads, which would otherwise queue behind
            // ~27 MB of weight traffic (measured: 2 us instead of 0.8 us until the activations arrive).
            asm volatile("griddepcontrol.wait;" ::: "memory");
            __nanosleep(300);
          }
          if (ok && round > 0) ok = ib_wait(bars_s + 8 * (kMaxStages + slot), (round - 1) & 1);
          ok = __all_sync(0xFFFFFFFFu, ok);
          if (!ok) continue;
          const int cs = min(kChunkSb, nsb - c * kChunkSb);
          const uint32_t cbytes = static_cast<uint32_t>(cs * UB_Q4K_BYTES);
          const uint32_t full = bars_s + 8 * slot;
          if (use_tm) {
            // one copy: 16 rows x (row_stride / 128) lines of 128 bytes; rows past N arrive as zeros, rows of
            // the next CTA's range are simply not used
            if (lane == 0) {
              ib_expect_tx(full, static_cast<uint32_t>(geo.stage_bytes));
              asm volatile(
                  "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
                  "%5}], [%2];" ::"r"(ring_s + slot * geo.stage_bytes),
                  "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(full), "r"(0), "r"(c * (geo.row_stride >> 7)),
                  "r"(tile_row0(mt))
                  : "memory");
            }
            continue;
          }
          if (lane == 0) ib_expect_tx(full, cbytes * rows_here);
          __syncwarp();
          if (lane < rows_here)
            ib_copy(ring_s + slot * geo.stage_bytes + lane * geo.row_stride,
                    wq + static_cast<size_t>(tile_row0(mt) + lane) * row_bytes +
                        static_cast<size_t>(c) * kChunkSb * UB_Q4K_BYTES,
                    cbytes, full);
        }
      }
    } else {
      // ---- consumers: warp w owns super-block w of every chunk ----
#pragma unroll
      for (int mt = 0; mt < kMT; mt++)
#pragma unroll
        for (int p = 0; p < MP; p++) acc[mt][p][0] = acc[mt][p][1] = 0.f;

#pragma unroll
      for (int mt = 0; mt < kMT; mt++) {
        if (mt < n_mt) {
          for (int c = 0; c < nchunks; c++, ring_next()) {
              if (ok) ok = __all_sync(0xFFFFFFFFu, ib_wait(bars_s + 8 * slot, round & 1));
            const int cs = min(kChunkSb, nsb - c * kChunkSb);
            if (ok && warp < cs) {
              const int sb = c * kChunkSb + warp;
              // rows g and g + 8 of the tile; offsets inside a row are swizzled identically for both
              const unsigned char* rowA = ismem + static_cast<size_t>(slot) * geo.stage_bytes;
              const unsigned char* rowB = rowA + 8 * geo.row_stride;
              const uint4 hA = *reinterpret_cast<const uint4*>(rowA + off_h);
              const uint4 hB = *reinterpret_cast<const uint4*>(rowB + off_h);
              uint2 wA[4], wB[4];
#pragma unroll
              for (int G = 0; G < 4; G++) {
                wA[G] = *reinterpret_cast<const uint2*>(rowA + off_q[G]);
                wB[G] = *reinterpret_cast<const uint2*>(rowB + off_q[G]);
              }
              // everything this warp needs from the stage is in registers: hand the slot back now (the
              // arrive is a release, so the loads above are performed before the producer sees it)
              __syncwarp();
              if (lane == 0) ib_arrive(bars_s + 8 * (kMaxStages + slot));
              uint32_t scA[2], mnA[2], scB[2], mnB[2];
              q4k_unpack_scales(hA.y, hA.z, hA.w, scA[0], scA[1], mnA[0], mnA[1]);
              q4k_unpack_scales(hB.y, hB.z, hB.w, scB[0], scB[1], mnB[0], mnB[1]);
              // this lane's columns belong to sub-blocks 2G + par: bring their scales to bytes 0 and 2
              scA[0] >>= 8 * par, scA[1] >>= 8 * par, scB[0] >>= 8 * par, scB[1] >>= 8 * par;
              // ... and to sub-blocks 4 par .. 4 par + 3 for the min term
              const uint32_t mA = par ? mnA[1] : mnA[0], mB = par ? mnB[1] : mnB[0];
              const float dA = half_bits_to_f32(hA.x), dminA = half_bits_to_f32(hA.x >> 16);
              const float dB = half_bits_to_f32(hB.x), dminB = half_bits_to_f32(hB.x >> 16);
#pragma unroll
              for (int p = 0; p < MP; p++) {
                if (!hoist) {
                  const uint2* f1 =
                      reinterpret_cast<const uint2*>(bfrag) + (static_cast<size_t>(p) * nsb + sb) * 256 + lane;
#pragma unroll
                  for (int G = 0; G < 4; G++) bq1[G] = f1[G * 64], bq2[G] = f1[G * 64 + 32];
                  mt4 = reinterpret_cast<const uint4*>(meta)[(static_cast<size_t>(p) * nsb + sb) * 4 + t];
                }
                // all eight MMAs first (four independent chains of two), then the scale arithmetic
                int d[4][4];
#pragma unroll
                for (int G = 0; G < 4; G++) {
                  imma_u8s8_first(d[G], wA[G].x, wB[G].x, wA[G].y, wB[G].y, bq1[G]);
                }
#pragma unroll
                for (int G = 0; G < 4; G++)
                  imma_u8s8(d[G], wA[G].x & 0xF0F0F0F0u, wB[G].x & 0xF0F0F0F0u, wA[G].y & 0xF0F0F0F0u,
                            wB[G].y & 0xF0F0F0F0u, bq2[G]);
                int hiA = 0, loA = 0, hiB = 0, loB = 0;
#pragma unroll
                for (int G = 0; G < 4; G++) {
                  const int sa = (G & 1) ? __byte_perm(scA[G >> 1], 0, 0x4442) : (scA[G >> 1] & 0xFF);
                  const int sbv = (G & 1) ? __byte_perm(scB[G >> 1], 0, 0x4442) : (scB[G >> 1] & 0xFF);
                  hiA += d[G][0] * sa, loA += d[G][1] * sa, hiB += d[G][2] * sbv, loB += d[G][3] * sbv;
                }
                const float xs = __uint_as_float(mt4.w);
                const float xsm = par ? xs * 0.0625f : xs;  // odd lanes carry 16 x the high nibbles
                const int tA = (dp4a_u_s(mA, mt4.z, 0) * 256 + static_cast<int>(__dp4a(mA, mt4.y, 0u))) * 256 +
                               static_cast<int>(__dp4a(mA, mt4.x, 0u));
                const int tB = (dp4a_u_s(mB, mt4.z, 0) * 256 + static_cast<int>(__dp4a(mB, mt4.y, 0u))) * 256 +
                               static_cast<int>(__dp4a(mB, mt4.x, 0u));
                const float fA = fmaf(static_cast<float>(hiA), 254.f, static_cast<float>(loA));
                const float fB = fmaf(static_cast<float>(hiB), 254.f, static_cast<float>(loB));
                acc[mt][p][0] += fmaf(dA * xsm, fA, -(dminA * xs) * static_cast<float>(tA));
                acc[mt][p][1] += fmaf(dB * xsm, fB, -(dminB * xs) * static_cast<float>(tB));
              }
            } else {
              __syncwarp();
              if (lane == 0) ib_arrive(bars_s + 8 * (kMaxStages + slot));
            }
          }
        }
      }
    }
    __syncthreads();  // (A) every stage of this batch has been consumed: the ring may hold the partial sums
    if (warp < kCW) {
      // the two lanes of a (row, token) pair hold its even and odd sub-blocks
#pragma unroll
      for (int mt = 0; mt < kMT; mt++)
#pragma unroll
        for (int p = 0; p < MP; p++)
#pragma unroll
          for (int rs = 0; rs < 2; rs++) {
            const float v = acc[mt][p][rs] + __shfl_xor_sync(0xFFFFFFFFu, acc[mt][p][rs], 1);
            if (par == 0) red[((((warp * kMT + mt) * MP + p) * 2 + rs) * 8 + g) * 2 + (t >> 1)] = v;
          }
    }
    __syncthreads();  // (B) partial sums visible
    if (b == 0 && warp == kCW) asm volatile("griddepcontrol.wait;" ::: "memory");  // before this warp's stores
    for (int o = threadIdx.x; o < n_mt * 16 * 2 * MP; o += kImmaThreads) {
      const int rl = o / (2 * MP), tok = o - rl * (2 * MP);
      const int row = tile_row0(rl >> 4) + (rl & 15);
      if (row < N && tok < M) {
        const int mt = rl >> 4, rs = (rl >> 3) & 1, gg = rl & 7, p = tok >> 1, tk = tok & 1;
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kCW; w++) tot += red[((((w * kMT + mt) * MP + p) * 2 + rs) * 8 + gg) * 2 + tk];
        if (ar.world > 1)  // fused all-reduce (one token): the row goes to every rank's staging slot
          ar_push(ar, ar_epoch(ar), row, tot);
        else
          st_y(y, static_cast<size_t>(tok) * N + row, y_dtype, tot);
      }
    }
    __syncthreads();  // (C) the ring is free again
  }
  if (ar.world > 1) ar_finish(ar, ar_epoch(ar), y, N, err_word);
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

template <typename XT, int MP>
int launch_imma(const uint8_t* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, const ArParams& ar,
                cudaStream_t s) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ub::tensor_map_encoder());
  bool use_tm = enc != nullptr && imma_tm_ok(K);
  CUtensorMap wmap;
  memset(&wmap, 0, sizeof(wmap));
  if (use_tm) {
    // rows as lines of 128 bytes: {128 bytes, lines per row, N rows}; box = {128, lines per chunk, 16 rows}
    const ImmaGeom gt = imma_geom(K, true);
    const cuuint64_t row_bytes = static_cast<cuuint64_t>(gt.nsb) * UB_Q4K_BYTES;
    const cuuint64_t dims[3] = {128, row_bytes / 128, static_cast<cuuint64_t>(N)};
    const cuuint64_t strides[2] = {128, row_bytes};
    const cuuint32_t box[3] = {128, static_cast<cuuint32_t>(gt.row_stride / 128), 16};
    const cuuint32_t estr[3] = {1, 1, 1};
    use_tm = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(wq), dims, strides, box, estr,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  const ImmaGeom geo = imma_geom(K, use_tm);
  const size_t fixed = static_cast<size_t>(MP) * geo.nsb * (2048 + 64);
  if (fixed + 2 * static_cast<size_t>(geo.stage_bytes) > kSmemBudget) return UB_ERR_UNSUPPORTED;
  int S = static_cast<int>((kSmemBudget - fixed) / geo.stage_bytes);
  if (S > kMaxStages) S = kMaxStages;
  const size_t red_bytes = static_cast<size_t>(kCW) * imma_mt(MP) * MP * 32 * sizeof(float);
  if (static_cast<size_t>(S) * geo.stage_bytes < red_bytes) return UB_ERR_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(S) * geo.stage_bytes + fixed + 1024;
  auto kernel = qgemv_q4k_imma_kernel<XT, MP>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  const int sms = ub::num_sms();
  const int tiles = (N + 15) / 16;
  const int grid = tiles < sms ? tiles : sms;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kImmaThreads), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, wq, x, y, M, N, K, y_dtype, S, fresh ? 0 : kEarlySlots, ub::device_error_word(),
                         use_tm ? 1 : 0, ar, wmap);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::check_launch();
}


// =====================================================================================================
// Q8_0 on the same scheme.  A block is 34 bytes: an f16 scale and 32 signed bytes, which are the MMA's A
// operand as they lie in memory (s8 x s8 -> s32); activations are quantised per 32-value block to the same
// two signed-byte limbs, so a token takes two of the eight B columns and a launch carries token QUADS.
// Replaces the reference's decode matmul for block_q8_0 weights (kernels/quant.cpp:98-104, dequantisation
// :188-268).  Tiles are 16 rows x 64 blocks (2176 bytes = 17 lines of 128 bytes per row), one swizzled
// tensor-map copy each; warp w owns blocks 4w .. 4w+3 of the chunk.  The 32 weight bytes of a block start
// 2 bytes after a 4-byte boundary in every other block: those are read as three aligned words and funnel
// shifted.
constexpr int kQ8ChunkBlocks = 64;
constexpr int kQ8RowStride = kQ8ChunkBlocks * UB_Q8_0_BYTES;  // 2176
constexpr int kQ8StageBytes = 16 * kQ8RowStride;              // 34816 = 34 KB

// d = A(16x32 s8, row) . B(32x8 s8, col)
__device__ __forceinline__ void imma_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "r"(0));
}
__device__ __forceinline__ uint32_t swz128(uint32_t L) { return L ^ (((L >> 7) & 7u) << 4); }

// MQ: token quads per launch (M <= 4 MQ, missing tokens are zeros).
template <typename XT, int MQ>
__global__ void __launch_bounds__(kImmaThreads, 1)
qgemv_q8_0_imma_kernel(const XT* __restrict__ x, void* __restrict__ y, int M, int N, int K, int y_dtype, int S,
                       int early, int* err_word, const __grid_constant__ CUtensorMap w_map) {
  constexpr int kMT = 7;
  extern __shared__ __align__(128) unsigned char ismem_raw[];
  unsigned char* const ismem =
      ismem_raw + ((1024u - (static_cast<uint32_t>(__cvta_generic_to_shared(ismem_raw)) & 1023u)) & 1023u);
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int nblk = K >> 5, nchunks = nblk / kQ8ChunkBlocks;
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ismem));
  const uint32_t bars_s = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  unsigned char* const bfrag = ismem + static_cast<size_t>(S) * kQ8StageBytes;  // [MQ][nblk][32 lanes] uint2
  float* const xscale = reinterpret_cast<float*>(bfrag + static_cast<size_t>(MQ) * nblk * 256);  // [MQ][nblk][4]
  float* const red = reinterpret_cast<float*>(ismem);

  const int total_tiles = (N + 15) >> 4;
  const int my_tiles =
      static_cast<int>(blockIdx.x) < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int nbatches = (my_tiles + kMT - 1) / kMT;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // barriers first (see the Q4_K kernel): the producer warp starts streaming while the compute warps wait
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      ib_init(bars_s + 8 * s, 1);
      ib_init(bars_s + 8 * (kMaxStages + s), kCW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp < kCW) asm volatile("griddepcontrol.wait;" ::: "memory");

  bool ok = true;
  // ring position of the next item (same sequence on the producer and the consumer side), kept as counters:
  // a division by the run-time ring depth per item would cost more than the item's address arithmetic
  int slot = 0, round = 0;
  auto ring_next = [&]() {
    if (++slot == S) {
      slot = 0;
      round++;
    }
  };

  if (warp < kCW) {
    // ---- activations -> B fragments: unit = (token, 256 values); lane i holds 8 values of block i / 4 ----
    const int groups = K >> 8;
    for (int u = warp; u < 4 * MQ * groups; u += kCW) {
      const int m = u / groups, grp = u - m * groups;
      const int quad = m >> 2, col = 2 * (m & 3);
      const int blk = grp * 8 + (lane >> 2), tt = lane & 3;
      uint2* f = reinterpret_cast<uint2*>(bfrag) + (static_cast<size_t>(quad) * nblk + blk) * 32;
      float* xsp = xscale + (static_cast<size_t>(quad) * nblk + blk) * 4 + (m & 3);
      if (m >= M) {
        f[col * 4 + tt] = f[(col + 1) * 4 + tt] = make_uint2(0, 0);
        if (tt == 0) *xsp = 0.f;
        continue;
      }
      float v[8];
      ld_x8<XT>(x + static_cast<size_t>(m) * K + grp * 256 + 8 * lane, v);
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));  // over the block's four lanes
      const float inv = amax > 0.f ? kXQMax / amax : 0.f;
      const float inv254 = inv * (1.f / 254.f);  // rounding through the mantissa of 1.5 * 2^23, as above
      int hi[8], lo[8];
#pragma unroll
      for (int e = 0; e < 8; e++) {
        const int q = __float_as_int(fmaf(v[e], inv, 12582912.f)) - 0x4B400000;
        hi[e] = __float_as_int(fmaf(v[e], inv254, 12582912.f)) - 0x4B400000;
        lo[e] = q - 254 * hi[e];
      }
      f[col * 4 + tt] = make_uint2(pack4(hi[0], hi[1], hi[2], hi[3]), pack4(hi[4], hi[5], hi[6], hi[7]));
      f[(col + 1) * 4 + tt] = make_uint2(pack4(lo[0], lo[1], lo[2], lo[3]), pack4(lo[4], lo[5], lo[6], lo[7]));
      if (tt == 0) *xsp = amax * (1.f / kXQMax);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory");
  }

  for (int b = 0; b < nbatches; b++) {
    const int n_mt = min(kMT, my_tiles - b * kMT);
    // first row of this batch's tile `mt`: tiles are dealt round robin, so that at any moment the grid as a
    // whole reads one contiguous window of the matrix
    auto tile_row0 = [&](int mt) { return 16 * (static_cast<int>(blockIdx.x) + (b * kMT + mt) * static_cast<int>(gridDim.x)); };
    float acc[kMT][MQ][2];
    if (warp == kCW) {
      for (int mt = 0; mt < n_mt; mt++) {
        for (int c = 0; c < nchunks; c++, ring_next()) {
          if (round == 0 && slot == early) {
            // Two tiles are requested before the previous kernel has finished; the rest of the ring waits
            // until the compute warps have sent their activation loads, which would otherwise queue behind
            // ~27 MB of weight traffic (measured: 2 us instead of 0.8 us until the activations arrive).
            asm volatile("griddepcontrol.wait;" ::: "memory");
            __nanosleep(300);
          }
          if (ok && round > 0) ok = ib_wait(bars_s + 8 * (kMaxStages + slot), (round - 1) & 1);
          ok = __all_sync(0xFFFFFFFFu, ok);
          if (!ok) continue;
          if (lane == 0) {
            const uint32_t full = bars_s + 8 * slot;
            ib_expect_tx(full, kQ8StageBytes);
            asm volatile(
                "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
                "%5}], [%2];" ::"r"(ring_s + slot * kQ8StageBytes),
                "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(full), "r"(0), "r"(c * (kQ8RowStride >> 7)),
                "r"(tile_row0(mt))
                : "memory");
          }
        }
      }
    } else {
#pragma unroll
      for (int mt = 0; mt < kMT; mt++)
#pragma unroll
        for (int q = 0; q < MQ; q++) acc[mt][q][0] = acc[mt][q][1] = 0.f;
#pragma unroll
      for (int mt = 0; mt < kMT; mt++) {
        if (mt < n_mt) {
          for (int c = 0; c < nchunks; c++, ring_next()) {
              if (ok) ok = __all_sync(0xFFFFFFFFu, ib_wait(bars_s + 8 * slot, round & 1));
            if (ok) {
              const unsigned char* st = ismem + static_cast<size_t>(slot) * kQ8StageBytes;
              // this warp's four blocks of rows g and g + 8: scales and weight bytes into registers
              uint32_t a[4][4];
              float dA[4], dB[4];
#pragma unroll
              for (int i = 0; i < 4; i++) {
                const uint32_t L = static_cast<uint32_t>(g * kQ8RowStride + (warp * 4 + i) * UB_Q8_0_BYTES);
                const uint32_t LB = L + 8 * kQ8RowStride;  // 8 rows = 136 lines further: same swizzle phase
                dA[i] = half_bits_to_f32(*reinterpret_cast<const unsigned short*>(st + swz128(L)));
                dB[i] = half_bits_to_f32(*reinterpret_cast<const unsigned short*>(st + swz128(LB)));
                const uint32_t q0 = L + 2 + 8 * t;
                if (i & 1) {  // 34 i + 2 is a multiple of 4 for odd i (warp * 4 is even): aligned words
                  a[i][0] = *reinterpret_cast<const uint32_t*>(st + swz128(q0));
                  a[i][2] = *reinterpret_cast<const uint32_t*>(st + swz128(q0 + 4));
                  a[i][1] = *reinterpret_cast<const uint32_t*>(st + swz128(q0 + 8 * kQ8RowStride));
                  a[i][3] = *reinterpret_cast<const uint32_t*>(st + swz128(q0 + 4 + 8 * kQ8RowStride));
                } else {      // 2 bytes past a word boundary: three words, funnel shifted by 16 bits
                  const uint32_t w0 = *reinterpret_cast<const uint32_t*>(st + swz128(q0 - 2));
                  const uint32_t w1 = *reinterpret_cast<const uint32_t*>(st + swz128(q0 + 2));
                  const uint32_t w2 = *reinterpret_cast<const uint32_t*>(st + swz128(q0 + 6));
                  a[i][0] = __funnelshift_r(w0, w1, 16), a[i][2] = __funnelshift_r(w1, w2, 16);
                  const uint32_t v0 = *reinterpret_cast<const uint32_t*>(st + swz128(q0 - 2 + 8 * kQ8RowStride));
                  const uint32_t v1 = *reinterpret_cast<const uint32_t*>(st + swz128(q0 + 2 + 8 * kQ8RowStride));
                  const uint32_t v2 = *reinterpret_cast<const uint32_t*>(st + swz128(q0 + 6 + 8 * kQ8RowStride));
                  a[i][1] = __funnelshift_r(v0, v1, 16), a[i][3] = __funnelshift_r(v1, v2, 16);
                }
              }
              __syncwarp();
              if (lane == 0) ib_arrive(bars_s + 8 * (kMaxStages + slot));
#pragma unroll
              for (int q = 0; q < MQ; q++) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                  const int blk = c * kQ8ChunkBlocks + warp * 4 + i;
                  const uint2 bf = reinterpret_cast<const uint2*>(bfrag)[(static_cast<size_t>(q) * nblk + blk) * 32 + lane];
                  const float xs = xscale[(static_cast<size_t>(q) * nblk + blk) * 4 + t];
                  int d[4];
                  imma_s8s8(d, a[i][0], a[i][1], a[i][2], a[i][3], bf);
                  // columns 2t, 2t+1 = token t's high and low limb
                  acc[mt][q][0] = fmaf(static_cast<float>(d[0] * 254 + d[1]), dA[i] * xs, acc[mt][q][0]);
                  acc[mt][q][1] = fmaf(static_cast<float>(d[2] * 254 + d[3]), dB[i] * xs, acc[mt][q][1]);
                }
              }
            } else {
              __syncwarp();
              if (lane == 0) ib_arrive(bars_s + 8 * (kMaxStages + slot));
            }
          }
        }
      }
    }
    __syncthreads();  // (A) every stage of this batch has been consumed: the ring may hold the partial sums
    if (warp < kCW) {
#pragma unroll
      for (int mt = 0; mt < kMT; mt++)
#pragma unroll
        for (int q = 0; q < MQ; q++)
#pragma unroll
          for (int rs = 0; rs < 2; rs++)
            red[((((warp * kMT + mt) * MQ + q) * 2 + rs) * 8 + g) * 4 + t] = acc[mt][q][rs];
    }
    __syncthreads();  // (B)
    if (b == 0 && warp == kCW) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int o = threadIdx.x; o < n_mt * 16 * 4 * MQ; o += kImmaThreads) {
      const int rl = o / (4 * MQ), tok = o - rl * (4 * MQ);
      const int row = tile_row0(rl >> 4) + (rl & 15);
      if (row < N && tok < M) {
        const int mt = rl >> 4, rs = (rl >> 3) & 1, gg = rl & 7, q = tok >> 2, tk = tok & 3;
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kCW; w++) tot += red[((((w * kMT + mt) * MQ + q) * 2 + rs) * 8 + gg) * 4 + tk];
        st_y(y, static_cast<size_t>(tok) * N + row, y_dtype, tot);
      }
    }
    __syncthreads();  // (C)
  }
  if (!ok && lane == 0) report_device_error(err_word, UB_ERR_TIMEOUT);
}

template <typename XT, int MQ>
int launch_q8_imma(const uint8_t* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ub::tensor_map_encoder());
  // whole 64-block chunks (rows are then whole 128-byte lines) and a 16-byte aligned base for the tensor map
  if (!enc || K % (32 * kQ8ChunkBlocks) != 0 || (reinterpret_cast<uintptr_t>(wq) & 15)) return UB_ERR_UNSUPPORTED;
  const int nblk = K / 32;
  const size_t fixed = static_cast<size_t>(MQ) * nblk * (256 + 16);
  if (fixed + 2 * static_cast<size_t>(kQ8StageBytes) > kSmemBudget) return UB_ERR_UNSUPPORTED;
  int S = static_cast<int>((kSmemBudget - fixed) / kQ8StageBytes);
  if (S > kMaxStages) S = kMaxStages;
  const size_t red_bytes = static_cast<size_t>(kCW) * 7 * MQ * 64 * sizeof(float);
  if (static_cast<size_t>(S) * kQ8StageBytes < red_bytes) return UB_ERR_UNSUPPORTED;
  CUtensorMap wmap;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(nblk) * UB_Q8_0_BYTES;
  const cuuint64_t dims[3] = {128, row_bytes / 128, static_cast<cuuint64_t>(N)};
  const cuuint64_t strides[2] = {128, row_bytes};
  const cuuint32_t box[3] = {128, static_cast<cuuint32_t>(kQ8RowStride / 128), 16};
  const cuuint32_t estr[3] = {1, 1, 1};
  if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(wq), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return UB_ERR_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(S) * kQ8StageBytes + fixed + 1024;
  auto kernel = qgemv_q8_0_imma_kernel<XT, MQ>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  const int sms = ub::num_sms();
  const int tiles = (N + 15) / 16;
  const int grid = tiles < sms ? tiles : sms;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kImmaThreads), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, x, y, M, N, K, y_dtype, S, fresh ? 0 : kEarlySlots, ub::device_error_word(), wmap);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::check_launch();
}

}  // namespace

namespace ub {

// y[M,N] = x[M,K] . dequant(Wq)^T for 1 <= M <= 8; returns UB_ERR_UNSUPPORTED (without setting the thread's
// status) when the shape does not fit this kernel's shared-memory plan, so that the caller can use another.
template <typename XT>
int q4k_gemv_imma(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, const ArParams* ar,
                  cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  ArParams none;
  memset(&none, 0, sizeof(none));
  if (ar && ar->world > 1 && M != 1) return UB_ERR_UNSUPPORTED;  // the fused exchange is a one-token path
  const ArParams& a = ar ? *ar : none;
  if (M <= 2) return launch_imma<XT, 1>(w, x, y, M, N, K, y_dtype, fresh, a, s);
  if (M <= 4) return launch_imma<XT, 2>(w, x, y, M, N, K, y_dtype, fresh, a, s);
  return launch_imma<XT, 4>(w, x, y, M, N, K, y_dtype, fresh, a, s);
}

// Q8_0 flavour, same contract.
template <typename XT>
int q8_0_gemv_imma(const void* wq, const XT* x, void* y, int M, int N, int K, int y_dtype, bool fresh, cudaStream_t s) {
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  if (M <= 4) return launch_q8_imma<XT, 1>(w, x, y, M, N, K, y_dtype, fresh, s);
  return launch_q8_imma<XT, 2>(w, x, y, M, N, K, y_dtype, fresh, s);
}

template int q8_0_gemv_imma<float>(const void*, const float*, void*, int, int, int, int, bool, cudaStream_t);
template int q8_0_gemv_imma<__nv_bfloat16>(const void*, const __nv_bfloat16*, void*, int, int, int, int, bool, cudaStream_t);
template int q4k_gemv_imma<float>(const void*, const float*, void*, int, int, int, int, bool, const ArParams*,
                                  cudaStream_t);
template int q4k_gemv_imma<__nv_bfloat16>(const void*, const __nv_bfloat16*, void*, int, int, int, int, bool,
                                          const ArParams*, cudaStream_t);

}  // namespace ub
