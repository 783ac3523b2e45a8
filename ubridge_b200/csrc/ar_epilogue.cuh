// All-reduce fused behind a row-split decode matmul: the matmul's own CTAs push their rows of the partial output
// into the peers' staging buffers as they finish them, and the LAST CTA of the grid to finish completes the
// exchange.  It stands where the reference's caller issues ecclAllReduce after the o and down projections
// (src/eccl.rs:209-245) and replaces the separate one-CTA kernel of p2p.cu for one-token calls, which removes
// one launch and one dependent-launch gap per exchange.
//
// Same staging buffer, same epoch / flag protocol and the same result bits as ub_allreduce_oneshot_bf16 (p2p.cu),
// so fused and stand-alone calls may alternate on one set of buffers:
//   [0]   u32 epoch of the last completed exchange (local)        [64]  u32 count of CTAs that have pushed (local)
//   [128] flags[2][world] u32                                     [1024] slots[2][world][max_bytes]
// Every CTA: bf16 value of each of its rows -> slot `rank` of EVERY rank (plain peer stores), system-scope
// fence, one atomic increment of the local count.  The CTA that observes count == gridDim.x - 1 resets the
// count, raises this rank's flag at every peer (release), waits - bounded - for all flags of this epoch in its
// own buffer, adds the slots in rank order in f32, rounds once to bf16 into y and publishes the epoch.
// No multimem, no cluster features, no TMA from peer memory: ordinary loads and stores only.
#pragma once

#include "common.cuh"

namespace ub {

constexpr int kArMaxWorld = 16;
constexpr size_t kArCountOff = 64, kArFlagsOff = 128, kArSlotsOff = 1024;

struct ArParams {
  unsigned char* base[kArMaxWorld];  // staging buffer of every rank, in rank order (own buffer at [rank])
  int rank, world;                   // world <= 1: no exchange, rows go straight to y
  uint32_t spin_limit;
  size_t max_bytes;
  const __nv_bfloat16* residual;     // optional [n]: y = residual + sum (the residual add of a decoder layer), else null
};

// Optional pieces of a one-token matmul launch, all off when null / zero.
struct M1Extras {
  const void* gamma;   // RMSNorm weight [K] in the activation type: the matmul runs on rmsnorm(x)
  float eps;
  const ArParams* ar;  // exchange over the ranks (world > 1) and / or a residual row added to the output
};

__device__ __forceinline__ uint32_t ar_epoch(const ArParams& ar) {
  return *reinterpret_cast<volatile uint32_t*>(ar.base[ar.rank]) + 1;
}

// one row of this rank's partial output -> slot `rank` of every rank
__device__ __forceinline__ void ar_push(const ArParams& ar, uint32_t epoch, int row, float v) {
  const __nv_bfloat16 b = __float2bfloat16_rn(v);
  const size_t off = kArSlotsOff + (static_cast<size_t>(epoch & 1) * ar.world + ar.rank) * ar.max_bytes +
                     static_cast<size_t>(row) * 2;
  for (int p = 0; p < ar.world; p++) *reinterpret_cast<__nv_bfloat16*>(ar.base[p] + off) = b;
}

// Called by every thread of every CTA after its last ar_push.  y: bf16 [n] (n % 8 == 0, 16-byte aligned).
__device__ __forceinline__ void ar_finish(const ArParams& ar, uint32_t epoch, void* y, int n, int* err_word) {
  __shared__ int s_last;
  unsigned char* const mine = ar.base[ar.rank];
  __threadfence_system();  // this thread's pushes are visible system-wide before the count moves
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned old = atomicAdd(reinterpret_cast<unsigned*>(mine + kArCountOff), 1u);
    s_last = old == gridDim.x - 1;
    if (s_last) *reinterpret_cast<volatile unsigned*>(mine + kArCountOff) = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();  // the other CTAs' pushes, ordered before their increments, are ordered before what follows
  const int set = epoch & 1;
  if (static_cast<int>(threadIdx.x) < ar.world) {
    uint32_t* f = reinterpret_cast<uint32_t*>(ar.base[threadIdx.x] + kArFlagsOff) + set * ar.world + ar.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    const uint32_t* w = reinterpret_cast<const uint32_t*>(mine + kArFlagsOff) + set * ar.world + threadIdx.x;
    bool seen = false;
    for (uint32_t it = 0; it < ar.spin_limit; it++) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(w) : "memory");
      if (v == epoch) {
        seen = true;
        break;
      }
      __nanosleep(100);
    }
    if (!seen) report_device_error(err_word, UB_ERR_TIMEOUT);
  }
  __syncthreads();
  const unsigned char* slots = mine + kArSlotsOff + static_cast<size_t>(set) * ar.world * ar.max_bytes;
  for (int i = threadIdx.x; i < n / 8; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; e++) acc[e] = 0.f;
    if (ar.residual) {  // the residual comes first, then the ranks in order: the same bits on every rank
      const uint4 r = __ldg(reinterpret_cast<const uint4*>(ar.residual) + i);
      const uint32_t r4[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int e = 0; e < 4; e++) {
        acc[2 * e] = __uint_as_float(r4[e] << 16);
        acc[2 * e + 1] = __uint_as_float(r4[e] & 0xFFFF0000u);
      }
    }
    for (int p = 0; p < ar.world; p++) {
      uint4 v;  // written by a peer: not through L1
      asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                   : "l"(slots + static_cast<size_t>(p) * ar.max_bytes + static_cast<size_t>(i) * 16));
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; e++) {
        acc[2 * e] += __uint_as_float(w4[e] << 16);
        acc[2 * e + 1] += __uint_as_float(w4[e] & 0xFFFF0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      o[e] = *reinterpret_cast<const uint32_t*>(&b);
    }
    reinterpret_cast<uint4*>(y)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  __syncthreads();
  if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(mine) = epoch;
}

}  // namespace ub
