// Prefill GEMM for Q4_K weights on the 5th-generation tensor cores (tcgen05 / TMEM), with the
// dequantisation fused into the main loop.
//
//   y[M,N] (bf16) = x[M,K] (bf16) . dequant(Wq[N rows of K/256 super-blocks])^T,   f32 accumulation.
//
// Replaces the reference's two-kernel sequence dequantize_block_q4_k_* (kernels/quant.cpp:477-488) +
// matmul_bf16 (kernels/matmul.cpp:1143-1184), whose W4 flavour dequantises a weight tile in on-chip memory
// and then calls the matrix engine (kernels/matmul.cpp:1039-1109).
//
// Tile and roles.  One persistent CTA per SM walks over (128 weight rows) x (TOK tokens) output tiles.
// The weight tile is the UMMA "A" operand (M = 128) and is read by the MMA from TENSOR MEMORY: producers
// dequantise straight from registers into TMEM with tcgen05.st, so weights never touch shared memory.
// The token tile is the "B" operand (N = TOK <= 256, trimmed to the valid tokens of a ragged last tile),
// K-major bf16 in the 128-byte-swizzled canonical layout, written to shared memory by 2-D tensor-map
// copies.  The accumulator D[128 lanes x TOK columns] lives in tensor memory next to the weight stages
// (columns 0..255 accumulators, 256.. weight stages of 32 columns each).  K is consumed 64 values per
// stage (one 64-value Q4_K group), four UMMA K=16 steps each.
//
//   warp 0        allocates TMEM, then one elected lane issues tcgen05.mma and tcgen05.commit
//   warps 1-4     epilogue: tcgen05.ld -> bf16 -> staging tile in shared memory (accumulator released
//                 here) -> 16-byte coalesced stores to y, overlapping the next tile's main loop
//   warps 5-12    weight producers: read their row's packed super-block from a shared-memory ring, turn
//                 nibbles into bf16 (128 + q) with one byte permute per pair, minus 128 (exact), times d*sc
//                 minus dmin*m with packed bf16 FMAs; tcgen05.st, tcgen05.wait::st, mbarrier arrive
//   warp 13       one lane issues all bulk copies: packed weight tiles ([128 rows][144 bytes], one 2-D
//                 tensor-map copy per super-block column, two super-blocks ahead) and token tiles (one
//                 copy per K step, as far ahead as the ring allows)
//
// Every mbarrier wait is bounded; on expiry the CTA sets a shared abort flag, records UB_ERR_TIMEOUT in
// the device error word, all roles leave their loops, and TMEM is freed before the kernel returns.
#include <cuda.h>  // CUtensorMap type and enums only; the encoder is resolved at run time

#include <string.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace {

using namespace ub;

constexpr int kTcProducerWarps = 8;   // warps that dequantise one K step (128 rows x 2 nibble halves)
// Sets of such warps (template parameter SETS); set i takes the K steps with step % SETS == i.  Measured on B200:
// a second set does not help, neither with 256-token tiles (C3 204 us against 191 us with one) nor with 16 to 128
// tokens (14336x4096: 27.9 us against 26.1 us at 16 tokens, where a K step takes 0.42 us whatever the token
// count: 0.20 us of producer arithmetic, 0.10 us until tcgen05.st has landed, 0.20 us for the issuing thread to
// get four MMAs and a commit out).  Every launch uses one set.
constexpr int tc_threads(int sets) { return (5 + kTcProducerWarps * sets + 1) * 32; }
constexpr int kTcBK = 64;
constexpr uint32_t kTcWaitLimit = 2000000;

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait that also gives up when another role has raised the abort flag.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (tc_mbar_try(bar, parity)) return true;
  for (uint32_t i = 0; i < kTcWaitLimit; i++) {
    if (tc_mbar_try(bar, parity)) return true;
    if (i > 16) __nanosleep(i > 256 ? 256 : 32);  // back off: spinning warps share issue slots with the producers
    if ((i & 255) == 255 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// The same bounded wait with acquire semantics at cluster scope: what other CTAs of the cluster wrote into this
// CTA's shared memory before their (release) arrivals is visible afterwards.
__device__ __forceinline__ bool tc_mbar_try_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool tc_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (tc_mbar_try_cluster(bar, parity)) return true;
  for (uint32_t i = 0; i < kTcWaitLimit; i++) {
    if (tc_mbar_try_cluster(bar, parity)) return true;
    if (i > 16) __nanosleep(i > 256 ? 256 : 32);
    if ((i & 255) == 255 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
// address of this CTA's shared-memory location `addr` in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t tc_peer_addr(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void tc_peer_arrive(uint32_t peer_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(peer_bar) : "memory");
}
// four bytes into another CTA's shared memory, counted on a barrier of that CTA (no fence on this side)
__device__ __forceinline__ void tc_peer_store_tx(uint32_t peer_addr, uint32_t v, uint32_t peer_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(peer_addr), "r"(v),
               "r"(peer_bar)
               : "memory");
}
__device__ __forceinline__ void tc_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the same without ordering memory: only "every CTA of the cluster has come this far"
__device__ __forceinline__ void tc_cluster_sync_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}

__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t smem_addr) {
  // K-major, 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO), LBO unused (1), descriptor version 1
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// same, with the A operand read from tensor memory (128 lanes x 8 columns of packed bf16 pairs per K = 16)
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
      "%15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
      "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ uint32_t bf162_bits(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// Two nibbles (bytes A and B of a word masked with 0x0F0F0F0F) -> packed bf16 (dsc*qA - dm, dsc*qB - dm)
template <int SEL>
__device__ __forceinline__ uint32_t deq_pair(uint32_t w4, __nv_bfloat162 dsc, __nv_bfloat162 ndm) {
  const uint32_t biased = __byte_perm(w4, 0x43434343u, SEL);  // bf16 (128 + q) in each half
  const uint32_t c128 = 0x43004300u;
  const __nv_bfloat162 q = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&biased),
                                   *reinterpret_cast<const __nv_bfloat162*>(&c128));
  return bf162_bits(__hfma2(q, dsc, ndm));
}

// Two signed bytes A and B of a word (given as its low seven bits and its sign bits) -> packed bf16 (d*qA, d*qB):
// 0x43 over the low seven bits is bf16 (128 + m), 0x43 over the sign bit is 128 or 256, their difference is q.
template <int SEL>
__device__ __forceinline__ uint32_t deq8_pair(uint32_t lo7, uint32_t sg, __nv_bfloat162 dh, __nv_bfloat162 dl) {
  const uint32_t biased = __byte_perm(lo7, 0x43434343u, SEL), off = __byte_perm(sg, 0x43434343u, SEL);
  const __nv_bfloat162 q = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&biased),
                                   *reinterpret_cast<const __nv_bfloat162*>(&off));
  return bf162_bits(__hfma2(q, dh, __hmul2(q, dl)));
}

constexpr int kTcMaxStages = 8;
constexpr int kTcWStages = 8;                        // most slots a ring of packed weight tiles has
// Shared-memory plan per token-tile size: the 256-token tile spends its memory on token stages (the
// copies' latency, not their bandwidth, bounds a K step) and keeps the other two areas small.
// With two CTAs per SM (the producer-bound MoE tiles of up to 128 tokens) every area is halved again.
// packed weight ring: WST slots when the launch names a depth, else 2 or 3
constexpr int tc_wstages(int tok, int ctas, int wst = 0) { return wst ? wst : ((tok > 128 || ctas > 1) ? 2 : 3); }
constexpr int tc_stage_tok(int tok, int ctas) {  // staging rows
  return (tok > 128 || ctas > 1) ? 64 : (tok < 128 ? tok : 128);
}
// Shared memory of a launch: token stages, output staging tile (none with a K split: those store from registers),
// packed-weight ring, f32 partial sums of a K split ([source rank][TOK / KS tokens][128 rows]), 1 KB for alignment.
constexpr size_t tc_smem_bytes(int tok, int stages, int ctas, int wst, int fmt, int ks) {
  return static_cast<size_t>(stages) * (tok * 128) + (ks > 1 ? 0 : static_cast<size_t>(tc_stage_tok(tok, ctas)) * 256) +
         static_cast<size_t>(tc_wstages(tok, ctas, wst)) * (128 * (fmt ? 8 * 34 : 144)) +
         (ks > 1 ? static_cast<size_t>(tok) * 512 : 0) + 1024;
}
// One slot of the packed-weight ring holds 256 K values of 128 rows: a Q4_K super-block (144 bytes) or eight
// Q8_0 blocks (272 bytes, the shortest run of 34-byte blocks that is a whole number of 16-byte pieces).
constexpr uint32_t kTcQ8RowBytes = 8 * 34;
constexpr uint32_t tc_wrow(int fmt) { return fmt ? kTcQ8RowBytes : UB_Q4K_BYTES; }
constexpr uint32_t tc_wbytes(int fmt) { return 128 * tc_wrow(fmt); }

constexpr int kTcMaxRuns = 256;  // token runs (consecutive alignment blocks of one expert) a grouped launch handles

// Grouped (MoE) launch: rows of A are in aligned order (position i holds the token of sorted_ids[i]).
struct TcGroup {
  const int32_t* experts_ids;   // [blocks] expert of each alignment block, -1 = not on this rank
  const int32_t* num_post_pad;  // [1] padded number of positions
  const int32_t* sorted_ids;    // [positions] slot id (token * top_k + j) or a padding value >= num_valid
  const float* topk_w;          // [num_valid] routed weights (mode 2, may be null)
  int block;                    // alignment block size (multiple of 16, <= TOK)
  int num_valid;                // T * top_k
  int rows_per_expert;          // weight rows per expert in the packed tensor (2 I for mode 1, N for mode 2)
};

struct TcRun {
  int e, m0, len;
};

struct TcShared {
  unsigned long long full[kTcMaxStages], empty[kTcMaxStages], tmem_full[2], tmem_empty[2];
  unsigned long long wfull[kTcWStages], wempty[kTcWStages];
  unsigned long long pfull, pempty;  // partial sums of a K split: all arrived here / all read everywhere else
  uint32_t tmem_base;
  int abort_flag;
  int nruns;
};

// TOK: tokens per tile (UMMA N): 64, 128 or 256.  STAGES: ring depth (token tiles in shared memory and
// weight stages in tensor memory advance together).
// MODE 0: dense y[M,N].  MODE 1 (grouped): weight tile = 64 gate rows + the 64 matching up rows of the run's
// expert, output act[position, N] = silu(gate) * up.  MODE 2 (grouped): output row sorted_ids[position],
// multiplied by the routed weight.  In the grouped modes M is the number of positions of A.
// CTAS: CTAs per SM the launch is planned for (2: each takes half of the SM's tensor memory and shared memory).
// WST: slots of the packed-weight ring (0: the default of tc_wstages).  Measured on B200: deeper rings do not
// help (MoE layer of 256 tokens, one CTA per SM: 3 -> 5 slots 589 -> 567 us; dense M = 2048: 2 -> 4 slots no
// change), the packed tiles are not what a K step waits for.
// FMT: 0 = Q4_K super-blocks, 1 = Q8_0 blocks (dense mode only).
// KS: K split (dense mode, up to 64 tokens).  A tile then belongs to a thread-block cluster of KS CTAs, each of which
// runs K / KS of the reduction into an accumulator of its own.  With so few tokens a K step costs the same 0.4 us of
// barrier round trips whatever it computes, and 14336 rows are only 112 tiles: the split puts more of those chains
// side by side (two CTAs per SM).  The partial sums meet in shared memory: token t of the tile belongs to rank
// t % KS, every rank writes its 128 partial sums of that token into the owner's buffer (st.async, counted in bytes on
// a barrier of the owner), and the owner adds the KS slots in rank order (deterministic) and stores the row.
// These launches also overlap with their neighbours in the stream (programmatic dependent launch): barriers and
// tensor memory are set up before the dependency wait, every access to global memory comes after it.
template <int TOK, int STAGES, int MODE, int CTAS, int WST, int FMT, int SETS, int KS>
__global__ void __launch_bounds__(tc_threads(SETS), CTAS)
qgemm_q4k_tc_kernel(__nv_bfloat16* __restrict__ y, int M, int N, int K, int early, int* err_word,
                    const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                    const TcGroup grp) {
  if (KS > 1) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {  // the copies' descriptors are on their way before the first copy needs them
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&x_map)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&w_map)) : "memory");
    }
  }
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  __shared__ TcShared sh;
  __shared__ TcRun runs[MODE == 0 ? 1 : kTcMaxRuns];
  __shared__ float run_w[MODE == 2 ? TOK : 1];
  __shared__ int run_dst[MODE == 2 ? TOK : 1];
  static_assert(STAGES <= kTcMaxStages, "barrier arrays");
  constexpr uint32_t kBBytes = TOK * 128;              // TOK token rows x 64 bf16
  constexpr int kStageTok = tc_stage_tok(TOK, CTAS);   // tokens the output staging tile holds
  constexpr int kWStages = tc_wstages(TOK, CTAS, WST);
  static_assert(kWStages <= kTcWStages, "barrier arrays");
  static_assert(FMT == 0 || MODE == 0, "the grouped modes take Q4_K experts");
  constexpr uint32_t kTcWBytes = tc_wbytes(FMT);
  constexpr uint32_t kWRow = tc_wrow(FMT);
  constexpr uint32_t kStagingOff = STAGES * kBBytes;   // [kStageTok tokens][128 weight rows] bf16
  constexpr uint32_t kWOff = kStagingOff + (KS > 1 ? 0 : kStageTok * 256);  // packed weight ring: [128 rows][144 bytes] each
  constexpr uint32_t kPartOff = kWOff + kWStages * kTcWBytes;  // [KS source ranks][TOK / KS tokens][128 rows] f32
  static_assert(KS == 1 || (MODE == 0 && TOK <= 64 && TOK % KS == 0), "K split: dense mode, few tokens");
  constexpr int kAccBufs = (TOK > 128 || CTAS > 1 || KS > 1) ? 1 : 2;  // accumulator buffers at the start of the allocation
  constexpr uint32_t kAccStride = 128;
  constexpr uint32_t kTmemCols = CTAS > 1 ? 256 : 512;        // columns this CTA allocates
  constexpr uint32_t kATmemCol = CTAS > 1 ? 128 : 256;        // first column of the weight stages (32 each)
  static_assert(TOK * kAccBufs <= static_cast<int>(kATmemCol) && kATmemCol + 32 * STAGES <= kTmemCols, "TMEM plan");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the swizzled tiles need 1024-byte alignment; the launch reserves 1 KB of slack for rounding the base up
  const uint32_t smem_raw = static_cast<uint32_t>(__cvta_generic_to_shared(tc_smem));
  const uint32_t smem_base = (smem_raw + 1023u) & ~1023u;
  unsigned char* const tiles = tc_smem + (smem_base - smem_raw);
  const uint32_t bars = static_cast<uint32_t>(__cvta_generic_to_shared(&sh));
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * kTcMaxStages + 8u * s; };
  auto tfull_bar = [&](int b) { return bars + 16u * kTcMaxStages + 8u * b; };
  auto tempty_bar = [&](int b) { return bars + 16u * kTcMaxStages + 16u + 8u * b; };
  auto wfull_bar = [&](int b) { return bars + 16u * kTcMaxStages + 32u + 8u * b; };
  auto wempty_bar = [&](int b) { return bars + 16u * kTcMaxStages + 32u + 8u * kTcWStages + 8u * b; };
  const uint32_t pfull_bar = bars + 16u * kTcMaxStages + 32u + 16u * kTcWStages;
  const uint32_t pempty_bar = pfull_bar + 8u;
  // K split: rank of this CTA in its cluster (= which part of K it takes); clusters walk over the tiles
  uint32_t krank = 0;
  if (KS > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(krank));
  const int vblock = static_cast<int>(blockIdx.x) / KS, vgrid = static_cast<int>(gridDim.x) / KS;
  volatile int* abort_flag = &sh.abort_flag;

  constexpr int kTileCols = MODE == 1 ? 64 : 128;  // output columns per tile
  const int w_tiles = (N + kTileCols - 1) / kTileCols, t_tiles = (M + TOK - 1) / TOK;
  const int ksteps = K / kTcBK / KS;  // of this CTA

  if (MODE != 0) {
    // Token runs: consecutive alignment blocks of one expert, merged up to TOK tokens.  Every CTA builds
    // the same table (expert ids staged through the output staging tile, then one thread scans them).
    int* ids = reinterpret_cast<int*>(tiles + kStagingOff);
    const int padded = *grp.num_post_pad;
    int nblocks = padded > 0 ? (padded + grp.block - 1) / grp.block : 0;
    if (nblocks > kTcMaxRuns) nblocks = kTcMaxRuns;  // the launcher guarantees this never cuts
    for (int i = threadIdx.x; i < nblocks; i += tc_threads(SETS)) ids[i] = grp.experts_ids[i];
    __syncthreads();
    if (threadIdx.x == 0) {
      int n = 0;
      for (int b = 0; b < nblocks; b++) {
        const int e = ids[b];
        if (e < 0) continue;
        if (n > 0 && runs[n - 1].e == e && runs[n - 1].m0 + runs[n - 1].len == b * grp.block &&
            runs[n - 1].len + grp.block <= TOK) {
          runs[n - 1].len += grp.block;
        } else {
          runs[n].e = e, runs[n].m0 = b * grp.block, runs[n].len = grp.block;
          n++;
        }
      }
      sh.nruns = n;
    }
    __syncthreads();
  }
  const int ntiles = MODE == 0 ? w_tiles * t_tiles : sh.nruns * w_tiles;
  // tile -> (first token row of A, valid tokens, first weight row in the packed tensor, first output column)
  auto tile_info = [&](int tile, int& m0, int& valid, int& wrow0, int& n0) {
    if (MODE == 0) {
      const int wt = tile / t_tiles, tt = tile - wt * t_tiles;
      m0 = tt * TOK, valid = min(TOK, M - m0), wrow0 = wt * 128, n0 = wt * 128;
    } else {
      const int run = tile / w_tiles, wt = tile - run * w_tiles;
      const TcRun r = runs[run];
      m0 = r.m0, valid = r.len, n0 = wt * kTileCols, wrow0 = r.e * grp.rows_per_expert + n0;
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      tc_mbar_init(full_bar(s), kTcProducerWarps + 1);  // eight weight warps + the token copy's expect_tx
      tc_mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; b++) {
      tc_mbar_init(tfull_bar(b), 1);
      tc_mbar_init(tempty_bar(b), 4);
    }
    for (int b = 0; b < kWStages; b++) {
      tc_mbar_init(wfull_bar(b), 1);
      tc_mbar_init(wempty_bar(b), kTcProducerWarps * SETS);
    }
    tc_mbar_init(pfull_bar, 1);
    tc_mbar_init(pempty_bar, (KS - 1) * 128 + (KS == 1));
    sh.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (KS > 1) tc_cluster_sync();  // the other ranks' barriers exist before anything arrives on them
  if (warp == 0) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(&sh.tmem_base));
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sh.tmem_base;
  // Everything below reads what the previous kernel may have written or writes what it may still read; only the
  // thread that issues the copies first requests its first packed weight tiles (early: nothing on the stream
  // writes the weights), whose way from memory is the longest wait of a launch.
  const bool copy_warp = warp > 4 + kTcProducerWarps * SETS;
  if (KS > 1 && !(early && copy_warp)) asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0, acc_phase = 0;
      int buf = 0;
      bool ok = true;
      for (int tile = vblock; tile < ntiles && ok; tile += vgrid) {
        int m0_, valid, wrow0_, n0_;
        tile_info(tile, m0_, valid, wrow0_, n0_);
        // UMMA N = the tile's valid tokens rounded up to 16 (a ragged last tile costs less)
        const uint32_t n_mma = valid >= TOK ? TOK : static_cast<uint32_t>((valid + 15) & ~15);
        // instruction descriptor: D = f32, A = B = bf16, both K-major, N = n_mma, M = 128
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((n_mma >> 3) << 17) | (8u << 24);
        ok = tc_wait(tempty_bar(buf), acc_phase ^ 1, abort_flag);  // epilogue has drained this accumulator
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf) * kAccStride;
        for (int ks = 0; ks < ksteps; ks++) {
          ok = tc_wait(full_bar(s), phase, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t b_desc = make_sw128_desc(smem_base + s * kBBytes);
          const uint32_t a_tmem = tmem_base + kATmemCol + 32u * s;
#pragma unroll
          for (int j = 0; j < 4; j++)  // K = 16 per instruction: 8 TMEM columns of A, 32 bytes of a B row
            umma_bf16_ts(d_tmem, a_tmem + 8u * j, b_desc + 2 * j, idesc, (ks > 0 || j > 0) ? 1u : 0u);
          umma_commit(empty_bar(s));  // stage is free once these MMAs have read it
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(tfull_bar(buf));  // accumulator complete
        if (++buf == kAccBufs) {
          buf = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp <= 4) {
    // ------------------------------------------------------------ epilogue (TMEM lanes 32*(warp%4) ..)
    const int lane_base = 32 * (warp & 3);
    const int ew = warp - 1;  // 0..3: which quarter of the tile's tokens this warp writes out
    unsigned char* const staging = tiles + kStagingOff;
    const bool vec_ok = (N % 8) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    bool ok = true;
    if constexpr (KS > 1) {
      // K split: partial sums to their owners, then this rank's tokens (t % KS == krank) summed in rank order
      constexpr int kSlots = TOK / KS;  // tokens a rank owns at most
      const int row = lane_base + lane;
      const uint32_t part_s = smem_base + kPartOff;
      const float* const part = reinterpret_cast<const float*>(tiles + kPartOff);
      uint32_t it = 0;
      auto agree = [&](bool mine_ok) {  // the four warps take the same decision
        uint32_t all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 1, 128, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(all_ok)
            : "r"(mine_ok ? 1u : 0u)
            : "memory");
        return all_ok != 0;
      };
      for (int tile = vblock; tile < ntiles && ok; tile += vgrid, it++) {
        int m0, valid, wrow0_, n0;
        tile_info(tile, m0, valid, wrow0_, n0);
        bool mine = tc_wait(tfull_bar(0), acc_phase, abort_flag);
        // the buffers everywhere have been read for the previous tile before anybody writes them again
        if (mine && it > 0) mine = tc_wait_cluster(pempty_bar, (it - 1) & 1, abort_flag);
        ok = agree(mine);
        if (!ok) break;
        // bytes the other ranks will send for the tokens this rank owns
        if (warp == 1 && lane == 0) {
          const int nown = (valid - static_cast<int>(krank) + KS - 1) / KS;
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pfull_bar),
                       "r"(static_cast<uint32_t>((KS - 1) * (nown > 0 ? nown : 0) * 512))
                       : "memory");
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c = 0; c < valid; c += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_base + (static_cast<uint32_t>(lane_base) << 16) + c, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const int t = c + j;
            if (t < valid) {
              const uint32_t owner = static_cast<uint32_t>(t) & (KS - 1);
              const uint32_t a = part_s + ((krank * kSlots + (t / KS)) * 128 + row) * 4;
              if (owner == krank)
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(v[j]) : "memory");
              else
                tc_peer_store_tx(tc_peer_addr(a, owner), v[j], tc_peer_addr(pfull_bar, owner));
            }
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) tc_mbar_arrive(tempty_bar(0));  // this warp's lanes of the accumulator are drained
        acc_phase ^= 1;
        ok = agree(tc_wait_cluster(pfull_bar, it & 1, abort_flag));
        if (!ok) break;
        for (int t = krank, i = 0; t < valid; t += KS, i++) {
          float f = 0.f;
#pragma unroll
          for (int r = 0; r < KS; r++) f += part[(r * kSlots + i) * 128 + row];
          if (n0 + row < N) y[static_cast<size_t>(m0 + t) * N + n0 + row] = __float2bfloat16_rn(f);
        }
        if (tile + vgrid < ntiles) {  // the buffers here may be written for the next tile
#pragma unroll
          for (uint32_t d = 0; d < KS; d++)
            if (d != krank) tc_peer_arrive(tc_peer_addr(pempty_bar, d));
        }
      }
    } else
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      int m0, valid, wrow0_, n0;
      tile_info(tile, m0, valid, wrow0_, n0);
      if (MODE == 2) {
        // destination row and routed weight of every token of the run (visible after the barrier below)
        for (int tk = threadIdx.x - 32; tk < valid; tk += 128) {
          const int sid = grp.sorted_ids[m0 + tk];
          const bool live = sid >= 0 && sid < grp.num_valid;
          run_dst[tk] = live ? sid : -1;
          run_w[tk] = live ? (grp.topk_w ? grp.topk_w[sid] : 1.f) : 0.f;
        }
      }
      {
        // all four epilogue warps take the same decision, so nobody is left alone at the named barrier
        const uint32_t mine = tc_wait(tfull_bar(buf), acc_phase, abort_flag) ? 1u : 0u;
        uint32_t all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 1, 128, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(all_ok)
            : "r"(mine)
            : "memory");
        ok = all_ok != 0;
      }
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // accumulator -> bf16 -> staging[token][weight row] -> y, kStageTok tokens at a time.  A warp's 32
      // lanes write 64 contiguous bytes of a staging row; token rows leave as 256 contiguous bytes.
      __nv_bfloat16* const st_col = reinterpret_cast<__nv_bfloat16*>(staging) + lane_base + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < valid; c0 += kStageTok) {
        const int part = min(kStageTok, valid - c0);
#pragma unroll 1
        for (int c = 0; c < part; c += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_base + (static_cast<uint32_t>(lane_base) << 16) + static_cast<uint32_t>(buf) * kAccStride +
                        c0 + c, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 32; j++) {
            float f = __uint_as_float(v[j]);
            if (MODE == 2) f *= run_w[c0 + c + j];
            st_col[(c + j) * 128] = __float2bfloat16_rn(f);
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps: staging complete
        // after the last part the next tile's MMAs may overwrite the accumulator
        if (c0 + kStageTok >= valid && lane == 0) tc_mbar_arrive(tempty_bar(buf));
        if (MODE == 1) {
          // staging row = 64 gate values then 64 up values of one position: eight lanes per position
          const int ch = lane & 7;
          const bool n_in = n0 + 8 * ch < N;
          for (int t = 4 * ew + (lane >> 3); t < part; t += 16) {
            const uint4 gv = *reinterpret_cast<const uint4*>(staging + t * 256 + ch * 16);
            const uint4 uv = *reinterpret_cast<const uint4*>(staging + t * 256 + 128 + ch * 16);
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
            uint32_t ow[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const float g0 = __uint_as_float(gw[i] << 16), g1 = __uint_as_float(gw[i] & 0xFFFF0000u);
              const float u0 = __uint_as_float(uw[i] << 16), u1 = __uint_as_float(uw[i] & 0xFFFF0000u);
              const __nv_bfloat162 o2 =
                  __floats2bfloat162_rn(__fdividef(g0, 1.f + __expf(-g0)) * u0, __fdividef(g1, 1.f + __expf(-g1)) * u1);
              ow[i] = bf162_bits(o2);
            }
            if (n_in)
              *reinterpret_cast<uint4*>(y + static_cast<size_t>(m0 + c0 + t) * N + n0 + 8 * ch) =
                  make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
        } else if (vec_ok) {
          const int ch = lane & 15;
          const bool n_in = n0 + 8 * ch < N;
          for (int t = 2 * ew + (lane >> 4); t < part; t += 8) {
            const uint4 val = *reinterpret_cast<const uint4*>(staging + t * 256 + ch * 16);
            const int row = MODE == 2 ? run_dst[c0 + t] : m0 + c0 + t;
            if (n_in && row >= 0) *reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * N + n0 + 8 * ch) = val;
          }
        } else {
          for (int t = ew; t < part; t += 4) {
            const int row = MODE == 2 ? run_dst[c0 + t] : m0 + c0 + t;
#pragma unroll
            for (int r = lane; r < 128; r += 32)
              if (n0 + r < N && row >= 0)
                y[static_cast<size_t>(row) * N + n0 + r] = reinterpret_cast<const __nv_bfloat16*>(staging)[t * 128 + r];
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // staging may be overwritten
      }
      if (++buf == kAccBufs) {
        buf = 0;
        acc_phase ^= 1;
      }
    }
  } else if (warp <= 4 + kTcProducerWarps * SETS) {
    // ------------------------------------------------------------ weight producers (256 threads per set)
    // One flat loop over (tile, super-block); the super-block's four K steps (its four 64-value groups) are
    // dealt round robin to the producer sets.  Packed weights arrive in shared memory as
    // [128 rows][144 bytes] per super-block; a thread owns one weight row (= its TMEM lane) and one nibble
    // half and reads its row's header and 32-byte pieces from there (rows are 144 bytes apart, so a
    // quarter-warp's 16-byte reads hit all 32 banks once).
    static_assert(STAGES % SETS == 0, "a set must return to the same stages every ring turn");
    // weight row inside the tile = the TMEM lane this warp may access (32 * (warp % 4) + lane);
    // half: 0 = low nibbles (even sub-blocks), 1 = high nibbles
    const int wrow = 32 * (warp & 3) + lane, half = ((warp - 5) >> 2) & 1, set = (warp - 5) >> 3;
    const int nsb = (K >> 8) / KS;
    const int my_tiles = vblock < ntiles ? (ntiles - vblock + vgrid - 1) / vgrid : 0;
    const int total_sb = my_tiles * nsb;  // super-block iterations
    const unsigned char* const w_ring = tiles + kWOff + wrow * kWRow;
    const uint32_t a_lane = tmem_base + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + kATmemCol;

    int s = set;  // stage of the step being dequantised
    uint32_t phase = 0;
    int ws = 0;  // packed-weight ring slot
    uint32_t wphase = 0;
    bool ok = true;

    // one super-block (four K steps); HALF is a compile-time copy of `half` so that nibble selection and
    // the scale bytes' positions are immediate operands.  (Measured on B200: one rolled code path for both
    // halves, with the half as a run-time shift, is no faster, although instruction fetch is the second largest
    // stall of the grouped launches.)
    auto super_block = [&](auto half_c, auto set_c) {
      constexpr int HALF = decltype(half_c)::value, SET = decltype(set_c)::value;
      ok = __all_sync(0xFFFFFFFFu, tc_wait(wfull_bar(ws), wphase, abort_flag));
      if (!ok) return;
      const unsigned char* blk = w_ring + ws * kTcWBytes;
      uint32_t scw[2] = {0, 0}, mnw[2] = {0, 0};
      float d = 0.f, dmin = 0.f;
      if (FMT == 0) {
        const uint4 hdr = *reinterpret_cast<const uint4*>(blk);  // rows past N arrive as zeros: d = dmin = 0
        d = half_bits_to_f32(hdr.x), dmin = half_bits_to_f32(hdr.x >> 16);
        q4k_unpack_scales(hdr.y, hdr.z, hdr.w, scw[0], scw[1], mnw[0], mnw[1]);
      }
#pragma unroll
      for (int Gi = 0; Gi < 4 / SETS; Gi++) {
        constexpr int kSets = SETS;
        const int G = kSets * Gi + SET;
        uint32_t ot[16];  // this thread's 32 values of the step = 16 TMEM columns of packed pairs
        if (FMT == 0) {
          const int j = 2 * G + HALF;
          const uint32_t sc = (scw[j >> 2] >> (8 * (j & 3))) & 0xFF, mn = (mnw[j >> 2] >> (8 * (j & 3))) & 0xFF;
          const __nv_bfloat162 dsc = __float2bfloat162_rn(d * static_cast<float>(sc));
          const __nv_bfloat162 ndm = __float2bfloat162_rn(-dmin * static_cast<float>(mn));
          const uint4 qa = *reinterpret_cast<const uint4*>(blk + 16 + 32 * G);
          const uint4 qb = *reinterpret_cast<const uint4*>(blk + 32 + 32 * G);
          const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
          for (int cc = 0; cc < 4; cc++) {  // 8 values = bytes 8cc .. 8cc+7
            const uint32_t w0 = HALF ? (w[2 * cc] >> 4) & 0x0F0F0F0Fu : w[2 * cc] & 0x0F0F0F0Fu;
            const uint32_t w1 = HALF ? (w[2 * cc + 1] >> 4) & 0x0F0F0F0Fu : w[2 * cc + 1] & 0x0F0F0F0Fu;
            ot[4 * cc] = deq_pair<0x4140>(w0, dsc, ndm);
            ot[4 * cc + 1] = deq_pair<0x4342>(w0, dsc, ndm);
            ot[4 * cc + 2] = deq_pair<0x4140>(w1, dsc, ndm);
            ot[4 * cc + 3] = deq_pair<0x4342>(w1, dsc, ndm);
          }
        } else {
          // Q8_0 block 2G + HALF of the row's eight: 34 bytes at byte 34 (2G + HALF) of a 272-byte row, i.e. three
          // aligned 16-byte pieces from piece (34 (2G + HALF)) / 16; inside them the f16 scale sits at byte
          // 4G + 2 HALF and the 32 signed bytes follow it, so the even blocks' words straddle two loaded words.
          const uint4* pc = reinterpret_cast<const uint4*>(blk) + ((34 * (2 * G + HALF)) >> 4);
          const uint4 p0 = pc[0], p1 = pc[1], p2 = pc[2];
          const uint32_t c[12] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w, p2.x, p2.y, p2.z, p2.w};
          const float df = half_bits_to_f32(HALF ? c[G] >> 16 : c[G]);
          const __nv_bfloat16 dh1 = __float2bfloat16_rn(df);
          // d = dh + dl in two bf16 pieces: fma(q, dh, q * dl) is the f32 product d * q rounded once
          const __nv_bfloat162 dh = __bfloat162bfloat162(dh1);
          const __nv_bfloat162 dl = __float2bfloat162_rn(df - __bfloat162float(dh1));
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const uint32_t w = HALF ? c[G + 1 + i] : __funnelshift_r(c[G + i], c[G + i + 1], 16);
            const uint32_t lo7 = w & 0x7F7F7F7Fu, sg = w & 0x80808080u;
            ot[2 * i] = deq8_pair<0x4140>(lo7, sg, dh, dl);
            ot[2 * i + 1] = deq8_pair<0x4342>(lo7, sg, dh, dl);
          }
        }
        // the MMAs that read this weight stage one ring turn ago must have completed
        ok = __all_sync(0xFFFFFFFFu, tc_wait(empty_bar(s), phase ^ 1, abort_flag));
        if (!ok) return;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem_st16(a_lane + 32u * s + 16u * HALF, ot);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) tc_mbar_arrive(full_bar(s));
        s += SETS;
        if (s >= STAGES) {
          s -= STAGES;
          phase ^= 1;
        }
      }
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(wempty_bar(ws));  // this warp has read all it needs from the slot
      if (++ws == kWStages) {
        ws = 0;
        wphase ^= 1;
      }
    };
    using I0 = std::integral_constant<int, 0>;
    using I1 = std::integral_constant<int, 1>;
    if (SETS == 1 || set == 0) {
      if (half) {
        for (int q = 0; q < total_sb && ok; q++) super_block(I1{}, I0{});
      } else {
        for (int q = 0; q < total_sb && ok; q++) super_block(I0{}, I0{});
      }
    } else if constexpr (SETS > 1) {
      if (half) {
        for (int q = 0; q < total_sb && ok; q++) super_block(I1{}, I1{});
      } else {
        for (int q = 0; q < total_sb && ok; q++) super_block(I0{}, I1{});
      }
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  } else {
    // ------------------------------------------------------------ bulk copies (one lane)
    // Packed weight tiles run kWStages - 1 super-blocks ahead of the token tiles; token tiles run as far
    // ahead of the MMA as the ring allows.
    if (lane == 0) {
      const int nsb = (K >> 8) / KS, sb0 = static_cast<int>(krank) * nsb;  // this CTA's super-blocks of a row
      const int my_tiles = vblock < ntiles ? (ntiles - vblock + vgrid - 1) / vgrid : 0;
      const int total_sb = my_tiles * nsb;
      int s = 0, ws = 0;
      uint32_t phase = 0, wphase = 0;
      bool ok = true;
      int wq_next = 0;  // next super-block (flat index) whose packed weights have not been requested
      auto issue_w = [&]() {
        const int ti = wq_next / nsb, sb = sb0 + wq_next - ti * nsb;
        int m0_, valid_, wrow0, n0_;
        tile_info(vblock + ti * vgrid, m0_, valid_, wrow0, n0_);
        ok = tc_wait(wempty_bar(ws), wphase ^ 1, abort_flag);
        if (!ok) return;
        const uint32_t bar = wfull_bar(ws);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kTcWBytes) : "memory");
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
                "r"(smem_base + kWOff + ws * kTcWBytes),
            "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(bar), "r"(sb * (FMT ? kWRow / 2 : kWRow)), "r"(wrow0)
            : "memory");
        if (MODE == 1)  // second half of the tile: the up rows matching the 64 gate rows (box = 64 rows)
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
                  "r"(smem_base + kWOff + ws * kTcWBytes + kTcWBytes / 2),
              "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(bar), "r"(sb * kWRow), "r"(wrow0 + N)
              : "memory");
        wq_next++;
        if (++ws == kWStages) {
          ws = 0;
          wphase ^= 1;
        }
      };
      for (int i = 0; i < kWStages - 1 && wq_next < total_sb && ok; i++) issue_w();
      if (KS > 1 && early) asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int q = 0; q < total_sb && ok; q++) {
        if (wq_next < total_sb) issue_w();
        if (!ok) break;
        const int ti = q / nsb, sb = sb0 + q - ti * nsb;
        int m0, valid_, wrow0_, n0_;
        tile_info(vblock + ti * vgrid, m0, valid_, wrow0_, n0_);
        for (int G = 0; G < 4; G++) {
          ok = tc_wait(empty_bar(s), phase ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t bar = full_bar(s);
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kBBytes) : "memory");
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
                  "r"(smem_base + s * kBBytes),
              "l"(reinterpret_cast<uint64_t>(&x_map)), "r"(bar), "r"((sb * 4 + G) * kTcBK), "r"(m0)
              : "memory");
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  }

  // ---- teardown: every role arrives here, whether it finished or gave up ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // nobody leaves while another rank may still write or arrive here (after a wait that gave up; otherwise every
  // rank has received all it was sent by now)
  if (KS > 1) tc_cluster_sync_relaxed();
  if (threadIdx.x == 0 && sh.abort_flag) report_device_error(err_word, UB_ERR_TIMEOUT);
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// cuTensorMapEncodeTiled, resolved once through the runtime (no link-time dependency on libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  std::lock_guard<std::mutex> lk(mu);
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

template <int TOK, int STAGES, int MODE, int CTAS = 1, int WST = 0, int FMT = 0, int SETS = 1, int KS = 1>
int launch_tc(void* y, const void* x, const void* wq, int M, int N, int K, const TcGroup& grp, int w_rows_total,
              cudaStream_t s, int early = 0) {
  constexpr size_t smem = tc_smem_bytes(TOK, STAGES, CTAS, WST, FMT, KS);
  static_assert(smem <= 227 * 1024 / CTAS, "shared memory plan");
  const int sms = ub::num_sms();
  int grid = sms * CTAS;  // grouped launches learn their tile count on the device; idle CTAs leave at once
  if (MODE == 0) {
    const int tiles = ((N + 127) / 128) * ((M + TOK - 1) / TOK);
    const int slots = KS > 1 ? sms * CTAS / KS : sms;  // clusters (CTAs) resident at once
    grid = (tiles < slots ? tiles : slots) * KS;
  }
  // token matrix as a 2-D tensor map: inner dimension K (bf16), outer M; box = 64 x TOK, 128-byte swizzle;
  // rows beyond M read as zeros
  CUtensorMap map;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return ub::fail(UB_ERR_UNSUPPORTED);
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(TOK)};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return ub::fail(UB_ERR_UNSUPPORTED);
  // packed weights as a 2-D byte tensor: inner dimension = one row's bytes, outer = all weight rows (of all
  // experts); box = one super-block (144 bytes) of 128 rows (64 for the gate/up halves of mode 1), no
  // swizzle; rows beyond the tensor read as zeros.  Q8_0: a box of eight blocks is 272 bytes, wider than the
  // 256 elements a box may have, so that map counts 16-bit elements (136 per box).
  CUtensorMap wmap;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(K / UB_QK_K) * tc_wrow(FMT);
  const cuuint64_t wdims[2] = {FMT ? row_bytes / 2 : row_bytes, static_cast<cuuint64_t>(w_rows_total)};
  const cuuint64_t wstrides[1] = {row_bytes};
  const cuuint32_t wbox[2] = {FMT ? tc_wrow(FMT) / 2 : tc_wrow(FMT), MODE == 1 ? 64u : 128u};
  if (enc(&wmap, FMT ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(wq), wdims,
          wstrides, wbox, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return ub::fail(UB_ERR_UNSUPPORTED);
  auto kernel = qgemm_q4k_tc_kernel<TOK, STAGES, MODE, CTAS, WST, FMT, SETS, KS>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  if (KS > 1) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid), cfg.blockDim = dim3(tc_threads(SETS)), cfg.dynamicSmemBytes = smem, cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = KS, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 2;
    e = cudaLaunchKernelEx(&cfg, kernel, static_cast<__nv_bfloat16*>(y), M, N, K, early, ub::device_error_word(), map, wmap,
                           grp);
    if (e != cudaSuccess) {
      ub::set_cuda_error(e);
      return ub::fail(UB_ERR_CUDA);
    }
    return ub::check_launch();
  }
  kernel<<<grid, tc_threads(SETS), smem, s>>>(static_cast<__nv_bfloat16*>(y), M, N, K, 0, ub::device_error_word(), map,
                                        wmap, grp);
  return ub::check_launch();
}

// xg[i, :] = hidden[sorted_ids[i] / top_k, :] for the positions the alignment produced (zeros for padding)
__global__ void __launch_bounds__(256) moe_gather_rows_kernel(__nv_bfloat16* __restrict__ xg,
                                                              const __nv_bfloat16* __restrict__ hidden,
                                                              const int32_t* __restrict__ sorted_ids,
                                                              const int32_t* __restrict__ num_post_pad, int num_valid,
                                                              int top_k, int H) {
  const int i = blockIdx.x;
  if (i >= *num_post_pad) return;
  const int sid = sorted_ids[i];
  const bool live = sid >= 0 && sid < num_valid;
  const uint4* src = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(live ? sid / top_k : 0) * H);
  uint4* dst = reinterpret_cast<uint4*>(xg + static_cast<size_t>(i) * H);
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = live ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
}

}  // namespace

namespace ub {

// cuTensorMapEncodeTiled of the running driver as an untyped pointer (null when unavailable), for the other
// kernels of this library that build tensor maps.
void* tensor_map_encoder() { return reinterpret_cast<void*>(encode_tiled_fn()); }

// y (bf16) [M,N] = x (bf16) [M,K] . dequant(Wq)^T on tcgen05; K % 256 == 0, pointers 16-byte aligned.
// Returns UB_ERR_UNSUPPORTED when the driver offers no tensor-map encoder (the caller falls back).
int q4k_gemm_tc(void* y, const void* x, const void* wq, int M, int N, int K, bool fresh, cudaStream_t s) {
  const TcGroup none = {nullptr, nullptr, nullptr, nullptr, 0, 0, 0};
  if (M <= 64) {
    // few tokens: K split over clusters, two CTAs per SM; the widest split that still fills one round of CTA slots
    const int tiles = (N + 127) / 128, slots = 2 * ub::num_sms(), nsb = K / UB_QK_K;
    const int early = fresh ? 0 : 1;
    // Measured on B200 at 16 tokens: 14336x4096 27.4 us unsplit, 23.1 us in two; 4096x4096 26.4 / 19.3 / 12.7 / 11.3 us
    // unsplit / in two / four / eight.
    int ks = 1;
    while (ks < 8 && tiles * (2 * ks) <= slots && nsb % (2 * ks) == 0 && nsb / (2 * ks) >= 2) ks *= 2;
    if (ks == 1 && nsb % 2 == 0) ks = 2;
    if (ks == 8) return launch_tc<64, 4, 0, 2, 0, 0, 1, 8>(y, x, wq, M, N, K, none, N, s, early);
    if (ks == 4) return launch_tc<64, 4, 0, 2, 0, 0, 1, 4>(y, x, wq, M, N, K, none, N, s, early);
    if (ks == 2) return launch_tc<64, 4, 0, 2, 0, 0, 1, 2>(y, x, wq, M, N, K, none, N, s, early);
    return launch_tc<64, 6, 0>(y, x, wq, M, N, K, none, N, s);
  }
  if (M <= 128) return launch_tc<128, 6, 0>(y, x, wq, M, N, K, none, N, s);
  return launch_tc<256, 5, 0>(y, x, wq, M, N, K, none, N, s);
}

// Same product for Q8_0 rows (K/32 blocks of 34 bytes); K % 256 == 0 (a row must be whole 16-byte pieces) and wq
// 16-byte aligned, else UB_ERR_UNSUPPORTED and the caller keeps the decode kernel.  The 272-byte slots of the
// packed ring leave room for four token stages at 256 tokens.  Measured on B200, 4096x4096 with 512 tokens
// (64 tiles of 256 tokens on 148 SMs): 505 TFLOP/s; with 128-token tiles (128 tiles) 400: the producers'
// work per flop doubles, which costs more than the idle SMs.
int q8_0_gemm_tc(void* y, const void* x, const void* wq, int M, int N, int K, bool fresh, cudaStream_t s) {
  if (K % UB_QK_K || (reinterpret_cast<uintptr_t>(wq) & 15)) return UB_ERR_UNSUPPORTED;
  const TcGroup none = {nullptr, nullptr, nullptr, nullptr, 0, 0, 0};
  if (M <= 64) {
    const int tiles = (N + 127) / 128, slots = ub::num_sms(), nsb = K / UB_QK_K;
    const int early = fresh ? 0 : 1;
    int ks = 1;
    while (ks < 8 && tiles * (2 * ks) <= slots && nsb % (2 * ks) == 0 && nsb / (2 * ks) >= 2) ks *= 2;
    if (ks == 8) return launch_tc<64, 6, 0, 1, 0, 1, 1, 8>(y, x, wq, M, N, K, none, N, s, early);
    if (ks == 4) return launch_tc<64, 6, 0, 1, 0, 1, 1, 4>(y, x, wq, M, N, K, none, N, s, early);
    if (ks == 2) return launch_tc<64, 6, 0, 1, 0, 1, 1, 2>(y, x, wq, M, N, K, none, N, s, early);
    return launch_tc<64, 6, 0, 1, 0, 1>(y, x, wq, M, N, K, none, N, s);
  }
  if (M <= 128) return launch_tc<128, 6, 0, 1, 2, 1>(y, x, wq, M, N, K, none, N, s);
  return launch_tc<256, 4, 0, 1, 0, 1>(y, x, wq, M, N, K, none, N, s);
}

// Limits of the grouped tcgen05 path; outside them the caller keeps the mma.sync kernels.
bool q4k_moe_tc_supported(int positions, int K, int N, int block) {
  return encode_tiled_fn() != nullptr && block > 0 && block % 16 == 0 && block <= 128 && K % UB_QK_K == 0 &&
         N % 8 == 0 && (positions + block - 1) / block <= kTcMaxRuns;
}

// Gathers hidden rows into aligned order: xg[positions, H].
int moe_gather_rows(void* xg, const void* hidden, const int32_t* sorted_ids, const int32_t* num_post_pad, int positions,
                    int num_valid, int top_k, int H, cudaStream_t s) {
  if (positions <= 0) return UB_OK;
  moe_gather_rows_kernel<<<positions, 256, 0, s>>>(static_cast<__nv_bfloat16*>(xg),
                                                   static_cast<const __nv_bfloat16*>(hidden), sorted_ids, num_post_pad,
                                                   num_valid, top_k, H);
  return ub::check_launch();
}

// Grouped expert GEMM over rows in aligned order (A[positions, K] bf16).
//   act_silu_mul != 0: Bq = [E][2N rows: gate then up][K], C[position, N] = silu(gate) * up
//   else:              Bq = [E][N rows][K], C[sorted_ids[position], N] = (A . W^T) * topk_w[slot]
int q4k_moe_gemm_tc(void* C, const void* A, const void* Bq, const float* topk_w, const int32_t* sorted_ids,
                    const int32_t* experts_ids, const int32_t* num_post_pad, int positions, int K, int N, int E,
                    int num_valid, int block, int act_silu_mul, cudaStream_t s) {
  if (!q4k_moe_tc_supported(positions, K, N, block)) return UB_ERR_UNSUPPORTED;
  TcGroup g;
  g.experts_ids = experts_ids, g.num_post_pad = num_post_pad, g.sorted_ids = sorted_ids, g.topk_w = topk_w;
  g.block = block, g.num_valid = num_valid, g.rows_per_expert = act_silu_mul ? 2 * N : N;
  const int rows_total = E * g.rows_per_expert;
  // token runs are capped at the tile's token count: short runs (few tokens per expert) take the 128 tile
  const bool small = num_valid / (E > 0 ? E : 1) <= 128;
  if (act_silu_mul)
    return small ? launch_tc<128, 3, 1, 2>(C, A, Bq, positions, N, K, g, rows_total, s)
                 : launch_tc<256, 5, 1>(C, A, Bq, positions, N, K, g, rows_total, s);
  return small ? launch_tc<128, 3, 2, 2>(C, A, Bq, positions, N, K, g, rows_total, s)
               : launch_tc<256, 5, 2>(C, A, Bq, positions, N, K, g, rows_total, s);
}

}  // namespace ub
