// Grouped Q4_K GEMM on warp-level tensor-core mma (m16n8k16 bf16, f32 accumulate): the expert GEMMs
// of the fused MoE layer and the general-M fallback of the quantized matmul.
//
// Contract = invoke_fused_moe_bf16 (kernels/fused_moe_host.cpp:43-250) with the expert weights given
// as Q4_K blocks instead of dense bf16: for aligned block b with expert e = experts_ids[b],
//   C[sid,:] = A[sid / topk_str,:] . dequant(Bq[e])^T  (x topk_weights[sid] when mul_routed_weight),
// e == -1 zero-fills, slots >= topk_ids_size are padding.  With act_silu_mul the weight rows are
// [gate; up] and the epilogue writes silu(gate)*up (kernels/topsaten_ops_wrapper.cpp:375-391), each
// GEMM result rounded to bf16 first, as the reference's separate kernels do.
//
// One CTA = one block of slots x (4 warps x 16 weight rows).  Token rows are the mma M operand, weight
// rows the N operand.  Per 64-value Q4_K group lane (g,t) reads 8 bytes of nibbles of weight row g
// (bytes 8t..8t+7): their low nibbles are k = 8t..8t+7 of sub-block 2G, their high nibbles the same k
// of sub-block 2G+1, which feeds four mma steps.  Activations are read with the same k assignment, so
// the reduction order inside a group is permuted but complete.  Weights are dequantised exactly in
// f32 ((d*sc)*q - dmin*m) and rounded once to bf16 for the tensor core.
#include "common.cuh"

namespace {

using namespace ub;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// exact float(nibble) for byte I of a word masked with 0x0F0F0F0F
template <int I>
__device__ __forceinline__ float nib_exact(uint32_t w4) {
  return __uint_as_float(__byte_perm(w4, 0x4B000000u, 0x7440u | I)) - 8388608.0f;
}

// Four nibbles (one masked word) -> two bf16x2 registers holding (d*q0-m, d*q1-m), (d*q2-m, d*q3-m)
__device__ __forceinline__ void dequant4(uint32_t w4, float d, float m, uint32_t& p01, uint32_t& p23) {
  p01 = pack_bf16(__fsub_rn(__fmul_rn(d, nib_exact<0>(w4)), m), __fsub_rn(__fmul_rn(d, nib_exact<1>(w4)), m));
  p23 = pack_bf16(__fsub_rn(__fmul_rn(d, nib_exact<2>(w4)), m), __fsub_rn(__fmul_rn(d, nib_exact<3>(w4)), m));
}

constexpr int kMT = 4;  // 16-row token tiles per pass

// IDENTITY: plain matmul (no routing): slot r of block b is row b*block + r, expert 0.
// ACT: weight rows [gate (D rows); up (D rows)], N = 2D, C row stride D.
template <bool IDENTITY, bool ACT>
__global__ void __launch_bounds__(128) q4k_grouped_mma_kernel(
    __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ A, const uint8_t* __restrict__ Bq,
    const float* __restrict__ topk_w, const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ experts_ids,
    const int32_t* __restrict__ num_post_pad, int K, int N, int E, int topk_ids_size, int top_k, int block,
    int mul_routed_weight, int* err_word) {
  const int blk = blockIdx.x;
  int e = 0;
  if (!IDENTITY) {
    const int padded = *num_post_pad;
    if (padded <= 0 || blk * block >= padded) return;
    e = experts_ids[blk];
  } else if (blk * block >= topk_ids_size) {
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int D = ACT ? N / 2 : N;       // output columns
  const int cols_per_warp = ACT ? 8 : 16;
  const int n_warp = (blockIdx.y * 4 + warp) * cols_per_warp;  // first output column of this warp
  const int32_t* sids = IDENTITY ? nullptr : sorted_ids + static_cast<size_t>(blk) * block;

  if (e < 0 || e >= E) {
    if (e != -1 && threadIdx.x == 0) report_device_error(err_word, UB_ERR_BAD_INDEX);
    for (int r = 0; r < block; r++) {
      const int sid = sids[r];
      if (sid < 0 || sid >= topk_ids_size) continue;
      for (int n = n_warp + lane; n < n_warp + cols_per_warp && n < D; n += 32)
        C[static_cast<size_t>(sid) * D + n] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  if (n_warp >= D) return;

  const int topk_str = (IDENTITY || mul_routed_weight) ? 1 : top_k;
  const int nsb = K >> 8;
  const size_t row_bytes = static_cast<size_t>(nsb) * UB_Q4K_BYTES;
  const uint8_t* Be = Bq + static_cast<size_t>(e) * N * row_bytes;
  // weight rows feeding the two n8 tiles of this lane
  const int wr0 = n_warp + g;
  const int wr1 = ACT ? (D + n_warp + g) : (n_warp + 8 + g);
  const bool wv0 = wr0 < (ACT ? D : N), wv1 = ACT ? wv0 : (wr1 < N);
  const uint8_t* brow0 = Be + static_cast<size_t>(wv0 ? wr0 : 0) * row_bytes;
  const uint8_t* brow1 = Be + static_cast<size_t>(wv1 ? wr1 : 0) * row_bytes;

  for (int r0 = 0; r0 < block; r0 += 16 * kMT) {
    int sid_lo[kMT], sid_hi[kMT];
    const __nv_bfloat16* arow_lo[kMT];
    const __nv_bfloat16* arow_hi[kMT];
#pragma unroll
    for (int mt = 0; mt < kMT; mt++) {
      const int ra = r0 + 16 * mt + g, rb = ra + 8;
      int sa, sb;
      if (IDENTITY) {
        sa = (ra < block) ? blk * block + ra : -1;
        sb = (rb < block) ? blk * block + rb : -1;
      } else {
        sa = (ra < block) ? sids[ra] : -1;
        sb = (rb < block) ? sids[rb] : -1;
      }
      if (sa < 0 || sa >= topk_ids_size) sa = -1;
      if (sb < 0 || sb >= topk_ids_size) sb = -1;
      sid_lo[mt] = sa;
      sid_hi[mt] = sb;
      arow_lo[mt] = (sa >= 0) ? A + static_cast<size_t>(sa / topk_str) * K : nullptr;
      arow_hi[mt] = (sb >= 0) ? A + static_cast<size_t>(sb / topk_str) * K : nullptr;
    }
    float acc[kMT][2][4];
#pragma unroll
    for (int mt = 0; mt < kMT; mt++)
#pragma unroll
      for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[mt][nt][i] = 0.f;

    for (int sb = 0; sb < nsb; sb++) {
      const uint4 h0 = __ldg(reinterpret_cast<const uint4*>(brow0 + static_cast<size_t>(sb) * UB_Q4K_BYTES));
      const uint4 h1 = __ldg(reinterpret_cast<const uint4*>(brow1 + static_cast<size_t>(sb) * UB_Q4K_BYTES));
      const float d0 = half_bits_to_f32(h0.x), dm0 = half_bits_to_f32(h0.x >> 16);
      const float d1 = half_bits_to_f32(h1.x), dm1 = half_bits_to_f32(h1.x >> 16);
      uint32_t sc0[2], mn0[2], sc1[2], mn1[2];
      q4k_unpack_scales(h0.y, h0.z, h0.w, sc0[0], sc0[1], mn0[0], mn0[1]);
      q4k_unpack_scales(h1.y, h1.z, h1.w, sc1[0], sc1[1], mn1[0], mn1[1]);
#pragma unroll
      for (int G = 0; G < 4; G++) {
        const uint2 q0 = __ldg(reinterpret_cast<const uint2*>(brow0 + static_cast<size_t>(sb) * UB_Q4K_BYTES + 16 + G * 32 + 8 * t));
        const uint2 q1 = __ldg(reinterpret_cast<const uint2*>(brow1 + static_cast<size_t>(sb) * UB_Q4K_BYTES + 16 + G * 32 + 8 * t));
        const int sh = (G & 1) * 16;
        // sub-blocks 2G (low nibbles) and 2G+1 (high nibbles) of both weight rows
        const float dl0 = d0 * static_cast<float>((sc0[G >> 1] >> sh) & 0xFF), ml0 = dm0 * static_cast<float>((mn0[G >> 1] >> sh) & 0xFF);
        const float dh0 = d0 * static_cast<float>((sc0[G >> 1] >> (sh + 8)) & 0xFF), mh0 = dm0 * static_cast<float>((mn0[G >> 1] >> (sh + 8)) & 0xFF);
        const float dl1 = d1 * static_cast<float>((sc1[G >> 1] >> sh) & 0xFF), ml1 = dm1 * static_cast<float>((mn1[G >> 1] >> sh) & 0xFF);
        const float dh1 = d1 * static_cast<float>((sc1[G >> 1] >> (sh + 8)) & 0xFF), mh1 = dm1 * static_cast<float>((mn1[G >> 1] >> (sh + 8)) & 0xFF);
        // bfrag[tile][step][2]; steps: 0 = low of word x, 1 = low of word y, 2 = high of x, 3 = high of y
        uint32_t bf0[4][2], bf1[4][2];
        dequant4(q0.x & 0x0F0F0F0Fu, dl0, ml0, bf0[0][0], bf0[0][1]);
        dequant4(q0.y & 0x0F0F0F0Fu, dl0, ml0, bf0[1][0], bf0[1][1]);
        dequant4((q0.x >> 4) & 0x0F0F0F0Fu, dh0, mh0, bf0[2][0], bf0[2][1]);
        dequant4((q0.y >> 4) & 0x0F0F0F0Fu, dh0, mh0, bf0[3][0], bf0[3][1]);
        dequant4(q1.x & 0x0F0F0F0Fu, dl1, ml1, bf1[0][0], bf1[0][1]);
        dequant4(q1.y & 0x0F0F0F0Fu, dl1, ml1, bf1[1][0], bf1[1][1]);
        dequant4((q1.x >> 4) & 0x0F0F0F0Fu, dh1, mh1, bf1[2][0], bf1[2][1]);
        dequant4((q1.y >> 4) & 0x0F0F0F0Fu, dh1, mh1, bf1[3][0], bf1[3][1]);
        const int kg = sb * 256 + G * 64 + 8 * t;  // this lane's k for the low half; +32 for the high half
#pragma unroll
        for (int mt = 0; mt < kMT; mt++) {
          if (r0 + 16 * mt >= block) break;
          const uint4 z = make_uint4(0, 0, 0, 0);
          const uint4 al = arow_lo[mt] ? __ldg(reinterpret_cast<const uint4*>(arow_lo[mt] + kg)) : z;
          const uint4 ah = arow_hi[mt] ? __ldg(reinterpret_cast<const uint4*>(arow_hi[mt] + kg)) : z;
          const uint4 al2 = arow_lo[mt] ? __ldg(reinterpret_cast<const uint4*>(arow_lo[mt] + kg + 32)) : z;
          const uint4 ah2 = arow_hi[mt] ? __ldg(reinterpret_cast<const uint4*>(arow_hi[mt] + kg + 32)) : z;
          const uint32_t a0[4] = {al.x, ah.x, al.y, ah.y};
          const uint32_t a1[4] = {al.z, ah.z, al.w, ah.w};
          const uint32_t a2[4] = {al2.x, ah2.x, al2.y, ah2.y};
          const uint32_t a3[4] = {al2.z, ah2.z, al2.w, ah2.w};
          mma_bf16(acc[mt][0], a0, bf0[0][0], bf0[0][1]);
          mma_bf16(acc[mt][0], a1, bf0[1][0], bf0[1][1]);
          mma_bf16(acc[mt][0], a2, bf0[2][0], bf0[2][1]);
          mma_bf16(acc[mt][0], a3, bf0[3][0], bf0[3][1]);
          mma_bf16(acc[mt][1], a0, bf1[0][0], bf1[0][1]);
          mma_bf16(acc[mt][1], a1, bf1[1][0], bf1[1][1]);
          mma_bf16(acc[mt][1], a2, bf1[2][0], bf1[2][1]);
          mma_bf16(acc[mt][1], a3, bf1[3][0], bf1[3][1]);
        }
      }
    }

    // epilogue: lane holds rows (g, g+8) x columns (2t, 2t+1) of each n8 tile
#pragma unroll
    for (int mt = 0; mt < kMT; mt++) {
      if (r0 + 16 * mt >= block) break;
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int sid = half ? sid_hi[mt] : sid_lo[mt];
        if (sid < 0) continue;
        const float w = mul_routed_weight ? topk_w[sid] : 1.f;
        if (ACT) {
          // tile 0 = gate columns, tile 1 = the matching up columns
          const int n = n_warp + 2 * t;
          float o[2];
#pragma unroll
          for (int i = 0; i < 2; i++) {
            const float gte = __bfloat162float(__float2bfloat16_rn(acc[mt][0][2 * half + i] * w));
            const float up = __bfloat162float(__float2bfloat16_rn(acc[mt][1][2 * half + i] * w));
            o[i] = __fmul_rn(__fdiv_rn(gte, 1.f + expf(-gte)), up);
          }
          __nv_bfloat16* dst = C + static_cast<size_t>(sid) * D + n;
          if (n + 1 < D && ((reinterpret_cast<uintptr_t>(dst) & 3) == 0)) {
            *reinterpret_cast<uint32_t*>(dst) = pack_bf16(o[0], o[1]);
          } else {
            if (n < D) dst[0] = __float2bfloat16_rn(o[0]);
            if (n + 1 < D) dst[1] = __float2bfloat16_rn(o[1]);
          }
        } else {
#pragma unroll
          for (int nt = 0; nt < 2; nt++) {
            const int n = n_warp + 8 * nt + 2 * t;
            const float v0 = acc[mt][nt][2 * half] * w, v1 = acc[mt][nt][2 * half + 1] * w;
            __nv_bfloat16* dst = C + static_cast<size_t>(sid) * D + n;
            if (n + 1 < D && ((reinterpret_cast<uintptr_t>(dst) & 3) == 0)) {
              *reinterpret_cast<uint32_t*>(dst) = pack_bf16(v0, v1);
            } else {
              if (n < D) dst[0] = __float2bfloat16_rn(v0);
              if (n + 1 < D) dst[1] = __float2bfloat16_rn(v1);
            }
          }
        }
      }
    }
  }
}

__global__ void bf16_to_f32_kernel(float* __restrict__ out, const __nv_bfloat16* __restrict__ in, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __bfloat162float(in[i]);
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

namespace ub {

int moe_align(int32_t* sorted_ids, int32_t* experts_ids, int32_t* num_post_pad, const int32_t* topk_ids,
              const int32_t* real_token_num, const int32_t* expert_map, int E, int block, int T, int k, cudaStream_t s);
int topk_softmax_bf16_impl(const void* in, void* out_w, int* out_idx, int T, int E, int k, int norm, cudaStream_t s);

// Plain y[M,N] = x[M,K] . dequant(Wq)^T through the grouped kernel (bf16 in, bf16 out).
int q4k_gemm_mma(void* y, const void* x, const void* wq, int M, int N, int K, cudaStream_t s) {
  const int block = 64;
  dim3 grid((M + block - 1) / block, (N + 63) / 64);
  q4k_grouped_mma_kernel<true, false><<<grid, 128, 0, s>>>(
      static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(x), static_cast<const uint8_t*>(wq), nullptr,
      nullptr, nullptr, nullptr, K, N, 1, M, 1, block, 0, ub::device_error_word());
  return ub::check_launch();
}

}  // namespace ub

namespace ub {
bool q4k_moe_tc_supported(int positions, int K, int N, int block);
int moe_gather_rows(void* xg, const void* hidden, const int32_t* sorted_ids, const int32_t* num_post_pad, int positions,
                    int num_valid, int top_k, int H, cudaStream_t s);
int q4k_moe_gemm_tc(void* C, const void* A, const void* Bq, const float* topk_w, const int32_t* sorted_ids,
                    const int32_t* experts_ids, const int32_t* num_post_pad, int positions, int K, int N, int E,
                    int num_valid, int block, int act_silu_mul, cudaStream_t s);
}  // namespace ub

extern "C" {

int ub_fused_moe_q4k_gemm(void* C, const void* A, const void* Bq, const float* topk_weights, const int32_t* sorted_ids,
                          const int32_t* experts_ids, const int32_t* num_tokens_post_pad, int M, int K, int N, int E,
                          int topk_ids_size, int top_k, int block_size, int mul_routed_weight, int act_silu_mul,
                          void* workspace, size_t ws_bytes, void* stream) {
  (void)M;
  (void)workspace;
  (void)ws_bytes;
  if (!C || !A || !Bq || !sorted_ids || !experts_ids || !num_tokens_post_pad || K <= 0 || N <= 0 || E <= 0 ||
      block_size <= 0 || top_k <= 0 || topk_ids_size < 0 || (mul_routed_weight && !topk_weights))
    return ub::fail(UB_ERR_INVALID_ARG);
  if (K % UB_QK_K != 0 || (act_silu_mul && (N % 2)) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(Bq) & 15))
    return ub::fail(UB_ERR_INVALID_ARG);
  if (topk_ids_size == 0) return ub::fail(UB_OK);
  const int max_blocks = (topk_ids_size + E * (block_size - 1)) / block_size;
  if (max_blocks == 0) return ub::fail(UB_OK);
  cudaStream_t s = ub::as_stream(stream);
  __nv_bfloat16* c = static_cast<__nv_bfloat16*>(C);
  const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(A);
  const uint8_t* b = static_cast<const uint8_t*>(Bq);
  if (act_silu_mul) {
    dim3 grid(max_blocks, (N / 2 + 31) / 32);
    q4k_grouped_mma_kernel<false, true><<<grid, 128, 0, s>>>(c, a, b, topk_weights, sorted_ids, experts_ids,
                                                             num_tokens_post_pad, K, N, E, topk_ids_size, top_k,
                                                             block_size, mul_routed_weight, ub::device_error_word());
  } else {
    dim3 grid(max_blocks, (N + 63) / 64);
    q4k_grouped_mma_kernel<false, false><<<grid, 128, 0, s>>>(c, a, b, topk_weights, sorted_ids, experts_ids,
                                                              num_tokens_post_pad, K, N, E, topk_ids_size, top_k,
                                                              block_size, mul_routed_weight, ub::device_error_word());
  }
  return ub::check_launch();
}

// Workspace layout of ub_moe_layer_q4k (each region 256-byte aligned):
//   w_t [T*k] bf16 | w_f32 [T*k] f32 | idx [T*k] i32 | sorted_ids [T*k + E*(block-1)] i32 |
//   experts_ids [max_blocks] i32 | num_post_pad [1] i32 | act [max_padded, I] bf16 | c2 [T*k, H] bf16 |
//   xg [max_padded, H] bf16
// (act holds slot-indexed rows on the mma.sync path and aligned-order rows on the tcgen05 path; xg is the
// hidden states gathered into aligned order for the tcgen05 path.)
size_t ub_moe_layer_q4k_workspace_bytes(int T, int H, int I, int E, int top_k, int block_size) {
  if (T <= 0 || H <= 0 || I <= 0 || E <= 0 || top_k <= 0 || block_size <= 0) return 0;
  const size_t slots = static_cast<size_t>(T) * top_k;
  const size_t max_padded = slots + static_cast<size_t>(E) * (block_size - 1);
  size_t b = 0;
  b += align_up(slots * 2, 256);
  b += align_up(slots * 4, 256);
  b += align_up(slots * 4, 256);
  b += align_up(max_padded * 4, 256);
  b += align_up((max_padded / block_size + 1) * 4, 256);
  b += 256;
  b += align_up(max_padded * I * 2, 256);
  b += align_up(slots * H * 2, 256);
  b += align_up(max_padded * H * 2, 256);
  return b;
}

int ub_moe_layer_q4k(void* out, const void* hidden, const void* router_logits, const void* w13q, const void* w2q,
                     const int32_t* expert_map, int T, int H, int I, int E, int top_k, int block_size,
                     int norm_topk_prob, void* workspace, size_t ws_bytes, void* stream) {
  if (T == 0) return ub::fail(UB_OK);
  if (!out || !hidden || !router_logits || !w13q || !w2q || T < 0 || H <= 0 || I <= 0 || E <= 0 || top_k <= 0 ||
      block_size <= 0)
    return ub::fail(UB_ERR_INVALID_ARG);
  if (H % UB_QK_K || I % UB_QK_K) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t need = ub_moe_layer_q4k_workspace_bytes(T, H, I, E, top_k, block_size);
  if (!workspace || ws_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return ub::fail(UB_ERR_WORKSPACE);
  cudaStream_t s = ub::as_stream(stream);
  const size_t slots = static_cast<size_t>(T) * top_k;
  const size_t max_padded = slots + static_cast<size_t>(E) * (block_size - 1);
  char* p = static_cast<char*>(workspace);
  __nv_bfloat16* w_t = reinterpret_cast<__nv_bfloat16*>(p); p += align_up(slots * 2, 256);
  float* w_f32 = reinterpret_cast<float*>(p); p += align_up(slots * 4, 256);
  int32_t* idx = reinterpret_cast<int32_t*>(p); p += align_up(slots * 4, 256);
  int32_t* sorted_ids = reinterpret_cast<int32_t*>(p); p += align_up(max_padded * 4, 256);
  int32_t* experts_ids = reinterpret_cast<int32_t*>(p); p += align_up((max_padded / block_size + 1) * 4, 256);
  int32_t* npp = reinterpret_cast<int32_t*>(p); p += 256;
  __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(p); p += align_up(max_padded * I * 2, 256);
  __nv_bfloat16* c2 = reinterpret_cast<__nv_bfloat16*>(p); p += align_up(slots * H * 2, 256);
  __nv_bfloat16* xg = reinterpret_cast<__nv_bfloat16*>(p);

  int st = ub::topk_softmax_bf16_impl(router_logits, w_t, idx, T, E, top_k, norm_topk_prob != 0, s);
  if (st != UB_OK) return st;
  bf16_to_f32_kernel<<<static_cast<int>((slots + 255) / 256), 256, 0, s>>>(w_f32, w_t, static_cast<int>(slots));
  st = ub::moe_align(sorted_ids, experts_ids, npp, idx, nullptr, expert_map, E, block_size, T, top_k, s);
  if (st != UB_OK) return st;
  const int positions = static_cast<int>(max_padded);
  if (ub::q4k_moe_tc_supported(positions, H, I, block_size) && ub::q4k_moe_tc_supported(positions, I, H, block_size) &&
      (reinterpret_cast<uintptr_t>(w13q) & 15) == 0 && (reinterpret_cast<uintptr_t>(w2q) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(hidden) & 15) == 0) {
    // tcgen05 path: gather the tokens into aligned order once, keep the SiLU.up activations in that order
    st = ub::moe_gather_rows(xg, hidden, sorted_ids, npp, positions, static_cast<int>(slots), top_k, H, s);
    if (st != UB_OK) return st;
    st = ub::q4k_moe_gemm_tc(act, xg, w13q, nullptr, sorted_ids, experts_ids, npp, positions, H, I, E,
                             static_cast<int>(slots), block_size, 1, s);
    if (st != UB_OK) return ub::fail(st);
    if (expert_map) {  // slots of experts held elsewhere contribute zeros
      cudaError_t ce = cudaMemsetAsync(c2, 0, slots * H * 2, s);
      if (ce != cudaSuccess) {
        ub::set_cuda_error(ce);
        return ub::fail(UB_ERR_CUDA);
      }
    }
    st = ub::q4k_moe_gemm_tc(c2, act, w2q, w_f32, sorted_ids, experts_ids, npp, positions, I, H, E,
                             static_cast<int>(slots), block_size, 0, s);
    if (st != UB_OK) return ub::fail(st);
    return ub_topk_sum(out, c2, T, top_k, H, UB_DTYPE_BF16, stream);
  }
  st = ub_fused_moe_q4k_gemm(act, hidden, w13q, nullptr, sorted_ids, experts_ids, npp, T, H, 2 * I, E,
                             static_cast<int>(slots), top_k, block_size, 0, 1, nullptr, 0, stream);
  if (st != UB_OK) return st;
  st = ub_fused_moe_q4k_gemm(c2, act, w2q, w_f32, sorted_ids, experts_ids, npp, static_cast<int>(slots), I, H, E,
                             static_cast<int>(slots), top_k, block_size, 1, 0, nullptr, 0, stream);
  if (st != UB_OK) return st;
  return ub_topk_sum(out, c2, T, top_k, H, UB_DTYPE_BF16, stream);
}

}  // extern "C"
