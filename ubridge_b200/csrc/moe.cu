// MoE routing and dense expert kernels behind the reference's host-launcher names.
//
//   topk_softmax_{f32,f16,bf16}   replaces kernels/topk_softmax_host.cpp:103-208
//   moe_align_block_size          replaces kernels/moe_align_host.cpp:51-99,318-935
//   invoke_fused_moe_{f16,bf16}   replaces kernels/fused_moe_host.cpp:43-536 (dense expert weights)
//   moe_{f16,bf16}                replaces kernels/moe_host.cpp:26-94   (weighted combine)
//   indexed_moe_{f16,bf16}        replaces kernels/moe_host.cpp:117-293 (per-slot expert GEMV)
//   ub_silu_and_mul, ub_topk_sum  the two elementwise steps the reference's caller runs around the
//                                 grouped GEMMs (kernels/topsaten_ops_wrapper.cpp:375-391; src/ffi.rs:841-849)
//
// Where the reference traps the device on a bad expert id (kernels/utils/moe_kernel_compat.h:21-28)
// these kernels record UB_ERR_BAD_INDEX in the device error word, skip the access and carry on.
#include "common.cuh"

namespace {

using namespace ub;

// ------------------------------------------------------------------ topk_softmax
// One warp per token.  Softmax in f32; the denominator is summed left to right (the scalar
// reference's order) when E <= 64, lane-partial + shuffle tree above that.  k rounds of arg-max
// with strict '>' inside a lane (ascending e) and (value, lower index) across lanes, so ties go
// to the lowest expert index exactly as the scalar scan does.
template <typename T>
__global__ void __launch_bounds__(128) topk_softmax_kernel(const T* __restrict__ in, T* __restrict__ out_w,
                                                            int* __restrict__ out_idx, int* __restrict__ out_src,
                                                            int T_tokens, int E, int k, int norm) {
  extern __shared__ float smem_prob[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* prob = smem_prob + static_cast<size_t>(warp) * E;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + warp; t < T_tokens; t += gridDim.x * wpb) {
    const T* row = in + static_cast<size_t>(t) * E;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, to_f32(row[e]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    float part = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float ex = expf(to_f32(row[e]) - mx);
      prob[e] = ex;
      part += ex;
    }
    __syncwarp();
    float sum;
    if (E <= 64) {
      sum = 0.f;
      for (int e = 0; e < E; e++) sum += prob[e];
    } else {
      sum = warp_sum(part);
    }
    const float inv_sum = sum > 0.f ? __fdiv_rn(1.f, sum) : 1.f;
    for (int e = lane; e < E; e += 32) prob[e] = __fmul_rn(prob[e], inv_sum);
    __syncwarp();

    float wsum = 0.f;
    int got = 0;
    for (int j = 0; j < k; j++) {
      float best = -INFINITY;
      int bi = -1;
      for (int e = lane; e < E; e += 32) {
        const float v = prob[e];
        if (v > best) {
          best = v;
          bi = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi < bi))) {
          best = ov;
          bi = oi;
        }
      }
      if (bi < 0) break;
      if (lane == 0) {
        out_w[static_cast<size_t>(t) * k + j] = from_f32<T>(best);
        out_idx[static_cast<size_t>(t) * k + j] = bi;
        // source-row id of slot (t, j) in the expanded [k, T] layout, as vLLM's router kernel numbers them
        if (out_src) out_src[static_cast<size_t>(t) * k + j] = j * T_tokens + t;
        prob[bi] = -INFINITY;
      }
      wsum += best;
      got++;
      __syncwarp();
    }
    if (norm && wsum > 0.f) {
      const float inv = __fdiv_rn(1.f, wsum);
      for (int j = lane; j < got; j += 32) {
        T* p = out_w + static_cast<size_t>(t) * k + j;
        *p = from_f32<T>(__fmul_rn(to_f32(*p), inv));
      }
    }
    __syncwarp();
  }
}

template <typename T>
int topk_softmax_launch(const void* in, void* out_w, int* out_idx, int T_tokens, int E, int k, int norm,
                        cudaStream_t s, int* out_src = nullptr) {
  if (T_tokens == 0) return ub::fail(UB_OK);
  // same limits as the reference (kernels/topk_softmax_host.cpp:108-110): silently do nothing beyond them
  if (E > 4096 || k > 4096) return ub::fail(UB_ERR_INVALID_ARG);
  if (!in || !out_w || !out_idx || T_tokens < 0 || E <= 0 || k <= 0) return ub::fail(UB_ERR_INVALID_ARG);
  const int threads = 128;
  const size_t smem = static_cast<size_t>(threads / 32) * E * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(topk_softmax_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) {
      ub::set_cuda_error(e);
      return ub::fail(UB_ERR_CUDA);
    }
  }
  int blocks = (T_tokens + 3) / 4;
  const int cap = ub::num_sms() * 8;
  if (blocks > cap) blocks = cap;
  topk_softmax_kernel<T><<<blocks, threads, smem, s>>>(static_cast<const T*>(in), static_cast<T*>(out_w), out_idx,
                                                       out_src, T_tokens, E, k, norm);
  return ub::check_launch();
}

// ------------------------------------------------------------------ moe_align_block_size
// Every CTA rebuilds the per-expert histogram and its padded prefix sum in shared memory (the
// slot list is a few KB), then owns experts blockIdx.x, blockIdx.x + gridDim.x, ...: it writes
// those experts' entries of experts_ids, scatters their slots in ascending slot order (ballot +
// prefix inside a warp, a 32-entry scan across warps) and pads their tails.  CTA 0 also fills
// everything beyond num_tokens_post_pad.  CTAs never write the same word, so no grid sync is needed.
constexpr int kAlignThreads = 256;

__global__ void __launch_bounds__(kAlignThreads) moe_align_kernel(
    int32_t* __restrict__ sorted_ids, int32_t* __restrict__ experts_ids, int32_t* __restrict__ num_post_pad,
    const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ real_token_num,
    const int32_t* __restrict__ expert_map, int E, int block, int T, int k, int* err_word) {
  extern __shared__ int32_t sm[];
  int32_t* cnt = sm;            // [E]
  int32_t* off = sm + E;        // [E+1] padded prefix (in slots)
  __shared__ int32_t warp_tot[kAlignThreads / 32];
  __shared__ int32_t chunk_base;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pad_value = T * k;
  const int max_padded = T * k + E * (block - 1);
  const int max_blocks = max_padded / block;
  int tn = T;
  if (real_token_num) {
    tn = *real_token_num;
    if (tn < 0 || tn > T) {
      if (tid == 0 && blockIdx.x == 0) report_device_error(err_word, UB_ERR_BAD_INDEX);
      tn = tn < 0 ? 0 : T;
    }
  }
  const int slots = tn * k;

  for (int e = tid; e < E; e += kAlignThreads) cnt[e] = 0;
  __syncthreads();
  for (int i = tid; i < slots; i += kAlignThreads) {
    const int e = topk_ids[i];
    if (e < 0 || e >= E) {
      if (blockIdx.x == 0) report_device_error(err_word, UB_ERR_BAD_INDEX);
    } else {
      atomicAdd(&cnt[e], 1);
    }
  }
  if (expert_map && blockIdx.x == 0)
    for (int e = tid; e < E; e += kAlignThreads)
      if (expert_map[e] < -1 || expert_map[e] >= E) report_device_error(err_word, UB_ERR_BAD_INDEX);
  __syncthreads();

  // padded exclusive prefix over experts, warp 0, 32 experts per step
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + lane;
      const int padded = (e < E) ? ((cnt[e] + block - 1) / block) * block : 0;
      int incl = padded;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (lane >= o) incl += v;
      }
      if (e < E) off[e] = carry + incl - padded;
      carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
    }
    if (lane == 0) off[E] = carry;
  }
  __syncthreads();
  const int total_padded = off[E];

  if (blockIdx.x == 0) {
    if (tid == 0) *num_post_pad = total_padded;
    for (int i = total_padded + tid; i < max_padded; i += kAlignThreads) sorted_ids[i] = pad_value;
    for (int i = total_padded / block + tid; i < max_blocks; i += kAlignThreads) experts_ids[i] = 0;
  }

  for (int e = blockIdx.x; e < E; e += gridDim.x) {
    const int c = cnt[e];
    if (c == 0) continue;  // uniform across the CTA
    const int begin = off[e], end = off[e + 1];
    const int id_out = expert_map ? expert_map[e] : e;
    for (int b = begin / block + tid; b < end / block; b += kAlignThreads) experts_ids[b] = id_out;
    for (int i = begin + c + tid; i < end; i += kAlignThreads) sorted_ids[i] = pad_value;
    if (tid == 0) chunk_base = begin;
    __syncthreads();
    for (int base = 0; base < slots; base += kAlignThreads) {
      const int i = base + tid;
      const bool hit = (i < slots) && (topk_ids[i] == e);
      const unsigned mask = __ballot_sync(0xFFFFFFFFu, hit);
      if (lane == 0) warp_tot[warp] = __popc(mask);
      __syncthreads();
      int before = 0;
#pragma unroll
      for (int w = 0; w < kAlignThreads / 32; w++) before += (w < warp) ? warp_tot[w] : 0;
      const int cb = chunk_base;
      if (hit) sorted_ids[cb + before + __popc(mask & ((1u << lane) - 1u))] = i;
      __syncthreads();
      if (tid == 0) {
        int tot = 0;
#pragma unroll
        for (int w = 0; w < kAlignThreads / 32; w++) tot += warp_tot[w];
        chunk_base = cb + tot;
      }
      __syncthreads();
    }
  }
}

int moe_align_launch(int32_t* sorted_ids, int32_t* experts_ids, int32_t* num_post_pad, const int32_t* topk_ids,
                     const int32_t* real_token_num, const int32_t* expert_map, int E, int block, int T, int k,
                     cudaStream_t s) {
  if (!sorted_ids || !experts_ids || !num_post_pad || E <= 0 || block <= 0 || T < 0 || k <= 0 ||
      (T > 0 && !topk_ids))
    return ub::fail(UB_ERR_INVALID_ARG);
  const size_t smem = static_cast<size_t>(2 * E + 1) * sizeof(int32_t);
  if (smem > 200 * 1024) return ub::fail(UB_ERR_TOO_LARGE);
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(moe_align_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) {
      ub::set_cuda_error(e);
      return ub::fail(UB_ERR_CUDA);
    }
  }
  const int blocks = E < 64 ? E : 64;
  moe_align_kernel<<<blocks, kAlignThreads, smem, s>>>(sorted_ids, experts_ids, num_post_pad, topk_ids,
                                                       real_token_num, expert_map, E, block, T, k,
                                                       ub::device_error_word());
  return ub::check_launch();
}

// ------------------------------------------------------------------ dense grouped GEMM (reference signature)
// Tensor-core path with warp-level mma (m16n8k16, f32 accumulate).  One CTA = one aligned block of
// slots x 64 output columns; each of its 4 warps owns 16 columns and walks the block's rows in
// 16-row tiles.  Operands are read straight from global memory with 16-byte loads: lane (g,t)
// takes k = 8t..8t+7 of a 32-wide k chunk for its row, which feeds two mma steps; A and B use the
// same k assignment, so the reduction order inside a chunk is permuted but complete.
template <typename T> struct MmaType;
template <> struct MmaType<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct MmaType<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int kMoeTileN = 64;   // output columns per CTA
constexpr int kMoeMaxMT = 4;    // 16-row tiles per pass (64 rows)

template <typename T>
__global__ void __launch_bounds__(128) fused_moe_dense_kernel(
    T* __restrict__ C, const T* __restrict__ A, const T* __restrict__ B, const T* __restrict__ bias,
    const float* __restrict__ topk_w, const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ experts_ids,
    const int32_t* __restrict__ num_post_pad, int K, int N, int E, int topk_ids_size, int top_k, int block,
    int mul_routed_weight, int bias_flag, int* err_word) {
  const int padded = *num_post_pad;
  const int blk = blockIdx.x;
  if (padded <= 0 || blk * block >= padded) return;
  const int e = experts_ids[blk];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n_cta = blockIdx.y * kMoeTileN;
  const int32_t* sids = sorted_ids + static_cast<size_t>(blk) * block;

  if (e < 0 || e >= E) {
    if (e != -1 && threadIdx.x == 0) report_device_error(err_word, UB_ERR_BAD_INDEX);
    // expert not on this rank: zero-fill the rows this block names (kernels/fused_moe_host.cpp:161-176)
    for (int r = warp; r < block; r += 4) {
      const int sid = sids[r];
      if (sid < 0 || sid >= topk_ids_size) continue;
      for (int n = n_cta + lane; n < n_cta + kMoeTileN && n < N; n += 32)
        C[static_cast<size_t>(sid) * N + n] = from_f32<T>(0.f);
    }
    return;
  }

  const int topk_str = mul_routed_weight ? 1 : top_k;
  const int n_warp = n_cta + warp * 16;
  const T* Be = B + static_cast<size_t>(e) * N * K;

  for (int r0 = 0; r0 < block; r0 += 16 * kMoeMaxMT) {
    // rows this lane touches: r0 + 16*mt + g and + 8
    int sid_lo[kMoeMaxMT], sid_hi[kMoeMaxMT];
    const T* arow_lo[kMoeMaxMT];
    const T* arow_hi[kMoeMaxMT];
#pragma unroll
    for (int mt = 0; mt < kMoeMaxMT; mt++) {
      const int ra = r0 + 16 * mt + g, rb = ra + 8;
      int sa = (ra < block) ? sids[ra] : -1, sb = (rb < block) ? sids[rb] : -1;
      if (sa < 0 || sa >= topk_ids_size) sa = -1;
      if (sb < 0 || sb >= topk_ids_size) sb = -1;
      sid_lo[mt] = sa;
      sid_hi[mt] = sb;
      arow_lo[mt] = (sa >= 0) ? A + static_cast<size_t>(sa / topk_str) * K : nullptr;
      arow_hi[mt] = (sb >= 0) ? A + static_cast<size_t>(sb / topk_str) * K : nullptr;
    }
    float acc[kMoeMaxMT][2][4];
#pragma unroll
    for (int mt = 0; mt < kMoeMaxMT; mt++)
#pragma unroll
      for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[mt][nt][i] = 0.f;

    const int nb0 = n_warp + g, nb1 = n_warp + 8 + g;
    const T* brow0 = (nb0 < N) ? Be + static_cast<size_t>(nb0) * K : nullptr;
    const T* brow1 = (nb1 < N) ? Be + static_cast<size_t>(nb1) * K : nullptr;

    for (int k0 = 0; k0 < K; k0 += 32) {
      const int kk = k0 + 8 * t;
      const bool kin = kk < K;  // K is a multiple of 8
      const uint4 z = make_uint4(0, 0, 0, 0);
      const uint4 b0 = (brow0 && kin) ? __ldg(reinterpret_cast<const uint4*>(brow0 + kk)) : z;
      const uint4 b1 = (brow1 && kin) ? __ldg(reinterpret_cast<const uint4*>(brow1 + kk)) : z;
#pragma unroll
      for (int mt = 0; mt < kMoeMaxMT; mt++) {
        if (r0 + 16 * mt >= block) break;
        const uint4 al = (arow_lo[mt] && kin) ? __ldg(reinterpret_cast<const uint4*>(arow_lo[mt] + kk)) : z;
        const uint4 ah = (arow_hi[mt] && kin) ? __ldg(reinterpret_cast<const uint4*>(arow_hi[mt] + kk)) : z;
        const uint32_t a_s0[4] = {al.x, ah.x, al.y, ah.y};
        const uint32_t a_s1[4] = {al.z, ah.z, al.w, ah.w};
        MmaType<T>::mma(acc[mt][0], a_s0, b0.x, b0.y);
        MmaType<T>::mma(acc[mt][0], a_s1, b0.z, b0.w);
        MmaType<T>::mma(acc[mt][1], a_s0, b1.x, b1.y);
        MmaType<T>::mma(acc[mt][1], a_s1, b1.z, b1.w);
      }
    }

#pragma unroll
    for (int mt = 0; mt < kMoeMaxMT; mt++) {
      if (r0 + 16 * mt >= block) break;
#pragma unroll
      for (int nt = 0; nt < 2; nt++) {
        const int n = n_warp + 8 * nt + 2 * t;
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const int sid = half ? sid_hi[mt] : sid_lo[mt];
          if (sid < 0) continue;
          float v0 = acc[mt][nt][2 * half], v1 = acc[mt][nt][2 * half + 1];
          if (bias_flag) {
            if (n < N) v0 += to_f32(bias[static_cast<size_t>(e) * N + n]);
            if (n + 1 < N) v1 += to_f32(bias[static_cast<size_t>(e) * N + n + 1]);
          }
          if (mul_routed_weight) {
            const float w = topk_w[sid];
            v0 *= w;
            v1 *= w;
          }
          T* dst = C + static_cast<size_t>(sid) * N + n;
          if (n + 1 < N && ((reinterpret_cast<uintptr_t>(dst) & 3) == 0)) {
            *reinterpret_cast<uint32_t*>(dst) = pack2<T>(v0, v1);
          } else {
            if (n < N) dst[0] = from_f32<T>(v0);
            if (n + 1 < N) dst[1] = from_f32<T>(v1);
          }
        }
      }
    }
  }
}

template <typename T>
int fused_moe_dense_launch(void* C, const void* A, const void* B, const void* bias, const float* topk_w,
                           const int32_t* sorted_ids, const int32_t* experts_ids, const int32_t* num_post_pad, int M,
                           int K, int N, int E, int topk_ids_size, int top_k, int block, int mul_routed_weight,
                           int bias_flag, cudaStream_t s) {
  (void)M;
  if (!C || !A || !B || !sorted_ids || !experts_ids || !num_post_pad || K <= 0 || N <= 0 || E <= 0 || block <= 0 ||
      top_k <= 0 || topk_ids_size < 0 || (mul_routed_weight && !topk_w) || (bias_flag && !bias))
    return ub::fail(UB_ERR_INVALID_ARG);
  if (K % 8 != 0 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return ub::fail(UB_ERR_INVALID_ARG);  // 16-byte operand loads
  if (topk_ids_size == 0) return ub::fail(UB_OK);
  const int max_blocks = (topk_ids_size + E * (block - 1)) / block;
  if (max_blocks == 0) return ub::fail(UB_OK);
  dim3 grid(max_blocks, (N + kMoeTileN - 1) / kMoeTileN);
  fused_moe_dense_kernel<T><<<grid, 128, 0, s>>>(static_cast<T*>(C), static_cast<const T*>(A),
                                                 static_cast<const T*>(B), static_cast<const T*>(bias), topk_w,
                                                 sorted_ids, experts_ids, num_post_pad, K, N, E, topk_ids_size, top_k,
                                                 block, mul_routed_weight, bias_flag, ub::device_error_word());
  return ub::check_launch();
}

// ------------------------------------------------------------------ weighted combine (moe_*)
// y[idx[k],:] = T( y[idx[k],:] + T(e_out[k,:] * w[idx[k]*topk + top[k]]) ), applied in ascending k.
// One CTA per output row: warp 0 compacts the matching k in order, then all threads walk columns.
constexpr int kCombineMaxList = 1024;

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(T* __restrict__ y, const T* __restrict__ e_out,
                                                           const float* __restrict__ w,
                                                           const uint32_t* __restrict__ idx,
                                                           const uint32_t* __restrict__ top, int N, int K, int M,
                                                           int topk) {
  __shared__ int list[kCombineMaxList];
  __shared__ int list_n;
  const int r = blockIdx.x;
  const int lane = threadIdx.x & 31;
  for (int kbase = 0; kbase < K; kbase += kCombineMaxList) {
    const int kend = min(K, kbase + kCombineMaxList);
    if (threadIdx.x < 32) {
      int n = 0;
      for (int k0 = kbase; k0 < kend; k0 += 32) {
        const int kk = k0 + lane;
        const bool hit = kk < kend && idx[kk] == static_cast<uint32_t>(r) && top[kk] < static_cast<uint32_t>(topk);
        const unsigned mask = __ballot_sync(0xFFFFFFFFu, hit);
        if (hit) list[n + __popc(mask & ((1u << lane) - 1u))] = kk;
        n += __popc(mask);
      }
      if (lane == 0) list_n = n;
    }
    __syncthreads();
    const int n = list_n;
    if (n > 0) {
      for (int j = threadIdx.x; j < M; j += blockDim.x) {
        float cur = to_f32(y[static_cast<size_t>(r) * M + j]);
        for (int i = 0; i < n; i++) {
          const int kk = list[i];
          const float wv = w[static_cast<size_t>(r) * topk + top[kk]];
          const float prod = to_f32(from_f32<T>(__fmul_rn(to_f32(e_out[static_cast<size_t>(kk) * M + j]), wv)));
          cur = to_f32(from_f32<T>(__fadd_rn(cur, prod)));
        }
        y[static_cast<size_t>(r) * M + j] = from_f32<T>(cur);
      }
    }
    __syncthreads();
  }
}

template <typename T>
int moe_combine_launch(void* y, const void* e_out, const float* w, const uint32_t* idx, const uint32_t* top, int N,
                       int K, int M, int topk, cudaStream_t s) {
  if (N == 0 || K == 0 || M == 0) return ub::fail(UB_OK);
  if (!y || !e_out || !w || !idx || !top || N < 0 || K < 0 || M < 0 || topk <= 0) return ub::fail(UB_ERR_INVALID_ARG);
  moe_combine_kernel<T><<<N, 256, 0, s>>>(static_cast<T*>(y), static_cast<const T*>(e_out), w, idx, top, N, K, M,
                                          topk);
  return ub::check_launch();
}

// ------------------------------------------------------------------ indexed_moe (dense per-slot GEMV)
// out[b,t,n] = sum_k in[b,(M==1?0:t),k] * w[indices[b,t],n,k]; one warp per output element.
template <typename T>
__global__ void __launch_bounds__(256) indexed_moe_kernel(const T* __restrict__ in, const T* __restrict__ w,
                                                           T* __restrict__ out, const uint32_t* __restrict__ indices,
                                                           int N, int K, int M, int batch, int topk, int num_experts,
                                                           int* err_word) {
  const int lane = threadIdx.x & 31;
  const size_t warp = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
  const size_t total = static_cast<size_t>(batch) * topk * N;
  for (size_t o = warp; o < total; o += nwarps) {
    const int n = static_cast<int>(o % N);
    const size_t bt = o / N;
    const int tt = static_cast<int>(bt % topk);
    const size_t b = bt / topk;
    const uint32_t e = indices[bt];
    if (e >= static_cast<uint32_t>(num_experts)) {
      if (lane == 0) {
        report_device_error(err_word, UB_ERR_BAD_INDEX);
        out[o] = from_f32<T>(0.f);
      }
      continue;
    }
    const T* xr = in + (b * M + (M == 1 ? 0 : tt)) * static_cast<size_t>(K);
    const T* wr = w + (static_cast<size_t>(e) * N + n) * static_cast<size_t>(K);
    float acc = 0.f;
    for (int kk = lane * 8; kk < K; kk += 256) {
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(xr + kk));
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wr + kk));
      const T* xs = reinterpret_cast<const T*>(&xv);
      const T* ws = reinterpret_cast<const T*>(&wv);
#pragma unroll
      for (int i = 0; i < 8; i++) acc = fmaf(to_f32(xs[i]), to_f32(ws[i]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[o] = from_f32<T>(acc);
  }
}

template <typename T>
int indexed_moe_launch(const void* in, const void* w, void* out, const uint32_t* indices, int N, int K, int M,
                       int batch, int topk, int num_experts, cudaStream_t s) {
  if (batch == 0 || topk == 0 || N == 0) return ub::fail(UB_OK);
  if (!in || !w || !out || !indices || N < 0 || K <= 0 || M <= 0 || batch < 0 || topk < 0 || num_experts <= 0)
    return ub::fail(UB_ERR_INVALID_ARG);
  if (K % 8 != 0 || (reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return ub::fail(UB_ERR_INVALID_ARG);
  if (M != 1 && M != topk) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t total = static_cast<size_t>(batch) * topk * N;
  size_t blocks = (total + 7) / 8;
  const size_t cap = static_cast<size_t>(ub::num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  indexed_moe_kernel<T><<<static_cast<int>(blocks), 256, 0, s>>>(static_cast<const T*>(in), static_cast<const T*>(w),
                                                                 static_cast<T*>(out), indices, N, K, M, batch, topk,
                                                                 num_experts, ub::device_error_word());
  return ub::check_launch();
}

// ------------------------------------------------------------------ elementwise helpers
template <typename T>
__global__ void __launch_bounds__(256) silu_and_mul_kernel(T* __restrict__ out, const T* __restrict__ in, size_t rows,
                                                            int D) {
  const size_t total = rows * D;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = i / D;
    const int j = static_cast<int>(i - r * D);
    const float gte = to_f32(in[r * 2 * D + j]), up = to_f32(in[r * 2 * D + D + j]);
    const float sg = __fdiv_rn(gte, 1.f + expf(-gte));
    out[i] = from_f32<T>(__fmul_rn(sg, up));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) topk_sum_kernel(T* __restrict__ out, const T* __restrict__ in, size_t T_tokens,
                                                        int topk, int H) {
  const size_t total = T_tokens * H;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t tk = i / H;
    const int h = static_cast<int>(i - tk * H);
    float sacc = 0.f;
    for (int j = 0; j < topk; j++) sacc = __fadd_rn(sacc, to_f32(in[(tk * topk + j) * H + h]));
    out[i] = from_f32<T>(sacc);
  }
}

inline int ew_grid(size_t total) {
  size_t blocks = (total + 255) / 256;
  const size_t cap = static_cast<size_t>(ub::num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  return static_cast<int>(blocks ? blocks : 1);
}

}  // namespace

namespace ub {
int moe_align(int32_t* sorted_ids, int32_t* experts_ids, int32_t* num_post_pad, const int32_t* topk_ids,
              const int32_t* real_token_num, const int32_t* expert_map, int E, int block, int T, int k,
              cudaStream_t s) {
  return moe_align_launch(sorted_ids, experts_ids, num_post_pad, topk_ids, real_token_num, expert_map, E, block, T, k,
                          s);
}
int topk_softmax_bf16_impl(const void* in, void* out_w, int* out_idx, int T, int E, int k, int norm, cudaStream_t s) {
  return topk_softmax_launch<__nv_bfloat16>(in, out_w, out_idx, T, E, k, norm, s);
}
}  // namespace ub

extern "C" {

void topk_softmax_f32(float* input, float* output, int* index, int32_t num_tokens, int32_t num_experts, int32_t topk,
                      int32_t norm_topk_prob, void* stream) {
  topk_softmax_launch<float>(input, output, index, num_tokens, num_experts, topk, norm_topk_prob != 0,
                             ub::as_stream(stream));
}
void topk_softmax_f16(void* input, void* output, int* index, int32_t num_tokens, int32_t num_experts, int32_t topk,
                      int32_t norm_topk_prob, void* stream) {
  topk_softmax_launch<__half>(input, output, index, num_tokens, num_experts, topk, norm_topk_prob != 0,
                              ub::as_stream(stream));
}
void topk_softmax_bf16(void* input, void* output, int* index, int32_t num_tokens, int32_t num_experts, int32_t topk,
                       int32_t norm_topk_prob, void* stream) {
  topk_softmax_launch<__nv_bfloat16>(input, output, index, num_tokens, num_experts, topk, norm_topk_prob != 0,
                                     ub::as_stream(stream));
}

void moe_align_block_size(int32_t* sorted_ids, int32_t* experts_ids, int32_t* num_tokens_post_pad, int32_t* topk_ids,
                          int32_t* real_token_num, int32_t* expert_map, int32_t num_experts, int32_t block_size,
                          int32_t token_num, int32_t topk, void* stream) {
  moe_align_launch(sorted_ids, experts_ids, num_tokens_post_pad, topk_ids, real_token_num, expert_map, num_experts,
                   block_size, token_num, topk, ub::as_stream(stream));
}

void invoke_fused_moe_f16(void* C, void* A, void* B, void* bias, float* topk_weights, int32_t* sorted_ids,
                          int32_t* experts_ids, int32_t* num_tokens_post_pad, int32_t M, int32_t K, int32_t N,
                          int32_t E, int32_t topk_ids_size, int32_t top_k, int32_t block_size,
                          int32_t mul_routed_weight, int32_t bias_flag, void* stream) {
  fused_moe_dense_launch<__half>(C, A, B, bias, topk_weights, sorted_ids, experts_ids, num_tokens_post_pad, M, K, N, E,
                                 topk_ids_size, top_k, block_size, mul_routed_weight, bias_flag,
                                 ub::as_stream(stream));
}
void invoke_fused_moe_bf16(void* C, void* A, void* B, void* bias, float* topk_weights, int32_t* sorted_ids,
                           int32_t* experts_ids, int32_t* num_tokens_post_pad, int32_t M, int32_t K, int32_t N,
                           int32_t E, int32_t topk_ids_size, int32_t top_k, int32_t block_size,
                           int32_t mul_routed_weight, int32_t bias_flag, void* stream) {
  fused_moe_dense_launch<__nv_bfloat16>(C, A, B, bias, topk_weights, sorted_ids, experts_ids, num_tokens_post_pad, M,
                                        K, N, E, topk_ids_size, top_k, block_size, mul_routed_weight, bias_flag,
                                        ub::as_stream(stream));
}

void moe_f16(void* y, void* e_out, float* w, uint32_t* idx, uint32_t* top, int N, int K, int M, int topk,
             void* stream) {
  moe_combine_launch<__half>(y, e_out, w, idx, top, N, K, M, topk, ub::as_stream(stream));
}
void moe_bf16(void* y, void* e_out, float* w, uint32_t* idx, uint32_t* top, int N, int K, int M, int topk,
              void* stream) {
  moe_combine_launch<__nv_bfloat16>(y, e_out, w, idx, top, N, K, M, topk, ub::as_stream(stream));
}

void indexed_moe_f16(void* in, void* w, void* out, uint32_t* indices, int N, int K, int M, int batch, int topk,
                     int num_experts, void* stream) {
  indexed_moe_launch<__half>(in, w, out, indices, N, K, M, batch, topk, num_experts, ub::as_stream(stream));
}
void indexed_moe_bf16(void* in, void* w, void* out, uint32_t* indices, int N, int K, int M, int batch, int topk,
                      int num_experts, void* stream) {
  indexed_moe_launch<__nv_bfloat16>(in, w, out, indices, N, K, M, batch, topk, num_experts, ub::as_stream(stream));
}

int topsaten_topk_softmax_f32(float* gating_output, float* topk_weights, int32_t* topk_indices,
                              int32_t* token_expert_indices, int32_t num_tokens, int32_t num_experts, int32_t topk,
                              int32_t norm_topk_prob, void* stream) {
  // token_expert_indices [num_tokens, topk] is an output tensor of the vendor op
  // (kernels/topsaten_moe_wrapper.cpp:95-100); it receives slot (t, j) -> j * num_tokens + t, the
  // source-row numbering of vLLM's topk_softmax, which that op mirrors.  NULL is accepted.
  return topk_softmax_launch<float>(gating_output, topk_weights, topk_indices, num_tokens, num_experts, topk,
                                    norm_topk_prob != 0, ub::as_stream(stream), token_expert_indices);
}

int topsaten_moe_align_block_size(int32_t* sorted_token_ids, int32_t* experts_ids, int32_t* num_tokens_post_pad,
                                  int32_t* topk_ids, int32_t num_tokens, int32_t topk, int32_t num_experts,
                                  int32_t block_size, void* stream) {
  return moe_align_launch(sorted_token_ids, experts_ids, num_tokens_post_pad, topk_ids, nullptr, nullptr, num_experts,
                          block_size, num_tokens, topk, ub::as_stream(stream));
}

int topsaten_fused_moe_gemm(void* c, void* a, void* b, float* topk_weights, int32_t* topk_ids,
                            int32_t* sorted_token_ids, int32_t* expert_ids, int32_t* num_tokens_post_padded,
                            int32_t mul_routed_weight, int32_t topk, int32_t block_size, int32_t num_tokens,
                            int32_t hidden_dim, int32_t inter_dim, int32_t num_experts, int32_t dtype_code,
                            void* stream) {
  (void)topk_ids;
  // C [num_tokens, topk, inter_dim], A [num_tokens, hidden_dim] (or [num_tokens*topk, hidden_dim] when the
  // routed weight is applied), B [num_experts, inter_dim, hidden_dim]  (kernels/topsaten_moe_wrapper.cpp:143-151)
  const int slots = num_tokens * topk;
  if (dtype_code == UB_DTYPE_F16)
    return fused_moe_dense_launch<__half>(c, a, b, nullptr, topk_weights, sorted_token_ids, expert_ids,
                                          num_tokens_post_padded, num_tokens, hidden_dim, inter_dim, num_experts,
                                          slots, topk, block_size, mul_routed_weight, 0, ub::as_stream(stream));
  if (dtype_code == UB_DTYPE_BF16)
    return fused_moe_dense_launch<__nv_bfloat16>(c, a, b, nullptr, topk_weights, sorted_token_ids, expert_ids,
                                                 num_tokens_post_padded, num_tokens, hidden_dim, inter_dim,
                                                 num_experts, slots, topk, block_size, mul_routed_weight, 0,
                                                 ub::as_stream(stream));
  return ub::fail(UB_ERR_UNSUPPORTED);
}

void topsaten_release_graph_workspace_pool(void* stream) { (void)stream; }

int ub_silu_and_mul(void* out, const void* in, int rows, int D, int dtype, void* stream) {
  if (rows == 0 || D == 0) return ub::fail(UB_OK);
  if (!out || !in || rows < 0 || D < 0) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t total = static_cast<size_t>(rows) * D;
  UB_DISPATCH_FLOAT(dtype, T, (silu_and_mul_kernel<T><<<ew_grid(total), 256, 0, ub::as_stream(stream)>>>(
                                  static_cast<T*>(out), static_cast<const T*>(in), static_cast<size_t>(rows), D)));
  return ub::check_launch();
}

int ub_topk_sum(void* out, const void* in, int T_tokens, int topk, int H, int dtype, void* stream) {
  if (T_tokens == 0 || H == 0) return ub::fail(UB_OK);
  if (!out || !in || T_tokens < 0 || topk <= 0 || H < 0) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t total = static_cast<size_t>(T_tokens) * H;
  UB_DISPATCH_FLOAT(dtype, T, (topk_sum_kernel<T><<<ew_grid(total), 256, 0, ub::as_stream(stream)>>>(
                                  static_cast<T*>(out), static_cast<const T*>(in), static_cast<size_t>(T_tokens), topk,
                                  H)));
  return ub::check_launch();
}

}  // extern "C"
