// Entry points of the fused quantized matmul and the M-bucket dispatch behind them.
//
// The reference picks a matmul variant per shape with AtenGemmTuner (src/gemm_tuner.rs:326-359,
// small-M special cases :502-514) and kernels/matmul.cpp:1197-1208 (LHS-resident decode kernel when it
// fits, batched kernel otherwise).  The same idea here is a three-way split on M:
//   M <= 16           bandwidth-bound decode GEMV (qgemv.cu), f32 or bf16 activations, no workspace;
//                     from M = 9 on, Q4_K with bf16 activations AND bf16 output takes the tensor-core kernel
//                     instead (one pass of it is faster than two passes of eight tokens; no workspace either);
//   M  > 16, Q4_K     tcgen05 tensor-core GEMM with in-kernel dequantisation (bf16 activations and output;
//                     other types are converted through the caller's workspace);
//   M  > 16, Q8_0     the same tensor-core kernel with a Q8_0 producer (K % 256 == 0, 16-byte aligned weights,
//                     workspace as for Q4_K when the types are not bf16); otherwise the decode kernel in passes.
#include <string.h>

#include <mutex>

#include "ar_epilogue.cuh"
#include "common.cuh"

namespace ub {
template <typename XT>
int qgemv(bool is_q4k, void* y, const XT* x, const void* wq, int M, int N, int K, int y_dtype, bool fresh,
          cudaStream_t s);
template <typename XT>
int qgemv_ar(bool is_q4k, void* y, const XT* x, const void* wq, int M, int N, int K, int y_dtype, bool fresh,
             const ArParams* ar, cudaStream_t s);
template <typename XT>
int q4k_gemv_m1_gate_up(const void* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, const void* gamma,
                        float eps, cudaStream_t s);
template <typename XT>
int q4k_gemv_m1x(const void* wq, const XT* x, void* y, int N, int K, int y_dtype, bool fresh, const M1Extras& ex,
                 cudaStream_t s);
int q4k_gemm_mma(void* y, const void* x, const void* wq, int M, int N, int K, cudaStream_t s);
uint32_t oneshot_spin_limit();
void* tensor_map_encoder();
int q4k_gemm_tc(void* y, const void* x, const void* wq, int M, int N, int K, bool fresh, cudaStream_t s);
int q8_0_gemm_tc(void* y, const void* x, const void* wq, int M, int N, int K, bool fresh, cudaStream_t s);
}  // namespace ub

namespace {

constexpr int kDecodeMaxM = 16;
constexpr int kDecodeOnePassM = 8;  // tokens one launch of the decode kernel covers

__global__ void convert_f32_to_bf16_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ in, size_t n) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16_rn(in[i]);
}

template <typename T>
__global__ void convert_bf16_to_kernel(T* __restrict__ out, const __nv_bfloat16* __restrict__ in, size_t n) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[i] = ub::from_f32<T>(__bfloat162float(in[i]));
}

// RMSNorm of rows: out = T(T(x * rsqrt(mean(x^2) + eps)) * gamma), the normalised value rounded to the storage
// type before the weight is applied (the usual definition).  One warp per row.
template <typename T>
__global__ void __launch_bounds__(256) rms_norm_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                       const T* __restrict__ gamma, int rows, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* x = in + static_cast<size_t>(row) * H;
  float ss = 0.f;
  for (int k = lane; k < H; k += 32) {
    const float v = ub::to_f32(x[k]);
    ss = fmaf(v, v, ss);
  }
  ss = ub::warp_sum(ss);
  const float scale = rsqrtf(ss / static_cast<float>(H) + eps);
  T* o = out + static_cast<size_t>(row) * H;
  for (int k = lane; k < H; k += 32)
    o[k] = ub::from_f32<T>(ub::to_f32(ub::from_f32<T>(ub::to_f32(x[k]) * scale)) * ub::to_f32(gamma[k]));
}

// y += r (bf16), the residual add behind a matmul that could not carry it in its epilogue
__global__ void add_bf16_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ r, size_t n) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    y[i] = __float2bfloat16_rn(__bfloat162float(r[i]) + __bfloat162float(y[i]));
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline int conv_grid(size_t n) {
  size_t b = (n + 255) / 256;
  const size_t cap = static_cast<size_t>(ub::num_sms()) * 8;
  return static_cast<int>(b > cap ? cap : (b ? b : 1));
}

// x_dtype: UB_DTYPE_F32 or UB_DTYPE_BF16
int qmatmul(bool is_q4k, int x_dtype, void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype,
            void* workspace, size_t ws_bytes, void* stream) {
  // UB_QMATMUL_WEIGHTS_FRESH rides in the upper bits of out_dtype
  bool fresh = (out_dtype & UB_QMATMUL_WEIGHTS_FRESH) != 0;
  out_dtype &= ~UB_QMATMUL_WEIGHTS_FRESH;
  if (M == 0 || N == 0) return ub::fail(UB_OK);
  if (!y || !x || !wq || M < 0 || N < 0 || K <= 0) return ub::fail(UB_ERR_INVALID_ARG);
  if (K % (is_q4k ? UB_QK_K : UB_QK8_0)) return ub::fail(UB_ERR_INVALID_ARG);
  if (out_dtype != UB_DTYPE_F32 && out_dtype != UB_DTYPE_BF16 && out_dtype != UB_DTYPE_F16)
    return ub::fail(UB_ERR_INVALID_ARG);
  // 16-byte loads on activations and (Q4_K) weight rows
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (is_q4k && (reinterpret_cast<uintptr_t>(wq) & 15)) ||
      (!is_q4k && (reinterpret_cast<uintptr_t>(wq) & 1)) || (x_dtype == UB_DTYPE_BF16 && (K % 8)) ||
      (x_dtype == UB_DTYPE_F32 && (K % 4)))
    return ub::fail(UB_ERR_INVALID_ARG);
  cudaStream_t s = ub::as_stream(stream);
  if (ub::take_weights_written(s)) fresh = true;

  if (is_q4k && M > kDecodeOnePassM && M <= kDecodeMaxM && x_dtype == UB_DTYPE_BF16 && out_dtype == UB_DTYPE_BF16) {
    const int st = ub::q4k_gemm_tc(y, x, wq, M, N, K, fresh, s);
    if (st != UB_ERR_UNSUPPORTED) return st;  // unsupported shape or driver: the decode kernel below
  }
  auto decode = [&]() {
    if (x_dtype == UB_DTYPE_F32)
      return ub::qgemv<float>(is_q4k, y, static_cast<const float*>(x), wq, M, N, K, out_dtype, fresh, s);
    return ub::qgemv<__nv_bfloat16>(is_q4k, y, static_cast<const __nv_bfloat16*>(x), wq, M, N, K, out_dtype, fresh, s);
  };
  if (M <= kDecodeMaxM) return decode();

  // tensor-core path: bf16 in, bf16 out; convert around it when the caller's types differ
  const size_t need = ub_qmatmul_workspace_bytes(M, N, K, 1);
  const bool conv_in = x_dtype != UB_DTYPE_BF16, conv_out = out_dtype != UB_DTYPE_BF16;
  const bool ws_ok = workspace && ws_bytes >= need && !(reinterpret_cast<uintptr_t>(workspace) & 255);
  if (!is_q4k) {
    // Q8_0 keeps the decode kernel (passes of eight tokens) where the tensor-core kernel cannot run: rows that are
    // not whole 16-byte pieces, unaligned weights, or a caller that brought no workspace for the conversions
    if (K % UB_QK_K || (reinterpret_cast<uintptr_t>(wq) & 15) || ((conv_in || conv_out) && !ws_ok) ||
        !ub::tensor_map_encoder())
      return decode();
  } else if ((conv_in || conv_out) && !ws_ok) {
    return ub::fail(UB_ERR_WORKSPACE);
  }
  char* ws = static_cast<char*>(workspace);
  const void* xin = x;
  void* yout = y;
  if (conv_in) {
    __nv_bfloat16* xb = reinterpret_cast<__nv_bfloat16*>(ws);
    const size_t n = static_cast<size_t>(M) * K;
    convert_f32_to_bf16_kernel<<<conv_grid(n), 256, 0, s>>>(xb, static_cast<const float*>(x), n);
    xin = xb;
  }
  if (conv_out) yout = ws + align_up(static_cast<size_t>(M) * K * 2, 256);
  int st = is_q4k ? ub::q4k_gemm_tc(yout, xin, wq, M, N, K, fresh, s) : ub::q8_0_gemm_tc(yout, xin, wq, M, N, K, fresh, s);
  // no tensor-map encoder in this driver: the mma.sync kernel computes the same product
  if (st == UB_ERR_UNSUPPORTED && is_q4k) st = ub::q4k_gemm_mma(yout, xin, wq, M, N, K, s);
  if (st != UB_OK) return st;
  if (conv_out) {
    const size_t n = static_cast<size_t>(M) * N;
    if (out_dtype == UB_DTYPE_F32)
      convert_bf16_to_kernel<float><<<conv_grid(n), 256, 0, s>>>(static_cast<float*>(y),
                                                                static_cast<const __nv_bfloat16*>(yout), n);
    else
      convert_bf16_to_kernel<__half><<<conv_grid(n), 256, 0, s>>>(static_cast<__half*>(y),
                                                                 static_cast<const __nv_bfloat16*>(yout), n);
  }
  return ub::check_launch();
}

// ---- scratch of ub_qmatmul_q4k_f32_static: lives in the library's device image, one copy per GPU ----
constexpr size_t kStaticScratchBytes = static_cast<size_t>(8) << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel may use.
// The device address is looked up once per device (with that device current) and cached here.
std::mutex g_static_mu;
void* g_static_ptr[64] = {nullptr};

int static_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  if (dev < 0 || dev >= 64) return ub::fail(UB_ERR_INVALID_ARG);  // more devices than the address table holds
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      ub::set_cuda_error(e);
      return ub::fail(UB_ERR_CUDA);
    }
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return UB_OK;
}

}  // namespace

extern "C" {

// Scratch for the tensor-core path when the caller's activation or output type is not bf16:
// a bf16 copy of x and a bf16 staging copy of y.  0 for the decode kernel.  Q8_0 (is_q4k == 0) may be called
// without it: it then keeps the decode kernel in passes of eight tokens.
size_t ub_qmatmul_workspace_bytes(int M, int N, int K, int is_q4k) {
  (void)is_q4k;
  if (M <= kDecodeMaxM || M <= 0 || N <= 0 || K <= 0) return 0;
  return align_up(static_cast<size_t>(M) * K * 2, 256) + align_up(static_cast<size_t>(M) * N * 2, 256);
}

int ub_qmatmul_q8_0_f32(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* workspace,
                        size_t ws_bytes, void* stream) {
  return qmatmul(false, UB_DTYPE_F32, y, x, wq, M, N, K, out_dtype, workspace, ws_bytes, stream);
}
int ub_qmatmul_q8_0_bf16(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* workspace,
                         size_t ws_bytes, void* stream) {
  return qmatmul(false, UB_DTYPE_BF16, y, x, wq, M, N, K, out_dtype, workspace, ws_bytes, stream);
}
int ub_qmatmul_q4k_f32(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* workspace,
                       size_t ws_bytes, void* stream) {
  return qmatmul(true, UB_DTYPE_F32, y, x, wq, M, N, K, out_dtype, workspace, ws_bytes, stream);
}
int ub_qmatmul_q4k_bf16(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* workspace,
                        size_t ws_bytes, void* stream) {
  return qmatmul(true, UB_DTYPE_BF16, y, x, wq, M, N, K, out_dtype, workspace, ws_bytes, stream);
}

// ---- gate/up projection with the SiLU.up step in the matmul's epilogue ----
// y[M, I] = silu(x . Wgate^T) * (x . Wup^T) with wq = [gate rows; up rows] (2 I rows of K), bf16 activations.
// One token with K a multiple of 2048 up to 12288 is ONE launch; everything else is the matmul into the
// workspace followed by ub_silu_and_mul (the reference's own sequence, kernels/topsaten_ops_wrapper.cpp:375-391).
size_t ub_qmatmul_q4k_gate_up_workspace_bytes(int M, int I, int K) {
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  return align_up(static_cast<size_t>(M) * 2 * I * 2, 256) + align_up(ub_qmatmul_workspace_bytes(M, 2 * I, K, 1), 256);
}

int ub_qmatmul_q4k_gate_up_bf16(void* y, const void* x, const void* wq, int M, int I, int K, int out_dtype,
                                void* workspace, size_t ws_bytes, void* stream) {
  bool fresh = (out_dtype & UB_QMATMUL_WEIGHTS_FRESH) != 0;
  out_dtype &= ~UB_QMATMUL_WEIGHTS_FRESH;
  if (M == 0 || I == 0) return ub::fail(UB_OK);
  if (!y || !x || !wq || M < 0 || I < 0 || K <= 0 || K % UB_QK_K) return ub::fail(UB_ERR_INVALID_ARG);
  if (out_dtype != UB_DTYPE_BF16 && out_dtype != UB_DTYPE_F16 && out_dtype != UB_DTYPE_F32)
    return ub::fail(UB_ERR_INVALID_ARG);
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15)) return ub::fail(UB_ERR_INVALID_ARG);
  cudaStream_t s = ub::as_stream(stream);
  if (ub::take_weights_written(s)) fresh = true;
  if (M == 1) {
    const int st = ub::q4k_gemv_m1_gate_up<__nv_bfloat16>(wq, static_cast<const __nv_bfloat16*>(x), y, I, K, out_dtype,
                                                         fresh, nullptr, 0.f, s);
    if (st != UB_ERR_UNSUPPORTED) return st;
  }
  const size_t need = ub_qmatmul_q4k_gate_up_workspace_bytes(M, I, K);
  if (!workspace || ws_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255)) return ub::fail(UB_ERR_WORKSPACE);
  char* ws = static_cast<char*>(workspace);
  const size_t gu_bytes = align_up(static_cast<size_t>(M) * 2 * I * 2, 256);
  // the intermediate is bf16 (f16 when that is the output type), as in the two-call sequence
  const int mid = out_dtype == UB_DTYPE_F16 ? UB_DTYPE_F16 : UB_DTYPE_BF16;
  int st = qmatmul(true, UB_DTYPE_BF16, ws, x, wq, M, 2 * I, K, mid | (fresh ? UB_QMATMUL_WEIGHTS_FRESH : 0),
                   ws + gu_bytes, ws_bytes - gu_bytes, stream);
  if (st != UB_OK) return st;
  if (out_dtype == UB_DTYPE_F32) return ub::fail(UB_ERR_UNSUPPORTED);  // f32 output exists on the one-token path only
  return ub_silu_and_mul(y, ws, M, I, out_dtype, stream);
}

// ---- RMSNorm in front of the matmul ----
// The reference's stand-alone norm (src/ffi.rs:719-728): output[t,:] = rmsnorm(input[t,:]) * gamma.
int topsaten_rms_norm(void* output, const void* input, const void* gamma, int num_tokens, int hidden_size, float epsilon,
                      int dtype_code, void* stream) {
  if (num_tokens == 0 || hidden_size == 0) return ub::fail(UB_OK);
  if (!output || !input || !gamma || num_tokens < 0 || hidden_size < 0) return ub::fail(UB_ERR_INVALID_ARG);
  const int grid = (num_tokens + 7) / 8;
  cudaStream_t s = ub::as_stream(stream);
  UB_DISPATCH_FLOAT(dtype_code, T, (rms_norm_kernel<T><<<grid, 256, 0, s>>>(static_cast<T*>(output),
                                                                          static_cast<const T*>(input),
                                                                          static_cast<const T*>(gamma), num_tokens,
                                                                          hidden_size, epsilon)));
  return ub::check_launch();
}

size_t ub_qmatmul_q4k_rmsnorm_workspace_bytes(int M, int N, int K, int gate_up) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const size_t inner = gate_up ? ub_qmatmul_q4k_gate_up_workspace_bytes(M, N, K) : ub_qmatmul_workspace_bytes(M, N, K, 1);
  return align_up(static_cast<size_t>(M) * K * 2, 256) + align_up(inner, 256);
}

// y = rmsnorm(x; gamma, eps) . W^T (gate_up == 0, y [M,N]) or silu(. Wgate^T) * (. Wup^T) (gate_up != 0, y [M,N] with
// W = [gate rows; up rows] of 2 N rows), x and gamma bf16.  One token with K a multiple of 2048 up to 12288 is one
// launch: every CTA of the matmul normalises the activation row in its prologue.  Other shapes run
// topsaten_rms_norm into the workspace and then the matmul.
int ub_qmatmul_q4k_rmsnorm_bf16(void* y, const void* x, const void* gamma, float eps, const void* wq, int M, int N,
                                int K, int gate_up, int out_dtype, void* workspace, size_t ws_bytes, void* stream) {
  if (M == 0 || N == 0) return ub::fail(UB_OK);
  if (!y || !x || !gamma || !wq || M < 0 || N < 0 || K <= 0 || K % UB_QK_K) return ub::fail(UB_ERR_INVALID_ARG);
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(gamma) & 15) ||
      (reinterpret_cast<uintptr_t>(wq) & 15))
    return ub::fail(UB_ERR_INVALID_ARG);
  cudaStream_t s = ub::as_stream(stream);
  if (M == 1) {
    const bool fresh = ub::take_weights_written(s);
    int st;
    if (gate_up) {
      st = ub::q4k_gemv_m1_gate_up<__nv_bfloat16>(wq, static_cast<const __nv_bfloat16*>(x), y, N, K, out_dtype, fresh,
                                                  gamma, eps, s);
    } else {
      const ub::M1Extras ex = {gamma, eps, nullptr};
      st = ub::q4k_gemv_m1x<__nv_bfloat16>(wq, static_cast<const __nv_bfloat16*>(x), y, N, K, out_dtype, fresh, ex, s);
    }
    if (st != UB_ERR_UNSUPPORTED) return st;
  }
  const size_t need = ub_qmatmul_q4k_rmsnorm_workspace_bytes(M, N, K, gate_up);
  if (!workspace || ws_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255)) return ub::fail(UB_ERR_WORKSPACE);
  char* ws = static_cast<char*>(workspace);
  const size_t xn_bytes = align_up(static_cast<size_t>(M) * K * 2, 256);
  int st = topsaten_rms_norm(ws, x, gamma, M, K, eps, UB_DTYPE_BF16, stream);
  if (st != UB_OK) return st;
  if (gate_up) return ub_qmatmul_q4k_gate_up_bf16(y, ws, wq, M, N, K, out_dtype, ws + xn_bytes, ws_bytes - xn_bytes, stream);
  return qmatmul(true, UB_DTYPE_BF16, y, ws, wq, M, N, K, out_dtype, ws + xn_bytes, ws_bytes - xn_bytes, stream);
}

// ---- row-split matmul with the all-reduce over the ranks in its epilogue ----
// y[M, N] (bf16, summed over the ranks, identical bits on every rank) = sum_r x_r[M, K] . W_r^T.  `staging`,
// rank, world, max_bytes as for ub_allreduce_oneshot_bf16 (the same buffers serve both; M*N*2 <= max_bytes).
// One token is ONE launch on every kernel that takes the shape (the matmul's CTAs push their rows to the
// peers, the last CTA completes the exchange); other shapes run the matmul and then the one-shot exchange.
int ub_qmatmul_q4k_allreduce_bf16(void* y, const void* x, const void* wq, int M, int N, int K, void* const* staging,
                                  int rank, int world, size_t max_bytes, void* stream) {
  return ub_qmatmul_q4k_allreduce_residual_bf16(y, x, wq, nullptr, M, N, K, staging, rank, world, max_bytes, stream);
}

// The same with the residual add of a decoder layer: y = residual + sum over the ranks (residual bf16 [M,N], may
// be null, must not alias y).  world <= 1: y = residual + x . W^T in the matmul's epilogue for one token.
int ub_qmatmul_q4k_allreduce_residual_bf16(void* y, const void* x, const void* wq, const void* residual, int M, int N,
                                           int K, void* const* staging, int rank, int world, size_t max_bytes,
                                           void* stream) {
  if (M == 0 || N == 0) return ub::fail(UB_OK);
  if (!y || !x || !wq || M < 0 || N < 0 || K <= 0 || K % UB_QK_K) return ub::fail(UB_ERR_INVALID_ARG);
  if (residual && (residual == y || (reinterpret_cast<uintptr_t>(residual) & 15))) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t n_out = static_cast<size_t>(M) * N;
  auto add_residual = [&]() -> int {
    if (!residual) return UB_OK;
    size_t blocks = (n_out + 255) / 256;
    const size_t cap = static_cast<size_t>(ub::num_sms()) * 8;
    add_bf16_kernel<<<static_cast<unsigned>(blocks > cap ? cap : blocks), 256, 0, ub::as_stream(stream)>>>(
        static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(residual), n_out);
    return ub::check_launch();
  };
  if (world <= 1) {
    if (M == 1 && residual && !(reinterpret_cast<uintptr_t>(x) & 15)) {
      ub::ArParams ar;
      memset(&ar, 0, sizeof(ar));
      ar.residual = static_cast<const __nv_bfloat16*>(residual);
      const ub::M1Extras ex = {nullptr, 0.f, &ar};
      const int st = ub::q4k_gemv_m1x<__nv_bfloat16>(wq, static_cast<const __nv_bfloat16*>(x), y, N, K, UB_DTYPE_BF16,
                                                     ub::take_weights_written(ub::as_stream(stream)), ex,
                                                     ub::as_stream(stream));
      if (st != UB_ERR_UNSUPPORTED) return st;
    }
    const int st = qmatmul(true, UB_DTYPE_BF16, y, x, wq, M, N, K, UB_DTYPE_BF16, nullptr, 0, stream);
    return st != UB_OK ? st : add_residual();
  }
  if (!staging || world > ub::kArMaxWorld || rank < 0 || rank >= world || (max_bytes & 15))
    return ub::fail(UB_ERR_INVALID_ARG);
  const size_t count = static_cast<size_t>(M) * N;
  if (count % 8 || (reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(wq) & 15))
    return ub::fail(UB_ERR_INVALID_ARG);
  if (count * 2 > max_bytes) return ub::fail(UB_ERR_TOO_LARGE);
  cudaStream_t s = ub::as_stream(stream);
  if (M == 1) {
    ub::ArParams ar;
    memset(&ar, 0, sizeof(ar));
    for (int p = 0; p < world; p++) {
      ar.base[p] = static_cast<unsigned char*>(staging[p]);
      if (!ar.base[p] || (reinterpret_cast<uintptr_t>(ar.base[p]) & 15)) return ub::fail(UB_ERR_INVALID_ARG);
    }
    ar.rank = rank, ar.world = world, ar.max_bytes = max_bytes;
    ar.residual = static_cast<const __nv_bfloat16*>(residual);
    ar.spin_limit = ub::oneshot_spin_limit();
    const bool fresh = ub::take_weights_written(s);
    const int st = ub::qgemv_ar<__nv_bfloat16>(true, y, static_cast<const __nv_bfloat16*>(x), wq, 1, N, K, UB_DTYPE_BF16,
                                               fresh, &ar, s);
    if (st != UB_ERR_UNSUPPORTED) return st;
  }
  int st = qmatmul(true, UB_DTYPE_BF16, y, x, wq, M, N, K, UB_DTYPE_BF16, nullptr, 0, stream);
  if (st != UB_OK) return st;
  st = ub_allreduce_oneshot_bf16(y, count, staging, rank, world, max_bytes, stream);
  return st != UB_OK ? st : add_residual();
}

// ub_qmatmul_q4k_f32 for callers that have no way to hand over a workspace: the type-conversion
// scratch of the M > 16 path sits in a fixed 8 MiB array inside the library's device image instead of
// a caller buffer, and this function never allocates (no cudaMalloc / cudaFree, no allocating library
// call).  Shapes whose scratch need (ub_qmatmul_workspace_bytes) exceeds 8 MiB get UB_ERR_TOO_LARGE.
// The first call on each device resolves the array's device address; make that call outside any
// stream capture.  All calls on a device share the one array, so two calls that can overlap on the
// GPU (different streams) race on it; nothing in it has to start at zero, every byte that is read is
// written earlier in the same call.
int ub_qmatmul_q4k_f32_static(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype,
                              void* stream) {
  const size_t need = ub_qmatmul_workspace_bytes(M, N, K, 1);
  if (need > kStaticScratchBytes) return ub::fail(UB_ERR_TOO_LARGE);
  void* scratch = nullptr;
  const int st = static_scratch(&scratch);
  if (st != UB_OK) return st;
  return qmatmul(true, UB_DTYPE_F32, y, x, wq, M, N, K, out_dtype, scratch, kStaticScratchBytes, stream);
}

}  // extern "C"
