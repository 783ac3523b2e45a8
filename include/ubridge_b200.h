/*
 * ubridge_b200 — C-ABI of the B200 (sm_100a) quantized-linear + fused-MoE path.
 *
 * Plain C: pointers, sizes and ints only.  Every pointer is caller-owned DEVICE memory
 * unless a comment says "host".  Every call enqueues on the CUDA stream passed as the
 * trailing `void* stream` (a cudaStream_t; NULL = the legacy default stream) and returns
 * without synchronising, exactly like the reference's host launchers.  Outputs and
 * workspaces are pre-allocated by the caller; the library allocates nothing on these
 * paths and keeps no pointer after a call returns.
 *
 * Each declaration cites the reference interface it replaces as  file:line  (paths
 * inside the reference project).  Exports that keep a reference name keep its argument
 * order, meaning and `void` return; status of the last such call on the calling thread
 * is readable through ub_last_status().  New exports return an int status.
 */
#ifndef UBRIDGE_B200_H_
#define UBRIDGE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status codes */
enum {
  UB_OK = 0,
  UB_ERR_INVALID_ARG = 1,   /* bad shape, null pointer, unsupported dtype            */
  UB_ERR_UNSUPPORTED = 2,   /* name not in the registry / path not built             */
  UB_ERR_WORKSPACE = 3,     /* workspace missing or too small                        */
  UB_ERR_CUDA = 4,          /* a CUDA runtime call failed (see ub_last_cuda_error)   */
  UB_ERR_BAD_INDEX = 5,     /* device saw an expert id / slot outside its range      */
  UB_ERR_TIMEOUT = 6,       /* a bounded device-side wait ran out                    */
  UB_ERR_NCCL = 7,          /* NCCL missing or a collective call failed              */
  UB_ERR_TOO_LARGE = 8,     /* size beyond a fixed limit of the entry point          */
  UB_ERR_NOT_READY = 9      /* ub_stream_query: work is still pending on the stream  */
};

/* element type codes: the reference's DATATYPE enum, src/lib.rs:87-106 (kernels/utils/utils.h:31-49) */
enum { UB_DTYPE_I8 = 0, UB_DTYPE_U8 = 1, UB_DTYPE_F16 = 4, UB_DTYPE_BF16 = 5, UB_DTYPE_I32 = 6, UB_DTYPE_F32 = 8, UB_DTYPE_I4 = 15 };

/* opcodes of the shim: src/device_opcode.rs:16-46 keeps an (unused) opcode enum; the
 * quantized path's operations are numbered here in the same spirit. */
enum {
  UB_OP_DEQUANT_Q8_0 = 100,
  UB_OP_DEQUANT_Q4K = 101,
  UB_OP_QUANTIZE_Q8_0 = 102,
  UB_OP_QMATMUL_Q8_0 = 110,
  UB_OP_QMATMUL_Q4K = 111,
  UB_OP_TOPK_SOFTMAX = 120,
  UB_OP_MOE_ALIGN = 121,
  UB_OP_FUSED_MOE = 122,
  UB_OP_MOE_COMBINE = 123,
  UB_OP_INDEXED_MOE = 124,
  UB_OP_FUSED_MOE_Q4K = 125,
  UB_OP_MATMUL = 130,
  UB_OP_MATMUL_W4 = 131,
  UB_OP_MATMUL_W8 = 132
};

int ub_version(void);
const char* ub_status_string(int status);
/* status of the most recent call made by the calling thread (void exports included) */
int ub_last_status(void);
/* last cudaError_t seen by the calling thread, as an int */
int ub_last_cuda_error(void);
/* Reads (and clears) the per-device error word that kernels set instead of trapping:
 * the reference traps the device on a bad expert id (kernels/utils/moe_kernel_compat.h:21-28,
 * kernels/moe_align_host.cpp:101-163).  Synchronises `stream`.  Returns UB_OK,
 * UB_ERR_BAD_INDEX or UB_ERR_TIMEOUT. */
int ub_device_status(void* stream);

/* ------------------------------------------------------------------ device, memory, stream
 * Mirrors GcuDevice (src/gcu_device.rs:61-635): one device + one non-blocking stream,
 * stream-ordered alloc/free, H2D / D2H / D2D copies, synchronize. */
typedef struct ub_device ub_device;
int ub_device_count(void);                                         /* gcu_device.rs: GcuDevice::count */
int ub_device_new(int ordinal, ub_device** out);                   /* gcu_device.rs:108-139 */
void ub_device_free(ub_device* dev);
int ub_device_ordinal(const ub_device* dev);
void* ub_device_stream(const ub_device* dev);                      /* the device's cudaStream_t */
int ub_device_bind(const ub_device* dev);                          /* gcu_device.rs:144-147 (select device) */
int ub_alloc(ub_device* dev, size_t bytes, void** out);            /* gcu_device.rs:216-260 */
int ub_alloc_zeros(ub_device* dev, size_t bytes, void** out);      /* gcu_device.rs:262-324 */
int ub_free(ub_device* dev, void* ptr);                            /* gcu_slice.rs:62-101 (stream-ordered free) */
int ub_memcpy_htod(ub_device* dev, void* dst, const void* host_src, size_t bytes); /* gcu_device.rs:337-420 */
/* Enqueues the copy on the device's stream and returns: the host bytes are valid only after ub_synchronize
 * (the reference's dtoh_sync_copy synchronises itself; the Python mirror's dtoh_sync_copy does the same). */
int ub_memcpy_dtoh(ub_device* dev, void* host_dst, const void* src, size_t bytes); /* gcu_device.rs:500-588 */
int ub_memcpy_dtod(ub_device* dev, void* dst, const void* src, size_t bytes);      /* gcu_device.rs:422-498 */
/* strided rows: `height` rows of `width_bytes`, source/destination pitches in bytes */
int ub_memcpy_dtod_2d(ub_device* dev, void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t height); /* gcu_device.rs:422-498 */
int ub_synchronize(ub_device* dev);                                /* gcu_device.rs:610-618 */
/* Non-blocking: UB_OK once everything enqueued on `stream` has completed, UB_ERR_NOT_READY while work is
 * pending.  What a host polls against a deadline instead of blocking in ub_synchronize when a peer rank may
 * have gone away (no counterpart in the reference, whose synchronize blocks: gcu_device.rs:610-618). */
int ub_stream_query(void* stream);
/* Free and total bytes of the device's memory (the mem_get_info the reference's own allocation test reads,
 * src/gcu_device.rs:708-718). */
int ub_mem_info(ub_device* dev, size_t* free_bytes, size_t* total_bytes);

/* ------------------------------------------------------------------ name -> launcher registry
 * Mirrors DeviceExecutor.function_map + GcuDevice::get_or_load_func + GcuFunction::launch
 * (src/device_executor.rs:57-61,295-308,361-376; src/gcu_device.rs:160-183;
 * src/gcu_launch.rs:183-328).  `params` is the same void*[] the reference hands to
 * topsModuleLaunchKernel: params[i] points at the i-th kernel argument.  Grid, block and
 * shared-memory fields are accepted for source compatibility and ignored: each launcher
 * sizes its own grid.  Unlike the reference (silent no-op handle, gcu_device.rs:176-182)
 * an unknown name returns NULL and launching NULL returns UB_ERR_UNSUPPORTED.
 * Registered: module "quant": dequantize_block_{q8_0,q4_k}_{f16,bf16,f32}, quantize_block_q8_0_{f16,bf16,f32}
 * (kernels/quant.cpp:257-268,341-353,477-488); module "matmul": matmul_{f32,f16,bf16} with the reference's
 * 20-parameter list and matmul_{f16,bf16}_{4bit,8bit} with its 23-parameter list
 * (kernels/matmul.cpp:1143-1150,1186-1194; W4/W8 packing as documented at dequant_f16 below). */
typedef struct ub_function ub_function;
typedef struct {
  unsigned grid_dim[3];
  unsigned block_dim[3];
  unsigned shared_mem_bytes;
  int is_cooperative_launch;
} ub_launch_config;                                                /* src/gcu_launch.rs:40-90 */

const ub_function* ub_get_function(const char* module_name, const char* func_name);
int ub_has_function(const char* module_name, const char* func_name); /* device_executor.rs:533-538 */
int ub_function_count(void);
const char* ub_function_name(int index);                           /* "module::name" */
int ub_function_opcode(const ub_function* f);
int ub_launch(const ub_function* f, const ub_launch_config* cfg, void** params, void* stream);

/* Kernels reachable by name, module "quant" (kernels/quant.cpp:257-268,341-353,477-488):
 *   dequantize_block_q8_0_{f16,bf16,f32}(int8_t* in, T* out, size_t numel)
 *   dequantize_block_q4_k_{f16,bf16,f32}(int8_t* in, T* out, size_t numel)
 *   quantize_block_q8_0_{f16,bf16,f32}(T* in, int8_t* out, size_t in_bytes, size_t out_bytes)
 * `in`/`out` use the reference's de-interleaved device layout: all block headers first,
 * then all quants (kernels/quant.cpp:219-220,300-301,441-442).  quantize_block_q4_k_* is
 * absent on purpose: the reference's own is a stub whose body is commented out
 * (kernels/quant.cpp:639-640). */

/* ------------------------------------------------------------------ GGUF block (de)quantisation
 * New entry points on INTERLEAVED GGUF blocks (34-byte Q8_0, 144-byte Q4_K; formats at
 * kernels/quant.cpp:98-104,145-150,356-363).  `numel` counts weights, a multiple of the
 * block size.  Output is bit-exact: the f32 value d*q (Q8_0) or (d*sc)*q - dmin*m (Q4_K),
 * rounded once (nearest-even) to out_dtype.  Replaces kernels/quant.cpp:188-268,372-488. */
int ub_dequant_q8_0(void* out, const void* blocks, size_t numel, int out_dtype, void* stream);
int ub_dequant_q4k(void* out, const void* blocks, size_t numel, int out_dtype, void* stream);
/* x (in_dtype) -> interleaved Q8_0 blocks; replaces kernels/quant.cpp:270-353. */
int ub_quantize_q8_0(void* blocks, const void* x, size_t numel, int in_dtype, void* stream);
/* interleaved <-> the reference's split device layout (kernels/quant.cpp:219-220,441-442) */
int ub_repack_to_split(void* split, const void* interleaved, size_t nblocks, int is_q4k, void* stream);
int ub_repack_to_interleaved(void* interleaved, const void* split, size_t nblocks, int is_q4k, void* stream);

/* ------------------------------------------------------------------ GGUF Q6_K
 * The reference declares block_q6_K (kernels/quant.cpp:170-177: ql[128], qh[64], int8 scales[16],
 * f16 d; 210 bytes per 256 weights) and ships no kernel for it; Q4_K_M model files hold their
 * output and embedding matrices in it.  Blocks are interleaved as in a .gguf file, 2-byte aligned.
 * ub_dequant_q6k: the f32 value (d*scale)*(q-32) rounded once to out_dtype, bit-exact.
 * ub_qmatmul_q6k_*: y[M,N] = x[M,K] . W^T with W = N rows of K/256 blocks, f32 accumulation, a
 * weight-streaming decode kernel that takes the tokens four at a time (any M, no workspace).  With K a multiple of
 * 2048 (up to 14336 for one token) and 16-byte aligned wq each pass runs a kernel that stages whole rows by bulk copies and requests
 * its first rows before it waits for the kernel in front of it on the stream: the precondition on the weights and
 * UB_QMATMUL_WEIGHTS_FRESH (below, ORed into out_dtype) apply to it as to ub_qmatmul_*. */
int ub_dequant_q6k(void* out, const void* blocks, size_t numel, int out_dtype, void* stream);
int ub_qmatmul_q6k_f32(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* stream);
int ub_qmatmul_q6k_bf16(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* stream);

/* ------------------------------------------------------------------ fused quantized matmul
 * y[M,N] = x[M,K] . W^T, W given as N rows of K/32 (Q8_0) or K/256 (Q4_K) interleaved GGUF
 * blocks; f32 accumulation.  The reference reaches the same result with two kernels and a
 * dense temporary: dequantize_block_* (kernels/quant.cpp:257-268,477-488) followed by
 * matmul_* (kernels/matmul.cpp:1143-1184; small-M shape in
 * kernels/third_party/matmul_decoding.h:12-570).  The suffix names the activation type;
 * out_dtype is UB_DTYPE_F32 / UB_DTYPE_BF16 / UB_DTYPE_F16.  M <= 16 runs the
 * bandwidth-bound decode kernels (Q4_K with bf16 activations and bf16 output: M <= 8), larger M
 * the tensor-core kernel — see ub_qmatmul_workspace_bytes for the scratch it needs when the
 * activation or output type is not bf16 (0 whenever M <= 16).  Q8_0 takes the tensor-core kernel when
 * K % 256 == 0 and wq is 16-byte aligned; otherwise, or when called without the scratch, it runs the
 * decode kernel in passes of eight tokens (same result within the matmul tolerance, slower).
 *
 * Precondition on the weights.  The decode kernels (M <= 16) and the tensor-core kernel up to 64 tokens are
 * launched with programmatic dependent launch
 * and request their first weight tiles BEFORE they wait for the kernel in front of them on the stream.  The
 * weight bytes must therefore be complete before that preceding kernel starts: uploaded by a copy, written
 * by a kernel that is followed by an event / synchronisation / any non-kernel operation, or simply written
 * long ago (model weights).  If the kernel launched immediately before the matmul on the same stream is the
 * one that WRITES wq (a dequantise / upload / repack kernel of the caller), OR UB_QMATMUL_WEIGHTS_FRESH into
 * out_dtype: the launch then requests nothing ahead of its dependency wait.  ub_quantize_q8_0 and
 * ub_repack_to_interleaved set this for the next matmul on their stream by themselves.  x and y carry no
 * such condition. */
#define UB_QMATMUL_WEIGHTS_FRESH 0x100
size_t ub_qmatmul_workspace_bytes(int M, int N, int K, int is_q4k);
int ub_qmatmul_q8_0_f32(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* workspace, size_t ws_bytes, void* stream);
/* Gate/up projection with SiLU.up in the matmul's epilogue: y[M,I] = silu(x . Wgate^T) * (x . Wup^T), wq = [gate
 * rows; up rows] (2 I rows of K/256 Q4_K super-blocks), x bf16, out_dtype bf16 / f16 (f32 for one token only).
 * The reference's caller runs the matmul and then silu_and_mul (kernels/topsaten_ops_wrapper.cpp:375-391); the
 * result here has the bits of that sequence (gate and up rounded to the output type first).  One token with K a
 * multiple of 2048 up to 12288 is one launch and needs no workspace; other shapes need
 * ub_qmatmul_q4k_gate_up_workspace_bytes. */
/* RMSNorm in front of the matmul.  topsaten_rms_norm is the reference's stand-alone norm (src/ffi.rs:719-728):
 * output[t,:] = T(T(input[t,:] * rsqrt(mean(input[t,:]^2) + epsilon)) * gamma), dtype_code f32 / f16 / bf16.
 * ub_qmatmul_q4k_rmsnorm_bf16 runs the Q4_K matmul (gate_up == 0: y[M,N] = xn . W^T; gate_up != 0: W = [gate
 * rows; up rows] of 2 N rows and y[M,N] = silu(xn . Wgate^T) * (xn . Wup^T)) on xn = that norm of x: for one
 * token with K a multiple of 2048 up to 12288 as ONE launch (every CTA normalises the row in its prologue),
 * otherwise norm into the workspace, then matmul (ub_qmatmul_q4k_rmsnorm_workspace_bytes). */
int topsaten_rms_norm(void* output, const void* input, const void* gamma, int num_tokens, int hidden_size, float epsilon, int dtype_code, void* stream);
size_t ub_qmatmul_q4k_rmsnorm_workspace_bytes(int M, int N, int K, int gate_up);
int ub_qmatmul_q4k_rmsnorm_bf16(void* y, const void* x, const void* gamma, float eps, const void* wq, int M, int N, int K, int gate_up, int out_dtype, void* workspace, size_t ws_bytes, void* stream);
size_t ub_qmatmul_q4k_gate_up_workspace_bytes(int M, int I, int K);
int ub_qmatmul_q4k_gate_up_bf16(void* y, const void* x, const void* wq, int M, int I, int K, int out_dtype, void* workspace, size_t ws_bytes, void* stream);
int ub_qmatmul_q8_0_bf16(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* workspace, size_t ws_bytes, void* stream);
int ub_qmatmul_q4k_f32(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* workspace, size_t ws_bytes, void* stream);
int ub_qmatmul_q4k_bf16(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* workspace, size_t ws_bytes, void* stream);
/* No counterpart in the reference.  ub_qmatmul_q4k_f32 without a workspace argument, for hosts that
 * cannot give the library device memory of their own: a plugin that only receives input and output
 * pointers from its framework, or a serving loop whose memory pool is closed after start-up, where a
 * cudaMalloc would either fail or stall every stream.  The scratch of the M > 16 path is a fixed
 * 8 MiB array in the library's device image (held by every GPU that loads the library until the
 * process exits); the call allocates nothing.  Limit: ub_qmatmul_workspace_bytes(M,N,K,1) <= 8 MiB,
 * i.e. about M*(K+N) <= 4M elements; beyond it the call returns UB_ERR_TOO_LARGE.  The first call on a
 * device looks up the array's address and should come before any stream capture.  Calls share the
 * array: do not let two of them overlap on one GPU.  The array used is the one of the CURRENT device of the
 * calling thread, which must be the device `stream` belongs to (device ordinals up to 63; UB_ERR_INVALID_ARG
 * beyond). */
int ub_qmatmul_q4k_f32_static(void* y, const void* x, const void* wq, int M, int N, int K, int out_dtype, void* stream);

/* ------------------------------------------------------------------ GGUF tensor blobs
 * A GGUF file stores a tensor as (GGML type tag, dims, interleaved block bytes); these entries take the blob's
 * bytes as they lie in the file and dispatch on the tag.  The reference declares the block structs of the family
 * (kernels/quant.cpp:64-185) and ships kernels for Q8_0 and Q4_K; taken here: Q4_0 (2), Q8_0 (8), Q4_K (12),
 * Q5_K (13), Q6_K (14); other tags return UB_ERR_UNSUPPORTED.  x_dtype f32 / bf16; Q4_K with more than 16 tokens
 * and non-bf16 types needs ub_qmatmul_gguf_workspace_bytes of workspace, the other formats none.  Q4_0, Q5_K and
 * Q6_K with rows of whole 2048 values and 16-byte aligned blob and activations run, up to four tokens per pass,
 * kernels that stage whole rows by bulk copies and request their first rows before they wait for the kernel in
 * front of them on the stream: the precondition on the weights and UB_QMATMUL_WEIGHTS_FRESH (ORed into out_dtype)
 * apply to them as to ub_qmatmul_*. */
int ub_gguf_block_values(int ggml_type);
int ub_gguf_block_bytes(int ggml_type);
size_t ub_gguf_tensor_bytes(int ggml_type, size_t numel);
int ub_dequant_gguf(void* out, const void* blob, int ggml_type, size_t numel, int out_dtype, void* stream);
size_t ub_qmatmul_gguf_workspace_bytes(int ggml_type, int M, int N, int K);
int ub_qmatmul_gguf(void* y, const void* x, const void* blob, int ggml_type, int M, int N, int K, int x_dtype, int out_dtype, void* workspace, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------ MoE: reference-named host launchers */
/* src/ffi.rs:205-236, kernels/topk_softmax_host.cpp:178-208 */
void topk_softmax_f32(float* input, float* output, int32_t* index, int32_t num_tokens, int32_t num_experts, int32_t topk, int32_t norm_topk_prob, void* stream);
void topk_softmax_f16(void* input, void* output, int32_t* index, int32_t num_tokens, int32_t num_experts, int32_t topk, int32_t norm_topk_prob, void* stream);
void topk_softmax_bf16(void* input, void* output, int32_t* index, int32_t num_tokens, int32_t num_experts, int32_t topk, int32_t norm_topk_prob, void* stream);

/* src/ffi.rs:149-161, kernels/moe_align_host.cpp:923-935.  sorted_ids holds
 * token_num*topk + num_experts*(block_size-1) ints, experts_ids that count / block_size.
 * real_token_num and expert_map may be NULL.  A bad expert id sets the device error word
 * (ub_device_status) instead of trapping. */
void moe_align_block_size(int32_t* sorted_ids, int32_t* experts_ids, int32_t* num_tokens_post_pad, int32_t* topk_ids, int32_t* real_token_num, int32_t* expert_map, int32_t num_experts, int32_t block_size, int32_t token_num, int32_t topk, void* stream);

/* src/ffi.rs:163-203, kernels/fused_moe_host.cpp:504-536.  Dense expert weights B[E,N,K]. */
void invoke_fused_moe_f16(void* c, void* a, void* b, void* bias, float* topk_weights, int32_t* sorted_ids, int32_t* experts_ids, int32_t* num_tokens_post_pad, int32_t m, int32_t k, int32_t n, int32_t e, int32_t topk_ids_size, int32_t top_k, int32_t block_size, int32_t mul_routed_weight, int32_t bias_flag, void* stream);
void invoke_fused_moe_bf16(void* c, void* a, void* b, void* bias, float* topk_weights, int32_t* sorted_ids, int32_t* experts_ids, int32_t* num_tokens_post_pad, int32_t m, int32_t k, int32_t n, int32_t e, int32_t topk_ids_size, int32_t top_k, int32_t block_size, int32_t mul_routed_weight, int32_t bias_flag, void* stream);

/* src/ffi.rs:44-68, kernels/moe_host.cpp:83-94: y[idx[k],:] += e_out[k,:] * w[idx[k]*topk + top[k]] */
void moe_f16(void* y, void* e_out, float* w, uint32_t* idx, uint32_t* top, int N, int K, int M, int topk, void* stream);
void moe_bf16(void* y, void* e_out, float* w, uint32_t* idx, uint32_t* top, int N, int K, int M, int topk, void* stream);

/* src/ffi.rs:121-147, kernels/moe_host.cpp:278-293: out[b,t,:] = in[b,(M==1?0:t),:] . w[indices[b,t]]^T */
void indexed_moe_f16(void* input, void* w, void* out, uint32_t* idx, int N, int K, int M, int batch, int topk, int num_experts, void* stream);
void indexed_moe_bf16(void* input, void* w, void* out, uint32_t* idx, int N, int K, int M, int batch, int topk, int num_experts, void* stream);

/* src/ffi.rs:70-92, kernels/dequant_host.cpp:298-306: Enflame W4A16 weights -> dense T [K, N].
 * rhs is u8 [K/2, N] (weight_transpose != 0: [N, K/2]), scale / zeros are T [K/group_size, N] (group_size <= 0:
 * one group; zeros may be NULL), out[k,n] = (q - zeros[k/g,n]) * scale[k/g,n].  ASSUMED packing (the reference
 * unpacks inside a vendor routine outside its source tree, so parity with it is unpinned): the byte at
 * packed row r holds reduction index 2r in its low nibble and 2r+1 in its high nibble; K counts dequantised
 * rows.  The same convention serves the name-launched matmul_{f16,bf16}_{4bit,8bit} (module "matmul"). */
void dequant_f16(void* out, uint8_t* rhs, void* scale, void* zeros, int K, int N, int weight_transpose, int group_size, void* stream);
void dequant_bf16(void* out, uint8_t* rhs, void* scale, void* zeros, int K, int N, int weight_transpose, int group_size, void* stream);

/* status-returning twins: src/ffi.rs:671-713, kernels/topsaten_moe_wrapper.cpp:80-213.  Argument order as
 * declared there (the align twin takes num_tokens, topk BEFORE num_experts, block_size, unlike
 * moe_align_block_size above).  token_expert_indices [num_tokens, topk] is written with
 * slot (t, j) -> j * num_tokens + t (vLLM's source-row numbering, which the vendor op mirrors); NULL skips it. */
int topsaten_topk_softmax_f32(float* gating_output, float* topk_weights, int32_t* topk_indices, int32_t* token_expert_indices, int32_t num_tokens, int32_t num_experts, int32_t topk, int32_t norm_topk_prob, void* stream);
int topsaten_moe_align_block_size(int32_t* sorted_token_ids, int32_t* experts_ids, int32_t* num_tokens_post_pad, int32_t* topk_ids, int32_t num_tokens, int32_t topk, int32_t num_experts, int32_t block_size, void* stream);
int topsaten_fused_moe_gemm(void* c_ptr, void* a_ptr, void* b_ptr, float* topk_weights, int32_t* topk_ids, int32_t* sorted_token_ids, int32_t* expert_ids, int32_t* num_tokens_post_padded, int32_t mul_routed_weight, int32_t topk_val, int32_t block_size, int32_t num_tokens, int32_t hidden_dim, int32_t inter_dim, int32_t num_experts, int32_t dtype_code, void* stream);
void topsaten_release_graph_workspace_pool(void* stream);

/* ------------------------------------------------------------------ MoE: new fused entry points */
/* out[t, :D] = silu(in[t, :D]) * in[t, D:2D]  (kernels/topsaten_ops_wrapper.cpp:375-391) */
int ub_silu_and_mul(void* out, const void* in, int rows, int D, int dtype, void* stream);
/* out[t,:] = sum_j in[t,j,:]  (the reference's caller uses topsaten_sum, src/ffi.rs:841-849) */
int ub_topk_sum(void* out, const void* in, int T, int topk, int H, int dtype, void* stream);

/* Grouped GEMM over aligned blocks with Q4_K expert weights Bq[E][N rows of K/256
 * super-blocks]: same contract as invoke_fused_moe_bf16 (kernels/fused_moe_host.cpp:43-250)
 * with A and C bf16.  act_silu_mul != 0 treats B as [gate rows; up rows] (N = 2*D) and
 * writes C[slot, :D] = silu(gate)*up (the SiLU.up step the reference's caller runs between
 * its two GEMMs, kernels/topsaten_ops_wrapper.cpp:375-391), C row stride D. */
int ub_fused_moe_q4k_gemm(void* C, const void* A, const void* Bq, const float* topk_weights, const int32_t* sorted_ids, const int32_t* experts_ids, const int32_t* num_tokens_post_pad, int M, int K, int N, int E, int topk_ids_size, int top_k, int block_size, int mul_routed_weight, int act_silu_mul, void* workspace, size_t ws_bytes, void* stream);

/* indexed_moe on Q4_K experts (decode-time sibling of the grouped GEMM; the reference's dense contract is
 * indexed_moe_{f16,bf16}, src/ffi.rs:121-147, kernels/moe_host.cpp:100-109,278-293):
 * out[b,t,:] = in[b,(M==1?0:t),:] . dequant(wq[indices[b,t]])^T with in [batch,M,K] (M = 1 or topk),
 * wq [num_experts][N rows of K/256 super-blocks], indices [batch,topk], out [batch,topk,N]; dtype bf16 / f16.
 * An index outside [0,num_experts) gives a zero row and UB_ERR_BAD_INDEX in the device error word. */
int ub_indexed_moe_q4k(void* out, const void* in, const void* wq, const uint32_t* indices, int N, int K, int M, int batch, int topk, int num_experts, int dtype, void* stream);

/* Whole expert layer: router logits -> out[T,H].  topk_softmax -> moe_align_block_size ->
 * grouped Q4_K GEMM (w13, SiLU.up) -> grouped Q4_K GEMM (w2, routed weight) -> sum over
 * top-k; the sequence of src/ffi.rs calls the reference's caller issues (five to six
 * launches), on one stream with one caller-provided workspace.  expert_map may be NULL
 * (expert-parallel ranks pass local ids / -1, kernels/moe_align_host.cpp:298,535-543). */
size_t ub_moe_layer_q4k_workspace_bytes(int T, int H, int I, int E, int top_k, int block_size);
int ub_moe_layer_q4k(void* out, const void* hidden, const void* router_logits, const void* w13q, const void* w2q, const int32_t* expert_map, int T, int H, int I, int E, int top_k, int block_size, int norm_topk_prob, void* workspace, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------ one-shot all-reduce over peer memory
 * No reference counterpart as an entry point: it stands where the reference's caller issues ecclAllReduce
 * (src/eccl.rs:209-245) after a row-split matmul, for messages of a few KB where a library all-reduce is
 * latency bound.  Every rank allocates one staging buffer of
 * ub_allreduce_oneshot_staging_bytes(world, max_bytes) with ub_p2p_alloc and makes it reachable from its peers: other processes
 * open it through ub_ipc_get_handle / ub_ipc_open_handle (64-byte handle shipped out of band), threads of one
 * process call ub_enable_peer_access and use the pointer itself.  `staging` is a host array of `world` device
 * pointers in rank order (own buffer at [rank]).  data (bf16, count % 8 == 0, 16-byte aligned, count*2 <=
 * max_bytes) is summed in place over the ranks, in rank order, on every rank.  All ranks must issue the same
 * sequence of calls.  The wait for the peers is bounded (UB_ERR_TIMEOUT in the device error word, see
 * ub_allreduce_oneshot_set_spin_limit). */
int ub_p2p_alloc(size_t bytes, void** out_ptr);   /* zero-filled, mappable by peers (cudaMalloc, synchronous) */
int ub_p2p_free(void* ptr);
int ub_ipc_get_handle(void* dev_ptr, void* handle64);
int ub_ipc_open_handle(const void* handle64, void** out_ptr);
int ub_ipc_close_handle(void* ptr);
int ub_enable_peer_access(int peer_device);
size_t ub_allreduce_oneshot_staging_bytes(int world, size_t max_bytes);
int ub_allreduce_oneshot_bf16(void* data, size_t count, void* const* staging, int rank, int world, size_t max_bytes, void* stream);
/* Polls of a peer's flag (about half a microsecond each; default 2 000 000, i.e. one to two seconds) before a
 * call gives up, records UB_ERR_TIMEOUT in the device error word and returns with an undefined result: read
 * ub_device_status before trusting the output of a run in which a rank may have gone away.  0 restores the
 * default; applies to later launches, process-wide; returns the previous limit.  No reference counterpart
 * (the reference has no bounded waits). */
unsigned ub_allreduce_oneshot_set_spin_limit(unsigned polls);

/* Row-split Q4_K matmul with the all-reduce over the ranks in its epilogue: y[M,N] bf16 = sum over ranks of
 * x_r[M,K] . W_r^T, identical bits on every rank (rank-ordered f32 sum of the bf16 partials, as
 * ub_allreduce_oneshot_bf16 gives).  It stands where the reference's caller runs a matmul and then ecclAllReduce
 * (src/eccl.rs:209-245).  staging / rank / world / max_bytes as above (the same buffers serve both entry points,
 * M*N*2 <= max_bytes, M*N % 8 == 0).  With one token the matmul's own CTAs push their rows to the peers and the
 * last CTA of the grid completes the exchange: ONE launch; other shapes run the matmul and then the one-shot
 * exchange.  world <= 1 is the plain matmul.  No reference counterpart as an entry point. */
int ub_qmatmul_q4k_allreduce_bf16(void* y, const void* x, const void* wq, int M, int N, int K, void* const* staging, int rank, int world, size_t max_bytes, void* stream);
/* The same with the residual add of a decoder layer in the exchange's epilogue: y = residual + sum over the
 * ranks (residual bf16 [M,N], may be NULL, must not alias y; the residual enters the rank-ordered f32 sum first,
 * one rounding).  world <= 1: y = residual + x . W^T, for one token in the matmul's own epilogue. */
int ub_qmatmul_q4k_allreduce_residual_bf16(void* y, const void* x, const void* wq, const void* residual, int M, int N, int K, void* const* staging, int rank, int world, size_t max_bytes, void* stream);

/* ------------------------------------------------------------------ collectives
 * ECCL-shaped surface (src/eccllib.rs:7-169, src/eccl.rs:14-426) forwarding to NCCL over
 * NVLink.  Types and enum values below are ECCL's names with NCCL's layout.  The NCCL
 * library is opened at first use (dlopen "libnccl.so.2"); without it every call returns
 * UB-side failure code ecclSystemError. */
typedef struct ecclComm* ecclComm_t;
typedef struct { char internal[128]; } ecclUniqueId;               /* src/eccl.rs:24-43 */
typedef enum { ecclSuccess = 0, ecclUnhandledCudaError = 1, ecclSystemError = 2, ecclInternalError = 3, ecclInvalidArgument = 4, ecclInvalidUsage = 5, ecclRemoteError = 6, ecclInProgress = 7 } ecclResult_t;
typedef enum { ecclSum = 0, ecclProd = 1, ecclMax = 2, ecclMin = 3, ecclAvg = 4 } ecclRedOp_t;             /* src/eccl.rs:45-61 */
typedef enum { ecclInt8 = 0, ecclUint8 = 1, ecclInt32 = 2, ecclUint32 = 3, ecclInt64 = 4, ecclUint64 = 5, ecclFloat16 = 6, ecclFloat32 = 7, ecclFloat64 = 8, ecclBfloat16 = 9 } ecclDataType_t; /* src/eccl.rs:86-96 */

ecclResult_t ecclGetVersion(int* version);                                                              /* eccllib.rs:15-21 */
ecclResult_t ecclGetUniqueId(ecclUniqueId* id);                                                         /* eccllib.rs:23-29 */
ecclResult_t ecclCommInitRank(ecclComm_t* comm, int nranks, ecclUniqueId id, int rank);                 /* eccllib.rs:31-38 */
ecclResult_t ecclCommInitAll(ecclComm_t* comm, int ndev, const int* devlist);                          /* eccllib.rs:40-46 */
ecclResult_t ecclCommDestroy(ecclComm_t comm);                                                          /* eccllib.rs:7-9  */
ecclResult_t ecclCommAbort(ecclComm_t comm);                                                            /* eccllib.rs:11-13 */
ecclResult_t ecclCommCount(ecclComm_t comm, int* count);                                                /* eccllib.rs:48-52 */
ecclResult_t ecclCommDevice(ecclComm_t comm, int* device);                                              /* eccllib.rs:54-58 */
ecclResult_t ecclCommUserRank(ecclComm_t comm, int* rank);                                              /* eccllib.rs:60-64 */
ecclResult_t ecclReduce(const void* sendbuff, void* recvbuff, size_t count, ecclDataType_t datatype, ecclRedOp_t op, int root, ecclComm_t comm, void* stream);          /* eccllib.rs:67-80 */
ecclResult_t ecclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ecclDataType_t datatype, int root, ecclComm_t comm, void* stream);                      /* eccllib.rs:82-94 */
ecclResult_t ecclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ecclDataType_t datatype, ecclRedOp_t op, ecclComm_t comm, void* stream);                /* eccllib.rs:96-108 */
ecclResult_t ecclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, ecclDataType_t datatype, ecclRedOp_t op, ecclComm_t comm, void* stream);        /* eccllib.rs:110-122 */
ecclResult_t ecclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ecclDataType_t datatype, ecclComm_t comm, void* stream);                            /* eccllib.rs:124-135 */
ecclResult_t ecclSend(const void* sendbuff, size_t count, ecclDataType_t datatype, int peer, ecclComm_t comm, void* stream);                                           /* eccllib.rs:137-148 */
ecclResult_t ecclRecv(void* recvbuff, size_t count, ecclDataType_t datatype, int peer, ecclComm_t comm, void* stream);                                                 /* eccllib.rs:150-161 */
ecclResult_t ecclGroupStart(void);                                                                      /* eccllib.rs:167-169 */
ecclResult_t ecclGroupEnd(void);                                                                        /* eccllib.rs:163-165 */
/* Asynchronous error state of a communicator (ncclCommGetAsyncError): *async_error = ecclSuccess while all is
 * well.  Not part of eccllib.rs; together with ub_stream_query it lets the host bound a collective by a deadline
 * and call ecclCommAbort (what the reference's Drop does, src/eccl.rs:63-70) instead of blocking for ever. */
ecclResult_t ub_eccl_comm_async_error(ecclComm_t comm, ecclResult_t* async_error);

#ifdef __cplusplus
}
#endif
#endif /* UBRIDGE_B200_H_ */
