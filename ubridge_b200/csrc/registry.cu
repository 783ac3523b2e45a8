// Name -> launcher registry: the shim's counterpart of DeviceExecutor.function_map
// (src/device_executor.rs:57-61, name tables :295-308 and :361-376), GcuDevice::get_or_load_func
// (src/gcu_device.rs:160-183) and GcuFunction::launch (src/gcu_launch.rs:183-328).
//
// A launcher receives the reference's kernel parameter array: params[i] points at argument i, in
// the order of the kernel's signature (kernels/quant.cpp:257-268,341-353,477-488).  The reference
// resolves names through a HashMap<String, ...>; here the table is a fixed array searched once per
// lookup, and callers keep the returned handle, so the per-launch cost is one indirect call.
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace ub {
int dequant_q8_0_split(void* out, const void* in, size_t numel, int dt, cudaStream_t s);
int dequant_q4k_split(void* out, const void* in, size_t numel, int dt, cudaStream_t s);
int quantize_q8_0_split(void* out, const void* x, size_t numel, int dt, cudaStream_t s);
int dense_matmul(int dtype, int quant, const void* a, const void* b, void* out, const void* scales, const void* zeros,
                 int B, int M, int K, int N, int lhs_t, int rhs_t, int bcast_w, int group, cudaStream_t s);
}  // namespace ub

struct ub_function {
  const char* module;
  const char* name;
  int opcode;
  int dtype;
  int (*launch)(const ub_function* self, void** params, cudaStream_t s);
};

namespace {

template <typename V>
V arg(void** params, int i) {
  return *static_cast<V*>(params[i]);
}

// (int8_t* in, T* out, size_t numel)
int launch_dequant_q8_0(const ub_function* f, void** p, cudaStream_t s) {
  return ub::dequant_q8_0_split(arg<void*>(p, 1), arg<void*>(p, 0), arg<size_t>(p, 2), f->dtype, s);
}
int launch_dequant_q4k(const ub_function* f, void** p, cudaStream_t s) {
  return ub::dequant_q4k_split(arg<void*>(p, 1), arg<void*>(p, 0), arg<size_t>(p, 2), f->dtype, s);
}
// (T* in, int8_t* out, size_t in_bytes, size_t out_bytes)
int launch_quantize_q8_0(const ub_function* f, void** p, cudaStream_t s) {
  const size_t esz = f->dtype == UB_DTYPE_F32 ? 4 : 2;
  const size_t numel = arg<size_t>(p, 2) / esz;
  const size_t out_bytes = arg<size_t>(p, 3);
  if (numel % UB_QK8_0 || out_bytes < numel / UB_QK8_0 * UB_Q8_0_BYTES) return ub::fail(UB_ERR_INVALID_ARG);
  return ub::quantize_q8_0_split(arg<void*>(p, 1), arg<void*>(p, 0), numel, f->dtype, s);
}

// module "matmul", 20 parameters (kernels/matmul.cpp:1143-1150,1171-1177):
// (T* a, T* b, T* out, int dtype, int B, int M, int K, int N, int lhs_multicore, int rhs_multicore,
//  int batch_multicore, int lhs_transpose, int rhs_transpose, float alpha, float beta, float addmm_beta,
//  int sip_m, int sip_k, int sip_n, int broadcasted_weight)
int launch_matmul(const ub_function* f, void** p, cudaStream_t s) {
  return ub::dense_matmul(f->dtype, 0, arg<void*>(p, 0), arg<void*>(p, 1), arg<void*>(p, 2), nullptr, nullptr,
                          arg<int>(p, 4), arg<int>(p, 5), arg<int>(p, 6), arg<int>(p, 7), arg<int>(p, 11),
                          arg<int>(p, 12), arg<int>(p, 19), -1, s);
}
// 23 parameters (kernels/matmul.cpp:1186-1194): (T* a, W* b, T* out, T* scales, T* zeros, int dtype, int B, int M,
//  int K, int N, 3 x multicore, lhs_transpose, rhs_transpose, alpha, beta, addmm_beta, sip_m, sip_k, sip_n,
//  int broadcasted_weight, int group_size)
template <int QUANT>
int launch_matmul_quant(const ub_function* f, void** p, cudaStream_t s) {
  return ub::dense_matmul(f->dtype, QUANT, arg<void*>(p, 0), arg<void*>(p, 1), arg<void*>(p, 2), arg<void*>(p, 3),
                          arg<void*>(p, 4), arg<int>(p, 6), arg<int>(p, 7), arg<int>(p, 8), arg<int>(p, 9),
                          arg<int>(p, 13), arg<int>(p, 14), arg<int>(p, 21), arg<int>(p, 22), s);
}

const ub_function kTable[] = {
    {"quant", "dequantize_block_q8_0_f16", UB_OP_DEQUANT_Q8_0, UB_DTYPE_F16, launch_dequant_q8_0},
    {"quant", "dequantize_block_q8_0_bf16", UB_OP_DEQUANT_Q8_0, UB_DTYPE_BF16, launch_dequant_q8_0},
    {"quant", "dequantize_block_q8_0_f32", UB_OP_DEQUANT_Q8_0, UB_DTYPE_F32, launch_dequant_q8_0},
    {"quant", "dequantize_block_q4_k_f16", UB_OP_DEQUANT_Q4K, UB_DTYPE_F16, launch_dequant_q4k},
    {"quant", "dequantize_block_q4_k_bf16", UB_OP_DEQUANT_Q4K, UB_DTYPE_BF16, launch_dequant_q4k},
    {"quant", "dequantize_block_q4_k_f32", UB_OP_DEQUANT_Q4K, UB_DTYPE_F32, launch_dequant_q4k},
    {"quant", "quantize_block_q8_0_f16", UB_OP_QUANTIZE_Q8_0, UB_DTYPE_F16, launch_quantize_q8_0},
    {"quant", "quantize_block_q8_0_bf16", UB_OP_QUANTIZE_Q8_0, UB_DTYPE_BF16, launch_quantize_q8_0},
    {"quant", "quantize_block_q8_0_f32", UB_OP_QUANTIZE_Q8_0, UB_DTYPE_F32, launch_quantize_q8_0},
    // src/device_executor.rs:361-376
    {"matmul", "matmul_f32", UB_OP_MATMUL, UB_DTYPE_F32, launch_matmul},
    {"matmul", "matmul_f16", UB_OP_MATMUL, UB_DTYPE_F16, launch_matmul},
    {"matmul", "matmul_bf16", UB_OP_MATMUL, UB_DTYPE_BF16, launch_matmul},
    {"matmul", "matmul_f16_4bit", UB_OP_MATMUL_W4, UB_DTYPE_F16, launch_matmul_quant<1>},
    {"matmul", "matmul_bf16_4bit", UB_OP_MATMUL_W4, UB_DTYPE_BF16, launch_matmul_quant<1>},
    {"matmul", "matmul_f16_8bit", UB_OP_MATMUL_W8, UB_DTYPE_F16, launch_matmul_quant<2>},
    {"matmul", "matmul_bf16_8bit", UB_OP_MATMUL_W8, UB_DTYPE_BF16, launch_matmul_quant<2>},
};
constexpr int kTableSize = sizeof(kTable) / sizeof(kTable[0]);

thread_local char t_name_buf[128];

}  // namespace

extern "C" {

const ub_function* ub_get_function(const char* module_name, const char* func_name) {
  if (!module_name || !func_name) {
    ub::set_status(UB_ERR_INVALID_ARG);
    return nullptr;
  }
  for (int i = 0; i < kTableSize; i++)
    if (!strcmp(kTable[i].module, module_name) && !strcmp(kTable[i].name, func_name)) {
      ub::set_status(UB_OK);
      return &kTable[i];
    }
  ub::set_status(UB_ERR_UNSUPPORTED);
  return nullptr;
}

int ub_has_function(const char* module_name, const char* func_name) {
  return ub_get_function(module_name, func_name) != nullptr;
}

int ub_function_count(void) { return kTableSize; }

const char* ub_function_name(int index) {
  if (index < 0 || index >= kTableSize) return nullptr;
  snprintf(t_name_buf, sizeof(t_name_buf), "%s::%s", kTable[index].module, kTable[index].name);
  return t_name_buf;
}

int ub_function_opcode(const ub_function* f) { return f ? f->opcode : -1; }

int ub_launch(const ub_function* f, const ub_launch_config* cfg, void** params, void* stream) {
  (void)cfg;  // grid/block/shared-memory hints of the reference's launch config are not needed here
  if (!f) return ub::fail(UB_ERR_UNSUPPORTED);
  if (!params) return ub::fail(UB_ERR_INVALID_ARG);
  return f->launch(f, params, ub::as_stream(stream));
}

}  // extern "C"
