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
