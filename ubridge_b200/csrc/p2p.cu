// One-shot all-reduce over peer memory for the small exchanges of the tensor-parallel decode path.
//
// After a row-split GEMV every rank holds a partial [M, hidden] bf16 vector (16 KB at M = 1, hidden = 8192) and
// the reference sums them with ecclAllReduce (src/eccl.rs:209-245).  A library all-reduce costs tens of
// microseconds for such a message; here each rank PUSHES its vector into a slot of every peer's staging
// buffer with plain peer stores over NVLink, raises a flag there, waits for the flags of all ranks in its own
// buffer and adds the slots in rank order, so every rank obtains the same bits.  One kernel, one CTA.
//
// Staging buffer of a rank (allocated by the caller, one per rank, same size everywhere):
//   [0]            u32 epoch of the last completed call (local)
//   [128 ..]       flags[2][world] u32: flags[set][r] = epoch once rank r's vector of that epoch has landed
//   [1024 ..]      slots[2][world][max_bytes]
// Two sets alternate by epoch parity: a rank can start epoch k+2 only after it has seen every peer's flag of
// epoch k+1, which a peer raises only after it has finished reading epoch k.
// The wait on the flags is bounded (a launch parameter, ub_allreduce_oneshot_set_spin_limit; the default is one
// to two seconds of polling); on expiry the kernel records UB_ERR_TIMEOUT in the device error word and still
// leaves: it adds whatever the slots hold, so the result of that call is undefined and the caller must read
// ub_device_status before trusting it.  No multimem, no cluster features: peer loads and stores only.
#include <string.h>

#include <atomic>

#include "common.cuh"

namespace {

using namespace ub;

constexpr uint32_t kDefaultFlagSpinLimit = 2000000;  // polls of ~0.5 us each: one to two seconds
std::atomic<uint32_t> g_flag_spin_limit{kDefaultFlagSpinLimit};
constexpr size_t kFlagsOff = 128, kSlotsOff = 1024;
constexpr int kMaxWorld = 16;

struct PeerTable {
  unsigned char* base[kMaxWorld];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_cg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__global__ void __launch_bounds__(1024, 1)
allreduce_oneshot_bf16_kernel(__nv_bfloat16* __restrict__ data, size_t count, PeerTable peers, int rank, int world,
                              size_t max_bytes, uint32_t spin_limit, int* err_word) {
  __shared__ uint32_t s_epoch;
  unsigned char* const mine = peers.base[rank];
  if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(mine) + 1;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int set = epoch & 1;
  const size_t nvec = count / 8;  // 16-byte pieces; the launcher guarantees count % 8 == 0
  const size_t slot_off = kSlotsOff + (static_cast<size_t>(set) * world + rank) * max_bytes;

  // 1. push this rank's vector into slot `rank` of every rank's staging buffer (its own included)
  for (size_t i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(data)[i];
    for (int p = 0; p < world; p++) reinterpret_cast<uint4*>(peers.base[p] + slot_off)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  // 2. raise this rank's flag everywhere, then wait for everybody's flag here
  if (threadIdx.x < world)
    st_release_sys(reinterpret_cast<uint32_t*>(peers.base[threadIdx.x] + kFlagsOff) + set * world + rank, epoch);
  if (threadIdx.x < world) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(mine + kFlagsOff) + set * world + threadIdx.x;
    bool seen = false;
    for (uint32_t it = 0; it < spin_limit; it++) {
      if (ld_acquire_sys(f) == epoch) {
        seen = true;
        break;
      }
      __nanosleep(100);
    }
    if (!seen) report_device_error(err_word, UB_ERR_TIMEOUT);
  }
  __syncthreads();
  // 3. add the slots in rank order (f32), round once
  const unsigned char* slots = mine + kSlotsOff + static_cast<size_t>(set) * world * max_bytes;
  for (size_t i = threadIdx.x; i < nvec; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; e++) acc[e] = 0.f;
    for (int p = 0; p < world; p++) {
      const uint4 v = ld_cg16(slots + static_cast<size_t>(p) * max_bytes + i * 16);  // written by a peer: not through L1
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; e++) {
        acc[2 * e] += __uint_as_float(w[e] << 16);
        acc[2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      o[e] = *reinterpret_cast<const uint32_t*>(&b);
    }
    reinterpret_cast<uint4*>(data)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  __syncthreads();
  if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(mine) = epoch;
}

}  // namespace

namespace ub {
uint32_t oneshot_spin_limit() { return g_flag_spin_limit.load(std::memory_order_relaxed); }
}  // namespace ub

extern "C" {

// Zero-filled device memory that peers can map: plain cudaMalloc (allocations of the stream-ordered pool behind
// ub_alloc are neither exportable through IPC nor covered by cudaDeviceEnablePeerAccess).  Synchronous.
int ub_p2p_alloc(size_t bytes, void** out_ptr) {
  if (!out_ptr || bytes == 0) return ub::fail(UB_ERR_INVALID_ARG);
  cudaError_t e = cudaMalloc(out_ptr, bytes);
  if (e == cudaSuccess) e = cudaMemset(*out_ptr, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::fail(UB_OK);
}

int ub_p2p_free(void* ptr) {
  if (!ptr) return ub::fail(UB_OK);
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::fail(UB_OK);
}

int ub_ipc_get_handle(void* dev_ptr, void* handle64) {
  if (!dev_ptr || !handle64) return ub::fail(UB_ERR_INVALID_ARG);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaError_t e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), dev_ptr);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::fail(UB_OK);
}

int ub_ipc_open_handle(const void* handle64, void** out_ptr) {
  if (!handle64 || !out_ptr) return ub::fail(UB_ERR_INVALID_ARG);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::fail(UB_OK);
}

int ub_ipc_close_handle(void* ptr) {
  if (!ptr) return ub::fail(UB_OK);
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::fail(UB_OK);
}

int ub_enable_peer_access(int peer_device) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    e = cudaSuccess;
  }
  if (e != cudaSuccess) {
    ub::set_cuda_error(e);
    return ub::fail(UB_ERR_CUDA);
  }
  return ub::fail(UB_OK);
}

size_t ub_allreduce_oneshot_staging_bytes(int world, size_t max_bytes) {
  if (world <= 0 || world > kMaxWorld) return 0;
  return kSlotsOff + 2 * static_cast<size_t>(world) * max_bytes;
}

// Polls of a peer's flag (about half a microsecond each) before a call gives up with UB_ERR_TIMEOUT in the
// device error word; 0 restores the default.  Applies to launches made after the call, process-wide.
// Returns the previous limit.
unsigned ub_allreduce_oneshot_set_spin_limit(unsigned polls) {
  return g_flag_spin_limit.exchange(polls ? polls : kDefaultFlagSpinLimit, std::memory_order_relaxed);
}

int ub_allreduce_oneshot_bf16(void* data, size_t count, void* const* staging, int rank, int world, size_t max_bytes,
                              void* stream) {
  if (!data || !staging || world <= 0 || world > kMaxWorld || rank < 0 || rank >= world)
    return ub::fail(UB_ERR_INVALID_ARG);
  if (count % 8 || (reinterpret_cast<uintptr_t>(data) & 15) || (max_bytes & 15)) return ub::fail(UB_ERR_INVALID_ARG);
  if (count * 2 > max_bytes) return ub::fail(UB_ERR_TOO_LARGE);
  if (count == 0) return ub::fail(UB_OK);
  PeerTable t;
  for (int p = 0; p < kMaxWorld; p++) t.base[p] = p < world ? static_cast<unsigned char*>(staging[p]) : nullptr;
  for (int p = 0; p < world; p++)
    if (!t.base[p] || (reinterpret_cast<uintptr_t>(t.base[p]) & 15)) return ub::fail(UB_ERR_INVALID_ARG);
  const size_t nvec = count / 8;
  const int threads = nvec >= 1024 ? 1024 : static_cast<int>((nvec + 31) / 32 * 32);  // >= 32 >= world
  allreduce_oneshot_bf16_kernel<<<1, threads, 0, ub::as_stream(stream)>>>(
      static_cast<__nv_bfloat16*>(data), count, t, rank, world, max_bytes,
      g_flag_spin_limit.load(std::memory_order_relaxed), ub::device_error_word());
  return ub::check_launch();
}

}  // extern "C"
