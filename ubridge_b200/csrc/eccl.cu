// ECCL-shaped collectives over NCCL: replaces src/eccl.rs:14-426 and src/eccllib.rs:1-169, which wrap
// Enflame's ECCL (an NCCL work-alike reached through tops_backend::driv_eccl::lib()).
//
// Every export forwards 1:1 to the NCCL call of the same shape; ECCL's enums are declared with
// NCCL's numeric values so no translation table is needed.  NCCL is opened lazily with dlopen, so
// the quantized-linear library itself has no link-time dependency on it and single-GPU users never
// load it.  If a process already holds an NCCL (PyTorch's bundled copy, for instance) the same image
// is reused, since dlopen resolves "libnccl.so.2" to the loaded one.  UB_NCCL_PATH overrides the
// library file.
#include <dlfcn.h>
#include <stdlib.h>

#include <mutex>

#include "common.cuh"

namespace {

struct Nccl {
  void* handle = nullptr;
  bool tried = false;
  int (*GetVersion)(int*) = nullptr;
  int (*GetUniqueId)(ecclUniqueId*) = nullptr;
  int (*CommInitRank)(ecclComm_t*, int, ecclUniqueId, int) = nullptr;
  int (*CommInitAll)(ecclComm_t*, int, const int*) = nullptr;
  int (*CommDestroy)(ecclComm_t) = nullptr;
  int (*CommAbort)(ecclComm_t) = nullptr;
  int (*CommCount)(ecclComm_t, int*) = nullptr;
  int (*CommCuDevice)(ecclComm_t, int*) = nullptr;
  int (*CommUserRank)(ecclComm_t, int*) = nullptr;
  int (*Reduce)(const void*, void*, size_t, int, int, int, ecclComm_t, cudaStream_t) = nullptr;
  int (*Bcast)(const void*, void*, size_t, int, int, ecclComm_t, cudaStream_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ecclComm_t, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, ecclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ecclComm_t, cudaStream_t) = nullptr;
  int (*Send)(const void*, size_t, int, int, ecclComm_t, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, ecclComm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*CommGetAsyncError)(ecclComm_t, int*) = nullptr;  // optional
};

Nccl g_nccl;
std::mutex g_nccl_mu;

template <typename F>
bool sym(void* h, const char* name, F& out) {
  out = reinterpret_cast<F>(dlsym(h, name));
  return out != nullptr;
}

Nccl* nccl() {
  std::lock_guard<std::mutex> lk(g_nccl_mu);
  if (!g_nccl.tried) {
    g_nccl.tried = true;
    const char* override_path = getenv("UB_NCCL_PATH");
    void* h = nullptr;
    if (override_path && *override_path) h = dlopen(override_path, RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (h) {
      bool ok = sym(h, "ncclGetVersion", g_nccl.GetVersion) && sym(h, "ncclGetUniqueId", g_nccl.GetUniqueId) &&
                sym(h, "ncclCommInitRank", g_nccl.CommInitRank) && sym(h, "ncclCommInitAll", g_nccl.CommInitAll) &&
                sym(h, "ncclCommDestroy", g_nccl.CommDestroy) && sym(h, "ncclCommAbort", g_nccl.CommAbort) &&
                sym(h, "ncclCommCount", g_nccl.CommCount) && sym(h, "ncclCommCuDevice", g_nccl.CommCuDevice) &&
                sym(h, "ncclCommUserRank", g_nccl.CommUserRank) && sym(h, "ncclReduce", g_nccl.Reduce) &&
                sym(h, "ncclBroadcast", g_nccl.Bcast) && sym(h, "ncclAllReduce", g_nccl.AllReduce) &&
                sym(h, "ncclReduceScatter", g_nccl.ReduceScatter) && sym(h, "ncclAllGather", g_nccl.AllGather) &&
                sym(h, "ncclSend", g_nccl.Send) && sym(h, "ncclRecv", g_nccl.Recv) &&
                sym(h, "ncclGroupStart", g_nccl.GroupStart) && sym(h, "ncclGroupEnd", g_nccl.GroupEnd);
      sym(h, "ncclCommGetAsyncError", g_nccl.CommGetAsyncError);
      if (ok)
        g_nccl.handle = h;
      else
        dlclose(h);
    }
  }
  return g_nccl.handle ? &g_nccl : nullptr;
}

inline ecclResult_t done(int rc) {
  ub::set_status(rc == 0 ? UB_OK : UB_ERR_NCCL);
  return static_cast<ecclResult_t>(rc);
}

#define UB_NCCL_OR_FAIL()              \
  Nccl* n = nccl();                    \
  if (!n) {                            \
    ub::set_status(UB_ERR_NCCL);       \
    return ecclSystemError;            \
  }

}  // namespace

extern "C" {

ecclResult_t ecclGetVersion(int* version) {
  UB_NCCL_OR_FAIL();
  return done(n->GetVersion(version));
}
ecclResult_t ecclGetUniqueId(ecclUniqueId* id) {
  UB_NCCL_OR_FAIL();
  return done(n->GetUniqueId(id));
}
ecclResult_t ecclCommInitRank(ecclComm_t* comm, int nranks, ecclUniqueId id, int rank) {
  UB_NCCL_OR_FAIL();
  return done(n->CommInitRank(comm, nranks, id, rank));
}
ecclResult_t ecclCommInitAll(ecclComm_t* comms, int ndev, const int* devlist) {
  UB_NCCL_OR_FAIL();
  return done(n->CommInitAll(comms, ndev, devlist));
}
ecclResult_t ecclCommDestroy(ecclComm_t comm) {
  UB_NCCL_OR_FAIL();
  return done(n->CommDestroy(comm));
}
ecclResult_t ecclCommAbort(ecclComm_t comm) {
  UB_NCCL_OR_FAIL();
  return done(n->CommAbort(comm));
}
ecclResult_t ecclCommCount(ecclComm_t comm, int* count) {
  UB_NCCL_OR_FAIL();
  return done(n->CommCount(comm, count));
}
ecclResult_t ecclCommDevice(ecclComm_t comm, int* device) {
  UB_NCCL_OR_FAIL();
  return done(n->CommCuDevice(comm, device));
}
ecclResult_t ecclCommUserRank(ecclComm_t comm, int* rank) {
  UB_NCCL_OR_FAIL();
  return done(n->CommUserRank(comm, rank));
}
ecclResult_t ecclReduce(const void* sendbuff, void* recvbuff, size_t count, ecclDataType_t dt, ecclRedOp_t op, int root,
                        ecclComm_t comm, void* stream) {
  UB_NCCL_OR_FAIL();
  return done(n->Reduce(sendbuff, recvbuff, count, dt, op, root, comm, ub::as_stream(stream)));
}
ecclResult_t ecclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ecclDataType_t dt, int root,
                           ecclComm_t comm, void* stream) {
  UB_NCCL_OR_FAIL();
  return done(n->Bcast(sendbuff, recvbuff, count, dt, root, comm, ub::as_stream(stream)));
}
ecclResult_t ecclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ecclDataType_t dt, ecclRedOp_t op,
                           ecclComm_t comm, void* stream) {
  UB_NCCL_OR_FAIL();
  return done(n->AllReduce(sendbuff, recvbuff, count, dt, op, comm, ub::as_stream(stream)));
}
ecclResult_t ecclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, ecclDataType_t dt,
                               ecclRedOp_t op, ecclComm_t comm, void* stream) {
  UB_NCCL_OR_FAIL();
  return done(n->ReduceScatter(sendbuff, recvbuff, recvcount, dt, op, comm, ub::as_stream(stream)));
}
ecclResult_t ecclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ecclDataType_t dt, ecclComm_t comm,
                           void* stream) {
  UB_NCCL_OR_FAIL();
  return done(n->AllGather(sendbuff, recvbuff, sendcount, dt, comm, ub::as_stream(stream)));
}
ecclResult_t ecclSend(const void* sendbuff, size_t count, ecclDataType_t dt, int peer, ecclComm_t comm, void* stream) {
  UB_NCCL_OR_FAIL();
  return done(n->Send(sendbuff, count, dt, peer, comm, ub::as_stream(stream)));
}
ecclResult_t ecclRecv(void* recvbuff, size_t count, ecclDataType_t dt, int peer, ecclComm_t comm, void* stream) {
  UB_NCCL_OR_FAIL();
  return done(n->Recv(recvbuff, count, dt, peer, comm, ub::as_stream(stream)));
}
ecclResult_t ecclGroupStart(void) {
  UB_NCCL_OR_FAIL();
  return done(n->GroupStart());
}
ecclResult_t ecclGroupEnd(void) {
  UB_NCCL_OR_FAIL();
  return done(n->GroupEnd());
}
ecclResult_t ub_eccl_comm_async_error(ecclComm_t comm, ecclResult_t* async_error) {
  UB_NCCL_OR_FAIL();
  if (!async_error || !n->CommGetAsyncError) return done(ecclInvalidArgument);
  int st = 0;
  const int rc = n->CommGetAsyncError(comm, &st);
  *async_error = static_cast<ecclResult_t>(st);
  return done(rc);
}

}  // extern "C"
