// nccl_dl.cuh -- NCCL resolved at run time (dlopen of libnccl.so.2), so that the single-GPU path
// has no link-time dependency and a host process that already loaded an NCCL keeps using that one.
#pragma once
#include <dlfcn.h>
#include "common.cuh"

namespace gn {

struct NcclUniqueId { char internal[GN_UNIQUE_ID_BYTES]; };

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(void** comm, int nranks, NcclUniqueId id, int rank) = nullptr;
  int (*CommDestroy)(void* comm) = nullptr;
  int (*AllReduce)(const void* send, void* recv, size_t count, int dtype, int op, void* comm, cudaStream_t s) = nullptr;
  int (*AllGather)(const void* send, void* recv, size_t sendcount, int dtype, void* comm, cudaStream_t s) = nullptr;
  int (*CommGetAsyncError)(void* comm, int* err) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};
constexpr int NCCL_FLOAT32 = 7, NCCL_SUM = 0;

inline NcclApi* nccl_api() {
  static NcclApi api; static std::once_flag once; static bool ok = false;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) { api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (api.handle) break; }
    if (!api.handle) return;
    api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
    api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
    api.AllReduce = (decltype(api.AllReduce))dlsym(api.handle, "ncclAllReduce");
    api.AllGather = (decltype(api.AllGather))dlsym(api.handle, "ncclAllGather");
    api.CommGetAsyncError = (decltype(api.CommGetAsyncError))dlsym(api.handle, "ncclCommGetAsyncError");
    api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
    ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather && api.GetErrorString;
  });
  return ok ? &api : nullptr;
}

}  // namespace gn
