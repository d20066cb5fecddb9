// The one collective of the path: the fp32 filter gradients of the batch shards are summed over the
// ranks with ncclAllReduce.  The reference is single-device and has no counterpart.
//
// NCCL is not linked: its entry points are looked up in the process (the copy PyTorch loads, or
// libnccl.so.2 from the loader path), so that the library has no hard dependency on it and a
// single-GPU user never needs it.  One communicator per process and GPU, created from a 128-byte
// unique id that rank 0 makes and hands to the other ranks by whatever channel the host has (a
// key-value store, MPI, torch.distributed).
#include <dlfcn.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace pdnn {
namespace {

struct NcclUniqueId {
  char internal[128];
};
using NcclComm = void*;

struct NcclApi {
  int (*get_unique_id)(NcclUniqueId*) = nullptr;
  int (*comm_init_rank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
  int (*all_reduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*comm_destroy)(NcclComm) = nullptr;
  const char* (*get_error_string)(int) = nullptr;
  bool ok = false;
};

const NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);  // already in the process?
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) return;
    api.get_unique_id = reinterpret_cast<decltype(api.get_unique_id)>(dlsym(h, "ncclGetUniqueId"));
    api.comm_init_rank = reinterpret_cast<decltype(api.comm_init_rank)>(dlsym(h, "ncclCommInitRank"));
    api.all_reduce = reinterpret_cast<decltype(api.all_reduce)>(dlsym(h, "ncclAllReduce"));
    api.comm_destroy = reinterpret_cast<decltype(api.comm_destroy)>(dlsym(h, "ncclCommDestroy"));
    api.get_error_string = reinterpret_cast<decltype(api.get_error_string)>(dlsym(h, "ncclGetErrorString"));
    api.ok = api.get_unique_id && api.comm_init_rank && api.all_reduce && api.comm_destroy;
  });
  return api;
}

int nccl_status(int rc, const char* what) {
  if (rc == 0) return PDNN_OK;
  const NcclApi& api = nccl();
  return fail(PDNN_ALLOCATION_PROBLEM, "%s: %s", what, api.get_error_string ? api.get_error_string(rc) : "NCCL error");
}

constexpr int kNcclFloat32 = 7, kNcclSum = 0;  // ncclDataType_t / ncclRedOp_t values of nccl.h

}  // namespace
}  // namespace pdnn

using namespace pdnn;

extern "C" {

int pdnn_comm_unique_id(void* id128) {
  if (id128 == nullptr) return fail(PDNN_INVALID_PARAMETER, "comm: null id");
  if (!nccl().ok) return fail(PDNN_ALLOCATION_PROBLEM, "comm: libnccl.so.2 is not available in this process");
  NcclUniqueId id;
  const int st = nccl_status(nccl().get_unique_id(&id), "ncclGetUniqueId");
  if (st == PDNN_OK) std::memcpy(id128, id.internal, sizeof(id.internal));
  return st;
}

int pdnn_comm_init(void** comm, const void* id128, int world_size, int rank) {
  if (comm == nullptr || id128 == nullptr || world_size < 1 || rank < 0 || rank >= world_size)
    return fail(PDNN_INVALID_PARAMETER, "comm: bad arguments");
  if (!nccl().ok) return fail(PDNN_ALLOCATION_PROBLEM, "comm: libnccl.so.2 is not available in this process");
  NcclUniqueId id;
  std::memcpy(id.internal, id128, sizeof(id.internal));
  NcclComm c = nullptr;
  const int st = nccl_status(nccl().comm_init_rank(&c, world_size, id, rank), "ncclCommInitRank");
  *comm = st == PDNN_OK ? c : nullptr;
  return st;
}

int pdnn_allreduce_filter_grads(void* comm, float* gradients, size_t count, void* stream) {
  if (count == 0) return PDNN_OK;
  if (comm == nullptr || gradients == nullptr) return fail(PDNN_INVALID_PARAMETER, "all-reduce: null argument");
  if (!nccl().ok) return fail(PDNN_ALLOCATION_PROBLEM, "all-reduce: libnccl.so.2 is not available in this process");
  return nccl_status(nccl().all_reduce(gradients, gradients, count, kNcclFloat32, kNcclSum, comm,
                                       static_cast<cudaStream_t>(stream)),
                     "ncclAllReduce");
}

int pdnn_comm_destroy(void* comm) {
  if (comm == nullptr) return PDNN_OK;
  if (!nccl().ok) return fail(PDNN_ALLOCATION_PROBLEM, "comm: libnccl.so.2 is not available in this process");
  return nccl_status(nccl().comm_destroy(comm), "ncclCommDestroy");
}

}  // extern "C"
