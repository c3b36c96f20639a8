// Collectives for tensor parallelism: a thin binding of NCCL (all-reduce over NVLink 5 / NVSwitch), loaded at run time.
//
// The reference has no collective at all: devices exchange whole tensors with cuMemcpyPeer inside one process
// (TensorSharp.CUDA/KernelOps/CopyOps.cs:47-97, Seq2SeqSharp/MultiProcessorNetworkWrapper.cs:81-124).  Here every GPU is
// driven by its own process; the 7B-class model is sharded over heads and FFN columns, and the partial results of the
// attention out-projection and of the FFN down-projection are summed with one all-reduce each.
// libnccl is not linked: it is opened with dlopen (the copy already loaded into the process, e.g. by torch, is
// preferred), so the library itself has no NCCL dependency for single-GPU users.
#include <dlfcn.h>

#include <cstring>

#include "kernels.cuh"

namespace tsb {

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclFloat32 = 7, ncclSum = 0 };

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
};

static NcclApi* nccl() {
  static NcclApi api;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW);
    if (h) {
      api.handle = h;
      api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
      api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
      api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
      api.AllReduce = (decltype(api.AllReduce))dlsym(h, "ncclAllReduce");
      api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
      api.CommGetAsyncError = (decltype(api.CommGetAsyncError))dlsym(h, "ncclCommGetAsyncError");
      if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce) api.handle = nullptr;
    }
  }
  return api.handle ? &api : nullptr;
}

struct Comm {
  ncclComm_t comm = nullptr;
  int rank = 0, nranks = 1, device = 0;
};

int comm_all_reduce_f32(void* c, float* buf, int64_t count, cudaStream_t s) {
  Comm* cm = (Comm*)c;
  NcclApi* api = nccl();
  TSB_CHECK(cm && api, "all_reduce: no communicator");
  const ncclResult_t r = api->AllReduce(buf, buf, (size_t)count, ncclFloat32, ncclSum, cm->comm, s);
  TSB_CHECK(r == 0, "ncclAllReduce failed: %s", api->GetErrorString ? api->GetErrorString(r) : "?");
  return 1;
}
int comm_nranks(void* c) { return c ? ((Comm*)c)->nranks : 1; }
int comm_rank(void* c) { return c ? ((Comm*)c)->rank : 0; }

}  // namespace tsb

using namespace tsb;

extern "C" {

int TSB200_CommGetUniqueId(void* id128) {
  TSB_CHECK(id128, "comm_get_unique_id: null buffer");
  NcclApi* api = nccl();
  TSB_CHECK(api, "comm: libnccl.so.2 could not be opened (%s)", dlerror() ? dlerror() : "not found");
  ncclUniqueId id;
  const ncclResult_t r = api->GetUniqueId(&id);
  TSB_CHECK(r == 0, "ncclGetUniqueId failed: %s", api->GetErrorString ? api->GetErrorString(r) : "?");
  std::memcpy(id128, &id, sizeof(id));
  return 1;
}

int TSB200_CommInitRank(const void* id128, int rank, int nranks, int device, void** comm) {
  TSB_CHECK(id128 && comm, "comm_init_rank: null argument");
  TSB_CHECK(nranks >= 1 && rank >= 0 && rank < nranks, "comm_init_rank: bad rank %d of %d", rank, nranks);
  TSB_TRY(use_device(device, nullptr));
  NcclApi* api = nccl();
  TSB_CHECK(api, "comm: libnccl.so.2 could not be opened");
  ncclUniqueId id;
  std::memcpy(&id, id128, sizeof(id));
  Comm* c = new Comm();
  c->rank = rank; c->nranks = nranks; c->device = device;
  const ncclResult_t r = api->CommInitRank(&c->comm, nranks, id, rank);
  if (r != 0) {
    delete c;
    TSB_FAIL("ncclCommInitRank failed: %s", api->GetErrorString ? api->GetErrorString(r) : "?");
  }
  *comm = c;
  return 1;
}

int TSB200_CommDestroy(void* comm) {
  if (!comm) return 1;
  Comm* c = (Comm*)comm;
  NcclApi* api = nccl();
  if (api && c->comm) {
    cudaSetDevice(c->device);
    api->CommDestroy(c->comm);
  }
  delete c;
  return 1;
}

int TSB200_AllReduceSumF32(void* comm, float* buf, int64_t count, void* stream) {
  Comm* c = (Comm*)comm;
  TSB_CHECK(c && buf && count >= 0, "all_reduce: bad arguments");
  DeviceState* st;
  TSB_TRY(use_device(c->device, &st));
  return comm_all_reduce_f32(comm, buf, count, pick_stream(st, stream));
}

}  // extern "C"
