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

constexpr int kMaxPeers = 8;
constexpr int kPeerFlagBytes = 1024;  // [0..kMaxPeers) arrival flags written by the peers, [64] call counter, [65] CTA counter

struct Comm {
  ncclComm_t comm = nullptr;
  int rank = 0, nranks = 1, device = 0;
  // peer-memory all-reduce (small messages): one region per rank, mapped into every peer
  unsigned char* region = nullptr;        // [flags 1 KB][buffer 0][buffer 1]
  int64_t peer_cap = 0;                   // floats per buffer
  unsigned char* peer_base[kMaxPeers] = {};  // every rank's region as seen from this process (own region included)
  bool peer_open[kMaxPeers] = {};
  bool peers_ready = false;
  long long calls = 0;                    // all-reduces enqueued so far (chooses the buffer a producer writes)
};

// x[i] += sum over ranks (in rank order, so every rank computes bitwise the same) of that rank's partial[i].
// One-shot all-reduce over NVLink for the few KB a decode step exchanges: every rank keeps its partial in its own
// buffer, raises a flag in every peer's memory (release at system scope), waits for the flags of all peers (bounded
// acquire-polls) and reads the partials straight from the peers' buffers.  Two buffers alternate, so a rank that is one
// call ahead never overwrites what a peer is still reading: to get two calls ahead it would need that peer's next flag.
struct PeerArgs {
  unsigned char* base[kMaxPeers];
  int rank, nranks;
  int parity;
  int64_t count, stride;   // floats per call, floats between the two buffers
  float* x;
  int* error_flag;
};
__device__ int g_peer_error;

__global__ void __launch_bounds__(256) peer_reduce_kernel(PeerArgs a) {
  unsigned int* flags = reinterpret_cast<unsigned int*>(a.base[a.rank]);
  const unsigned int seq = *reinterpret_cast<volatile unsigned int*>(flags + 64) + 1u;  // the mark of this call
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < a.nranks && (int)threadIdx.x != a.rank) {
    // this rank's partial was written by an earlier kernel of this stream; order it before the flag for the peer
    __threadfence_system();
    unsigned int* pf = reinterpret_cast<unsigned int*>(a.base[threadIdx.x]) + a.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pf), "r"(seq) : "memory");
  }
  if (threadIdx.x < a.nranks && (int)threadIdx.x != a.rank) {
    const unsigned int* lf = flags + threadIdx.x;
    bool ok = false;
    for (unsigned i = 0; i < (1u << 22); ++i) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(lf) : "memory");
      if ((int)(v - seq) >= 0) {
        ok = true;
        break;
      }
    }
    if (!ok) s_fail = 1;
  }
  __syncthreads();
  if (!s_fail) {
    const size_t off = kPeerFlagBytes + (size_t)a.parity * a.stride * sizeof(float);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.count; i += (int64_t)gridDim.x * blockDim.x) {
      float sum = 0.0f;
      for (int r = 0; r < a.nranks; ++r) sum += __ldcv(reinterpret_cast<const float*>(a.base[r] + off) + i);
      a.x[i] += sum;
    }
  } else if (threadIdx.x == 0) {
    g_peer_error = 1;
    if (a.error_flag) *a.error_flag = 1;
  }
  // the last CTA out advances the call counter
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(flags + 65, 1u);
    if (prev == gridDim.x - 1) {
      flags[65] = 0u;
      *reinterpret_cast<volatile unsigned int*>(flags + 64) = seq;
    }
  }
}

int comm_all_reduce_f32(void* c, float* buf, int64_t count, cudaStream_t s) {
  Comm* cm = (Comm*)c;
  NcclApi* api = nccl();
  TSB_CHECK(cm && api, "all_reduce: no communicator");
  const ncclResult_t r = api->AllReduce(buf, buf, (size_t)count, ncclFloat32, ncclSum, cm->comm, s);
  TSB_CHECK(r == 0, "ncclAllReduce failed: %s", api->GetErrorString ? api->GetErrorString(r) : "?");
  return 1;
}
// The buffer the producer of the next peer all-reduce must write its partial sums to (count floats), or NULL when
// the peer path is not set up / the message does not fit (the caller then uses NCCL).
float* comm_peer_buffer(void* c, int64_t count) {
  Comm* cm = (Comm*)c;
  if (!cm || !cm->peers_ready || count > cm->peer_cap) return nullptr;
  return reinterpret_cast<float*>(cm->region + kPeerFlagBytes + (size_t)(cm->calls & 1) * cm->peer_cap * sizeof(float));
}
// x += sum of all ranks' buffers written through comm_peer_buffer(c, count).
int comm_peer_reduce(void* c, float* x, int64_t count, int* error_flag, int sm_count, cudaStream_t s) {
  Comm* cm = (Comm*)c;
  TSB_CHECK(cm && cm->peers_ready && count <= cm->peer_cap, "peer all-reduce: not set up");
  PeerArgs a{};
  for (int r = 0; r < cm->nranks; ++r) a.base[r] = cm->peer_base[r];
  a.rank = cm->rank; a.nranks = cm->nranks; a.parity = (int)(cm->calls & 1); a.count = count; a.stride = cm->peer_cap; a.x = x; a.error_flag = error_flag;
  cm->calls += 1;
  int grid = (int)((count + 255) / 256);
  if (grid > sm_count) grid = sm_count;
  if (grid < 1) grid = 1;
  peer_reduce_kernel<<<grid, 256, 0, s>>>(a);
  return check_launch("peer_reduce");
}
int comm_peer_take_error() {
  int e = 0;
  if (cudaMemcpyFromSymbol(&e, g_peer_error, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (e) {
    const int z = 0;
    cudaMemcpyToSymbol(g_peer_error, &z, sizeof(int));
  }
  return e;
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

int TSB200_CommPeerExport(void* comm, int64_t max_count, void* handle64) {
  Comm* c = (Comm*)comm;
  TSB_CHECK(c && handle64 && max_count > 0, "comm_peer_export: bad arguments");
  TSB_CHECK(c->nranks <= kMaxPeers, "comm_peer_export: at most %d ranks", kMaxPeers);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  TSB_TRY(use_device(c->device, nullptr));
  if (!c->region) {
    const size_t bytes = kPeerFlagBytes + 2 * (size_t)max_count * sizeof(float);
    TSB_CUDA(cudaMalloc((void**)&c->region, bytes));
    TSB_CUDA(cudaMemset(c->region, 0, bytes));
    c->peer_cap = max_count;
  }
  cudaIpcMemHandle_t h;
  TSB_CUDA(cudaIpcGetMemHandle(&h, c->region));
  std::memcpy(handle64, &h, sizeof(h));
  return 1;
}

int TSB200_CommPeerImport(void* comm, const void* handles, int n) {
  Comm* c = (Comm*)comm;
  TSB_CHECK(c && handles && n == c->nranks && c->region, "comm_peer_import: bad arguments (export first; one 64-byte handle per rank)");
  TSB_TRY(use_device(c->device, nullptr));
  for (int r = 0; r < n; ++r) {
    if (r == c->rank) {
      c->peer_base[r] = c->region;
      continue;
    }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, (const unsigned char*)handles + (size_t)r * 64, sizeof(h));
    void* p = nullptr;
    TSB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    c->peer_base[r] = (unsigned char*)p;
    c->peer_open[r] = true;
  }
  c->peers_ready = true;
  return 1;
}

// First phase of a collective teardown: waits for this device's work, then unmaps the peers' regions.  After EVERY rank
// has returned from this call (a host-side barrier between the ranks) each rank may free its own region with
// TSB200_CommDestroy: freeing exported memory while an importer still has it mapped is undefined, and a peer's kernel
// may still be reading it.
int TSB200_CommPeerClose(void* comm) {
  if (!comm) return 1;
  Comm* c = (Comm*)comm;
  TSB_TRY(use_device(c->device, nullptr));
  cudaDeviceSynchronize();
  c->peers_ready = false;
  for (int r = 0; r < kMaxPeers; ++r)
    if (c->peer_open[r]) {
      cudaIpcCloseMemHandle(c->peer_base[r]);
      c->peer_open[r] = false;
      c->peer_base[r] = nullptr;
    }
  cudaGetLastError();
  return 1;
}

int TSB200_CommDestroy(void* comm) {
  if (!comm) return 1;
  Comm* c = (Comm*)comm;
  cudaSetDevice(c->device);
  for (int r = 0; r < kMaxPeers; ++r)
    if (c->peer_open[r]) cudaIpcCloseMemHandle(c->peer_base[r]);
  if (c->region) cudaFree(c->region);
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
