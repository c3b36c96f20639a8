// Lifecycle, error reporting and memory entry points of libtsb200.
#include <mutex>

#include "common.cuh"

namespace tsb {

static thread_local std::string g_last_error;

void set_last_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
}
const char* last_error() { return g_last_error.c_str(); }

static thread_local bool g_pdl = false;
bool pdl_enabled() { return g_pdl; }
PdlScope::PdlScope(bool on) : prev(g_pdl) { g_pdl = on; }
PdlScope::~PdlScope() { g_pdl = prev; }

static DeviceState g_dev[kMaxDevices];
static std::mutex g_dev_mu;

int use_device(int device, DeviceState** st) {
  TSB_CHECK(device >= 0 && device < kMaxDevices, "device id %d out of range", device);
  DeviceState& d = g_dev[device];
  if (!d.ready) {
    std::lock_guard<std::mutex> lk(g_dev_mu);
    if (!d.ready) {
      int n = 0;
      cudaError_t e = cudaGetDeviceCount(&n);
      if (e != cudaSuccess) {
        cudaGetLastError();
        TSB_FAIL("no CUDA device available: %s (this backend has no CPU fallback)", cudaGetErrorString(e));
      }
      TSB_CHECK(device < n, "device %d does not exist (%d visible)", device, n);
      cudaDeviceProp p;
      TSB_CUDA(cudaGetDeviceProperties(&p, device));
      TSB_CUDA(cudaSetDevice(device));
      d.usable = (p.major == 10);
      d.sm_count = p.multiProcessorCount;
      if (d.usable) TSB_CUDA(cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking));
      d.ready = true;
    }
  }
  TSB_CHECK(d.usable, "device %d is not compute capability 10.x; libtsb200 ships sm_100a code only", device);
  TSB_CUDA(cudaSetDevice(device));
  if (st) *st = &d;
  return 1;
}

void count_launch(int device, long long n) {
  if (device >= 0 && device < kMaxDevices) g_dev[device].launches += n;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) TSB_FAIL("kernel launch failed (%s): %s", what, cudaGetErrorString(e));
  return 1;
}

int check_tensor(const TSB200Tensor* t, const char* name) {
  TSB_CHECK(t != nullptr, "%s: null tensor", name);
  TSB_CHECK(t->data != nullptr, "%s: null data pointer", name);
  TSB_CHECK(t->ndim >= 1 && t->ndim <= 4, "%s: ndim %d not in 1..4", name, t->ndim);
  for (int i = 0; i < t->ndim; ++i) TSB_CHECK(t->sizes[i] >= 0, "%s: negative size", name);
  return 1;
}

}  // namespace tsb

using namespace tsb;

extern "C" {

const char* TSB200_GetLastError(void) { return last_error(); }

int TSB200_DeviceCount(int* count) {
  TSB_CHECK(count, "count is null");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    *count = 0;
    TSB_FAIL("cudaGetDeviceCount: %s", cudaGetErrorString(e));
  }
  *count = n;
  return 1;
}

int TSB200_IsAvailable(int device) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (device < 0 || device >= n) return 0;
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return p.major == 10 ? 1 : 0;
}

const char* TSB200_BuildInfo(void) {
#define TSB_STR2(x) #x
#define TSB_STR(x) TSB_STR2(x)
  return "sm_100a;nvcc " TSB_STR(__CUDACC_VER_MAJOR__) "." TSB_STR(__CUDACC_VER_MINOR__) "." TSB_STR(__CUDACC_VER_BUILD__);
}

int TSB200_LaunchCount(int device, int64_t* launches) {
  TSB_CHECK(launches, "launches is null");
  TSB_CHECK(device >= 0 && device < kMaxDevices, "device id out of range");
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  *launches = st->launches;
  return 1;
}

int TSB200_Alloc(int device, int64_t bytes, void** ptr) {
  TSB_CHECK(ptr, "ptr is null");
  TSB_CHECK(bytes >= 0, "negative size");
  TSB_TRY(use_device(device, nullptr));
  *ptr = nullptr;
  if (bytes == 0) bytes = 256;
  cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    TSB_FAIL("OOM: cudaMalloc of %lld bytes on device %d failed: %s", (long long)bytes, device, cudaGetErrorString(e));
  }
  return 1;
}

int TSB200_Free(int device, void* ptr) {
  if (!ptr) return 1;
  TSB_TRY(use_device(device, nullptr));
  TSB_CUDA(cudaFree(ptr));
  return 1;
}

int TSB200_MemcpyH2D(int device, void* dst, const void* src, int64_t bytes, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  cudaStream_t s = pick_stream(st, stream);
  TSB_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, s));
  TSB_CUDA(cudaStreamSynchronize(s));
  return 1;
}

int TSB200_MemcpyD2H(int device, void* dst, const void* src, int64_t bytes, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  cudaStream_t s = pick_stream(st, stream);
  TSB_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost, s));
  TSB_CUDA(cudaStreamSynchronize(s));
  return 1;
}

int TSB200_MemcpyD2D(int device, void* dst, const void* src, int64_t bytes, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, pick_stream(st, stream)));
  return 1;
}

int TSB200_MemcpyPeer(int dst_device, void* dst, int src_device, const void* src, int64_t bytes) {
  DeviceState* st;
  TSB_TRY(use_device(src_device, nullptr));
  TSB_TRY(use_device(dst_device, &st));
  TSB_CUDA(cudaMemcpyPeerAsync(dst, dst_device, src, src_device, (size_t)bytes, st->stream));
  TSB_CUDA(cudaStreamSynchronize(st->stream));
  return 1;
}

int TSB200_Synchronize(int device, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CUDA(cudaStreamSynchronize(pick_stream(st, stream)));
  return 1;
}

int TSB200_MemoryInfo(int device, int64_t* free_bytes, int64_t* total_bytes) {
  TSB_TRY(use_device(device, nullptr));
  size_t f = 0, t = 0;
  TSB_CUDA(cudaMemGetInfo(&f, &t));
  if (free_bytes) *free_bytes = (int64_t)f;
  if (total_bytes) *total_bytes = (int64_t)t;
  return 1;
}

}  // extern "C"
