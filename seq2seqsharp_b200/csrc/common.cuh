// Shared host/device helpers for libtsb200: error convention, device/stream bookkeeping, dtype utilities.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/tsb200.h"

namespace tsb {

// ---- error convention: 1 = success, 0 = failure, message in a thread-local string ----------------
void set_last_error(const char* fmt, ...);
const char* last_error();

#define TSB_FAIL(...)                  \
  do {                                 \
    ::tsb::set_last_error(__VA_ARGS__); \
    return 0;                          \
  } while (0)

#define TSB_CHECK(cond, ...)   \
  do {                         \
    if (!(cond)) TSB_FAIL(__VA_ARGS__); \
  } while (0)

#define TSB_CUDA(expr)                                                                         \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess) {                                                                   \
      if (_e == cudaErrorMemoryAllocation) TSB_FAIL("OOM: %s (%s)", cudaGetErrorString(_e), #expr); \
      TSB_FAIL("CUDA error %d: %s at %s:%d (%s)", (int)_e, cudaGetErrorString(_e), __FILE__, __LINE__, #expr); \
    }                                                                                          \
  } while (0)

#define TSB_TRY(expr)      \
  do {                     \
    if (!(expr)) return 0; \
  } while (0)

// ---- device state -----------------------------------------------------------------------------------
constexpr int kMaxDevices = 16;
struct DeviceState {
  bool ready = false;
  bool usable = false;  // compute capability 10.x
  int sm_count = 0;
  cudaStream_t stream = nullptr;  // library-owned non-blocking stream
  long long launches = 0;
};
// Makes `device` current, lazily creates its state.  Fails when the device is absent or not sm_100.
int use_device(int device, DeviceState** st);
inline cudaStream_t pick_stream(DeviceState* st, void* stream) { return stream ? (cudaStream_t)stream : st->stream; }
void count_launch(int device, long long n = 1);
int check_launch(const char* what);

// ---- programmatic dependent launch ------------------------------------------------------------------
// Kernels of a decode step are chained with programmatic stream serialization: a kernel may become resident while its
// predecessor is still running.  It calls pdl_wait() before it touches anything an earlier kernel wrote (a no-op when
// the launch carried no such attribute) and pdl_trigger() as early as possible so that its own successor can be
// scheduled.  The engine switches the attribute on for the launches it issues (PdlScope); stand-alone ops never use it.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif
bool pdl_enabled();
struct PdlScope {
  bool prev;
  explicit PdlScope(bool on);
  ~PdlScope();
};
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- dtype helpers ----------------------------------------------------------------------------------
inline size_t dtype_size(int dt) {
  switch (dt) {
    case TSB200_F32: return 4;
    case TSB200_F16: return 2;
    case TSB200_F64: return 8;
    case TSB200_I32: return 4;
    case TSB200_U8: return 1;
  }
  return 0;
}

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blockDim.x a multiple of 32 (<= 1024); `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.0f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

// Descriptor helpers
inline int64_t numel(const TSB200Tensor* t) {
  int64_t n = 1;
  for (int i = 0; i < t->ndim; ++i) n *= t->sizes[i];
  return n;
}
inline bool is_contiguous(const TSB200Tensor* t) {
  int64_t expect = 1;
  for (int i = t->ndim - 1; i >= 0; --i) {
    if (t->sizes[i] != 1 && t->strides[i] != expect) return false;
    expect *= t->sizes[i];
  }
  return true;
}
int check_tensor(const TSB200Tensor* t, const char* name);

struct View4 {  // a tensor padded to 4-D (outermost first) for strided kernels
  int64_t size[4];
  int64_t stride[4];
};
inline View4 view4(const TSB200Tensor* t) {
  View4 v;
  const int pad = 4 - t->ndim;
  for (int i = 0; i < 4; ++i) {
    if (i < pad) {
      v.size[i] = 1;
      v.stride[i] = 0;
    } else {
      v.size[i] = t->sizes[i - pad];
      v.stride[i] = t->strides[i - pad];
    }
  }
  return v;
}

}  // namespace tsb
