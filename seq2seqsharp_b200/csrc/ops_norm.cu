// LayerNorm / RMSNorm: the unfused "layernorm"/"rmsnorm" ops and the fused residual+norm used by the decode path.
// One CTA per row; the row is held in shared memory as fp32, statistics are reduced with warp shuffles.
// Numerics follow the reference: LayerNorm sigma = sqrt(eps + mean((x-mu)^2)), y = alpha*((x-mu)/sigma)+beta
// (TensorSharp/TensorApplyCPU.cs:1360-1447; TensorSharp.CUDA/DeviceCode/AdvFuncKernels.cs:613-685);
// RMSNorm rms = sqrt(mean(x^2)+eps), y = gamma*(x/rms)+beta (TensorApplyCPU.cs:1451-1496; AdvFuncKernels.cs:791-845).
#include "kernels.cuh"

namespace tsb {

// TX: type of the row source/destination; TH: type of the normalised output and of gamma/beta/delta.
// FUSED: x is fp32 residual stream, optionally x += delta (written back), h = norm(x).
template <typename TX, typename TH, bool FUSED>
__global__ void __launch_bounds__(1024) norm_kernel(TH* __restrict__ h, TX* __restrict__ x, const TH* __restrict__ delta,
                                                    const TH* __restrict__ gamma, const TH* __restrict__ beta,
                                                    int norm_type, float eps, int rows, int cols, int64_t x_row_stride,
                                                    int64_t h_row_stride) {
  extern __shared__ float row[];
  __shared__ float red[32];
  pdl_trigger();  // chained launches of a decode step: let the next kernel become resident,
  pdl_wait();     // and read the rows only after the previous kernel has completed
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    TX* xr = x + (int64_t)r * x_row_stride;
    TH* hr = h + (int64_t)r * h_row_stride;
    float s = 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
      float v = to_f<TX>(xr[i]);
      if (FUSED && delta) {
        v += to_f<TH>(delta[(int64_t)r * cols + i]);
        xr[i] = from_f<TX>(v);
      }
      row[i] = v;
      s += (norm_type == 0) ? v : v * v;
    }
    s = block_sum(s, red);
    if (norm_type == 0) {
      const float mean = s / cols;
      float sq = 0.0f;
      for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float e = row[i] - mean;
        sq += e * e;
      }
      sq = block_sum(sq, red);
      const float sigma = sqrtf(eps + sq / cols);
      for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float t = to_f<TH>(gamma[i]) * ((row[i] - mean) / sigma);
        if (beta) t += to_f<TH>(beta[i]);
        hr[i] = from_f<TH>(t);
      }
    } else {
      const float rms = sqrtf(s / (float)cols + eps);
      for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float t = to_f<TH>(gamma[i]) * (row[i] / rms);
        if (beta) t += to_f<TH>(beta[i]);
        hr[i] = from_f<TH>(t);
      }
    }
    __syncthreads();
  }
}

static inline int norm_threads(int cols) {
  int t = 128;
  while (t < 1024 && t * 4 < cols) t <<= 1;
  return t;
}

template <typename T>
static int launch_unfused(int device, DeviceState* st, const TSB200Tensor* result, const TSB200Tensor* src,
                          const TSB200Tensor* gamma, const TSB200Tensor* beta, int norm_type, float eps, void* stream) {
  const int cols = (int)src->sizes[src->ndim - 1];
  const int64_t rows = cols ? numel(src) / cols : 0;
  if (rows == 0) return 1;
  TSB_CHECK(numel(gamma) == cols && (!beta || numel(beta) == cols), "norm: gamma/beta must have %d elements", cols);
  TSB_CHECK(is_contiguous(gamma) && (!beta || is_contiguous(beta)), "norm: gamma/beta must be contiguous");
  TSB_CHECK(is_contiguous(result), "norm: result must be contiguous");
  // src: contiguous, or a 2-D view with unit column stride
  int64_t xs = cols;
  if (!is_contiguous(src)) {
    TSB_CHECK(src->ndim == 2 && src->strides[1] == 1, "norm: src must be contiguous or a 2-D row-strided view");
    xs = src->strides[0];
  }
  cudaStream_t s = pick_stream(st, stream);
  const int g = (int)(rows < (int64_t)st->sm_count * 8 ? rows : (int64_t)st->sm_count * 8);
  norm_kernel<T, T, false><<<g, norm_threads(cols), cols * sizeof(float), s>>>(
      (T*)result->data, (T*)src->data, nullptr, (const T*)gamma->data, beta ? (const T*)beta->data : nullptr, norm_type, eps,
      (int)rows, cols, xs, cols);
  count_launch(device);
  return check_launch(norm_type == 0 ? "layernorm" : "rmsnorm");
}

static int norm_entry(int device, const TSB200Tensor* result, const TSB200Tensor* src, const TSB200Tensor* gamma,
                      const TSB200Tensor* beta, int norm_type, float eps, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_TRY(check_tensor(result, "result"));
  TSB_TRY(check_tensor(src, "src"));
  TSB_TRY(check_tensor(gamma, "gamma"));
  if (beta) TSB_TRY(check_tensor(beta, "beta"));
  TSB_CHECK(result->dtype == src->dtype && gamma->dtype == src->dtype && (!beta || beta->dtype == src->dtype),
            "norm: all tensors must have the same element type");
  TSB_CHECK(numel(result) == numel(src), "norm: result/src size mismatch");
  TSB_CHECK(src->sizes[src->ndim - 1] * sizeof(float) <= 48 * 1024, "norm: rows longer than 12288 elements are not supported");
  if (src->dtype == TSB200_F32) return launch_unfused<float>(device, st, result, src, gamma, beta, norm_type, eps, stream);
  if (src->dtype == TSB200_F16) return launch_unfused<__half>(device, st, result, src, gamma, beta, norm_type, eps, stream);
  TSB_FAIL("norm: unsupported dtype %d", src->dtype);
}

// Internal launcher shared with the engine.
int launch_norm_residual(int device, DeviceState* st, int dtype, void* h, float* x, const void* delta, const void* gamma,
                         const void* beta, int norm_type, float eps, int M, int d, cudaStream_t s) {
  if (M == 0) return 1;
  const int g = M < st->sm_count * 8 ? M : st->sm_count * 8;
  const int th = norm_threads(d);
  if (dtype == TSB200_F32)
    TSB_CUDA(launch_k(norm_kernel<float, float, true>, dim3(g), dim3(th), d * sizeof(float), s, (float*)h, x, (const float*)delta,
                      (const float*)gamma, (const float*)beta, norm_type, eps, M, d, (int64_t)d, (int64_t)d));
  else
    TSB_CUDA(launch_k(norm_kernel<float, __half, true>, dim3(g), dim3(th), d * sizeof(float), s, (__half*)h, x, (const __half*)delta,
                      (const __half*)gamma, (const __half*)beta, norm_type, eps, M, d, (int64_t)d, (int64_t)d));
  count_launch(device);
  return check_launch("norm_residual");
}

}  // namespace tsb

using namespace tsb;

extern "C" {

int TSB200_LayerNorm(int device, const TSB200Tensor* result, const TSB200Tensor* src, const TSB200Tensor* gamma,
                     const TSB200Tensor* beta, float eps, void* stream) {
  return norm_entry(device, result, src, gamma, beta, 0, eps, stream);
}
int TSB200_RMSNorm(int device, const TSB200Tensor* result, const TSB200Tensor* src, const TSB200Tensor* gamma,
                   const TSB200Tensor* beta, float eps, void* stream) {
  return norm_entry(device, result, src, gamma, beta, 1, eps, stream);
}

int TSB200_NormResidual(int device, int dtype, void* h, float* x_f32, const void* delta, const void* gamma,
                        const void* beta, int norm_type, float eps, int M, int d, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(h && x_f32 && gamma, "norm_residual: null pointer");
  TSB_CHECK(dtype == TSB200_F32 || dtype == TSB200_F16, "norm_residual: unsupported dtype %d", dtype);
  TSB_CHECK(norm_type == 0 || norm_type == 1, "norm_residual: norm_type must be 0 or 1");
  TSB_CHECK(M >= 0 && d > 0 && (size_t)d * sizeof(float) <= 48 * 1024, "norm_residual: bad shape (d <= 12288)");
  return launch_norm_residual(device, st, dtype, h, x_f32, delta, gamma, beta, norm_type, eps, M, d, pick_stream(st, stream));
}

}  // extern "C"
