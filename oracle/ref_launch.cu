// Launcher for the reference's own CUDA kernels (test infrastructure; see build_ref_kernels.py).  The kernel text is
// NOT in this file: it is extracted from the reference checkout at build time into adv_func_kernels_extracted.cu.
// Each entry point starts one kernel with the launch shape the reference's host code uses for it
// (TensorSharp.CUDA/DeviceCode/AdvFuncKernels.cs: LayerNorm :2866-2896, RMSNorm :2911-2953, IndexSelect :3141-3189,
// RoPE :3192-3235, BuildSelfTriMask / BuildTriMask :3075-3140, Softmax :3385-3438): block = min(512, cols) threads,
// grid = min(1024, rows) blocks, block.x floats of dynamic shared memory, the NULL stream.  Returns the CUDA error code.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "adv_func_kernels_extracted.cu"

namespace {
struct Shape {
  dim3 grid, block;
  size_t smem;
};
Shape shape_of(long rows, long cols) {
  Shape s;
  s.block = dim3((unsigned)(cols < 512 ? cols : 512));
  s.grid = dim3((unsigned)(rows < 1024 ? rows : 1024));
  s.smem = s.block.x * sizeof(float);
  return s;
}
int finish() {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  return (int)e;
}
}  // namespace

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API int ref_layernorm(void* out, const void* in, const void* alpha, const void* beta, int rows, int cols, float eps, int half) {
  const Shape s = shape_of(rows, cols);
  if (half) gLNormalizationHalf<<<s.grid, s.block, s.smem>>>((__half*)out, (const __half*)in, (const __half*)alpha, (const __half*)beta, rows, cols, eps);
  else gLNormalization<<<s.grid, s.block, s.smem>>>((float*)out, (const float*)in, (const float*)alpha, (const float*)beta, rows, cols, eps);
  return finish();
}

REF_API int ref_rmsnorm(void* out, const void* in, const void* alpha, const void* beta, int rows, int cols, float eps, int half) {
  const Shape s = shape_of(rows, cols);
  const bool bias = beta != nullptr;
  if (half) RMSNormHalf<<<s.grid, s.block, s.smem>>>((__half*)out, (const __half*)in, (const __half*)alpha, (const __half*)beta, rows, cols, eps, bias);
  else RMSNorm<<<s.grid, s.block, s.smem>>>((float*)out, (const float*)in, (const float*)alpha, (const float*)beta, rows, cols, eps, bias);
  return finish();
}

REF_API int ref_rope(void* out, void* in, int rows, int cols, int seq_len, int row_offset, int half) {
  const Shape s = shape_of(rows, cols);
  if (half) RoPEHalf<<<s.grid, s.block, s.smem>>>((__half*)out, (__half*)in, rows, cols, seq_len, row_offset);
  else RoPE<<<s.grid, s.block, s.smem>>>((float*)out, (float*)in, rows, cols, seq_len, row_offset);
  return finish();
}

REF_API int ref_softmax(void* out, void* in, int rows, int cols, int half) {
  const Shape s = shape_of(rows, cols);
  if (half) gSoftmaxHalf<<<s.grid, s.block, s.smem>>>((__half*)out, (__half*)in, (unsigned)rows, (unsigned)cols);
  else gSoftmax<<<s.grid, s.block, s.smem>>>((float*)out, (float*)in, (unsigned)rows, (unsigned)cols);
  return finish();
}

// indices travel as floats in the reference (one per result row; a negative index leaves the row untouched)
REF_API int ref_indexselect(void* out, void* src, float* indice, int rows, int cols, int is_add, int half) {
  const Shape s = shape_of(rows, cols);
  if (half) IndexSelectHalf<<<s.grid, s.block, s.smem>>>((__half*)out, (__half*)src, indice, rows, cols, is_add);
  else IndexSelect<<<s.grid, s.block, s.smem>>>((float*)out, (float*)src, indice, rows, cols, is_add);
  return finish();
}

REF_API int ref_build_tri_mask(void* out, int rows, int cols, float value, float masked_value, int half) {
  const Shape s = shape_of(rows, cols);
  if (half) BuildTriMaskHalf<<<s.grid, s.block, s.smem>>>((__half*)out, rows, cols, value, masked_value);
  else BuildTriMask<<<s.grid, s.block, s.smem>>>((float*)out, rows, cols, value, masked_value);
  return finish();
}

REF_API int ref_build_self_tri_mask(void* out, float* original_lengths, int rows, int cols, int padded_len, float value, float masked_value, int half) {
  const Shape s = shape_of(rows, cols);
  if (half) BuildSelfTriMaskHalf<<<s.grid, s.block, s.smem>>>((__half*)out, original_lengths, rows, cols, padded_len, value, masked_value);
  else BuildSelfTriMask<<<s.grid, s.block, s.smem>>>((float*)out, original_lengths, rows, cols, padded_len, value, masked_value);
  return finish();
}
