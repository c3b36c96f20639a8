// Unfused element-wise ops behind the OpRegistry names "copy", "fill", "addt", "mult", "mulv", "divv", "relu",
// "SiLU", "LeakyReLU", "float2half", "half2float", "indexselect", "buildtrimask", "buildselftrimask".
// They stand in for the generated pointwise-apply kernels of the reference
// (TensorSharp.CUDA/DeviceCode/ElementwiseKernels.cs:20-128, ElementwiseActKernels.cs:27-59) and exist so that
// unmodified model code runs on this backend; the fused decode path does not use them.
#include "common.cuh"

namespace tsb {

struct Idx4 {
  int64_t s1, s2, s3;          // sizes of dims 1..3 (dim 0 implied by n)
  int64_t r[4], a[4], b[4];    // element strides of result, first and second operand
};

__device__ __forceinline__ void decompose(int64_t i, const Idx4& ix, int64_t& ro, int64_t& ao, int64_t& bo) {
  const int64_t i3 = i % ix.s3;
  int64_t t = i / ix.s3;
  const int64_t i2 = t % ix.s2;
  t /= ix.s2;
  const int64_t i1 = t % ix.s1;
  const int64_t i0 = t / ix.s1;
  ro = i0 * ix.r[0] + i1 * ix.r[1] + i2 * ix.r[2] + i3 * ix.r[3];
  ao = i0 * ix.a[0] + i1 * ix.a[1] + i2 * ix.a[2] + i3 * ix.a[3];
  bo = i0 * ix.b[0] + i1 * ix.b[1] + i2 * ix.b[2] + i3 * ix.b[3];
}

enum UnOp { U_COPY, U_RELU, U_SILU, U_LEAKY, U_MULV, U_DIVV, U_FILL };
enum BinOp { B_ADD, B_MUL };

template <typename TR, typename TA, int OP>
__global__ void unary_kernel(TR* __restrict__ r, const TA* __restrict__ a, int64_t n, Idx4 ix, float scalar) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t ro, ao, bo;
    decompose(i, ix, ro, ao, bo);
    float v = (OP == U_FILL) ? scalar : to_f<TA>(a[ao]);
    if (OP == U_RELU) v = v < 0.0f ? 0.0f : v;
    if (OP == U_SILU) v = v / (1.0f + expf(-v));
    if (OP == U_LEAKY) v = v < 0.0f ? 0.01f * v : v;
    if (OP == U_MULV) v = v * scalar;
    if (OP == U_DIVV) v = v / scalar;
    r[ro] = from_f<TR>(v);
  }
}

template <typename T, int OP>
__global__ void binary_kernel(T* __restrict__ r, const T* __restrict__ a, const T* __restrict__ b, int64_t n, Idx4 ix) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t ro, ao, bo;
    decompose(i, ix, ro, ao, bo);
    const float x = to_f<T>(a[ao]), y = to_f<T>(b[bo]);
    r[ro] = from_f<T>(OP == B_ADD ? x + y : x * y);
  }
}

static int make_idx(const TSB200Tensor* r, const TSB200Tensor* a, const TSB200Tensor* b, Idx4* ix, int64_t* n) {
  View4 vr = view4(r);
  *n = numel(r);
  ix->s1 = vr.size[1];
  ix->s2 = vr.size[2];
  ix->s3 = vr.size[3];
  for (int i = 0; i < 4; ++i) ix->r[i] = vr.stride[i];
  auto fill = [&](const TSB200Tensor* t, int64_t* out, const char* nm) -> int {
    if (!t) {
      for (int i = 0; i < 4; ++i) out[i] = 0;
      return 1;
    }
    TSB_CHECK(numel(t) == *n || true, "%s", nm);
    View4 v = view4(t);
    for (int i = 0; i < 4; ++i) {
      TSB_CHECK(v.size[i] == vr.size[i] || v.size[i] == 1, "%s: size mismatch in dim %d (%lld vs %lld)", nm, i,
                (long long)v.size[i], (long long)vr.size[i]);
      out[i] = (v.size[i] == 1 && vr.size[i] != 1) ? 0 : v.stride[i];
    }
    return 1;
  };
  TSB_TRY(fill(a, ix->a, "operand 1"));
  TSB_TRY(fill(b, ix->b, "operand 2"));
  return 1;
}

static inline int grid_for(int64_t n, DeviceState* st) {
  int64_t g = (n + 255) / 256;
  const int64_t cap = (int64_t)st->sm_count * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

template <int OP>
static int run_unary(int device, const TSB200Tensor* result, const TSB200Tensor* src, float scalar, void* stream,
                     const char* what) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_TRY(check_tensor(result, "result"));
  if (OP != U_FILL) TSB_TRY(check_tensor(src, "src"));
  Idx4 ix;
  int64_t n;
  if (OP != U_FILL && src->ndim != result->ndim) {
    // different rank: allowed when both are contiguous with the same element count (a View in the reference)
    TSB_CHECK(numel(src) == numel(result) && is_contiguous(src) && is_contiguous(result),
              "%s: rank mismatch on non-contiguous tensors", what);
    TSB200Tensor fr = *result, fs = *src;
    fr.ndim = fs.ndim = 1;
    fr.sizes[0] = fs.sizes[0] = numel(result);
    fr.strides[0] = fs.strides[0] = 1;
    TSB_TRY(make_idx(&fr, &fs, nullptr, &ix, &n));
  } else {
    TSB_TRY(make_idx(result, OP == U_FILL ? nullptr : src, nullptr, &ix, &n));
  }
  if (n == 0) return 1;
  cudaStream_t s = pick_stream(st, stream);
  const int g = grid_for(n, st);
  const int rd = result->dtype, sd = (OP == U_FILL) ? rd : src->dtype;
  if (rd == TSB200_F32 && sd == TSB200_F32)
    unary_kernel<float, float, OP><<<g, 256, 0, s>>>((float*)result->data, OP == U_FILL ? nullptr : (const float*)src->data, n, ix, scalar);
  else if (rd == TSB200_F16 && sd == TSB200_F16)
    unary_kernel<__half, __half, OP><<<g, 256, 0, s>>>((__half*)result->data, OP == U_FILL ? nullptr : (const __half*)src->data, n, ix, scalar);
  else if (rd == TSB200_F16 && sd == TSB200_F32 && OP == U_COPY)
    unary_kernel<__half, float, U_COPY><<<g, 256, 0, s>>>((__half*)result->data, (const float*)src->data, n, ix, scalar);
  else if (rd == TSB200_F32 && sd == TSB200_F16 && OP == U_COPY)
    unary_kernel<float, __half, U_COPY><<<g, 256, 0, s>>>((float*)result->data, (const __half*)src->data, n, ix, scalar);
  else
    TSB_FAIL("%s: unsupported dtype combination result=%d src=%d", what, rd, sd);
  count_launch(device);
  return check_launch(what);
}

template <int OP>
static int run_binary(int device, const TSB200Tensor* result, const TSB200Tensor* lhs, const TSB200Tensor* rhs,
                      void* stream, const char* what) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_TRY(check_tensor(result, "result"));
  TSB_TRY(check_tensor(lhs, "lhs"));
  TSB_TRY(check_tensor(rhs, "rhs"));
  TSB_CHECK(result->dtype == lhs->dtype && result->dtype == rhs->dtype, "%s: all tensors must have the same element type", what);
  TSB_CHECK(result->ndim == lhs->ndim && result->ndim == rhs->ndim, "%s: rank mismatch", what);
  Idx4 ix;
  int64_t n;
  TSB_TRY(make_idx(result, lhs, rhs, &ix, &n));
  if (n == 0) return 1;
  cudaStream_t s = pick_stream(st, stream);
  const int g = grid_for(n, st);
  if (result->dtype == TSB200_F32)
    binary_kernel<float, OP><<<g, 256, 0, s>>>((float*)result->data, (const float*)lhs->data, (const float*)rhs->data, n, ix);
  else if (result->dtype == TSB200_F16)
    binary_kernel<__half, OP><<<g, 256, 0, s>>>((__half*)result->data, (const __half*)lhs->data, (const __half*)rhs->data, n, ix);
  else
    TSB_FAIL("%s: unsupported dtype %d", what, result->dtype);
  count_launch(device);
  return check_launch(what);
}

// Row gather by float (or int32) indices; negative index = leave the row untouched
// (TensorSharp.CUDA/DeviceCode/AdvFuncKernels.cs:1214-1243).
template <typename T, typename TI>
__global__ void indexselect_kernel(T* __restrict__ out, const T* __restrict__ src, const TI* __restrict__ idx, int rows,
                                   int cols, int64_t src_rows, int isAdd) {
  for (int j = blockIdx.x; j < rows; j += gridDim.x) {
    const long long s = (long long)idx[j];
    if (s < 0 || s >= src_rows) continue;
    T* o = out + (int64_t)j * cols;
    const T* p = src + (int64_t)s * cols;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) o[i] = isAdd ? from_f<T>(to_f<T>(o[i]) + to_f<T>(p[i])) : p[i];
  }
}

template <typename T>
__global__ void trimask_kernel(T* __restrict__ out, int rows, int cols, float value, float masked) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (int64_t)rows * cols; i += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(i / cols), id = (int)(i % cols);
    out[i] = from_f<T>(id <= j ? value : masked);
  }
}

// out [B, L, L]: value where key <= query and both inside the row's original length, else masked
// (AdvFuncKernels.cs:1383-1412).
template <typename T>
__global__ void selftrimask_kernel(T* __restrict__ out, const float* __restrict__ lens, int B, int L, float value,
                                   float masked) {
  const int64_t n = (int64_t)B * L * L;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int b = (int)(i / ((int64_t)L * L));
    const int q = (int)((i / L) % L), k = (int)(i % L);
    const int len = (int)lens[b];
    out[i] = from_f<T>((k <= q && q < len && k < len) ? value : masked);
  }
}

}  // namespace tsb

using namespace tsb;

extern "C" {

int TSB200_Copy(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream) {
  return run_unary<U_COPY>(device, result, src, 0.0f, stream, "copy");
}
int TSB200_Fill(int device, const TSB200Tensor* result, float value, void* stream) {
  return run_unary<U_FILL>(device, result, nullptr, value, stream, "fill");
}
int TSB200_Add(int device, const TSB200Tensor* result, const TSB200Tensor* lhs, const TSB200Tensor* rhs, void* stream) {
  return run_binary<B_ADD>(device, result, lhs, rhs, stream, "addt");
}
int TSB200_Mul(int device, const TSB200Tensor* result, const TSB200Tensor* lhs, const TSB200Tensor* rhs, void* stream) {
  return run_binary<B_MUL>(device, result, lhs, rhs, stream, "mult");
}
int TSB200_MulScalar(int device, const TSB200Tensor* result, const TSB200Tensor* src, float value, void* stream) {
  return run_unary<U_MULV>(device, result, src, value, stream, "mulv");
}
int TSB200_DivScalar(int device, const TSB200Tensor* result, const TSB200Tensor* src, float value, void* stream) {
  return run_unary<U_DIVV>(device, result, src, value, stream, "divv");
}
int TSB200_Relu(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream) {
  return run_unary<U_RELU>(device, result, src, 0.0f, stream, "relu");
}
int TSB200_SiLU(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream) {
  return run_unary<U_SILU>(device, result, src, 0.0f, stream, "SiLU");
}
int TSB200_LeakyReLU(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream) {
  return run_unary<U_LEAKY>(device, result, src, 0.0f, stream, "LeakyReLU");
}
int TSB200_Float2Half(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream) {
  TSB_CHECK(result && src && result->dtype == TSB200_F16 && src->dtype == TSB200_F32, "float2half: needs F32 -> F16");
  return run_unary<U_COPY>(device, result, src, 0.0f, stream, "float2half");
}
int TSB200_Half2Float(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream) {
  TSB_CHECK(result && src && result->dtype == TSB200_F32 && src->dtype == TSB200_F16, "half2float: needs F16 -> F32");
  return run_unary<U_COPY>(device, result, src, 0.0f, stream, "half2float");
}

int TSB200_IndexSelect(int device, const TSB200Tensor* result, const TSB200Tensor* src, const TSB200Tensor* indices,
                       int isAdd, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_TRY(check_tensor(result, "result"));
  TSB_TRY(check_tensor(src, "src"));
  TSB_TRY(check_tensor(indices, "indices"));
  TSB_CHECK(result->ndim == 2 && src->ndim == 2, "indexselect: result and src must be matrices");
  TSB_CHECK(is_contiguous(result) && is_contiguous(src) && is_contiguous(indices), "indexselect: tensors must be contiguous");
  TSB_CHECK(result->dtype == src->dtype, "indexselect: dtype mismatch");
  TSB_CHECK(result->sizes[1] == src->sizes[1], "indexselect: column count mismatch");
  const int rows = (int)result->sizes[0], cols = (int)result->sizes[1];
  TSB_CHECK(numel(indices) == rows, "indexselect: need one index per result row");
  if (rows == 0) return 1;
  cudaStream_t s = pick_stream(st, stream);
  const int g = rows < st->sm_count * 8 ? rows : st->sm_count * 8;
#define TSB_IS(T, TI) indexselect_kernel<T, TI><<<g, 256, 0, s>>>((T*)result->data, (const T*)src->data, (const TI*)indices->data, rows, cols, src->sizes[0], isAdd)
  if (result->dtype == TSB200_F32 && indices->dtype == TSB200_F32) TSB_IS(float, float);
  else if (result->dtype == TSB200_F16 && indices->dtype == TSB200_F32) TSB_IS(__half, float);
  else if (result->dtype == TSB200_F32 && indices->dtype == TSB200_I32) TSB_IS(float, int);
  else if (result->dtype == TSB200_F16 && indices->dtype == TSB200_I32) TSB_IS(__half, int);
  else TSB_FAIL("indexselect: unsupported dtypes");
#undef TSB_IS
  count_launch(device);
  return check_launch("indexselect");
}

int TSB200_BuildTriMask(int device, const TSB200Tensor* result, float value, float maskedValue, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_TRY(check_tensor(result, "result"));
  TSB_CHECK(is_contiguous(result), "buildtrimask: result must be contiguous");
  const int cols = (int)result->sizes[result->ndim - 1];
  const int rows = (int)(numel(result) / (cols ? cols : 1));
  if (numel(result) == 0) return 1;
  cudaStream_t s = pick_stream(st, stream);
  const int g = grid_for(numel(result), st);
  if (result->dtype == TSB200_F32) trimask_kernel<float><<<g, 256, 0, s>>>((float*)result->data, rows, cols, value, maskedValue);
  else if (result->dtype == TSB200_F16) trimask_kernel<__half><<<g, 256, 0, s>>>((__half*)result->data, rows, cols, value, maskedValue);
  else TSB_FAIL("buildtrimask: unsupported dtype");
  count_launch(device);
  return check_launch("buildtrimask");
}

int TSB200_BuildSelfTriMask(int device, const TSB200Tensor* result, const TSB200Tensor* originalLengths,
                            int paddedSeqLen, float value, float maskedValue, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_TRY(check_tensor(result, "result"));
  TSB_TRY(check_tensor(originalLengths, "originalLengths"));
  TSB_CHECK(is_contiguous(result) && originalLengths->dtype == TSB200_F32, "buildselftrimask: contiguous result and F32 lengths required");
  const int64_t n = numel(result);
  TSB_CHECK(paddedSeqLen > 0 && n % ((int64_t)paddedSeqLen * paddedSeqLen) == 0, "buildselftrimask: result is not [B, L, L]");
  const int B = (int)(n / ((int64_t)paddedSeqLen * paddedSeqLen));
  TSB_CHECK(numel(originalLengths) == B, "buildselftrimask: need one length per sequence");
  cudaStream_t s = pick_stream(st, stream);
  const int g = grid_for(n, st);
  if (result->dtype == TSB200_F32) selftrimask_kernel<float><<<g, 256, 0, s>>>((float*)result->data, (const float*)originalLengths->data, B, paddedSeqLen, value, maskedValue);
  else if (result->dtype == TSB200_F16) selftrimask_kernel<__half><<<g, 256, 0, s>>>((__half*)result->data, (const float*)originalLengths->data, B, paddedSeqLen, value, maskedValue);
  else TSB_FAIL("buildselftrimask: unsupported dtype");
  count_launch(device);
  return check_launch("buildselftrimask");
}

}  // extern "C"
