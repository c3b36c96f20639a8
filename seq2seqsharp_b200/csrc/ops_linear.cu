// Linear layers: y = act(bias + x W) (+ residual), the unfused "addmm"/"addmmbatch" ops, and the decode GEMV.
//
// Replaces Affine = bias broadcast copy + cublasGemmEx (Seq2SeqSharp/Tools/ComputeGraphTensor.cs:1848-1880,
// TensorSharp.CUDA/MatrixMul/CudaMatrixMulMM.cs:305-362) and the batched products of attention (:390-504).
// Weights stay in the reference's [in, out] row-major layout; accumulation is always fp32, bias is added first.
//
// gemv_kernel (M <= 8 rows, the decode case) is bandwidth-bound: every weight byte is read exactly once with
// 128-bit loads that are contiguous along `out` across the warp; K is split over the warps of a CTA and over
// CTAs, partial sums meet in a scratch buffer and the last-arriving CTA of a column tile reduces them in a
// fixed order (bitwise deterministic) and applies the fused epilogue.
#include "kernels.cuh"

namespace tsb {


__device__ __forceinline__ float apply_act(int act, float v) {
  switch (act) {
    case TSB200_ACT_RELU: return v < 0.0f ? 0.0f : v;
    case TSB200_ACT_SILU:
    case TSB200_ACT_SWIGLU: return v / (1.0f + expf(-v));
    case TSB200_ACT_LEAKYRELU: return v < 0.0f ? 0.01f * v : v;
    case TSB200_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    default: return v;  // NONE, GLU_NOACT
  }
}

template <typename T>
__device__ __forceinline__ void store_out(const Epilogue& ep, int64_t idx, float v) {
  if (ep.residual) v += ep.residual[idx];
  if (ep.y32) ep.y32[idx] = v;
  else reinterpret_cast<T*>(ep.y)[idx] = from_f<T>(v);
}

template <typename T> struct WVec;
template <> struct WVec<__half> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ void load(const __half* p) { raw = __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void zero() { raw = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void get(float* f) const {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};
template <> struct WVec<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void load(const float* p) { raw = __ldg(reinterpret_cast<const float4*>(p)); }
  __device__ __forceinline__ void zero() { raw = make_float4(0, 0, 0, 0); }
  __device__ __forceinline__ void get(float* f) const {
    f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w;
  }
};

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvUnroll = 4;

template <typename T, int M>
__global__ void __launch_bounds__(kGemvThreads) gemv_kernel(const T* __restrict__ x, const T* __restrict__ W, int K, int N,
                                                            int kchunk, int ksplit, float* partials, unsigned int* counters,
                                                            Epilogue ep, int packedKB) {
  constexpr int VEC = WVec<T>::N;
  constexpr int NT = 32 * VEC;
  extern __shared__ float smem[];  // phase 1: xs[M][kchunk]; phase 2: red[warps][M][NT]
  __shared__ int s_last;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int ct = blockIdx.x, ks = blockIdx.y;
  const int c0 = ct * NT + lane * VEC;
  const bool col_ok = c0 < N;
  const int k0 = ks * kchunk, k1 = min(K, k0 + kchunk);

  for (int i = threadIdx.x; i < M * kchunk; i += kGemvThreads) {
    const int m = i / kchunk, kk = k0 + (i % kchunk);
    smem[i] = (kk < k1) ? to_f<T>(x[(int64_t)m * K + kk]) : 0.0f;
  }
  __syncthreads();

  float acc[M][VEC];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[m][e] = 0.0f;

  // row-major [K,N] (packedKB == 0) or the engine's tiled layout [ct][kb][32][NT] (packedKB = tiles along K)
  const T* wp = packedKB ? W + (int64_t)ct * packedKB * (32 * NT) + lane * VEC : W + c0;
  for (int k = k0 + w; k < k1; k += kGemvWarps * kGemvUnroll) {
    WVec<T> wv[kGemvUnroll];
#pragma unroll
    for (int u = 0; u < kGemvUnroll; ++u) {
      const int kk = k + u * kGemvWarps;
      if (kk < k1 && (col_ok || packedKB))
        wv[u].load(packedKB ? wp + (int64_t)(kk >> 5) * (32 * NT) + packed_tile_off<T>(kk & 31, lane * VEC) - lane * VEC : wp + (int64_t)kk * N);
      else wv[u].zero();
    }
#pragma unroll
    for (int u = 0; u < kGemvUnroll; ++u) {
      const int kk = k + u * kGemvWarps;
      float wf[VEC];
      wv[u].get(wf);
      const int ki = min(kk, k1 - 1) - k0;
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float xv = smem[m * kchunk + ki];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[m][e] = fmaf(xv, wf[e], acc[m][e]);
      }
    }
  }
  __syncthreads();  // everyone is done with xs
  float* red = smem;
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int e = 0; e < VEC; ++e) red[((w * M) + m) * NT + lane * VEC + e] = acc[m][e];
  __syncthreads();
  // fin[m][c] = sum over warps, kept in red[0][..]
  for (int i = threadIdx.x; i < M * NT; i += kGemvThreads) {
    float v = 0.0f;
#pragma unroll
    for (int ww = 0; ww < kGemvWarps; ++ww) v += red[ww * M * NT + i];
    red[i] = v;  // slot i of warp 0's region is only ever read by this thread
  }
  __syncthreads();
  if (ksplit > 1) {
    float* mine = partials + ((int64_t)ct * ksplit + ks) * (M * NT);
    for (int i = threadIdx.x; i < M * NT; i += kGemvThreads) mine[i] = red[i];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int prev = atomicAdd(&counters[ct], 1u);
      s_last = (prev == (unsigned int)(ksplit - 1));
      if (s_last) counters[ct] = 0u;  // self-reset for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* all = partials + (int64_t)ct * ksplit * (M * NT);
    for (int i = threadIdx.x; i < M * NT; i += kGemvThreads) {
      float v = 0.0f;
      for (int s = 0; s < ksplit; ++s) v += __ldcg(all + (int64_t)s * (M * NT) + i);
      red[i] = v;
    }
    __syncthreads();
  }
  // epilogue: bias first, activation, optional gate product, residual
  const T* bias = reinterpret_cast<const T*>(ep.bias);
  if (!ep.glu) {
    for (int i = threadIdx.x; i < M * NT; i += kGemvThreads) {
      const int m = i / NT, c = ct * NT + (i % NT);
      if (c < N) {
        float v = red[i] + (bias ? to_f<T>(bias[c]) : 0.0f);
        v = apply_act(ep.act, v);
        store_out<T>(ep, (int64_t)m * N + c, v);
      }
    }
  } else {
    const int No = N / 2;
    for (int i = threadIdx.x; i < M * (NT / 2); i += kGemvThreads) {
      const int m = i / (NT / 2), j = i % (NT / 2);
      const int c = ct * NT + 2 * j;
      if (c + 1 < N) {
        const float a = red[m * NT + 2 * j] + (bias ? to_f<T>(bias[c]) : 0.0f);
        const float g = red[m * NT + 2 * j + 1] + (bias ? to_f<T>(bias[c + 1]) : 0.0f);
        store_out<T>(ep, (int64_t)m * No + (c >> 1), apply_act(ep.act, a) * g);
      }
    }
  }
}

// ---- generic strided GEMM (any M, any strides, batched): correctness path for views and for prefill until the
// tensor-core kernel takes the contiguous fp16 case.  64x64x16 tiles, 4x4 per thread, fp32 accumulate.
struct GemmArgs {
  const void* A; const void* B; const void* src; void* C;
  int M, N, K, batch;
  int64_t a_m, a_k, a_b;      // element strides of A over m, k, batch
  int64_t b_k, b_n, b_b;
  int64_t s_m, s_n, s_b;      // src (beta term / bias broadcast)
  int64_t c_m, c_n, c_b;
  float alpha, beta;
  int b_packedKB, b_NT;       // B in the engine's tiled layout when b_packedKB > 0
};

template <typename T, bool EPI>
__global__ void __launch_bounds__(256) gemm_generic_kernel(GemmArgs g, Epilogue ep) {
  __shared__ float As[16][64 + 4];
  __shared__ float Bs[16][64 + 4];
  const int bz = blockIdx.z;
  const T* A = reinterpret_cast<const T*>(g.A) + bz * g.a_b;
  const T* B = reinterpret_cast<const T*>(g.B) + bz * g.b_b;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < g.K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int mm = i / 16, kk = i % 16;
      const int m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < g.M && k < g.K) ? to_f<T>(A[m * g.a_m + k * g.a_k]) : 0.0f;
    }
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int kk = i / 64, nn = i % 64;
      const int k = k0 + kk, n = n0 + nn;
      float bv = 0.0f;
      if (k < g.K && n < g.N)
        bv = g.b_packedKB ? to_f<T>(B[((int64_t)(n / g.b_NT) * g.b_packedKB + k / 32) * (32 * g.b_NT) + packed_tile_off<T>(k % 32, n % g.b_NT)])
                          : to_f<T>(B[k * g.b_k + n * g.b_n]);
      Bs[kk][nn] = bv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  if (!EPI) {
    const T* S = g.src ? reinterpret_cast<const T*>(g.src) + bz * g.s_b : nullptr;
    T* C = reinterpret_cast<T*>(g.C) + bz * g.c_b;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
        if (m < g.M && n < g.N) {
          float v = g.alpha * acc[i][j];
          if (g.beta != 0.0f && S) v += g.beta * to_f<T>(S[m * g.s_m + n * g.s_n]);
          C[m * g.c_m + n * g.c_n] = from_f<T>(v);
        }
      }
  } else {
    const T* bias = reinterpret_cast<const T*>(ep.bias);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = m0 + ty * 4 + i;
      if (m >= g.M) continue;
      if (!ep.glu) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + tx * 4 + j;
          if (n < g.N) {
            float v = acc[i][j] + (bias ? to_f<T>(bias[n]) : 0.0f);
            store_out<T>(ep, (int64_t)m * g.N + n, apply_act(ep.act, v));
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
          const int n = n0 + tx * 4 + j;
          if (n + 1 < g.N) {
            const float a = acc[i][j] + (bias ? to_f<T>(bias[n]) : 0.0f);
            const float gg = acc[i][j + 1] + (bias ? to_f<T>(bias[n + 1]) : 0.0f);
            store_out<T>(ep, (int64_t)m * (g.N / 2) + (n >> 1), apply_act(ep.act, a) * gg);
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ host side
struct GemvPlan {
  int ctiles, ksplit, kchunk;
  size_t smem;
};

template <typename T>
static GemvPlan plan_gemv(DeviceState* st, int M, int K, int N) {
  constexpr int NT = 32 * WVec<T>::N;
  GemvPlan p;
  p.ctiles = (N + NT - 1) / NT;
  const int target = st->sm_count * 4;
  int ks = (target + p.ctiles - 1) / p.ctiles;
  int kchunk = (K + ks - 1) / ks;
  kchunk = (kchunk + 31) & ~31;
  if (kchunk < 64) kchunk = 64;
  if (kchunk > 2048) kchunk = 2048;
  if (kchunk > ((K + 31) & ~31)) kchunk = (K + 31) & ~31;
  p.kchunk = kchunk;
  p.ksplit = (K + kchunk - 1) / kchunk;
  const size_t a = (size_t)M * kchunk, b = (size_t)kGemvWarps * M * NT;
  p.smem = (a > b ? a : b) * sizeof(float);
  return p;
}

int64_t linear_workspace_bytes(int M, int K, int N) {
  (void)K;
  // partials for up to sm*4 + ctiles CTAs of M x NT floats, plus one counter per column tile (generous bound)
  const int Mb = M > 8 ? 8 : (M < 1 ? 1 : M);
  const int64_t ctiles = (N + 127) / 128;
  const int64_t ctas = 148 * 8 + ctiles * 2;
  return ctas * Mb * 256 * 4 + kWsCounterBytes + 1024;
}

template <typename T, int M>
static int gemv_attr(int) {
  TSB_CUDA(cudaFuncSetAttribute(gemv_kernel<T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 8 * 256 * 4));
  return 1;
}
// Opt every GEMV instantiation into 64 KB of dynamic shared memory, once per device (never during graph capture).
int init_linear_attrs(int device) {
  static bool done[kMaxDevices] = {};
  if (done[device]) return 1;
#define TSB_ATTR(M) TSB_TRY((gemv_attr<float, M>(device))); TSB_TRY((gemv_attr<__half, M>(device)))
  TSB_ATTR(1); TSB_ATTR(2); TSB_ATTR(3); TSB_ATTR(4); TSB_ATTR(5); TSB_ATTR(6); TSB_ATTR(7); TSB_ATTR(8);
#undef TSB_ATTR
  done[device] = true;
  return 1;
}

template <typename T, int M>
static int launch_gemv_m(int device, DeviceState* st, const T* x, const T* W, int K, int N, const Epilogue& ep, void* ws,
                         int64_t ws_bytes, cudaStream_t s, int packedKB) {
  constexpr int NT = 32 * WVec<T>::N;
  GemvPlan p = plan_gemv<T>(st, M, K, N);
  const int64_t cnt_bytes = kWsCounterBytes;
  const int64_t need = cnt_bytes + (int64_t)p.ctiles * p.ksplit * M * NT * 4;
  if (p.ksplit > 1 && (!ws || ws_bytes < need)) {
    // no scratch: fall back to one CTA per column tile over the whole K range (chunked through shared memory
    // is not possible here, so restrict to what fits)
    TSB_FAIL("linear: workspace too small for split-K GEMV (%lld < %lld bytes)", (long long)ws_bytes, (long long)need);
  }
  TSB_TRY(init_linear_attrs(device));
  unsigned int* counters = reinterpret_cast<unsigned int*>(ws);
  float* partials = ws ? reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + cnt_bytes) : nullptr;
  dim3 grid(p.ctiles, p.ksplit);
  gemv_kernel<T, M><<<grid, kGemvThreads, p.smem, s>>>(x, W, K, N, p.kchunk, p.ksplit, partials, counters, ep, packedKB);
  count_launch(device);
  return check_launch("gemv");
}

template <typename T>
static int launch_generic(int device, const GemmArgs& g, const Epilogue* ep, cudaStream_t s) {
  if (g.M == 0 || g.N == 0 || g.batch == 0) return 1;
  dim3 grid((g.N + 63) / 64, (g.M + 63) / 64, g.batch);
  TSB_CHECK(grid.y <= 65535 && grid.z <= 65535, "gemm: grid too large");
  if (ep) gemm_generic_kernel<T, true><<<grid, 256, 0, s>>>(g, *ep);
  else gemm_generic_kernel<T, false><<<grid, 256, 0, s>>>(g, Epilogue{});
  count_launch(device);
  return check_launch("gemm_generic");
}

// y = epilogue(x[M,K] W[K,N]); x, W contiguous.  counters in `ws` must be zero on first use (they self-reset).
int launch_linear(int device, DeviceState* st, int dtype, const void* x, const void* W, int M, int K, int N,
                  const Epilogue& ep, void* ws, int64_t ws_bytes, cudaStream_t s, bool packed) {
  if (M == 0) return 1;
  const int vec = dtype == TSB200_F16 ? 8 : 4;
  const int packedKB = packed ? (K + 31) / 32 : 0;
  if (packed && dtype == TSB200_F16 && M > 16 && M <= 64) {
    // 17..64 rows: the weights stream once through tcgen05 with the activation rows as the N dimension
    const int r = launch_gemm_stream_tc(device, st, x, W, M, K, N, ep, nullptr, true, ws, ws_bytes, s);
    if (r != 2) return r;
  }
  if (packed && dtype == TSB200_F16 && M >= 1 && M <= 64) {
    // decode batches: weights streamed once through a ring, mma.sync consumers (measured: for 33..64 rows and wide
    // outputs the split-K tcgen05 kernel below is faster, its partial sums being a smaller share of the traffic)
    const int r = launch_gemm_stream_mma(device, st, x, W, M, K, N, ep, nullptr, true, ws, ws_bytes, s);
    if (r != 2) return r;
  }
  if (packed && dtype == TSB200_F16 && M > 16) {
    const int r = launch_gemm_tc(device, st, x, W, M, K, N, ep, nullptr, ws, ws_bytes, s);
    if (r != 2) return r;
  }
  const bool gemv_ok = (packed || N % vec == 0) && (((uintptr_t)W % 16) == 0) && M <= 16;
  if (gemv_ok) {
    for (int m0 = 0; m0 < M; m0 += 8) {
      const int mb = M - m0 < 8 ? M - m0 : 8;
      Epilogue e2 = ep;
      const int No = ep.glu ? N / 2 : N;
      if (e2.residual) e2.residual += (int64_t)m0 * No;
      if (e2.y32) e2.y32 += (int64_t)m0 * No;
      if (e2.y) e2.y = (char*)e2.y + (int64_t)m0 * No * (dtype == TSB200_F16 ? 2 : 4);
#define TSB_GEMV(T, MM) launch_gemv_m<T, MM>(device, st, (const T*)x + (int64_t)m0 * K, (const T*)W, K, N, e2, ws, ws_bytes, s, packedKB)
#define TSB_GEMV_SW(T)                                  \
  switch (mb) {                                         \
    case 1: TSB_TRY(TSB_GEMV(T, 1)); break;             \
    case 2: TSB_TRY(TSB_GEMV(T, 2)); break;             \
    case 3: TSB_TRY(TSB_GEMV(T, 3)); break;             \
    case 4: TSB_TRY(TSB_GEMV(T, 4)); break;             \
    case 5: TSB_TRY(TSB_GEMV(T, 5)); break;             \
    case 6: TSB_TRY(TSB_GEMV(T, 6)); break;             \
    case 7: TSB_TRY(TSB_GEMV(T, 7)); break;             \
    default: TSB_TRY(TSB_GEMV(T, 8)); break;            \
  }
      if (dtype == TSB200_F16) { TSB_GEMV_SW(__half) } else { TSB_GEMV_SW(float) }
#undef TSB_GEMV_SW
#undef TSB_GEMV
    }
    return 1;
  }
  GemmArgs g{};
  g.A = x; g.B = W; g.src = nullptr; g.C = nullptr;
  g.M = M; g.N = N; g.K = K; g.batch = 1;
  g.a_m = K; g.a_k = 1; g.b_k = N; g.b_n = 1;
  g.alpha = 1.0f; g.beta = 0.0f;
  g.b_packedKB = packedKB;
  g.b_NT = 32 * vec;
  if (dtype == TSB200_F16) return launch_generic<__half>(device, g, &ep, s);
  return launch_generic<float>(device, g, &ep, s);
}

}  // namespace tsb

using namespace tsb;

static int addmm_common(int device, const TSB200Tensor* result, float beta, const TSB200Tensor* src, float alpha,
                        const TSB200Tensor* m1, const TSB200Tensor* m2, void* stream, int nd, const char* what) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_TRY(check_tensor(result, "result"));
  TSB_TRY(check_tensor(src, "src"));
  TSB_TRY(check_tensor(m1, "m1"));
  TSB_TRY(check_tensor(m2, "m2"));
  TSB_CHECK(result->ndim == nd && src->ndim == nd && m1->ndim == nd && m2->ndim == nd, "%s: all tensors must be %d-D", what, nd);
  TSB_CHECK(src->dtype == m1->dtype && src->dtype == m2->dtype && result->dtype == src->dtype,
            "%s: all tensors must have the same element type", what);
  const int o = nd - 2;
  GemmArgs g{};
  g.batch = nd == 3 ? (int)result->sizes[0] : 1;
  g.M = (int)m1->sizes[o];
  g.K = (int)m1->sizes[o + 1];
  g.N = (int)m2->sizes[o + 1];
  TSB_CHECK(m2->sizes[o] == g.K && result->sizes[o] == g.M && result->sizes[o + 1] == g.N && src->sizes[o] == g.M &&
                src->sizes[o + 1] == g.N, "%s: size mismatch", what);
  if (nd == 3)
    TSB_CHECK(m1->sizes[0] == g.batch && m2->sizes[0] == g.batch && src->sizes[0] == g.batch, "%s: batch size mismatch", what);
  g.A = m1->data; g.B = m2->data; g.src = src->data; g.C = result->data;
  g.a_m = m1->strides[o]; g.a_k = m1->strides[o + 1]; g.a_b = nd == 3 ? m1->strides[0] : 0;
  g.b_k = m2->strides[o]; g.b_n = m2->strides[o + 1]; g.b_b = nd == 3 ? m2->strides[0] : 0;
  g.s_m = src->strides[o]; g.s_n = src->strides[o + 1]; g.s_b = nd == 3 ? src->strides[0] : 0;
  g.c_m = result->strides[o]; g.c_n = result->strides[o + 1]; g.c_b = nd == 3 ? result->strides[0] : 0;
  g.alpha = alpha;
  g.beta = beta;
  cudaStream_t s = pick_stream(st, stream);
  if (src->dtype == TSB200_F32) return launch_generic<float>(device, g, nullptr, s);
  if (src->dtype == TSB200_F16) return launch_generic<__half>(device, g, nullptr, s);
  TSB_FAIL("%s: unsupported dtype %d", what, src->dtype);
}

extern "C" {

int TSB200_Addmm(int device, const TSB200Tensor* result, float beta, const TSB200Tensor* src, float alpha,
                 const TSB200Tensor* m1, const TSB200Tensor* m2, void* stream) {
  return addmm_common(device, result, beta, src, alpha, m1, m2, stream, 2, "addmm");
}
int TSB200_AddmmBatch(int device, const TSB200Tensor* result, float beta, const TSB200Tensor* src, float alpha,
                      const TSB200Tensor* m1, const TSB200Tensor* m2, void* stream) {
  return addmm_common(device, result, beta, src, alpha, m1, m2, stream, 3, "addmmbatch");
}

int64_t TSB200_LinearWorkspaceBytes(int M, int K, int N) { return linear_workspace_bytes(M, K, N); }

int TSB200_LinearBiasAct(int device, int dtype, void* y, float* y_f32, const void* x, const void* W, const void* bias,
                         const float* residual_f32, int M, int K, int N, int act, void* workspace, int64_t workspace_bytes,
                         void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(dtype == TSB200_F32 || dtype == TSB200_F16, "linear: unsupported dtype %d", dtype);
  TSB_CHECK(x && W && (y || y_f32), "linear: null pointer");
  TSB_CHECK(M >= 0 && K > 0 && N > 0, "linear: bad shape");
  Epilogue ep{};
  ep.bias = bias;
  ep.residual = residual_f32;
  ep.y = y_f32 ? nullptr : y;
  ep.y32 = y_f32;
  ep.act = act;
  ep.glu = (act == TSB200_ACT_GLU_NOACT || act == TSB200_ACT_SWIGLU) ? 1 : 0;
  TSB_CHECK(!ep.glu || N % 2 == 0, "linear: gated activations need an even (interleaved) column count");
  cudaStream_t s = pick_stream(st, stream);
  if (workspace && workspace_bytes > 0) {
    // the split-K counters live at the start of the workspace and must start at zero
    const int64_t z = workspace_bytes < 65536 ? workspace_bytes : 65536;
    TSB_CUDA(cudaMemsetAsync(workspace, 0, (size_t)z, s));
  }
  return launch_linear(device, st, dtype, x, W, M, K, N, ep, workspace, workspace_bytes, s, false);
}

}  // extern "C"
