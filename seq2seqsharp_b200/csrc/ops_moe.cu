// Mixture-of-experts feed-forward of the GPT decoder at inference (Seq2SeqSharp/Layers/MoEFeedForward.cs:72-160): after
// the layer's own LayerNorm, a router picks experts_per_token experts per token (softmax of an affine map, TopK), each
// chosen expert runs x W1_e -> activation -> W2_e (no biases), the results are weighted by the token's router
// probabilities, summed per token in ascending expert order and added to the residual stream.
//
// Three kernels, all reading the experts in place from [E, d, 4d] / [E, 4d, d] row-major tensors (which expert a token
// uses is only known on the device, so the weight pointer is formed there):
//   moe_route_kernel  one CTA per token: router logits in fp32, the reference's constant -65000 "mask" added in fp32
//                     (which rounds the logits to multiples of 2^-7: part of the reference's behaviour), softmax, TopK with
//                     the reference's tie rule (TensorApplyCPU.cs:1097-1146: a value equal to the current k-th one
//                     replaces it), picks sorted by expert index;
//   moe_up_kernel     hidden[token, pick, :] = act(x[token] W1[expert]): one CTA per (token, pick, 256 columns), the input
//                     row in shared memory, every thread one column, coalesced over columns;
//   moe_down_kernel   x32[token] += sum over picks (ascending expert) of score * (hidden[token, pick] W2[expert]).
// These are plain HBM-bound GEMVs; a mixture layer's decode step reads experts_per_token / E of its weights.
#include "kernels.cuh"

namespace tsb {

TSB_CHECKED_WORD(moe)
#ifndef TSB200_CHECKED
int chk_take_moe() { return 0; }
#endif

constexpr int kMoeMaxExperts = 256;
constexpr int kMoeMaxPicks = 8;

template <typename T>
__global__ void __launch_bounds__(256) moe_route_kernel(int* picks, float* scores, const T* h, const T* Wr, const T* br, int d, int E, int k) {
  __shared__ float s_r[kMoeMaxExperts];
  __shared__ float s_part[8][kMoeMaxExperts / 8 > 32 ? kMoeMaxExperts / 8 : 32];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const T* x = h + (size_t)row * d;
  // router logits: thread t sums over k = t, t + 256, ... for every expert; the partial sums meet in shared memory
  for (int e0 = 0; e0 < E; e0 += 32) {
    const int ne = E - e0 < 32 ? E - e0 : 32;
    float acc[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) acc[e] = 0.0f;
    for (int kk = tid; kk < d; kk += 256) {
      const float xv = to_f<T>(x[kk]);
      const T* wrow = Wr + (size_t)kk * E + e0;
#pragma unroll
      for (int e = 0; e < 32; ++e)
        if (e < ne) acc[e] += xv * to_f<T>(wrow[e]);
    }
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      float v = acc[e];
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) s_part[w][e] = v;
    }
    __syncthreads();
    if (tid < ne) {
      float v = 0.0f;
      for (int q = 0; q < 8; ++q) v += s_part[q][tid];
      v += br ? to_f<T>(br[e0 + tid]) : 0.0f;
      s_r[e0 + tid] = v + (-65000.0f);
    }
    __syncthreads();
  }
  if (tid == 0) {
    // softmax over E (TensorApplyCPU softmax: max, exp, sum, divide) and TopK, sequentially: E is small
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) mx = fmaxf(mx, s_r[e]);
    float sum = 0.0f;
    for (int e = 0; e < E; ++e) {
      s_r[e] = expf(s_r[e] - mx);
      sum += s_r[e];
    }
    float val[kMoeMaxPicks];
    int idx[kMoeMaxPicks];
    for (int i = 0; i < k; ++i) {
      val[i] = -1.70141e+38f;
      idx[i] = -1;
    }
    for (int e = 0; e < E; ++e) {
      const float data = s_r[e] / sum;
      s_r[e] = data;
      if (data < val[k - 1]) continue;
      int j = k - 2;
      for (; j >= 0; --j) {
        if (data > val[j]) {
          val[j + 1] = val[j];
          idx[j + 1] = idx[j];
        } else {
          break;
        }
      }
      val[j + 1] = data;
      idx[j + 1] = e;
    }
    // the reference runs the experts in ascending order: sort the picks by expert index (k is tiny)
    for (int i = 1; i < k; ++i)
      for (int j = i; j > 0 && idx[j] < idx[j - 1]; --j) {
        const int ti = idx[j]; idx[j] = idx[j - 1]; idx[j - 1] = ti;
      }
    for (int i = 0; i < k; ++i) {
      TSB_DEV_CHECK(moe, idx[i] >= 0 && idx[i] < E, 0x301, (void)0)   // the router picked no expert for a slot (NaN scores): the slot is skipped downstream
      picks[(size_t)row * k + i] = idx[i];
      scores[(size_t)row * k + i] = idx[i] >= 0 ? s_r[idx[i]] : 0.0f;
    }
  }
}

__device__ __forceinline__ float moe_act(float v, int act) {
  switch (act) {   // MoEFeedForward.RunActivateFunction has branches for SiLU, ReLU and LeakyReLU only (:162-178)
    case TSB200_ACT_RELU: return v < 0.0f ? 0.0f : v;
    case TSB200_ACT_SILU: return v / (1.0f + expf(-v));
    case TSB200_ACT_LEAKYRELU: return v < 0.0f ? 0.01f * v : v;
    default: return v;
  }
}

// hidden [rows, k, Fh]; grid (ceil(Fh / 256), rows * k)
template <typename T>
__global__ void __launch_bounds__(256) moe_up_kernel(T* hidden, const T* h, const T* W1, const int* picks, int d, int Fh, int k, int act) {
  extern __shared__ float s_x[];
  pdl_trigger();
  pdl_wait();
  const int rp = blockIdx.y, row = rp / k;
  const int e = picks[rp];
  for (int i = threadIdx.x; i < d; i += 256) s_x[i] = to_f<T>(h[(size_t)row * d + i]);
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= Fh || e < 0) return;
  const T* W = W1 + (size_t)e * d * Fh + c;
  float acc = 0.0f;
#pragma unroll 8
  for (int kk = 0; kk < d; ++kk) acc += s_x[kk] * to_f<T>(W[(size_t)kk * Fh]);
  hidden[(size_t)rp * Fh + c] = from_f<T>(moe_act(acc, act));
}

// x32 [rows, d] += sum over picks of score * (hidden[row, pick] W2[expert]); grid (ceil(d / 256), rows)
template <typename T>
__global__ void __launch_bounds__(256) moe_down_kernel(float* x32, const T* hidden, const T* W2, const int* picks, const float* scores, int d,
                                                       int Fh, int k) {
  extern __shared__ float s_x[];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.y;
  const int c = blockIdx.x * 256 + threadIdx.x;
  float total = 0.0f;
  for (int j = 0; j < k; ++j) {
    const int e = picks[(size_t)row * k + j];
    __syncthreads();
    for (int i = threadIdx.x; i < Fh; i += 256) s_x[i] = to_f<T>(hidden[((size_t)row * k + j) * Fh + i]);
    __syncthreads();
    if (c < d && e >= 0) {
      const T* W = W2 + (size_t)e * Fh * d + c;
      float acc = 0.0f;
#pragma unroll 8
      for (int kk = 0; kk < Fh; ++kk) acc += s_x[kk] * to_f<T>(W[(size_t)kk * d]);
      // the reference rounds the expert's output to the model's type before it is weighted (Mul, then EltMul)
      total += to_f<T>(from_f<T>(acc)) * scores[(size_t)row * k + j];
    }
  }
  if (c < d) x32[(size_t)row * d + c] += total;
}

template <typename T>
static int moe_launch(int device, float* x32, const void* h, const void* Wr, const void* br, const void* W1, const void* W2, void* hidden,
                      int* picks, float* scores, int rows, int d, int E, int k, int act, cudaStream_t s) {
  const int Fh = 4 * d;
  TSB_CUDA(launch_k(moe_route_kernel<T>, dim3(rows), dim3(256), 0, s, picks, scores, (const T*)h, (const T*)Wr, (const T*)br, d, E, k));
  count_launch(device);
  TSB_CUDA(launch_k(moe_up_kernel<T>, dim3((Fh + 255) / 256, rows * k), dim3(256), (size_t)d * 4, s, (T*)hidden, (const T*)h, (const T*)W1,
                    (const int*)picks, d, Fh, k, act));
  count_launch(device);
  TSB_CUDA(launch_k(moe_down_kernel<T>, dim3((d + 255) / 256, rows), dim3(256), (size_t)Fh * 4, s, x32, (const T*)hidden, (const T*)W2,
                    (const int*)picks, (const float*)scores, d, Fh, k));
  count_launch(device);
  return check_launch("moe feed-forward");
}

// h: the layer's normed input [rows, d] in the model type; x32: the residual stream (updated in place).
// hidden: scratch [rows, k, 4d] model type; picks / scores: scratch [rows, k].
int launch_moe_ffn(int device, DeviceState* st, int dtype, float* x32, const void* h, const void* router_w, const void* router_b,
                   const void* W1, const void* W2, void* hidden, int* picks, float* scores, int rows, int d, int E, int k, int act,
                   cudaStream_t s) {
  (void)st;
  TSB_CHECK(E >= 2 && E <= kMoeMaxExperts && k >= 1 && k <= kMoeMaxPicks && k <= E, "moe: %d experts with %d per token is not supported (at most %d and %d)",
            E, k, kMoeMaxExperts, kMoeMaxPicks);
  TSB_CHECK((size_t)4 * d * 4 <= 160 * 1024, "moe: hidden size %d is too large for the expert kernels", d);
  if (rows == 0) return 1;
  static bool attr_done[kMaxDevices] = {};
  if (!attr_done[device]) {
    TSB_CUDA(cudaFuncSetAttribute(moe_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    TSB_CUDA(cudaFuncSetAttribute(moe_down_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    attr_done[device] = true;
  }
  if (dtype == TSB200_F32) return moe_launch<float>(device, x32, h, router_w, router_b, W1, W2, hidden, picks, scores, rows, d, E, k, act, s);
  return moe_launch<__half>(device, x32, h, router_w, router_b, W1, W2, hidden, picks, scores, rows, d, E, k, act, s);
}

}  // namespace tsb
