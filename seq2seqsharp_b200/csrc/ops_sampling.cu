// Softmax, ArgMax, fused logits softmax + ArgMax, Top-P sort-and-sample and the Philox uniform stream.
//
//  * "softmax"  : row max -> exp(x - max) -> / sum, fp32 internally (TensorSharp/TensorApplyCPU.cs:1230-1268;
//                 TensorSharp.CUDA/DeviceCode/AdvFuncKernels.cs:1534-1600).
//  * "argmax"   : lowest index among equal maxima (TensorApplyCPU.cs:339-360;
//                 TensorSharp.CUDA/DeviceCode/ReduceDimIndexKernels.cs:25,96-119 scans one thread per row — here a
//                 whole CTA reduces (value, index) pairs with warp shuffles and the same tie rule).
//  * Top-P      : device version of the host loop ComputeGraphTensor.TopPSample
//                 (Seq2SeqSharp/Tools/ComputeGraphTensor.cs:2305-2403); see topp_kernel.
#include <mutex>
#include <cstdlib>

#include "kernels.cuh"

namespace tsb {

TSB_CHECKED_WORD(sampling)
#ifndef TSB200_CHECKED
int chk_take_sampling() { return 0; }
#endif

struct ValIdx {
  float v;
  int i;
};
// "a beats b": strictly greater value, or equal value and lower index (first-max rule).
__device__ __forceinline__ ValIdx better(ValIdx a, ValIdx b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ValIdx warp_argmax(ValIdx x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ValIdx y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  return x;
}
__device__ __forceinline__ ValIdx block_argmax(ValIdx x, ValIdx* red /* 32 */) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  x = warp_argmax(x);
  __syncthreads();
  if (lane == 0) red[w] = x;
  __syncthreads();
  ValIdx r;
  r.v = -INFINITY;
  r.i = 0x7fffffff;
  if (lane < nw) r = red[lane];
  return warp_argmax(r);
}

// ------------------------------------------------------------------------------------------------ softmax
template <typename T>
__global__ void __launch_bounds__(1024) softmax_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t rows, int cols,
                                                       int64_t in_row_stride, int64_t in_col_stride) {
  __shared__ float red[32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* x = in + r * in_row_stride;
    T* y = out + r * (int64_t)cols;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) mx = fmaxf(mx, to_f<T>(x[(int64_t)i * in_col_stride]));
    mx = block_max(mx, red);
    float s = 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) s += expf(to_f<T>(x[(int64_t)i * in_col_stride]) - mx);
    s = block_sum(s, red);
    for (int i = threadIdx.x; i < cols; i += blockDim.x)
      y[i] = from_f<T>(expf(to_f<T>(x[(int64_t)i * in_col_stride]) - mx) / s);
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------ argmax
// src viewed as [outer, n, inner] with the reduced dimension in the middle.
template <typename T, typename TO>
__global__ void __launch_bounds__(256) argmax_kernel(TO* __restrict__ out, const T* __restrict__ in, int64_t outer, int n,
                                                     int64_t inner, int64_t so, int64_t sn, int64_t si) {
  __shared__ ValIdx red[32];
  for (int64_t r = blockIdx.x; r < outer * inner; r += gridDim.x) {
    const int64_t o = r / inner, ii = r % inner;
    const T* x = in + o * so + ii * si;
    ValIdx best;
    best.v = -INFINITY;
    best.i = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      ValIdx c;
      c.v = to_f<T>(x[(int64_t)i * sn]);
      c.i = i;
      if (best.i == 0x7fffffff || c.v > best.v) best = c;  // strictly greater, as the reference scan
    }
    best = block_argmax(best, red);
    if (threadIdx.x == 0) out[r] = (TO)(best.i == 0x7fffffff ? 0 : best.i);
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------ fused softmax + argmax
// logits [B,V] fp32 -> probs (optionally stored) -> first index of the row maximum of the PROBABILITIES, which is
// what the reference compares (Decoder.cs:732-761): logits that differ can round to equal probabilities, and
// the lowest index must then win.  Blocked ids get p += -1 (Decoder.cs:744-752).
__global__ void __launch_bounds__(1024) softmax_argmax_kernel(int* out_ids, float* probs,
                                                              const float* logits, int V, float inv_temp_div,
                                                              int use_temp, const int* blocked, int n_blocked) {
  __shared__ float red[32];
  __shared__ ValIdx redi[32];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* z = logits + (int64_t)r * V;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = z[i];
    if (use_temp) v = v / inv_temp_div;
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, red);
  float s = 0.0f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = z[i];
    if (use_temp) v = v / inv_temp_div;
    s += expf(v - mx);
  }
  s = block_sum(s, red);
  ValIdx best;
  best.v = -INFINITY;
  best.i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = z[i];
    if (use_temp) v = v / inv_temp_div;
    float p = expf(v - mx) / s;
    for (int j = 0; j < n_blocked; ++j)
      if (blocked[j] == i) p += -1.0f;
    if (probs) probs[(int64_t)r * V + i] = p;
    ValIdx c;
    c.v = p;
    c.i = i;
    best = better(best, c);
  }
  best = block_argmax(best, redi);
  if (threadIdx.x == 0 && out_ids) out_ids[r] = best.i == 0x7fffffff ? 0 : best.i;
}

// ------------------------------------------------------------------------------------------------ Philox4x32-10
__host__ __device__ inline void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
    const uint32_t n3 = (uint32_t)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}
// key = (seed lo, seed hi), counter = (step, 0, seq lo, seq hi); u = (x0 >> 8) * 2^-24 in [0,1)
__host__ __device__ inline float philox_uniform(uint64_t seed, uint64_t seq, uint32_t step) {
  uint32_t c[4] = {step, 0u, (uint32_t)seq, (uint32_t)(seq >> 32)};
  philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
  return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}
// dstate: the engine's device step state (kernels.cuh), or NULL: then every row uses step_arg
__global__ void philox_kernel(float* u, int n, uint64_t seed, uint64_t seq_first, uint32_t step_arg, const int* dstate) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) u[i] = philox_uniform(seed, seq_first + (uint64_t)i, (uint32_t)state_step(dstate, i, (int)step_arg));
}

// ------------------------------------------------------------------------------------------------ Top-P
// One CTA of 1024 threads per row.  Workspace per row (uint32 words): keyA[V] keyB[V] idxA[V] idxB[V] last[V].
//  1. key[j] = bits(w_j) for w_j > 0 else 0, where w_j = probs[j] * (float)pow(dist/len, repeatPenalty) for ids
//     already in the row's history (dist counted from the LAST occurrence), computed as the reference does:
//     float ratio -> double pow -> float -> float multiply.
//  2. stable LSD radix sort, 4 x 8 bits, descending by key: equal keys keep ascending index order, which is the
//     reference's SortedDictionary<float, List<int>> iterated in reverse with insertion-ordered lists.
//  3. one lane accumulates acc += w sequentially in fp32 (the reference's rounding order) and stops at the first
//     acc >= topP; accumulated values are kept.
//  4. all threads search the first k with acc[k] / acc_final >= u.
constexpr int kTopPThreads = 1024;
constexpr int kTopPWarps = kTopPThreads / 32;
constexpr int kScanChunk = 1024;   // head of the prefix sum staged in shared memory
constexpr int kRadixUnroll = 8;

struct ToppSmem {
  uint32_t hist[kTopPWarps][256];  // per-warp digit counters / offsets
  uint32_t warp_tot[32];
  float chunk[kScanChunk];
  int n_cand;
  float acc_final;
  int stop;
  int best_k;
  int n_valid;
  int ov_idx, stop_idx;   // first index of the window whose sum left the binade / reached topP
  int k_next;
  uint32_t acc_bits;
  int2 warp_pair[32];
  uint32_t tot[256];    // cluster sort: this CTA's count per digit (read by the other CTAs of the cluster)
  uint32_t base[256];   // cluster sort: global offset of this CTA's first key of a digit, minus its local offset
};

// The buffers are written earlier in the same kernel, so they are deliberately NOT const __restrict__ (no
// non-coherent read-only loads).
__device__ __forceinline__ void radix_pass(const uint32_t* kin, const uint32_t* iin, uint32_t* kout, uint32_t* iout, int n,
                                           int shift, bool first, ToppSmem& sm) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int per_warp = ((n + kTopPWarps - 1) / kTopPWarps + 31) & ~31;
  const int beg = w * per_warp, end = min(n, beg + per_warp);
  for (int i = threadIdx.x; i < kTopPWarps * 256; i += blockDim.x) (&sm.hist[0][0])[i] = 0;
  __syncthreads();
  // A: per-warp histogram of the (descending) digit; kRadixUnroll loads are in flight per lane
  for (int base0 = beg; base0 < end; base0 += 32 * kRadixUnroll) {
    uint32_t keys[kRadixUnroll];
#pragma unroll
    for (int q = 0; q < kRadixUnroll; ++q) {
      const int j = base0 + q * 32 + lane;
      keys[q] = j < end ? kin[j] : 0u;
    }
#pragma unroll
    for (int q = 0; q < kRadixUnroll; ++q) {
      const int j = base0 + q * 32 + lane;
      if (base0 + q * 32 >= end) break;
      const bool ok = j < end;
      const uint32_t dg = ok ? (255u - ((keys[q] >> shift) & 255u)) : 256u;
      const uint32_t peers = __match_any_sync(0xffffffffu, dg);
      if (ok && lane == (__ffs(peers) - 1)) sm.hist[w][dg] += __popc(peers);
      __syncwarp();
    }
  }
  __syncthreads();
  // B: exclusive scan in (digit-major, warp-minor) order
  {
    uint32_t v[8];
    uint32_t tsum = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int li = threadIdx.x * 8 + e;  // li = digit * 32 + warp
      v[e] = sm.hist[li & 31][li >> 5];
      tsum += v[e];
    }
    uint32_t incl = tsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) sm.warp_tot[w] = incl;
    __syncthreads();
    if (w == 0) {
      uint32_t t = sm.warp_tot[lane];
      uint32_t ti = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t u2 = __shfl_up_sync(0xffffffffu, ti, o);
        if (lane >= o) ti += u2;
      }
      sm.warp_tot[lane] = ti - t;
    }
    __syncthreads();
    uint32_t run = sm.warp_tot[w] + incl - tsum;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int li = threadIdx.x * 8 + e;
      sm.hist[li & 31][li >> 5] = run;
      run += v[e];
    }
  }
  __syncthreads();
  // C: stable scatter
  for (int base0 = beg; base0 < end; base0 += 32 * kRadixUnroll) {
    uint32_t keys[kRadixUnroll], idxs[kRadixUnroll];
#pragma unroll
    for (int q = 0; q < kRadixUnroll; ++q) {
      const int j = base0 + q * 32 + lane;
      keys[q] = j < end ? kin[j] : 0u;
      idxs[q] = j < end ? (first ? (uint32_t)j : iin[j]) : 0u;
    }
#pragma unroll
    for (int q = 0; q < kRadixUnroll; ++q) {
      const int j = base0 + q * 32 + lane;
      if (base0 + q * 32 >= end) break;
      const bool ok = j < end;
      const uint32_t dg = ok ? (255u - ((keys[q] >> shift) & 255u)) : 256u;
      const uint32_t peers = __match_any_sync(0xffffffffu, dg);
      const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
      uint32_t pos = 0;
      if (ok) pos = sm.hist[w][dg] + rank;
      __syncwarp();
      if (ok) {
        kout[pos] = keys[q];
        iout[pos] = idxs[q];
        if (lane == (__ffs(peers) - 1)) sm.hist[w][dg] += __popc(peers);
      }
      __syncwarp();
    }
  }
  __syncthreads();
}

// ---- exact parallel evaluation of   acc = 0; for k: acc = fl32(acc + w[k])   for sorted positive w ------------------
// While acc stays inside one binade [2^e, 2^(e+1)) it is a multiple of ulp = 2^(e-23) and fl32(acc + w) equals
// acc + ulp * (q + r), where w/ulp = q + f and r rounds f to nearest, ties to even of (acc/ulp + q).  So in units of
// ulp every element is the map A -> A + inc[A & 1] with two integer increments, these maps compose associatively, and
// a block-wide scan of the composed maps gives every partial sum of a window bit-exactly.  The first element whose
// sum leaves the binade (A >= 2^24) is added with one ordinary fp32 add (the hardware rounds on the coarser grid) and
// the next window starts from there.  The first kHead elements, where binades change every few elements, are added
// one by one from shared memory.
struct IncPair {
  int i0, i1;  // increment when the incoming A is even / odd
};
__device__ __forceinline__ int sat_add(int a, int b) { return min(a + b, 1 << 29); }
__device__ __forceinline__ IncPair compose(IncPair f, IncPair g) {  // first f, then g
  IncPair h;
  h.i0 = sat_add(f.i0, (f.i0 & 1) ? g.i1 : g.i0);
  h.i1 = sat_add(f.i1, ((1 + f.i1) & 1) ? g.i1 : g.i0);
  return h;
}
__device__ __forceinline__ void split_float(uint32_t bits, int& e, uint32_t& m) {
  const uint32_t E = bits >> 23;
  if (E == 0) {
    e = -126;
    m = bits & 0x7fffffu;
  } else {
    e = (int)E - 127;
    m = (bits & 0x7fffffu) | 0x800000u;
  }
}
__device__ __forceinline__ IncPair inc_of(uint32_t wbits, int e) {
  int ew;
  uint32_t m;
  split_float(wbits, ew, m);
  const int shift = e - ew;
  IncPair r;
  if (shift <= 0) {  // w is in the same (or a higher) binade: the sum leaves the binade at once
    r.i0 = r.i1 = 1 << 29;
    return r;
  }
  if (shift >= 32) {
    r.i0 = r.i1 = 0;
    return r;
  }
  const uint32_t q = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  const int up = rem > half ? 1 : 0, tie = rem == half ? 1 : 0;
  r.i0 = (int)q + up + (tie & (int)(q & 1u));          // A even: A+q is odd iff q is odd
  r.i1 = (int)q + up + (tie & (int)((q & 1u) ^ 1u));   // A odd
  return r;
}
constexpr int kHead = 1024;
constexpr int kPerThread = 8;

__device__ void exact_prefix(const uint32_t* keys, float* accs, int n_valid, float topP, ToppSmem& sm) {
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  // ---- head: plain sequential adds out of shared memory, eight at a time
  const int nh = min(n_valid, kHead);
  for (int i = tid; i < nh; i += blockDim.x) sm.chunk[i] = __uint_as_float(__ldcg(keys + i));
  __syncthreads();
  if (tid == 0) {
    float acc = 0.0f;
    int i = 0, stop = 0;
    while (i < nh && !stop) {
      float v[8];
      const int c = min(8, nh - i);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = j < c ? sm.chunk[i + j] : 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < c && !stop) {
          acc += v[j];
          sm.chunk[i + j] = acc;
          if (acc >= topP) {
            stop = 1;
            sm.n_cand = i + j + 1;
          }
        }
      }
      i += c;
    }
    if (!stop) sm.n_cand = nh;
    sm.stop = stop || (nh == n_valid);
    sm.acc_final = acc;
    sm.k_next = nh;
    sm.acc_bits = __float_as_uint(acc);
  }
  __syncthreads();
  for (int i = tid; i < sm.n_cand && i < nh; i += blockDim.x) accs[i] = sm.chunk[i];
  // ---- windows of blockDim * kPerThread elements
  while (true) {
    __syncthreads();
    if (sm.stop) break;
    const int k0 = sm.k_next;
    int e;
    uint32_t A0;
    split_float(sm.acc_bits, e, A0);
    if (tid == 0) {
      sm.ov_idx = 0x7fffffff;
      sm.stop_idx = 0x7fffffff;
    }
    const int base = k0 + tid * kPerThread;
    uint32_t wb[kPerThread];
    IncPair f[kPerThread], F;
    F.i0 = F.i1 = 0;
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
      wb[j] = (base + j < n_valid) ? __ldcg(keys + base + j) : 0u;
      if (wb[j]) f[j] = inc_of(wb[j], e);
      else f[j].i0 = f[j].i1 = 0;
      F = compose(F, f[j]);
    }
    // inclusive scan of the per-thread maps across the block
    IncPair incl = F;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      IncPair prev;
      prev.i0 = __shfl_up_sync(0xffffffffu, incl.i0, o);
      prev.i1 = __shfl_up_sync(0xffffffffu, incl.i1, o);
      if (lane >= o) incl = compose(prev, incl);
    }
    if (lane == 31) sm.warp_pair[w] = make_int2(incl.i0, incl.i1);
    __syncthreads();
    if (w == 0) {
      const int2 t = sm.warp_pair[lane];
      IncPair x;
      x.i0 = t.x;
      x.i1 = t.y;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        IncPair prev;
        prev.i0 = __shfl_up_sync(0xffffffffu, x.i0, o);
        prev.i1 = __shfl_up_sync(0xffffffffu, x.i1, o);
        if (lane >= o) x = compose(prev, x);
      }
      sm.warp_pair[lane] = make_int2(x.i0, x.i1);  // inclusive over warps
    }
    __syncthreads();
    // exclusive map for this thread = (all earlier warps) then (earlier lanes of this warp)
    IncPair excl;
    excl.i0 = excl.i1 = 0;
    if (w > 0) {
      const int2 t = sm.warp_pair[w - 1];
      excl.i0 = t.x;
      excl.i1 = t.y;
    }
    {
      IncPair lane_prev;
      lane_prev.i0 = __shfl_up_sync(0xffffffffu, incl.i0, 1);
      lane_prev.i1 = __shfl_up_sync(0xffffffffu, incl.i1, 1);
      if (lane > 0) excl = compose(excl, lane_prev);
    }
    int A = sat_add((int)A0, (A0 & 1u) ? excl.i1 : excl.i0);
    const uint32_t ebits = (uint32_t)(e + 126) << 23;
    float outv[kPerThread];
    int n_ok = 0;
    bool live = A < (1 << 24);
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
      if (live && base + j < n_valid) {
        A = sat_add(A, (A & 1) ? f[j].i1 : f[j].i0);
        if (A >= (1 << 24)) {
          atomicMin(&sm.ov_idx, base + j);
          live = false;
        } else {
          const float v = __uint_as_float(ebits + (uint32_t)A);
          outv[j] = v;
          n_ok = j + 1;
          if (v >= topP) {
            atomicMin(&sm.stop_idx, base + j);
            live = false;
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kPerThread; ++j)
      if (j < n_ok) accs[base + j] = outv[j];
    __syncthreads();
    if (tid == 0) {
      const int wend = min(n_valid, k0 + (int)blockDim.x * kPerThread);
      const int ov = sm.ov_idx, st = sm.stop_idx;
      if (st < ov) {  // reached topP inside the valid part of the window
        sm.n_cand = st + 1;
        sm.stop = 1;
      } else if (ov < wend) {  // element `ov` carries the sum into the next binade: one ordinary fp32 add
        const float prev = (ov == k0) ? __uint_as_float(sm.acc_bits) : accs[ov - 1];
        const float acc = prev + __uint_as_float(__ldcg(keys + ov));
        accs[ov] = acc;
        sm.acc_bits = __float_as_uint(acc);
        sm.k_next = ov + 1;
        sm.n_cand = ov + 1;
        if (acc >= topP || ov + 1 >= n_valid) sm.stop = 1;
      } else {
        sm.k_next = wend;
        sm.n_cand = wend;
        sm.acc_bits = __float_as_uint(accs[wend - 1]);
        if (wend >= n_valid) sm.stop = 1;
      }
    }
  }
  __syncthreads();
  if (tid == 0) sm.acc_final = sm.n_cand > 0 ? accs[sm.n_cand - 1] : 0.0f;
}

__global__ void __launch_bounds__(kTopPThreads) topp_kernel(int* out, const float* probs, int V,
                                                            float topP, float repeatPenalty,
                                                            const int* history,
                                                            const int* history_len, int history_stride,
                                                            const float* u, uint32_t* ws) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ToppSmem& sm = *reinterpret_cast<ToppSmem*>(smem_raw);
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  uint32_t* keyA = ws + (size_t)r * 5 * V;
  uint32_t* keyB = keyA + V;
  uint32_t* idxA = keyB + V;
  uint32_t* idxB = idxA + V;
  int* last = reinterpret_cast<int*>(idxB + V);
  const float* p = probs + (size_t)r * V;
  const int* hist = history ? history + (size_t)r * history_stride : nullptr;
  const int len = (history && history_len) ? history_len[r] : 0;

  // 1. keys (+ repeat penalty on the last occurrence of each id in the history)
  for (int j = threadIdx.x; j < V; j += blockDim.x) {
    const float w = p[j];
    keyA[j] = (w > 0.0f) ? __float_as_uint(w) : 0u;
  }
  for (int q = threadIdx.x; q < len; q += blockDim.x) {
    const int t = hist[q];
    if (t >= 0 && t < V) last[t] = -1;
  }
  __syncthreads();
  for (int q = threadIdx.x; q < len; q += blockDim.x) {
    const int t = hist[q];
    if (t >= 0 && t < V) atomicMax(&last[t], q);
  }
  __syncthreads();
  for (int q = threadIdx.x; q < len; q += blockDim.x) {
    const int t = hist[q];
    if (t >= 0 && t < V && last[t] == q) {
      float w = p[t];
      if (w > 0.0f) {
        const float ratio = (float)(len - q) / (float)len;
        const float rp = (float)pow((double)ratio, (double)repeatPenalty);
        w = w * rp;
        keyA[t] = __float_as_uint(w);  // may become +0: stays in the list with weight 0, as in the reference
        if (w == 0.0f) keyA[t] = 0u;   // a zero weight sorts with the dropped entries; it adds nothing to acc
      }
    }
  }
  __syncthreads();

  // 2. sort descending, stable
  radix_pass(keyA, nullptr, keyB, idxB, V, 0, true, sm);
  radix_pass(keyB, idxB, keyA, idxA, V, 8, false, sm);
  radix_pass(keyA, idxA, keyB, idxB, V, 16, false, sm);
  radix_pass(keyB, idxB, keyA, idxA, V, 24, false, sm);
  // sorted: keyA / idxA

  // 3. fp32 prefix sum with the reference's left-to-right rounding, computed exactly but in parallel (see exact_prefix)
  if (threadIdx.x == 0) {
    sm.n_cand = 0;
    sm.acc_final = 0.0f;
    sm.stop = 0;
    sm.best_k = 0x7fffffff;
    sm.n_valid = 0;
  }
  __syncthreads();
  // number of entries with w > 0 (they sort first)
  for (int j = threadIdx.x; j < V; j += blockDim.x)
    if (keyA[j] != 0u && (j + 1 == V || keyA[j + 1] == 0u)) sm.n_valid = j + 1;
  __syncthreads();
  float* accs = reinterpret_cast<float*>(keyB);  // accumulated values, reusing a sort buffer
  exact_prefix(keyA, accs, sm.n_valid, topP, sm);
  __syncthreads();

  // 4. first k with acc[k] / acc_final >= u
  const int n = sm.n_cand;
  const float tot = sm.acc_final, uu = u[r];
  int mine = 0x7fffffff;
  for (int k = threadIdx.x; k < n; k += blockDim.x)
    if (accs[k] / tot >= uu) {
      mine = k;
      break;
    }
  if (mine != 0x7fffffff) atomicMin(&sm.best_k, mine);
  __syncthreads();
  if (threadIdx.x == 0) out[r] = (sm.best_k == 0x7fffffff) ? 0 : (int)idxA[sm.best_k];
}


// ------------------------------------------------------------------------------------------------ Top-P on a cluster
// The same algorithm with the stable radix sort spread over a thread-block cluster of kToppCluster CTAs (one cluster
// per row): CTA c ranks the c-th slice of the current key order, the 256 digit totals of every CTA are read through
// distributed shared memory after a cluster barrier, and the scatter goes to the global ping-pong buffers (L2).
// A slice is 1/8 of the vocabulary, so the latency-bound ranking chains are 8 times shorter than on one SM.  CTA 0
// then runs the exact prefix sum and the search.  Keys and indices written by other CTAs are read with L2 loads.
constexpr int kToppCluster = 8;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t ld_dsmem_u32(const uint32_t* local_ptr, uint32_t cta) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(local_ptr), ra, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(cta));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(ra) : "memory");
  return v;
}

__device__ __forceinline__ void radix_pass_cluster(const uint32_t* kin, const uint32_t* iin, uint32_t* kout, uint32_t* iout, int n,
                                                   int shift, bool first, ToppSmem& sm, int crank) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int n_per = ((n + kToppCluster - 1) / kToppCluster + 31) & ~31;
  const int s_beg = min(n, crank * n_per), s_end = min(n, s_beg + n_per);
  const int n_loc = s_end - s_beg;
  const int per_warp = ((n_loc + kTopPWarps - 1) / kTopPWarps + 31) & ~31;
  const int beg = min(s_end, s_beg + w * per_warp), end = min(s_end, beg + per_warp);
  for (int i = threadIdx.x; i < kTopPWarps * 256; i += blockDim.x) (&sm.hist[0][0])[i] = 0;
  __syncthreads();
  // A: per-warp histogram of the (descending) digit
  for (int base0 = beg; base0 < end; base0 += 32 * kRadixUnroll) {
    uint32_t keys[kRadixUnroll];
#pragma unroll
    for (int q = 0; q < kRadixUnroll; ++q) {
      const int j = base0 + q * 32 + lane;
      keys[q] = j < end ? __ldcg(kin + j) : 0u;
    }
#pragma unroll
    for (int q = 0; q < kRadixUnroll; ++q) {
      const int j = base0 + q * 32 + lane;
      if (base0 + q * 32 >= end) break;
      const bool ok = j < end;
      const uint32_t dg = ok ? (255u - ((keys[q] >> shift) & 255u)) : 256u;
      const uint32_t peers = __match_any_sync(0xffffffffu, dg);
      if (ok && lane == (__ffs(peers) - 1)) sm.hist[w][dg] += __popc(peers);
      __syncwarp();
    }
  }
  __syncthreads();
  // B: exclusive scan inside the CTA in (digit-major, warp-minor) order
  {
    uint32_t v[8];
    uint32_t tsum = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int li = threadIdx.x * 8 + e;  // li = digit * 32 + warp
      v[e] = sm.hist[li & 31][li >> 5];
      tsum += v[e];
    }
    uint32_t incl = tsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) sm.warp_tot[w] = incl;
    __syncthreads();
    if (w == 0) {
      uint32_t t = sm.warp_tot[lane];
      uint32_t ti = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t u2 = __shfl_up_sync(0xffffffffu, ti, o);
        if (lane >= o) ti += u2;
      }
      sm.warp_tot[lane] = ti - t;
    }
    __syncthreads();
    uint32_t run = sm.warp_tot[w] + incl - tsum;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int li = threadIdx.x * 8 + e;
      sm.hist[li & 31][li >> 5] = run;
      run += v[e];
    }
  }
  __syncthreads();
  // this CTA's keys per digit: difference of the offsets of warp 0
  if (threadIdx.x < 256) {
    const int d = threadIdx.x;
    sm.tot[d] = (d == 255 ? (uint32_t)n_loc : sm.hist[0][d + 1]) - sm.hist[0][d];
  }
  cluster_sync_all();  // every CTA's totals are in place (and all reads of the previous pass are done)
  // C: global base of (digit, this CTA): keys of smaller digits anywhere + keys of this digit in earlier CTAs
  if (threadIdx.x < 256) {
    const int d = threadIdx.x;
    uint32_t all = 0, before = 0;
#pragma unroll
    for (int c = 0; c < kToppCluster; ++c) {
      const uint32_t t = ld_dsmem_u32(&sm.tot[d], (uint32_t)c);
      all += t;
      if (c < crank) before += t;
    }
    uint32_t incl = all;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) sm.warp_tot[w] = incl;  // 8 warps take part
    asm volatile("bar.sync 2, 256;" ::: "memory");
    uint32_t wbase = 0;
    for (int i = 0; i < w; ++i) wbase += sm.warp_tot[i];
    sm.base[d] = wbase + incl - all + before - sm.hist[0][d];
  }
  __syncthreads();
  // D: stable scatter into the global buffers
  for (int base0 = beg; base0 < end; base0 += 32 * kRadixUnroll) {
    uint32_t keys[kRadixUnroll], idxs[kRadixUnroll];
#pragma unroll
    for (int q = 0; q < kRadixUnroll; ++q) {
      const int j = base0 + q * 32 + lane;
      keys[q] = j < end ? __ldcg(kin + j) : 0u;
      idxs[q] = j < end ? (first ? (uint32_t)j : __ldcg(iin + j)) : 0u;
    }
#pragma unroll
    for (int q = 0; q < kRadixUnroll; ++q) {
      const int j = base0 + q * 32 + lane;
      if (base0 + q * 32 >= end) break;
      const bool ok = j < end;
      const uint32_t dg = ok ? (255u - ((keys[q] >> shift) & 255u)) : 256u;
      const uint32_t peers = __match_any_sync(0xffffffffu, dg);
      const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
      uint32_t pos = 0;
      if (ok) pos = sm.hist[w][dg] + sm.base[dg] + rank;
      __syncwarp();
      if (ok) {
        kout[pos] = keys[q];
        iout[pos] = idxs[q];
        if (lane == (__ffs(peers) - 1)) sm.hist[w][dg] += __popc(peers);
      }
      __syncwarp();
    }
  }
  cluster_sync_all();  // the scattered keys are visible to the whole cluster; sm.tot may be rewritten
}

__global__ void __launch_bounds__(kTopPThreads) topp_cluster_kernel(int* out, const float* probs, int V, float topP, float repeatPenalty,
                                                                    const int* history, const int* history_len, int history_stride,
                                                                    const float* u, uint32_t* ws) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ToppSmem& sm = *reinterpret_cast<ToppSmem*>(smem_raw);
  pdl_trigger();
  pdl_wait();
  const int crank = (int)cluster_rank();
  const int r = blockIdx.x / kToppCluster;
  uint32_t* keyA = ws + (size_t)r * 5 * V;
  uint32_t* keyB = keyA + V;
  uint32_t* idxA = keyB + V;
  uint32_t* idxB = idxA + V;
  int* last = reinterpret_cast<int*>(idxB + V);
  const float* p = probs + (size_t)r * V;
  const int* hist = history ? history + (size_t)r * history_stride : nullptr;
  const int len = (history && history_len) ? history_len[r] : 0;
  const int n_per = ((V + kToppCluster - 1) / kToppCluster + 31) & ~31;
  const int s_beg = min(V, crank * n_per), s_end = min(V, s_beg + n_per);

  // 1. keys of this CTA's slice (+ repeat penalty on the last occurrence of each id of the slice in the history)
  for (int j = s_beg + threadIdx.x; j < s_end; j += blockDim.x) {
    const float w = p[j];
    keyA[j] = (w > 0.0f) ? __float_as_uint(w) : 0u;
  }
  for (int q = threadIdx.x; q < len; q += blockDim.x) {
    const int t = hist[q];
    if (t >= s_beg && t < s_end) last[t] = -1;
  }
  __syncthreads();
  for (int q = threadIdx.x; q < len; q += blockDim.x) {
    const int t = hist[q];
    if (t >= s_beg && t < s_end) atomicMax(&last[t], q);
  }
  __syncthreads();
  for (int q = threadIdx.x; q < len; q += blockDim.x) {
    const int t = hist[q];
    if (t >= s_beg && t < s_end && last[t] == q) {
      float w = p[t];
      if (w > 0.0f) {
        const float ratio = (float)(len - q) / (float)len;
        const float rp = (float)pow((double)ratio, (double)repeatPenalty);
        w = w * rp;
        keyA[t] = (w == 0.0f) ? 0u : __float_as_uint(w);  // a zero weight sorts with the dropped entries
      }
    }
  }
  __syncthreads();

  // 2. sort descending, stable, over the cluster
  radix_pass_cluster(keyA, nullptr, keyB, idxB, V, 0, true, sm, crank);
  radix_pass_cluster(keyB, idxB, keyA, idxA, V, 8, false, sm, crank);
  radix_pass_cluster(keyA, idxA, keyB, idxB, V, 16, false, sm, crank);
  radix_pass_cluster(keyB, idxB, keyA, idxA, V, 24, false, sm, crank);
  if (crank != 0) return;  // the last cluster barrier is behind us: nobody reads this CTA's shared memory any more

  // 3. + 4. on CTA 0: exact fp32 prefix sum and search, as in topp_kernel
  if (threadIdx.x == 0) {
    sm.n_cand = 0;
    sm.acc_final = 0.0f;
    sm.stop = 0;
    sm.best_k = 0x7fffffff;
    sm.n_valid = 0;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < V; j += blockDim.x)
    if (__ldcg(keyA + j) != 0u && (j + 1 == V || __ldcg(keyA + j + 1) == 0u)) sm.n_valid = j + 1;
  __syncthreads();
  float* accs = reinterpret_cast<float*>(keyB);
  exact_prefix(keyA, accs, sm.n_valid, topP, sm);
  __syncthreads();
  const int n = sm.n_cand;
  const float tot = sm.acc_final, uu = u[r];
  int mine = 0x7fffffff;
  for (int k = threadIdx.x; k < n; k += blockDim.x)
    if (accs[k] / tot >= uu) {
      mine = k;
      break;
    }
  if (mine != 0x7fffffff) atomicMin(&sm.best_k, mine);
  __syncthreads();
  if (threadIdx.x == 0) out[r] = (sm.best_k == 0x7fffffff) ? 0 : (int)__ldcg(idxA + sm.best_k);
}

int init_topp_attrs(int device) {
  static bool attr_set[kMaxDevices] = {false};
  if (!attr_set[device]) {
    TSB_CUDA(cudaFuncSetAttribute(topp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ToppSmem)));
    TSB_CUDA(cudaFuncSetAttribute(topp_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ToppSmem)));
    attr_set[device] = true;
  }
  return 1;
}

int launch_softmax_argmax(int device, DeviceState* st, int* out_ids, float* probs, const float* logits, int B, int V,
                          float temperature, int use_temp, const int* blocked_dev, int n_blocked, cudaStream_t s) {
  (void)st;
  if (B == 0) return 1;
  TSB_CUDA(launch_k(softmax_argmax_kernel, dim3(B), dim3(1024), 0, s, out_ids, probs, logits, V, temperature, use_temp, blocked_dev, n_blocked));
  count_launch(device);
  return check_launch("softmax_argmax");
}

int launch_topp(int device, DeviceState* st, int* out, const float* probs, int rows, int V, float topP, float repeatPenalty,
                const int* history, const int* history_len, int history_stride, const float* u, void* ws, cudaStream_t s) {
  if (rows == 0) return 1;
  TSB_TRY(init_topp_attrs(device));
  static int use_cluster = -1;
  if (use_cluster < 0) {
    const char* e = getenv("TSB200_TOPP_CLUSTER");  // "0": one CTA per row (A/B measurements)
    use_cluster = (e && e[0] == '0') ? 0 : 1;
  }
  // A cluster per row cuts the latency of one row to a half (160 against 327 us at V = 32000) but takes eight SMs: once the
  // rows no longer fit the GPU in one wave (64 rows: 3.5 waves), one CTA per row finishes earlier.
  if (use_cluster && V >= 4096 && rows * kToppCluster <= (st ? st->sm_count : 148)) {
    // one cluster of kToppCluster CTAs per row
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(rows * kToppCluster);
    cfg.blockDim = dim3(kTopPThreads);
    cfg.dynamicSmemBytes = sizeof(ToppSmem);
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = kToppCluster;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    uint32_t* wsp = (uint32_t*)ws;
    TSB_CUDA(cudaLaunchKernelEx(&cfg, topp_cluster_kernel, out, probs, V, topP, repeatPenalty, history, history_len, history_stride, u, wsp));
    count_launch(device);
    return check_launch("topp_cluster");
  }
  TSB_CUDA(launch_k(topp_kernel, dim3(rows), dim3(kTopPThreads), sizeof(ToppSmem), s, out, probs, V, topP, repeatPenalty, history,
                    history_len, history_stride, u, (uint32_t*)ws));
  count_launch(device);
  return check_launch("topp");
}

int launch_philox(int device, float* u, int n, uint64_t seed, uint64_t seq_first, uint32_t step, const int* dstep,
                  cudaStream_t s) {
  if (n == 0) return 1;
  TSB_CUDA(launch_k(philox_kernel, dim3((n + 127) / 128), dim3(128), 0, s, u, n, seed, seq_first, step, dstep));
  count_launch(device);
  return check_launch("philox");
}

// ------------------------------------------------------------------------------------------------ beam candidates
// The reference takes the K candidates of a hypothesis by K rounds of (ArgMax, Gather, Log, ScatterFill 0) on the
// probabilities (Decoder.cs:459-517 `while (beamSearchSize > 0)`): the same here, one CTA per row, the rounds inside the
// kernel.  probs is changed as the reference changes it (the chosen entries end as 0).  Ties go to the lower index.
__global__ void __launch_bounds__(1024) beam_topk_kernel(int* __restrict__ out_ids, float* __restrict__ out_p, float* __restrict__ out_logp,
                                                         float* __restrict__ probs, int V, int K) {
  __shared__ ValIdx red[32];
  pdl_trigger();
  pdl_wait();
  float* p = probs + (size_t)blockIdx.x * V;
  for (int k = 0; k < K; ++k) {
    ValIdx best;
    best.v = -INFINITY;
    best.i = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      ValIdx c;
      c.v = p[i];
      c.i = i;
      best = better(best, c);
    }
    best = block_argmax(best, red);
    if (threadIdx.x == 0) {
      out_ids[(size_t)blockIdx.x * K + k] = best.i;
      out_p[(size_t)blockIdx.x * K + k] = best.v;
      out_logp[(size_t)blockIdx.x * K + k] = logf(best.v);
      TSB_DEV_CHECK(sampling, best.i >= 0 && best.i < V, 0x401, (void)0)   // no candidate found (a row of NaNs): nothing is zeroed
      if (best.i < V) p[best.i] = 0.0f;
    }
    __syncthreads();   // the zero is in place (same CTA, global memory) before the next round reads the row
  }
}

int launch_beam_topk(int device, DeviceState* st, int* out_ids, float* out_p, float* out_logp, float* probs, int rows, int V, int K,
                     cudaStream_t s) {
  (void)st;
  if (rows == 0 || K == 0) return 1;
  TSB_CUDA(launch_k(beam_topk_kernel, dim3(rows), dim3(V >= 8192 ? 1024 : 256), 0, s, out_ids, out_p, out_logp, probs, V, K));
  count_launch(device);
  return check_launch("beam_topk");
}

}  // namespace tsb

using namespace tsb;

extern "C" {

int TSB200_Softmax(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_TRY(check_tensor(result, "result"));
  TSB_TRY(check_tensor(src, "src"));
  TSB_CHECK(result->dtype == src->dtype, "softmax: dtype mismatch");
  TSB_CHECK(numel(result) == numel(src) && is_contiguous(result), "softmax: result must be contiguous and match src");
  const int cols = (int)src->sizes[src->ndim - 1];
  const int64_t rows = cols ? numel(src) / cols : 0;
  if (rows == 0) return 1;
  int64_t rs = cols, cs = 1;
  if (!is_contiguous(src)) {
    TSB_CHECK(src->ndim == 2, "softmax: non-contiguous src must be a 2-D view");
    rs = src->strides[0];
    cs = src->strides[1];
  }
  cudaStream_t s = pick_stream(st, stream);
  const int g = (int)(rows < (int64_t)st->sm_count * 4 ? rows : (int64_t)st->sm_count * 4);
  const int th = cols >= 4096 ? 1024 : (cols >= 512 ? 256 : 64);
  if (src->dtype == TSB200_F32) softmax_kernel<float><<<g, th, 0, s>>>((float*)result->data, (const float*)src->data, rows, cols, rs, cs);
  else if (src->dtype == TSB200_F16) softmax_kernel<__half><<<g, th, 0, s>>>((__half*)result->data, (const __half*)src->data, rows, cols, rs, cs);
  else TSB_FAIL("softmax: unsupported dtype %d", src->dtype);
  count_launch(device);
  return check_launch("softmax");
}

int TSB200_Argmax(int device, const TSB200Tensor* result, const TSB200Tensor* src, int dim, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_TRY(check_tensor(result, "result"));
  TSB_TRY(check_tensor(src, "src"));
  if (dim < 0) dim = src->ndim - 1;
  TSB_CHECK(dim < src->ndim, "argmax: dim out of range");
  TSB_CHECK(is_contiguous(result), "argmax: result must be contiguous");
  const int n = (int)src->sizes[dim];
  TSB_CHECK(n > 0, "argmax: empty dimension");
  // collapse to [outer, n, inner]; needs the outer and inner groups to be uniformly strided
  int64_t outer = 1, inner = 1, so = 0, si = 1;
  for (int i = 0; i < dim; ++i) outer *= src->sizes[i];
  for (int i = dim + 1; i < src->ndim; ++i) inner *= src->sizes[i];
  if (is_contiguous(src)) {
    so = (int64_t)n * inner;
    si = 1;
  } else {
    TSB_CHECK(src->ndim == 2, "argmax: non-contiguous src must be a 2-D view");
    so = dim == 1 ? src->strides[0] : 0;
    si = dim == 0 ? src->strides[1] : 1;
  }
  const int64_t sn = src->strides[dim];
  TSB_CHECK(numel(result) == outer * inner, "argmax: result must have the reduced dimension of size 1");
  cudaStream_t s = pick_stream(st, stream);
  const int64_t work = outer * inner;
  const int g = (int)(work < (int64_t)st->sm_count * 8 ? work : (int64_t)st->sm_count * 8);
#define TSB_AM(T, TO) argmax_kernel<T, TO><<<g, 256, 0, s>>>((TO*)result->data, (const T*)src->data, outer, n, inner, so, sn, si)
  if (src->dtype == TSB200_F32 && result->dtype == TSB200_F32) TSB_AM(float, float);
  else if (src->dtype == TSB200_F32 && result->dtype == TSB200_I32) TSB_AM(float, int);
  else if (src->dtype == TSB200_F16 && result->dtype == TSB200_F16) TSB_AM(__half, __half);
  else if (src->dtype == TSB200_F16 && result->dtype == TSB200_F32) TSB_AM(__half, float);
  else if (src->dtype == TSB200_F16 && result->dtype == TSB200_I32) TSB_AM(__half, int);
  else TSB_FAIL("argmax: unsupported dtypes src=%d result=%d", src->dtype, result->dtype);
#undef TSB_AM
  count_launch(device);
  return check_launch("argmax");
}

int TSB200_SoftmaxArgmax(int device, int32_t* out_ids, float* probs_out, const float* logits, int B, int V,
                         float temperature, const int32_t* blocked, int n_blocked, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(logits && (out_ids || probs_out), "softmax_argmax: null pointer");
  TSB_CHECK(B >= 0 && V > 0, "softmax_argmax: bad shape");
  TSB_CHECK(n_blocked == 0 || blocked, "softmax_argmax: blocked list is null");
  return launch_softmax_argmax(device, st, out_ids, probs_out, logits, B, V, temperature, temperature != 1.0f ? 1 : 0,
                               blocked, n_blocked, pick_stream(st, stream));
}

int64_t TSB200_TopPWorkspaceBytes(int rows, int V) { return (int64_t)rows * V * 5 * 4; }

int TSB200_TopPSample(int device, int32_t* out, const float* probs, int rows, int V, float topP, float repeatPenalty,
                      const int32_t* history, const int32_t* history_len, int history_stride, const float* u,
                      void* workspace, int64_t workspace_bytes, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(out && probs && u && workspace, "topp: null pointer");
  TSB_CHECK(rows >= 0 && V > 0, "topp: bad shape");
  TSB_CHECK(workspace_bytes >= TSB200_TopPWorkspaceBytes(rows, V), "topp: workspace too small (%lld < %lld)",
            (long long)workspace_bytes, (long long)TSB200_TopPWorkspaceBytes(rows, V));
  TSB_CHECK(!history || history_len, "topp: history given without history_len");
  return launch_topp(device, st, out, probs, rows, V, topP, repeatPenalty, history, history_len, history_stride, u,
                     workspace, pick_stream(st, stream));
}

int TSB200_PhiloxUniform(int device, float* u, int n, uint64_t seed, uint64_t seq_first, uint32_t step, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(u && n >= 0, "philox: bad arguments");
  return launch_philox(device, u, n, seed, seq_first, step, nullptr, pick_stream(st, stream));
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------ Top-P without any allocation
// Scratch for TSB200_TopPSampleStatic: a fixed block of device memory that is part of the library image.  Every GPU
// that loads the library holds these 5 MiB until the process exits.
namespace tsb {
constexpr int64_t kStaticToppBytes = 4LL * 65536 * 20;  // up to rows * V = 262144 probabilities per call (5 x uint32 each)
static __device__ __align__(256) unsigned char g_topp_static_scratch[kStaticToppBytes];
// Host code must not hand `g_topp_static_scratch` itself to a kernel: on the host that name is only a stand-in for the
// symbol.  The real device address is looked up once per device, with that device current, and cached here.
static void* g_topp_static_addr[kMaxDevices] = {};
static std::mutex g_topp_static_mu;  // two host threads may make the first call on one device at the same time

static int topp_static_setup(int device) {
  std::lock_guard<std::mutex> lk(g_topp_static_mu);
  if (g_topp_static_addr[device]) return 1;
  void* p = nullptr;
  TSB_CUDA(cudaGetSymbolAddress(&p, g_topp_static_scratch));
  TSB_CHECK(p != nullptr, "topp_static: the scratch symbol has no device address");
  TSB_TRY(init_topp_attrs(device));
  g_topp_static_addr[device] = p;
  return 1;
}
}  // namespace tsb

extern "C" int TSB200_TopPSampleStatic(int device, int32_t* out, const float* probs, int rows, int V, float topP,
                                        float repeatPenalty, const int32_t* history, const int32_t* history_len,
                                        int history_stride, const float* u, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(out && probs && u, "topp_static: null pointer");
  TSB_CHECK(rows >= 0 && V > 0, "topp_static: bad shape");
  TSB_CHECK(!history || history_len, "topp_static: history given without history_len");
  const int64_t need = TSB200_TopPWorkspaceBytes(rows, V);
  TSB_CHECK(need <= kStaticToppBytes,
            "topp_static: rows*V = %lld exceeds the built-in scratch (at most %lld probabilities per call); use "
            "TSB200_TopPSample with a caller-provided workspace", (long long)rows * V, (long long)(kStaticToppBytes / 20));
  TSB_TRY(topp_static_setup(device));  // first call on this device: address lookup + kernel attribute, no allocation
  return launch_topp(device, st, out, probs, rows, V, topP, repeatPenalty, history, history_len, history_stride, u,
                     g_topp_static_addr[device], pick_stream(st, stream));
}
