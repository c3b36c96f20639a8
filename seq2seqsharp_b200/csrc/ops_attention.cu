// RoPE, fused RoPE + KV-cache append, split-K flash-decode attention and causal prefill attention.
//
// Cache layout (this backend's own, laid out for streaming): K and V are both [B, Hkv, Tmax, hd], token-major,
// un-expanded for GQA — the reference materialises K as [B*H, hd, T] and V as [B*H, T, hd] with the KV heads
// repeated H/Hkv times and re-copies the whole cache every step (Seq2SeqSharp/Layers/GroupQueryAttention.cs:156-188,
// TensorSharp/Core/TensorConcatenation.cs:9-45).  Query head h reads KV head h / (H/Hkv).
//
// RoPE follows TensorSharp/TensorApplyCPU.cs:1148-1178 (same math as TensorSharp.CUDA/DeviceCode/
// AdvFuncKernels.cs:1245-1279 without fast-math): interleaved pairs (2i, 2i+1), theta_i = base^(-2i/hd) rounded to
// float, angle = theta_i * position in float, cos/sin evaluated in double and rounded to float.
#include <cstdlib>

#include "kernels.cuh"

namespace tsb {

TSB_CHECKED_WORD(attention)
#ifndef TSB200_CHECKED
int chk_take_attention() { return 0; }
#endif

__device__ __forceinline__ void rope_cs(int i, int cols, int m, double base, float& c, float& s) {
  const float theta = (float)pow(base, -2.0 * i / cols);
  const float tm = theta * (float)m;
  c = (float)cos((double)tm);
  s = (float)sin((double)tm);
}

// Unfused "rope": rows flattened [.., seqLen], position = (row % seqLen) + rowOffset.
template <typename T>
__global__ void rope_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t rows, int cols, int seqLen, int rowOffset,
                            double base) {
  const int64_t pairs = rows * (cols / 2);
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < pairs; p += (int64_t)gridDim.x * blockDim.x) {
    const int64_t j = p / (cols / 2);
    const int i = (int)(p % (cols / 2));
    const int m = (int)(j % seqLen) + rowOffset;
    float c, s;
    rope_cs(i, cols, m, base, c, s);
    const float a = to_f<T>(in[j * cols + 2 * i]), b = to_f<T>(in[j * cols + 2 * i + 1]);
    out[j * cols + 2 * i] = from_f<T>(a * c - b * s);
    out[j * cols + 2 * i + 1] = from_f<T>(b * c + a * s);
  }
}

// cos/sin table [Tmax, hd/2] (float2) built once per model so the decode path does no transcendental work.
__global__ void rope_table_kernel(float2* __restrict__ tab, int Tmax, int hd, double base) {
  const int64_t n = (int64_t)Tmax * (hd / 2);
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += (int64_t)gridDim.x * blockDim.x) {
    const int m = (int)(p / (hd / 2)), i = (int)(p % (hd / 2));
    float c, s;
    rope_cs(i, hd, m, base, c, s);
    tab[p] = make_float2(c, s);
  }
}

// q [B,S,H,hd] rotated in place; k rotated and stored with v into the cache at positions T0 + s.
// One thread per pair.  tab may be NULL (then cos/sin are evaluated here).
template <typename T>
__global__ void rope_append_kernel(T* q, const T* k, const T* v, int64_t q_rs,
                                   int64_t kv_rs, T* cK, T* cV, int B, int S, int H, int Hkv, int hd,
                                   int T0_arg, const int* dT0, int Tmax, int use_rope, double base,
                                   const float2* tab) {
  pdl_trigger();
  pdl_wait();
  const int hp = hd / 2;
  const int64_t per_row = (int64_t)(H + 2 * Hkv) * hp;
  const int64_t n = (int64_t)B * S * per_row;
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = p / per_row;  // b*S + s
    int rem = (int)(p % per_row);
    const int b = (int)(row / S), s = (int)(row % S);
    const int T0 = state_len(dT0, b, T0_arg);  // the engine keeps the cache lengths on the device so one CUDA graph serves every step
    const int pos = T0 + s;
    TSB_DEV_CHECK(attention, pos >= 0 && pos < Tmax, 0x201, (void)0)   // append position outside the cache (row skipped)
    if (pos >= Tmax) continue;  // capacity is checked on the host; never write past the cache
    const int head = rem / hp, i = rem % hp;
    float c = 1.0f, sn = 0.0f;
    if (use_rope && head < H + Hkv) {
      if (tab) {
        const float2 cs = tab[(int64_t)pos * hp + i];
        c = cs.x;
        sn = cs.y;
      } else {
        rope_cs(i, hd, pos, base, c, sn);
      }
    }
    if (head < H) {
      T* qp = q + row * q_rs + (int64_t)head * hd + 2 * i;
      const float a = to_f<T>(qp[0]), bb = to_f<T>(qp[1]);
      if (use_rope) {
        qp[0] = from_f<T>(a * c - bb * sn);
        qp[1] = from_f<T>(bb * c + a * sn);
      }
    } else if (head < H + Hkv) {
      const int g = head - H;
      const T* kp = k + row * kv_rs + (int64_t)g * hd + 2 * i;
      const float a = to_f<T>(kp[0]), bb = to_f<T>(kp[1]);
      T* dst = cK + (((int64_t)b * Hkv + g) * Tmax + pos) * hd + 2 * i;
      dst[0] = from_f<T>(use_rope ? a * c - bb * sn : a);
      dst[1] = from_f<T>(use_rope ? bb * c + a * sn : bb);
    } else {
      const int g = head - H - Hkv;
      const T* vp = v + row * kv_rs + (int64_t)g * hd + 2 * i;
      T* dst = cV + (((int64_t)b * Hkv + g) * Tmax + pos) * hd + 2 * i;
      dst[0] = vp[0];
      dst[1] = vp[1];
    }
  }
}

// ------------------------------------------------------------------------------------------------ attention
// One CTA handles one (sequence b, query position s, group of G query heads sharing a KV head, split of the key
// range).  Lanes are grouped LPT = hd*sizeof(T)/16 per cached token, each lane owning 16 bytes (EPL elements) of
// the K row and the V row, so every load is a 128-bit coalesced read and K/V are read exactly once for all G
// heads.  Each lane group runs an online softmax over its own token subsequence; the partial (max, sum, acc)
// states are merged through shared memory, and across splits by attn_combine_kernel.
// Scores: (q . k) * (1/sqrt(hd)) in fp32; softmax in fp32; P.V accumulated in fp32
// (the reference promotes Q and K to fp32 for the scores as well: MultiHeadAttention.cs:203-221).
template <typename T> struct Vec16;
template <> struct Vec16<__half> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ void load(const __half* p) { raw = *reinterpret_cast<const uint4*>(p); }
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
template <> struct Vec16<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void get(float* f) const {
    f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w;
  }
};

constexpr int kAttnThreads = 128;

template <typename T, int G>
__global__ void __launch_bounds__(kAttnThreads) attn_kernel(T* out, float* part,
                                                            const T* q, int64_t q_rs,
                                                            const T* cK, const T* cV, int S, int H,
                                                            int Hkv, int hd, int T0_arg, const int* dT0, int Tmax,
                                                            int splits, float scale) {
  constexpr int EPL = Vec16<T>::N;
  pdl_trigger();
  pdl_wait();
  const int T0 = state_len(dT0, (int)blockIdx.z / S, T0_arg);
  const int lpt = hd / EPL;              // lanes per token (power of two, <= 32)
  const int tpw = 32 / lpt;              // tokens per warp iteration
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int sub = lane / lpt, li = lane % lpt;
  const int nwarps = kAttnThreads / 32;
  const int split = blockIdx.x;
  const int groups_per_kv = (H / Hkv) / G;
  const int kvh = blockIdx.y / groups_per_kv;
  const int h0 = kvh * (H / Hkv) + (blockIdx.y % groups_per_kv) * G;
  const int row = blockIdx.z;  // b*S + s
  const int b = row / S, s = row % S;
  const int Tk = min(T0 + s + 1, Tmax);  // causal: keys 0 .. T0+s
  const int per_split = (Tk + splits - 1) / splits;
  const int t_beg = split * per_split, t_end = min(Tk, t_beg + per_split);

  float qf[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    Vec16<T> qv;
    qv.load(q + (int64_t)row * q_rs + (int64_t)(h0 + g) * hd + li * EPL);
    qv.get(qf[g]);
#pragma unroll
    for (int e = 0; e < EPL; ++e) qf[g][e] *= scale;
  }
  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.0f;
  }
  const T* Kb = cK + ((int64_t)b * Hkv + kvh) * Tmax * hd + li * EPL;
  const T* Vb = cV + ((int64_t)b * Hkv + kvh) * Tmax * hd + li * EPL;
  const int stride = nwarps * tpw;
  for (int tb = t_beg + w * tpw; tb < t_end; tb += stride) {
    // all lanes of the warp iterate together (shuffles below need full participation); `live` masks the tail
    const int t = tb + sub;
    const bool live = t < t_end;
    float kf[EPL], vf[EPL];
    if (live) {
      Vec16<T> kv, vv;
      kv.load(Kb + (int64_t)t * hd);
      vv.load(Vb + (int64_t)t * hd);
      kv.get(kf);
      vv.get(vf);
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) kf[e] = vf[e] = 0.0f;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float d = 0.0f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) d += qf[g][e] * kf[e];
      for (int o = lpt >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (live) {
        const float mn = fmaxf(m[g], d);
        const float corr = __expf(m[g] - mn);  // exp(-inf) = 0 on the first token
        const float p = __expf(d - mn);
        l[g] = l[g] * corr + p;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * corr + p * vf[e];
        m[g] = mn;
      }
    }
  }
  // merge the nwarps*tpw lane-group states through shared memory
  extern __shared__ float sm[];  // [nstates][G][hd + 2]
  const int nstates = nwarps * tpw;
  const int st = w * tpw + sub;
  const int rec = hd + 2;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float* r = sm + ((int64_t)st * G + g) * rec;
    if (li == 0) {
      r[0] = m[g];
      r[1] = l[g];
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) r[2 + li * EPL + e] = acc[g][e];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * hd; idx += kAttnThreads) {
    const int g = idx / hd, e = idx % hd;
    float mx = -INFINITY;
    for (int i = 0; i < nstates; ++i) mx = fmaxf(mx, sm[((int64_t)i * G + g) * rec]);
    float L = 0.0f, A = 0.0f;
    for (int i = 0; i < nstates; ++i) {
      const float* r = sm + ((int64_t)i * G + g) * rec;
      const float c = (r[0] == -INFINITY) ? 0.0f : __expf(r[0] - mx);
      L += r[1] * c;
      A += r[2 + e] * c;
    }
    const int h = h0 + g;
    if (splits == 1) {
      out[((int64_t)row * H + h) * hd + e] = from_f<T>(L > 0.0f ? A / L : 0.0f);
    } else {
      float* pr = part + (((int64_t)row * H + h) * splits + split) * rec;
      if (e == 0) {
        pr[0] = mx;
        pr[1] = L;
      }
      pr[2 + e] = A;
    }
  }
}

// Decode variant (one query position per sequence) with the cached K/V rows staged through shared memory by
// cp.async: three stages of kStageTokens tokens are in flight per CTA and several CTAs fit on an SM, so ~150 KB per SM
// are outstanding instead of the two 16-byte loads per lane of attn_kernel — at large batch the cache read is bound
// by memory latency x bytes in flight, not by arithmetic.  Same arithmetic and the same merge as attn_kernel.
constexpr int kStageTokens = 32;
constexpr int kAttnStages = 3;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T, int G>
__global__ void __launch_bounds__(kAttnThreads) attn_staged_kernel(T* out, float* part, const T* q, int64_t q_rs, const T* cK,
                                                                   const T* cV, int H, int Hkv, int hd, int T0_arg, const int* dT0,
                                                                   int Tmax, int splits, float scale) {
  constexpr int EPL = Vec16<T>::N;
  extern __shared__ __align__(16) unsigned char attn_smem[];
  pdl_trigger();
  pdl_wait();
  const int T0 = state_len(dT0, (int)blockIdx.z, T0_arg);
  const int lpt = hd / EPL;              // lanes per token (power of two, <= 32)
  const int tpw = 32 / lpt;              // tokens per warp pass
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int sub = lane / lpt, li = lane % lpt;
  const int nwarps = kAttnThreads / 32;
  const int split = blockIdx.x;
  const int groups_per_kv = (H / Hkv) / G;
  const int kvh = blockIdx.y / groups_per_kv;
  const int h0 = kvh * (H / Hkv) + (blockIdx.y % groups_per_kv) * G;
  const int row = blockIdx.z;  // sequence
  const int Tk = min(T0 + 1, Tmax);
  const int per_split = (Tk + splits - 1) / splits;
  const int t_beg = split * per_split, t_end = min(Tk, t_beg + per_split);
  const size_t row_bytes = (size_t)hd * sizeof(T);
  const size_t stage_bytes = 2 * kStageTokens * row_bytes;   // K rows then V rows
  const T* Kb = cK + ((int64_t)row * Hkv + kvh) * Tmax * hd;
  const T* Vb = cV + ((int64_t)row * Hkv + kvh) * Tmax * hd;
  const int n_tiles = (max(t_end - t_beg, 0) + kStageTokens - 1) / kStageTokens;
  const int vec_per_row = hd / EPL;                           // 16-byte vectors per row
  const int vec_per_tile = kStageTokens * vec_per_row;

  auto issue = [&](int tile) {
    if (tile < n_tiles) {
      unsigned char* st = attn_smem + (size_t)(tile % kAttnStages) * stage_bytes;
      const int t0 = t_beg + tile * kStageTokens;
      for (int v = threadIdx.x; v < vec_per_tile; v += kAttnThreads) {
        const int tt = v / vec_per_row, c = v % vec_per_row;
        const int t = min(t0 + tt, t_end - 1);  // the tail re-reads the last token of the range; it is masked below
        cp_async_16(st + (size_t)tt * row_bytes + c * 16, Kb + (int64_t)t * hd + c * EPL);
        cp_async_16(st + (size_t)(kStageTokens + tt) * row_bytes + c * 16, Vb + (int64_t)t * hd + c * EPL);
      }
    }
    cp_async_commit();
  };
  for (int i = 0; i < kAttnStages - 1; ++i) issue(i);

  float qf[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    Vec16<T> qv;
    qv.load(q + (int64_t)row * q_rs + (int64_t)(h0 + g) * hd + li * EPL);
    qv.get(qf[g]);
#pragma unroll
    for (int e = 0; e < EPL; ++e) qf[g][e] *= scale;
  }
  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.0f;
  }
  for (int tile = 0; tile < n_tiles; ++tile) {
    issue(tile + kAttnStages - 1);
    cp_async_wait<kAttnStages - 1>();
    __syncthreads();
    const unsigned char* st = attn_smem + (size_t)(tile % kAttnStages) * stage_bytes;
    const int t0 = t_beg + tile * kStageTokens;
    for (int tt = w * tpw + sub; tt < kStageTokens; tt += nwarps * tpw) {
      const bool live = t0 + tt < t_end;  // uniform trip count: kStageTokens is a multiple of nwarps * tpw
      Vec16<T> kv, vv;
      kv.load(reinterpret_cast<const T*>(st + (size_t)tt * row_bytes) + li * EPL);
      vv.load(reinterpret_cast<const T*>(st + (size_t)(kStageTokens + tt) * row_bytes) + li * EPL);
      float kf[EPL], vf[EPL];
      kv.get(kf);
      vv.get(vf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) d += qf[g][e] * kf[e];
        for (int o = lpt >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (live) {
          const float mn = fmaxf(m[g], d);
          const float corr = __expf(m[g] - mn);  // exp(-inf) = 0 on the first token
          const float p = __expf(d - mn);
          l[g] = l[g] * corr + p;
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * corr + p * vf[e];
          m[g] = mn;
        }
      }
    }
    __syncthreads();  // the stage is overwritten by the copy issued in the next iteration
  }
  cp_async_wait<0>();
  __syncthreads();
  // merge the nwarps*tpw lane-group states through shared memory (the stage area is free now)
  float* sm = reinterpret_cast<float*>(attn_smem);  // [nstates][G][hd + 2]
  const int nstates = nwarps * tpw;
  const int stt = w * tpw + sub;
  const int rec = hd + 2;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float* r = sm + ((int64_t)stt * G + g) * rec;
    if (li == 0) {
      r[0] = m[g];
      r[1] = l[g];
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) r[2 + li * EPL + e] = acc[g][e];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * hd; idx += kAttnThreads) {
    const int g = idx / hd, e = idx % hd;
    float mx = -INFINITY;
    for (int i = 0; i < nstates; ++i) mx = fmaxf(mx, sm[((int64_t)i * G + g) * rec]);
    float L = 0.0f, A = 0.0f;
    for (int i = 0; i < nstates; ++i) {
      const float* r = sm + ((int64_t)i * G + g) * rec;
      const float c = (r[0] == -INFINITY) ? 0.0f : __expf(r[0] - mx);
      L += r[1] * c;
      A += r[2 + e] * c;
    }
    const int h = h0 + g;
    if (splits == 1) {
      out[((int64_t)row * H + h) * hd + e] = from_f<T>(L > 0.0f ? A / L : 0.0f);
    } else {
      float* pr = part + (((int64_t)row * H + h) * splits + split) * rec;
      if (e == 0) {
        pr[0] = mx;
        pr[1] = L;
      }
      pr[2 + e] = A;
    }
  }
}

// Decode attention on the warp-level tensor cores (fp16, head_dim 64 or 128, up to 8 query heads per KV head), for
// large batches: one CTA = (sequence, KV head, split of the key range), the query heads of the group are the rows of
// the m16n8k16 A operand (rows beyond the group are zero), so K and V are read once for the whole group and a 16-token
// slice costs a warp 2*(hd/16) + hd/8 mma instructions instead of ~60 shuffle/FMA instructions per token.
//   S = Q K^T : A = Q fragments held in registers, B = K rows staged in shared memory (ldmatrix);
//   online softmax per 16-token slice in fp32 (scores scaled by 1/sqrt(hd) after the product, as the reference does);
//   O += P V  : A = P rounded to fp16, taken straight from the S accumulator fragments, B = V rows (ldmatrix.trans).
// K/V rows are staged by cp.async, 64 tokens per stage, three stages in flight; every 16-byte chunk is stored at
// chunk ^ (row & 7) so that the ldmatrix row reads are bank-conflict free.  Each warp owns 16 tokens of a stage and its
// own (max, sum, O) state; the four states are merged like the lane-group states of attn_kernel.
constexpr int kMmaStageTokens = 64;
constexpr int kMmaStages = 3;

__device__ __forceinline__ void at_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void at_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void at_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int HD>
__global__ void __launch_bounds__(kAttnThreads) attn_mma_kernel(__half* out, float* part, const __half* q, int64_t q_rs,
                                                                const __half* cK, const __half* cV, int H, int Hkv, int T0_arg,
                                                                const int* dT0, int Tmax, int splits, float scale) {
  constexpr int RB = HD * 2;            // bytes per row
  constexpr int CPR = RB / 16;          // 16-byte chunks per row
  constexpr int KS = HD / 16;           // k steps of Q K^T
  constexpr int NBO = HD / 8;           // n blocks of O
  extern __shared__ __align__(128) unsigned char attn_smem[];
  pdl_trigger();
  pdl_wait();
  const int T0 = state_len(dT0, (int)blockIdx.z, T0_arg);
  TSB_DEV_CHECK(attention, T0 >= 0 && T0 < Tmax, 0x202, (void)0)   // cache length beyond the capacity (keys are clamped to Tmax below)
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int G = H / Hkv;                // query heads per KV head (<= 8)
  const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
  const int h0 = kvh * G;
  const int Tk = min(T0 + 1, Tmax);
  const int per_split = (Tk + splits - 1) / splits;
  const int t_beg = split * per_split, t_end = min(Tk, t_beg + per_split);
  const size_t stage_bytes = 2 * (size_t)kMmaStageTokens * RB;
  const __half* Kb = cK + ((int64_t)row * Hkv + kvh) * Tmax * HD;
  const __half* Vb = cV + ((int64_t)row * Hkv + kvh) * Tmax * HD;
  const int n_tiles = (max(t_end - t_beg, 0) + kMmaStageTokens - 1) / kMmaStageTokens;

  auto issue = [&](int tile) {
    if (tile < n_tiles) {
      unsigned char* st = attn_smem + (size_t)(tile % kMmaStages) * stage_bytes;
      const int t0 = t_beg + tile * kMmaStageTokens;
      for (int v = threadIdx.x; v < kMmaStageTokens * CPR; v += kAttnThreads) {
        const int tt = v / CPR, c = v % CPR;
        const int t = min(t0 + tt, t_end - 1);  // the tail re-reads the last token of the range; its scores are masked
        const int pc = (c ^ (tt & 7)) * 16;
        cp_async_16(st + (size_t)tt * RB + pc, Kb + (int64_t)t * HD + c * 8);
        cp_async_16(st + (size_t)(kMmaStageTokens + tt) * RB + pc, Vb + (int64_t)t * HD + c * 8);
      }
    }
    cp_async_commit();
  };
  for (int i = 0; i < kMmaStages - 1; ++i) issue(i);

  // Q fragments: row g8 = head h0 + g8 (zero rows beyond the group), a0 = k 2*t4.., a2 = k 8 + 2*t4..
  uint32_t qa[KS][2];
  {
    const bool live = g8 < G;
    const __half* qp = q + (int64_t)row * q_rs + (int64_t)(h0 + (live ? g8 : 0)) * HD + 2 * t4;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qa[ks][0] = live ? *reinterpret_cast<const uint32_t*>(qp + ks * 16) : 0u;
      qa[ks][1] = live ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8) : 0u;
    }
  }
  float m_run = -INFINITY, l_run = 0.0f;   // state of head g8 (this lane's part of the row sum)
  float o[NBO][4];
#pragma unroll
  for (int nb = 0; nb < NBO; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nb][e] = 0.0f;

  for (int tile = 0; tile < n_tiles; ++tile) {
    issue(tile + kMmaStages - 1);
    cp_async_wait<kMmaStages - 1>();
    __syncthreads();
    const uint32_t kbase = (uint32_t)__cvta_generic_to_shared(attn_smem + (size_t)(tile % kMmaStages) * stage_bytes);
    const uint32_t vbase = kbase + kMmaStageTokens * RB;
    const int tw = w * 16;                                   // this warp's 16 tokens of the stage
    const int t_first = t_beg + tile * kMmaStageTokens + tw;
    if (t_first < t_end) {
      // ---- S = Q K^T for two 8-token blocks
      float sc[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[nb][e] = 0.0f;
        const int r = tw + nb * 8 + (lane & 7);
#pragma unroll
        for (int kp = 0; kp < KS / 2; ++kp) {
          uint32_t b0, b1, b2, b3;
          const int c = kp * 4 + (lane >> 3);
          at_ldmatrix_x4(kbase + r * RB + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
          at_mma(sc[nb], qa[2 * kp][0], 0u, qa[2 * kp][1], 0u, b0, b1);
          at_mma(sc[nb], qa[2 * kp + 1][0], 0u, qa[2 * kp + 1][1], 0u, b2, b3);
        }
      }
      // ---- online softmax of row g8 over these 16 tokens (this lane: tokens nb*8 + 2*t4, +1)
      float mx = -INFINITY;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int t = t_first + nb * 8 + 2 * t4 + e;
          sc[nb][e] = (t < t_end) ? sc[nb][e] * scale : -INFINITY;
          mx = fmaxf(mx, sc[nb][e]);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);   // finite: the slice has at least one valid token
      const float corr = __expf(m_run - m_new);
      float p[2][2];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          p[nb][e] = __expf(sc[nb][e] - m_new);
          l_run = (nb == 0 && e == 0) ? l_run * corr + p[nb][e] : l_run + p[nb][e];
        }
      m_run = m_new;
      // P as the A operand of the second product (rows beyond the group stay zero)
      __half2 h0p = __floats2half2_rn(p[0][0], p[0][1]), h1p = __floats2half2_rn(p[1][0], p[1][1]);
      const uint32_t pa0 = *reinterpret_cast<uint32_t*>(&h0p), pa2 = *reinterpret_cast<uint32_t*>(&h1p);
      // ---- O = O * corr + P V
      const int vr = tw + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int np = 0; np < NBO / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        const int c = np * 2 + (lane >> 4);
        at_ldmatrix_x4_trans(vbase + vr * RB + ((c ^ (vr & 7)) << 4), b0, b1, b2, b3);
        o[2 * np][0] *= corr; o[2 * np][1] *= corr;
        o[2 * np + 1][0] *= corr; o[2 * np + 1][1] *= corr;
        at_mma(o[2 * np], pa0, 0u, pa2, 0u, b0, b1);
        at_mma(o[2 * np + 1], pa0, 0u, pa2, 0u, b2, b3);
      }
    }
    __syncthreads();  // the stage is overwritten by the copy issued in the next iteration
  }
  cp_async_wait<0>();
  __syncthreads();
  // this lane's part of the row sum -> whole row
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  // merge the four warp states through shared memory: [warp][head][hd + 2]
  float* sm = reinterpret_cast<float*>(attn_smem);
  const int rec = HD + 2;
  if (g8 < G) {
    float* r = sm + ((int64_t)w * G + g8) * rec;
    if (t4 == 0) {
      r[0] = m_run;
      r[1] = l_run;
    }
#pragma unroll
    for (int nb = 0; nb < NBO; ++nb) {
      r[2 + nb * 8 + 2 * t4] = o[nb][0];
      r[2 + nb * 8 + 2 * t4 + 1] = o[nb][1];
    }
  }
  __syncthreads();
  const int nstates = kAttnThreads / 32;
  for (int idx = threadIdx.x; idx < G * HD; idx += kAttnThreads) {
    const int g = idx / HD, e = idx % HD;
    float mx = -INFINITY;
    for (int i = 0; i < nstates; ++i) mx = fmaxf(mx, sm[((int64_t)i * G + g) * rec]);
    float L = 0.0f, A = 0.0f;
    for (int i = 0; i < nstates; ++i) {
      const float* r = sm + ((int64_t)i * G + g) * rec;
      const float c = (r[0] == -INFINITY) ? 0.0f : __expf(r[0] - mx);
      L += r[1] * c;
      A += r[2 + e] * c;
    }
    const int h = h0 + g;
    if (splits == 1) {
      out[((int64_t)row * H + h) * HD + e] = __float2half_rn(L > 0.0f ? A / L : 0.0f);
    } else {
      float* pr = part + (((int64_t)row * H + h) * splits + split) * rec;
      if (e == 0) {
        pr[0] = mx;
        pr[1] = L;
      }
      pr[2 + e] = A;
    }
  }
}

// Causal prefill attention on the warp-level tensor cores (fp16, head_dim 64 / 128, 1, 2, 4 or 8 query heads per KV
// head).  One CTA = (sequence, KV head, tile of 64 / G query positions): its 64 rows are the (query, head) pairs of
// the tile, 16 per warp, so the K/V rows of the tile's key range are staged once (cp.async, 64 tokens per stage,
// chunk-XOR swizzle) for all heads of the group and all queries of the tile — the one-CTA-per-query kernel re-read
// the whole prefix for every query.  Per 16-key slice a warp does S = Q K^T (mma.sync), the causal mask, an online
// softmax in fp32 for its 16 rows and O += P V (mma.sync); slices beyond the warp's last query are skipped.
template <int HD>
__global__ void __launch_bounds__(kAttnThreads) attn_prefill_mma_kernel(__half* out, const __half* q, int64_t q_rs, const __half* cK,
                                                                        const __half* cV, int S, int H, int Hkv, int T0_arg,
                                                                        const int* dT0, int Tmax, float scale) {
  constexpr int RB = HD * 2, CPR = RB / 16, KS = HD / 16, NBO = HD / 8;
  extern __shared__ __align__(128) unsigned char attn_smem[];
  pdl_trigger();
  pdl_wait();
  const int T0 = state_len(dT0, (int)blockIdx.z, T0_arg);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int G = H / Hkv;                       // 1, 2, 4 or 8
  const int QT = 64 / G;                       // query positions per CTA
  const int q0 = blockIdx.x * QT, kvh = blockIdx.y, b = blockIdx.z;
  const int h0 = kvh * G;
  // this lane's two rows: (query, head) pairs r0 and r0 + 8 of the CTA's 64
  const int rA = w * 16 + g8, rB = rA + 8;
  const int qiA = rA / G, gA = rA % G, qiB = rB / G, gB = rB % G;
  const int sA = q0 + qiA, sB = q0 + qiB;      // query positions (may be >= S in the last tile)
  const bool liveA = sA < S, liveB = sB < S;
  const int q_last_cta = min(S, q0 + QT) - 1;  // last live query of the tile
  const int n_keys = min(T0 + q_last_cta + 1, Tmax);
  const int w_last_q = min(S - 1, q0 + (w * 16 + 15) / G);   // last query of this warp
  const int w_keys = min(T0 + w_last_q + 1, Tmax);           // keys this warp needs
  const size_t stage_bytes = 2 * (size_t)kMmaStageTokens * RB;
  const __half* Kb = cK + ((int64_t)b * Hkv + kvh) * Tmax * HD;
  const __half* Vb = cV + ((int64_t)b * Hkv + kvh) * Tmax * HD;
  const int n_tiles = (max(n_keys, 0) + kMmaStageTokens - 1) / kMmaStageTokens;

  auto issue = [&](int tile) {
    if (tile < n_tiles) {
      unsigned char* st = attn_smem + (size_t)(tile % kMmaStages) * stage_bytes;
      const int t0 = tile * kMmaStageTokens;
      for (int v = threadIdx.x; v < kMmaStageTokens * CPR; v += kAttnThreads) {
        const int tt = v / CPR, c = v % CPR;
        const int t = min(t0 + tt, n_keys - 1);
        const int pc = (c ^ (tt & 7)) * 16;
        cp_async_16(st + (size_t)tt * RB + pc, Kb + (int64_t)t * HD + c * 8);
        cp_async_16(st + (size_t)(kMmaStageTokens + tt) * RB + pc, Vb + (int64_t)t * HD + c * 8);
      }
    }
    cp_async_commit();
  };
  for (int i = 0; i < kMmaStages - 1; ++i) issue(i);

  // Q fragments of the two rows: a0 / a2 = row A (k 2*t4.., 8 + 2*t4..), a1 / a3 = row B
  uint32_t qa[KS][4];
  {
    const __half* qpA = q + ((int64_t)b * S + (liveA ? sA : 0)) * q_rs + (int64_t)(h0 + gA) * HD + 2 * t4;
    const __half* qpB = q + ((int64_t)b * S + (liveB ? sB : 0)) * q_rs + (int64_t)(h0 + gB) * HD + 2 * t4;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qa[ks][0] = liveA ? *reinterpret_cast<const uint32_t*>(qpA + ks * 16) : 0u;
      qa[ks][1] = liveB ? *reinterpret_cast<const uint32_t*>(qpB + ks * 16) : 0u;
      qa[ks][2] = liveA ? *reinterpret_cast<const uint32_t*>(qpA + ks * 16 + 8) : 0u;
      qa[ks][3] = liveB ? *reinterpret_cast<const uint32_t*>(qpB + ks * 16 + 8) : 0u;
    }
  }
  const int limA = liveA ? min(T0 + sA + 1, Tmax) : 0, limB = liveB ? min(T0 + sB + 1, Tmax) : 0;  // keys [0, lim) are visible
  float mA = -INFINITY, mB = -INFINITY, lA = 0.0f, lB = 0.0f;
  float o[NBO][4];
#pragma unroll
  for (int nb = 0; nb < NBO; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nb][e] = 0.0f;

  for (int tile = 0; tile < n_tiles; ++tile) {
    issue(tile + kMmaStages - 1);
    cp_async_wait<kMmaStages - 1>();
    __syncthreads();
    const uint32_t kbase = (uint32_t)__cvta_generic_to_shared(attn_smem + (size_t)(tile % kMmaStages) * stage_bytes);
    const uint32_t vbase = kbase + kMmaStageTokens * RB;
#pragma unroll 1
    for (int sl = 0; sl < kMmaStageTokens / 16; ++sl) {
      const int tw = sl * 16;
      const int t_first = tile * kMmaStageTokens + tw;
      if (t_first >= w_keys) break;   // causal: nothing further in this stage is visible to this warp (warp-uniform)
      float sc[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[nb][e] = 0.0f;
        const int r = tw + nb * 8 + (lane & 7);
#pragma unroll
        for (int kp = 0; kp < KS / 2; ++kp) {
          uint32_t b0, b1, b2, b3;
          const int c = kp * 4 + (lane >> 3);
          at_ldmatrix_x4(kbase + r * RB + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
          at_mma(sc[nb], qa[2 * kp][0], qa[2 * kp][1], qa[2 * kp][2], qa[2 * kp][3], b0, b1);
          at_mma(sc[nb], qa[2 * kp + 1][0], qa[2 * kp + 1][1], qa[2 * kp + 1][2], qa[2 * kp + 1][3], b2, b3);
        }
      }
      // scale, causal mask, row maxima (row A: elements 0,1; row B: elements 2,3; keys nb*8 + 2*t4 + e)
      float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int t = t_first + nb * 8 + 2 * t4 + e;
          sc[nb][e] = (t < limA) ? sc[nb][e] * scale : -INFINITY;
          sc[nb][2 + e] = (t < limB) ? sc[nb][2 + e] * scale : -INFINITY;
          mxA = fmaxf(mxA, sc[nb][e]);
          mxB = fmaxf(mxB, sc[nb][2 + e]);
        }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      // a row may see none of these 16 keys: keep its state (no exp(-inf - -inf))
      const float mnA = fmaxf(mA, mxA), mnB = fmaxf(mB, mxB);
      const float corrA = (mnA == -INFINITY) ? 1.0f : __expf(mA - mnA), corrB = (mnB == -INFINITY) ? 1.0f : __expf(mB - mnB);
      float p[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          p[nb][e] = (mnA == -INFINITY) ? 0.0f : __expf(sc[nb][e] - mnA);
          p[nb][2 + e] = (mnB == -INFINITY) ? 0.0f : __expf(sc[nb][2 + e] - mnB);
        }
      lA = lA * corrA + (p[0][0] + p[0][1]) + (p[1][0] + p[1][1]);
      lB = lB * corrB + (p[0][2] + p[0][3]) + (p[1][2] + p[1][3]);
      mA = mnA;
      mB = mnB;
      __half2 hA0 = __floats2half2_rn(p[0][0], p[0][1]), hB0 = __floats2half2_rn(p[0][2], p[0][3]);
      __half2 hA1 = __floats2half2_rn(p[1][0], p[1][1]), hB1 = __floats2half2_rn(p[1][2], p[1][3]);
      const uint32_t pa0 = *reinterpret_cast<uint32_t*>(&hA0), pa1 = *reinterpret_cast<uint32_t*>(&hB0);
      const uint32_t pa2 = *reinterpret_cast<uint32_t*>(&hA1), pa3 = *reinterpret_cast<uint32_t*>(&hB1);
      const int vr = tw + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int np = 0; np < NBO / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        const int c = np * 2 + (lane >> 4);
        at_ldmatrix_x4_trans(vbase + vr * RB + ((c ^ (vr & 7)) << 4), b0, b1, b2, b3);
        o[2 * np][0] *= corrA; o[2 * np][1] *= corrA; o[2 * np][2] *= corrB; o[2 * np][3] *= corrB;
        o[2 * np + 1][0] *= corrA; o[2 * np + 1][1] *= corrA; o[2 * np + 1][2] *= corrB; o[2 * np + 1][3] *= corrB;
        at_mma(o[2 * np], pa0, pa1, pa2, pa3, b0, b1);
        at_mma(o[2 * np + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
    }
    __syncthreads();  // the stage is overwritten by the copy issued in the next iteration
  }
  cp_async_wait<0>();
  lA += __shfl_xor_sync(0xffffffffu, lA, 1);
  lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1);
  lB += __shfl_xor_sync(0xffffffffu, lB, 2);
  const float iA = lA > 0.0f ? 1.0f / lA : 0.0f, iB = lB > 0.0f ? 1.0f / lB : 0.0f;
  if (liveA) {
    __half* op = out + (((int64_t)b * S + sA) * H + h0 + gA) * HD + 2 * t4;
#pragma unroll
    for (int nb = 0; nb < NBO; ++nb) *reinterpret_cast<__half2*>(op + nb * 8) = __floats2half2_rn(o[nb][0] * iA, o[nb][1] * iA);
  }
  if (liveB) {
    __half* op = out + (((int64_t)b * S + sB) * H + h0 + gB) * HD + 2 * t4;
#pragma unroll
    for (int nb = 0; nb < NBO; ++nb) *reinterpret_cast<__half2*>(op + nb * 8) = __floats2half2_rn(o[nb][2] * iB, o[nb][3] * iB);
  }
}

template <typename T>
__global__ void attn_combine_kernel(T* out, const float* part, int hd, int splits) {
  pdl_trigger();
  pdl_wait();
  const int64_t rh = blockIdx.x;  // row*H + h
  const int rec = hd + 2;
  const float* p = part + rh * splits * rec;
  float mx = -INFINITY;
  for (int i = 0; i < splits; ++i) mx = fmaxf(mx, p[i * rec]);
  for (int e = threadIdx.x; e < hd; e += blockDim.x) {
    float L = 0.0f, A = 0.0f;
    for (int i = 0; i < splits; ++i) {
      const float c = (p[i * rec] == -INFINITY) ? 0.0f : __expf(p[i * rec] - mx);
      L += p[i * rec + 1] * c;
      A += p[i * rec + 2 + e] * c;
    }
    out[rh * hd + e] = from_f<T>(L > 0.0f ? A / L : 0.0f);
  }
}

static int pick_splits(DeviceState* st, int B, int Hkv_groups, int T, int min_keys = 32) {
  // enough CTAs to cover the SMs about twice, at least min_keys keys per split (a CTA of the shuffle / FMA kernels covers
  // 8..16 keys per iteration: 32; the tensor-core kernel stages 64 keys at a time: 128 - with 32 a 530-token context was cut
  // into 17..32 splits whose start-up and merge cost more than they gained: 7B-class, two sequences, 3.38 against 3.20 ms per step)
  const int64_t base = (int64_t)B * Hkv_groups;
  int s = (int)((2LL * st->sm_count + base - 1) / base);
  const int max_by_len = (T + min_keys - 1) / min_keys;
  if (s > max_by_len) s = max_by_len;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return s;
}

// fp16, head size 64 / 128, 1, 2, 4 or 8 query heads per KV head: the tensor-core flash-decode kernel serves the shape
static bool mma_decode_shape(int dtype, int H, int Hkv, int hd) {
  if (Hkv <= 0 || H % Hkv != 0) return false;
  const int group = H / Hkv;
  return dtype == TSB200_F16 && (hd == 64 || hd == 128) && (group == 1 || group == 2 || group == 4 || group == 8);
}

int64_t attn_workspace_bytes(int B, int H, int hd, int T) {
  (void)T;
  return (int64_t)B * H * 64 * (hd + 2) * sizeof(float);
}

template <typename T>
static int launch_attn_t(int device, DeviceState* st, T* out, const T* q, int64_t q_rs, const T* cK, const T* cV, int B, int S,
                         int H, int Hkv, int hd, int T0, const int* dT0, int Tmax, int splits_hint, float* ws, int64_t ws_bytes,
                         cudaStream_t s) {
  constexpr int EPL = Vec16<T>::N;
  const int lpt = hd / EPL;
  TSB_CHECK(hd % EPL == 0 && lpt >= 1 && lpt <= 32 && (lpt & (lpt - 1)) == 0,
            "attention: head_dim %d unsupported for this dtype (hd*sizeof(T)/16 must be a power of two <= 32)", hd);
  TSB_CHECK(H % Hkv == 0, "attention: H must be divisible by Hkv");
  TSB_CHECK(dT0 || T0 + S <= Tmax, "attention: cache capacity exceeded (%d + %d > %d)", T0, S, Tmax);
  TSB_CHECK(q_rs % EPL == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)cK % 16) == 0 && ((uintptr_t)cV % 16) == 0,
            "attention: pointers and row strides must be 16-byte aligned");
  const int group = H / Hkv;
  int G = 1;
  if (group % 8 == 0) G = 8;
  else if (group % 4 == 0) G = 4;
  else if (group % 2 == 0) G = 2;
  const int ygroups = Hkv * (group / G);
  const bool mma_shape = mma_decode_shape(sizeof(T) == 2 ? TSB200_F16 : TSB200_F32, H, Hkv, hd);
  int splits = (S == 1) ? (splits_hint > 0 ? splits_hint : pick_splits(st, B, ygroups, T0 + 1, mma_shape ? 256 : 32)) : 1;
  if (splits > 1) {
    const int64_t need = (int64_t)B * S * H * splits * (hd + 2) * sizeof(float);
    if (!ws || ws_bytes < need) splits = 1;
  }
  const int tpw = 32 / lpt;
  const size_t smem = (size_t)(kAttnThreads / 32) * tpw * G * (hd + 2) * sizeof(float);
  TSB_CHECK(smem <= 48 * 1024, "attention: shared memory need %zu exceeds 48 KB", smem);
  dim3 grid(splits, ygroups, B * S);
  const float scale = 1.0f / sqrtf((float)hd);
  // cached decode at batch: K/V rows staged through shared memory (cp.async), several tiles in flight per CTA
  static int staged = -1;
  if (staged < 0) {
    const char* e = getenv("TSB200_ATTN_STAGED");  // "0": register-only kernel for every case (A/B measurements)
    staged = (e && e[0] == '0') ? 0 : 1;
  }
  // fp16, head_dim 64 / 128, up to 8 query heads per KV head: scores and P V on the warp-level tensor cores
  static int use_mma = -1;
  if (use_mma < 0) {
    const char* e = getenv("TSB200_ATTN_MMA");  // "0": keep the shuffle/FMA kernels (A/B measurements)
    use_mma = (e && e[0] == '0') ? 0 : 1;
  }
  if constexpr (sizeof(T) == 2) {
    if (use_mma && S >= 16 && (hd == 64 || hd == 128) && (group == 1 || group == 2 || group == 4 || group == 8)) {
      // causal prefill on the tensor cores: K/V staged once per tile of 64 / group query positions
      const size_t sm3 = (size_t)kMmaStages * 2 * kMmaStageTokens * hd * 2;
      const int QT = 64 / group;
      dim3 g3((S + QT - 1) / QT, Hkv, B);
      static bool attr_done2[kMaxDevices] = {};
      if (!attr_done2[device]) {
        TSB_CUDA(cudaFuncSetAttribute(attn_prefill_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        TSB_CUDA(cudaFuncSetAttribute(attn_prefill_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        attr_done2[device] = true;
      }
      if (hd == 64)
        TSB_CUDA(launch_k(attn_prefill_mma_kernel<64>, g3, dim3(kAttnThreads), sm3, s, (__half*)out, (const __half*)q, q_rs, (const __half*)cK,
                          (const __half*)cV, S, H, Hkv, T0, dT0, Tmax, scale));
      else
        TSB_CUDA(launch_k(attn_prefill_mma_kernel<128>, g3, dim3(kAttnThreads), sm3, s, (__half*)out, (const __half*)q, q_rs, (const __half*)cK,
                          (const __half*)cV, S, H, Hkv, T0, dT0, Tmax, scale));
      count_launch(device);
      return check_launch("attention_prefill_mma");
    }
    // at every grid size (7B-class model, sequences of 530 tokens: faster than the shuffle / FMA kernels from 16 CTAs on)
    if (use_mma && staged && S == 1 && (hd == 64 || hd == 128) && group <= 8 && ygroups == Hkv) {
      const size_t sm3 = (size_t)kMmaStages * 2 * kMmaStageTokens * hd * 2;
      dim3 g3(splits, Hkv, B);
      static bool attr_done[kMaxDevices] = {};
      if (!attr_done[device]) {
        TSB_CUDA(cudaFuncSetAttribute(attn_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        TSB_CUDA(cudaFuncSetAttribute(attn_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        attr_done[device] = true;
      }
      if (hd == 64)
        TSB_CUDA(launch_k(attn_mma_kernel<64>, g3, dim3(kAttnThreads), sm3, s, (__half*)out, ws, (const __half*)q, q_rs, (const __half*)cK,
                          (const __half*)cV, H, Hkv, T0, dT0, Tmax, splits, scale));
      else
        TSB_CUDA(launch_k(attn_mma_kernel<128>, g3, dim3(kAttnThreads), sm3, s, (__half*)out, ws, (const __half*)q, q_rs, (const __half*)cK,
                          (const __half*)cV, H, Hkv, T0, dT0, Tmax, splits, scale));
      count_launch(device);
      TSB_TRY(check_launch("attention_mma"));
      if (splits > 1) {
        TSB_CUDA(launch_k(attn_combine_kernel<T>, dim3(B * S * H), dim3(hd < 128 ? 64 : 128), 0, s, out, (const float*)ws, hd, splits));
        count_launch(device);
        TSB_TRY(check_launch("attention_combine"));
      }
      return 1;
    }
  }
  const size_t stage_smem = (size_t)kAttnStages * 2 * kStageTokens * hd * sizeof(T);
  if (staged && S == 1 && kStageTokens % ((kAttnThreads / 32) * tpw) == 0 && B * ygroups * splits >= 2 * st->sm_count) {
    const size_t sm2 = stage_smem > smem ? stage_smem : smem;
    if (sm2 <= 96 * 1024) {
#define TSB_ATTN_S(GG)                                                                                                          \
  do {                                                                                                                          \
    static bool attr_done[kMaxDevices] = {};                                                                                    \
    if (!attr_done[device]) {                                                                                                   \
      TSB_CUDA(cudaFuncSetAttribute(attn_staged_kernel<T, GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));        \
      attr_done[device] = true;                                                                                                 \
    }                                                                                                                           \
    TSB_CUDA(launch_k(attn_staged_kernel<T, GG>, grid, dim3(kAttnThreads), sm2, s, out, ws, q, q_rs, cK, cV, H, Hkv, hd, T0, dT0, \
                      Tmax, splits, scale));                                                                                    \
  } while (0)
      switch (G) {
        case 8: TSB_ATTN_S(8); break;
        case 4: TSB_ATTN_S(4); break;
        case 2: TSB_ATTN_S(2); break;
        default: TSB_ATTN_S(1); break;
      }
#undef TSB_ATTN_S
      count_launch(device);
      TSB_TRY(check_launch("attention_staged"));
      if (splits > 1) {
        TSB_CUDA(launch_k(attn_combine_kernel<T>, dim3(B * S * H), dim3(hd < 128 ? 64 : 128), 0, s, out, (const float*)ws, hd, splits));
        count_launch(device);
        TSB_TRY(check_launch("attention_combine"));
      }
      return 1;
    }
  }
#define TSB_ATTN(GG) TSB_CUDA(launch_k(attn_kernel<T, GG>, grid, dim3(kAttnThreads), smem, s, out, ws, q, q_rs, cK, cV, S, H, Hkv, hd, T0, dT0, Tmax, splits, scale))
  switch (G) {
    case 8: TSB_ATTN(8); break;
    case 4: TSB_ATTN(4); break;
    case 2: TSB_ATTN(2); break;
    default: TSB_ATTN(1); break;
  }
#undef TSB_ATTN
  count_launch(device);
  TSB_TRY(check_launch("attention"));
  if (splits > 1) {
    TSB_CUDA(launch_k(attn_combine_kernel<T>, dim3(B * S * H), dim3(hd < 128 ? 64 : 128), 0, s, out, (const float*)ws, hd, splits));
    count_launch(device);
    TSB_TRY(check_launch("attention_combine"));
  }
  return 1;
}

int attn_pick_splits(DeviceState* st, int dtype, int B, int H, int Hkv, int hd, int T) {
  const int group = H / Hkv;
  int G = 1;
  if (group % 8 == 0) G = 8;
  else if (group % 4 == 0) G = 4;
  else if (group % 2 == 0) G = 2;
  return pick_splits(st, B, Hkv * (group / G), T, mma_decode_shape(dtype, H, Hkv, hd) ? 256 : 32);
}

int launch_attention(int device, DeviceState* st, int dtype, void* out, const void* q, int64_t q_rs, const void* cK,
                     const void* cV, int B, int S, int H, int Hkv, int hd, int T0, const int* dT0, int Tmax, int splits_hint,
                     void* ws, int64_t ws_bytes, cudaStream_t s) {
  if (B == 0 || S == 0) return 1;
  if (dtype == TSB200_F32)
    return launch_attn_t<float>(device, st, (float*)out, (const float*)q, q_rs, (const float*)cK, (const float*)cV, B, S, H, Hkv,
                                hd, T0, dT0, Tmax, splits_hint, (float*)ws, ws_bytes, s);
  if (dtype == TSB200_F16)
    return launch_attn_t<__half>(device, st, (__half*)out, (const __half*)q, q_rs, (const __half*)cK, (const __half*)cV, B, S, H,
                                 Hkv, hd, T0, dT0, Tmax, splits_hint, (float*)ws, ws_bytes, s);
  TSB_FAIL("attention: unsupported dtype %d", dtype);
}

int launch_rope_table(int device, DeviceState* st, float2* tab, int Tmax, int hd, double base, cudaStream_t s) {
  const int64_t n = (int64_t)Tmax * (hd / 2);
  const int g = (int)((n + 255) / 256 < (int64_t)st->sm_count * 8 ? (n + 255) / 256 : (int64_t)st->sm_count * 8);
  rope_table_kernel<<<g > 0 ? g : 1, 256, 0, s>>>(tab, Tmax, hd, base);
  count_launch(device);
  return check_launch("rope_table");
}

int launch_rope_append(int device, DeviceState* st, int dtype, void* q, const void* k, const void* v, int64_t q_rs,
                       int64_t kv_rs, void* cK, void* cV, int B, int S, int H, int Hkv, int hd, int T0, const int* dT0,
                       int Tmax, int use_rope, double base, const float2* tab, cudaStream_t s) {
  if (B == 0 || S == 0) return 1;
  TSB_CHECK(hd % 2 == 0, "rope_append: head_dim must be even");
  TSB_CHECK(dT0 || (T0 >= 0 && T0 + S <= Tmax), "rope_append: cache capacity exceeded (%d + %d > %d)", T0, S, Tmax);
  const int64_t n = (int64_t)B * S * (H + 2 * Hkv) * (hd / 2);
  int64_t g = (n + 255) / 256;
  if (g > (int64_t)st->sm_count * 16) g = (int64_t)st->sm_count * 16;
  if (dtype == TSB200_F32)
    TSB_CUDA(launch_k(rope_append_kernel<float>, dim3((int)g), dim3(256), 0, s, (float*)q, (const float*)k, (const float*)v, q_rs, kv_rs,
                      (float*)cK, (float*)cV, B, S, H, Hkv, hd, T0, dT0, Tmax, use_rope, base, tab));
  else if (dtype == TSB200_F16)
    TSB_CUDA(launch_k(rope_append_kernel<__half>, dim3((int)g), dim3(256), 0, s, (__half*)q, (const __half*)k, (const __half*)v, q_rs,
                      kv_rs, (__half*)cK, (__half*)cV, B, S, H, Hkv, hd, T0, dT0, Tmax, use_rope, base, tab));
  else
    TSB_FAIL("rope_append: unsupported dtype %d", dtype);
  count_launch(device);
  return check_launch("rope_append");
}

}  // namespace tsb

using namespace tsb;

extern "C" {

int TSB200_RoPEEx(int device, const TSB200Tensor* result, const TSB200Tensor* src, int seqLen, int rowOffset, float base,
                  void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_TRY(check_tensor(result, "result"));
  TSB_TRY(check_tensor(src, "src"));
  TSB_CHECK(result->dtype == src->dtype, "rope: dtype mismatch");
  // the reference requires contiguous tensors here (AdvFuncKernels.cs:3198-3205)
  TSB_CHECK(is_contiguous(result) && is_contiguous(src) && numel(result) == numel(src), "rope: tensors must be contiguous and equal-sized");
  const int cols = (int)src->sizes[src->ndim - 1];
  TSB_CHECK(cols > 0 && cols % 2 == 0 && seqLen > 0, "rope: even column count and positive seqLen required");
  const int64_t rows = numel(src) / cols;
  if (rows == 0) return 1;
  cudaStream_t s = pick_stream(st, stream);
  int64_t g = (rows * (cols / 2) + 255) / 256;
  if (g > (int64_t)st->sm_count * 8) g = (int64_t)st->sm_count * 8;
  if (src->dtype == TSB200_F32) rope_kernel<float><<<(int)g, 256, 0, s>>>((float*)result->data, (const float*)src->data, rows, cols, seqLen, rowOffset, (double)base);
  else if (src->dtype == TSB200_F16) rope_kernel<__half><<<(int)g, 256, 0, s>>>((__half*)result->data, (const __half*)src->data, rows, cols, seqLen, rowOffset, (double)base);
  else TSB_FAIL("rope: unsupported dtype %d", src->dtype);
  count_launch(device);
  return check_launch("rope");
}

int TSB200_RoPE(int device, const TSB200Tensor* result, const TSB200Tensor* src, int seqLen, int rowOffset, void* stream) {
  return TSB200_RoPEEx(device, result, src, seqLen, rowOffset, 500000.0f, stream);
}

int TSB200_RopeAppend(int device, int dtype, void* q, const void* k, const void* v, int64_t q_row_stride,
                      int64_t kv_row_stride, void* cacheK, void* cacheV, int B, int S, int H, int Hkv, int hd, int T0,
                      int Tmax, int use_rope, float rope_base, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(q && k && v && cacheK && cacheV, "rope_append: null pointer");
  return launch_rope_append(device, st, dtype, q, k, v, q_row_stride, kv_row_stride, cacheK, cacheV, B, S, H, Hkv, hd, T0,
                            nullptr, Tmax, use_rope, (double)rope_base, nullptr, pick_stream(st, stream));
}

int64_t TSB200_FlashDecodeWorkspaceBytes(int B, int H, int hd, int T) { return attn_workspace_bytes(B, H, hd, T); }

int TSB200_FlashDecode(int device, int dtype, void* out, const void* q, int64_t q_row_stride, const void* cacheK,
                       const void* cacheV, int B, int H, int Hkv, int hd, int T, int Tmax, void* workspace,
                       int64_t workspace_bytes, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(out && q && cacheK && cacheV, "flash_decode: null pointer");
  TSB_CHECK(T >= 1, "flash_decode: empty cache");
  return launch_attention(device, st, dtype, out, q, q_row_stride, cacheK, cacheV, B, 1, H, Hkv, hd, T - 1, nullptr, Tmax, 0,
                          workspace, workspace_bytes, pick_stream(st, stream));
}

int TSB200_PrefillAttention(int device, int dtype, void* out, const void* q, int64_t q_row_stride, const void* cacheK,
                            const void* cacheV, int B, int S, int H, int Hkv, int hd, int T0, int Tmax, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(out && q && cacheK && cacheV, "prefill_attention: null pointer");
  return launch_attention(device, st, dtype, out, q, q_row_stride, cacheK, cacheV, B, S, H, Hkv, hd, T0, nullptr, Tmax, 0,
                          nullptr, 0, pick_stream(st, stream));
}

}  // extern "C"
