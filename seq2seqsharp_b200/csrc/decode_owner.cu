// Owner-partitioned persistent decode step, fp16, one GPU (see decode_owner.cuh for the partition and the weight layout).
//
// One CTA per SM.  Warp 8 (one lane) streams the CTA's private, contiguous weight stream through a ring of 16 KB
// stages with TMA bulk copies; it never waits for activations.  Warps 0-7 follow the program: per layer an attention
// block and an FFN block, then the LM head.  A block starts with ONE grid-wide wait (the residual stream of the previous
// block is complete), stages the normed row into shared memory and runs its jobs; results that other CTAs need are
// added with 64-bit integer atomics (fixed point) into the group accumulator or into the next residual buffer.
//
// Residual stream: three buffers X[0..2] of int64 [rows, d], fixed point.  Block p reads X[p % 3], every CTA adds its
// contributions to X[(p+1) % 3] (one CTA per column slice also adds the old value and the bias), and clears its slice of
// X[(p+2) % 3].  Readers of a buffer have all arrived at the block's counter before anybody clears or refills it.
#include <cstdlib>
#include <cstring>
#include <vector>

#include "decode_owner.cuh"
#include "decode_stack.cuh"

namespace tsb {

constexpr float kOwnFix = 268435456.0f;          // 2^28
constexpr float kOwnUnfix = 1.0f / 268435456.0f;
constexpr int kOwnCntStride = 8;                 // one 32-byte sector per counter

struct OwnLayerDev {
  const __half *g1, *b1n, *bqkv, *bo, *g2, *b2n, *bup, *bdown;
  __half *cK, *cV;
};

struct OwnArgs {
  const unsigned char* wstream;   // all CTAs' streams
  const long long* cta_row0;      // [G] first 4 KB row of each CTA's stream
  const int* cta_tiles;           // [G] 16 KB tiles of each CTA's stream
  const OwnJob* jobs;             // [G][5]
  const OwnLayerDev* layers;      // [L]
  const __half *gF, *bF, *head_b; // final norm, LM head bias
  float* logits;                  // [M, V]
  long long* X[3];                // residual stream, fixed point [kOwnMaxRows, d]
  long long* QA[2];               // group accumulators of q|k|v [Hkv][kOwnMaxRows][QW], fixed point
  float* AP;                      // partial softmax states [rows][Hkv][grp][gmax][hd + 2]
  unsigned* cnt;                  // [2L block counters | L*Hkv*2 group counters | exit], kOwnCntStride words apart
  const float2* rope_tab;
  const int* dT;
  int* error_flag;
  unsigned poll_limit;
  int L, M, d, H, Hkv, hd, grp, F, V, Tmax, glu, act, xmode, use_rope, gmax;
  float eps, scale;
  int stages;
  // shared memory (bytes from the aligned base, after the ring)
  int xstride, ystride, hstride, qstride;    // elements between rows
  int off_xs, off_red, off_merge, off_ys, off_hs, off_qs, off_gsum, off_bar, gsum_cols;
};

__device__ __forceinline__ long long own_fix(float v) { return __float2ll_rn(v * kOwnFix); }
__device__ __forceinline__ float own_unfix(long long v) { return __ll2float_rn(v) * kOwnUnfix; }
__device__ __forceinline__ void own_add(long long* p, long long v) {
  atomicAdd(reinterpret_cast<unsigned long long*>(p), static_cast<unsigned long long>(v));
}
__device__ __forceinline__ long long own_ldcg(const long long* p) { return __ldcg(p); }
__device__ __forceinline__ void own_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ------------------------------------------------------------------------------------------- the weight ring (consumer side)
struct OwnRing {
  uint32_t stage0;
  uint64_t *full, *empty;
  int S, slot, r;
  unsigned par;
  bool dead;
  volatile int* s_err;
  // the next block of warp `w`: one 16-byte load per lane; a stage goes back to the producer after its fourth row
  __device__ __forceinline__ uint4 next(int w, int lane) {
    if (r == 0 && !dead) {
      if (!mbar_wait(&full[slot], par, kSpinLimit)) {
        *s_err = 1;
        dead = true;
      }
    }
    uint4 v;
    const uint32_t addr = stage0 + (uint32_t)slot * kOwnTileBytes + (uint32_t)r * kOwnRowBytes + (uint32_t)w * kOwnBlockBytes + (uint32_t)lane * 16u;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    if (++r == 4) {
      r = 0;
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[slot]);
      if (++slot == S) {
        slot = 0;
        par ^= 1u;
      }
    }
    return v;
  }
};

// ------------------------------------------------------------------------------------------- jobs (consumer side)
// K-split job: see OwnJob.  `xb` is the B operand (activations, fp16 [rows][xstride]) whose element 0 is the job's first k.
// emit(column of the job, row, sum) is called once per output by some thread after the eight warps' sums have met.
template <typename Emit>
__device__ __forceinline__ void own_job_ksplit(const OwnJob& j, OwnRing& R, const __half* xb, int xstride, int M, float* red, int w,
                                               int lane, int tid, Emit emit) {
  if (j.nrows == 0) return;
  const int g8 = lane >> 2, t4 = lane & 3;
  const bool row_live = g8 < M;
  const __half* xrow = xb + (size_t)(row_live ? g8 : 0) * xstride + 2 * t4;
  for (int c = 0; c < j.nchunks; ++c) {
    const int left = j.ws - c * kOwnKChunk;
    const int wc = left < kOwnKChunk ? left : kOwnKChunk;
    float acc[kOwnKChunk][4];
#pragma unroll
    for (int s = 0; s < kOwnKChunk; ++s)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[s][e] = 0.0f;
    for (int kk = 0; kk < j.ksw; ++kk) {
      const int kst = w * j.ksw + kk;
      const bool klive = kst < j.ks;
      uint32_t b0 = 0u, b1 = 0u;
      if (row_live && klive) {
        b0 = *reinterpret_cast<const uint32_t*>(xrow + kst * 16);
        b1 = *reinterpret_cast<const uint32_t*>(xrow + kst * 16 + 8);
      }
#pragma unroll
      for (int s = 0; s < kOwnKChunk; ++s) {
        if (s < wc) {
          const uint4 av = R.next(w, lane);
          own_mma(acc[s], av.x, av.y, av.z, av.w, b0, b1);
        }
      }
    }
    // the eight warps' sums meet: red[warp][column of the chunk][row]
#pragma unroll
    for (int s = 0; s < kOwnKChunk; ++s) {
      if (s < wc) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = 2 * t4 + (e & 1), col = s * 16 + g8 + ((e >> 1) << 3);
          if (n < M) red[(w * (kOwnKChunk * 16) + col) * M + n] = acc[s][e];
        }
      }
    }
    consumers_sync();
    for (int idx = tid; idx < wc * 16 * M; idx += 256) {
      const int n = idx % M, col = idx / M;
      float v = 0.0f;
#pragma unroll
      for (int ww = 0; ww < kConsumerWarps; ++ww) v += red[(ww * (kOwnKChunk * 16) + col) * M + n];
      emit(c * kOwnKChunk * 16 + col, n, v);
    }
    consumers_sync();
  }
}

// strip-split job: a warp holds the complete sums of its strips; emit is called from the accumulator registers.
template <typename Emit>
__device__ __forceinline__ void own_job_ssplit(const OwnJob& j, OwnRing& R, const __half* xb, int xstride, int M, int w, int lane,
                                               Emit emit) {
  if (j.nrows == 0) return;
  const int g8 = lane >> 2, t4 = lane & 3;
  const bool row_live = g8 < M;
  const __half* xrow = xb + (size_t)(row_live ? g8 : 0) * xstride + 2 * t4;
  for (int c = 0; c < j.nchunks; ++c) {
    float acc[kOwnMaxSpw][4];
#pragma unroll
    for (int s = 0; s < kOwnMaxSpw; ++s)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[s][e] = 0.0f;
    for (int k = 0; k < j.ks; ++k) {
      uint32_t b0 = 0u, b1 = 0u;
      if (row_live) {
        b0 = *reinterpret_cast<const uint32_t*>(xrow + k * 16);
        b1 = *reinterpret_cast<const uint32_t*>(xrow + k * 16 + 8);
      }
#pragma unroll
      for (int s = 0; s < kOwnMaxSpw; ++s) {
        if (s < j.spw) {
          const uint4 av = R.next(w, lane);
          own_mma(acc[s], av.x, av.y, av.z, av.w, b0, b1);
        }
      }
    }
#pragma unroll
    for (int s = 0; s < kOwnMaxSpw; ++s) {
      const int strip = c * 8 * j.spw + w * j.spw + s;
      if (s < j.spw && strip < j.ws) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = 2 * t4 + (e & 1), col = strip * 16 + g8 + ((e >> 1) << 3);
          if (n < M) emit(col, n, acc[s][e]);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------- staging with the fused norm
struct OwnNormConsts {
  uint2 g[4], b[4];   // four groups of four consecutive halves per thread: rows of up to 4096 elements
  float beta_on;
};
__device__ __forceinline__ void own_norm_consts(OwnNormConsts& nc, const __half* gamma, const __half* beta_or_null, int d, int tid) {
  const __half* beta = beta_or_null ? beta_or_null : gamma;  // every address a thread can form stays valid
  nc.beta_on = beta_or_null ? 1.0f : 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int k = (j * 256 + tid) * 4;
    const int kc = k < d ? k : 0;
    nc.g[j] = *reinterpret_cast<const uint2*>(gamma + kc);
    nc.b[j] = *reinterpret_cast<const uint2*>(beta + kc);
  }
}
__device__ __forceinline__ void own_half4(const uint2& raw, float* f) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
  const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
// xs[m][k] = norm(X[m])[k] in fp16; RMSNorm (xmode 1) or LayerNorm (xmode 2), the arithmetic of the stand-alone kernels
// (fp32 sums, sqrt, divide).  d <= 4096, d % 4 == 0.
__device__ __forceinline__ void own_stage_norm(__half* xs, int xstride, const long long* X, const OwnNormConsts& nc, int xmode, float eps,
                                               int M, int d, int tid, float* s_stat) {
  const int lane = tid & 31, w = tid >> 5;
  for (int m = 0; m < M; ++m) {
    float v[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = (j * 256 + tid) * 4;
      const longlong2* p = reinterpret_cast<const longlong2*>(X + (size_t)m * d + (k < d ? k : 0));
      const longlong2 a = __ldcg(p), b = __ldcg(p + 1);
      const bool ok = k < d;
      v[j][0] = ok ? own_unfix(a.x) : 0.0f;
      v[j][1] = ok ? own_unfix(a.y) : 0.0f;
      v[j][2] = ok ? own_unfix(b.x) : 0.0f;
      v[j][3] = ok ? own_unfix(b.y) : 0.0f;
    }
    float s1 = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      s1 += (xmode == 2) ? (v[j][0] + v[j][1]) + (v[j][2] + v[j][3])
                         : (v[j][0] * v[j][0] + v[j][1] * v[j][1]) + (v[j][2] * v[j][2] + v[j][3] * v[j][3]);
    s1 = warp_sum(s1);
    if (lane == 0) s_stat[(m & 3) * 8 + w] = s1;
    consumers_sync();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kConsumerWarps; ++i) tot += s_stat[(m & 3) * 8 + i];
    float mean = 0.0f, inv;
    if (xmode == 2) {
      mean = tot / d;
      float s2 = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if ((j * 256 + tid) * 4 < d) {
          const float e0 = v[j][0] - mean, e1 = v[j][1] - mean, e2 = v[j][2] - mean, e3 = v[j][3] - mean;
          s2 += (e0 * e0 + e1 * e1) + (e2 * e2 + e3 * e3);
        }
      }
      s2 = warp_sum(s2);
      if (lane == 0) s_stat[32 + (m & 3) * 8 + w] = s2;
      consumers_sync();
      float t2 = 0.0f;
#pragma unroll
      for (int i = 0; i < kConsumerWarps; ++i) t2 += s_stat[32 + (m & 3) * 8 + i];
      inv = sqrtf(eps + t2 / d);
    } else {
      inv = sqrtf(tot / (float)d + eps);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = (j * 256 + tid) * 4;
      if (k < d) {
        float gf[4], bf[4], o[4];
        own_half4(nc.g[j], gf);
        own_half4(nc.b[j], bf);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = gf[e] * ((v[j][e] - mean) / inv) + nc.beta_on * bf[e];
        St4<__half>::st(xs + (size_t)m * xstride + k, o);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------- waits between CTAs
// One thread polls (bounded); everybody learns the outcome.  A CTA that gave up keeps going without waiting.
__device__ __forceinline__ void own_wait(const unsigned* p, unsigned target, const OwnArgs& a, volatile int* s_err, bool& dead, int tid) {
  if (tid == 0) {
    if (!poll_count(p, target, dead ? 1u : a.poll_limit, a.error_flag)) {
      *s_err = 1;
      *a.error_flag = 1;
    }
  }
  consumers_sync();
  if (*s_err) dead = true;
}
// Every thread's earlier stores and atomics are published by ONE release-add after a CTA barrier (cumulativity).
__device__ __forceinline__ void own_arrive(unsigned* p, int tid) {
  consumers_sync();
  if (tid == 0) red_release_add(p, 1u);
}

// ------------------------------------------------------------------------------------------- attention of one KV-head group
// CTA `i` of the group takes the cached tokens [t_beg, t_end) of every row and GH query heads at a time; lane groups of
// hd/8 lanes own one token per iteration (16-byte loads, four tokens in flight), each runs an online softmax, the lane
// groups' states are merged through shared memory and written as this CTA's partial state of (row, head).
// q (rotated, rounded to fp16, unscaled), the new k and the new v of the group come from shared memory (`qs`).
template <int GH>
__device__ __forceinline__ void own_attention(const OwnArgs& a, const OwnLayerDev& Lr, int g, int i, int gsz, int T0, const float* qs,
                                              float* merge, int tid) {
  constexpr int EPL = 8;
  const int hd = a.hd, grp = a.grp, Hkv = a.Hkv, Tmax = a.Tmax;
  const int lpt = hd / EPL, tpw = 32 / lpt;
  const int lane = tid & 31, w = tid >> 5;
  const int sub = lane / lpt, li = lane % lpt;
  const int Tk = T0 + 1;
  const int per = (Tk + gsz - 1) / gsz;
  const int t_beg = min(Tk, i * per), t_end = min(Tk, t_beg + per);
  const int t_cached_end = min(t_end, T0);
  const bool has_new = (t_beg <= T0) && (T0 < t_end);
  const int rec = hd + 2;
  const int nstates = kConsumerWarps * tpw;
  for (int m = 0; m < a.M; ++m) {
    const float* qrow = qs + (size_t)m * a.qstride;
    const size_t head_off = ((size_t)m * Hkv + g) * Tmax * hd + li * EPL;
    const __half* Kb = Lr.cK + head_off;
    const __half* Vb = Lr.cV + head_off;
    for (int h0 = 0; h0 < grp; h0 += GH) {
      float qf[GH][EPL];
#pragma unroll
      for (int gg = 0; gg < GH; ++gg)
#pragma unroll
        for (int e = 0; e < EPL; ++e) qf[gg][e] = qrow[(h0 + gg) * hd + li * EPL + e] * a.scale;
      float mx[GH], l[GH], acc[GH][EPL];
#pragma unroll
      for (int gg = 0; gg < GH; ++gg) {
        mx[gg] = -INFINITY;
        l[gg] = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[gg][e] = 0.0f;
      }
      for (int tb = t_beg + w * tpw; tb < t_cached_end; tb += 4 * nstates) {
        TileVec<__half> kv[4], vv[4];
        bool live[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int t = tb + q * nstates + sub;
          live[q] = t < t_cached_end;  // all lanes iterate together (full-warp shuffles); dead lanes re-read token t_beg
          const size_t o = (size_t)(live[q] ? t : t_beg) * hd;
          kv[q].lds(Kb + o);
          vv[q].lds(Vb + o);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float kf[EPL], vf[EPL];
          kv[q].get(kf);
          vv[q].get(vf);
          attn_update<GH, EPL>(qf, kf, vf, mx, l, acc, lpt, live[q]);
        }
      }
      if (has_new && w == 0) {  // the token of this step, from shared memory
        float kf[EPL], vf[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          kf[e] = qrow[grp * hd + li * EPL + e];
          vf[e] = qrow[(grp + 1) * hd + li * EPL + e];
        }
        attn_update<GH, EPL>(qf, kf, vf, mx, l, acc, lpt, sub == 0);
      }
      const int st = w * tpw + sub;
#pragma unroll
      for (int gg = 0; gg < GH; ++gg) {
        float* r = merge + ((size_t)st * GH + gg) * rec;
        if (li == 0) {
          r[0] = mx[gg];
          r[1] = l[gg];
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) r[2 + li * EPL + e] = acc[gg][e];
      }
      consumers_sync();
      for (int idx = tid; idx < GH * hd; idx += 256) {
        const int gg = idx / hd, e = idx % hd;
        float mm = -INFINITY;
        for (int q = 0; q < nstates; ++q) mm = fmaxf(mm, merge[((size_t)q * GH + gg) * rec]);
        float Ls = 0.0f, As = 0.0f;
        for (int q = 0; q < nstates; ++q) {
          const float* r = merge + ((size_t)q * GH + gg) * rec;
          const float cc = (r[0] == -INFINITY) ? 0.0f : __expf(r[0] - mm);
          Ls += r[1] * cc;
          As += r[2 + e] * cc;
        }
        float* pr = a.AP + ((((size_t)m * Hkv + g) * grp + h0 + gg) * a.gmax + i) * rec;
        if (e == 0) {
          pr[0] = mm;
          pr[1] = Ls;
        }
        pr[2 + e] = As;
      }
      consumers_sync();  // the merge area is free again
    }
  }
}

// ------------------------------------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(kStreamThreads, 1) decode_owner_kernel(OwnArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.stages;
  unsigned char* stage_mem = smem;
  unsigned char* un = smem + (size_t)S * kOwnTileBytes;
  __half* xs = reinterpret_cast<__half*>(un + a.off_xs);
  float* red = reinterpret_cast<float*>(un + a.off_red);
  float* merge = reinterpret_cast<float*>(un + a.off_merge);   // aliases xs + red (attention runs between QKV and W0)
  __half* ys = reinterpret_cast<__half*>(un + a.off_ys);
  __half* hs = reinterpret_cast<__half*>(un + a.off_hs);
  float* qs = reinterpret_cast<float*>(un + a.off_qs);
  float* gsum = reinterpret_cast<float*>(un + a.off_gsum);
  uint64_t* full = reinterpret_cast<uint64_t*>(un + a.off_bar);
  uint64_t* empty = full + 16;
  __shared__ int s_err, s_last;
  __shared__ float s_stat[64];
  __shared__ OwnJob s_jobs[5];

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kConsumerWarps);
    }
    s_err = 0;
    s_last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  {
    const int words = 5 * (int)(sizeof(OwnJob) / 4);
    const int* src = reinterpret_cast<const int*>(a.jobs + (size_t)cta * 5);
    int* dst = reinterpret_cast<int*>(s_jobs);
    for (int i = tid; i < words; i += kStreamThreads) dst[i] = src[i];
  }
  __syncthreads();

  if (w == kConsumerWarps) {
    // producer: the CTA's stream is one contiguous range; weights never depend on earlier kernels
    if (lane == 0) {
      const unsigned char* src = a.wstream + (size_t)a.cta_row0[cta] * kOwnRowBytes;
      const int n_tiles = a.cta_tiles[cta];
      int issued = 0;
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % S;
        if (t >= S) {
          const unsigned par = (unsigned)((t / S - 1) & 1);
          bool got = false;
          for (unsigned q = 0; q < (kSpinLimit >> 10) && !got && !*(volatile int*)&s_err; ++q) got = mbar_wait(&empty[s], par, 1024u);
          if (!got) {
            *(volatile int*)&s_err = 1;
            break;
          }
        }
        if (*(volatile int*)&s_err) break;
        mbar_expect_tx(&full[s], kOwnTileBytes);
        bulk_g2s(stage_mem + (size_t)s * kOwnTileBytes, src + (size_t)t * kOwnTileBytes, kOwnTileBytes, &full[s]);
        ++issued;
      }
      if (*(volatile int*)&s_err) {
        // await (bounded) every copy that may still be in flight, so nothing lands after the CTA has left
        const int first = issued > S ? issued - S : 0;
        for (int q = first; q < issued; ++q) mbar_wait(&full[q % S], (unsigned)((q / S) & 1));
        *a.error_flag = 1;
      }
    }
    return;
  }

  grid_dep_wait();  // the residual row of this step, the cache length and last step's cache appends are visible
  const int M = a.M, d = a.d, hd = a.hd, grp = a.grp, Hkv = a.Hkv;
  const int T0 = min(__ldcg(a.dT), a.Tmax - 1);
  const OwnJob& jq = s_jobs[OWN_QKV];
  const int g = jq.group;
  const int gb = own_group_begin(g, G, Hkv), gsz = own_group_begin(g + 1, G, Hkv) - gb, gi = cta - gb;
  const int QW = (grp + 2) * hd;
  const int c0 = own_split(d, G, cta), c1 = own_split(d, G, cta + 1);   // this CTA's slice of the residual columns
  unsigned* cntP = a.cnt;                                               // [2L] block counters
  unsigned* cntG = a.cnt + (size_t)2 * a.L * kOwnCntStride;             // [L][Hkv][2] group counters
  unsigned* cntExit = cntG + (size_t)a.L * Hkv * 2 * kOwnCntStride;
  OwnRing R;
  R.stage0 = smem_u32(stage_mem);
  R.full = full;
  R.empty = empty;
  R.S = S;
  R.slot = 0;
  R.r = 0;
  R.par = 0u;
  R.dead = false;
  R.s_err = &s_err;
  bool dead = false;

  // duties of a block: add the old residual value and the bias of the block's last linear to the CTA's slice of the
  // next buffer, clear the slice of the buffer after that
  auto duties = [&](const long long* Xc, long long* Xn, long long* Xz, const __half* bias) {
    const int wdt = c1 - c0;
    for (int idx = tid; idx < M * wdt; idx += 256) {
      const int m = idx / wdt, col = c0 + idx % wdt;
      long long v = own_ldcg(Xc + (size_t)m * d + col);
      if (bias) v += own_fix(__half2float(bias[col]));
      own_add(Xn + (size_t)m * d + col, v);
      Xz[(size_t)m * d + col] = 0;
    }
  };

  for (int layer = 0; layer < a.L; ++layer) {
    const OwnLayerDev& Lr = a.layers[layer];
    // =================================================================== attention block
    {
      const int p = 2 * layer;
      const long long* Xc = a.X[p % 3];
      long long* Xn = a.X[(p + 1) % 3];
      long long* Xz = a.X[(p + 2) % 3];
      long long* qa = a.QA[layer & 1] + (size_t)g * kOwnMaxRows * QW;
      long long* qz = a.QA[(layer + 1) & 1] + (size_t)g * kOwnMaxRows * QW;
      OwnNormConsts nc;
      own_norm_consts(nc, Lr.g1, Lr.b1n, d, tid);
      if (p > 0) own_wait(cntP + (size_t)(p - 1) * kOwnCntStride, (unsigned)G, a, &s_err, dead, tid);
      R.dead = R.dead || dead;
      own_stage_norm(xs, a.xstride, Xc, nc, a.xmode, a.eps, M, d, tid, s_stat);
      duties(Xc, Xn, Xz, Lr.bo);
      {
        // clear this CTA's part of the group accumulator the NEXT layer uses
        const int n = kOwnMaxRows * QW, z0 = own_split(n, gsz, gi), z1 = own_split(n, gsz, gi + 1);
        for (int idx = z0 + tid; idx < z1; idx += 256) qz[idx] = 0;
      }
      consumers_sync();
      // q|k|v of the group: this CTA's range of K, sums meet in the group accumulator
      own_job_ssplit(jq, R, xs + jq.kbase, a.xstride, M, w, lane,
                     [&](int col, int n, float v) { own_add(qa + (size_t)n * QW + col, own_fix(v)); });
      unsigned* gc = cntG + ((size_t)(layer * Hkv + g) * 2) * kOwnCntStride;
      own_arrive(gc, tid);
      own_wait(gc, (unsigned)gsz, a, &s_err, dead, tid);
      // bias, rounding to fp16 (the model's activation type), RoPE
      for (int idx = tid; idx < M * QW; idx += 256) {
        const int m = idx / QW, jcol = idx % QW;
        float v = own_unfix(own_ldcg(qa + (size_t)m * QW + jcol));
        v += __half2float(Lr.bqkv[own_qkv_col(jcol, g, grp, hd, a.H, Hkv)]);
        qs[(size_t)m * a.qstride + jcol] = __half2float(__float2half_rn(v));
      }
      consumers_sync();
      if (a.use_rope) {
        const int npair = (grp + 1) * hd / 2;   // q heads and k
        for (int idx = tid; idx < M * npair; idx += 256) {
          const int m = idx / npair, pr = idx % npair;
          const float2 cs = a.rope_tab[(size_t)T0 * (hd / 2) + pr % (hd / 2)];
          float* q2 = qs + (size_t)m * a.qstride + 2 * pr;
          const float x0 = q2[0], x1 = q2[1];
          q2[0] = __half2float(__float2half_rn(x0 * cs.x - x1 * cs.y));
          q2[1] = __half2float(__float2half_rn(x1 * cs.x + x0 * cs.y));
        }
        consumers_sync();
      }
      if (gi == 0) {  // the first CTA of the group appends the new k and v rows to the cache
        for (int idx = tid; idx < M * hd; idx += 256) {
          const int m = idx / hd, e = idx % hd;
          const size_t o = (((size_t)m * Hkv + g) * a.Tmax + T0) * hd + e;
          Lr.cK[o] = __float2half_rn(qs[(size_t)m * a.qstride + grp * hd + e]);
          Lr.cV[o] = __float2half_rn(qs[(size_t)m * a.qstride + (grp + 1) * hd + e]);
        }
      }
      if (grp % 4 == 0) own_attention<4>(a, Lr, g, gi, gsz, T0, qs, merge, tid);
      else own_attention<1>(a, Lr, g, gi, gsz, T0, qs, merge, tid);
      own_arrive(gc + kOwnCntStride, tid);
      own_wait(gc + kOwnCntStride, (unsigned)gsz, a, &s_err, dead, tid);
      // merge the group's partial states: attention output of the group's heads, fp16, in shared memory
      {
        const int rec = hd + 2, per_row = grp * hd;
        for (int idx = tid; idx < M * per_row; idx += 256) {
          const int m = idx / per_row, r = idx % per_row, head = r / hd, e = r % hd;
          const float* base = a.AP + ((((size_t)m * Hkv + g) * grp + head) * a.gmax) * rec;
          float mm = -INFINITY;
          for (int s = 0; s < gsz; ++s) mm = fmaxf(mm, __ldcg(base + (size_t)s * rec));
          float Ls = 0.0f, As = 0.0f;
          for (int s = 0; s < gsz; ++s) {
            const float mi = __ldcg(base + (size_t)s * rec);
            const float cc = (mi == -INFINITY) ? 0.0f : __expf(mi - mm);
            Ls += __ldcg(base + (size_t)s * rec + 1) * cc;
            As += __ldcg(base + (size_t)s * rec + 2 + e) * cc;
          }
          ys[(size_t)m * a.ystride + r] = __float2half_rn(Ls > 0.0f ? As / Ls : 0.0f);
        }
      }
      consumers_sync();
      // the group's rows of W0, this CTA's range of output columns
      const OwnJob& jo = s_jobs[OWN_W0];
      R.dead = R.dead || dead;
      own_job_ksplit(jo, R, ys, a.ystride, M, red, w, lane, tid, [&](int col, int n, float v) {
        own_add(Xn + (size_t)n * d + jo.cbase + col, own_fix(v));
      });
      own_arrive(cntP + (size_t)p * kOwnCntStride, tid);
    }
    // =================================================================== FFN block
    {
      const int p = 2 * layer + 1;
      const long long* Xc = a.X[p % 3];
      long long* Xn = a.X[(p + 1) % 3];
      long long* Xz = a.X[(p + 2) % 3];
      OwnNormConsts nc;
      own_norm_consts(nc, Lr.g2, Lr.b2n, d, tid);
      own_wait(cntP + (size_t)(p - 1) * kOwnCntStride, (unsigned)G, a, &s_err, dead, tid);
      R.dead = R.dead || dead;
      own_stage_norm(xs, a.xstride, Xc, nc, a.xmode, a.eps, M, d, tid, s_stat);
      duties(Xc, Xn, Xz, Lr.bdown);
      const OwnJob& ju = s_jobs[OWN_UP];
      const OwnJob& jd = s_jobs[OWN_DOWN];
      for (int idx = tid; idx < M * a.hstride; idx += 256) hs[idx] = __float2half_rn(0.0f);
      consumers_sync();
      own_job_ksplit(ju, R, xs, a.xstride, M, red, w, lane, tid,
                     [&](int col, int n, float v) { gsum[(size_t)n * a.gsum_cols + col] = v; });
      consumers_sync();
      // bias, activation, gate: this CTA's hidden units, fp16, in shared memory
      if (a.glu) {
        const int nh = ju.ws * 8;
        for (int idx = tid; idx < M * nh; idx += 256) {
          const int m = idx / nh, jl = idx % nh;
          float av = gsum[(size_t)m * a.gsum_cols + 2 * jl] + __half2float(Lr.bup[ju.cbase + 2 * jl]);
          const float gv = gsum[(size_t)m * a.gsum_cols + 2 * jl + 1] + __half2float(Lr.bup[ju.cbase + 2 * jl + 1]);
          if (a.act == TSB200_ACT_SWIGLU) av = av / (1.0f + expf(-av));
          hs[(size_t)m * a.hstride + jl] = __float2half_rn(av * gv);
        }
      } else {
        const int nh = ju.ws * 16;
        for (int idx = tid; idx < M * nh; idx += 256) {
          const int m = idx / nh, jl = idx % nh;
          float v = gsum[(size_t)m * a.gsum_cols + jl] + __half2float(Lr.bup[ju.cbase + jl]);
          switch (a.act) {
            case TSB200_ACT_RELU: v = v < 0.0f ? 0.0f : v; break;
            case TSB200_ACT_SILU: v = v / (1.0f + expf(-v)); break;
            case TSB200_ACT_LEAKYRELU: v = v < 0.0f ? 0.01f * v : v; break;
            case TSB200_ACT_GELU: v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)); break;
            default: break;
          }
          hs[(size_t)m * a.hstride + jl] = __float2half_rn(v);
        }
      }
      consumers_sync();
      // the matching rows of W2: all d output columns, sums go straight into the next residual buffer
      own_job_ssplit(jd, R, hs, a.hstride, M, w, lane, [&](int col, int n, float v) { own_add(Xn + (size_t)n * d + col, own_fix(v)); });
      own_arrive(cntP + (size_t)p * kOwnCntStride, tid);
    }
  }
  // =================================================================== LM head
  {
    const int p = 2 * a.L;
    const long long* Xc = a.X[p % 3];
    OwnNormConsts nc;
    own_norm_consts(nc, a.gF, a.bF, d, tid);
    grid_dep_launch();  // the sampling kernels may become resident while the LM head streams
    own_wait(cntP + (size_t)(p - 1) * kOwnCntStride, (unsigned)G, a, &s_err, dead, tid);
    R.dead = R.dead || dead;
    own_stage_norm(xs, a.xstride, Xc, nc, a.xmode, a.eps, M, d, tid, s_stat);
    consumers_sync();
    const OwnJob& jh = s_jobs[OWN_HEAD];
    own_job_ksplit(jh, R, xs, a.xstride, M, red, w, lane, tid, [&](int col, int n, float v) {
      const int c = jh.cbase + col;
      if (c < a.V) a.logits[(size_t)n * a.V + c] = v + __half2float(a.head_b[c]);
    });
  }
  // leave: the last CTA out clears the counters for the next launch
  consumers_sync();
  if (tid == 0) {
    if (*(volatile int*)&s_err) *a.error_flag = 1;
    __threadfence();
    const unsigned prev = atomicAdd(cntExit, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
  }
  consumers_sync();
  if (s_last) {
    const int n = 2 * a.L + a.L * Hkv * 2 + 1;
    for (int i = tid; i < n; i += 256) a.cnt[(size_t)i * kOwnCntStride] = 0u;
  }
}

// x (fp32 rows from the embedding kernel) -> X[0] in fixed point; X[1], X[2] and the first group accumulator start at zero
__global__ void own_init_kernel(long long* X0, long long* X1, long long* X2, long long* QA0, const float* x, int M, int d, int qa_words) {
  pdl_trigger();
  pdl_wait();
  const int n = kOwnMaxRows * d;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    X0[i] = (i < M * d) ? own_fix(x[i]) : 0;
    X1[i] = 0;
    X2[i] = 0;
  }
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < qa_words; i += gridDim.x * blockDim.x) QA0[i] = 0;
}

// ------------------------------------------------------------------------------------------- weight re-packing
// Source: a matrix in the engine's packed tile layout (kernels.cuh: packed_tile_off).  Element (k, c).
__device__ __forceinline__ __half own_src_elem(const __half* Wp, int KB, int K, int N, int k, int c) {
  if (k >= K || c >= N) return __float2half_rn(0.0f);
  const size_t tile = (size_t)(c >> 8) * KB + (k >> 5);
  return Wp[tile * (kTileBytes / 2) + packed_tile_off<__half>(k & 31, c & 255)];
}
struct OwnPackArgs {
  unsigned char* wstream;
  const long long* cta_row0;
  const OwnJob* jobs;     // [G][5]
  const __half* Wp;       // packed source matrix [K, N]
  int K, N;
  int kind;
  int layer;              // the layer's rows start layer * (rows of one layer) into a CTA's stream; HEAD jobs carry an absolute row0
  int grp, hd, H, Hkv;
};
__global__ void own_pack_kernel(OwnPackArgs p) {
  const OwnJob* mine = p.jobs + (size_t)blockIdx.x * 5;
  const OwnJob j = mine[p.kind];
  const int KB = (p.K + kKT - 1) / kKT;
  long long rows_layer = 0;
  for (int q = 0; q < 4; ++q) rows_layer += mine[q].nrows;
  const long long row_base = (p.kind == OWN_HEAD) ? 0 : (long long)p.layer * rows_layer;
  uint4* dst = reinterpret_cast<uint4*>(p.wstream + (size_t)(p.cta_row0[blockIdx.x] + row_base + j.row0) * kOwnRowBytes);
  const long long units = (long long)j.nrows * 256;   // 16-byte units: 8 warps x 32 lanes per row
  for (long long u = threadIdx.x; u < units; u += blockDim.x) {
    const int row = (int)(u >> 8), w = (int)((u >> 5) & 7), lane = (int)(u & 31);
    int kstep, strip;
    bool live;
    own_block_coords(j, row, w, kstep, strip, live);
    __align__(16) __half v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      int kk, cc;
      own_frag_coords(lane, e, kk, cc);
      const int k = j.kbase + kstep * 16 + kk;
      const int cl = strip * 16 + cc;
      const int c = (p.kind == OWN_QKV) ? own_qkv_col(cl, j.group, p.grp, p.hd, p.H, p.Hkv) : j.cbase + cl;
      v[e] = live ? own_src_elem(p.Wp, KB, p.K, p.N, k, c) : __float2half_rn(0.0f);
    }
    dst[u] = *reinterpret_cast<const uint4*>(v);
  }
}

// ------------------------------------------------------------------------------------------- host side
struct OwnerModel {
  int device = 0, G = 0;
  OwnDims D{};
  int norm_type = 0, act = 0, use_rope = 0, Tmax = 0;
  float eps = 0.0f;
  std::vector<OwnJob> jobs;            // [G][5], row0 relative to the layer (HEAD: to the end of the layers)
  std::vector<long long> cta_row0;     // [G]
  std::vector<int> cta_tiles;          // [G]
  std::vector<long long> rows_layer;   // [G] rows of one layer in a CTA's stream
  long long total_rows = 0;
  int gmax = 0, up_cols_max = 0, hid_max = 0;
  std::vector<OwnLayerPtrs> layers;
  const void *nf_g = nullptr, *nf_b = nullptr, *head_w = nullptr, *head_b = nullptr;
  // device
  unsigned char* wstream = nullptr;
  long long* d_row0 = nullptr;
  int* d_tiles = nullptr;
  OwnJob* d_jobs = nullptr;
  OwnLayerDev* d_layers = nullptr;
  long long* X = nullptr;     // 3 buffers
  long long* QA = nullptr;    // 2 buffers
  float* AP = nullptr;
  unsigned* cnt = nullptr;
  size_t cnt_bytes = 0;
  bool packed = false;
};

int owner_applicable(const OwnDims& D, int dtype, int sm_count) {
  if (dtype != TSB200_F16) return 0;
  if (D.d % 16 != 0 || D.d > 4096 || D.hd % 16 != 0 || D.hd > 256 || D.F % 16 != 0) return 0;
  const int lpt = D.hd / 8;
  if (lpt > 32 || (lpt & (lpt - 1)) != 0) return 0;
  if (D.H % D.Hkv != 0 || D.Hkv > sm_count) return 0;
  return 1;
}

void owner_destroy(OwnerModel* m) {
  if (!m) return;
  cudaSetDevice(m->device);
  void* ptrs[] = {m->wstream, m->d_row0, m->d_tiles, m->d_jobs, m->d_layers, m->X, m->QA, m->AP, m->cnt};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  delete m;
}

// The plan: every CTA's jobs and the place of its stream.  Pure host arithmetic (also used by the layout self-test).
void owner_plan(OwnerModel* m) {
  const int G = m->G;
  m->jobs.assign((size_t)G * 5, OwnJob{});
  m->cta_row0.assign(G, 0);
  m->cta_tiles.assign(G, 0);
  m->rows_layer.assign(G, 0);
  m->gmax = 0;
  m->up_cols_max = 16;
  m->hid_max = 16;
  long long row = 0;
  for (int c = 0; c < G; ++c) {
    OwnJob* j = &m->jobs[(size_t)c * 5];
    own_plan_cta(m->D, G, c, j);
    long long r = 0;
    for (int q = 0; q < 4; ++q) {
      j[q].row0 = r;
      r += j[q].nrows;
    }
    m->rows_layer[c] = r;
    j[OWN_HEAD].row0 = r * m->D.L;
    const long long rows = r * m->D.L + j[OWN_HEAD].nrows;
    const long long tiles = (rows + 3) / 4;
    m->cta_row0[c] = row;
    m->cta_tiles[c] = (int)tiles;
    row += tiles * 4;
    if (j[OWN_UP].ws * 16 > m->up_cols_max) m->up_cols_max = j[OWN_UP].ws * 16;
    if (j[OWN_DOWN].ks * 16 > m->hid_max) m->hid_max = j[OWN_DOWN].ks * 16;
  }
  m->total_rows = row;
  for (int g = 0; g < m->D.Hkv; ++g) {
    const int sz = own_group_begin(g + 1, G, m->D.Hkv) - own_group_begin(g, G, m->D.Hkv);
    if (sz > m->gmax) m->gmax = sz;
  }
}

int owner_create(int device, DeviceState* st, const OwnDims& D, int norm_type, int act, int use_rope, float eps, int Tmax,
                 const OwnLayerPtrs* layers, const void* nf_g, const void* nf_b, const void* head_w, const void* head_b,
                 OwnerModel** out) {
  *out = nullptr;
  OwnerModel* m = new OwnerModel();
  m->device = device;
  m->G = st->sm_count;
  m->D = D;
  m->norm_type = norm_type;
  m->act = act;
  m->use_rope = use_rope;
  m->eps = eps;
  m->Tmax = Tmax;
  m->layers.assign(layers, layers + D.L);
  m->nf_g = nf_g; m->nf_b = nf_b; m->head_w = head_w; m->head_b = head_b;
  owner_plan(m);
  const int G = m->G, grp = D.H / D.Hkv, QW = (grp + 2) * D.hd;
  auto alloc = [&](void** p, size_t bytes, bool zero) -> int {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 256);
    if (e != cudaSuccess) {
      cudaGetLastError();
      set_last_error("OOM: owner-partitioned decode step: cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
      return 0;
    }
    if (zero && cudaMemset(*p, 0, bytes ? bytes : 256) != cudaSuccess) {
      set_last_error("owner-partitioned decode step: cudaMemset failed");
      return 0;
    }
    return 1;
  };
  std::vector<OwnLayerDev> ld(D.L);
  for (int k = 0; k < D.L; ++k) {
    const OwnLayerPtrs& s = layers[k];
    OwnLayerDev& t = ld[k];
    t.g1 = (const __half*)s.n1_g; t.b1n = norm_type == 0 ? (const __half*)s.n1_b : nullptr;
    t.bqkv = (const __half*)s.bqkv; t.bo = (const __half*)s.bo;
    t.g2 = (const __half*)s.n2_g; t.b2n = norm_type == 0 ? (const __half*)s.n2_b : nullptr;
    t.bup = (const __half*)s.b1; t.bdown = (const __half*)s.b2;
    t.cK = (__half*)s.cK; t.cV = (__half*)s.cV;
  }
  m->cnt_bytes = (size_t)(2 * D.L + D.L * D.Hkv * 2 + 1) * kOwnCntStride * sizeof(unsigned);
  const bool ok = alloc((void**)&m->wstream, (size_t)m->total_rows * kOwnRowBytes, false) &&
                  alloc((void**)&m->d_row0, (size_t)G * sizeof(long long), false) && alloc((void**)&m->d_tiles, (size_t)G * sizeof(int), false) &&
                  alloc((void**)&m->d_jobs, m->jobs.size() * sizeof(OwnJob), false) &&
                  alloc((void**)&m->d_layers, ld.size() * sizeof(OwnLayerDev), false) &&
                  alloc((void**)&m->X, (size_t)3 * kOwnMaxRows * D.d * sizeof(long long), true) &&
                  alloc((void**)&m->QA, (size_t)2 * D.Hkv * kOwnMaxRows * QW * sizeof(long long), true) &&
                  alloc((void**)&m->AP, (size_t)kOwnMaxRows * D.Hkv * grp * m->gmax * (D.hd + 2) * sizeof(float), true) &&
                  alloc((void**)&m->cnt, m->cnt_bytes, true);
  if (!ok || cudaMemcpy(m->d_row0, m->cta_row0.data(), (size_t)G * sizeof(long long), cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaMemcpy(m->d_tiles, m->cta_tiles.data(), (size_t)G * sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaMemcpy(m->d_jobs, m->jobs.data(), m->jobs.size() * sizeof(OwnJob), cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaMemcpy(m->d_layers, ld.data(), ld.size() * sizeof(OwnLayerDev), cudaMemcpyHostToDevice) != cudaSuccess) {
    if (ok) set_last_error("owner-partitioned decode step: table upload failed");
    owner_destroy(m);
    return 0;
  }
  *out = m;
  return 1;
}

// (Re)builds the CTAs' weight streams from the engine's packed matrices.
int owner_repack(OwnerModel* m, cudaStream_t s) {
  const OwnDims& D = m->D;
  const int grp = D.H / D.Hkv;
  const int Nqkv = (D.H + 2 * D.Hkv) * D.hd;
  OwnPackArgs p{};
  p.wstream = m->wstream; p.cta_row0 = m->d_row0; p.jobs = m->d_jobs;
  p.grp = grp; p.hd = D.hd; p.H = D.H; p.Hkv = D.Hkv;
  for (int k = 0; k <= D.L; ++k) {
    for (int q = 0; q < 5; ++q) {
      if ((k < D.L) != (q != OWN_HEAD)) continue;
      p.kind = q;
      switch (q) {
        case OWN_QKV: p.Wp = (const __half*)m->layers[k].wqkv; p.K = D.d; p.N = Nqkv; break;
        case OWN_W0: p.Wp = (const __half*)m->layers[k].wo; p.K = D.H * D.hd; p.N = D.d; break;
        case OWN_UP: p.Wp = (const __half*)m->layers[k].w1; p.K = D.d; p.N = D.F * (D.glu ? 2 : 1); break;
        case OWN_DOWN: p.Wp = (const __half*)m->layers[k].w2; p.K = D.F; p.N = D.d; break;
        default: p.Wp = (const __half*)m->head_w; p.K = D.d; p.N = D.V; break;
      }
      p.layer = k;
      own_pack_kernel<<<m->G, 256, 0, s>>>(p);
    }
  }
  // the tail of a CTA's last tile (rows beyond its last job) is read by the ring but never used: clear it once
  for (int c = 0; c < m->G; ++c) {
    const long long rows = m->rows_layer[c] * D.L + m->jobs[(size_t)c * 5 + OWN_HEAD].nrows;
    const long long pad = (long long)m->cta_tiles[c] * 4 - rows;
    if (pad > 0) TSB_CUDA(cudaMemsetAsync(m->wstream + (size_t)(m->cta_row0[c] + rows) * kOwnRowBytes, 0, (size_t)pad * kOwnRowBytes, s));
  }
  TSB_TRY(check_launch("owner repack"));
  m->packed = true;
  return 1;
}

bool owner_packed(const OwnerModel* m) { return m && m->packed; }
void owner_invalidate(OwnerModel* m) {
  if (m) m->packed = false;
}
int owner_reset_counters(OwnerModel* m) {
  if (m && m->cnt) cudaMemset(m->cnt, 0, m->cnt_bytes);
  return 1;
}
long long owner_stream_bytes(const OwnerModel* m) { return m ? m->total_rows * (long long)kOwnRowBytes : 0; }

// One decode step for M rows whose embedded fp32 rows are in `x`.  Returns 1 ok, 0 error, 2 not applicable (the caller
// takes another path).
int owner_launch(OwnerModel* m, DeviceState* st, int M, const float* x, float* logits, const float2* rope_tab, const int* dT,
                 int* error_flag, unsigned poll_limit, bool pdl, cudaStream_t s) {
  if (!m || !m->packed || M < 1 || M > kOwnMaxRows || !error_flag || !dT) return 2;
  const OwnDims& D = m->D;
  const int grp = D.H / D.Hkv, QW = (grp + 2) * D.hd;
  OwnArgs a{};
  a.wstream = m->wstream; a.cta_row0 = m->d_row0; a.cta_tiles = m->d_tiles; a.jobs = m->d_jobs; a.layers = m->d_layers;
  a.gF = (const __half*)m->nf_g; a.bF = m->norm_type == 0 ? (const __half*)m->nf_b : nullptr; a.head_b = (const __half*)m->head_b;
  a.logits = logits;
  for (int i = 0; i < 3; ++i) a.X[i] = m->X + (size_t)i * kOwnMaxRows * D.d;
  for (int i = 0; i < 2; ++i) a.QA[i] = m->QA + (size_t)i * D.Hkv * kOwnMaxRows * QW;
  a.AP = m->AP; a.cnt = m->cnt; a.rope_tab = rope_tab; a.dT = dT; a.error_flag = error_flag;
  a.poll_limit = poll_limit ? poll_limit : kPollLimit;
  a.L = D.L; a.M = M; a.d = D.d; a.H = D.H; a.Hkv = D.Hkv; a.hd = D.hd; a.grp = grp; a.F = D.F; a.V = D.V; a.Tmax = m->Tmax;
  a.glu = D.glu; a.act = m->act; a.xmode = m->norm_type == 0 ? 2 : 1; a.use_rope = m->use_rope; a.gmax = m->gmax;
  a.eps = m->eps; a.scale = 1.0f / sqrtf((float)D.hd);
  if (a.use_rope && !rope_tab) return 2;
  // shared memory behind the ring: {xs | red} aliased by the attention merge area, then ys, hs, qs, gsum, barriers
  auto up = [](size_t v, size_t al) { return (v + al - 1) / al * al; };
  a.xstride = D.d + 8; a.ystride = grp * D.hd + 8; a.hstride = m->hid_max + 8; a.qstride = QW;
  const size_t xs_b = up((size_t)M * a.xstride * 2, 128);
  const size_t red_b = up((size_t)kConsumerWarps * kOwnKChunk * 16 * M * 4, 128);
  const int lpt = D.hd / 8, tpw = 32 / lpt, GH = (grp % 4 == 0) ? 4 : 1;
  const size_t merge_b = up((size_t)kConsumerWarps * tpw * GH * (D.hd + 2) * 4, 128);
  size_t off = 0;
  a.off_xs = 0; a.off_red = (int)xs_b; a.off_merge = 0;
  off = xs_b + red_b > merge_b ? xs_b + red_b : merge_b;
  a.off_ys = (int)off; off += up((size_t)M * a.ystride * 2, 128);
  a.off_hs = (int)off; off += up((size_t)M * a.hstride * 2, 128);
  a.off_qs = (int)off; off += up((size_t)M * a.qstride * 4, 128);
  a.gsum_cols = m->up_cols_max;
  a.off_gsum = (int)off; off += up((size_t)M * a.gsum_cols * 4, 128);
  a.off_bar = (int)off; off += 32 * sizeof(uint64_t);
  const size_t fixed = off + 1024 /* alignment slack */ + 128;
  const size_t budget = 225 * 1024;  // the kernel also has some static shared memory
  if (fixed + 4 * (size_t)kOwnTileBytes > budget) return 2;
  int stages = (int)((budget - fixed) / kOwnTileBytes);
  if (stages > 16) stages = 16;
  a.stages = stages;
  const size_t smem = fixed + (size_t)stages * kOwnTileBytes;
  {
    // the CTAs wait on one another: the whole grid must be resident at once
    int per_sm = 0;
    TSB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_owner_kernel, kStreamThreads, smem));
    if ((long long)per_sm * st->sm_count < m->G) return 2;
  }
  {
    const int qa_words = D.Hkv * kOwnMaxRows * QW;
    TSB_CUDA(launch_k(own_init_kernel, dim3(16), dim3(256), 0, s, a.X[0], a.X[1], a.X[2], a.QA[0], x, M, D.d, qa_words));
    count_launch(m->device);
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(m->G);
  cfg.blockDim = dim3(kStreamThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  TSB_CUDA(cudaLaunchKernelEx(&cfg, decode_owner_kernel, a));
  count_launch(m->device);
  return 1;
}

// ------------------------------------------------------------------------------------------- layout self-test (host only)
// Walks every CTA's jobs the way the kernel's consumer warps do (the loop nests of own_job_ksplit / own_job_ssplit,
// restated on the host) and checks, block by block, that the re-packer's placement rule (own_block_coords) puts exactly
// the block the consumer expects at the row it reads next, that every (k-step, strip) of a share is visited once, that
// shares tile each matrix without gaps or overlaps, and that the streams are contiguous.  Needs no GPU.
static int own_selftest_job(const OwnJob& j, std::vector<int>& seen, int ks_total_stride) {
  (void)ks_total_stride;
  seen.assign((size_t)(j.ks > 0 ? j.ks : 1) * (j.ws > 0 ? j.ws : 1), 0);
  if (j.nrows == 0) return 1;
  for (int w = 0; w < 8; ++w) {
    int row = 0;
    if (j.mode == OWN_KSPLIT) {
      for (int c = 0; c < j.nchunks; ++c) {
        const int left = j.ws - c * kOwnKChunk, wc = left < kOwnKChunk ? left : kOwnKChunk;
        for (int kk = 0; kk < j.ksw; ++kk) {
          const int kst = w * j.ksw + kk;
          for (int s = 0; s < kOwnKChunk; ++s) {
            if (s >= wc) continue;
            int kstep, strip;
            bool live;
            own_block_coords(j, row, w, kstep, strip, live);
            TSB_CHECK(kstep == kst && strip == c * kOwnKChunk + s && live == (kst < j.ks),
                      "owner layout: K-split job kind %d: row %d warp %d holds (k-step %d, strip %d) but the consumer expects (%d, %d)",
                      j.kind, row, w, kstep, strip, kst, c * kOwnKChunk + s);
            if (live) seen[(size_t)kstep * j.ws + strip] += 1;
            ++row;
          }
        }
      }
    } else {
      for (int c = 0; c < j.nchunks; ++c)
        for (int k = 0; k < j.ks; ++k)
          for (int s = 0; s < kOwnMaxSpw; ++s) {
            if (s >= j.spw) continue;
            const int want = c * 8 * j.spw + w * j.spw + s;
            int kstep, strip;
            bool live;
            own_block_coords(j, row, w, kstep, strip, live);
            TSB_CHECK(kstep == k && strip == want && live == (want < j.ws),
                      "owner layout: strip-split job kind %d: row %d warp %d holds (k-step %d, strip %d) but the consumer expects (%d, %d)",
                      j.kind, row, w, kstep, strip, k, want);
            if (live) seen[(size_t)kstep * j.ws + strip] += 1;
            ++row;
          }
    }
    TSB_CHECK(row == j.nrows, "owner layout: job kind %d: warp %d consumes %d rows, the job has %d", j.kind, w, row, j.nrows);
  }
  for (size_t i = 0; i < (size_t)j.ks * j.ws; ++i)
    TSB_CHECK(seen[i] == 1, "owner layout: job kind %d: block %zu of the share is visited %d times", j.kind, i, seen[i]);
  return 1;
}

int owner_layout_selftest(const OwnDims& D, int G) {
  OwnerModel m;
  m.G = G;
  m.D = D;
  owner_plan(&m);
  const int grp = D.H / D.Hkv, KS = D.d / 16, DS = D.d / 16, VS = own_ceil(D.V, 16);
  const int up_strips = D.F / 16 * (D.glu ? 2 : 1);
  // coverage of every matrix by the CTAs' shares: count how often each (k-step, strip) of the matrix is owned
  std::vector<int> qkv((size_t)D.Hkv * KS, 0), w0((size_t)D.Hkv * DS, 0), up(up_strips, 0), down(D.F / 16, 0), head(VS, 0), seen;
  long long expect_row = 0;
  for (int c = 0; c < G; ++c) {
    const OwnJob* j = &m.jobs[(size_t)c * 5];
    TSB_CHECK(m.cta_row0[c] == expect_row, "owner layout: the stream of CTA %d does not follow its predecessor", c);
    long long r = 0;
    for (int q = 0; q < 4; ++q) {
      TSB_CHECK(j[q].row0 == r, "owner layout: CTA %d job %d starts at row %lld, expected %lld", c, q, j[q].row0, r);
      r += j[q].nrows;
    }
    TSB_CHECK(j[OWN_HEAD].row0 == r * D.L, "owner layout: CTA %d: LM-head rows do not follow the layers", c);
    const long long rows = r * D.L + j[OWN_HEAD].nrows;
    TSB_CHECK((long long)m.cta_tiles[c] * 4 >= rows && (long long)m.cta_tiles[c] * 4 < rows + 4, "owner layout: CTA %d: tile count", c);
    expect_row += (long long)m.cta_tiles[c] * 4;
    for (int q = 0; q < 5; ++q) {
      TSB_TRY(own_selftest_job(j[q], seen, 0));
      TSB_CHECK(j[q].mode == OWN_SSPLIT ? (j[q].spw <= kOwnMaxSpw) : true, "owner layout: strips per warp");
    }
    const int g = j[OWN_QKV].group;
    TSB_CHECK(g >= 0 && g < D.Hkv && c >= own_group_begin(g, G, D.Hkv) && c < own_group_begin(g + 1, G, D.Hkv), "owner layout: group of CTA %d", c);
    TSB_CHECK(j[OWN_QKV].ws == 0 || j[OWN_QKV].ws == (grp + 2) * D.hd / 16, "owner layout: q|k|v width");
    for (int k = 0; k < j[OWN_QKV].ks; ++k) qkv[(size_t)g * KS + j[OWN_QKV].kbase / 16 + k] += 1;
    TSB_CHECK(j[OWN_W0].ws == 0 || (j[OWN_W0].ks == grp * D.hd / 16 && j[OWN_W0].kbase == g * grp * D.hd), "owner layout: W0 rows of CTA %d", c);
    for (int s = 0; s < j[OWN_W0].ws; ++s) w0[(size_t)g * DS + j[OWN_W0].cbase / 16 + s] += 1;
    for (int s = 0; s < j[OWN_UP].ws; ++s) up[j[OWN_UP].cbase / 16 + s] += 1;
    TSB_CHECK(j[OWN_UP].ws == 0 || j[OWN_UP].ks == KS, "owner layout: FFN up covers all of K");
    for (int k = 0; k < j[OWN_DOWN].ks; ++k) down[j[OWN_DOWN].kbase / 16 + k] += 1;
    TSB_CHECK(j[OWN_DOWN].ks == 0 || j[OWN_DOWN].ws == DS, "owner layout: FFN down covers all columns");
    // the hidden units a CTA produces are the rows of W2 it multiplies
    TSB_CHECK(j[OWN_UP].cbase == j[OWN_DOWN].kbase * (D.glu ? 2 : 1) && j[OWN_UP].ws == j[OWN_DOWN].ks * (D.glu ? 2 : 1),
              "owner layout: CTA %d: FFN up columns and FFN down rows do not match", c);
    for (int s = 0; s < j[OWN_HEAD].ws; ++s) head[j[OWN_HEAD].cbase / 16 + s] += 1;
  }
  TSB_CHECK(expect_row == m.total_rows, "owner layout: total rows");
  for (int v : qkv) TSB_CHECK(v == 1, "owner layout: a k-step of a group's q|k|v is owned %d times", v);
  for (int v : w0) TSB_CHECK(v == 1, "owner layout: a column strip of a group's W0 is owned %d times", v);
  for (int v : up) TSB_CHECK(v == 1, "owner layout: a column strip of FFN up is owned %d times", v);
  for (int v : down) TSB_CHECK(v == 1, "owner layout: a k-step of FFN down is owned %d times", v);
  for (int v : head) TSB_CHECK(v == 1, "owner layout: a column strip of the LM head is owned %d times", v);
  // fragment coordinates: the 32 x 8 values of a block are the 16 x 16 block, each once
  int cover[16][16] = {};
  for (int lane = 0; lane < 32; ++lane)
    for (int e = 0; e < 8; ++e) {
      int k, c;
      own_frag_coords(lane, e, k, c);
      TSB_CHECK(k >= 0 && k < 16 && c >= 0 && c < 16, "owner layout: fragment coordinates out of range");
      cover[k][c] += 1;
    }
  for (int k = 0; k < 16; ++k)
    for (int c = 0; c < 16; ++c) TSB_CHECK(cover[k][c] == 1, "owner layout: fragment element (%d, %d) appears %d times", k, c, cover[k][c]);
  // group-local q|k|v columns map onto distinct columns of the packed matrix
  std::vector<int> cols((size_t)(D.H + 2 * D.Hkv) * D.hd, 0);
  for (int g = 0; g < D.Hkv; ++g)
    for (int jc = 0; jc < (grp + 2) * D.hd; ++jc) cols[own_qkv_col(jc, g, grp, D.hd, D.H, D.Hkv)] += 1;
  for (int v : cols) TSB_CHECK(v == 1, "owner layout: a q|k|v column is mapped %d times", v);
  return 1;
}

int init_owner_attrs() {
  TSB_CUDA(cudaFuncSetAttribute(decode_owner_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  return 1;
}

}  // namespace tsb

extern "C" int TSB200_OwnerLayoutSelfTest(int L, int d, int H, int Hkv, int hd, int F, int V, int glu, int n_ctas) {
  using namespace tsb;
  OwnDims D{};
  D.L = L; D.d = d; D.H = H; D.Hkv = Hkv; D.hd = hd; D.F = F; D.V = V; D.glu = glu;
  TSB_CHECK(n_ctas >= 1 && L >= 1 && Hkv >= 1 && H % Hkv == 0, "owner_layout_self_test: bad arguments");
  TSB_CHECK(owner_applicable(D, TSB200_F16, n_ctas), "owner_layout_self_test: this shape is not served by the owner-partitioned kernel");
  return owner_layout_selftest(D, n_ctas);
}
