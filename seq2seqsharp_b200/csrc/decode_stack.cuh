// Device code shared by the persistent decode-step kernels (decode_stack.cu: CUDA-core consumers, any dtype;
// decode_stack_mma.cu: warp-level tensor-core consumers, fp16): the argument block, the global-counter protocol between CTAs, input
// staging with the fused norms, and the in-kernel RoPE + cache append + split-K attention.
#pragma once
#include "kernels.cuh"
#include "stream_common.cuh"

namespace tsb {

constexpr unsigned kPollLimit = 1u << 21;   // acquire-polls of a global counter before giving up (~1 s)
constexpr int kDoneStride = 8;              // one 32-byte sector per operation counter
constexpr int kMaxStackSplits = 16;

struct StackArgs {
  const StackOp* ops;
  int n_ops;
  int stages;
  int union_bytes;          // shared memory shared by {x staging (+ warp reduction)} and the attention merge
  int xs_bytes;             // bytes of the x staging area inside the union
  StackConfig c;
  float scale;              // 1/sqrt(hd)
  float* partials;          // linear: [CT][max_contrib][M][NT]
  unsigned int* counters;   // linear: per column tile, self-resetting
  unsigned int* attn_cnt;   // attention: per (row, head group), self-resetting
  unsigned int* done;       // [n_ops + 1][kDoneStride]; the last slot counts CTAs that left the kernel
  float* attn_part;         // [M*H][kMaxStackSplits][hd + 2]
  int* error_flag;
  int defer;                // when the ring slots of an operation's last tiles go back to the producer: 0 at once, 1 after the
                            // partial sums are published, 2 after the operation's epilogue (default)
  long long* trace;         // optional [grid][n_ops][8] timestamps (+ [grid][8] cycle counters of the MMA warp)
  unsigned poll_limit;      // acquire-polls of a dependency counter before a CTA gives up (kPollLimit unless the host set one)
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Counting arrival with release + acquire semantics at GPU scope.  Called by ONE thread after a CTA barrier: the
// release is cumulative, so it also publishes the stores the other threads made before the barrier, and the acquire
// lets the CTA (after the next barrier) read what earlier arrivers published.  One round trip instead of a fence by
// every thread followed by the atomic.
__device__ __forceinline__ unsigned atom_add_acq_rel(unsigned* p, unsigned v) {
  unsigned old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
// System-scope forms for counters that other GPUs increment over NVLink (tensor parallelism).  Counters are
// monotonic across launches (epochs), compared wrap-safe.
__device__ __forceinline__ void red_release_add_sys(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// fence.sys by the caller + this relaxed add form a release pattern; used when one thread per peer signals, so that the
// fences (each waits for the peer stores to be acknowledged over NVLink) run side by side instead of one after another
__device__ __forceinline__ void red_relaxed_add_sys(unsigned* p, unsigned v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool poll_count_sys(const unsigned* p, unsigned want, unsigned limit, const int* err) {
  for (unsigned i = 0; i < limit; ++i) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    if ((int)(v - want) >= 0) return true;
    if ((i & 1023u) == 1023u && *(volatile const int*)err) return false;
  }
  return false;
}
__device__ __forceinline__ float* stack_xch(const StackConfig& c, int dest_rank, int site, int src_rank) {
  return reinterpret_cast<float*>(c.peer[dest_rank] + kStackXchHeader) +
         ((size_t)(site * c.tp_size + src_rank) * kStackXchRows) * c.d;
}
// Bounded acquire-poll until *p >= target.  Also gives up early when another CTA has raised the error word.
__device__ __forceinline__ bool poll_count(const unsigned* p, unsigned target, unsigned limit, const int* err) {
  for (unsigned i = 0; i < limit; ++i) {
    if (ld_acquire_u32(p) >= target) return true;
    if ((i & 1023u) == 1023u && *(volatile const int*)err) return false;
  }
  return false;
}
// the eight worker (consumer) warps are threads 0..255 in both kernels
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Geometry of one linear for a grid of G CTAs: CTAs 0..Gop-1 each own a contiguous, evenly sized range of the
// KB*CT tiles (column-tile-major), so no range is empty.
struct LinGeom {
  int KB, CT, Gop;
  long long U;
};
template <typename T>
__host__ __device__ __forceinline__ LinGeom lin_geom(int K, int N, int G) {
  constexpr int NT = 32 * (16 / (int)sizeof(T));
  LinGeom g;
  g.KB = (K + kKT - 1) / kKT;
  g.CT = (N + NT - 1) / NT;
  g.U = (long long)g.KB * g.CT;
  g.Gop = g.U < G ? (int)g.U : G;
  return g;
}

// Walks this CTA's weight tiles over the linear operations of the program, in the order they are streamed.
template <typename T>
struct TileCursor {
  int op_i = -1, u = 0, u_end = 0;
  const unsigned char* src = nullptr;
  __device__ __forceinline__ bool next(const StackArgs& a, const unsigned char*& out) {
    while (u >= u_end) {
      if (++op_i >= a.n_ops) return false;
      const StackOp* op = a.ops + op_i;
      if (op->type != 0) continue;
      const LinGeom g = lin_geom<T>(op->K, op->N, (int)gridDim.x);
      if ((int)blockIdx.x >= g.Gop) continue;
      u = (int)(g.U * blockIdx.x / g.Gop);
      u_end = (int)(g.U * (blockIdx.x + 1) / g.Gop);
      src = reinterpret_cast<const unsigned char*>(op->Wp) + (size_t)u * kTileBytes;
    }
    out = src;
    src += kTileBytes;
    ++u;
    return true;
  }
};
// The weight stream of one CTA (one lane): tiles go through the shared-memory ring in program order, across the
// boundaries of the operations, never waiting for activations.  (Requesting tiles into L2 ahead of the ring was
// measured and does not help: refilling the ring from L2 is no faster than from HBM.)
template <typename T>
__device__ __forceinline__ void stack_stream_tiles(const StackArgs& a, unsigned char* stage_mem, uint64_t* full, uint64_t* empty,
                                                   volatile int* s_err) {
  const int S = a.stages;
  int s = 0;
  unsigned round = 0;
  long long issued = 0;
  TileCursor<T> fetch;
  const unsigned char* src;
  while (fetch.next(a, src)) {
    if (round > 0) {
      // short waits, so that a CTA whose workers gave up (they stop handing slots back) leaves at once
      bool got = false;
      for (unsigned t = 0; t < (kSpinLimit >> 10) && !got && !*s_err; ++t) got = mbar_wait(&empty[s], (round - 1u) & 1u, 1024u);
      if (!got) {
        *s_err = 1;
        break;
      }
    }
    if (*s_err) break;
    mbar_expect_tx(&full[s], kTileBytes);
    bulk_g2s(stage_mem + (size_t)s * kTileBytes, src, kTileBytes, &full[s]);
    ++issued;
    if (++s == S) {
      s = 0;
      ++round;
    }
  }
  if (*s_err) {
    // drain: await (bounded) every copy that was issued and possibly not consumed, so nothing lands after exit
    const long long first = issued > S ? issued - S : 0;
    for (long long j = first; j < issued; ++j) mbar_wait(&full[(int)(j % S)], (unsigned)((j / S) & 1));
    if (a.error_flag) *a.error_flag = 1;
  }
}

// Time stamps for kernel development exist only in builds with -DTSB200_TRACE; the shipped kernels carry none.
#ifdef TSB200_TRACE
#define STRACE(op_i, slot)                                                                        \
  do {                                                                                            \
    if (a.trace && threadIdx.x == 0) a.trace[((size_t)blockIdx.x * a.n_ops + (op_i)) * 8 + (slot)] = gtimer(); \
  } while (0)
#else
#define STRACE(op_i, slot) do { } while (0)
#endif

// ------------------------------------------------------------------------------------------- x staging (workers)
// All loads of activations are L2-coherent (__ldcg): they were written by other SMs earlier in this same kernel.
// Loads are gathered into registers in batches before anything is stored to shared memory, so that their
// latencies overlap.
template <typename T>
__device__ __forceinline__ void stage_plain(T* xs, const T* x, int M, int K, int Kp, int tid) {
  constexpr int XB = 8;
  for (int m = 0; m < M; ++m) {
    for (int k0 = 0; k0 < Kp; k0 += 256 * XB) {
      T v[XB];
#pragma unroll
      for (int j = 0; j < XB; ++j) {
        const int k = k0 + j * 256 + tid;
        const T xv = __ldcg(x + (size_t)m * K + (k < K ? k : 0));
        v[j] = (k < K) ? xv : from_f<T>(0.0f);
      }
#pragma unroll
      for (int j = 0; j < XB; ++j) {
        const int k = k0 + j * 256 + tid;
        if (k < Kp) xs[m * Kp + k] = v[j];
      }
    }
  }
}

// 16-byte variant of stage_plain for rows whose length is a multiple of 16 bytes: up to 8 vectors per thread in
// flight, so rows of up to 2048 vectors (16 K halves) cost ONE memory round trip instead of one per 2048 elements.
template <typename T>
__device__ __forceinline__ void stage_plain_vec(T* xs, const T* x, int M, int K, int Kp, int tid) {
  constexpr int EPV = 16 / (int)sizeof(T);
  const int nv = K / EPV, nvp = Kp / EPV;  // K % EPV == 0 (checked by the caller); Kp is a multiple of 32
  for (int m = 0; m < M; ++m) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)m * K);
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)m * Kp);
    for (int v0 = 0; v0 < nvp; v0 += 256 * 8) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = v0 + j * 256 + tid;
        const uint4 t = __ldcg(src + (i < nv ? i : 0));
        v[j] = (i < nv) ? t : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = v0 + j * 256 + tid;
        if (i < nvp) dst[i] = v[j];
      }
    }
  }
}

// Slice variant: a CTA whose tile range is shorter than one pass over K only needs the n_t k-tiles it streams
// (k-tile (kb0 + i) % KB for i < n_t); they are staged back to back, so a wide FFN-down input costs a few KB of shared
// memory per sequence instead of the whole row.  K % 8 == 0.
__device__ __forceinline__ void stage_plain_slice(__half* xs, const __half* x, int M, int K, int KB, int kb0, int n_t, int Ks, int tid) {
  const int nv = n_t * 4;  // 16-byte vectors per row: four per k-tile
  for (int m = 0; m < M; ++m) {
    for (int v0 = 0; v0 < nv; v0 += 256 * 4) {
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = v0 + j * 256 + tid;
        int kb = kb0 + (i >> 2);
        if (kb >= KB) kb -= KB;
        const int k = kb * kKT + (i & 3) * 8;
        const bool ok = i < nv && k + 8 <= K;
        const uint4 t = __ldcg(reinterpret_cast<const uint4*>(x + (size_t)m * K + (ok ? k : 0)));
        v[j] = ok ? t : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = v0 + j * 256 + tid;
        if (i < nv) *reinterpret_cast<uint4*>(xs + (size_t)m * Ks + i * 8) = v[j];
      }
    }
  }
}

// Norm gains (and LayerNorm biases) of a row of up to 256*16 elements, fetched BEFORE the dependency wait: they are
// constants, and their HBM latency would otherwise sit on the critical path of every layer.
template <typename T>
struct NormConsts {
  T g[16], b[16];
};
template <typename T>
__device__ __forceinline__ void load_norm_consts(NormConsts<T>& nc, const T* gamma, const T* beta_or_null, int K, int tid) {
  const T* beta = beta_or_null ? beta_or_null : gamma;  // every address a thread can form stays valid
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int k = j * 256 + tid;
    const int kc = k < K ? k : 0;
    nc.g[j] = gamma[kc];
    nc.b[j] = beta[kc];
  }
}

// RMSNorm (xmode 1) or LayerNorm (xmode 2) of the fp32 rows; XR*256 >= K elements of a row live in registers.
// Same arithmetic as the stand-alone norm kernels: fp32 sums, sqrt, divide.  `nc` (XR == 16 only) holds the
// pre-fetched gains; otherwise they are loaded here.
template <typename T, int XR>
__device__ __forceinline__ void stage_norm(T* xs, const float* x, const T* gamma, const T* beta_or_null, const NormConsts<T>* nc,
                                           int xmode, float eps, int M, int K, int Kp, int tid, float* s_stat) {
  constexpr int XB = 8;
  const int lane = tid & 31, w = tid >> 5;
  const float beta_on = beta_or_null ? 1.0f : 0.0f;
  const T* beta = beta_or_null ? beta_or_null : gamma;
  for (int m = 0; m < M; ++m) {
    float xr[XR];
#pragma unroll
    for (int j = 0; j < XR; ++j) {
      const int k = j * 256 + tid;
      const float xv = __ldcg(x + (size_t)m * K + (k < K ? k : 0));
      xr[j] = (k < K) ? xv : 0.0f;
    }
    float s1 = 0.0f;
#pragma unroll
    for (int j = 0; j < XR; ++j) s1 += (xmode == 2) ? xr[j] : xr[j] * xr[j];
    s1 = warp_sum(s1);
    if (lane == 0) s_stat[(m & 3) * 8 + w] = s1;
    consumers_sync();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kConsumerWarps; ++i) tot += s_stat[(m & 3) * 8 + i];
    float mean = 0.0f, inv;
    if (xmode == 2) {
      mean = tot / K;
      float s2 = 0.0f;
#pragma unroll
      for (int j = 0; j < XR; ++j) {
        const float e = (j * 256 + tid < K) ? xr[j] - mean : 0.0f;
        s2 += e * e;
      }
      s2 = warp_sum(s2);
      if (lane == 0) s_stat[32 + (m & 3) * 8 + w] = s2;
      consumers_sync();
      float t2 = 0.0f;
#pragma unroll
      for (int i = 0; i < kConsumerWarps; ++i) t2 += s_stat[32 + (m & 3) * 8 + i];
      inv = sqrtf(eps + t2 / K);
    } else {
      inv = sqrtf(tot / (float)K + eps);
    }
#pragma unroll
    for (int j0 = 0; j0 < XR; j0 += XB) {
      if (j0 * 256 >= Kp) break;
      float gv[XB], bv[XB];
#pragma unroll
      for (int j = 0; j < XB; ++j) {
        const int k = (j0 + j) * 256 + tid;
        const int kc = k < K ? k : 0;
        if (XR == 16 && nc) {
          gv[j] = to_f<T>(nc->g[(j0 + j) & 15]);
          bv[j] = beta_on * to_f<T>(nc->b[(j0 + j) & 15]);
        } else {
          gv[j] = to_f<T>(gamma[kc]);
          bv[j] = beta_on * to_f<T>(beta[kc]);
        }
      }
#pragma unroll
      for (int j = 0; j < XB; ++j) {
        const int k = (j0 + j) * 256 + tid;
        if (k < Kp) xs[m * Kp + k] = from_f<T>((k < K) ? gv[j] * ((xr[j0 + j] - mean) / inv) + bv[j] : 0.0f);
      }
    }
  }
}

// RMSNorm / LayerNorm prologue for rows of up to 4096 elements with K % 4 == 0: every thread owns up to four groups
// of four consecutive elements (float4 loads of the fp32 row, 8-byte loads of the gains, one 8- or 16-byte store per
// group).  Same arithmetic as stage_norm (fp32 sums in a different, fixed order; sqrt; divide).  The gains are
// fetched BEFORE the dependency wait (norm_vec_consts) because they are constants.
template <typename T>
struct NormVecConsts {
  T g[4][4], b[4][4];
  float beta_on;
};
template <typename T>
__device__ __forceinline__ void norm_vec_consts(NormVecConsts<T>& nc, const T* gamma, const T* beta_or_null, int K, int tid) {
  const T* beta = beta_or_null ? beta_or_null : gamma;  // every address a thread can form stays valid
  nc.beta_on = beta_or_null ? 1.0f : 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int k = (j * 256 + tid) * 4;
    const int kc = k < K ? k : 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      nc.g[j][e] = gamma[kc + e];
      nc.b[j][e] = beta[kc + e];
    }
  }
}
template <typename T> struct St4;
template <> struct St4<__half> {
  static __device__ __forceinline__ void st(__half* p, const float* f) {
    uint2 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
    h[0] = __floats2half2_rn(f[0], f[1]);
    h[1] = __floats2half2_rn(f[2], f[3]);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};
template <> struct St4<float> {
  static __device__ __forceinline__ void st(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
template <typename T>
__device__ __forceinline__ void stage_norm_vec(T* xs, const float* x, const NormVecConsts<T>& nc, int xmode, float eps, int M, int K,
                                               int Kp, int tid, float* s_stat, const float* xsum = nullptr, int n_sum = 0,
                                               size_t sum_stride = 0, float* x_out = nullptr) {
  const int lane = tid & 31, w = tid >> 5;
  for (int m = 0; m < M; ++m) {
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = (j * 256 + tid) * 4;
      const float4 t = __ldcg(reinterpret_cast<const float4*>(x + (size_t)m * K + (k < K ? k : 0)));
      v[j] = (k < K) ? t : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (xsum) {
      // tensor parallelism: the row is the old residual plus every rank's partial sum, added in rank order (the same
      // bits on every rank); the block with index 0 also stores the new residual row
      // two ranks' rows in flight per round trip; added in rank order
      for (int r = 0; r < n_sum; r += 2) {
        const bool two = r + 1 < n_sum;
        float4 p[4], q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = (j * 256 + tid) * 4;
          const size_t o = (size_t)m * K + (k < K ? k : 0);
          p[j] = __ldcg(reinterpret_cast<const float4*>(xsum + (size_t)r * sum_stride + o));
          q[j] = __ldcg(reinterpret_cast<const float4*>(xsum + (size_t)(two ? r + 1 : r) * sum_stride + o));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if ((j * 256 + tid) * 4 < K) {
            v[j].x += p[j].x; v[j].y += p[j].y; v[j].z += p[j].z; v[j].w += p[j].w;
            if (two) {
              v[j].x += q[j].x; v[j].y += q[j].y; v[j].z += q[j].z; v[j].w += q[j].w;
            }
          }
        }
      }
      if (x_out) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = (j * 256 + tid) * 4;
          if (k < K) *reinterpret_cast<float4*>(x_out + (size_t)m * K + k) = v[j];
        }
      }
    }
    float s1 = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      s1 += (xmode == 2) ? (v[j].x + v[j].y) + (v[j].z + v[j].w) : (v[j].x * v[j].x + v[j].y * v[j].y) + (v[j].z * v[j].z + v[j].w * v[j].w);
    s1 = warp_sum(s1);
    if (lane == 0) s_stat[(m & 3) * 8 + w] = s1;
    consumers_sync();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kConsumerWarps; ++i) tot += s_stat[(m & 3) * 8 + i];
    float mean = 0.0f, inv;
    if (xmode == 2) {
      mean = tot / K;
      float s2 = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if ((j * 256 + tid) * 4 < K) {
          const float e0 = v[j].x - mean, e1 = v[j].y - mean, e2 = v[j].z - mean, e3 = v[j].w - mean;
          s2 += (e0 * e0 + e1 * e1) + (e2 * e2 + e3 * e3);
        }
      }
      s2 = warp_sum(s2);
      if (lane == 0) s_stat[32 + (m & 3) * 8 + w] = s2;
      consumers_sync();
      float t2 = 0.0f;
#pragma unroll
      for (int i = 0; i < kConsumerWarps; ++i) t2 += s_stat[32 + (m & 3) * 8 + i];
      inv = sqrtf(eps + t2 / K);
    } else {
      inv = sqrtf(tot / (float)K + eps);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = (j * 256 + tid) * 4;
      if (k < Kp) {
        float o[4];
        const float xv[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = (k < K) ? to_f<T>(nc.g[j][e]) * ((xv[e] - mean) / inv) + nc.beta_on * to_f<T>(nc.b[j][e]) : 0.0f;
        St4<T>::st(xs + (size_t)m * Kp + k, o);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------- attention (workers)
template <typename T> struct Ld16;
template <> struct Ld16<__half> {
  static __device__ __forceinline__ void cg(const __half* p, float* f) {
    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ void st(__half* p, const float* f) {
    uint4 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};
template <> struct Ld16<float> {
  static __device__ __forceinline__ void cg(const float* p, float* f) {
    const float4 raw = __ldcg(reinterpret_cast<const float4*>(p));
    f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w;
  }
  static __device__ __forceinline__ void st(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

// Rotates the EPL elements a lane holds (interleaved pairs) and rounds them to T, as the stand-alone kernel stores them.
template <typename T, int EPL>
__device__ __forceinline__ void rope_round(float* f, const float* cs, const float* sn) {
#pragma unroll
  for (int j = 0; j < EPL / 2; ++j) {
    const float x0 = f[2 * j], x1 = f[2 * j + 1];
    f[2 * j] = to_f<T>(from_f<T>(x0 * cs[j] - x1 * sn[j]));
    f[2 * j + 1] = to_f<T>(from_f<T>(x1 * cs[j] + x0 * sn[j]));
  }
}

// Number of key-range splits of the in-kernel attention: enough items to give every CTA one, at least 32 keys each.
__device__ __forceinline__ int stack_splits(int grid, int M, int ygroups, int Tk) {
  int s = grid / (M * ygroups);
  const int by_len = (Tk + 31) / 32;
  if (s > by_len) s = by_len;
  if (s > kMaxStackSplits) s = kMaxStackSplits;
  if (s < 1) s = 1;
  return s;
}

template <int G, int EPL>
__device__ __forceinline__ void attn_update(const float (*qf)[EPL], const float* kf, const float* vf, float* mx, float* l,
                                            float (*acc)[EPL], int lpt, bool live) {
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float d = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) d += qf[g][e] * kf[e];
    for (int o = lpt >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    if (live) {
      const float mn = fmaxf(mx[g], d);
      const float corr = __expf(mx[g] - mn);  // exp(-inf) = 0 on the first token
      const float p = __expf(d - mn);
      l[g] = l[g] * corr + p;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * corr + p * vf[e];
      mx[g] = mn;
    }
  }
}

// One item = (sequence row, group of G query heads sharing a KV head, split of the key range).  Lane groups of
// lpt = hd/EPL lanes own one cached token per iteration (16-byte loads of its K and V rows, two tokens in flight);
// each lane group runs an online softmax, the 8*tpw states are merged through shared memory and written as this
// split's partial state.  The CTA that delivers the last split of a (row, head group) combines the partial states
// in split order (bitwise reproducible) and stores the attention output rows in T.
// cs / sn: cos / sin of this step's position for the pairs this lane holds (loaded once per kernel).
template <typename T, int G>
__device__ __forceinline__ void stack_attention(const StackArgs& a, const StackOp* op, int op_i, float* merge, volatile int* s_last,
                                                int T0, int splits, const float* cs, const float* sn) {
  constexpr int EPL = TileVec<T>::N;
  const StackConfig& c = a.c;
  const int hd = c.hd, H = c.H, Hkv = c.Hkv, Tmax = c.Tmax;
  const int lpt = hd / EPL, tpw = 32 / lpt;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int sub = lane / lpt, li = lane % lpt;
  const int group = H / Hkv, gpk = group / G, yg = Hkv * gpk;
  const int Tk = min(T0 + 1, Tmax);
  const int per_split = (Tk + splits - 1) / splits;
  const int items = c.M * yg * splits;
  const int rec = hd + 2;
  const T* qkv = reinterpret_cast<const T*>(op->x);
  const T* cK = reinterpret_cast<const T*>(op->cK);
  const T* cV = reinterpret_cast<const T*>(op->cV);
  T* out = reinterpret_cast<T*>(op->ep.y);
  const int nstates = kConsumerWarps * tpw;
  const int stride = kConsumerWarps * tpw;

  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int split = item % splits, y = (item / splits) % yg, row = item / (splits * yg);
    const int kvh = y / gpk, h0 = kvh * group + (y % gpk) * G;
    const int t_beg = split * per_split, t_end = min(Tk, t_beg + per_split);
    const int t_cached_end = min(t_end, T0);
    const T* qrow = qkv + (size_t)row * c.qkv_rs;

    float qf[G][EPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      Ld16<T>::cg(qrow + (size_t)(h0 + g) * hd + li * EPL, qf[g]);
      if (c.use_rope) rope_round<T, EPL>(qf[g], cs, sn);
#pragma unroll
      for (int e = 0; e < EPL; ++e) qf[g][e] *= a.scale;
    }
#ifdef TSB200_TRACE
    if (qf[0][0] == 12345.678f) STRACE(op_i, 7);  // keeps the stamp below after the q loads
#endif
    STRACE(op_i, 4);
    float mx[G], l[G], acc[G][EPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      mx[g] = -INFINITY;
      l[g] = 0.0f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[g][e] = 0.0f;
    }
    const size_t head_off = ((size_t)row * Hkv + kvh) * Tmax * hd + li * EPL;
    const T* Kb = cK + head_off;
    const T* Vb = cV + head_off;
    // cached tokens of this split, four per lane group in flight (one memory round trip for typical split lengths)
    for (int tb = t_beg + w * tpw; tb < t_cached_end; tb += 4 * stride) {
      TileVec<T> kv[4], vv[4];
      bool live[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = tb + i * stride + sub;
        live[i] = t < t_cached_end;  // all lanes iterate together (full-warp shuffles); dead lanes re-read token t_beg
        const size_t o = (size_t)(live[i] ? t : t_beg) * hd;
        kv[i].lds(Kb + o);
        vv[i].lds(Vb + o);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float kf[EPL], vf[EPL];
        kv[i].get(kf);
        vv[i].get(vf);
        attn_update<G, EPL>(qf, kf, vf, mx, l, acc, lpt, live[i]);
      }
    }
    // the token of this step, in the split whose range holds position T0: k (rotated) and v come straight from the
    // q|k|v rows; the first head group of each KV head also appends them to the cache (nobody reads that slot now)
    if ((t_beg <= T0) && (T0 < t_end) && w == 0) {
      float kf[EPL], vf[EPL];
      Ld16<T>::cg(qrow + (size_t)H * hd + (size_t)kvh * hd + li * EPL, kf);
      if (c.use_rope) rope_round<T, EPL>(kf, cs, sn);
      Ld16<T>::cg(qrow + (size_t)(H + Hkv) * hd + (size_t)kvh * hd + li * EPL, vf);
      const bool live = sub == 0;
      if (live && (y % gpk) == 0) {
        Ld16<T>::st(reinterpret_cast<T*>(op->cK) + head_off + (size_t)T0 * hd, kf);
        Ld16<T>::st(reinterpret_cast<T*>(op->cV) + head_off + (size_t)T0 * hd, vf);
      }
      attn_update<G, EPL>(qf, kf, vf, mx, l, acc, lpt, live);
    }
#ifdef TSB200_TRACE
    if (l[0] == 12345.678f) STRACE(op_i, 7);
#endif
    STRACE(op_i, 5);
    // merge the lane-group states through shared memory, write this split's partial state
    const int st = w * tpw + sub;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float* r = merge + ((size_t)st * G + g) * rec;
      if (li == 0) {
        r[0] = mx[g];
        r[1] = l[g];
      }
#pragma unroll
      for (int e = 0; e < EPL; ++e) r[2 + li * EPL + e] = acc[g][e];
    }
    consumers_sync();
    for (int idx = tid; idx < G * hd; idx += 256) {
      const int g = idx / hd, e = idx % hd;
      float mm = -INFINITY;
      for (int i = 0; i < nstates; ++i) mm = fmaxf(mm, merge[((size_t)i * G + g) * rec]);
      float L = 0.0f, A = 0.0f;
      for (int i = 0; i < nstates; ++i) {
        const float* r = merge + ((size_t)i * G + g) * rec;
        const float cc = (r[0] == -INFINITY) ? 0.0f : __expf(r[0] - mm);
        L += r[1] * cc;
        A += r[2 + e] * cc;
      }
      if (splits == 1) {
        out[((size_t)row * H + h0 + g) * hd + e] = from_f<T>(L > 0.0f ? A / L : 0.0f);
      } else {
        float* pr = a.attn_part + (((size_t)row * H + h0 + g) * kMaxStackSplits + split) * rec;
        if (e == 0) {
          pr[0] = mm;
          pr[1] = L;
        }
        pr[2 + e] = A;
      }
    }
    consumers_sync();  // all partial stores issued (published by the release below); the merge area is free again
    STRACE(op_i, 6);
    bool finished = (splits == 1);
    if (splits > 1) {
      if (tid == 0) {
        unsigned int* cnt = a.attn_cnt + (row * yg + y);
        const unsigned int prev = atom_add_acq_rel(cnt, 1u);
        const int last = (prev == (unsigned int)(splits - 1));
        if (last) *cnt = 0u;
        *s_last = last;
      }
      consumers_sync();
      if (*s_last) {
        for (int idx = tid; idx < G * hd; idx += 256) {
          const int g = idx / hd, e = idx % hd;
          const float* p = a.attn_part + (((size_t)row * H + h0 + g) * kMaxStackSplits) * rec;
          float mi[kMaxStackSplits], li_[kMaxStackSplits], ai[kMaxStackSplits];
#pragma unroll
          for (int i = 0; i < kMaxStackSplits; ++i) {
            const int ic = i < splits ? i : 0;  // clamped: every address is valid, all loads are independent
            mi[i] = __ldcg(p + ic * rec);
            li_[i] = __ldcg(p + ic * rec + 1);
            ai[i] = __ldcg(p + ic * rec + 2 + e);
          }
          float mm = -INFINITY;
#pragma unroll
          for (int i = 0; i < kMaxStackSplits; ++i)
            if (i < splits) mm = fmaxf(mm, mi[i]);
          float L = 0.0f, A = 0.0f;
#pragma unroll
          for (int i = 0; i < kMaxStackSplits; ++i)
            if (i < splits) {
              const float cc = (mi[i] == -INFINITY) ? 0.0f : __expf(mi[i] - mm);
              L += li_[i] * cc;
              A += ai[i] * cc;
            }
          out[((size_t)row * H + h0 + g) * hd + e] = from_f<T>(L > 0.0f ? A / L : 0.0f);
        }
        finished = true;
      }
      consumers_sync();  // s_last is reused; the combined rows are fenced
    }
    if (finished && tid == 0) red_release_add(&a.done[op_i * kDoneStride], 1u);
  }
}

// ------------------------------------------------------------------------------------------- host side (decode_stack.cu)
struct StackPlan {
  int64_t partial_bytes, counter_words;
  size_t xs_bytes, union_bytes;
};
// mode: 0 FMA consumers, 2 mma.sync consumers
StackPlan stack_plan(const StackConfig& c, const StackOp* ops, int n_ops, int grid, int mode);
int stack_fill_args(StackArgs& a, const StackPlan& p, const StackConfig& c, const StackOp* ops_dev, const StackOp* ops_host, int n_ops,
                    void* partials, void* counters, void* attn_part, int* error_flag, long long* trace);
// mma.sync variant (decode_stack_mma.cu), fp16 and up to 8 sequences
int launch_decode_stack_mma(int device, DeviceState* st, const StackConfig& c, const StackOp* ops_dev, const StackOp* ops_host,
                            int n_ops, void* partials, void* counters, void* attn_part, int* error_flag,
                            long long* trace, bool pdl, cudaStream_t s);
int init_stack_mma_attrs();

}  // namespace tsb
