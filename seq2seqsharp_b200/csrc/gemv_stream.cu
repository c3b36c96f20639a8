// Decode GEMV for the GPT engine: y[M,N] = epilogue(prologue(x)[M,K] * W[K,N]), M <= 4, bandwidth-bound.
//
// Blackwell-first design:
//  * weights are pre-packed at load time into contiguous 16 KB tiles [KT=32 rows][NT=32*VEC columns] ordered
//    column-tile-major, so the units a CTA works on are ONE contiguous byte range of HBM (fp16 tiles are stored
//    in the 128-byte-swizzled box order of packed_tile_off(), which this kernel's 16-byte reads follow);
//  * each CTA is persistent over a contiguous, evenly sized range of tiles (stream-K: the K dimension of a column
//    tile may be shared by several CTAs), so all SMs stream the same number of bytes regardless of the shape;
//  * one producer warp feeds a ring of shared-memory stages with TMA bulk copies (cp.async.bulk, completion on an
//    mbarrier); eight consumer warps read the tiles with conflict-free 128-bit shared loads and accumulate in fp32;
//    stages are handed back through a second set of mbarriers, so no block-wide barrier sits in the main loop;
//  * the producer starts streaming weights before the grid dependency is resolved (programmatic dependent launch):
//    weights never depend on the previous kernel, activations are read only after griddepcontrol.wait;
//  * the preceding LayerNorm / RMSNorm is a prologue (each CTA normalises the M activation rows itself from the fp32
//    residual stream: d*4 bytes from L2 instead of a separate launch), and bias, activation, gate product and
//    residual add are the epilogue;
//  * partial sums of a column tile shared by several CTAs meet in a scratch buffer; the last CTA to arrive adds them
//    in a fixed order, so results are bitwise reproducible.
// Every wait on an mbarrier is bounded; on timeout the kernel raises an error flag that the host reads, stops
// issuing copies, drains the copies in flight (bounded) and returns.
//
// Replaces, per decode step and layer, LayerNorm/RMSNorm + bias copy + cublasGemmEx + activation / gate / residual
// kernels of the reference (TensorSharp.CUDA/DeviceCode/AdvFuncKernels.cs:613-685,791-845,
// TensorSharp.CUDA/MatrixMul/CudaMatrixMulMM.cs:305-362, Seq2SeqSharp/Layers/PositionwiseFeedForward.cs:72-98).
#include "kernels.cuh"
#include "stream_common.cuh"

namespace tsb {

// Time stamps for kernel development exist only in builds with -DTSB200_TRACE; the shipped kernel carries none.
#ifdef TSB200_TRACE
#define TRACE(slot)                                                                     \
  do {                                                                                  \
    if (a.trace && (tid & 31) == 0 && ((tid >> 5) == 0 || (tid >> 5) == kConsumerWarps)) \
      a.trace[(size_t)blockIdx.x * 8 + (slot)] = gtimer();                              \
  } while (0)
#else
#define TRACE(slot) do { } while (0)
#endif
struct StreamArgs {
  const void* Wp;        // packed tiles
  const void* x;         // xmode 0: T [M,K]; xmode 1/2: fp32 residual stream [M,K]
  const void* gamma;     // norm gain (T), xmode 1/2
  const void* beta;      // LayerNorm bias (T) or null
  int xmode;             // 0 plain, 1 RMSNorm prologue, 2 LayerNorm prologue
  float eps;
  int K, N;              // logical sizes
  int KB, CT;            // tiles along K and along N
  int stages;
  int max_contrib;
  float* partials;       // [CT][max_contrib][M][NT]
  unsigned int* counters;  // [CT], zero on entry, self-resetting
  int* error_flag;       // set to 1 on a wait timeout
  long long* trace;      // optional [grid][8] globaltimer stamps (profiling aid), null in normal use
  Epilogue ep;
};

template <typename T, int M>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_stream_kernel(StreamArgs a) {
  constexpr int VEC = TileVec<T>::N;
  constexpr int NT = 32 * VEC;
  extern __shared__ __align__(128) unsigned char smem[];
  const int S = a.stages;
  const int Kp = a.KB * kKT;
  unsigned char* stage_mem = smem;                                        // [S][16 KB]
  T* xs = reinterpret_cast<T*>(smem + (size_t)S * kTileBytes);            // [M][Kp]
  float* red = reinterpret_cast<float*>(smem + (size_t)S * kTileBytes + (((size_t)M * Kp * sizeof(T) + 127) & ~(size_t)127));  // [8][M][NT]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + kConsumerWarps * M * NT);
  uint64_t* empty = full + 8;
  __shared__ int s_err, s_last;
  __shared__ float s_stat[2 * 4 * 8];

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  if (w == 0) TRACE(0);  // CTA start
  const long long U = (long long)a.KB * a.CT;
  const long long G = gridDim.x;
  const int u_begin = (int)(U * blockIdx.x / G), u_end = (int)(U * (blockIdx.x + 1) / G);

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    s_err = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  grid_dep_launch();  // let the next kernel's CTAs become resident and start streaming their weights

  if (w == kConsumerWarps) {
    // ---------------- producer warp: stream this CTA's contiguous tile range through the stage ring
    if (lane == 0) {
      const unsigned char* src = reinterpret_cast<const unsigned char*>(a.Wp) + (size_t)u_begin * kTileBytes;
      int issued = 0, s = 0;
      unsigned ph = 1;  // parity of the "empty" phase to wait for once the ring has wrapped (first wrap waits phase 0)
      for (int u = u_begin; u < u_end; ++u, ++issued) {
        if (issued >= S) {
          if (!mbar_wait(&empty[s], ph ^ 1u)) {
            s_err = 1;
            break;
          }
        }
        if (*(volatile int*)&s_err) break;
        mbar_expect_tx(&full[s], kTileBytes);
        bulk_g2s(stage_mem + (size_t)s * kTileBytes, src + (size_t)issued * kTileBytes, kTileBytes, &full[s]);
        if (++s == S) {
          s = 0;
          if (issued >= S) ph ^= 1u;
        }
      }
      if (*(volatile int*)&s_err) {
        // drain: wait (bounded) for every copy that was issued so nothing lands in shared memory after exit
        for (int i = (issued > S ? issued - S : 0); i < issued; ++i) mbar_wait(&full[i % S], (unsigned)((i / S) & 1));
        if (a.error_flag) *a.error_flag = 1;
      }
    }
    return;
  }

  // ---------------- consumer warps
  grid_dep_wait();  // activations and outputs of earlier kernels are visible from here on
  if (w == 0) TRACE(1);  // dependency resolved
  // prologue: stage x (optionally normalised) in shared memory as T.  Loads are gathered into registers in batches
  // before anything is stored (a store to shared memory between two global loads would serialise their latencies).
  constexpr int XB = 8;  // loads in flight per thread
  if (a.xmode == 0) {
    const T* __restrict__ x = reinterpret_cast<const T*>(a.x);
    const int K = a.K;
    for (int m = 0; m < M; ++m) {
      for (int k0 = 0; k0 < Kp; k0 += 256 * XB) {
        T v[XB];
#pragma unroll
        for (int j = 0; j < XB; ++j) {
          const int k = k0 + j * 256 + tid;
          const T xv = x[(size_t)m * K + (k < K ? k : 0)];  // plain (coherent) load, clamped index
          v[j] = (k < K) ? xv : from_f<T>(0.0f);
        }
#pragma unroll
        for (int j = 0; j < XB; ++j) {
          const int k = k0 + j * 256 + tid;
          if (k < Kp) xs[m * Kp + k] = v[j];
        }
      }
    }
  } else {
    const float* __restrict__ x = reinterpret_cast<const float*>(a.x);
    const T* gamma = reinterpret_cast<const T*>(a.gamma);
    // A guarded load may be hoisted above its guard by the compiler; so that every address a thread can form is
    // valid, a missing beta aliases gamma and is switched off by a factor instead of by a null test.
    const float beta_on = a.beta ? 1.0f : 0.0f;
    const T* beta = a.beta ? reinterpret_cast<const T*>(a.beta) : gamma;
    const int K = a.K;
    constexpr int XR = 48;  // row elements kept in registers per thread: rows up to 256*48 = 12288
    for (int m = 0; m < M; ++m) {
      float xr[XR];
#pragma unroll
      for (int j = 0; j < XR; ++j) {
        const int k = j * 256 + tid;
        const float xv = __ldcg(x + (size_t)m * K + (k < K ? k : 0));  // L2-coherent load (written by the previous kernel), clamped index
        xr[j] = (k < K) ? xv : 0.0f;
      }
      // statistics over the row: sum (LayerNorm) or sum of squares (RMSNorm), then centred squares for LayerNorm
      float s1 = 0.0f;
#pragma unroll
      for (int j = 0; j < XR; ++j) s1 += (a.xmode == 2) ? xr[j] : xr[j] * xr[j];
      s1 = warp_sum(s1);
      if (lane == 0) s_stat[m * 8 + w] = s1;
      consumer_sync();
      float tot = 0.0f;
#pragma unroll
      for (int i = 0; i < kConsumerWarps; ++i) tot += s_stat[m * 8 + i];
      float mean = 0.0f, inv;
      if (a.xmode == 2) {
        mean = tot / K;
        float s2 = 0.0f;
#pragma unroll
        for (int j = 0; j < XR; ++j) {
          const float e = (j * 256 + tid < K) ? xr[j] - mean : 0.0f;
          s2 += e * e;
        }
        s2 = warp_sum(s2);
        if (lane == 0) s_stat[32 + m * 8 + w] = s2;
        consumer_sync();
        float t2 = 0.0f;
#pragma unroll
        for (int i = 0; i < kConsumerWarps; ++i) t2 += s_stat[32 + m * 8 + i];
        inv = sqrtf(a.eps + t2 / K);      // sigma
      } else {
        inv = sqrtf(tot / (float)K + a.eps);  // rms
      }
#pragma unroll
      for (int j0 = 0; j0 < XR; j0 += XB) {
        if (j0 * 256 >= Kp) break;
        float gv[XB], bv[XB];
#pragma unroll
        for (int j = 0; j < XB; ++j) {
          const int k = (j0 + j) * 256 + tid;
          const int kc = k < K ? k : 0;  // clamped: always in range
          gv[j] = to_f<T>(gamma[kc]);
          bv[j] = beta_on * to_f<T>(beta[kc]);
        }
#pragma unroll
        for (int j = 0; j < XB; ++j) {
          const int k = (j0 + j) * 256 + tid;
          if (k < Kp) xs[m * Kp + k] = from_f<T>((k < K) ? gv[j] * ((xr[j0 + j] - mean) / inv) + bv[j] : 0.0f);
        }
      }
    }
  }
  consumer_sync();

  float acc[M][VEC];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[m][e] = 0.0f;

  int seg_begin = u_begin;
  int s = 0;
  unsigned ph = 0;
  int ct = u_begin / a.KB, kb = u_begin % a.KB;
  const T* bias = reinterpret_cast<const T*>(a.ep.bias);
  // A warp whose wait ran out keeps walking the loop (short waits only, so that every copy in flight is still
  // awaited and every named barrier is still reached by all eight warps); results are then garbage and the host
  // sees the error flag.
  bool dead = false;
  if (w == 0) TRACE(2);  // x staged
  constexpr int RPW = kKT / kConsumerWarps;  // rows of a tile per warp (consecutive rows, so x is one vector load)
  for (int u = u_begin; u < u_end; ++u) {
    if (*(volatile int*)&s_err) dead = true;
    if (!mbar_wait(&full[s], ph, dead ? 4096u : kSpinLimit)) {
      s_err = 1;
      dead = true;
    }
    if (w == 0 && u == u_begin) TRACE(3);  // first tile landed
    const unsigned char* tile = stage_mem + (size_t)s * kTileBytes;
    TileVec<T> wv[RPW];
#pragma unroll
    for (int rr = 0; rr < RPW; ++rr) wv[rr].lds(tile + (size_t)packed_tile_off<T>(w * RPW + rr, lane * VEC) * sizeof(T));
    float xv[M][RPW];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int rr = 0; rr < RPW; ++rr) xv[m][rr] = to_f<T>(xs[m * Kp + kb * kKT + w * RPW + rr]);
#pragma unroll
    for (int rr = 0; rr < RPW; ++rr) {
      float wf[VEC];
      wv[rr].get(wf);
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[m][e] = fmaf(xv[m][rr], wf[e], acc[m][e]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
    if (++s == S) {
      s = 0;
      ph ^= 1u;
    }
    const int cur_ct = ct, cur_kb = kb;
    if (++kb == a.KB) {
      kb = 0;
      ++ct;
    }
    const bool seg_end = (cur_kb == a.KB - 1) || (u == u_end - 1);
    if (w == 0 && u == u_end - 1) TRACE(4);  // last tile consumed
    if (!seg_end) continue;
    // ---- end of this CTA's share of column tile ct: reduce over warps, then finish or hand over a partial
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        red[(w * M + m) * NT + lane * VEC + e] = acc[m][e];
        acc[m][e] = 0.0f;
      }
    consumer_sync();
    for (int idx = tid; idx < M * NT; idx += 256) {
      float v = 0.0f;
#pragma unroll
      for (int ww = 0; ww < kConsumerWarps; ++ww) v += red[ww * M * NT + idx];
      red[idx] = v;
    }
    consumer_sync();
    const long long ct_first_u = (long long)cur_ct * a.KB, ct_last_u = ct_first_u + a.KB - 1;
    const bool whole = (seg_begin <= ct_first_u) && (u == ct_last_u);
    bool finish = whole;
    if (!whole) {
      const int c_first = (int)(((ct_first_u + 1) * G + U - 1) / U - 1);
      const int c_last = (int)(((ct_last_u + 1) * G + U - 1) / U - 1);
      const int n_contrib = c_last - c_first + 1;
      const int slot = blockIdx.x - c_first;
      float* mine = a.partials + (((size_t)cur_ct * a.max_contrib + slot) * M) * NT;
      for (int idx = tid; idx < M * NT; idx += 256) mine[idx] = red[idx];
      __threadfence();
      consumer_sync();
      if (tid == 0) {
        const unsigned int prev = atomicAdd(&a.counters[cur_ct], 1u);
        s_last = (prev == (unsigned int)(n_contrib - 1));
        if (s_last) a.counters[cur_ct] = 0u;
      }
      consumer_sync();
      if (s_last) {
        __threadfence();
        const float* all = a.partials + ((size_t)cur_ct * a.max_contrib * M) * NT;
        for (int idx = tid; idx < M * NT; idx += 256) {
          float v = 0.0f;
          for (int j = 0; j < n_contrib; ++j) v += __ldcg(all + (size_t)j * M * NT + idx);
          red[idx] = v;
        }
        consumer_sync();
        finish = true;
      }
    }
    if (finish) {
      if (!a.ep.glu) {
        for (int idx = tid; idx < M * NT; idx += 256) {
          const int m = idx / NT, c = cur_ct * NT + (idx % NT);
          if (c < a.N) {
            float v = red[idx] + (bias ? to_f<T>(bias[c]) : 0.0f);
            switch (a.ep.act) {
              case TSB200_ACT_RELU: v = v < 0.0f ? 0.0f : v; break;
              case TSB200_ACT_SILU: v = v / (1.0f + expf(-v)); break;
              case TSB200_ACT_LEAKYRELU: v = v < 0.0f ? 0.01f * v : v; break;
              case TSB200_ACT_GELU: v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)); break;
              default: break;
            }
            const size_t o = (size_t)m * a.N + c;
            if (a.ep.residual) v += a.ep.residual[o];
            if (a.ep.y32) a.ep.y32[o] = v;
            else reinterpret_cast<T*>(a.ep.y)[o] = from_f<T>(v);
          }
        }
      } else {
        const int No = a.N / 2;
        for (int idx = tid; idx < M * (NT / 2); idx += 256) {
          const int m = idx / (NT / 2), j = idx % (NT / 2);
          const int c = cur_ct * NT + 2 * j;
          if (c + 1 < a.N) {
            float av = red[m * NT + 2 * j] + (bias ? to_f<T>(bias[c]) : 0.0f);
            const float gv = red[m * NT + 2 * j + 1] + (bias ? to_f<T>(bias[c + 1]) : 0.0f);
            if (a.ep.act == TSB200_ACT_SWIGLU) av = av / (1.0f + expf(-av));
            float v = av * gv;
            const size_t o = (size_t)m * No + (c >> 1);
            if (a.ep.residual) v += a.ep.residual[o];
            if (a.ep.y32) a.ep.y32[o] = v;
            else reinterpret_cast<T*>(a.ep.y)[o] = from_f<T>(v);
          }
        }
      }
    }
    consumer_sync();  // red is reused by the next segment
    seg_begin = u + 1;
  }
  if (w == 0) TRACE(5);  // done
  if (tid == 0 && *(volatile int*)&s_err && a.error_flag) *a.error_flag = 1;
}

// ---- packing: row-major logical columns [c0 + j*cs] of a [K, Np] matrix into the tiled layout -----------------------
template <typename TD, typename TS>
__global__ void pack_tiles_kernel(TD* __restrict__ dst, const TS* __restrict__ src, int rows, int cols, int src_ld, int KB,
                                  int NT, int c0, int cs) {
  const long long n = (long long)rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i / cols), j = (int)(i % cols);
    const int c = c0 + j * cs;
    const long long tile = (long long)(c / NT) * KB + (k / kKT);
    dst[tile * (kKT * NT) + packed_tile_off<TD>(k % kKT, c % NT)] = from_f<TD>(to_f<TS>(src[(long long)k * src_ld + j]));
  }
}

int packed_tile_cols(int dtype) { return dtype == TSB200_F16 ? 256 : 128; }
int64_t packed_bytes(int dtype, int K, int N) {
  const int NT = packed_tile_cols(dtype);
  const int64_t KB = (K + kKT - 1) / kKT, CT = (N + NT - 1) / NT;
  return KB * CT * kTileBytes;
}

int launch_pack(int device, DeviceState* st, int dst_dtype, void* dst, int src_dtype, const void* src, int rows, int cols,
                int src_ld, int K, int c0, int cs, cudaStream_t s) {
  const int NT = packed_tile_cols(dst_dtype);
  const int KB = (K + kKT - 1) / kKT;
  const long long n = (long long)rows * cols;
  if (n == 0) return 1;
  long long g = (n + 255) / 256;
  if (g > (long long)st->sm_count * 16) g = (long long)st->sm_count * 16;
#define TSB_PACK(TD, TS) pack_tiles_kernel<TD, TS><<<(int)g, 256, 0, s>>>((TD*)dst, (const TS*)src, rows, cols, src_ld, KB, NT, c0, cs)
  if (dst_dtype == TSB200_F16 && src_dtype == TSB200_F16) TSB_PACK(__half, __half);
  else if (dst_dtype == TSB200_F16 && src_dtype == TSB200_F32) TSB_PACK(__half, float);
  else if (dst_dtype == TSB200_F32 && src_dtype == TSB200_F32) TSB_PACK(float, float);
  else if (dst_dtype == TSB200_F32 && src_dtype == TSB200_F16) TSB_PACK(float, __half);
  else TSB_FAIL("pack: unsupported dtypes");
#undef TSB_PACK
  count_launch(device);
  return check_launch("pack_tiles");
}

struct StreamPlan {
  int KB, CT, stages, grid, max_contrib;
  size_t smem;
};

template <typename T>
static bool plan_stream(DeviceState* st, int M, int K, int N, StreamPlan* p) {
  constexpr int NT = 32 * TileVec<T>::N;
  p->KB = (K + kKT - 1) / kKT;
  p->CT = (N + NT - 1) / NT;
  const long long U = (long long)p->KB * p->CT;
  const size_t xs = (((size_t)M * p->KB * kKT * sizeof(T)) + 127) & ~(size_t)127;
  const size_t red = (size_t)kConsumerWarps * M * NT * sizeof(float);
  const size_t fixed = xs + red + 16 * sizeof(uint64_t) + 128;
  // two CTAs per SM (so that the next kernel's CTAs can sit beside this kernel's and prefetch) when it fits
  const size_t budget2 = 112 * 1024, budget1 = 226 * 1024;
  int stages = 0;
  if (fixed + 3 * (size_t)kTileBytes <= budget2) stages = (int)((budget2 - fixed) / kTileBytes);
  else if (fixed + 2 * (size_t)kTileBytes <= budget1) stages = (int)((budget1 - fixed) / kTileBytes);
  else return false;
  if (stages > 8) stages = 8;
  p->stages = stages;
  p->smem = fixed + (size_t)stages * kTileBytes;
  long long g = st->sm_count;
  if (g > U) g = U;
  p->grid = (int)g;
  const long long per = U / g;  // >= 1
  p->max_contrib = (int)(p->KB / per) + 2;
  return true;
}

int64_t stream_workspace_bytes(int dtype, int M, int K, int N, int sm_count) {
  const int NT = packed_tile_cols(dtype);
  const long long KB = (K + kKT - 1) / kKT, CT = (N + NT - 1) / NT;
  long long g = sm_count;
  if (g > KB * CT) g = KB * CT;
  const long long per = (KB * CT) / (g > 0 ? g : 1);
  const long long mc = KB / (per > 0 ? per : 1) + 2;
  return kWsCounterBytes + 768 + CT * mc * M * NT * 4;
}

template <typename T, int M>
static int launch_stream_m(int device, DeviceState* st, const StreamPlan& p, StreamArgs& a, bool pdl, cudaStream_t s) {
  static bool attr_done[kMaxDevices] = {};
  if (!attr_done[device]) {
    TSB_CUDA(cudaFuncSetAttribute(gemv_stream_kernel<T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    attr_done[device] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.grid);
  cfg.blockDim = dim3(kStreamThreads);
  cfg.dynamicSmemBytes = p.smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  TSB_CUDA(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<T, M>, a));
  count_launch(device);
  return 1;
}

int init_stream_attrs(int device);

template <typename T>
static int launch_stream_t(int device, DeviceState* st, StreamArgs& a, int M, bool pdl, void* ws, int64_t ws_bytes, cudaStream_t s) {
  constexpr int NT = 32 * TileVec<T>::N;
  StreamPlan p;
  if (!plan_stream<T>(st, M, a.K, a.N, &p)) return 2;
  // [counters | 256 spare bytes (the stand-alone entry point keeps its error word there) | partials]
  const int64_t cnt_bytes = kWsCounterBytes;
  TSB_CHECK((int64_t)p.CT * 4 <= kWsCounterBytes - 256, "gemv_stream: too many column tiles (%d)", p.CT);
  const int64_t need = cnt_bytes + (int64_t)p.CT * p.max_contrib * M * NT * 4;
  TSB_CHECK(ws && ws_bytes >= need, "gemv_stream: workspace too small (%lld < %lld)", (long long)ws_bytes, (long long)need);
  a.KB = p.KB;
  a.CT = p.CT;
  a.stages = p.stages;
  a.max_contrib = p.max_contrib;
  a.counters = reinterpret_cast<unsigned int*>(ws);
  a.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + cnt_bytes);
  switch (M) {
    case 1: return launch_stream_m<T, 1>(device, st, p, a, pdl, s);
    case 2: return launch_stream_m<T, 2>(device, st, p, a, pdl, s);
    case 3: return launch_stream_m<T, 3>(device, st, p, a, pdl, s);
    case 4: return launch_stream_m<T, 4>(device, st, p, a, pdl, s);
  }
  return 2;
}

#ifdef TSB200_TRACE
static long long* g_gemv_trace = nullptr;  // set through TSB200_DebugSetGemvTrace
void set_gemv_trace(long long* p) { g_gemv_trace = p; }
#endif

// Returns 1 on success, 0 on error, 2 when the shape is not handled by this kernel (caller falls back).
int launch_gemv_stream(int device, DeviceState* st, int dtype, const void* Wp, const void* x, int xmode, const void* gamma,
                       const void* beta, float eps, int M, int K, int N, const Epilogue& ep, int* error_flag, bool pdl, void* ws,
                       int64_t ws_bytes, cudaStream_t s) {
  if (M < 1 || M > 4) return 2;
  if (xmode != 0 && K > 12288) return 2;  // the norm prologue keeps a row in registers
  StreamArgs a{};
  a.Wp = Wp; a.x = x; a.gamma = gamma; a.beta = beta; a.xmode = xmode; a.eps = eps; a.K = K; a.N = N;
  a.error_flag = error_flag;
#ifdef TSB200_TRACE
  a.trace = g_gemv_trace;
#endif
  a.ep = ep;
  if (dtype == TSB200_F16) return launch_stream_t<__half>(device, st, a, M, pdl, ws, ws_bytes, s);
  return launch_stream_t<float>(device, st, a, M, pdl, ws, ws_bytes, s);
}

template <typename T, int M>
static int stream_attr_one() {
  TSB_CUDA(cudaFuncSetAttribute(gemv_stream_kernel<T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  return 1;
}
int init_stream_attrs(int device) {
  static bool done[kMaxDevices] = {};
  if (done[device]) return 1;
  TSB_TRY((stream_attr_one<float, 1>())); TSB_TRY((stream_attr_one<float, 2>())); TSB_TRY((stream_attr_one<float, 3>())); TSB_TRY((stream_attr_one<float, 4>()));
  TSB_TRY((stream_attr_one<__half, 1>())); TSB_TRY((stream_attr_one<__half, 2>())); TSB_TRY((stream_attr_one<__half, 3>())); TSB_TRY((stream_attr_one<__half, 4>()));
  done[device] = true;
  return 1;
}

}  // namespace tsb

using namespace tsb;

extern "C" {

int64_t TSB200_PackedWeightBytes(int dtype, int K, int N) { return packed_bytes(dtype, K, N); }

#ifdef TSB200_TRACE
int TSB200_DebugSetGemvTrace(void* device_buffer) {
  set_gemv_trace(reinterpret_cast<long long*>(device_buffer));
  return 1;
}
#endif

int TSB200_PackWeight(int device, int dtype, void* packed, const void* W, int src_dtype, int K, int N, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(packed && W && K > 0 && N > 0, "pack_weight: bad arguments");
  TSB_CHECK(dtype == TSB200_F32 || dtype == TSB200_F16, "pack_weight: unsupported dtype %d", dtype);
  cudaStream_t s = pick_stream(st, stream);
  TSB_CUDA(cudaMemsetAsync(packed, 0, (size_t)packed_bytes(dtype, K, N), s));
  return launch_pack(device, st, dtype, packed, src_dtype, W, K, N, N, K, 0, 1, s);
}

int64_t TSB200_LinearPackedWorkspaceBytes(int dtype, int M, int K, int N) {
  const int64_t a = stream_workspace_bytes(dtype, M > 4 ? 4 : (M < 1 ? 1 : M), K, N, 160);
  int64_t b = linear_workspace_bytes(M, K, N);
  const int64_t c = dtype == TSB200_F16 && M > 16 ? gemm_tc_workspace_bytes(M, N, 132) : 0;
  if (c > b) b = c;
  const int64_t d = dtype == TSB200_F16 && M >= 1 && M <= 64 ? gemm_stream_mma_workspace_bytes(M, K, N, 132) : 0;
  if (d > b) b = d;
  const int64_t e = dtype == TSB200_F16 && M > 16 && M <= 64 ? gemm_stream_tc_workspace_bytes(M, K, N, 160) : 0;
  if (e > b) b = e;
  return (a > b ? a : b) + 256;
}

int TSB200_LinearPacked(int device, int dtype, void* y, float* y_f32, const void* x, const float* x_f32, const void* gamma,
                        const void* beta, int norm_type, float eps, const void* Wp, const void* bias, const float* residual_f32,
                        int M, int K, int N, int act, void* workspace, int64_t workspace_bytes, void* stream) {
  DeviceState* st;
  TSB_TRY(use_device(device, &st));
  TSB_CHECK(dtype == TSB200_F32 || dtype == TSB200_F16, "linear_packed: unsupported dtype %d", dtype);
  TSB_CHECK(Wp && (y || y_f32) && M >= 0 && K > 0 && N > 0, "linear_packed: bad arguments");
  TSB_CHECK(norm_type >= -1 && norm_type <= 1, "linear_packed: norm_type must be -1 (none), 0 (LayerNorm) or 1 (RMSNorm)");
  TSB_CHECK(norm_type < 0 ? x != nullptr : (x_f32 != nullptr && gamma != nullptr), "linear_packed: missing input for the chosen prologue");
  TSB_CHECK(workspace && workspace_bytes >= TSB200_LinearPackedWorkspaceBytes(dtype, M, K, N), "linear_packed: workspace too small");
  if (M == 0) return 1;
  Epilogue ep{};
  ep.bias = bias;
  ep.residual = residual_f32;
  ep.y = y_f32 ? nullptr : y;
  ep.y32 = y_f32;
  ep.act = act;
  ep.glu = (act == TSB200_ACT_GLU_NOACT || act == TSB200_ACT_SWIGLU) ? 1 : 0;
  TSB_CHECK(!ep.glu || N % 2 == 0, "linear_packed: gated activations need an even (interleaved) column count");
  cudaStream_t s = pick_stream(st, stream);
  TSB_TRY(init_stream_attrs(device));
  // counters at the head of the workspace must start at zero; the last word of the workspace is the error flag
  const int64_t z = workspace_bytes < kWsCounterBytes ? workspace_bytes : kWsCounterBytes;
  TSB_CUDA(cudaMemsetAsync(workspace, 0, (size_t)z, s));
  int* err = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + kWsCounterBytes - 256);
  static int gemv_rows = -1;
  if (gemv_rows < 0) {
    const char* e = getenv("TSB200_GEMV_MAXROWS");  // rows served by the FMA streaming GEMV here (default 4; the engine has its own default)
    gemv_rows = e ? atoi(e) : 4;
  }
  if (M <= 4 && M <= gemv_rows) {
    const int r = launch_gemv_stream(device, st, dtype, Wp, norm_type < 0 ? x : (const void*)x_f32, norm_type < 0 ? 0 : (norm_type == 0 ? 2 : 1),
                                     gamma, norm_type == 0 ? beta : nullptr, eps, M, K, N, ep, err, false, workspace, workspace_bytes - 256, s);
    if (r != 2) return r;
  }
  if (norm_type >= 0 && dtype == TSB200_F16 && M <= 8) {
    // up to eight rows of a fp16 model of width 1024 / 2048 / 4096: the tensor-core streaming kernel norms the rows itself
    const int r = launch_gemm_stream_mma_norm(device, st, x_f32, gamma, norm_type == 0 ? beta : nullptr, norm_type, eps, Wp, M, K, N, ep, err, false,
                                              workspace, workspace_bytes - 256, s);
    if (r != 2) return r;
  }
  TSB_CHECK(norm_type < 0, "linear_packed: the norm prologue is fused for M <= 4 (and for M <= 8 on fp16 models of width 1024 / 2048 / 4096 "
                           "with M * width <= 16384); normalise separately otherwise");
  return launch_linear(device, st, dtype, x, Wp, M, K, N, ep, workspace, workspace_bytes - 256, s, true);
}

}  // extern "C"
