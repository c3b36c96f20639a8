// One persistent kernel for the whole layer stack of a cached decode step (batch <= 4).
//
// A decode step of a 7B-class model is ~130 dependent matrix-vector products, each streaming 30..260 MB of weights
// once.  Launched one by one, every product pays a start-up (activations staged, first tiles in flight) and a tail
// (cross-CTA reduction, launch of the next kernel) during which HBM idles.  Weights, however, never depend on the
// activations.  So here one CTA per SM stays resident for the whole step and its producer warp streams the packed
// weight tiles of product after product through a deep shared-memory ring (cp.async.bulk + mbarrier) without ever
// waiting for the dependency chain; only the eight consumer warps follow the chain:
//
//   for each operation of the program (per layer: QKV, attention, out-projection, FFN up, FFN down; then LM head)
//     wait until the previous operation is complete everywhere   (one acquire-poll of a global counter)
//     linear:    stage x in shared memory (fused RMSNorm / LayerNorm of the fp32 residual stream, or the combine of
//                the attention partials), consume this CTA's contiguous tile range from the ring, hand partial
//                sums of shared column tiles to the last arriver (fixed order => bitwise reproducible), epilogue
//                (bias, activation, gate product, residual), release-increment the operation's counter
//     attention: RoPE of q and of the new key in registers, append of k/v to the cache, split-K online softmax
//                over the cached keys; partial states go to scratch, the out-projection's prologue combines them
//
// While consumers sit in a dependency wait the ring keeps filling (up to ~190 KB per SM, ~28 MB over the GPU, about
// 4 us of HBM time), which is what hides the chain latency.  Every wait (mbarrier or global counter) is bounded; a
// wait that runs out raises the error word, after which all waits become short, copies in flight are still awaited
// and the kernel returns.  Activations written inside the kernel are read with L2-coherent loads only.
//
// Replaces the per-layer launch sequence of the reference's cached decode (Seq2SeqSharp/Networks/GPTDecoder.cs:86-131,
// Layers/MultiHeadAttention.cs:141-252, Layers/PositionwiseFeedForward.cs:72-98).
#include <cstdlib>
#include <cstring>

#include "decode_stack.cuh"

namespace tsb {

// ------------------------------------------------------------------------------------------- linear (consumers)
template <typename T, int M>
__device__ __forceinline__ void stack_linear(const StackArgs& a, const StackOp* op, int op_i, const LinGeom& g,
                                             unsigned char* stage_mem, T* xs, float* red, uint64_t* full, uint64_t* empty,
                                             int& s, unsigned& round, volatile int* s_err, volatile int* s_last, float* s_stat,
                                             bool& dead, const NormConsts<T>* nc) {
  constexpr int VEC = TileVec<T>::N;
  constexpr int NT = 32 * VEC;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int S = a.stages;
  const int K = op->K, N = op->N, KB = g.KB;
  const int Kp = KB * kKT;
  const long long U = g.U, G = g.Gop;
  const int u_begin = (int)(U * blockIdx.x / G), u_end = (int)(U * (blockIdx.x + 1) / G);
  const int max_contrib = (int)(KB / (U / G)) + 2;
  const Epilogue ep = op->ep;

  if (op->xmode == 0) {
    stage_plain<T>(xs, reinterpret_cast<const T*>(op->x), M, K, Kp, tid);
  } else if (K <= 256 * 16) {
    stage_norm<T, 16>(xs, reinterpret_cast<const float*>(op->x), reinterpret_cast<const T*>(op->gamma),
                      reinterpret_cast<const T*>(op->beta), nc, op->xmode, op->eps, M, K, Kp, tid, s_stat);
  } else {
    stage_norm<T, 48>(xs, reinterpret_cast<const float*>(op->x), reinterpret_cast<const T*>(op->gamma),
                      reinterpret_cast<const T*>(op->beta), nullptr, op->xmode, op->eps, M, K, Kp, tid, s_stat);
  }
  consumers_sync();
  STRACE(op_i, 1);

  float acc[M][VEC];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[m][e] = 0.0f;

  int seg_begin = u_begin;
  int ct = u_begin / KB, kb = u_begin % KB;
  const T* bias = reinterpret_cast<const T*>(ep.bias);
  constexpr int RPW = kKT / kConsumerWarps;
  for (int u = u_begin; u < u_end; ++u) {
    if (*s_err) dead = true;
    // a CTA that gave up walks through the rest of its program without waiting (its results are discarded)
    if (!dead && !mbar_wait(&full[s], round & 1u, kSpinLimit)) {
      *s_err = 1;
      dead = true;
    }
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
      ++round;
    }
    const int cur_ct = ct, cur_kb = kb;
    if (++kb == KB) {
      kb = 0;
      ++ct;
    }
    const bool seg_end = (cur_kb == KB - 1) || (u == u_end - 1);
    if (u == u_end - 1) STRACE(op_i, 2);
    if (!seg_end) continue;
    // ---- end of this CTA's share of column tile cur_ct: reduce over warps, then finish or hand over a partial
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        red[(w * M + m) * NT + lane * VEC + e] = acc[m][e];
        acc[m][e] = 0.0f;
      }
    consumers_sync();
    for (int idx = tid; idx < M * NT; idx += 256) {
      float v = 0.0f;
#pragma unroll
      for (int ww = 0; ww < kConsumerWarps; ++ww) v += red[ww * M * NT + idx];
      red[idx] = v;
    }
    consumers_sync();
    const long long ct_first_u = (long long)cur_ct * KB, ct_last_u = ct_first_u + KB - 1;
    const bool whole = (seg_begin <= ct_first_u) && (u == ct_last_u);
    bool finish = whole;
    if (!whole) {
      const int c_first = (int)(((ct_first_u + 1) * G + U - 1) / U - 1);
      const int c_last = (int)(((ct_last_u + 1) * G + U - 1) / U - 1);
      const int n_contrib = c_last - c_first + 1;
      const int slot = blockIdx.x - c_first;
      float* mine = a.partials + (((size_t)cur_ct * max_contrib + slot) * M) * NT;
      for (int idx = tid; idx < M * NT; idx += 256) mine[idx] = red[idx];
      __threadfence();
      consumers_sync();
      if (tid == 0) {
        const unsigned int prev = atomicAdd(&a.counters[cur_ct], 1u);
        const int last = (prev == (unsigned int)(n_contrib - 1));
        if (last) a.counters[cur_ct] = 0u;
        *s_last = last;
      }
      consumers_sync();
      if (*s_last) {
        __threadfence();
        const float* all = a.partials + ((size_t)cur_ct * max_contrib * M) * NT;
        for (int idx = tid; idx < M * NT; idx += 256) {
          // the slots are read eight at a time (one L2 round trip per batch) and added in slot order
          float v = 0.0f;
          for (int j0 = 0; j0 < n_contrib; j0 += 8) {
            float t[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) t[q] = j0 + q < n_contrib ? __ldcg(all + (size_t)(j0 + q) * M * NT + idx) : 0.0f;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (j0 + q < n_contrib) v += t[q];
          }
          red[idx] = v;
        }
        consumers_sync();
        finish = true;
      }
    }
    if (finish) {
      if (!ep.glu) {
        for (int idx = tid; idx < M * NT; idx += 256) {
          const int m = idx / NT, c = cur_ct * NT + (idx % NT);
          if (c < N) {
            float v = red[idx] + (bias ? to_f<T>(bias[c]) : 0.0f);
            switch (ep.act) {
              case TSB200_ACT_RELU: v = v < 0.0f ? 0.0f : v; break;
              case TSB200_ACT_SILU: v = v / (1.0f + expf(-v)); break;
              case TSB200_ACT_LEAKYRELU: v = v < 0.0f ? 0.01f * v : v; break;
              case TSB200_ACT_GELU: v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)); break;
              default: break;
            }
            const size_t o = (size_t)m * N + c;
            if (ep.residual) v += __ldcg(ep.residual + o);
            if (ep.y32) ep.y32[o] = v;
            else reinterpret_cast<T*>(ep.y)[o] = from_f<T>(v);
          }
        }
      } else {
        const int No = N / 2;
        for (int idx = tid; idx < M * (NT / 2); idx += 256) {
          const int m = idx / (NT / 2), j = idx % (NT / 2);
          const int c = cur_ct * NT + 2 * j;
          if (c + 1 < N) {
            float av = red[m * NT + 2 * j] + (bias ? to_f<T>(bias[c]) : 0.0f);
            const float gv = red[m * NT + 2 * j + 1] + (bias ? to_f<T>(bias[c + 1]) : 0.0f);
            if (ep.act == TSB200_ACT_SWIGLU) av = av / (1.0f + expf(-av));
            float v = av * gv;
            const size_t o = (size_t)m * No + (c >> 1);
            if (ep.residual) v += __ldcg(ep.residual + o);
            if (ep.y32) ep.y32[o] = v;
            else reinterpret_cast<T*>(ep.y)[o] = from_f<T>(v);
          }
        }
      }
      __threadfence();
    }
    consumers_sync();  // red is reused by the next segment; all epilogue stores are fenced
    if (finish && tid == 0) red_release_add(&a.done[op_i * kDoneStride], 1u);
    seg_begin = u + 1;
  }
}

// ------------------------------------------------------------------------------------------- the kernel
template <typename T, int M>
__global__ void __launch_bounds__(kStreamThreads, 1) decode_stack_kernel(StackArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int S = a.stages;
  unsigned char* stage_mem = smem;                                  // [S][16 KB]
  unsigned char* un = smem + (size_t)S * kTileBytes;                // union: {xs, red} | attention merge
  T* xs = reinterpret_cast<T*>(un);
  float* red = reinterpret_cast<float*>(un + a.xs_bytes);
  float* merge = reinterpret_cast<float*>(un);
  uint64_t* full = reinterpret_cast<uint64_t*>(un + a.union_bytes);
  uint64_t* empty = full + 16;
  __shared__ int s_err, s_last;
  __shared__ float s_stat[64];

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kConsumerWarps);
    }
    s_err = 0;
    s_last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (w == kConsumerWarps) {
    // weights never depend on earlier kernels: start streaming at once
    if (lane == 0) stack_stream_tiles<T>(a, stage_mem, full, empty, &s_err);
    return;
  }

  grid_dep_wait();  // the embedding rows, the cache length and last step's cache appends are visible from here on
  const StackConfig& c = a.c;
  const int T0 = __ldcg(c.dT);
  const int group = c.H / c.Hkv;
  const int AG = (group % 4 == 0) ? 4 : 1;
  const int yg = c.Hkv * (group / AG);
  const int splits = stack_splits((int)gridDim.x, M, yg, min(T0 + 1, c.Tmax));
  // cos / sin of this step's position for the pairs this lane holds in the attention (the same for every layer)
  constexpr int EPLA = TileVec<T>::N;
  float rcs[EPLA / 2], rsn[EPLA / 2];
  {
    const int lpt = c.hd / EPLA, li = (tid & 31) % lpt;
#pragma unroll
    for (int j = 0; j < EPLA / 2; ++j) {
      rcs[j] = 1.0f;
      rsn[j] = 0.0f;
      if (c.use_rope) {
        const float2 v = c.rope_tab[(size_t)min(T0, c.Tmax - 1) * (c.hd / 2) + li * (EPLA / 2) + j];
        rcs[j] = v.x;
        rsn[j] = v.y;
      }
    }
  }
  int s = 0;
  unsigned round = 0;
  bool dead = false;
  unsigned prev_target = 0;
  for (int i = 0; i < a.n_ops; ++i) {
    const StackOp* op = a.ops + i;
    LinGeom g{};
    unsigned target;
    bool mine;
    if (op->type == 0) {
      g = lin_geom<T>(op->K, op->N, (int)gridDim.x);
      target = (unsigned)g.CT;
      mine = (int)blockIdx.x < g.Gop;
    } else {
      target = (unsigned)(M * yg);
      mine = (int)blockIdx.x < M * yg * splits;
    }
    if (i == a.n_ops - 1) grid_dep_launch();  // the sampling kernels may become resident while the LM head streams
    if (mine) {
      // constants of this operation that can be fetched before its input exists
      NormConsts<T> nc;
      const bool hoist = op->type == 0 && op->xmode != 0 && op->K <= 256 * 16;
      if (hoist) load_norm_consts<T>(nc, reinterpret_cast<const T*>(op->gamma), reinterpret_cast<const T*>(op->beta), op->K, tid);
      if (i > 0) {
        if (tid == 0 && !poll_count(&a.done[(i - 1) * kDoneStride], prev_target, dead ? 64u : a.poll_limit, a.error_flag)) {
          s_err = 1;
          *a.error_flag = 1;
        }
        consumers_sync();
        if (*(volatile int*)&s_err) dead = true;
      }
      STRACE(i, 0);
      if (op->type == 0) {
        stack_linear<T, M>(a, op, i, g, stage_mem, xs, red, full, empty, s, round, &s_err, &s_last, s_stat, dead, hoist ? &nc : nullptr);
      } else if (AG == 4) {
        stack_attention<T, 4>(a, op, i, merge, &s_last, T0, splits, rcs, rsn);
      } else {
        stack_attention<T, 1>(a, op, i, merge, &s_last, T0, splits, rcs, rsn);
      }
      STRACE(i, 3);
    }
    prev_target = target;
  }
  // leave: the last CTA out clears the operation counters for the next launch
  if (tid == 0) {
    if (*(volatile int*)&s_err) *a.error_flag = 1;
    __threadfence();
    const unsigned prev = atomicAdd(&a.done[a.n_ops * kDoneStride], 1u);
    if (prev == gridDim.x - 1) {
      for (int i = 0; i <= a.n_ops; ++i) a.done[i * kDoneStride] = 0u;
    }
  }
}

// ------------------------------------------------------------------------------------------- host side
template <typename T>
static StackPlan stack_plan_t(const StackConfig& c, const StackOp* ops, int n_ops, int grid, int mode) {
  constexpr int NT = 32 * (16 / (int)sizeof(T));
  constexpr int EPL = 16 / (int)sizeof(T);
  StackPlan p{};
  size_t xs = 0;
  for (int i = 0; i < n_ops; ++i) {
    if (ops[i].type != 0) continue;
    const LinGeom g = lin_geom<T>(ops[i].K, ops[i].N, grid);
    const int64_t mc = g.KB / (g.U / g.Gop) + 2;
    const int64_t b = (int64_t)g.CT * mc * c.M * NT * 4;
    if (b > p.partial_bytes) p.partial_bytes = b;
    if (g.CT > p.counter_words) p.counter_words = g.CT;
    // staged k-tiles per row: the whole row, or (mma.sync variant, plain inputs) only the tiles a CTA streams
    int64_t kt = g.KB;
    const int64_t per = (g.U + g.Gop - 1) / g.Gop;
    if (mode == 2 && ops[i].xmode == 0 && ops[i].K % 8 == 0 && per < g.KB) kt = per;
    const size_t x = (((size_t)c.M * kt * kKT * sizeof(T)) + 127) & ~(size_t)127;
    if (x > xs) xs = x;
  }
  // mode 0 (FMA consumers): the eight warps' sums meet in shared memory; 2 (mma.sync): every warp owns its columns,
  // one [M][NT] block carries them to the epilogue
  const size_t red = (size_t)(mode == 2 ? 1 : kConsumerWarps) * c.M * NT * sizeof(float);
  const int lpt = c.hd / EPL;
  const int tpw = lpt > 0 ? 32 / lpt : 1;
  const int group = c.H / c.Hkv;
  const int AG = (group % 4 == 0) ? 4 : 1;
  const size_t merge = (size_t)kConsumerWarps * tpw * AG * (c.hd + 2) * sizeof(float);
  size_t un = xs + red;
  if (merge > un) un = merge;
  p.xs_bytes = xs;
  p.union_bytes = (un + 1023) & ~(size_t)1023;
  return p;
}

StackPlan stack_plan(const StackConfig& c, const StackOp* ops, int n_ops, int grid, int mode) {
  return c.dtype == TSB200_F16 ? stack_plan_t<__half>(c, ops, n_ops, grid, mode) : stack_plan_t<float>(c, ops, n_ops, grid, mode);
}

// counter scratch: [column-tile counters | operation counters | attention group counters]
static void counter_layout(int64_t counter_words, int n_ops, int M, int H, int64_t* off_done, int64_t* off_attn, int64_t* total) {
  *off_done = (counter_words * 4 + 255) & ~255LL;
  *off_attn = *off_done + (((int64_t)(n_ops + 1) * kDoneStride * 4 + 255) & ~255LL);
  *total = *off_attn + (((int64_t)M * H * 4 + 255) & ~255LL);
}

void decode_stack_scratch(const StackConfig& c, const StackOp* ops, int n_ops, int sm_count, int64_t* partial_bytes,
                          int64_t* counter_bytes, int64_t* attn_part_bytes) {
  const StackPlan p = stack_plan(c, ops, n_ops, sm_count, 0);
  int64_t od, oa, tot;
  counter_layout(p.counter_words, n_ops, c.M, c.H, &od, &oa, &tot);
  *partial_bytes = p.partial_bytes + 256;
  *counter_bytes = tot + 256;
  *attn_part_bytes = (int64_t)c.M * c.H * kMaxStackSplits * (c.hd + 2) * 4 + 256;
}

// Checks shared by both kernels; fills everything of the argument block except the shared-memory split.
int stack_fill_args(StackArgs& a, const StackPlan& p, const StackConfig& c, const StackOp* ops_dev, const StackOp* ops_host, int n_ops,
                    void* partials, void* counters, void* attn_part, int* error_flag, long long* trace) {
  const int EPL = c.dtype == TSB200_F16 ? 8 : 4;
  if (n_ops < 1 || c.M < 1) return 2;
  const int lpt = c.hd / EPL;
  if (c.hd % EPL != 0 || lpt < 1 || lpt > 32 || (lpt & (lpt - 1)) != 0 || c.H % c.Hkv != 0) return 2;
  if (c.use_rope && !c.rope_tab) return 2;
  for (int i = 0; i < n_ops; ++i)
    if (ops_host[i].type == 0 && (ops_host[i].xmode == 1 || ops_host[i].xmode == 2) && ops_host[i].K > 12288) return 2;
  int64_t od, oa, tot;
  counter_layout(p.counter_words, n_ops, c.M, c.H, &od, &oa, &tot);
  a = StackArgs{};
  a.ops = ops_dev;
  a.n_ops = n_ops;
  a.union_bytes = (int)p.union_bytes;
  a.xs_bytes = (int)p.xs_bytes;
  a.c = c;
  a.scale = 1.0f / sqrtf((float)c.hd);
  a.partials = reinterpret_cast<float*>(partials);
  a.counters = reinterpret_cast<unsigned int*>(counters);
  a.done = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(counters) + od);
  a.attn_cnt = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(counters) + oa);
  a.attn_part = reinterpret_cast<float*>(attn_part);
  a.error_flag = error_flag;
  a.trace = trace;
  a.poll_limit = c.poll_limit ? c.poll_limit : kPollLimit;
  return 1;
}

template <typename T, int M>
static int stack_launch_m(int device, const StackArgs& a, int grid, size_t smem, bool pdl, cudaStream_t s) {
  {
    // the CTAs wait on one another: the whole grid must be resident at once, else the caller launches per operation
    int per_sm = 0, sms = 0;
    TSB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stack_kernel<T, M>, kStreamThreads, smem));
    TSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    if ((long long)per_sm * sms < grid) return 2;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kStreamThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  TSB_CUDA(cudaLaunchKernelEx(&cfg, decode_stack_kernel<T, M>, a));
  count_launch(device);
  return 1;
}

template <typename T>
static int stack_launch_t(int device, DeviceState* st, const StackConfig& c, const StackOp* ops_dev, const StackOp* ops_host,
                          int n_ops, void* partials, void* counters, void* attn_part, int* error_flag, long long* trace, bool pdl,
                          cudaStream_t s) {
  const int grid = st->sm_count;
  if (c.M > 4) return 2;
  const StackPlan p = stack_plan(c, ops_host, n_ops, grid, 0);
  StackArgs a;
  const int r = stack_fill_args(a, p, c, ops_dev, ops_host, n_ops, partials, counters, attn_part, error_flag, trace);
  if (r != 1) return r;
  const size_t fixed = p.union_bytes + 32 * sizeof(uint64_t) + 128;
  const size_t budget = 226 * 1024;
  if (fixed + 3 * (size_t)kTileBytes > budget) return 2;
  int stages = (int)((budget - fixed) / kTileBytes);
  if (stages > 16) stages = 16;
  a.stages = stages;
  const size_t smem = fixed + (size_t)stages * kTileBytes;
  switch (c.M) {
    case 1: return stack_launch_m<T, 1>(device, a, grid, smem, pdl, s);
    case 2: return stack_launch_m<T, 2>(device, a, grid, smem, pdl, s);
    case 3: return stack_launch_m<T, 3>(device, a, grid, smem, pdl, s);
    case 4: return stack_launch_m<T, 4>(device, a, grid, smem, pdl, s);
  }
  return 2;
}

int launch_decode_stack(int device, DeviceState* st, const StackConfig& c, const StackOp* ops_dev, const StackOp* ops_host,
                        int n_ops, void* partials, void* counters, void* attn_part, int* error_flag,
                        long long* trace, bool pdl, cudaStream_t s) {
  if (!error_flag || !c.dT) return 2;
  if (c.tp_size > 1) {
    // tensor parallelism inside the kernel exists in the mma.sync variant only
    if (c.dtype != TSB200_F16 || c.tp_size > kStackMaxRanks || !c.peer[c.tp_rank]) return 2;
    return launch_decode_stack_mma(device, st, c, ops_dev, ops_host, n_ops, partials, counters, attn_part, error_flag, trace, pdl, s);
  }
  if (c.dtype == TSB200_F16) {
    // fp16: eight warps eat the weight stream with ldmatrix + mma.sync; shapes that kernel does not take fall through
    // to the CUDA-core consumers
    const int r = launch_decode_stack_mma(device, st, c, ops_dev, ops_host, n_ops, partials, counters, attn_part, error_flag, trace, pdl, s);
    if (r != 2) return r;
    return stack_launch_t<__half>(device, st, c, ops_dev, ops_host, n_ops, partials, counters, attn_part, error_flag, trace, pdl, s);
  }
  return stack_launch_t<float>(device, st, c, ops_dev, ops_host, n_ops, partials, counters, attn_part, error_flag, trace, pdl, s);
}

template <typename T, int M>
static int stack_attr_one() {
  TSB_CUDA(cudaFuncSetAttribute(decode_stack_kernel<T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  return 1;
}
int init_stack_attrs(int device) {
  static bool done[kMaxDevices] = {};
  if (done[device]) return 1;
  TSB_TRY((stack_attr_one<float, 1>())); TSB_TRY((stack_attr_one<float, 2>())); TSB_TRY((stack_attr_one<float, 3>())); TSB_TRY((stack_attr_one<float, 4>()));
  TSB_TRY((stack_attr_one<__half, 1>())); TSB_TRY((stack_attr_one<__half, 2>())); TSB_TRY((stack_attr_one<__half, 3>())); TSB_TRY((stack_attr_one<__half, 4>()));
  TSB_TRY(init_stack_mma_attrs());
  done[device] = true;
  return 1;
}

}  // namespace tsb
