// Persistent decode-step kernel, fp16, tensor-core consumers (tcgen05 + TMEM): the sm_100a form of the layer-stack
// kernel described in decode_stack.cu.
//
// What changes against the CUDA-core variant is who eats the weight tiles.  There, eight warps convert and
// multiply every fp16 weight on the FMA pipes (~110 instructions per warp and 16 KB tile), which caps a CTA at about
// its share of HBM bandwidth, so data prefetched during a dependency wait cannot be caught up on.  Here:
//   * warp 8 (one lane) streams the packed weight tiles with TMA bulk copies (cp.async.bulk, one linear 16 KB copy
//     per stage: the tiles are stored as their 128-byte-swizzled shared-memory image, four 64-column boxes each);
//   * warp 9 issues tcgen05.mma (cta_group::1, kind::f16, M = 128 weight columns, N = 16, K = 16): the weight
//     tile is the A operand, read in place from the stage (MN-major, SWIZZLE_128B), the B operand is a 1 KB window
//     [16 rows][32 k] that the warp fills from the staged activations just before issuing (rows = sequences, the
//     unused rows stay zero), the accumulator [128 columns][16 rows] fp32 lives in tensor memory, two halves per
//     256-column tile, double buffered across column tiles; tcgen05.commit returns the stage to the TMA warp;
//   * warps 0..7 follow the dependency chain only: wait for the previous operation, stage (and normalise) the
//     activations, read finished accumulators with tcgen05.ld, exchange partial sums of shared column tiles,
//     apply the epilogue, and run the in-kernel attention.
// The multiply itself costs the SM four instructions per tile, so a full ring is drained at shared-memory speed and
// the stream only ever waits for HBM.  Up to 8 sequences ride in the N dimension at no extra cost.
// Every wait is bounded; all roles reach the common exit, where tensor memory is released.
#include "decode_stack.cuh"

namespace tsb {

constexpr int kTcsThreads = 320;   // 8 worker warps, TMA warp, MMA warp
constexpr int kWinBytes = 1024;    // B-operand window per stage: [4 k-chunks][2 row groups][8 rows][16 B]
constexpr int kAccCols = 32;       // TMEM columns per accumulator buffer: two 128-column halves x 16 rows
constexpr int kTmemCols = 64;      // two buffers
constexpr int kMaxTcRows = 8;

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in 16-byte units,
// version 1, swizzle mode (0 none, 2 = 128 bytes).
__device__ __forceinline__ uint64_t ts_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)swizzle << 61;
  return d;
}
__device__ __forceinline__ void ts_umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void ts_umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ts_tmem_ld8(uint32_t taddr, float* f) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void ts_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void ts_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void ts_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

struct TcsSmem {
  unsigned char* stage_mem;
  unsigned char* un;
  unsigned char* win;
  uint64_t *full, *empty, *xready, *acc_full, *acc_empty;
  uint32_t* tmem_slot;
};

// ------------------------------------------------------------------------------------------- MMA warp
__device__ __forceinline__ void tcs_mma_warp(const StackArgs& a, const TcsSmem& sm, uint32_t tmem_base, volatile int* s_err) {
  const int S = a.stages, lane = threadIdx.x & 31, M = a.c.M;
  const __half* xs = reinterpret_cast<const __half*>(sm.un);
  // instruction descriptor: D fp32, A / B fp16, A MN-major (weights [k][n]), B K-major (activations [row][k]), N = 16, M = 128
  const uint32_t idesc = (1u << 4) | (1u << 15) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  int s = 0;
  unsigned round = 0, n_seg = 0, n_lin = 0;
  bool dead = false;
  long long cyc_x = 0, cyc_full = 0, cyc_win = 0, cyc_issue = 0, cyc_acc = 0, n_tiles = 0, t_mark = 0;
  const bool prof = a.trace != nullptr;
#define MMA_LAP(acc_var)                 \
  do {                                   \
    if (prof) {                          \
      const long long t_now = clock64(); \
      acc_var += t_now - t_mark;         \
      t_mark = t_now;                    \
    }                                    \
  } while (0)
  for (int i = 0; i < a.n_ops; ++i) {
    const StackOp* op = a.ops + i;
    if (op->type != 0) continue;
    const LinGeom g = lin_geom<__half>(op->K, op->N, (int)gridDim.x);
    if ((int)blockIdx.x >= g.Gop) continue;
    if (*s_err) dead = true;
    if (prof) t_mark = clock64();
    // the workers have staged this operation's activations
    if (!mbar_wait(sm.xready, n_lin & 1u, dead ? 4096u : kSpinLimit)) {
      *s_err = 1;
      dead = true;
    }
    ++n_lin;
    MMA_LAP(cyc_x);
    const int Kp = g.KB * kKT;
    const int u_begin = (int)(g.U * blockIdx.x / g.Gop), u_end = (int)(g.U * (blockIdx.x + 1) / g.Gop);
    int kb = u_begin % g.KB;
    bool seg_start = true;
    for (int u = u_begin; u < u_end; ++u) {
      const unsigned b = n_seg & 1u;
      if (*s_err) dead = true;
      if (seg_start && n_seg >= 2 && !mbar_wait(&sm.acc_empty[b], ((n_seg >> 1) - 1u) & 1u, dead ? 4096u : kSpinLimit)) {
        *s_err = 1;
        dead = true;
      }
      MMA_LAP(cyc_acc);
      if (!mbar_wait(&sm.full[s], round & 1u, dead ? 4096u : kSpinLimit)) {
        *s_err = 1;
        dead = true;
      }
      MMA_LAP(cyc_full);
      // B-operand window of this tile: rows 0..7 = sequences (zero beyond M), 32 k values, as 8x16-byte core matrices
      {
        const int r = lane & 7, kc = lane >> 3;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < M) v = *reinterpret_cast<const uint4*>(xs + (size_t)r * Kp + kb * kKT + kc * 8);
        *reinterpret_cast<uint4*>(sm.win + (size_t)s * kWinBytes + kc * 256 + r * 16) = v;
      }
      ts_fence_async_smem();  // the window was written through the generic proxy, the tensor core reads it through the async proxy
      __syncwarp();
      MMA_LAP(cyc_win);
      const bool seg_end = (kb == g.KB - 1) || (u == u_end - 1);
      if (lane == 0) {
        ts_fence_after();
        if (!dead) {
          const uint32_t a_base = smem_u32(sm.stage_mem + (size_t)s * kTileBytes);
          const uint32_t b_base = smem_u32(sm.win + (size_t)s * kWinBytes);
#pragma unroll
          for (int kk = 0; kk < 2; ++kk) {
            // B (K-major, no swizzle): core matrices 256 B apart along k (LBO), 128 B apart along the rows (SBO); 16 k = 512 B
            const uint64_t bd = ts_desc(b_base + kk * 512, 256, 128, 0);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              // A (MN-major, SWIZZLE_128B): 64-column boxes [32 k][128 B]; 8-k groups 1024 B apart (SBO), the next 64
              // columns 4096 B away (LBO); 16 k = 2048 B; the second 128-column half starts at 8192 B
              const uint64_t ad = ts_desc(a_base + h * 8192 + kk * 2048, 4096, 1024, 2);
              ts_umma_f16(tmem_base + b * kAccCols + h * 16, ad, bd, idesc, (seg_start && kk == 0) ? 0u : 1u);
            }
          }
        }
        ts_umma_commit(&sm.empty[s]);                  // the stage returns to the TMA warp when these MMAs have read it
        if (seg_end) ts_umma_commit(&sm.acc_full[b]);  // this CTA's share of the column tile is complete
      }
      __syncwarp();
      MMA_LAP(cyc_issue);
      ++n_tiles;
      seg_start = seg_end;
      if (seg_end) ++n_seg;
      if (++kb == g.KB) kb = 0;
      if (++s == S) {
        s = 0;
        ++round;
      }
    }
  }
#undef MMA_LAP
  if (prof && lane == 0) {
    long long* o = a.trace + (size_t)gridDim.x * a.n_ops * 8 + (size_t)blockIdx.x * 8;
    o[0] = cyc_x; o[1] = cyc_full; o[2] = cyc_win; o[3] = cyc_issue; o[4] = cyc_acc; o[5] = n_tiles;
  }
}

// ------------------------------------------------------------------------------------------- workers: one linear
// Fused epilogue of one output element.
__device__ __forceinline__ float tcs_act(float v, int act) {
  switch (act) {
    case TSB200_ACT_RELU: return v < 0.0f ? 0.0f : v;
    case TSB200_ACT_SILU: return v / (1.0f + expf(-v));
    case TSB200_ACT_LEAKYRELU: return v < 0.0f ? 0.01f * v : v;
    case TSB200_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    default: return v;
  }
}

__device__ __forceinline__ void tcs_linear(const StackArgs& a, const StackOp* op, int op_i, const LinGeom& g, const TcsSmem& sm,
                                           uint32_t tmem_base, unsigned& n_seg, volatile int* s_err, volatile int* s_last,
                                           float* s_stat, bool& dead, const NormConsts<__half>* nc) {
  typedef __half T;
  constexpr int NT = 256;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int M = a.c.M;
  const int K = op->K, N = op->N, KB = g.KB;
  const int Kp = KB * kKT;
  const long long U = g.U, G = g.Gop;
  const int u_begin = (int)(U * blockIdx.x / G), u_end = (int)(U * (blockIdx.x + 1) / G);
  const int max_contrib = (int)(KB / (U / G)) + 2;
  const Epilogue ep = op->ep;
  T* xs = reinterpret_cast<T*>(sm.un);

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
  if (tid == 0) mbar_arrive(sm.xready);  // release: the MMA warp may read the staged rows
  STRACE(op_i, 1);

  // this thread's column inside a 256-column tile: TMEM lane quarter q = warp % 4, column half h = warp / 4
  const int q = w & 3, h = w >> 2;
  const int c_local = h * 128 + q * 32 + lane;
  const T* bias = reinterpret_cast<const T*>(ep.bias);
  const int ct_first = u_begin / KB, ct_last = (u_end - 1) / KB;
  // the bias (and residual) lines of this CTA's columns are needed at the very end of the chain: pull them into L2 now
  if (bias && lane == 0)
    for (int ct = ct_first; ct <= ct_last; ++ct) {
      const int c = ct * NT + c_local;
      if (c < N) prefetch_l2(bias + c);
    }

  for (int ct = ct_first; ct <= ct_last; ++ct) {
    const long long ct_first_u = (long long)ct * KB, ct_last_u = ct_first_u + KB - 1;
    const bool whole = (u_begin <= ct_first_u) && (u_end - 1 >= ct_last_u);
    const unsigned b = n_seg & 1u;
    if (*s_err) dead = true;
    if (!mbar_wait(&sm.acc_full[b], (n_seg >> 1) & 1u, dead ? 4096u : kSpinLimit)) {
      *s_err = 1;
      dead = true;
    }
    ts_fence_after();
    float v[kMaxTcRows];
    ts_tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + b * kAccCols + h * 16, v);
    ts_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.acc_empty[b]);
    ++n_seg;
    if (ct == ct_last) STRACE(op_i, 2);

    bool finish = whole;
    if (!whole) {
      const int c_first = (int)(((ct_first_u + 1) * G + U - 1) / U - 1);
      const int c_last = (int)(((ct_last_u + 1) * G + U - 1) / U - 1);
      const int n_contrib = c_last - c_first + 1;
      const int slot = blockIdx.x - c_first;
      float* mine = a.partials + (((size_t)ct * max_contrib + slot) * M) * NT + c_local;
      for (int m = 0; m < M; ++m) mine[(size_t)m * NT] = v[m];
      __threadfence();
      consumers_sync();
      if (tid == 0) {
        const unsigned int prev = atomicAdd(&a.counters[ct], 1u);
        const int last = (prev == (unsigned int)(n_contrib - 1));
        if (last) a.counters[ct] = 0u;
        *s_last = last;
      }
      consumers_sync();
      if (*s_last) {
        __threadfence();
        const float* all = a.partials + ((size_t)ct * max_contrib * M) * NT + c_local;
#pragma unroll
        for (int m = 0; m < kMaxTcRows; ++m) v[m] = 0.0f;
        for (int j = 0; j < n_contrib; ++j)
          for (int m = 0; m < M; ++m) v[m] += __ldcg(all + ((size_t)j * M + m) * NT);
        finish = true;
      }
    }
    if (finish) {
      const int c = ct * NT + c_local;
      if (!ep.glu) {
        if (c < N) {
          const float bv = bias ? to_f<T>(bias[c]) : 0.0f;
          for (int m = 0; m < M; ++m) {
            float x = tcs_act(v[m] + bv, ep.act);
            const size_t o = (size_t)m * N + c;
            if (ep.residual) x += __ldcg(ep.residual + o);
            if (ep.y32) ep.y32[o] = x;
            else reinterpret_cast<T*>(ep.y)[o] = from_f<T>(x);
          }
        }
      } else {
        // interleaved (a_j, g_j) column pairs: the even lane takes the gate value from its odd neighbour
        const int No = N / 2;
        const float bv = (bias && c < N) ? to_f<T>(bias[c]) : 0.0f;
        for (int m = 0; m < M; ++m) {
          const float mine_v = v[m] + bv;
          const float other = __shfl_xor_sync(0xffffffffu, mine_v, 1);
          if ((lane & 1) == 0 && c + 1 < N) {
            float av = mine_v;
            if (ep.act == TSB200_ACT_SWIGLU) av = av / (1.0f + expf(-av));
            float x = av * other;
            const size_t o = (size_t)m * No + (c >> 1);
            if (ep.residual) x += __ldcg(ep.residual + o);
            if (ep.y32) ep.y32[o] = x;
            else reinterpret_cast<T*>(ep.y)[o] = from_f<T>(x);
          }
        }
      }
      __threadfence();
    }
    consumers_sync();  // s_last is reused by the next segment; all epilogue stores are fenced
    if (finish && tid == 0) red_release_add(&a.done[op_i * kDoneStride], 1u);
  }
}

// ------------------------------------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(kTcsThreads, 1) decode_stack_tc_kernel(StackArgs a) {
  typedef __half T;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.stages;
  TcsSmem sm;
  sm.stage_mem = smem;                                   // [S][16 KB], 1024-byte aligned (swizzle atoms)
  sm.un = smem + (size_t)S * kTileBytes;                 // staged activations | attention merge
  sm.win = sm.un + a.union_bytes;                        // [S][1 KB] B-operand windows
  sm.full = reinterpret_cast<uint64_t*>(sm.win + (size_t)S * kWinBytes);
  sm.empty = sm.full + 16;
  sm.xready = sm.empty + 16;
  sm.acc_full = sm.xready + 1;
  sm.acc_empty = sm.acc_full + 2;
  sm.tmem_slot = reinterpret_cast<uint32_t*>(sm.acc_empty + 2);
  __shared__ int s_err, s_last;
  __shared__ float s_stat[64];

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&sm.full[i], 1);
      mbar_init(&sm.empty[i], 1);
    }
    mbar_init(sm.xready, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.acc_full[i], 1);
      mbar_init(&sm.acc_empty[i], kConsumerWarps);
    }
    s_err = 0;
    s_last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // rows 8..15 of every window (and rows beyond M) are never written again: zero once
  for (int i = tid; i < S * kWinBytes / 16; i += kTcsThreads) reinterpret_cast<uint4*>(sm.win)[i] = make_uint4(0u, 0u, 0u, 0u);
  ts_fence_async_smem();
  if (w == 9) {  // tensor memory: two accumulator buffers (one warp, whole-warp instruction)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(sm.tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  ts_fence_before();
  __syncthreads();
  ts_fence_after();
  const uint32_t tmem_base = *sm.tmem_slot;

  if (w == 8) {
    // weights never depend on earlier kernels: start streaming at once
    if (lane == 0) stack_stream_tiles<__half>(a, sm.stage_mem, sm.full, sm.empty, &s_err);
  } else if (w == 9) {
    tcs_mma_warp(a, sm, tmem_base, &s_err);
  } else {
    grid_dep_wait();  // the embedding rows, the cache length and last step's cache appends are visible from here on
    const StackConfig& c = a.c;
    const int M = c.M;
    const int T0 = __ldcg(c.dT);
    const int group = c.H / c.Hkv;
    const int AG = (group % 4 == 0) ? 4 : 1;
    const int yg = c.Hkv * (group / AG);
    const int splits = stack_splits((int)gridDim.x, M, yg, min(T0 + 1, c.Tmax));
    float* merge = reinterpret_cast<float*>(sm.un);
    // cos / sin of this step's position for the pairs this lane holds in the attention (the same for every layer)
    float rcs[4], rsn[4];
    {
      const int lpt = c.hd / 8, li = lane % lpt;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        rcs[j] = 1.0f;
        rsn[j] = 0.0f;
        if (c.use_rope) {
          const float2 v = c.rope_tab[(size_t)min(T0, c.Tmax - 1) * (c.hd / 2) + li * 4 + j];
          rcs[j] = v.x;
          rsn[j] = v.y;
        }
      }
    }
    unsigned n_seg = 0;
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
          if (tid == 0 && !poll_count(&a.done[(i - 1) * kDoneStride], prev_target, dead ? 64u : kPollLimit, a.error_flag)) {
            s_err = 1;
            *a.error_flag = 1;
          }
          consumers_sync();
          if (*(volatile int*)&s_err) dead = true;
        }
        STRACE(i, 0);
        if (op->type == 0) {
          tcs_linear(a, op, i, g, sm, tmem_base, n_seg, &s_err, &s_last, s_stat, dead, hoist ? &nc : nullptr);
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
  // common exit of all roles: every MMA this CTA issued has been committed and awaited by the workers
  ts_fence_before();
  __syncthreads();
  if (w == 9) {
    ts_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------- host side
int init_stack_tc_attrs() {
  TSB_CUDA(cudaFuncSetAttribute(decode_stack_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  return 1;
}

int launch_decode_stack_tc(int device, DeviceState* st, const StackConfig& c, const StackOp* ops_dev, const StackOp* ops_host,
                           int n_ops, void* partials, void* counters, void* attn_part, int* error_flag,
                           long long* trace, bool pdl, cudaStream_t s) {
  if (c.dtype != TSB200_F16 || c.M > kMaxTcRows) return 2;
  const int grid = st->sm_count;
  const StackPlan p = stack_plan(c, ops_host, n_ops, grid, 1);
  StackArgs a;
  const int r = stack_fill_args(a, p, c, ops_dev, ops_host, n_ops, partials, counters, attn_part, error_flag, trace);
  if (r != 1) return r;
  const size_t fixed = p.union_bytes + 40 * sizeof(uint64_t) + 1024 /* alignment slack */ + 128;
  const size_t budget = 225 * 1024;  // the kernel also has ~1 KB of static shared memory
  const size_t per_stage = (size_t)kTileBytes + kWinBytes;
  if (fixed + 3 * per_stage > budget) return 2;
  int stages = (int)((budget - fixed) / per_stage);
  if (stages > 16) stages = 16;
  a.stages = stages;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kTcsThreads);
  cfg.dynamicSmemBytes = fixed + (size_t)stages * per_stage;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  TSB_CUDA(cudaLaunchKernelEx(&cfg, decode_stack_tc_kernel, a));
  count_launch(device);
  return 1;
}

}  // namespace tsb
