// Persistent decode-step kernel, fp16, warp-level tensor-core consumers (ldmatrix + mma.sync m16n8k16).
//
// Same program, protocol and producer as decode_stack.cu (TMA bulk copies of the packed weight tiles, which are
// stored as their 128-byte-swizzled shared-memory image, into a stage ring), but the weight stream is eaten by all eight worker warps in parallel: per 16 KB
// tile a warp owns 32 of the 256 columns, loads them as transposed 8x8 fragments (ldmatrix.trans, conflict-free on
// the swizzled stage) and multiplies them with the staged activations (up to 8 sequences in the n dimension of the
// instruction): 4 ldmatrix + 4 mma + 4 shared loads per warp and tile instead of ~110 FMA-pipe instructions, and no
// cross-warp reduction (a warp sees all 32 k of its columns).  Eight independent warps hide the latencies of the
// barrier handshakes (a single-warp tcgen05 consumer was measured slower for that reason), so a ring filled during a
// dependency wait is drained several times faster than HBM refills it.
#include <cstdlib>

#include "decode_stack.cuh"

namespace tsb {

constexpr int kMmaMaxRows = 8;

__device__ __forceinline__ void mm_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mm_mma_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ------------------------------------------------------------------------------------------- workers: one linear
template <bool TP>  // TP: tensor-parallel program (exchange sites); the single-GPU instantiation carries none of that code
__device__ __forceinline__ void mm_linear(const StackArgs& a, const StackOp* op, int op_i, const LinGeom& g, unsigned char* stage_mem,
                                          __half* xs, float* red, uint64_t* full, uint64_t* empty, int& s, unsigned& round,
                                          volatile int* s_err, volatile int* s_last, float* s_stat, bool& dead,
                                          const NormVecConsts<__half>* nvc) {
  typedef __half T;
  constexpr int NT = 256;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int S = a.stages, M = a.c.M;
  const int K = op->K, N = op->N, KB = g.KB;
  const int Kp = KB * kKT;
  const long long U = g.U, G = g.Gop;
  const int u_begin = (int)(U * blockIdx.x / G), u_end = (int)(U * (blockIdx.x + 1) / G);
  const int max_contrib = (int)(KB / (U / G)) + 2;
  const Epilogue ep = op->ep;

  // a plain input is staged as the slice of k-tiles this CTA streams when that is less than one pass over K
  const int n_t = u_end - u_begin;
  const bool slice = op->xmode == 0 && K % 8 == 0 && n_t < KB;
  const int xstride = slice ? n_t * kKT : Kp;  // elements between staged rows
  if (slice) {
    stage_plain_slice(xs, reinterpret_cast<const T*>(op->x), M, K, KB, u_begin % KB, n_t, xstride, tid);
  } else if (op->xmode == 0) {
    if (K % 8 == 0) stage_plain_vec<T>(xs, reinterpret_cast<const T*>(op->x), M, K, Kp, tid);
    else stage_plain<T>(xs, reinterpret_cast<const T*>(op->x), M, K, Kp, tid);
  } else if (nvc) {
    const bool summed = TP && op->ssite >= 0;
    stage_norm_vec<T>(xs, reinterpret_cast<const float*>(op->x), *nvc, op->xmode, op->eps, M, K, Kp, tid, s_stat,
                      summed ? stack_xch(a.c, a.c.tp_rank, op->ssite, 0) : nullptr, a.c.tp_size, (size_t)kStackXchRows * a.c.d,
                      (summed && blockIdx.x == 0) ? op->x_out : nullptr);
  } else if (K <= 256 * 16) {
    stage_norm<T, 16>(xs, reinterpret_cast<const float*>(op->x), reinterpret_cast<const T*>(op->gamma),
                      reinterpret_cast<const T*>(op->beta), nullptr, op->xmode, op->eps, M, K, Kp, tid, s_stat);
  } else {
    stage_norm<T, 48>(xs, reinterpret_cast<const float*>(op->x), reinterpret_cast<const T*>(op->gamma),
                      reinterpret_cast<const T*>(op->beta), nullptr, op->xmode, op->eps, M, K, Kp, tid, s_stat);
  }
  STRACE(op_i, 4);
  consumers_sync();
  STRACE(op_i, 1);

  // this warp's 32 columns of a tile: 64-column box `chunk`, half `hf`; two 16-column blocks, each one mma wide
  const int chunk = w >> 1, hf = w & 1;
  const int g8 = lane >> 2, t4 = lane & 3;
  // ldmatrix row addresses: lanes 0-7 / 8-15 / 16-23 / 24-31 give the rows of the four 8x8 blocks
  //   (k 0-7, cols 0-7), (k 0-7, cols 8-15), (k 8-15, cols 0-7), (k 8-15, cols 8-15) of a [16 k][16 columns] block
  const int lrow = (lane & 7) + ((lane >> 4) << 3);
  const int lunit = (lane >> 3) & 1;
  const bool row_live = g8 < M;                       // B fragment: n = lane / 4 is the sequence
  const __half* xrow = xs + (size_t)(row_live ? g8 : 0) * xstride + 2 * t4;
  float d[2][4];
#pragma unroll
  for (int cb = 0; cb < 2; ++cb)
#pragma unroll
    for (int e = 0; e < 4; ++e) d[cb][e] = 0.0f;

  int seg_begin = u_begin;
  int ct = u_begin / KB, kb = u_begin % KB;
  const T* bias = reinterpret_cast<const T*>(ep.bias);
  // Epilogue operands of this CTA's first two column tiles (it rarely touches more), fetched now: their memory
  // latency would otherwise sit at the very end of the dependency chain.  A missing bias / residual aliases the
  // weights and is switched off by a factor, indices are clamped: every address a thread can form is valid.
  const int ct0 = ct;
  const bool xchg = TP && op->xsite >= 0;  // row-sharded linear under tensor parallelism: partial sums go to every rank
  if (xchg && a.c.tp_rank != 0) bias = nullptr;  // the bias is added once, by rank 0
  const float b_on = bias ? 1.0f : 0.0f, r_on = ep.residual ? 1.0f : 0.0f;
  const T* bp = bias ? bias : reinterpret_cast<const T*>(op->Wp);
  const float* rp = ep.residual ? ep.residual : reinterpret_cast<const float*>(op->Wp);
  float pre_b0[2], pre_b1[2], pre_r[2];
#pragma unroll
  for (int sg = 0; sg < 2; ++sg) {
    if (!ep.glu) {
      const int c = (ct0 + sg) * NT + tid;
      const int cc = c < N ? c : 0;
      pre_b0[sg] = b_on * to_f<T>(bp[cc]);
      pre_b1[sg] = 0.0f;
      pre_r[sg] = r_on * __ldcg(rp + cc);
    } else {
      const int c = (ct0 + sg) * NT + 2 * (tid & 127);
      const int cc = c + 1 < N ? c : 0;
      pre_b0[sg] = b_on * to_f<T>(bp[cc]);
      pre_b1[sg] = b_on * to_f<T>(bp[cc + 1]);
      pre_r[sg] = 0.0f;
    }
  }
  // Per-lane constants of the tile loop: byte offsets of this lane's four ldmatrix rows inside a stage
  // (k half kk, 16-column block cb), shared-memory addresses of the ring.
  uint32_t loff[2][2];
#pragma unroll
  for (int kk = 0; kk < 2; ++kk)
#pragma unroll
    for (int cb = 0; cb < 2; ++cb) {
      const int k = kk * 16 + lrow, unit = hf * 4 + cb * 2 + lunit;
      loff[kk][cb] = (uint32_t)(chunk * 4096 + k * 128 + ((unit ^ (k & 7)) << 4));
    }
  const uint32_t stage0 = smem_u32(stage_mem);
  // kk = 0 and kk = 1 accumulate separately (two independent mma chains per column block), summed at the segment end
  float d2[2][4];
#pragma unroll
  for (int cb = 0; cb < 2; ++cb)
#pragma unroll
    for (int e = 0; e < 4; ++e) d2[cb][e] = 0.0f;
  // one tile: 4 shared loads of the activation fragments, 4 ldmatrix, 4 mma
  auto eat = [&](uint32_t sbase, const __half* xp) {
    uint32_t b00 = 0u, b01 = 0u, b10 = 0u, b11 = 0u;
    if (row_live) {
      b00 = *reinterpret_cast<const uint32_t*>(xp);
      b01 = *reinterpret_cast<const uint32_t*>(xp + 8);
      b10 = *reinterpret_cast<const uint32_t*>(xp + 16);
      b11 = *reinterpret_cast<const uint32_t*>(xp + 24);
    }
    uint32_t f0[4], f1[4], f2[4], f3[4];
    mm_ldmatrix_x4_trans(sbase + loff[0][0], f0[0], f0[1], f0[2], f0[3]);
    mm_ldmatrix_x4_trans(sbase + loff[0][1], f1[0], f1[1], f1[2], f1[3]);
    mm_ldmatrix_x4_trans(sbase + loff[1][0], f2[0], f2[1], f2[2], f2[3]);
    mm_ldmatrix_x4_trans(sbase + loff[1][1], f3[0], f3[1], f3[2], f3[3]);
    mm_mma_16816(d[0], f0[0], f0[1], f0[2], f0[3], b00, b01);
    mm_mma_16816(d[1], f1[0], f1[1], f1[2], f1[3], b00, b01);
    mm_mma_16816(d2[0], f2[0], f2[1], f2[2], f2[3], b10, b11);
    mm_mma_16816(d2[1], f3[0], f3[1], f3[2], f3[3], b10, b11);
  };
  // Slots of the operation's last tiles (no later tile of this operation needs them) can be held back: handing them
  // over starts the producer's burst for the next operation, whose traffic delays the round trips of the exchange.
  const int n_hold = a.defer ? min(S, u_end - u_begin) : 0;
  const int u_hold = u_end - n_hold;
  auto release_held = [&]() {
    if (lane == 0) {
      int sl = s;
      for (int k = 0; k < n_hold; ++k) {
        sl = (sl == 0) ? S - 1 : sl - 1;
        mbar_arrive(&empty[sl]);
      }
    }
  };
  int un = u_begin;  // next tile
  while (un < u_end) {
    // this CTA's share of column tile ct: n tiles, eaten two at a time (the loop carries no segment logic)
    const int n = min(u_end - un, KB - kb);
    const __half* xp = xrow + (size_t)(slice ? (un - u_begin) : kb) * kKT;
    if (*s_err) dead = true;
    // a CTA that gave up walks through the rest of its program without waiting (its results are discarded)
    const unsigned lim = kSpinLimit;
    int i = 0;
    for (; i + 2 <= n; i += 2) {
      int s1 = s + 1;
      unsigned r1 = round;
      if (s1 == S) {
        s1 = 0;
        ++r1;
      }
      if (!dead && (!mbar_wait(&full[s], round & 1u, lim) || !mbar_wait(&full[s1], r1 & 1u, lim))) {
        *s_err = 1;
        dead = true;
      }
      eat(stage0 + (uint32_t)s * kTileBytes, xp);
      eat(stage0 + (uint32_t)s1 * kTileBytes, xp + kKT);
      __syncwarp();
      if (lane == 0) {
        if (un + i < u_hold) mbar_arrive(&empty[s]);
        if (un + i + 1 < u_hold) mbar_arrive(&empty[s1]);
      }
      s = s1 + 1;
      round = r1;
      if (s == S) {
        s = 0;
        ++round;
      }
      xp += 2 * kKT;
    }
    if (i < n) {
      if (!dead && !mbar_wait(&full[s], round & 1u, lim)) {
        *s_err = 1;
        dead = true;
      }
      eat(stage0 + (uint32_t)s * kTileBytes, xp);
      __syncwarp();
      if (lane == 0 && un + i < u_hold) mbar_arrive(&empty[s]);
      if (++s == S) {
        s = 0;
        ++round;
      }
    }
    const int u = un + n - 1;  // the segment's last tile
    const int cur_ct = ct;
    ++ct;
    kb = 0;
    if (u == u_end - 1) STRACE(op_i, 2);
#pragma unroll
    for (int cb = 0; cb < 2; ++cb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        d[cb][e] += d2[cb][e];
        d2[cb][e] = 0.0f;
      }
    // ---- end of this CTA's share of column tile cur_ct: the accumulator fragments go to red[row][column]
    //      (fragment: d0,d1 = column g8, rows 2*t4, 2*t4+1; d2,d3 = column g8 + 8)
#pragma unroll
    for (int cb = 0; cb < 2; ++cb) {
      const int col = chunk * 64 + hf * 32 + cb * 16 + g8;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = 2 * t4 + (e & 1);
        if (n < M) red[n * NT + col + (e >> 1) * 8] = d[cb][e];
        d[cb][e] = 0.0f;
      }
    }
    consumers_sync();
    if (u == u_end - 1) STRACE(op_i, 5);
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
      consumers_sync();
      if (tid == 0) {
        const unsigned int prev = atom_add_acq_rel(&a.counters[cur_ct], 1u);  // publishes the CTA's partial, acquires the others'
        const int last = (prev == (unsigned int)(n_contrib - 1));
        if (last) a.counters[cur_ct] = 0u;
        *s_last = last;
      }
      consumers_sync();
      if (u == u_end - 1) STRACE(op_i, 6);
      if (u == u_end - 1 && a.defer == 1) release_held();
      if (*s_last) {
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
        if (u == u_end - 1) STRACE(op_i, 7);
        finish = true;
      }
    }
    if (finish) {
      const int sg = cur_ct - ct0;
      const bool pre = sg < 2;
      if (!ep.glu) {
        for (int idx = tid; idx < M * NT; idx += 256) {
          const int m = idx / NT, c = cur_ct * NT + (idx % NT);  // idx % NT == tid: one column per thread, rows in turn
          if (c < N) {
            float v = red[idx] + (pre ? (sg == 0 ? pre_b0[0] : pre_b0[1]) : (bias ? to_f<T>(bias[c]) : 0.0f));
            switch (ep.act) {
              case TSB200_ACT_RELU: v = v < 0.0f ? 0.0f : v; break;
              case TSB200_ACT_SILU: v = v / (1.0f + expf(-v)); break;
              case TSB200_ACT_LEAKYRELU: v = v < 0.0f ? 0.01f * v : v; break;
              case TSB200_ACT_GELU: v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)); break;
              default: break;
            }
            const size_t o = (size_t)m * N + c;
            if (xchg) {
              // this rank's slot of the exchange buffer on every rank (peer stores over NVLink for the others)
              for (int r = 0; r < a.c.tp_size; ++r) stack_xch(a.c, r, op->xsite, a.c.tp_rank)[o] = v;
              continue;
            }
            if (ep.residual) v += (pre && m == 0) ? (sg == 0 ? pre_r[0] : pre_r[1]) : __ldcg(ep.residual + o);
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
            // j == tid & 127: the pre-fetched pair belongs to this thread
            float av = red[m * NT + 2 * j] + (pre ? (sg == 0 ? pre_b0[0] : pre_b0[1]) : (bias ? to_f<T>(bias[c]) : 0.0f));
            const float gv = red[m * NT + 2 * j + 1] + (pre ? (sg == 0 ? pre_b1[0] : pre_b1[1]) : (bias ? to_f<T>(bias[c + 1]) : 0.0f));
            if (ep.act == TSB200_ACT_SWIGLU) av = av / (1.0f + expf(-av));
            float v = av * gv;
            const size_t o = (size_t)m * No + (c >> 1);
            if (ep.residual) v += __ldcg(ep.residual + o);
            if (ep.y32) ep.y32[o] = v;
            else reinterpret_cast<T*>(ep.y)[o] = from_f<T>(v);
          }
        }
      }
    }
    consumers_sync();  // red is reused by the next segment; the release below publishes the epilogue stores
    if (finish && xchg) {
      // one arrival per finished column tile on every rank's counter of this operation, signalled by one thread per
      // rank: system-scope fence (the stores above went to other GPUs' memory; the barrier makes the fence cumulative
      // over the CTA's stores), then a relaxed add on that rank's counter
      if (tid < a.c.tp_size) {
        __threadfence_system();
        red_relaxed_add_sys(reinterpret_cast<unsigned*>(a.c.peer[tid]) + op_i, 1u);
      }
    } else if (finish && tid == 0) {
      red_release_add(&a.done[op_i * kDoneStride], 1u);
    }
    if (u == u_end - 1 && (a.defer == 2 || (a.defer == 1 && whole))) release_held();
    seg_begin = u + 1;
    un = u + 1;
  }
}

// ------------------------------------------------------------------------------------------- the kernel
template <bool TP>
__global__ void __launch_bounds__(kStreamThreads, 1) decode_stack_mma_kernel(StackArgs a) {
  typedef __half T;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.stages;
  unsigned char* stage_mem = smem;                                  // [S][16 KB], 1024-byte aligned (swizzle atoms)
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
    if (lane == 0) stack_stream_tiles<__half>(a, stage_mem, full, empty, &s_err);
    return;
  }

  grid_dep_wait();  // the embedding rows, the cache length and last step's cache appends are visible from here on
  const StackConfig& c = a.c;
  const int M = c.M;
  const int T0 = __ldcg(c.dT);
  const int group = c.H / c.Hkv;
  const int AG = (group % 4 == 0) ? 4 : 1;
  const int yg = c.Hkv * (group / AG);
  const int splits = stack_splits((int)gridDim.x, M, yg, min(T0 + 1, c.Tmax));
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
  // tensor parallelism: counters that other ranks increment are monotonic; this launch is epoch `epoch`
  unsigned* xcnt = TP ? reinterpret_cast<unsigned*>(c.peer[c.tp_rank]) : nullptr;
  unsigned* epoch_ptr = TP ? reinterpret_cast<unsigned*>(c.peer[c.tp_rank] + kStackXchHeader - 4) : nullptr;
  const unsigned epoch = TP ? *reinterpret_cast<volatile unsigned*>(epoch_ptr) : 0u;
  int s = 0;
  unsigned round = 0;
  bool dead = false;
  unsigned prev_target = 0;
  bool prev_xchg = false;
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
      NormVecConsts<T> nc;
      const bool hoist = op->type == 0 && op->xmode != 0 && op->K <= 4096 && op->K % 4 == 0;
      if (hoist) norm_vec_consts<T>(nc, reinterpret_cast<const T*>(op->gamma), reinterpret_cast<const T*>(op->beta), op->K, tid);
      if (i > 0) {
        bool ok = true;
        if (tid == 0) {
          if (TP && prev_xchg)  // every rank's finishers arrive here: column tiles x ranks, per launch
            ok = poll_count_sys(xcnt + (i - 1), (epoch + 1u) * prev_target * (unsigned)c.tp_size, dead ? 64u : a.poll_limit, a.error_flag);
          else
            ok = poll_count(&a.done[(i - 1) * kDoneStride], prev_target, dead ? 64u : a.poll_limit, a.error_flag);
        }
        if (tid == 0 && !ok) {
          s_err = 1;
          *a.error_flag = 1;
        }
        consumers_sync();
        if (*(volatile int*)&s_err) dead = true;
      }
      STRACE(i, 0);
      if (op->type == 0) {
        mm_linear<TP>(a, op, i, g, stage_mem, xs, red, full, empty, s, round, &s_err, &s_last, s_stat, dead, hoist ? &nc : nullptr);
      } else if (AG == 4) {
        stack_attention<T, 4>(a, op, i, merge, &s_last, T0, splits, rcs, rsn);
      } else {
        stack_attention<T, 1>(a, op, i, merge, &s_last, T0, splits, rcs, rsn);
      }
      STRACE(i, 3);
    }
    prev_target = target;
    prev_xchg = TP && op->type == 0 && op->xsite >= 0;
  }
  // leave: the last CTA out clears the operation counters for the next launch
  if (tid == 0) {
    if (*(volatile int*)&s_err) *a.error_flag = 1;
    __threadfence();
    const unsigned prev = atomicAdd(&a.done[a.n_ops * kDoneStride], 1u);
    if (prev == gridDim.x - 1) {
      for (int i = 0; i <= a.n_ops; ++i) a.done[i * kDoneStride] = 0u;
      if (TP) *reinterpret_cast<volatile unsigned*>(epoch_ptr) = epoch + 1u;
    }
  }
}

// ------------------------------------------------------------------------------------------- host side
int init_stack_mma_attrs() {
  TSB_CUDA(cudaFuncSetAttribute(decode_stack_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  TSB_CUDA(cudaFuncSetAttribute(decode_stack_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  return 1;
}

int launch_decode_stack_mma(int device, DeviceState* st, const StackConfig& c, const StackOp* ops_dev, const StackOp* ops_host,
                            int n_ops, void* partials, void* counters, void* attn_part, int* error_flag,
                            long long* trace, bool pdl, cudaStream_t s) {
  if (c.dtype != TSB200_F16 || c.M > kMmaMaxRows) return 2;
  const int grid = st->sm_count;
  const StackPlan p = stack_plan(c, ops_host, n_ops, grid, 2);
  StackArgs a;
  const int r = stack_fill_args(a, p, c, ops_dev, ops_host, n_ops, partials, counters, attn_part, error_flag, trace);
  if (r != 1) return r;
  const size_t fixed = p.union_bytes + 32 * sizeof(uint64_t) + 1024 /* alignment slack */ + 128;
  const size_t budget = 225 * 1024;  // the kernel also has a few hundred bytes of static shared memory
  if (fixed + 3 * (size_t)kTileBytes > budget) return 2;
  int stages = (int)((budget - fixed) / kTileBytes);
  if (stages > 16) stages = 16;
  a.stages = stages;
  a.defer = 2;  // measured best: the ring slots of an operation's last tiles go back after its epilogue
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kStreamThreads);
  cfg.dynamicSmemBytes = fixed + (size_t)stages * kTileBytes;
  cfg.stream = s;
  {
    // The CTAs wait on one another, so all of them must be resident at the same time: one per SM with this much shared
    // memory.  If the device cannot hold the grid (fewer SMs available than it reports, a smaller carve-out), the caller
    // runs one launch per operation instead.
    int per_sm = 0;
    if (c.tp_size > 1) TSB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stack_mma_kernel<true>, kStreamThreads, cfg.dynamicSmemBytes));
    else TSB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stack_mma_kernel<false>, kStreamThreads, cfg.dynamicSmemBytes));
    if ((long long)per_sm * st->sm_count < grid) return 2;
  }
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  if (c.tp_size > 1) TSB_CUDA(cudaLaunchKernelEx(&cfg, decode_stack_mma_kernel<true>, a));
  else TSB_CUDA(cudaLaunchKernelEx(&cfg, decode_stack_mma_kernel<false>, a));
  count_launch(device);
  return 1;
}

}  // namespace tsb
