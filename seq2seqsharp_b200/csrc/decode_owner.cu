// Owner-partitioned persistent decode step, fp16, one GPU (see decode_owner.cuh for the partition and the weight layout).
//
// One CTA per SM, eight warps.  The CTA's private, contiguous weight stream runs through a ring of 32 KB stages filled by
// TMA bulk copies that the warps themselves issue (no producer warp); weights never wait for activations.  The warps
// follow the program: per layer an attention block and an FFN block, then the LM head.  A block starts with ONE grid-wide wait (the residual stream of the previous
// block is complete), stages the normed row into shared memory and runs its jobs; results that other CTAs need are
// added with 64-bit integer atomics (fixed point) into the group accumulator or into the next residual buffer.
//
// Residual stream: three buffers X[0..2] of int64 [rows, d], fixed point.  Block p reads X[p % 3], every CTA adds its
// contributions to X[(p+1) % 3] (one CTA per column slice also adds the old value and the bias), and clears its slice of
// X[(p+2) % 3].  Readers of a buffer have all arrived at the block's counter before anybody clears or refills it.
//
// Tensor parallelism (decode_owner_kernel<true>, one sequence): every rank runs this program on its share of the heads
// and of the FFN columns.  The sums of a block's last linear (out-projection, FFN down) are partial: the CTAs of a rank
// add them into a local buffer Y, meet at a local counter, and then every CTA adds ITS slice of Y into the next residual
// buffer of EVERY rank (64-bit integer atomics over NVLink: the same bits everywhere, whatever the order) and signals
// the block's counter on every rank; a block starts when its counter shows the arrivals of all CTAs of all ranks.
// Those counters are never reset (a rank may be a launch ahead): a launch counter kept on the device scales the
// targets, and it also rotates the roles of the three residual buffers from launch to launch so that the buffer a fast
// rank adds into first is the one the slower rank's previous launch left cleared.
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
  float* AP;                      // partial softmax states [rows][Hkv][grp][gmax][hd + 4]: max, sum, -, -, value[hd]
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
  int off_xs, off_red, off_merge, off_ys, off_hs, off_qs, off_gsum, off_qbias, off_qcol, off_bar, gsum_cols;
  long long* trace;               // -DTSB200_TRACE builds: [grid][2L + 1 blocks][16] %globaltimer stamps
  // tensor parallelism (decode_owner_kernel<true>)
  int tp_rank, tp_size;
  long long* Y[2];                // this rank's partial sums of a block's last linear [kOwnMaxRows, d], fixed point
  unsigned char* peer[kStackMaxRanks];   // every rank's exchange region as mapped here (own included)
  long long off_X, off_P;         // bytes from a region's base: residual buffers X[3]; block counters [2L] (never reset)
  unsigned* epoch;                // launches completed so far (this rank's own word)
};

#ifdef TSB200_TRACE
#define OTRACE(block, slot)                                                                                  \
  do {                                                                                                       \
    if (a.trace && threadIdx.x == 0) a.trace[((size_t)blockIdx.x * (2 * a.L + 1) + (block)) * 16 + (slot)] = gtimer(); \
  } while (0)
#else
#define OTRACE(block, slot) do { } while (0)
#endif

__device__ __forceinline__ long long own_fix(float v) { return __float2ll_rn(v * kOwnFix); }
__device__ __forceinline__ float own_unfix(long long v) { return __ll2float_rn(v) * kOwnUnfix; }
__device__ __forceinline__ void own_add(long long* p, long long v) {
  atomicAdd(reinterpret_cast<unsigned long long*>(p), static_cast<unsigned long long>(v));
}
__device__ __forceinline__ long long own_ldcg(const long long* p) { return __ldcg(p); }
// the same add into another GPU's memory (or this one's) at system scope
__device__ __forceinline__ void own_add_sys(long long* p, long long v) {
  asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void own_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ------------------------------------------------------------------------------------------- the weight ring (consumer side)
// Every warp reads its own 512-byte block of every 4 KB row, in order.  Waiting for tiles and handing them back is
// decoupled from the loads: before a burst of `cnt` blocks the warp makes sure the tiles that hold them have landed
// (need), then loads them with plain shared-memory loads whose addresses only advance (ptr / step), and after the
// matching mma instructions have consumed the registers it hands back every tile it has finished (release).  The loops
// that carry the loads contain no branches, so the compiler pipelines loads and mma instructions freely.
__device__ __forceinline__ bool own_wait_full(uint64_t* bar, unsigned par, bool dead) {
  if (dead) return true;   // a CTA that gave up does not wait any more
  return mbar_wait(bar, par, kSpinLimit);
}
// non-blocking look at a barrier phase
__device__ __forceinline__ bool mbar_test(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

struct OwnRing {
  unsigned char* base;         // stage memory
  const unsigned char* src;    // this CTA's stream in global memory
  uint64_t* full;              // per stage: the bytes of the tile have landed (one arrival + transaction bytes)
  uint64_t* empty;             // per stage: all eight warps have finished the tile (eight arrivals)
  int S, rows;                 // stages, rows of the ring (4 per stage)
  int n_tiles;                 // tiles of the CTA's stream
  int pos;                     // ring row of the next block
  int n;                       // rows consumed so far (this launch)
  int t_have, t_rel;           // tiles known to have landed / finished by this warp
  int w_slot, r_slot;
  int f_next, f_slot;          // the next tile this warp is responsible for refilling (tiles w, w + 8, ...) and its stage
  unsigned w_par, f_par;
  bool dead;
  volatile int* s_err;
  volatile int* s_code;        // which ring wait ran out (for the error message)
#ifdef TSB200_TRACE
  long long wait_cycles = 0, rel_cycles = 0;
  long long job_cycles[4] = {0, 0, 0, 0};   // K-split job: passes, wait before the reduction, reduction + emission, final refill
#endif
  __device__ __forceinline__ void issue(int slot, int tile) {
    mbar_expect_tx(&full[slot], kOwnTileBytes);
    bulk_g2s(base + (size_t)slot * kOwnTileBytes, src + (size_t)tile * kOwnTileBytes, kOwnTileBytes, &full[slot]);
  }
  // Hands back every tile this warp has finished (a fire-and-forget arrival).  There is no producer warp: tile t is
  // refilled (with tile t + S) by warp t % 8 once all eight warps have handed it back.  The warp only LOOKS at the
  // barrier (no wait): a tile that is not free yet is tried again at the warp's next hand-back, so no warp ever stalls
  // for a slower one.  `block`: wait (bounded) instead - used at the end of a job, before the warps go into a phase
  // without hand-backs.
  __device__ __forceinline__ void refill(int lane, bool block) {
    if (lane == 0 && !dead) {
#pragma unroll 1
      while (f_next < t_rel && f_next + S < n_tiles) {
        bool free_now = mbar_test(&empty[f_slot], f_par);
        if (!free_now && block) {
#pragma unroll 1
          for (unsigned q = 0; q < (kSpinLimit >> 10) && !free_now && !*s_err; ++q) free_now = mbar_wait(&empty[f_slot], f_par, 1024u);
          if (!free_now) {
            *s_err = 1;
            *s_code = 0x20000 | (f_next & 0xffff);   // a stage was not handed back by all warps
          }
        }
        if (!free_now) break;
        issue(f_slot, f_next + S);
        f_next += kConsumerWarps;
        f_slot += kConsumerWarps;
#pragma unroll 1
        while (f_slot >= S) {
          f_slot -= S;
          f_par ^= 1u;
        }
      }
    }
  }
  // makes sure the tiles that hold rows [n, n + cnt) have landed (never beyond the end of the stream).  A warp that
  // has to wait keeps looking after the stages it is responsible for refilling: the tile it waits for may be one of them.
  __device__ __forceinline__ void need(int cnt, int lane) {
    int t_need = (n + cnt + kOwnTileRows - 1) >> kOwnTileShift;
    if (t_need > n_tiles) t_need = n_tiles;
#pragma unroll 1
    while (t_have < t_need) {
#ifdef TSB200_TRACE
      const long long c0 = clock64();
#endif
      if (!dead && !mbar_test(&full[w_slot], w_par)) {
        bool ok = false;
#pragma unroll 1
        for (unsigned q = 0; q < (kSpinLimit >> 8) && !ok && !*s_err; ++q) {
          refill(lane, false);
          ok = mbar_wait(&full[w_slot], w_par, 256u);
        }
        if (!ok) {
          *s_err = 1;
          *s_code = 0x10000 | (t_have & 0xffff);   // a weight tile did not land
          dead = true;
        }
      }
#ifdef TSB200_TRACE
      wait_cycles += clock64() - c0;
#endif
      ++t_have;
      if (++w_slot == S) {
        w_slot = 0;
        w_par ^= 1u;
      }
    }
  }
  __device__ __forceinline__ const uint4* ptr(int w, int lane) const {
    return reinterpret_cast<const uint4*>(base + (size_t)pos * kOwnRowBytes + w * kOwnBlockBytes + lane * 16);
  }
  __device__ __forceinline__ void step() {
    pos = (pos + 1 == rows) ? 0 : pos + 1;
    ++n;
  }
  __device__ __forceinline__ void release(int w, int lane) {
    (void)w;
    const int t_done = n >> kOwnTileShift;
    if (t_rel < t_done) {
#ifdef TSB200_TRACE
      const long long c0 = clock64();
#endif
      __syncwarp();
#pragma unroll 1
      while (t_rel < t_done) {
        if (lane == 0) mbar_arrive(&empty[r_slot]);
        ++t_rel;
        if (++r_slot == S) r_slot = 0;
      }
      refill(lane, false);
#ifdef TSB200_TRACE
      __syncwarp();
      rel_cycles += clock64() - c0;
#endif
    }
  }
};

// ------------------------------------------------------------------------------------------- jobs (consumer side)
// K-split job: see OwnJob.  `xb` is the B operand (activations, fp16 [rows][xstride]) whose element 0 is the job's first k.
// emit(column of the job, row, sum) is called once per output by some thread after the eight warps' sums have met.
constexpr int kOwnRedCols = 256;   // columns the eight warps' sums can meet for at a time (16 strips)

// Where the finished sums of a job go.  The job loops are separate (not inlined) functions so that the kernel holds ONE
// copy of each: inlined at every use the kernel grew to 650 KB of code and ran out of the instruction cache, which
// slowed every phase of the program by a factor of two to three.
enum OwnEmitKind { OWN_EMIT_ADD64 = 0, OWN_EMIT_SMEM = 1, OWN_EMIT_LOGITS = 2 };
struct OwnEmit {
  int kind;
  long long* x64;       // ADD64: fixed-point accumulator, element [row * stride + cbase + column]
  float* f32;           // SMEM: f32[row * stride + column]; LOGITS: f32[row * stride + cbase + column] = sum + bias
  const __half* bias;
  int stride, cbase, limit;
};
__device__ __forceinline__ void own_emit(const OwnEmit& em, int col, int n, float v) {
  if (em.kind == OWN_EMIT_ADD64) {
    own_add(em.x64 + (size_t)n * em.stride + em.cbase + col, own_fix(v));
  } else if (em.kind == OWN_EMIT_SMEM) {
    em.f32[(size_t)n * em.stride + col] = v;
  } else {
    const int c = em.cbase + col;
    if (c < em.limit) em.f32[(size_t)n * em.stride + c] = v + __half2float(em.bias[c]);
  }
}

// The inner loops are instantiated for every burst width: with the width a compile-time constant they are straight-line
// code (no guards around the loads and the mma instructions), which is what lets eight warps eat the ring faster than
// HBM refills it (measured: the same loop with run-time guards ran at a third of the rate).
template <int WC>
__device__ __forceinline__ void own_ksplit_pass(float (&acc)[kOwnKChunk][4], OwnRing& R, const __half* xrow, bool row_live, int ksw, int ks,
                                                int w, int lane) {
  R.need(WC, lane);
#pragma unroll 1
  for (int kk = 0; kk < ksw; ++kk) {
    const int kst = w * ksw + kk;
    // every lane loads (dead lanes from a valid address), the values of dead lanes are replaced by zero: no divergent branch
    const bool blive = row_live && kst < ks;
    const int kc = kst < ks ? kst : 0;
    const uint32_t v0 = *reinterpret_cast<const uint32_t*>(xrow + kc * 16), v1 = *reinterpret_cast<const uint32_t*>(xrow + kc * 16 + 8);
    const uint32_t b0 = blive ? v0 : 0u, b1 = blive ? v1 : 0u;
    uint4 av[WC];
#pragma unroll
    for (int s = 0; s < WC; ++s) {
      av[s] = *R.ptr(w, lane);
      R.step();
    }
    R.need(WC, lane);   // tiles of the blocks to come: the barrier round trip overlaps the loads above and the mma below
#pragma unroll
    for (int s = 0; s < WC; ++s) own_mma(acc[s], av[s].x, av[s].y, av[s].z, av[s].w, b0, b1);
    R.release(w, lane);
  }
}

__device__ __noinline__ void own_job_ksplit(const OwnJob* jp, OwnRing* Rp, const __half* xb, int xstride, int M, float* red,
                                            const OwnEmit* emp) {
  const OwnJob& j = *jp;
  if (j.nrows == 0) return;
  OwnRing R = *Rp;        // the ring state lives in registers while the job runs
  const OwnEmit em = *emp;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;
  const bool row_live = g8 < M;
  const __half* xrow = xb + (size_t)(row_live ? g8 : 0) * xstride + 2 * t4;
  const int ws = j.ws, ksw = j.ksw, ks = j.ks, nchunks = j.nchunks;
  int held0 = 0, held = 0;   // strips [held0, held0 + held) wait in `red` for the reduction
#ifdef TSB200_TRACE
  long long tc0 = clock64();
  R.job_cycles[0] = R.job_cycles[1] = R.job_cycles[2] = R.job_cycles[3] = 0;
#endif
  for (int c = 0; c < nchunks; ++c) {
    const int wc = own_chunk_width(ws, nchunks, c);
    float acc[kOwnKChunk][4];
#pragma unroll
    for (int s = 0; s < kOwnKChunk; ++s)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[s][e] = 0.0f;
    switch (wc) {
      case 1: own_ksplit_pass<1>(acc, R, xrow, row_live, ksw, ks, w, lane); break;
      case 2: own_ksplit_pass<2>(acc, R, xrow, row_live, ksw, ks, w, lane); break;
      case 3: own_ksplit_pass<3>(acc, R, xrow, row_live, ksw, ks, w, lane); break;
      case 4: own_ksplit_pass<4>(acc, R, xrow, row_live, ksw, ks, w, lane); break;
      case 5: own_ksplit_pass<5>(acc, R, xrow, row_live, ksw, ks, w, lane); break;
      case 6: own_ksplit_pass<6>(acc, R, xrow, row_live, ksw, ks, w, lane); break;
      case 7: own_ksplit_pass<7>(acc, R, xrow, row_live, ksw, ks, w, lane); break;
      default: own_ksplit_pass<8>(acc, R, xrow, row_live, ksw, ks, w, lane); break;
    }
    // this warp's sums of the chunk go to red[warp][column][row]; the warps' sums meet when `red` is full or the job ends
#pragma unroll
    for (int s = 0; s < kOwnKChunk; ++s) {
      if (s < wc) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = 2 * t4 + (e & 1), col = (held + s) * 16 + g8 + ((e >> 1) << 3);
          if (n < M) red[(w * kOwnRedCols + col) * M + n] = acc[s][e];
        }
      }
    }
    held += wc;
    const bool last = c + 1 == nchunks;
    if (last || held + own_chunk_width(ws, nchunks, c + 1) > kOwnRedCols / 16) {
#ifdef TSB200_TRACE
      { const long long t = clock64(); R.job_cycles[0] += t - tc0; tc0 = t; }
#endif
      R.refill(lane, true);   // a warp that waits at the barrier cannot look after its stages: settle them first
      consumers_sync();
#ifdef TSB200_TRACE
      { const long long t = clock64(); R.job_cycles[1] += t - tc0; tc0 = t; }
#endif
#pragma unroll 1
      for (int idx = tid; idx < held * 16 * M; idx += 256) {
        const int n = idx % M, col = idx / M;
        float v = 0.0f;
#pragma unroll
        for (int ww = 0; ww < kConsumerWarps; ++ww) v += red[(ww * kOwnRedCols + col) * M + n];
        own_emit(em, held0 * 16 + col, n, v);
      }
      consumers_sync();
      held0 += held;
      held = 0;
#ifdef TSB200_TRACE
      { const long long t = clock64(); R.job_cycles[2] += t - tc0; tc0 = t; }
#endif
    }
  }
  R.refill(lane, true);
#ifdef TSB200_TRACE
  R.job_cycles[3] += clock64() - tc0;
#endif
  *Rp = R;
}

// strip-split job: a warp holds the complete sums of its strips; emit is called from the accumulator registers.
template <int SPW>
__device__ __forceinline__ void own_ssplit_pass(float (&acc)[kOwnMaxSpw][4], OwnRing& R, const __half* xrow, bool row_live, int ks, int w, int lane) {
  R.need(SPW, lane);
#pragma unroll 1
  for (int k = 0; k < ks; ++k) {
    const uint32_t v0 = *reinterpret_cast<const uint32_t*>(xrow + k * 16), v1 = *reinterpret_cast<const uint32_t*>(xrow + k * 16 + 8);
    const uint32_t b0 = row_live ? v0 : 0u, b1 = row_live ? v1 : 0u;
    uint4 av[SPW];
#pragma unroll
    for (int s = 0; s < SPW; ++s) {
      av[s] = *R.ptr(w, lane);
      R.step();
    }
    R.need(SPW, lane);
#pragma unroll
    for (int s = 0; s < SPW; ++s) own_mma(acc[s], av[s].x, av[s].y, av[s].z, av[s].w, b0, b1);
    R.release(w, lane);
  }
}

__device__ __noinline__ void own_job_ssplit(const OwnJob* jp, OwnRing* Rp, const __half* xb, int xstride, int M, float* red,
                                            const OwnEmit* emp) {
  const OwnJob& j = *jp;
  if (j.nrows == 0) return;
  OwnRing R = *Rp;
  const OwnEmit em = *emp;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;
  const bool row_live = g8 < M;
  const __half* xrow = xb + (size_t)(row_live ? g8 : 0) * xstride + 2 * t4;
  const int spw = j.spw, ks = j.ks, ws = j.ws, nchunks = j.nchunks;
  for (int c = 0; c < nchunks; ++c) {
    float acc[kOwnMaxSpw][4];
#pragma unroll
    for (int s = 0; s < kOwnMaxSpw; ++s)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[s][e] = 0.0f;
    switch (spw) {
      case 1: own_ssplit_pass<1>(acc, R, xrow, row_live, ks, w, lane); break;
      case 2: own_ssplit_pass<2>(acc, R, xrow, row_live, ks, w, lane); break;
      case 3: own_ssplit_pass<3>(acc, R, xrow, row_live, ks, w, lane); break;
      case 4: own_ssplit_pass<4>(acc, R, xrow, row_live, ks, w, lane); break;
      case 5: own_ssplit_pass<5>(acc, R, xrow, row_live, ks, w, lane); break;
      case 6: own_ssplit_pass<6>(acc, R, xrow, row_live, ks, w, lane); break;
      case 7: own_ssplit_pass<7>(acc, R, xrow, row_live, ks, w, lane); break;
      default: own_ssplit_pass<8>(acc, R, xrow, row_live, ks, w, lane); break;
    }
    // the warp's sums go through its own corner of shared memory so that all 32 lanes issue the atomic adds (for one
    // sequence only 8 lanes hold live sums) and the code stays small
    float* mine = red + (size_t)w * (kOwnMaxSpw * 16) * M;
    __syncwarp();
#pragma unroll
    for (int s = 0; s < kOwnMaxSpw; ++s) {
      if (s < spw) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = 2 * t4 + (e & 1), col = s * 16 + g8 + ((e >> 1) << 3);
          if (n < M) mine[col * M + n] = acc[s][e];
        }
      }
    }
    __syncwarp();
    const int strip0 = c * 8 * spw + w * spw;
    int live = ws - strip0;
    live = live < 0 ? 0 : (live > spw ? spw : live);
#pragma unroll 1
    for (int idx = lane; idx < live * 16 * M; idx += 32) {
      const int n = idx % M, col = idx / M;
      own_add(em.x64 + (size_t)n * em.stride + em.cbase + strip0 * 16 + col, own_fix(mine[idx]));
    }
  }
  R.refill(lane, true);
  *Rp = R;
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
__device__ __noinline__ void own_stage_norm(__half* xs, int xstride, const long long* X, const OwnNormConsts& nc, int xmode, float eps,
                                            int M, int d, int tid, float* s_stat) {
  const int lane = tid & 31, w = tid >> 5;
#pragma unroll 1
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
// `where` tells a failed wait apart in the engine's error message: (block of the program << 4) | 1 block counter,
// 2 / 3 first / second group counter of an attention block.
// `sys`: the counter is incremented by other GPUs too (system-scope acquire, wrap-safe comparison with a monotonic target).
__device__ __noinline__ void own_wait(const unsigned* p, unsigned target, const OwnArgs& a, volatile int* s_err, bool& dead, int tid,
                                      int where, bool sys = false) {
  if (tid == 0) {
    const unsigned limit = dead ? 1u : a.poll_limit;
    if (!(sys ? poll_count_sys(p, target, limit, a.error_flag) : poll_count(p, target, limit, a.error_flag))) {
      *s_err = 1;
      if (!dead) atomicCAS(a.error_flag + 1, 0, where);   // the first wait that ran out (a CTA that follows another's failure is `dead`)
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
// hd/8 lanes own one token per iteration (16-byte loads, two tokens in flight), each runs an online softmax, the lane
// groups' states are merged through shared memory and written as this CTA's partial state of (row, head).
// q (rotated, rounded to fp16, unscaled), the new k and the new v of the group come from shared memory (`qs`).
// The first batch of K/V rows (row 0) does not depend on q: it is fetched BEFORE the group's q|k|v sums are waited for
// (own_attn_prefetch) so that its HBM latency is off the dependency chain.
constexpr int kOwnTokensInFlight = 2;   // cached tokens a lane group has in flight (each inlined copy of the update is 7 KB of code)
struct OwnKvBatch {
  TileVec<__half> kv[kOwnTokensInFlight], vv[kOwnTokensInFlight];
};
struct OwnAttnGeom {
  int lpt, tpw, sub, li, nstates, t_beg, t_end, t_cached_end;
  bool has_new;
};
__device__ __forceinline__ OwnAttnGeom own_attn_geom(const OwnArgs& a, int i, int gsz, int T0, int lane) {
  OwnAttnGeom q;
  q.lpt = a.hd / 8;
  q.tpw = 32 / q.lpt;
  q.sub = lane / q.lpt;
  q.li = lane % q.lpt;
  q.nstates = kConsumerWarps * q.tpw;
  const int Tk = T0 + 1;
  const int per = (Tk + gsz - 1) / gsz;
  q.t_beg = min(Tk, i * per);
  q.t_end = min(Tk, q.t_beg + per);
  q.t_cached_end = min(q.t_end, T0);
  q.has_new = (q.t_beg <= T0) && (T0 < q.t_end);
  return q;
}
__device__ __forceinline__ void own_attn_load(OwnKvBatch& b, const OwnAttnGeom& q, const __half* Kb, const __half* Vb, int tb, int hd) {
#pragma unroll
  for (int u = 0; u < kOwnTokensInFlight; ++u) {
    const int t = tb + u * q.nstates + q.sub;
    const size_t o = (size_t)(t < q.t_cached_end ? t : q.t_beg) * hd;  // dead lanes re-read a valid row
    b.kv[u].lds(Kb + o);
    b.vv[u].lds(Vb + o);
  }
}
__device__ __forceinline__ void own_attn_prefetch(OwnKvBatch& b, const OwnArgs& a, const OwnLayerDev& Lr, const OwnAttnGeom& q, int g, int w) {
  const size_t head_off = ((size_t)0 * a.Hkv + g) * a.Tmax * a.hd + q.li * 8;
  const int tb = q.t_beg + w * q.tpw;
  if (tb < q.t_cached_end) own_attn_load(b, q, Lr.cK + head_off, Lr.cV + head_off, tb, a.hd);
}
template <int GH>
__device__ __noinline__ void own_attention(const OwnArgs& a, const OwnLayerDev& Lr, const OwnAttnGeom& q, OwnKvBatch& first, int g, int i,
                                           const float* qs, float* merge, int tid, int p) {
  (void)p;
  constexpr int EPL = 8;
  const int hd = a.hd, grp = a.grp, Hkv = a.Hkv, Tmax = a.Tmax;
  const int lane = tid & 31, w = tid >> 5;
  const int rec = hd + 4;
#pragma unroll 1
  for (int m = 0; m < a.M; ++m) {
    const float* qrow = qs + (size_t)m * a.qstride;
    const size_t head_off = ((size_t)m * Hkv + g) * Tmax * hd + q.li * EPL;
    const __half* Kb = Lr.cK + head_off;
    const __half* Vb = Lr.cV + head_off;
#pragma unroll 1
    for (int h0 = 0; h0 < grp; h0 += GH) {
      float qf[GH][EPL];
#pragma unroll
      for (int gg = 0; gg < GH; ++gg)
#pragma unroll
        for (int e = 0; e < EPL; ++e) qf[gg][e] = qrow[(h0 + gg) * hd + q.li * EPL + e] * a.scale;
      float mx[GH], l[GH], acc[GH][EPL];
#pragma unroll
      for (int gg = 0; gg < GH; ++gg) {
        mx[gg] = -INFINITY;
        l[gg] = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[gg][e] = 0.0f;
      }
      // One copy of the update code: the loop runs over this lane group's cached tokens (two loads in flight: the token
      // being used and the next one) and, on warp 0, once more for the token of this step, which comes from shared memory.
      const int tb0 = q.t_beg + w * q.tpw;
      const int n_c = q.t_cached_end > tb0 ? (q.t_cached_end - tb0 + q.nstates - 1) / q.nstates : 0;
      const int n_it = n_c + ((q.has_new && w == 0) ? 1 : 0);
      TileVec<__half> kc, vc, kn, vn;
      if (m == 0) {   // fetched ahead of the wait
        kc = first.kv[0]; vc = first.vv[0]; kn = first.kv[1]; vn = first.vv[1];
      } else if (n_c > 0) {
        OwnKvBatch b2;
        own_attn_load(b2, q, Kb, Vb, tb0, hd);
        kc = b2.kv[0]; vc = b2.vv[0]; kn = b2.kv[1]; vn = b2.vv[1];
      }
#pragma unroll 1
      for (int it = 0; it < n_it; ++it) {
        float kf[EPL], vf[EPL];
        bool live;
        if (it < n_c) {
          kc.get(kf);
          vc.get(vf);
          live = tb0 + it * q.nstates + q.sub < q.t_cached_end;
          kc = kn;
          vc = vn;
          if (it + 2 < n_c) {
            const int t = tb0 + (it + 2) * q.nstates + q.sub;
            const size_t o = (size_t)(t < q.t_cached_end ? t : q.t_beg) * hd;  // dead lanes re-read a valid row
            kn.lds(Kb + o);
            vn.lds(Vb + o);
          }
        } else {
#pragma unroll
          for (int e = 0; e < EPL; ++e) {
            kf[e] = qrow[grp * hd + q.li * EPL + e];
            vf[e] = qrow[(grp + 1) * hd + q.li * EPL + e];
          }
          live = q.sub == 0;
        }
        attn_update<GH, EPL>(qf, kf, vf, mx, l, acc, q.lpt, live);
      }
      if (m == 0 && h0 == 0) OTRACE(p, 10);
      const int st = w * q.tpw + q.sub;
      const int srec = hd + 2;   // records of the shared-memory merge area
#pragma unroll
      for (int gg = 0; gg < GH; ++gg) {
        float* r = merge + ((size_t)st * GH + gg) * srec;
        if (q.li == 0) {
          r[0] = mx[gg];
          r[1] = l[gg];
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) r[2 + q.li * EPL + e] = acc[gg][e];
      }
      consumers_sync();
#pragma unroll 1
      for (int idx = tid; idx < GH * hd; idx += 256) {
        const int gg = idx / hd, e = idx % hd;
        float mm = -INFINITY;
#pragma unroll 1
        for (int u = 0; u < q.nstates; ++u) mm = fmaxf(mm, merge[((size_t)u * GH + gg) * srec]);
        float Ls = 0.0f, As = 0.0f;
#pragma unroll 2
        for (int u = 0; u < q.nstates; ++u) {
          const float* r = merge + ((size_t)u * GH + gg) * srec;
          const float cc = (r[0] == -INFINITY) ? 0.0f : __expf(r[0] - mm);
          Ls += r[1] * cc;
          As += r[2 + e] * cc;
        }
        float* pr = a.AP + ((((size_t)m * Hkv + g) * grp + h0 + gg) * a.gmax + i) * rec;
        if (e == 0) {
          pr[0] = mm;
          pr[1] = Ls;
        }
        pr[4 + e] = As;
      }
      consumers_sync();  // the merge area is free again
      if (m == 0 && h0 == 0) OTRACE(p, 11);
    }
  }
}

// ---- short ranges: when a CTA's share of the cache is at most kOwnShortTokens tokens (contexts of up to about
// kOwnShortTokens x CTAs per group tokens) the lane-group scheme above spends its time merging 16-32 partial states.
// Instead the CTA's K and V rows are copied to shared memory with cp.async (row 0 before the group's q|k|v sums are
// awaited, so the HBM latency is off the dependency chain), scores are computed by 8 lanes per (head, token), one warp
// per head forms the softmax statistics, and every thread accumulates two output dimensions: three barriers, no merge.
constexpr int kOwnShortTokens = 48;
__device__ __forceinline__ void own_cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void own_cp_async_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// copies the cached rows [t_beg, t_cached_end) of (row m, KV head g) to Ks / Vs (rows of hd + 8 halves)
__device__ __forceinline__ void own_short_stage(const OwnArgs& a, const OwnLayerDev& Lr, const OwnAttnGeom& q, int g, int m, __half* Ks,
                                                __half* Vs, int tid) {
  const int hd = a.hd, v8 = hd / 8, n_c = q.t_cached_end - q.t_beg, rs = hd + 8;
  const size_t base = (((size_t)m * a.Hkv + g) * a.Tmax + q.t_beg) * hd;
#pragma unroll 1
  for (int idx = tid; idx < n_c * v8; idx += 256) {
    const int t = idx / v8, c = idx % v8;
    own_cp_async16(Ks + (size_t)t * rs + c * 8, Lr.cK + base + (size_t)t * hd + c * 8);
    own_cp_async16(Vs + (size_t)t * rs + c * 8, Lr.cV + base + (size_t)t * hd + c * 8);
  }
}
__device__ __noinline__ void own_attention_short(const OwnArgs& a, const OwnLayerDev& Lr, const OwnAttnGeom& q, int g, int i, const float* qs,
                                                 float* region, int tid) {
  const int hd = a.hd, grp = a.grp, rs = hd + 8, NTP = kOwnShortTokens + 1;
  __half* Ks = reinterpret_cast<__half*>(region);
  __half* Vs = Ks + (size_t)NTP * rs;
  float* Ss = reinterpret_cast<float*>(Vs + (size_t)NTP * rs);   // [grp][NTP] scores, then exp(score - max)
  float* stat = Ss + (size_t)grp * NTP;                            // [grp][2] max, sum
  const int lane = tid & 31, w = tid >> 5;
  const int n_c = q.t_cached_end - q.t_beg;
  const int n_tot = n_c + (q.has_new ? 1 : 0);
  const int rec = hd + 4;
#pragma unroll 1
  for (int m = 0; m < a.M; ++m) {
    const float* qrow = qs + (size_t)m * a.qstride;
    if (m > 0) {
      consumers_sync();   // the previous row's K/V are no longer read
      own_short_stage(a, Lr, q, g, m, Ks, Vs, tid);
    }
    if (q.has_new) {   // the token of this step joins as the last row
#pragma unroll 1
      for (int e = tid; e < hd; e += 256) {
        Ks[(size_t)n_c * rs + e] = __float2half_rn(qrow[grp * hd + e]);
        Vs[(size_t)n_c * rs + e] = __float2half_rn(qrow[(grp + 1) * hd + e]);
      }
    }
    own_cp_async_wait();
    consumers_sync();
    // scores: eight lanes per (head, token) pair, hd / 8 dimensions each
    {
      const int dpl = hd / 8, l8 = tid & 7;
#pragma unroll 1
      const int npair = grp * n_tot;
      for (int p0 = (tid >> 5) * 4; p0 < npair; p0 += 32) {   // warp-uniform trip count: the shuffles below need every lane
        const int pi = p0 + ((tid >> 3) & 3);
        const bool pon = pi < npair;
        const int h = pon ? pi / n_tot : 0, t = pon ? pi % n_tot : 0;
        const float* qh = qrow + h * hd + l8 * dpl;
        const __half* kr = Ks + (size_t)t * rs + l8 * dpl;
        float dsum = 0.0f;
#pragma unroll 1
        for (int c = 0; c < dpl; c += 8) {
          const uint4 raw = *reinterpret_cast<const uint4*>(kr + c);
          const float4 qa4 = *reinterpret_cast<const float4*>(qh + c), qb4 = *reinterpret_cast<const float4*>(qh + c + 4);
          const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
          const float2 k0 = __half22float2(h2[0]), k1 = __half22float2(h2[1]), k2 = __half22float2(h2[2]), k3 = __half22float2(h2[3]);
          dsum += (qa4.x * k0.x + qa4.y * k0.y) + (qa4.z * k1.x + qa4.w * k1.y) + (qb4.x * k2.x + qb4.y * k2.y) + (qb4.z * k3.x + qb4.w * k3.y);
        }
        dsum += __shfl_xor_sync(0xffffffffu, dsum, 4);
        dsum += __shfl_xor_sync(0xffffffffu, dsum, 2);
        dsum += __shfl_xor_sync(0xffffffffu, dsum, 1);
        if (l8 == 0 && pon) Ss[h * NTP + t] = dsum * a.scale;
      }
    }
    consumers_sync();
    // softmax statistics: one warp per head
#pragma unroll 1
    for (int h = w; h < grp; h += kConsumerWarps) {
      float mx = -INFINITY;
      for (int t = lane; t < n_tot; t += 32) mx = fmaxf(mx, Ss[h * NTP + t]);
      mx = warp_max(mx);
      float l = 0.0f;
      for (int t = lane; t < n_tot; t += 32) {
        const float pv = __expf(Ss[h * NTP + t] - mx);
        Ss[h * NTP + t] = pv;
        l += pv;
      }
      l = warp_sum(l);
      if (lane == 0) {
        stat[2 * h] = mx;
        stat[2 * h + 1] = l;
      }
    }
    consumers_sync();
    // values: two output dimensions per thread
#pragma unroll 1
    for (int o = 2 * tid; o < grp * hd; o += 512) {
      const int h = o / hd, e = o % hd;
      float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 4
      for (int t = 0; t < n_tot; ++t) {
        const float pv = Ss[h * NTP + t];
        const float2 vf = __half22float2(*reinterpret_cast<const __half2*>(Vs + (size_t)t * rs + e));
        a0 += pv * vf.x;
        a1 += pv * vf.y;
      }
      float* pr = a.AP + ((((size_t)m * a.Hkv + g) * grp + h) * a.gmax + i) * rec;
      if (e == 0) {
        pr[0] = n_tot > 0 ? stat[2 * h] : -INFINITY;
        pr[1] = n_tot > 0 ? stat[2 * h + 1] : 0.0f;
      }
      pr[4 + e] = a0;
      pr[4 + e + 1] = a1;
    }
  }
}

// Combines the group's partial softmax states (records [max, sum, -, -, value[hd]] per split) for four consecutive output
// elements, taking every `step`-th split from `first` on.  Eight splits are read at a time with 8- and 16-byte loads that
// do not depend on each other (one memory round trip per batch) and folded into a running (max, sum, value).
__device__ __forceinline__ void own_merge_splits(const float* base, int rec, int e4, int gsz, int first, int step, float& mm, float& Ls,
                                                 float (&As)[4]) {
  mm = -INFINITY;
  Ls = 0.0f;
  As[0] = As[1] = As[2] = As[3] = 0.0f;
#pragma unroll 1
  for (int s0 = first; s0 < gsz; s0 += 8 * step) {
    float2 ml[8];
    float4 av[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int sc = s0 + u * step < gsz ? s0 + u * step : first;   // clamped: every address is valid
      ml[u] = __ldcg(reinterpret_cast<const float2*>(base + (size_t)sc * rec));
      av[u] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)sc * rec + 4 + e4));
    }
    float bm = mm;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (s0 + u * step < gsz) bm = fmaxf(bm, ml[u].x);
    const float c0 = (mm == -INFINITY) ? 0.0f : __expf(mm - bm);
    Ls *= c0;
    As[0] *= c0; As[1] *= c0; As[2] *= c0; As[3] *= c0;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (s0 + u * step < gsz) {
        const float cc = (ml[u].x == -INFINITY) ? 0.0f : __expf(ml[u].x - bm);
        Ls += ml[u].y * cc;
        As[0] += av[u].x * cc; As[1] += av[u].y * cc; As[2] += av[u].z * cc; As[3] += av[u].w * cc;
      }
    mm = bm;
  }
}

// ------------------------------------------------------------------------------------------- the kernel
constexpr int kOwnThreads = kConsumerWarps * 32;   // eight consumer warps; the ring is refilled by the consumers themselves

template <bool TP>
__global__ void __launch_bounds__(kOwnThreads, 1) decode_owner_kernel(OwnArgs a) {
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
  float* s_qbias = reinterpret_cast<float*>(un + a.off_qbias);   // q|k|v biases of the group, this layer
  int* s_qcol = reinterpret_cast<int*>(un + a.off_qcol);         // group-local q|k|v column -> column of the packed matrix
  uint64_t* full = reinterpret_cast<uint64_t*>(un + a.off_bar);
  uint64_t* empty = full + 16;
  __shared__ int s_err, s_last, s_code;
  __shared__ float s_stat[64];
  __shared__ OwnJob s_jobs[5];
  __shared__ float2 s_rope[128];   // cos / sin of this step's position (head sizes up to 256)

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  OwnRing R;
  R.base = stage_mem;
  R.src = a.wstream + (size_t)a.cta_row0[cta] * kOwnRowBytes;
  R.full = full;
  R.empty = empty;
  R.S = S;
  R.rows = kOwnTileRows * S;
  R.n_tiles = a.cta_tiles[cta];
  R.pos = 0;
  R.n = 0;
  R.t_have = 0;
  R.t_rel = 0;
  R.w_slot = 0;
  R.r_slot = 0;
  R.w_par = 0u;
  R.f_next = w;
  R.f_slot = w % S;
  R.f_par = (unsigned)((w / S) & 1);
  R.dead = false;
  R.s_err = &s_err;
  R.s_code = &s_code;
  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kConsumerWarps);
    }
    s_err = 0;
    s_last = 0;
    s_code = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // weights never depend on earlier kernels: fill the ring at once
    for (int i = 0; i < S && i < R.n_tiles; ++i) R.issue(i, i);
  }
  {
    const int words = 5 * (int)(sizeof(OwnJob) / 4);
    const int* src = reinterpret_cast<const int*>(a.jobs + (size_t)cta * 5);
    int* dst = reinterpret_cast<int*>(s_jobs);
    for (int i = tid; i < words; i += kOwnThreads) dst[i] = src[i];
  }
  __syncthreads();

  grid_dep_wait();  // the residual row of this step, the cache length and last step's cache appends are visible
  const int M = a.M, d = a.d, hd = a.hd, grp = a.grp, Hkv = a.Hkv;
  const int T0 = min(__ldcg(a.dT), a.Tmax - 1);
  if (a.use_rope && tid < a.hd / 2) s_rope[tid] = a.rope_tab[(size_t)T0 * (a.hd / 2) + tid];   // visible after the first barrier below
  const OwnJob& jq = s_jobs[OWN_QKV];
  const int g = jq.group;
  const int gb = own_group_begin(g, G, Hkv), gsz = own_group_begin(g + 1, G, Hkv) - gb, gi = cta - gb;
  const int QW = (grp + 2) * hd;
  // CTAs of the group that take part in attention: about 32 tokens each, so that short contexts are not cut into
  // slivers whose partial states cost more to merge than the tokens cost to read
  int asz = (T0 + 1 + 31) / 32;
  asz = asz > gsz ? gsz : asz;
  const bool attn_on = gi < asz;
  for (int jc = tid; jc < QW; jc += 256) s_qcol[jc] = own_qkv_col(jc, g, grp, hd, a.H, Hkv);   // visible after the first barrier below
  const int c0 = own_split(d, G, cta), c1 = own_split(d, G, cta + 1);   // this CTA's slice of the residual columns
  // [2L] block counters: one GPU: local, cleared at the end of the launch; tensor parallel: in the exchange region,
  // incremented by every rank, never reset (the local [2L] then count this rank's CTAs whose partial sums are in Y)
  unsigned* cntP = TP ? reinterpret_cast<unsigned*>(a.peer[a.tp_rank] + a.off_P) : a.cnt;
  unsigned* cntL = a.cnt;
  unsigned* cntG = a.cnt + (size_t)2 * a.L * kOwnCntStride;             // [L][Hkv][2] group counters
  unsigned* cntExit = cntG + (size_t)a.L * Hkv * 2 * kOwnCntStride;
  bool dead = false;
  const unsigned epoch = TP ? *reinterpret_cast<volatile unsigned*>(a.epoch) : 0u;
  const unsigned ptarget = TP ? (epoch + 1u) * (unsigned)G * (unsigned)a.tp_size : (unsigned)G;
  // the residual buffer block 0 reads: a launch leaves X[(xb + 2L + 1) % 3] cleared, which must be the buffer block 0 of
  // the next launch adds into
  const int xb = TP ? (int)((epoch % 3u) * (unsigned)((2 * a.L) % 3) % 3u) : 0;

  // duties of a block: add the old residual value and the bias of the block's last linear to the CTA's slice of the
  // next buffer, clear the slice of the buffer after that
  // duties of a block: add the old residual value and the bias of the block's last linear to the CTA's slice of the
  // next buffer, clear the slice of the buffer after that.  Split in three so that the loads overlap other work: the bias
  // before the block's wait, the old value right after it (the norm staging's loads follow at once), the adds after the staging.
  const int wdt = c1 - c0;
  auto duty_bias = [&](const __half* bias) -> long long {
    return (bias && tid < M * wdt) ? own_fix(__half2float(bias[c0 + tid % wdt])) : 0;
  };
  auto duty_load = [&](const long long* Xc) -> long long {
    return (tid < M * wdt) ? own_ldcg(Xc + (size_t)(tid / wdt) * d + c0 + tid % wdt) : 0;
  };
  // Tensor parallel: the old value goes into this rank's own next buffer, the bias (held by rank 0 only) into the
  // partial sums that every rank receives; the slice of the partial buffer of the NEXT block is cleared as well.
  auto duty_commit = [&](const long long* Xc, long long* Xn, long long* Xz, const __half* bias, long long v0, long long vb, int p) {
    long long* Yc = TP ? a.Y[p & 1] : nullptr;
    long long* Yz = TP ? a.Y[(p + 1) & 1] : nullptr;
    if (tid < M * wdt) {
      const size_t o = (size_t)(tid / wdt) * d + c0 + tid % wdt;
      if (TP) {
        own_add(Xn + o, v0);
        if (vb != 0) own_add(Yc + o, vb);
        Yz[o] = 0;
      } else {
        own_add(Xn + o, v0 + vb);
      }
      Xz[o] = 0;
    }
#pragma unroll 1
    for (int idx = tid + 256; idx < M * wdt; idx += 256) {   // slices wider than one element per thread (few CTAs)
      const int m = idx / wdt, col = c0 + idx % wdt;
      const size_t o = (size_t)m * d + col;
      long long v = own_ldcg(Xc + o);
      const long long b = bias ? own_fix(__half2float(bias[col])) : 0;
      if (TP) {
        own_add(Xn + o, v);
        if (b != 0) own_add(Yc + o, b);
        Yz[o] = 0;
      } else {
        own_add(Xn + o, v + b);
      }
      Xz[o] = 0;
    }
  };
  // Tensor parallel, end of a block: this CTA's partial sums are in Y; when all CTAs of the rank have said so, the CTA
  // adds its slice of Y into the next residual buffer of every rank and signals the block's counter there.  The
  // release of the signalling threads covers the adds of all threads (they met at the barrier before it).
  auto block_done = [&](int p, int xn) {
    if (!TP) {
      own_arrive(cntP + (size_t)p * kOwnCntStride, tid);
      return;
    }
    own_arrive(cntL + (size_t)p * kOwnCntStride, tid);
    own_wait(cntL + (size_t)p * kOwnCntStride, (unsigned)G, a, &s_err, dead, tid, (p << 4) | 4);
    OTRACE(p, 15);
    const long long* Yc = a.Y[p & 1];
    const int nv = M * wdt;
#pragma unroll 1
    for (int idx = tid; idx < nv * a.tp_size; idx += 256) {
      const int r = idx / nv, e = idx % nv;
      const size_t o = (size_t)(e / wdt) * d + c0 + e % wdt;
      const long long v = own_ldcg(Yc + o);
      long long* dst = reinterpret_cast<long long*>(a.peer[r] + a.off_X) + (size_t)xn * kOwnMaxRows * d + o;
      if (v != 0) own_add_sys(dst, v);
    }
    consumers_sync();
    if (tid < a.tp_size) red_release_add_sys(reinterpret_cast<unsigned*>(a.peer[tid] + a.off_P) + (size_t)p * kOwnCntStride, 1u);
    OTRACE(p, 11);
  };

  for (int layer = 0; layer < a.L; ++layer) {
    const OwnLayerDev& Lr = a.layers[layer];
    // =================================================================== attention block
    {
      const int p = 2 * layer;
      const long long* Xc = a.X[(xb + p) % 3];
      long long* Xn = a.X[(xb + p + 1) % 3];
      long long* Xz = a.X[(xb + p + 2) % 3];
      long long* qa = a.QA[layer & 1] + (size_t)g * kOwnMaxRows * QW;
      long long* qz = a.QA[(layer + 1) & 1] + (size_t)g * kOwnMaxRows * QW;
      OwnNormConsts nc;
      own_norm_consts(nc, Lr.g1, Lr.b1n, d, tid);
      // this CTA's share of the cached K/V rows is asked into L2 now: by the time attention reads it, HBM has answered
      {
        const OwnAttnGeom pg = own_attn_geom(a, gi, asz, T0, lane);
        const int lines = attn_on ? (pg.t_cached_end - pg.t_beg) * hd * 2 / 128 : 0;   // 128-byte lines of one row's K (and V) share
#pragma unroll 1
        for (int idx = tid; idx < M * lines; idx += 256) {
          const size_t o = (((size_t)(idx / lines) * Hkv + g) * a.Tmax + pg.t_beg) * hd + (size_t)(idx % lines) * 64;
          prefetch_l2(Lr.cK + o);
          prefetch_l2(Lr.cV + o);
        }
      }
      // constants of the block that can be fetched before its input exists: the q|k|v biases of the group (to shared
      // memory) and the bias of the CTA's residual slice
#pragma unroll 1
      for (int jc = tid; jc < QW; jc += 256) s_qbias[jc] = __half2float(Lr.bqkv[s_qcol[jc]]);
      const long long dbias = duty_bias(Lr.bo);
      if (p > 0) own_wait(cntP + (size_t)(p - 1) * kOwnCntStride, ptarget, a, &s_err, dead, tid, (p << 4) | 1, TP);
      OTRACE(p, 0);
      R.dead = R.dead || dead;
      const long long dval = duty_load(Xc);
      own_stage_norm(xs, a.xstride, Xc, nc, a.xmode, a.eps, M, d, tid, s_stat);
      duty_commit(Xc, Xn, Xz, Lr.bo, dval, dbias, p);
      {
        // clear this CTA's part of the group accumulator the NEXT layer uses
        const int n = kOwnMaxRows * QW, z0 = own_split(n, gsz, gi), z1 = own_split(n, gsz, gi + 1);
#pragma unroll 1
        for (int idx = z0 + tid; idx < z1; idx += 256) qz[idx] = 0;
      }
      consumers_sync();
      OTRACE(p, 1);
      // q|k|v of the group: this CTA's range of K, sums meet in the group accumulator
      {
        const OwnEmit em{OWN_EMIT_ADD64, qa, nullptr, nullptr, QW, 0, 0};
        own_job_ssplit(&jq, &R, xs + jq.kbase, a.xstride, M, red, &em);
      }
      unsigned* gc = cntG + ((size_t)(layer * Hkv + g) * 2) * kOwnCntStride;
      OTRACE(p, 2);
      own_arrive(gc, tid);
      // the cached K/V rows do not depend on q: their loads fly while the group's sums are awaited
      const OwnAttnGeom ag = own_attn_geom(a, gi, asz, T0, lane);
      const bool short_range = (T0 + 1 + asz - 1) / asz <= kOwnShortTokens && hd % 64 == 0;   // the same for every CTA of the group
      OwnKvBatch kv0;
      if (!attn_on) {
        // more CTAs than the context can feed: this one takes no tokens
      } else if (short_range) {
        __half* Ks = reinterpret_cast<__half*>(merge);
        own_short_stage(a, Lr, ag, g, 0, Ks, Ks + (size_t)(kOwnShortTokens + 1) * (hd + 8), tid);
      } else {
        own_attn_prefetch(kv0, a, Lr, ag, g, w);
      }
      own_wait(gc, (unsigned)gsz, a, &s_err, dead, tid, (p << 4) | 2);
      OTRACE(p, 3);
      // bias, rounding to fp16 (the model's activation type)
#pragma unroll 1
      for (int idx = tid; idx < M * QW; idx += 256) {
        const int jc = idx < QW ? idx : idx % QW;
        const float v = own_unfix(own_ldcg(qa + idx)) + s_qbias[jc];
        qs[idx] = __half2float(__float2half_rn(v));   // rows of qs are QW apart, like the accumulator's
      }
      consumers_sync();
      OTRACE(p, 8);
      if (a.use_rope) {   // cos / sin of this step's position were staged in shared memory at the start of the kernel
        const int npair = (grp + 1) * hd / 2;   // q heads and k
#pragma unroll 1
        for (int idx = tid; idx < M * npair; idx += 256) {
          const int m = idx / npair, pr = idx % npair;
          const float2 cs = s_rope[pr % (hd / 2)];
          float* q2 = qs + (size_t)m * a.qstride + 2 * pr;
          const float x0 = q2[0], x1 = q2[1];
          q2[0] = __half2float(__float2half_rn(x0 * cs.x - x1 * cs.y));
          q2[1] = __half2float(__float2half_rn(x1 * cs.x + x0 * cs.y));
        }
        consumers_sync();
      }
      if (gi == 0) {  // the first CTA of the group appends the new k and v rows to the cache
#pragma unroll 1
        for (int idx = tid; idx < M * hd; idx += 256) {
          const int m = idx / hd, e = idx % hd;
          const size_t o = (((size_t)m * Hkv + g) * a.Tmax + T0) * hd + e;
          Lr.cK[o] = __float2half_rn(qs[(size_t)m * a.qstride + grp * hd + e]);
          Lr.cV[o] = __float2half_rn(qs[(size_t)m * a.qstride + (grp + 1) * hd + e]);
        }
      }
      OTRACE(p, 9);
      if (!attn_on) {
      } else if (short_range) own_attention_short(a, Lr, ag, g, gi, qs, merge, tid);
      else if (grp % 4 == 0) own_attention<4>(a, Lr, ag, kv0, g, gi, qs, merge, tid, p);
      else own_attention<1>(a, Lr, ag, kv0, g, gi, qs, merge, tid, p);
      OTRACE(p, 4);
      own_arrive(gc + kOwnCntStride, tid);
      own_wait(gc + kOwnCntStride, (unsigned)gsz, a, &s_err, dead, tid, (p << 4) | 3);
      OTRACE(p, 5);
      // merge the group's partial states: attention output of the group's heads, fp16, in shared memory.  A thread owns
      // four consecutive outputs; the two halves of the CTA take every other split and meet in shared memory.
      {
        const int rec = hd + 4, nq = grp * hd / 4;
        const int half = tid >> 7, ql = tid & 127;
#pragma unroll 1
        for (int m = 0; m < M; ++m) {
#pragma unroll 1
          for (int q0 = 0; q0 < nq; q0 += 128) {
            const int qd = q0 + ql;
            const bool on = qd < nq;
            const int qc = on ? qd : 0;
            const int head = (qc * 4) / hd, e4 = (qc * 4) % hd;
            const float* base = a.AP + ((((size_t)m * Hkv + g) * grp + head) * a.gmax) * rec;
            float mm, Ls, As[4];
            own_merge_splits(base, rec, e4, asz, half, 2, mm, Ls, As);
            float* mine = red + (size_t)ql * 6;
            if (half == 1) {
              mine[0] = mm; mine[1] = Ls; mine[2] = As[0]; mine[3] = As[1]; mine[4] = As[2]; mine[5] = As[3];
            }
            consumers_sync();
            if (half == 0 && on) {
              const float m2 = mine[0];
              const float bm = fmaxf(mm, m2);
              const float ca = (mm == -INFINITY) ? 0.0f : __expf(mm - bm), cb = (m2 == -INFINITY) ? 0.0f : __expf(m2 - bm);
              const float L = Ls * ca + mine[1] * cb;
              float o[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) o[e] = L > 0.0f ? (As[e] * ca + mine[2 + e] * cb) / L : 0.0f;
              St4<__half>::st(ys + (size_t)m * a.ystride + qc * 4, o);
            }
            consumers_sync();
          }
        }
      }
      consumers_sync();
      OTRACE(p, 6);
      // the group's rows of W0, this CTA's range of output columns
      const OwnJob& jo = s_jobs[OWN_W0];
      R.dead = R.dead || dead;
#ifdef TSB200_TRACE
      const long long w0_wait0 = R.wait_cycles, w0_rel0 = R.rel_cycles;
      if (a.trace && tid == 0) {
        // how many of the tiles the job is about to read have landed already
        int landed = 0, sl = R.w_slot;
        unsigned par = R.w_par;
        for (int i = 0; i < S && R.t_have + i < R.n_tiles; ++i) {
          if (!mbar_test(&full[sl], par)) break;
          ++landed;
          if (++sl == S) { sl = 0; par ^= 1u; }
        }
        a.trace[((size_t)blockIdx.x * (2 * a.L + 1) + p) * 16 + 15] = landed * 1000 + S * 10 + (R.t_have - (R.n >> kOwnTileShift));
      }
#endif
      {
        const OwnEmit em{OWN_EMIT_ADD64, TP ? a.Y[p & 1] : Xn, nullptr, nullptr, d, jo.cbase, 0};
        own_job_ksplit(&jo, &R, ys, a.ystride, M, red, &em);
      }
#ifdef TSB200_TRACE
      if (a.trace && tid == 0) {
        long long* tr = a.trace + ((size_t)blockIdx.x * (2 * a.L + 1) + p) * 16;
        tr[12] = R.job_cycles[0];            // cycles in the passes of the W0 job (warp 0)
        tr[13] = R.wait_cycles - w0_wait0;   // of which waiting for tiles
        tr[14] = R.rel_cycles - w0_rel0;     // and in hand-back + refill
      }
#endif
      OTRACE(p, 7);
      block_done(p, (xb + p + 1) % 3);
    }
    // =================================================================== FFN block
    {
      const int p = 2 * layer + 1;
      const long long* Xc = a.X[(xb + p) % 3];
      long long* Xn = a.X[(xb + p + 1) % 3];
      long long* Xz = a.X[(xb + p + 2) % 3];
      OwnNormConsts nc;
      own_norm_consts(nc, Lr.g2, Lr.b2n, d, tid);
      const long long dbias = duty_bias(Lr.bdown);
      own_wait(cntP + (size_t)(p - 1) * kOwnCntStride, ptarget, a, &s_err, dead, tid, (p << 4) | 1, TP);
      OTRACE(p, 0);
      R.dead = R.dead || dead;
      const long long dval = duty_load(Xc);
      own_stage_norm(xs, a.xstride, Xc, nc, a.xmode, a.eps, M, d, tid, s_stat);
      duty_commit(Xc, Xn, Xz, Lr.bdown, dval, dbias, p);
      const OwnJob& ju = s_jobs[OWN_UP];
      const OwnJob& jd = s_jobs[OWN_DOWN];
#pragma unroll 1
      for (int idx = tid; idx < M * a.hstride; idx += 256) hs[idx] = __float2half_rn(0.0f);
      consumers_sync();
      OTRACE(p, 1);
#ifdef TSB200_TRACE
      const long long wc0 = R.wait_cycles, rc0 = R.rel_cycles, cc0 = clock64();
#endif
      {
        const OwnEmit em{OWN_EMIT_SMEM, nullptr, gsum, nullptr, a.gsum_cols, 0, 0};
        own_job_ksplit(&ju, &R, xs, a.xstride, M, red, &em);
      }
#ifdef TSB200_TRACE
      if (a.trace && tid == 0) {
        a.trace[((size_t)blockIdx.x * (2 * a.L + 1) + p) * 16 + 12] = R.wait_cycles - wc0;   // cycles warp 0 waited for tiles
        a.trace[((size_t)blockIdx.x * (2 * a.L + 1) + p) * 16 + 13] = clock64() - cc0;        // cycles of the whole job
        a.trace[((size_t)blockIdx.x * (2 * a.L + 1) + p) * 16 + 14] = R.rel_cycles - rc0;   // cycles in release (hand-back + refill)
      }
#endif
      consumers_sync();
      OTRACE(p, 2);
      // bias, activation, gate: this CTA's hidden units, fp16, in shared memory
      if (a.glu) {
        const int nh = ju.ws * 8;
#pragma unroll 1
        for (int idx = tid; idx < M * nh; idx += 256) {
          const int m = idx / nh, jl = idx % nh;
          float av = gsum[(size_t)m * a.gsum_cols + 2 * jl] + __half2float(Lr.bup[ju.cbase + 2 * jl]);
          const float gv = gsum[(size_t)m * a.gsum_cols + 2 * jl + 1] + __half2float(Lr.bup[ju.cbase + 2 * jl + 1]);
          if (a.act == TSB200_ACT_SWIGLU) av = av / (1.0f + expf(-av));
          hs[(size_t)m * a.hstride + jl] = __float2half_rn(av * gv);
        }
      } else {
        const int nh = ju.ws * 16;
#pragma unroll 1
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
      OTRACE(p, 3);
      // the matching rows of W2: all d output columns, sums go straight into the next residual buffer
      {
        const OwnEmit em{OWN_EMIT_ADD64, TP ? a.Y[p & 1] : Xn, nullptr, nullptr, d, 0, 0};
        own_job_ssplit(&jd, &R, hs, a.hstride, M, red, &em);
      }
      OTRACE(p, 7);
      block_done(p, (xb + p + 1) % 3);
    }
  }
  // =================================================================== LM head
  {
    const int p = 2 * a.L;
    const long long* Xc = a.X[(xb + p) % 3];
    OwnNormConsts nc;
    own_norm_consts(nc, a.gF, a.bF, d, tid);
    grid_dep_launch();  // the sampling kernels may become resident while the LM head streams
    own_wait(cntP + (size_t)(p - 1) * kOwnCntStride, ptarget, a, &s_err, dead, tid, (p << 4) | 1, TP);
    OTRACE(p, 0);
    R.dead = R.dead || dead;
    own_stage_norm(xs, a.xstride, Xc, nc, a.xmode, a.eps, M, d, tid, s_stat);
    consumers_sync();
    OTRACE(p, 1);
    const OwnJob& jh = s_jobs[OWN_HEAD];
    {
      const OwnEmit em{OWN_EMIT_LOGITS, nullptr, a.logits, a.head_b, a.V, jh.cbase, a.V};
      own_job_ksplit(&jh, &R, xs, a.xstride, M, red, &em);
    }
    OTRACE(p, 7);
  }
  // a CTA that gave up did not wait for its tiles: let the copies in flight land (bounded) before the CTA leaves
  if (R.dead || dead) {
    for (int i = 0; i < S; ++i) mbar_wait(&full[i], 0u, 1u << 16), mbar_wait(&full[i], 1u, 1u << 16);
  }
  // leave: the last CTA out clears the counters for the next launch
  consumers_sync();
  if (tid == 0) {
    if (*(volatile int*)&s_err) {
      if (*(volatile int*)&s_code) atomicCAS(a.error_flag + 1, 0, *(volatile int*)&s_code);
      *a.error_flag = 1;
    }
    __threadfence();
    const unsigned prev = atomicAdd(cntExit, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
  }
  consumers_sync();
  if (s_last) {
    const int n = 2 * a.L + a.L * Hkv * 2 + 1;
    for (int i = tid; i < n; i += 256) a.cnt[(size_t)i * kOwnCntStride] = 0u;   // the local counters
    if (TP && tid == 0) *reinterpret_cast<volatile unsigned*>(a.epoch) = epoch + 1u;
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
// Tensor parallel form: other ranks add into this rank's residual buffers, also before this kernel runs (a rank may be
// a launch ahead), so only the buffer block 0 READS is written here; the rotation of the buffers' roles (see the kernel)
// makes the one block 0 adds into the buffer the previous launch left cleared.  Y0 and QA0 are local.
__global__ void own_init_tp_kernel(long long* X, long long* Y0, long long* QA0, const float* x, const unsigned* epoch, int L, int M, int d,
                                   int qa_words) {
  pdl_trigger();
  pdl_wait();
  const unsigned ep = *epoch;
  const int xb = (int)((ep % 3u) * (unsigned)((2 * L) % 3) % 3u);
  long long* X0 = X + (size_t)xb * kOwnMaxRows * d;
  const int n = kOwnMaxRows * d;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    X0[i] = (i < M * d) ? own_fix(x[i]) : 0;
    Y0[i] = 0;
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
  unsigned* cnt = nullptr;    // local counters, then (one sector further) the launch counter of the tensor-parallel form
  size_t cnt_bytes = 0;
  long long* Y = nullptr;     // 2 buffers (tensor parallel only)
  bool packed = false;
  bool tp_failed = false;     // a tensor-parallel step failed: the ranks' counters and buffers no longer agree
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
  void* ptrs[] = {m->wstream, m->d_row0, m->d_tiles, m->d_jobs, m->d_layers, m->X, m->QA, m->AP, m->cnt, m->Y};
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
    const long long tiles = (rows + kOwnTileRows - 1) / kOwnTileRows;
    m->cta_row0[c] = row;
    m->cta_tiles[c] = (int)tiles;
    row += tiles * kOwnTileRows;
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
                  alloc((void**)&m->AP, (size_t)kOwnMaxRows * D.Hkv * grp * m->gmax * (D.hd + 4) * sizeof(float), true) &&
                  alloc((void**)&m->cnt, m->cnt_bytes + kOwnCntStride * sizeof(unsigned), true) &&
                  alloc((void**)&m->Y, (size_t)2 * kOwnMaxRows * D.d * sizeof(long long), true);
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
    const long long pad = (long long)m->cta_tiles[c] * kOwnTileRows - rows;
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
  if (m && m->cnt) cudaMemset(m->cnt, 0, m->cnt_bytes);   // not the launch counter behind them
  return 1;
}
// Bytes of the part of a tensor-parallel engine's exchange region that this kernel uses: [2L block counters][X[3]].
static size_t own_xch_counters_bytes(int L) { return ((size_t)2 * L * kOwnCntStride * sizeof(unsigned) + 255) / 256 * 256; }
long long owner_xch_bytes(const OwnDims& D) {
  return (long long)(own_xch_counters_bytes(D.L) + (size_t)3 * kOwnMaxRows * D.d * sizeof(long long));
}
void owner_tp_failed(OwnerModel* m) {
  if (m) m->tp_failed = true;
}
long long owner_stream_bytes(const OwnerModel* m) { return m ? m->total_rows * (long long)kOwnRowBytes : 0; }

// One decode step for M rows whose embedded fp32 rows are in `x`.  Returns 1 ok, 0 error, 2 not applicable (the caller
// takes another path).
int owner_launch(OwnerModel* m, DeviceState* st, int M, const float* x, float* logits, const float2* rope_tab, const int* dT,
                 int* error_flag, unsigned poll_limit, bool pdl, long long* trace, const OwnTp* tp, cudaStream_t s) {
  if (!m || !m->packed || M < 1 || M > kOwnMaxRows || !error_flag || !dT) return 2;
  const bool is_tp = tp && tp->size > 1;
  if (is_tp) {
    if (M != 1 || tp->size > kStackMaxRanks) return 2;
    TSB_CHECK(!m->tp_failed, "an earlier step of this tensor-parallel engine failed: the ranks no longer agree on the state of the "
                             "exchange; close the job on every rank and build it again");
  }
  const OwnDims& D = m->D;
  const int grp = D.H / D.Hkv, QW = (grp + 2) * D.hd;
  OwnArgs a{};
  a.wstream = m->wstream; a.cta_row0 = m->d_row0; a.cta_tiles = m->d_tiles; a.jobs = m->d_jobs; a.layers = m->d_layers;
  a.gF = (const __half*)m->nf_g; a.bF = m->norm_type == 0 ? (const __half*)m->nf_b : nullptr; a.head_b = (const __half*)m->head_b;
  a.logits = logits;
  long long* Xbase = m->X;
  if (is_tp) {
    a.tp_rank = tp->rank; a.tp_size = tp->size;
    for (int r = 0; r < tp->size; ++r) a.peer[r] = tp->peer[r] + tp->offset;
    a.off_P = 0;
    a.off_X = (long long)own_xch_counters_bytes(D.L);
    a.epoch = m->cnt + m->cnt_bytes / sizeof(unsigned);
    for (int i = 0; i < 2; ++i) a.Y[i] = m->Y + (size_t)i * kOwnMaxRows * D.d;
    Xbase = reinterpret_cast<long long*>(a.peer[tp->rank] + a.off_X);
  }
  for (int i = 0; i < 3; ++i) a.X[i] = Xbase + (size_t)i * kOwnMaxRows * D.d;
  for (int i = 0; i < 2; ++i) a.QA[i] = m->QA + (size_t)i * D.Hkv * kOwnMaxRows * QW;
  a.AP = m->AP; a.cnt = m->cnt; a.rope_tab = rope_tab; a.dT = dT; a.error_flag = error_flag;
  a.poll_limit = poll_limit ? poll_limit : kPollLimit;
  a.trace = trace;
  a.L = D.L; a.M = M; a.d = D.d; a.H = D.H; a.Hkv = D.Hkv; a.hd = D.hd; a.grp = grp; a.F = D.F; a.V = D.V; a.Tmax = m->Tmax;
  a.glu = D.glu; a.act = m->act; a.xmode = m->norm_type == 0 ? 2 : 1; a.use_rope = m->use_rope; a.gmax = m->gmax;
  a.eps = m->eps; a.scale = 1.0f / sqrtf((float)D.hd);
  if (a.use_rope && !rope_tab) return 2;
  // shared memory behind the ring: {xs | red} aliased by the attention merge area, then ys, hs, qs, gsum, barriers
  auto up = [](size_t v, size_t al) { return (v + al - 1) / al * al; };
  a.xstride = D.d + 8; a.ystride = grp * D.hd + 8; a.hstride = m->hid_max + 8; a.qstride = QW;
  const size_t xs_b = up((size_t)M * a.xstride * 2, 128);
  const size_t red_b = up((size_t)kConsumerWarps * kOwnRedCols * M * 4, 128);
  const int lpt = D.hd / 8, tpw = 32 / lpt, GH = (grp % 4 == 0) ? 4 : 1;
  size_t merge_b = up((size_t)kConsumerWarps * tpw * GH * (D.hd + 2) * 4, 128);
  {
    const size_t short_b = up((size_t)2 * (kOwnShortTokens + 1) * (D.hd + 8) * 2 + (size_t)grp * (kOwnShortTokens + 1) * 4 + (size_t)grp * 8, 128);
    if (short_b > merge_b) merge_b = short_b;
  }
  size_t off = 0;
  a.off_xs = 0; a.off_red = (int)xs_b; a.off_merge = 0;
  off = xs_b + red_b > merge_b ? xs_b + red_b : merge_b;
  a.off_ys = (int)off; off += up((size_t)M * a.ystride * 2, 128);
  a.off_hs = (int)off; off += up((size_t)M * a.hstride * 2, 128);
  a.off_qs = (int)off; off += up((size_t)M * a.qstride * 4, 128);
  a.gsum_cols = m->up_cols_max;
  a.off_gsum = (int)off; off += up((size_t)M * a.gsum_cols * 4, 128);
  a.off_qbias = (int)off; off += up((size_t)QW * 4, 128);
  a.off_qcol = (int)off; off += up((size_t)QW * 4, 128);
  a.off_bar = (int)off; off += 32 * sizeof(uint64_t);
  const size_t fixed = off + 1024 /* alignment slack */ + 128;
  const size_t budget = 224 * 1024;  // the kernel also has about 2 KB of static shared memory
  if (fixed + 4 * (size_t)kOwnTileBytes > budget) return 2;   // a burst plus the look-ahead for the next one spans up to four tiles
  int stages = (int)((budget - fixed) / kOwnTileBytes);
  if (stages > 16) stages = 16;
  a.stages = stages;
  const size_t smem = fixed + (size_t)stages * kOwnTileBytes;
  {
    // the CTAs wait on one another: the whole grid must be resident at once
    int per_sm = 0;
    if (is_tp) TSB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_owner_kernel<true>, kOwnThreads, smem));
    else TSB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_owner_kernel<false>, kOwnThreads, smem));
    if ((long long)per_sm * st->sm_count < m->G) return 2;
  }
  {
    const int qa_words = D.Hkv * kOwnMaxRows * QW;
    if (is_tp) TSB_CUDA(launch_k(own_init_tp_kernel, dim3(16), dim3(256), 0, s, Xbase, a.Y[0], a.QA[0], x, (const unsigned*)a.epoch, D.L, M, D.d, qa_words));
    else TSB_CUDA(launch_k(own_init_kernel, dim3(16), dim3(256), 0, s, a.X[0], a.X[1], a.X[2], a.QA[0], x, M, D.d, qa_words));
    count_launch(m->device);
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(m->G);
  cfg.blockDim = dim3(kOwnThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  if (is_tp) TSB_CUDA(cudaLaunchKernelEx(&cfg, decode_owner_kernel<true>, a));
  else TSB_CUDA(cudaLaunchKernelEx(&cfg, decode_owner_kernel<false>, a));
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
      int held0 = 0, held = 0;
      for (int c = 0; c < j.nchunks; ++c) {
        const int wc = own_chunk_width(j.ws, j.nchunks, c);
        TSB_CHECK(wc >= 1 && wc <= kOwnKChunk, "owner layout: chunk width %d", wc);
        for (int kk = 0; kk < j.ksw; ++kk) {
          const int kst = w * j.ksw + kk;
          for (int s = 0; s < kOwnKChunk; ++s) {
            if (s >= wc) continue;
            int kstep, strip;
            bool live;
            own_block_coords(j, row, w, kstep, strip, live);
            // the consumer files the sums of this block under column strip held0 + held + s of the job
            TSB_CHECK(kstep == kst && strip == held0 + held + s && live == (kst < j.ks),
                      "owner layout: K-split job kind %d: row %d warp %d holds (k-step %d, strip %d) but the consumer expects (%d, %d)",
                      j.kind, row, w, kstep, strip, kst, held0 + held + s);
            if (live) seen[(size_t)kstep * j.ws + strip] += 1;
            ++row;
          }
        }
        held += wc;
        if (c + 1 == j.nchunks || held + own_chunk_width(j.ws, j.nchunks, c + 1) > 16) {
          held0 += held;
          held = 0;
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
    TSB_CHECK((long long)m.cta_tiles[c] * kOwnTileRows >= rows && (long long)m.cta_tiles[c] * kOwnTileRows < rows + kOwnTileRows,
              "owner layout: CTA %d: tile count", c);
    expect_row += (long long)m.cta_tiles[c] * kOwnTileRows;
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
  TSB_CUDA(cudaFuncSetAttribute(decode_owner_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
  TSB_CUDA(cudaFuncSetAttribute(decode_owner_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
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
