// Linear layer for decode batches of 5..64 rows on packed fp16 weights: y[M,N] = epilogue(x[M,K] * W[K,N]).
//
// At these row counts the product is still bound by streaming the weights once (HBM), but there are too many rows
// for FMA pipes and too few output tiles for a tile-per-CTA tensor-core GEMM (its split-K variants spend most of their
// time in pipeline fill, drain and partial-sum hand-over).  So this kernel keeps the structure of the streaming GEMV:
//   * persistent CTAs, one per SM, each owning a contiguous, evenly sized range of the packed 16 KB weight tiles
//     (stream-K over column-tile-major order);
//   * a producer lane feeds a shared-memory ring: per stage one linear bulk copy of a weight tile (stored as its
//     128-byte-swizzled shared-memory image) and one TMA tensor copy of the matching activation tile [rows][32 k]
//     (64-byte swizzle, rows beyond M zero-filled);
//   * eight consumer warps, 32 columns each: ldmatrix.trans of the weight fragments, ldmatrix of the activation
//     fragments, mma.sync m16n8k16 with fp32 accumulators for up to 8 row blocks;
//   * at the end of a CTA's share of a column tile the accumulators go to a scratch slot; the CTA that delivers the
//     last share adds the slots in fixed order (bitwise reproducible) and applies bias / activation / gate / residual.
// Every mbarrier wait is bounded; on timeout the error word is raised and the CTA drains and returns.
//
// Replaces cublasGemmEx + bias / activation kernels for decode batches (TensorSharp.CUDA/MatrixMul/CudaMatrixMulMM.cs:305-362).
#include <cuda.h>

#include <cstdlib>

#include "kernels.cuh"
#include "stream_common.cuh"

namespace tsb {

constexpr int kGsXBytes = 4096;                       // activation tile per stage: up to 64 rows x 32 k halves
constexpr int kGsStageBytes = kTileBytes + kGsXBytes;

// Raised by a kernel whose bounded wait ran out; read and cleared by gs_take_error().
__device__ int g_gs_error;

struct GsArgs {
  const unsigned char* Wp;
  int M, K, N, KB, CT;
  int stages, max_contrib;
  int prefetch;             // 1: the first ring-full of weight tiles is requested before the wait on the previous kernel
  // KQ > 0 instantiations: the rows come from the fp32 residual stream and are normed here (no activation tiles by TMA)
  const float* xres;        // [M][K]
  const __half* gamma;
  const __half* beta;       // may be null
  int norm_type;            // 0 LayerNorm, 1 RMSNorm
  float eps;
  int rope_on;              // 1: the epilogue rotates q / k and appends k / v to the cache (see RopeFuse)
  RopeFuse rope;
  float* partials;          // [CT][max_contrib][M][256]
  unsigned int* counters;   // [CT], zero on entry, self-resetting
  int* error_flag;
  Epilogue ep;
};

__device__ __forceinline__ void gs_tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void gs_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void gs_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void gs_mma_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned gs_atom_add_acq_rel(unsigned* p, unsigned v) {
  unsigned old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void gs_consumers_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ float gs_act(float v, int act) {
  switch (act) {
    case TSB200_ACT_RELU: return v < 0.0f ? 0.0f : v;
    case TSB200_ACT_SILU: return v / (1.0f + expf(-v));
    case TSB200_ACT_LEAKYRELU: return v < 0.0f ? 0.01f * v : v;
    case TSB200_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    default: return v;
  }
}

// KQ == 0: activation rows arrive as TMA tiles beside every weight tile.  KQ > 0 (NB == 1, K == KQ * 1024, M * KQ <= 16): the
// rows are read from the fp32 residual stream, normed by the consumer warps (LayerNorm / RMSNorm, the arithmetic of
// norm_kernel) and kept in shared memory as fp16 for the whole kernel - the norm launch in front of the linear disappears and
// a stage is the weight tile alone.
template <int NB, int KQ = 0>  // row blocks of 8: M <= 8 * NB
__global__ void __launch_bounds__(kStreamThreads, 1) gemm_stream_mma_kernel(const __grid_constant__ CUtensorMap mapX, GsArgs a) {
  constexpr int NT = 256;
  constexpr bool NORM = KQ > 0;
  constexpr int STAGE = NORM ? kTileBytes : kGsStageBytes;
  constexpr int XROW = KQ * 1024 * 2 + 16;   // bytes per normed row: 16 bytes of padding keep the ldmatrix row reads conflict-free
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)S * STAGE);
  uint64_t* empty = full + 16;
  unsigned char* xs = reinterpret_cast<unsigned char*>(empty + 16);   // NORM: [8][XROW]
  __shared__ int s_err, s_last;
  __shared__ float s_red[8][16];

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int M = a.M, N = a.N, KB = a.KB;
  const long long U = (long long)KB * a.CT, G = gridDim.x;  // the host launches at most U CTAs: no range is empty
  const int u_begin = (int)(U * blockIdx.x / G), u_end = (int)(U * (blockIdx.x + 1) / G);

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
  grid_dep_launch();

  if (w == kConsumerWarps) {
    if (lane == 0) {
      const unsigned char* src = a.Wp + (size_t)u_begin * kTileBytes;
      int s = 0, kb = u_begin % KB;
      unsigned round = 0;
      long long issued = 0;
      // The weights do not depend on the previous kernel: the first ring-full of tiles is requested before the wait on it,
      // so the stream starts while that kernel's last CTAs still reduce and store (and while a norm kernel in between runs).
      constexpr unsigned TX = NORM ? kTileBytes : kTileBytes + NB * 8 * 64;
      const int n_pre = (a.prefetch || NORM) ? min(S, u_end - u_begin) : 0;
      for (int i = 0; i < n_pre; ++i) {
        mbar_expect_tx(&full[i], TX);
        bulk_g2s(smem + (size_t)i * STAGE, src + (size_t)i * kTileBytes, kTileBytes, &full[i]);
      }
      if (!NORM) grid_dep_wait();  // the activation rows come from the previous kernel (read through TMA)
      for (int u = u_begin; u < u_end; ++u) {
        if (round > 0 && !mbar_wait(&empty[s], (round - 1u) & 1u)) {
          s_err = 1;
          break;
        }
        if (*(volatile int*)&s_err) break;
        unsigned char* dst = smem + (size_t)s * STAGE;
        if (u - u_begin >= n_pre) {
          mbar_expect_tx(&full[s], TX);
          bulk_g2s(dst, src, kTileBytes, &full[s]);
        }
        if (!NORM) gs_tma_load_2d(dst + kTileBytes, &mapX, kb * kKT, 0, &full[s]);  // x = kb * 32 halves: a 64-byte multiple
        src += kTileBytes;
        ++issued;
        if (++kb == KB) kb = 0;
        if (++s == S) {
          s = 0;
          ++round;
        }
      }
      if (*(volatile int*)&s_err) {
        // stages whose weight tile was requested ahead still lack their activation tile: request it (any k block), so
        // that every copy into this CTA's shared memory has landed before the CTA returns
        for (long long j = issued; j < n_pre; ++j) {
          if (!NORM) gs_tma_load_2d(smem + (size_t)j * STAGE + kTileBytes, &mapX, 0, 0, &full[(int)j]);
          ++issued;
        }
        const long long first = issued > S ? issued - S : 0;
        for (long long j = first; j < issued; ++j) mbar_wait(&full[(int)(j % S)], (unsigned)((j / S) & 1));
        g_gs_error = 1;
        if (a.error_flag) *a.error_flag = 1;
      }
    }
    return;
  }
  grid_dep_wait();  // consumers touch the scratch slots, counters and the residual rows of earlier kernels

  if constexpr (NORM) {
    // ---- norm of the M rows: thread t holds float4 t, t + 256, ... of every row (one round of loads), two block reductions
    constexpr int R = 16 / KQ < 8 ? 16 / KQ : 8;   // rows a thread can hold
    constexpr int K = KQ * 1024;
    const int M_ = a.M;
    float4 v[R][KQ];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < KQ; ++j)
        v[r][j] = r < M_ ? __ldcg(reinterpret_cast<const float4*>(a.xres + (size_t)r * K) + tid + 256 * j) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    auto reduce_rows = [&](float* part) {   // part[R] per thread -> totals over the 256 consumer threads, in every thread
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part[r] += __shfl_xor_sync(0xffffffffu, part[r], o);
      gs_consumers_sync();
      if (lane == 0)
#pragma unroll
        for (int r = 0; r < R; ++r) s_red[w][r] = part[r];
      gs_consumers_sync();
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float t = 0.0f;
#pragma unroll
        for (int q = 0; q < 8; ++q) t += s_red[q][r];
        part[r] = t;
      }
    };
    float sum[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      sum[r] = 0.0f;
#pragma unroll
      for (int j = 0; j < KQ; ++j)
        sum[r] += a.norm_type == 0 ? (v[r][j].x + v[r][j].y) + (v[r][j].z + v[r][j].w)
                                   : (v[r][j].x * v[r][j].x + v[r][j].y * v[r][j].y) + (v[r][j].z * v[r][j].z + v[r][j].w * v[r][j].w);
    }
    reduce_rows(sum);
    float shift[R], inv[R];
    if (a.norm_type == 0) {
      float sq[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        shift[r] = sum[r] / K;
        sq[r] = 0.0f;
#pragma unroll
        for (int j = 0; j < KQ; ++j) {
          const float e0 = v[r][j].x - shift[r], e1 = v[r][j].y - shift[r], e2 = v[r][j].z - shift[r], e3 = v[r][j].w - shift[r];
          sq[r] += (e0 * e0 + e1 * e1) + (e2 * e2 + e3 * e3);
        }
      }
      reduce_rows(sq);
#pragma unroll
      for (int r = 0; r < R; ++r) inv[r] = sqrtf(a.eps + sq[r] / K);
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        shift[r] = 0.0f;
        inv[r] = sqrtf(sum[r] / (float)K + a.eps);
      }
    }
#pragma unroll
    for (int j = 0; j < KQ; ++j) {
      const int c4 = tid + 256 * j;   // float4 index inside a row
      const __half2 g01 = reinterpret_cast<const __half2*>(a.gamma)[2 * c4], g23 = reinterpret_cast<const __half2*>(a.gamma)[2 * c4 + 1];
      __half2 b01 = __floats2half2_rn(0.0f, 0.0f), b23 = b01;
      if (a.beta) {
        b01 = reinterpret_cast<const __half2*>(a.beta)[2 * c4];
        b23 = reinterpret_cast<const __half2*>(a.beta)[2 * c4 + 1];
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        uint2 out = make_uint2(0u, 0u);   // rows beyond M are zero rows of the 8-row operand
        if (r < R && r < M_) {
          const int rr = r < R ? r : 0;
          float t0 = __low2float(g01) * ((v[rr][j].x - shift[rr]) / inv[rr]), t1 = __high2float(g01) * ((v[rr][j].y - shift[rr]) / inv[rr]);
          float t2 = __low2float(g23) * ((v[rr][j].z - shift[rr]) / inv[rr]), t3 = __high2float(g23) * ((v[rr][j].w - shift[rr]) / inv[rr]);
          if (a.beta) {
            t0 += __low2float(b01); t1 += __high2float(b01);
            t2 += __low2float(b23); t3 += __high2float(b23);
          }
          const __half2 h01 = __floats2half2_rn(t0, t1), h23 = __floats2half2_rn(t2, t3);
          out.x = *reinterpret_cast<const uint32_t*>(&h01);
          out.y = *reinterpret_cast<const uint32_t*>(&h23);
        }
        *reinterpret_cast<uint2*>(xs + (size_t)r * XROW + (size_t)c4 * 8) = out;
      }
    }
    gs_consumers_sync();
  }

  // ---------------- consumer warps: warp w owns columns [w*32, w*32+32) of every tile
  const int chunk = w >> 1, hf = w & 1;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int lrow = (lane & 7) + ((lane >> 4) << 3);   // weight fragments: k row inside a 16-k block
  const int lunit = (lane >> 3) & 1;                  //                   which 8-column unit of a 16-column block
  const int xr = lane & 7, xc = lane >> 3;            // activation fragments: row inside an 8-row block, 16-byte k chunk
  float d[2][NB][4];
#pragma unroll
  for (int cb = 0; cb < 2; ++cb)
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) d[cb][nb][e] = 0.0f;

  const int max_contrib = a.max_contrib;
  const Epilogue ep = a.ep;
  const __half* bias = reinterpret_cast<const __half*>(ep.bias);
  int s = 0;
  unsigned round = 0;
  bool dead = false;
  int ct = u_begin / KB, kb = u_begin % KB;
  for (int u = u_begin; u < u_end; ++u) {
    if (*(volatile int*)&s_err) dead = true;
    if (!mbar_wait(&full[s], round & 1u, dead ? 4096u : kSpinLimit)) {
      s_err = 1;
      dead = true;
    }
    const uint32_t wbase = smem_u32(smem + (size_t)s * STAGE) + chunk * 4096;
    uint32_t bf[NB][4];
    if constexpr (NORM) {
      // the normed rows stay in place: row xr, the four 16-byte chunks of k tile kb
      gs_ldmatrix_x4(smem_u32(xs) + xr * XROW + kb * 64 + (xc << 4), bf[0][0], bf[0][1], bf[0][2], bf[0][3]);
    } else {
      const uint32_t xbase = smem_u32(smem + (size_t)s * STAGE + kTileBytes);
      // activation fragments of all row blocks: [rows][32 k] with 64-byte rows, 16-byte chunks XOR-ed with (row / 2) & 3
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const int n = nb * 8 + xr;
        gs_ldmatrix_x4(xbase + n * 64 + ((xc ^ ((n >> 1) & 3)) << 4), bf[nb][0], bf[nb][1], bf[nb][2], bf[nb][3]);
      }
    }
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      const int k = kk * 16 + lrow;
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
        const int unit = hf * 4 + cb * 2 + lunit;
        uint32_t a0, a1, a2, a3;
        gs_ldmatrix_x4_trans(wbase + k * 128 + ((unit ^ (k & 7)) << 4), a0, a1, a2, a3);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) gs_mma_16816(d[cb][nb], a0, a1, a2, a3, bf[nb][2 * kk], bf[nb][2 * kk + 1]);
      }
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
    if (!seg_end) continue;
    // ---- end of this CTA's share of column tile cur_ct: accumulators -> scratch slot, last arriver finishes the tile
    const long long ct_first_u = (long long)cur_ct * KB, ct_last_u = ct_first_u + KB - 1;
    const int c_first = (int)(((ct_first_u + 1) * G + U - 1) / U - 1);
    const int c_last = (int)(((ct_last_u + 1) * G + U - 1) / U - 1);
    const int n_contrib = c_last - c_first + 1;
    const int slot = blockIdx.x - c_first;
    float* mine = a.partials + (((size_t)cur_ct * max_contrib + slot) * M) * NT;
#pragma unroll
    for (int cb = 0; cb < 2; ++cb) {
      const int col = chunk * 64 + hf * 32 + cb * 16 + g8;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = nb * 8 + 2 * t4 + (e & 1);
          if (row < M) mine[(size_t)row * NT + col + (e >> 1) * 8] = d[cb][nb][e];
          d[cb][nb][e] = 0.0f;
        }
    }
    gs_consumers_sync();
    if (tid == 0) {
      const unsigned int prev = gs_atom_add_acq_rel(&a.counters[cur_ct], 1u);  // publishes this CTA's slot, acquires the others'
      const int last = (prev == (unsigned int)(n_contrib - 1));
      if (last) a.counters[cur_ct] = 0u;
      s_last = last;
    }
    gs_consumers_sync();
    if (*(volatile int*)&s_last) {
      const float* all = a.partials + ((size_t)cur_ct * max_contrib * M) * NT;
      const int No = ep.glu ? N / 2 : N;
      // work items: (row, group of 4 columns); per item up to eight slots are read at once and added in slot order
      for (int idx = tid; idx < M * 64; idx += 256) {
        {
          float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          const float4* src = reinterpret_cast<const float4*>(all) + idx;
          const size_t slot_stride = (size_t)M * NT / 4;
          for (int j0 = 0; j0 < n_contrib; j0 += 8) {
            float4 t[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
              t[q] = j0 + q < n_contrib ? __ldcg(src + (size_t)(j0 + q) * slot_stride) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (j0 + q < n_contrib) {
                sum.x += t[q].x; sum.y += t[q].y; sum.z += t[q].z; sum.w += t[q].w;
              }
          }
          const int row = idx >> 6, c = cur_ct * NT + (idx & 63) * 4;
          const float v[4] = {sum.x, sum.y, sum.z, sum.w};
          if (a.rope_on) {
            // four columns = two rotation pairs of one head (hd and the section boundaries are multiples of four)
            if (c + 3 < N) {
              const RopeFuse& rf = a.rope;
              const int pos = state_len(rf.state, row, rf.T0);
              const int sec = c < rf.Hd ? 0 : (c < rf.Hd + rf.KVd ? 1 : 2);
              const int cc = c - (sec == 0 ? 0 : (sec == 1 ? rf.Hd : rf.Hd + rf.KVd));
              const int head = cc / rf.hd, e0 = cc % rf.hd;
              float t[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) t[e] = __half2float(__float2half_rn(v[e] + (bias ? __half2float(bias[c + e]) : 0.0f)));
              if (rf.use_rope && sec < 2 && pos < rf.Tmax) {
                const float2 cs0 = rf.tab[(int64_t)pos * (rf.hd / 2) + e0 / 2], cs1 = rf.tab[(int64_t)pos * (rf.hd / 2) + e0 / 2 + 1];
                const float a0 = t[0], b0 = t[1], a1 = t[2], b1 = t[3];
                t[0] = a0 * cs0.x - b0 * cs0.y; t[1] = b0 * cs0.x + a0 * cs0.y;
                t[2] = a1 * cs1.x - b1 * cs1.y; t[3] = b1 * cs1.x + a1 * cs1.y;
              }
              const __half2 h01 = __floats2half2_rn(t[0], t[1]), h23 = __floats2half2_rn(t[2], t[3]);
              uint2 out;
              out.x = *reinterpret_cast<const uint32_t*>(&h01);
              out.y = *reinterpret_cast<const uint32_t*>(&h23);
              if (sec == 0) {
                *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(ep.y) + (size_t)row * N + c) = out;
              } else if (pos < rf.Tmax) {   // capacity is checked on the host; never write past the cache
                __half* dst = reinterpret_cast<__half*>(sec == 1 ? rf.cK : rf.cV) + (((int64_t)row * (rf.KVd / rf.hd) + head) * rf.Tmax + pos) * rf.hd + e0;
                *reinterpret_cast<uint2*>(dst) = out;
              }
            }
          } else if (!ep.glu) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (c + e < N) {
                float x = gs_act(v[e] + (bias ? __half2float(bias[c + e]) : 0.0f), ep.act);
                const size_t o = (size_t)row * N + c + e;
                if (ep.residual) x += ep.residual[o];
                if (ep.y32) ep.y32[o] = x;
                else reinterpret_cast<__half*>(ep.y)[o] = __float2half_rn(x);
              }
            }
          } else {
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
              if (c + e + 1 < N) {
                float av = v[e] + (bias ? __half2float(bias[c + e]) : 0.0f);
                const float gv = v[e + 1] + (bias ? __half2float(bias[c + e + 1]) : 0.0f);
                if (ep.act == TSB200_ACT_SWIGLU) av = av / (1.0f + expf(-av));
                float x = av * gv;
                const size_t o = (size_t)row * No + ((c + e) >> 1);
                if (ep.residual) x += ep.residual[o];
                if (ep.y32) ep.y32[o] = x;
                else reinterpret_cast<__half*>(ep.y)[o] = __float2half_rn(x);
              }
            }
          }
        }
      }
    }
    gs_consumers_sync();  // s_last is rewritten at the next segment end
  }
  if (tid == 0 && *(volatile int*)&s_err) {
    g_gs_error = 1;
    if (a.error_flag) *a.error_flag = 1;
  }
}

// ---- column-chunk variant for 17..64 rows ------------------------------------------------------------------------------
// With many rows the stream-K hand-over is expensive: every CTA leaves M x 256 floats per shared column tile and the
// last arriver adds up to ten such slots alone.  Here a CTA owns ONE 64-column box of the packed tiles (4 KB per k tile,
// contiguous) over a K range, so a box has few contributors (ksplit, usually 1..4) and a partial is M x 64 floats.
// Stage = two k tiles of the box (2 x 4 KB bulk copies) + the activation tile [rows][64 k] (TMA tensor copy, 128-byte
// swizzle).  Four consumer warps own 16 columns each; three CTAs fit on an SM, so one CTA's prologue and epilogue
// overlap the others' streaming.
constexpr int kGcThreads = 160;            // 4 consumer warps + producer warp
constexpr int kGcStages = 4;
constexpr int kGcStageBytes = 8192 + 8192; // W: 2 k tiles x 4 KB; x: 64 rows x 128 B

struct GcArgs {
  const unsigned char* Wp;
  int M, K, N, KB, CT;
  int ksplit, k2_per;        // K ranges per box; stages (pairs of k tiles) per range
  int prefetch;              // 1: the first ring-full of weight tiles is requested before the wait on the previous kernel
  float* partials;           // [boxes][ksplit][M][64]
  unsigned int* counters;    // [boxes], zero on entry, self-resetting
  int* error_flag;
  Epilogue ep;
};

template <int NB>
__global__ void __launch_bounds__(kGcThreads, 3) gemm_chunk_mma_kernel(const __grid_constant__ CUtensorMap mapX, GcArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kGcStages * kGcStageBytes);
  uint64_t* empty = full + kGcStages;
  float* red = reinterpret_cast<float*>(smem);  // [M][64] after the main loop (the stages are free then)
  __shared__ int s_err, s_last;

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int M = a.M, N = a.N, KB = a.KB;
  const int box = blockIdx.x / a.ksplit, ks = blockIdx.x % a.ksplit;   // the K ranges of a box run side by side
  const int ct = box >> 2, j = box & 3;
  const int k2_total = (KB + 1) / 2;
  const int k2_beg = ks * a.k2_per, k2_end = min(k2_total, k2_beg + a.k2_per);
  const int n_st = max(k2_end - k2_beg, 0);

  if (tid == 0) {
    for (int i = 0; i < kGcStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 4);
    }
    s_err = 0;
    s_last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  grid_dep_launch();
  if (!(w == 4 && lane == 0)) grid_dep_wait();  // scratch slots, counters and residual rows belong to earlier kernels too

  if (w == 4) {
    if (lane == 0) {
      const unsigned char* wsrc = a.Wp + ((size_t)ct * KB) * kTileBytes + (size_t)j * 4096;
      auto put_w = [&](int i) {
        const int s = i % kGcStages;
        const int kb0 = (k2_beg + i) * 2;
        const bool two = kb0 + 1 < KB;
        unsigned char* dst = smem + (size_t)s * kGcStageBytes;
        mbar_expect_tx(&full[s], (two ? 8192 : 4096) + NB * 8 * 128);
        bulk_g2s(dst, wsrc + (size_t)kb0 * kTileBytes, 4096, &full[s]);
        if (two) bulk_g2s(dst + 4096, wsrc + (size_t)(kb0 + 1) * kTileBytes, 4096, &full[s]);
      };
      // the weights do not depend on the previous kernel: the first ring-full is requested before the wait on it
      const int n_pre = a.prefetch ? min(kGcStages, n_st) : 0;
      for (int i = 0; i < n_pre; ++i) put_w(i);
      grid_dep_wait();  // the activation rows come from the previous kernel
      int done = 0;
      for (int i = 0; i < n_st; ++i) {
        const int s = i % kGcStages, r = i / kGcStages;
        if (i >= kGcStages && !mbar_wait(&empty[s], (unsigned)((r - 1) & 1))) {
          s_err = 1;
          break;
        }
        if (i >= n_pre) put_w(i);
        gs_tma_load_2d(smem + (size_t)s * kGcStageBytes + 8192, &mapX, (k2_beg + i) * 2 * kKT, 0, &full[s]);  // x = kb0 * 32 halves: a 64-byte multiple
        done = i + 1;
      }
      if (*(volatile int*)&s_err) {
        // stages requested ahead get their activation tile too, so that every copy into this CTA has landed on return
        for (int i = done; i < n_pre; ++i) gs_tma_load_2d(smem + (size_t)(i % kGcStages) * kGcStageBytes + 8192, &mapX, 0, 0, &full[i % kGcStages]);
        if (done < n_pre) done = n_pre;
        const int first = done > kGcStages ? done - kGcStages : 0;
        for (int i = first; i < done; ++i) mbar_wait(&full[i % kGcStages], (unsigned)((i / kGcStages) & 1), 1u << 16);
        g_gs_error = 1;
        if (a.error_flag) *a.error_flag = 1;
      }
    }
  } else {
    // ---------------- consumer warps: warp w owns columns [w*16, w*16+16) of the box
    const int g8 = lane >> 2, t4 = lane & 3;
    const int lrow = (lane & 7) + ((lane >> 4) << 3);
    const int lunit = (lane >> 3) & 1;
    const int xr = lane & 7, xc = lane >> 3;
    float d[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) d[nb][e] = 0.0f;
    bool dead = false;
    for (int i = 0; i < n_st; ++i) {
      const int s = i % kGcStages, r = i / kGcStages;
      if (*(volatile int*)&s_err) dead = true;
      if (!mbar_wait(&full[s], (unsigned)(r & 1), dead ? 4096u : kSpinLimit)) {
        s_err = 1;
        dead = true;
      }
      const uint32_t wbase = smem_u32(smem + (size_t)s * kGcStageBytes);
      const uint32_t xbase = wbase + 8192;
      const int kk_end = ((k2_beg + i) * 2 + 1 < KB) ? 4 : 2;  // a missing second k tile was not copied
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {            // the two k tiles of the stage
        if (h2 * 2 >= kk_end) break;
        // activation fragments of this k tile: rows of 128 B, 16-byte chunks XOR-ed with row & 7
        uint32_t bf[NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const int n = nb * 8 + xr;
          const int c = h2 * 4 + xc;
          gs_ldmatrix_x4(xbase + n * 128 + ((c ^ (n & 7)) << 4), bf[nb][0], bf[nb][1], bf[nb][2], bf[nb][3]);
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int k = kk * 16 + lrow;
          const int unit = w * 2 + lunit;
          uint32_t a0, a1, a2, a3;
          gs_ldmatrix_x4_trans(wbase + h2 * 4096 + k * 128 + ((unit ^ (k & 7)) << 4), a0, a1, a2, a3);
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) gs_mma_16816(d[nb], a0, a1, a2, a3, bf[nb][2 * kk], bf[nb][2 * kk + 1]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
    // ---- accumulators -> red[row][64] (the stages are free: every copy has been consumed)
    asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = nb * 8 + 2 * t4 + (e & 1);
        if (row < M) red[row * 64 + w * 16 + g8 + (e >> 1) * 8] = d[nb][e];
      }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    bool finish = a.ksplit == 1;
    if (a.ksplit > 1) {
      float* mine = a.partials + ((size_t)blockIdx.x * M) * 64;   // [box][ks] = blockIdx.x
      for (int idx = tid; idx < M * 16; idx += 128) reinterpret_cast<float4*>(mine)[idx] = reinterpret_cast<const float4*>(red)[idx];
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (tid == 0) {
        const unsigned int prev = gs_atom_add_acq_rel(&a.counters[box], 1u);
        const int last = (prev == (unsigned int)(a.ksplit - 1));
        if (last) a.counters[box] = 0u;
        s_last = last;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*(volatile int*)&s_last) {
        const float4* all = reinterpret_cast<const float4*>(a.partials + ((size_t)box * a.ksplit * M) * 64);
        for (int idx = tid; idx < M * 16; idx += 128) {
          float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          for (int z = 0; z < a.ksplit; ++z) {
            const float4 t = __ldcg(all + (size_t)z * M * 16 + idx);
            acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
          }
          reinterpret_cast<float4*>(red)[idx] = acc;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        finish = true;
      }
    }
    if (finish) {
      const Epilogue ep = a.ep;
      const __half* bias = reinterpret_cast<const __half*>(ep.bias);
      const int No = ep.glu ? N / 2 : N;
      for (int idx = tid; idx < M * 16; idx += 128) {
        const int row = idx >> 4, c = ct * 256 + j * 64 + (idx & 15) * 4;
        const float4 t = reinterpret_cast<const float4*>(red)[idx];
        const float v[4] = {t.x, t.y, t.z, t.w};
        if (!ep.glu) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (c + e < N) {
              float x = gs_act(v[e] + (bias ? __half2float(bias[c + e]) : 0.0f), ep.act);
              const size_t o = (size_t)row * N + c + e;
              if (ep.residual) x += ep.residual[o];
              if (ep.y32) ep.y32[o] = x;
              else reinterpret_cast<__half*>(ep.y)[o] = __float2half_rn(x);
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; e += 2) {
            if (c + e + 1 < N) {
              float av = v[e] + (bias ? __half2float(bias[c + e]) : 0.0f);
              const float gv = v[e + 1] + (bias ? __half2float(bias[c + e + 1]) : 0.0f);
              if (ep.act == TSB200_ACT_SWIGLU) av = av / (1.0f + expf(-av));
              float x = av * gv;
              const size_t o = (size_t)row * No + ((c + e) >> 1);
              if (ep.residual) x += ep.residual[o];
              if (ep.y32) ep.y32[o] = x;
              else reinterpret_cast<__half*>(ep.y)[o] = __float2half_rn(x);
            }
          }
        }
      }
    }
    if (tid == 0 && *(volatile int*)&s_err) {
      g_gs_error = 1;
      if (a.error_flag) *a.error_flag = 1;
    }
  }
}

// ---- host side ---------------------------------------------------------------------------------------------------------
typedef CUresult (*GsEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static GsEncodeTiledFn gs_get_encode() {
  static GsEncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<GsEncodeTiledFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

template <int NB, int KQ = 0>
static int gs_launch(int device, const CUtensorMap& mapX, const GsArgs& a, int grid, size_t smem, bool pdl, cudaStream_t s) {
  static bool attr_done[kMaxDevices] = {};
  if (!attr_done[device]) {
    TSB_CUDA(cudaFuncSetAttribute(gemm_stream_mma_kernel<NB, KQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    attr_done[device] = true;
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
  TSB_CUDA(cudaLaunchKernelEx(&cfg, gemm_stream_mma_kernel<NB, KQ>, mapX, a));
  count_launch(device);
  return 1;
}

// 1 when a kernel of this file gave up waiting since the last call (and clears the mark).
int gs_take_error() {
  int e = 0;
  if (cudaMemcpyFromSymbol(&e, g_gs_error, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (e) {
    const int z = 0;
    cudaMemcpyToSymbol(g_gs_error, &z, sizeof(int));
  }
  return e;
}

int64_t gemm_stream_mma_workspace_bytes(int M, int K, int N, int sm_count) {
  const long long KB = (K + kKT - 1) / kKT, CT = (N + 255) / 256;
  long long g = sm_count;
  if (g > KB * CT) g = KB * CT;
  const long long per = (KB * CT) / (g > 0 ? g : 1);
  const long long mc = KB / (per > 0 ? per : 1) + 2;
  const long long chunk = (long long)((N + 63) / 64) * 8 * M * 64 * 4;  // column-chunk variant: up to 8 K ranges per box
  const long long stream = CT * mc * M * 256 * 4;
  return kWsCounterBytes + (chunk > stream ? chunk : stream) + 256;
}

static int gs_prefetch_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("TSB200_GEMM_PREFETCH");  // "0": weights are requested only after the previous kernel has ended (A/B measurements)
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on;
}

template <int NB>
static int gc_launch(int device, const CUtensorMap& mapX, const GcArgs& a, int grid, bool pdl, cudaStream_t s) {
  static bool attr_done[kMaxDevices] = {};
  const size_t smem = kGcStages * kGcStageBytes + 1024 + 128;
  if (!attr_done[device]) {
    TSB_CUDA(cudaFuncSetAttribute(gemm_chunk_mma_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done[device] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  TSB_CUDA(cudaLaunchKernelEx(&cfg, gemm_chunk_mma_kernel<NB>, mapX, a));
  count_launch(device);
  return 1;
}

// Column-chunk variant (17..64 rows).  1 ok, 0 error, 2 not handled.
static int launch_gemm_chunk_mma(int device, DeviceState* st, const void* x, const void* Wp, int M, int K, int N, const Epilogue& ep,
                                 int* error_flag, bool pdl, void* ws, int64_t ws_bytes, cudaStream_t s) {
  GsEncodeTiledFn enc = gs_get_encode();
  if (!enc) return 2;
  const int NB = M <= 32 ? 4 : 8;
  GcArgs a{};
  a.Wp = reinterpret_cast<const unsigned char*>(Wp);
  a.M = M; a.K = K; a.N = N;
  a.KB = (K + kKT - 1) / kKT;
  a.CT = (N + 255) / 256;
  const int boxes = (N + 63) / 64;                 // boxes that hold real columns (the last column tile may have fewer than 4)
  const int k2_total = (a.KB + 1) / 2;
  // about two CTAs per SM in flight (three fit); a K range is at least 8 stages long
  int ks = (2 * st->sm_count + boxes - 1) / boxes;
  if (ks > k2_total / 8) ks = k2_total / 8;
  if (ks < 1) ks = 1;
  if (ks > 8) ks = 8;
  a.k2_per = (k2_total + ks - 1) / ks;
  ks = (k2_total + a.k2_per - 1) / a.k2_per;       // no empty range
  a.ksplit = ks;
  a.prefetch = gs_prefetch_enabled();
  const int64_t need = kWsCounterBytes + (int64_t)boxes * ks * M * 64 * 4;
  if (ks > 1 && (!ws || ws_bytes < need || (int64_t)boxes * 4 > kWsCounterBytes - 256)) return 2;
  a.counters = reinterpret_cast<unsigned int*>(ws);
  a.partials = ws ? reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + kWsCounterBytes) : nullptr;
  a.error_flag = error_flag;
  a.ep = ep;
  CUtensorMap mapX;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)(NB * 8)};
    const cuuint32_t el[2] = {1, 1};
    const CUresult r = enc(&mapX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, el,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TSB_CHECK(r == CUDA_SUCCESS, "gemm_chunk: cuTensorMapEncodeTiled failed with %d", (int)r);
  }
  const int grid = boxes * ks;
  if (NB == 4) return gc_launch<4>(device, mapX, a, grid, pdl, s);
  return gc_launch<8>(device, mapX, a, grid, pdl, s);
}

// 1 ok, 0 error, 2 shape not handled (caller falls back).
int launch_gemm_stream_mma(int device, DeviceState* st, const void* x, const void* Wp, int M, int K, int N, const Epilogue& ep,
                           int* error_flag, bool pdl, void* ws, int64_t ws_bytes, cudaStream_t s) {
  {
    static int enabled = -1;
    if (enabled < 0) {
      const char* e = getenv("TSB200_GEMM_STREAM");  // "0": decode batches go to the tile-per-CTA tensor-core GEMM (A/B measurements)
      enabled = (e && e[0] == '0') ? 0 : 1;
    }
    if (!enabled) return 2;
  }
  if (M < 1 || M > 64 || K % 8 != 0 || ((uintptr_t)x % 16) != 0 || ((uintptr_t)Wp % 16) != 0) return 2;
  if (M > 16) {
    static int chunk = -1;
    if (chunk < 0) {
      const char* e = getenv("TSB200_GEMM_CHUNK");  // "0": stream-K hand-over for every row count (A/B measurements)
      chunk = (e && e[0] == '0') ? 0 : 1;
    }
    if (chunk) {
      const int r = launch_gemm_chunk_mma(device, st, x, Wp, M, K, N, ep, error_flag, pdl, ws, ws_bytes, s);
      if (r != 2) return r;
    }
  }
  GsEncodeTiledFn enc = gs_get_encode();
  if (!enc) return 2;
  const int NB = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  GsArgs a{};
  a.Wp = reinterpret_cast<const unsigned char*>(Wp);
  a.M = M; a.K = K; a.N = N;
  a.KB = (K + kKT - 1) / kKT;
  a.CT = (N + 255) / 256;
  const long long U = (long long)a.KB * a.CT;
  long long g = st->sm_count;
  if (g > U) g = U;
  a.max_contrib = (int)(a.KB / (U / g)) + 2;
  const size_t fixed = 32 * sizeof(uint64_t) + 1024 + 128;
  int stages = (int)((225 * 1024 - fixed) / kGsStageBytes);
  if (stages > 16) stages = 16;
  a.stages = stages;
  a.prefetch = gs_prefetch_enabled();
  const int64_t need = kWsCounterBytes + (int64_t)a.CT * a.max_contrib * M * 256 * 4;
  if (!ws || ws_bytes < need) return 2;
  a.counters = reinterpret_cast<unsigned int*>(ws);
  a.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + kWsCounterBytes);
  a.error_flag = error_flag;
  a.ep = ep;
  CUtensorMap mapX;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {32, (cuuint32_t)(NB * 8)};
    const cuuint32_t el[2] = {1, 1};
    const CUresult r = enc(&mapX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, el,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TSB_CHECK(r == CUDA_SUCCESS, "gemm_stream: cuTensorMapEncodeTiled failed with %d", (int)r);
  }
  const size_t smem = fixed + (size_t)stages * kGsStageBytes;
  switch (NB) {
    case 1: return gs_launch<1>(device, mapX, a, (int)g, smem, pdl, s);
    case 2: return gs_launch<2>(device, mapX, a, (int)g, smem, pdl, s);
    case 4: return gs_launch<4>(device, mapX, a, (int)g, smem, pdl, s);
    default: return gs_launch<8>(device, mapX, a, (int)g, smem, pdl, s);
  }
}

// y = epilogue(norm(x32[M,K]) * W[K,N]) in one launch, for up to 8 rows of a fp16 model whose width is 1024, 2048 or 4096
// (M * K <= 16384): the consumer warps norm the rows themselves.  1 ok, 0 error, 2 shape not handled (the caller runs the
// norm kernel and the plain linear).
int launch_gemm_stream_mma_norm(int device, DeviceState* st, const float* x32, const void* gamma, const void* beta, int norm_type, float eps,
                                const void* Wp, int M, int K, int N, const Epilogue& ep, int* error_flag, bool pdl, void* ws, int64_t ws_bytes,
                                cudaStream_t s, const RopeFuse* rope) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("TSB200_GEMM_FUSED_NORM");  // "0": a norm launch in front of every linear (A/B measurements)
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  if (!enabled || !gamma) return 2;
  if (K != 1024 && K != 2048 && K != 4096) return 2;
  const int KQ = K / 1024;
  if (M < 1 || M > 8 || M * KQ > 16 || ((uintptr_t)x32 % 16) != 0 || ((uintptr_t)Wp % 16) != 0 || ((uintptr_t)gamma % 4) != 0 ||
      (beta && ((uintptr_t)beta % 4) != 0))
    return 2;
  GsArgs a{};
  a.Wp = reinterpret_cast<const unsigned char*>(Wp);
  a.M = M; a.K = K; a.N = N;
  a.KB = (K + kKT - 1) / kKT;
  a.CT = (N + 255) / 256;
  const long long U = (long long)a.KB * a.CT;
  long long g = st->sm_count;
  if (g > U) g = U;
  a.max_contrib = (int)(a.KB / (U / g)) + 2;
  const size_t xs_bytes = (size_t)8 * ((size_t)K * 2 + 16);
  const size_t fixed = 32 * sizeof(uint64_t) + 1024 + 128 + xs_bytes;
  int stages = (int)((225 * 1024 - fixed) / kTileBytes);
  if (stages > 16) stages = 16;
  if (stages < 4) return 2;
  a.stages = stages;
  a.prefetch = 1;
  a.xres = x32;
  a.gamma = reinterpret_cast<const __half*>(gamma);
  a.beta = reinterpret_cast<const __half*>(beta);
  a.norm_type = norm_type;
  a.eps = eps;
  if (rope) {
    // q | k | v columns with whole heads of a multiple of four elements, fp16 output rows, no activation / gate / residual
    if (rope->hd % 4 != 0 || rope->Hd % rope->hd != 0 || rope->KVd % rope->hd != 0 || rope->Hd + 2 * rope->KVd != N || N % 4 != 0 || !ep.y ||
        ep.y32 || ep.residual || ep.glu || ep.act != TSB200_ACT_NONE || (rope->use_rope && !rope->tab) || ((uintptr_t)ep.y % 8) != 0 ||
        ((uintptr_t)rope->cK % 8) != 0 || ((uintptr_t)rope->cV % 8) != 0)
      return 2;
    a.rope_on = 1;
    a.rope = *rope;
  }
  const int64_t need = kWsCounterBytes + (int64_t)a.CT * a.max_contrib * M * 256 * 4;
  if (!ws || ws_bytes < need) return 2;
  a.counters = reinterpret_cast<unsigned int*>(ws);
  a.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + kWsCounterBytes);
  a.error_flag = error_flag;
  a.ep = ep;
  CUtensorMap none{};   // unused by these instantiations
  const size_t smem = fixed + (size_t)stages * kTileBytes;
  switch (KQ) {
    case 1: return gs_launch<1, 1>(device, none, a, (int)g, smem, pdl, s);
    case 2: return gs_launch<1, 2>(device, none, a, (int)g, smem, pdl, s);
    default: return gs_launch<1, 4>(device, none, a, (int)g, smem, pdl, s);
  }
}

}  // namespace tsb
