// Linear layer for decode batches of 17..64 rows on packed fp16 weights, on the 5th-generation tensor cores:
// y[M,N] = epilogue(x[M,K] * W[K,N]).
//
// At these row counts the product is bound by streaming the weights once, but every weight byte feeds 2 x 64 flops:
// mma.sync consumers cannot keep up with HBM.  Here the WEIGHTS are the 128-row operand of tcgen05.mma (A, read in
// place from the packed tiles, which are stored as the MN-major 128-byte-swizzled shared-memory image) and the
// activation rows are its N dimension (B: [64 rows][64 k], K-major, one TMA tensor copy per stage; rows beyond M are
// zero-filled by the copy), so the accumulator of a 128-column group of the output is 128 TMEM lanes x 64 columns.
//
//   * persistent CTAs, one per SM, each owning a contiguous, evenly sized range of the units (column group, pair of
//     k tiles) in column-group-major order (stream-K).  A column group is a whole packed column tile (256 columns, one
//     32 KB bulk copy per unit) when few CTAs then share a group, else half of one (128 columns, two 8 KB copies), so
//     that the sums of a group meet from few contributors;
//   * warp 0: TMA producer through a ring of stages; warp 1: one thread issues the MMAs and hands stages back with
//     tcgen05.commit; warp 2 owns the TMEM allocation; warps 4-7 drain finished accumulators (two sets in TMEM, so the
//     drain of a group overlaps the MMAs of the next one) into a scratch slot; the CTA that delivers the last share of a
//     group adds the slots in fixed order (bitwise reproducible) and applies bias / activation / gate / residual.
// Every mbarrier wait is bounded; on timeout the error word is raised and the CTA drains and returns.
//
// Replaces cublasGemmEx + bias / activation kernels for decode batches (TensorSharp.CUDA/MatrixMul/CudaMatrixMulMM.cs:305-504).
#include <cuda.h>

#include <cstdlib>

#include "kernels.cuh"
#include "stream_common.cuh"

namespace tsb {

constexpr int kStcThreads = 256;
constexpr int kStcXBytes = 64 * 128;   // activation tile of a stage: 64 rows x 64 k halves
constexpr int kStcRows = 64;           // N of the MMA (activation rows, zero-filled beyond M)
constexpr unsigned kStcSpin = 1u << 22;

// Raised by a kernel whose bounded wait ran out; read and cleared by stc_take_error().
__device__ int g_stc_error;
#ifdef TSB200_TRACE
__device__ long long g_stc_trace[160 * 32];   // per CTA: %globaltimer stamps of the last launch
#define STRC(slot) do { g_stc_trace[blockIdx.x * 32 + (slot)] = gtimer(); } while (0)
#else
#define STRC(slot) do { } while (0)
#endif

struct StcArgs {
  const unsigned char* Wp;
  int M, K, N, KB, CT;
  int nh;                   // column halves per unit: 2 = whole packed column tiles, 1 = 128-column halves
  int stages, max_contrib;
  float* partials;          // [groups][max_contrib][M][128 * nh]
  unsigned int* counters;   // [groups], zero on entry, self-resetting
  int* error_flag;
  Epilogue ep;
};

__device__ __forceinline__ uint32_t stc_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void stc_tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(stc_u32(dst)),
      "l"(map), "r"(stc_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in 16-byte units,
// version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t stc_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ void stc_umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void stc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(stc_u32(bar)) : "memory");
}
__device__ __forceinline__ void stc_tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned stc_atom_add_acq_rel(unsigned* p, unsigned v) {
  unsigned old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void stc_epi_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // the four epilogue warps
__device__ __forceinline__ float stc_act(float v, int act) {
  switch (act) {
    case TSB200_ACT_RELU: return v < 0.0f ? 0.0f : v;
    case TSB200_ACT_SILU: return v / (1.0f + expf(-v));
    case TSB200_ACT_LEAKYRELU: return v < 0.0f ? 0.01f * v : v;
    case TSB200_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    default: return v;
  }
}

// Epilogue for four consecutive columns (c a multiple of 4) of one row: bias, activation, gate product on interleaved
// (a_j, g_j) column pairs, fp32 residual, store.  8- and 16-byte accesses where the row length allows them.
// One copy of this code (not inlined): with the activation functions inlined at each of a thread's sixteen items the
// reduction of a group was 300 KB of instructions that every SM fetched cold at the tail of the kernel (measured:
// 44 us for stores that take 2 us).
__device__ __noinline__ void stc_store4(const StcArgs& a, int row, int c, float v0, float v1, float v2, float v3) {
  const float v[4] = {v0, v1, v2, v3};
  const Epilogue& ep = a.ep;
  const __half* bias = reinterpret_cast<const __half*>(ep.bias);
  const int N = a.N;
  float b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const bool full = c + 3 < N;
  if (bias) {
    if (full) {
      const uint2 raw = *reinterpret_cast<const uint2*>(bias + c);
      const __half2* h = reinterpret_cast<const __half2*>(&raw);
      const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]);
      b[0] = f0.x; b[1] = f0.y; b[2] = f1.x; b[3] = f1.y;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (c + e < N) b[e] = __half2float(bias[c + e]);
    }
  }
  if (!ep.glu) {
    float x[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = stc_act(v[e] + b[e], ep.act);
    const size_t o = (size_t)row * N + c;
    if (full && (N & 3) == 0) {
      if (ep.residual) {
        const float4 r = *reinterpret_cast<const float4*>(ep.residual + o);
        x[0] += r.x; x[1] += r.y; x[2] += r.z; x[3] += r.w;
      }
      if (ep.y32) {
        *reinterpret_cast<float4*>(ep.y32 + o) = make_float4(x[0], x[1], x[2], x[3]);
      } else {
        uint2 out;
        __half2* h = reinterpret_cast<__half2*>(&out);
        h[0] = __floats2half2_rn(x[0], x[1]);
        h[1] = __floats2half2_rn(x[2], x[3]);
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(ep.y) + o) = out;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (c + e < N) {
          float y = x[e];
          if (ep.residual) y += ep.residual[o + e];
          if (ep.y32) ep.y32[o + e] = y;
          else reinterpret_cast<__half*>(ep.y)[o + e] = __float2half_rn(y);
        }
      }
    }
  } else {
    const int No = N / 2;
#pragma unroll
    for (int e = 0; e < 4; e += 2) {
      if (c + e + 1 < N) {
        float av = v[e] + b[e];
        const float gv = v[e + 1] + b[e + 1];
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

// The CTA that delivered the last share of group `cur` adds the contributors' slots in slot order (two slots in flight
// per round trip) and applies the epilogue.  `t` of `nt` threads take part.  Used for groups that finish while the CTA
// still has work: their cost hides behind the MMAs of the next group.
__device__ __noinline__ void stc_finish_group(const StcArgs& a, int cur, int n_contrib, int t, int nt) {
  const int M = a.M, TW = 128 * a.nh;
  const float* all = a.partials + ((size_t)cur * a.max_contrib * M) * TW;
  const size_t slot_elems = (size_t)M * TW;
  const int q4 = TW / 4;                       // groups of 4 columns per row
  const int c_base = cur * TW;
  // work items: (row, group of 4 columns); eight items per thread, two contributors in flight
#pragma unroll 1
  for (int i0 = 0; i0 < M * q4; i0 += nt * 8) {
    float4 acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 1
    for (int j = 0; j < n_contrib; j += 2) {
      const bool two = j + 1 < n_contrib;
      const float4* s0 = reinterpret_cast<const float4*>(all + (size_t)j * slot_elems);
      const float4* s1 = reinterpret_cast<const float4*>(all + (size_t)(two ? j + 1 : j) * slot_elems);
      float4 t0[8], t1[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int idx = i0 + e * nt + t;
        const int ic = idx < M * q4 ? idx : 0;
        t0[e] = __ldcg(s0 + ic);
        t1[e] = __ldcg(s1 + ic);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        acc[e].x += t0[e].x; acc[e].y += t0[e].y; acc[e].z += t0[e].z; acc[e].w += t0[e].w;
        if (two) {
          acc[e].x += t1[e].x; acc[e].y += t1[e].y; acc[e].z += t1[e].z; acc[e].w += t1[e].w;
        }
      }
    }
#pragma unroll
    for (int e8 = 0; e8 < 8; ++e8) {
      const int idx = i0 + e8 * nt + t;
      if (idx >= M * q4) continue;
      stc_store4(a, idx / q4, c_base + (idx % q4) * 4, acc[e8].x, acc[e8].y, acc[e8].z, acc[e8].w);
    }
  }
}

// The same for the CTA's LAST group, whose reduction is the tail of the kernel: the ring is free by then, so the
// contributors' slots (contiguous, up to 64 KB each) are fetched into it with bulk copies that fly together - one
// memory round trip instead of one per slot - and all threads of the CTA add them from shared memory, in slot order.
__device__ __noinline__ void stc_finish_tail(const StcArgs& a, int cur, int n_contrib, unsigned char* ring, int ring_bytes, uint64_t* bar,
                                             volatile int* s_err, int tid) {
  const int M = a.M, TW = 128 * a.nh;
  const float* all = a.partials + ((size_t)cur * a.max_contrib * M) * TW;
  const size_t slot_elems = (size_t)M * TW;
  const int slot_bytes = (int)(slot_elems * 4);
  const int per_round = ring_bytes / slot_bytes;   // >= 1: the host sizes the ring for at least one slot
  const int q4 = TW / 4, items = M * q4;
  const int c_base = cur * TW;
  constexpr int kMaxItems = 16;   // (row, 4 columns) items per thread: 64 rows x 256 columns over 256 threads
  float4 acc[kMaxItems];
#pragma unroll
  for (int e = 0; e < kMaxItems; ++e) acc[e] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  unsigned parity = 0;
#pragma unroll 1
  for (int j0 = 0; j0 < n_contrib; j0 += per_round) {
    const int nj = n_contrib - j0 < per_round ? n_contrib - j0 : per_round;
    if (tid == 0) {
      // the slots were written by other SMs through the generic proxy (acquired with the arrival counter); the copies
      // below read them through the async proxy
      asm volatile("fence.proxy.async;" ::: "memory");
      mbar_expect_tx(bar, (unsigned)(nj * slot_bytes));
      for (int j = 0; j < nj; ++j) bulk_g2s(ring + (size_t)j * slot_bytes, all + (size_t)(j0 + j) * slot_elems, (unsigned)slot_bytes, bar);
    }
    if (!mbar_wait(bar, parity, kStcSpin)) *s_err = 1;
    if (tid == 0) STRC(28);
    parity ^= 1u;
    const float4* sm = reinterpret_cast<const float4*>(ring);
#pragma unroll 1
    for (int j = 0; j < nj; ++j) {
#pragma unroll
      for (int e = 0; e < kMaxItems; ++e) {
        const int idx = e * kStcThreads + tid;
        if (idx < items) {
          const float4 t = sm[(size_t)j * (slot_elems / 4) + idx];
          acc[e].x += t.x; acc[e].y += t.y; acc[e].z += t.z; acc[e].w += t.w;
        }
      }
    }
    __syncthreads();   // everybody has read the ring before the next round overwrites it
    if (tid == 0) STRC(29);
  }
  // Epilogue.  A thread's items share their four columns (256 threads step whole rows), so bias is fetched once; the
  // activation functions other than "none" are one non-inlined copy (see stc_store4 about code size).
  const Epilogue& ep = a.ep;
  const int N = a.N, c = c_base + (tid % q4) * 4, row0 = tid / q4, row_step = kStcThreads / q4;
  if (c + 3 < N && (N & 3) == 0 && !ep.glu && (ep.act == TSB200_ACT_NONE)) {
    float b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (ep.bias) {
      const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(ep.bias) + c);
      const __half2* h = reinterpret_cast<const __half2*>(&raw);
      const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]);
      b[0] = f0.x; b[1] = f0.y; b[2] = f1.x; b[3] = f1.y;
    }
    float4 r[kMaxItems];
    if (ep.residual) {
#pragma unroll
      for (int e = 0; e < kMaxItems; ++e) {
        const int row = row0 + e * row_step;
        r[e] = row < M ? *reinterpret_cast<const float4*>(ep.residual + (size_t)row * N + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    }
#pragma unroll
    for (int e = 0; e < kMaxItems; ++e) {
      const int row = row0 + e * row_step;
      if (row >= M) continue;
      float x0 = acc[e].x + b[0], x1 = acc[e].y + b[1], x2 = acc[e].z + b[2], x3 = acc[e].w + b[3];
      if (ep.residual) {
        x0 += r[e].x; x1 += r[e].y; x2 += r[e].z; x3 += r[e].w;
      }
      const size_t o = (size_t)row * N + c;
      if (ep.y32) {
        *reinterpret_cast<float4*>(ep.y32 + o) = make_float4(x0, x1, x2, x3);
      } else {
        uint2 out;
        __half2* h = reinterpret_cast<__half2*>(&out);
        h[0] = __floats2half2_rn(x0, x1);
        h[1] = __floats2half2_rn(x2, x3);
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(ep.y) + o) = out;
      }
    }
  } else if (c + 3 < N && (N & 3) == 0 && ep.glu && !ep.residual) {
    // gate product on interleaved (a_j, g_j) column pairs: two outputs per item
    float b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (ep.bias) {
      const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(ep.bias) + c);
      const __half2* h = reinterpret_cast<const __half2*>(&raw);
      const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]);
      b[0] = f0.x; b[1] = f0.y; b[2] = f1.x; b[3] = f1.y;
    }
    const bool silu = ep.act == TSB200_ACT_SWIGLU;
    const int No = N / 2;
#pragma unroll
    for (int e = 0; e < kMaxItems; ++e) {
      const int row = row0 + e * row_step;
      if (row >= M) continue;
      float a0 = acc[e].x + b[0], a1 = acc[e].z + b[2];
      const float g0 = acc[e].y + b[1], g1 = acc[e].w + b[3];
      if (silu) {
        a0 = a0 / (1.0f + expf(-a0));
        a1 = a1 / (1.0f + expf(-a1));
      }
      const size_t o = (size_t)row * No + (c >> 1);
      if (ep.y32) *reinterpret_cast<float2*>(ep.y32 + o) = make_float2(a0 * g0, a1 * g1);
      else *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(ep.y) + o) = __floats2half2_rn(a0 * g0, a1 * g1);
    }
  } else {
#pragma unroll
    for (int e = 0; e < kMaxItems; ++e) {
      const int row = row0 + e * row_step;
      if (row < M) stc_store4(a, row, c, acc[e].x, acc[e].y, acc[e].z, acc[e].w);
    }
  }
}

__global__ void __launch_bounds__(kStcThreads, 1) gemm_stream_tc_kernel(const __grid_constant__ CUtensorMap mapX, StcArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.stages, nh = a.nh;
  const int w_bytes = nh * 16384;               // weights of a stage: nh halves x 64 k
  const int stage_bytes = w_bytes + kStcXBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)S * stage_bytes);
  uint64_t* empty = full + 16;
  uint64_t* acc_full = empty + 16;    // [2]: the MMAs of a group have finished (tcgen05.commit)
  uint64_t* acc_empty = acc_full + 2; // [2]: the four epilogue warps have read the set
  uint64_t* tail_bar = acc_empty + 2;   // the bulk copies of the tail reduction
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail_bar + 1);
  __shared__ int s_err, s_last;
  __shared__ int s_tail[3];   // the CTA's last group: {this CTA delivered the last share, group, contributors}

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int M = a.M, N = a.N, KB = a.KB;
  const int KB2 = KB / 2;                       // the host sends only matrices with an even number of k tiles
  const int TW = 128 * nh;                      // columns of a group
  const int groups = a.CT * (2 / nh);
  const long long U = (long long)KB2 * groups, G = gridDim.x;   // the host launches at most U CTAs: no range is empty
  const int u_begin = (int)(U * blockIdx.x / G), u_end = (int)(U * (blockIdx.x + 1) / G);
  const uint32_t acc_cols = 64 * nh;            // TMEM columns of one accumulator set

  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    mbar_init(tail_bar, 1);
    s_err = 0;
    s_last = 0;
    s_tail[0] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (w == 2) {  // TMEM: two accumulator sets of up to 128 columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(stc_u32(tmem_slot)), "r"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  if (tid == 0) STRC(0);
  grid_dep_launch();
  // The activation rows, the scratch slots and the counters belong to the previous kernel until griddepcontrol.wait
  // returns; the weights do not: the producer starts their copies first and waits afterwards.
  if (!(w == 0 && lane == 0)) grid_dep_wait();

  if (w == 0) {
    if (lane == 0) {
      // ---------------- TMA producer
      auto weights = [&](int st, int grp, int k2) {
        unsigned char* dst = smem + (size_t)st * stage_bytes;
        mbar_expect_tx(&full[st], (unsigned)(w_bytes + kStcXBytes));
        if (nh == 2) {
          // two whole packed tiles of column tile `grp`: k tiles 2 k2 and 2 k2 + 1 follow each other
          bulk_g2s(dst, a.Wp + ((size_t)grp * KB + 2 * k2) * kTileBytes, 32768, &full[st]);
        } else {
          // boxes (2h, 2h + 1) of the column tile: 8 KB contiguous in each of the two k tiles
          const unsigned char* src = a.Wp + ((size_t)(grp >> 1) * KB + 2 * k2) * kTileBytes + (size_t)(grp & 1) * 8192;
          bulk_g2s(dst, src, 8192, &full[st]);
          bulk_g2s(dst + 8192, src + kTileBytes, 8192, &full[st]);
        }
      };
      const int n_pre = u_end - u_begin < S ? u_end - u_begin : S;
      for (int i = 0; i < n_pre; ++i) weights(i, (u_begin + i) / KB2, (u_begin + i) % KB2);
      grid_dep_wait();
      STRC(1);
      int s = 0, grp = u_begin / KB2, k2 = u_begin % KB2;
      unsigned round = 0;
      for (int u = u_begin; u < u_end; ++u) {
        if (round > 0) {
          if (!mbar_wait(&empty[s], (round - 1u) & 1u, kStcSpin)) {
            s_err = 1;
            break;
          }
          if (*(volatile int*)&s_err) break;
          weights(s, grp, k2);
        }
        stc_tma_load_2d(smem + (size_t)s * stage_bytes + w_bytes, &mapX, k2 * 64, 0, &full[s]);
        if (++k2 == KB2) {
          k2 = 0;
          ++grp;
        }
        if (++s == S) {
          s = 0;
          ++round;
        }
      }
    }
  } else if (w == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer.  Instruction descriptor: D fp32, A / B fp16, A MN-major (the weights), B K-major
      // (the activation rows), N = 64, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 15) | (0u << 16) | ((uint32_t)(kStcRows >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      int s = 0, k2 = u_begin % KB2, seg = 0;
      unsigned round = 0;
      bool seg_first = true;
      for (int u = u_begin; u < u_end; ++u) {
        const int set = seg & 1;
        if (seg_first && seg >= 2 && !mbar_wait(&acc_empty[set], (unsigned)(((seg >> 1) - 1) & 1), kStcSpin)) {
          s_err = 1;
          break;
        }
        if (!mbar_wait(&full[s], round & 1u, kStcSpin)) {
          s_err = 1;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t w_base = stc_u32(smem + (size_t)s * stage_bytes), x_base = w_base + (uint32_t)w_bytes;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          // B (K-major, SW128): rows of 128 B, 8-row atoms 1024 B apart; 16 k = 32 B along the row
          const uint64_t bd = stc_desc(x_base + kk * 32, 16, 1024);
          for (int h = 0; h < nh; ++h) {
            // A (MN-major, SW128): [64-column box][32 k][128 B]: k groups of 8 are 1024 B apart (SBO), the second box of
            // the half is 4096 B away (LBO); 16 k = two groups = 2048 B; the second k tile follows the first
            const uint32_t wa = w_base + (uint32_t)((kk >> 1) * (nh * 8192) + h * 8192 + (kk & 1) * 2048);
            const uint64_t ad = stc_desc(wa, 4096, 1024);
            stc_umma(tmem_base + (uint32_t)set * acc_cols + (uint32_t)h * 64, ad, bd, idesc, (seg_first && kk == 0) ? 0u : 1u);
          }
        }
        stc_commit(&empty[s]);   // frees the stage when these MMAs have read it
        seg_first = false;
        const bool seg_end = (k2 == KB2 - 1) || (u == u_end - 1);
        if (seg_end) {
          stc_commit(&acc_full[set]);
          STRC(2 + seg);   // 2..5: the MMAs of the CTA's groups are issued
          ++seg;
          seg_first = true;
        }
        if (++k2 == KB2) k2 = 0;
        if (++s == S) {
          s = 0;
          ++round;
        }
      }
    }
  } else if (w >= 4) {
    // ---------------- epilogue: warp (w - 4) owns TMEM lanes 32 (w - 4) .. + 31 = output columns of the group
    const int q = w - 4, et = tid - 128;
    const int max_contrib = a.max_contrib;
    int grp = u_begin / KB2, k2 = u_begin % KB2, seg = 0;
    bool dead = false;
    for (int u = u_begin; u < u_end;) {
      // this CTA's share of group `grp`: units up to the end of the group or of the CTA's range
      const int left_in_grp = KB2 - k2, left = u_end - u;
      const int n_units = left_in_grp < left ? left_in_grp : left;
      const int cur = grp;
      u += n_units;
      k2 += n_units;
      if (k2 == KB2) {
        k2 = 0;
        ++grp;
      }
      const int set = seg & 1;
      if (*(volatile int*)&s_err) dead = true;
      if (!mbar_wait(&acc_full[set], (unsigned)((seg >> 1) & 1), dead ? 4096u : kStcSpin)) {
        s_err = 1;
        dead = true;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (et == 0) STRC(8 + 4 * seg);    // accumulator complete
      const long long first_u = (long long)cur * KB2, last_u = first_u + KB2 - 1;
      const int c_first = (int)(((first_u + 1) * G + U - 1) / U - 1);
      const int c_last = (int)(((last_u + 1) * G + U - 1) / U - 1);
      const int n_contrib = c_last - c_first + 1;
      const int slot = blockIdx.x - c_first;
      float* mine = a.partials + (((size_t)cur * max_contrib + slot) * M) * TW;
      // The CTA's last group leaves through shared memory (the ring is idle once its MMAs have finished) and ONE bulk
      // store: its slot write is on the kernel's critical path, and 128 scalar stores per thread took 5 us there.
      const bool via_smem = u >= u_end;
      float* dst = via_smem ? reinterpret_cast<float*>(smem) : mine;
      for (int h = 0; h < nh; ++h) {
#pragma unroll 1
        for (int r0 = 0; r0 < kStcRows; r0 += 32) {
          uint32_t v[32];
          stc_tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)set * acc_cols + (uint32_t)h * 64 + (uint32_t)r0, v);
          // lane = column, register j = row r0 + j: for every row the warp stores 32 consecutive floats
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (r0 + j < M) dst[(size_t)(r0 + j) * TW + h * 128 + q * 32 + lane] = __uint_as_float(v[j]);
        }
      }
      if (via_smem) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the bulk store reads what these threads wrote
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[set]);   // the MMA thread may reuse the set
      if (et == 0) STRC(9 + 4 * seg);    // slot written
      ++seg;
      stc_epi_sync();
      if (et == 0) {
        if (via_smem) {
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(mine), "r"(stc_u32(smem)), "r"((unsigned)(M * TW * 4))
                       : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
          asm volatile("fence.proxy.async;" ::: "memory");   // the slot was written through the async proxy; the release below is generic
        }
        const unsigned int prev = stc_atom_add_acq_rel(&a.counters[cur], 1u);  // publishes this CTA's slot, acquires the others'
        const int last = (prev == (unsigned int)(n_contrib - 1));
        if (last) a.counters[cur] = 0u;
        s_last = last;
      }
      stc_epi_sync();
      if (et == 0) STRC(10 + 4 * (seg - 1));   // arrival counted
      // The CTA's last group is finished after the role loops by all eight warps (the producer and the MMA thread
      // are done by then): that reduction is the tail of the kernel.  Earlier groups overlap the MMAs of later ones.
      if (u >= u_end) {
        if (et == 0) {
          s_tail[0] = *(volatile int*)&s_last;
          s_tail[1] = cur;
          s_tail[2] = n_contrib;
        }
      } else if (*(volatile int*)&s_last) {
        stc_finish_group(a, cur, n_contrib, et, 128);
      }
      stc_epi_sync();  // s_last is rewritten at the next group's end
      if (et == 0) STRC(11 + 4 * (seg - 1));   // group finished (if this CTA was the last to arrive)
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (w == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
  }
  if (tid == 0) STRC(30);
  if (s_tail[0] && !*(volatile int*)&s_err) stc_finish_tail(a, s_tail[1], s_tail[2], smem, S * stage_bytes, tail_bar, &s_err, tid);
  if (tid == 0) STRC(31);
  if (tid == 0 && *(volatile int*)&s_err) {
    // copies in flight have a stage to land in until the CTA exits; give them (bounded) time
    for (int i = 0; i < S; ++i) mbar_wait(&full[i], 0u, 1u << 14), mbar_wait(&full[i], 1u, 1u << 14);
    g_stc_error = 1;
    if (a.error_flag) *a.error_flag = 1;
  }
}

// ---- host side ---------------------------------------------------------------------------------------------------------
typedef CUresult (*StcEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static StcEncodeTiledFn stc_get_encode() {
  static StcEncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<StcEncodeTiledFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

#ifdef TSB200_TRACE
int stc_read_trace(long long* host) { return cudaMemcpyFromSymbol(host, g_stc_trace, sizeof(long long) * 160 * 32) == cudaSuccess; }
#endif
int stc_take_error() {
  int e = 0;
  if (cudaMemcpyFromSymbol(&e, g_stc_error, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (e) {
    const int z = 0;
    cudaMemcpyToSymbol(g_stc_error, &z, sizeof(int));
  }
  return e;
}

// Column-group width and contributor bound for a matrix: whole column tiles when at most four CTAs then share one.
static void stc_geometry(int K, int N, int sm_count, int* nh, long long* grid, int* max_contrib) {
  const long long KB2 = ((K + kKT - 1) / kKT) / 2, CT = (N + 255) / 256;
  for (int h = 2; h >= 1; --h) {
    const long long groups = CT * (2 / h), U = KB2 * groups;
    long long g = sm_count;
    if (g > U) g = U;
    const long long per = U / (g > 0 ? g : 1);
    const long long mc = KB2 / (per > 0 ? per : 1) + 2;
    *nh = h;
    *grid = g;
    *max_contrib = (int)mc;
    if (mc <= 5) break;
  }
}

int64_t gemm_stream_tc_workspace_bytes(int M, int K, int N, int sm_count) {
  int nh, mc;
  long long g;
  stc_geometry(K, N, sm_count, &nh, &g, &mc);
  const long long groups = (long long)((N + 255) / 256) * (2 / nh);
  return kWsCounterBytes + groups * mc * M * (128 * nh) * 4 + 256;
}

// 1 ok, 0 error, 2 shape not handled (caller falls back).
int launch_gemm_stream_tc(int device, DeviceState* st, const void* x, const void* Wp, int M, int K, int N, const Epilogue& ep,
                          int* error_flag, bool pdl, void* ws, int64_t ws_bytes, cudaStream_t s) {
  {
    static int enabled = -1;
    if (enabled < 0) {
      const char* e = getenv("TSB200_GEMM_STC");  // "0": decode batches of 17..64 rows keep the mma.sync kernels (A/B measurements)
      enabled = (e && e[0] == '0') ? 0 : 1;
    }
    if (!enabled) return 2;
  }
  const int KB = (K + kKT - 1) / kKT;
  if (M < 17 || M > kStcRows || K % 64 != 0 || (KB & 1) || N % 8 != 0 || ((uintptr_t)x % 16) != 0 || ((uintptr_t)Wp % 16) != 0) return 2;
  StcEncodeTiledFn enc = stc_get_encode();
  if (!enc) return 2;
  StcArgs a{};
  a.Wp = reinterpret_cast<const unsigned char*>(Wp);
  a.M = M; a.K = K; a.N = N; a.KB = KB;
  a.CT = (N + 255) / 256;
  long long g;
  stc_geometry(K, N, st->sm_count, &a.nh, &g, &a.max_contrib);
  // The hand-over of partial sums at the end of the kernel costs about 10 us whatever the matrix: small matrices, short
  // K (measured at 32 rows, K = 2048: 29.7 against 26.5 us for N = 16384, 43.3 against 38.3 us for N = 32000) and narrow
  // matrices whose column groups are shared by many CTAs stay with the mma.sync kernels.
  if ((long long)K * N < (16LL << 20) || K < 4096 || a.max_contrib > 6) return 2;
  const long long groups = (long long)a.CT * (2 / a.nh);
  if (groups * 4 > kWsCounterBytes - 256) return 2;
  const int64_t need = kWsCounterBytes + groups * a.max_contrib * M * (128 * a.nh) * 4;
  if (!ws || ws_bytes < need) return 2;
  const size_t stage_bytes = (size_t)a.nh * 16384 + kStcXBytes;
  const size_t fixed = 40 * sizeof(uint64_t) + 1024 + 128;
  int stages = (int)((220 * 1024 - fixed) / stage_bytes);
  if (stages > 16) stages = 16;
  a.stages = stages;
  a.counters = reinterpret_cast<unsigned int*>(ws);
  a.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + kWsCounterBytes);
  a.error_flag = error_flag;
  a.ep = ep;
  CUtensorMap mapX;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)kStcRows};
    const cuuint32_t el[2] = {1, 1};
    const CUresult r = enc(&mapX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, el,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TSB_CHECK(r == CUDA_SUCCESS, "gemm_stream_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
  }
  const size_t smem = fixed + (size_t)stages * stage_bytes;
  static bool attr_done[kMaxDevices] = {};
  if (!attr_done[device]) {
    TSB_CUDA(cudaFuncSetAttribute(gemm_stream_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
    attr_done[device] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)g);
  cfg.blockDim = dim3(kStcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  TSB_CUDA(cudaLaunchKernelEx(&cfg, gemm_stream_tc_kernel, mapX, a));
  count_launch(device);
  return 1;
}

}  // namespace tsb

#ifdef TSB200_TRACE
extern "C" __attribute__((visibility("default"))) int TSB200_DebugStcTrace(long long* host) { return tsb::stc_read_trace(host); }
#endif
