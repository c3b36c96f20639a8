// Tensor-core GEMM for prefill and large-batch decode: y[M,N] = epilogue(x[M,K] * W[K,N]), fp16 in, fp32 accumulate.
//
// sm_100a design (5th-generation tensor cores):
//  * operands are staged in shared memory by TMA tensor copies (cp.async.bulk.tensor, 128-byte swizzle, completion
//    on mbarriers): A = activations [M,K] row-major (K-major operand, box 64 k x 128 rows); B = the engine's packed
//    weight tiles, which are stored pre-swizzled (packed_tile_off), so the 128 columns x 32 k a stage needs from a
//    tile are one contiguous 8 KB range that a plain bulk copy lands in operand layout (MN-major, SWIZZLE_128B):
//    decode GEMV and GEMM share ONE copy of the weights;
//  * one elected thread issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=128, K=16) with the accumulator in
//    tensor memory (TMEM, 128 lanes x 128 fp32 columns), tcgen05.commit hands shared-memory stages back to the
//    producer and signals the epilogue;
//  * four epilogue warps read the accumulator with tcgen05.ld (32 lanes x 32 columns per instruction) and apply the
//    same fused epilogue as the GEMV: bias first, activation, gate product on interleaved columns, fp32 residual;
//  * warp roles: 0 = TMA producer, 1 = MMA issuer, 2 = TMEM allocator, 4..7 = epilogue.
// Rows beyond M and K beyond the tensor are zero-filled by TMA, N is padded by the packed layout.
// Every mbarrier wait is bounded; on timeout an error word is raised, TMEM is freed and the kernel returns.
//
// Replaces cublasGemmEx (TensorSharp.CUDA/MatrixMul/CudaMatrixMulMM.cs:305-362, fp16 accumulate there) plus the bias
// copy, activation and residual kernels around it.
#include <cuda.h>

#include <cstdlib>

#include "kernels.cuh"

namespace tsb {

constexpr int kBM = 128, kBN = 128, kBK = 64;
constexpr int kTcStages = 3;   // 3 x 32 KB: two CTAs per SM, so one CTA's epilogue overlaps the other's mainloop
constexpr int kTcThreads = 256;
constexpr int kABytes = kBM * kBK * 2;  // 16 KB
constexpr int kBBytes = kBN * kBK * 2;  // 16 KB
constexpr unsigned kTcSpin = 1u << 22;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_u32(bar)), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tc_mbar_wait(uint64_t* bar, unsigned parity) {
  const uint32_t a = s_u32(bar);
  for (unsigned i = 0; i < kTcSpin; ++i) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(s_u32(dst)),
      "l"(map), "r"(s_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(s_u32(dst)),
               "l"(src), "r"(bytes), "r"(s_u32(bar))
               : "memory");
}
// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in 16-byte units,
// version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
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

// Raised by a kernel whose bounded wait ran out; read and cleared by tc_take_error().
__device__ int g_tc_error;

struct TcArgs {
  int M, N, K;        // logical sizes (N = packed column count actually used, multiple of 8)
  int KB;             // packed 32-row tiles along K
  int ksplit;         // CTAs sharing one output tile along K (grid.z); > 1 only when there are few tiles (small M)
  float* partials;    // [ksplit][M][Npad] raw fp32 accumulators, Npad = gridDim.x * 128
  unsigned int* counters;  // one per output tile, zero on entry, self-resetting
  int* error_flag;
  const unsigned char* Wp;  // packed weight tiles
  int vec_ok;               // pointers and sizes allow the 16-byte epilogue
  Epilogue ep;
};

// Fused epilogue for 32 consecutive columns of one row: bias first, activation, gate product on interleaved
// (a_j, g_j) column pairs, fp32 residual, store in fp16 or fp32.
__device__ __forceinline__ void tc_finish(const TcArgs& a, int row, int col0, const float* v) {
  const __half* bias = reinterpret_cast<const __half*>(a.ep.bias);
  if (!a.ep.glu) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int col = col0 + j;
      if (col < a.N) {
        float x = v[j] + (bias ? __half2float(bias[col]) : 0.0f);
        switch (a.ep.act) {
          case TSB200_ACT_RELU: x = x < 0.0f ? 0.0f : x; break;
          case TSB200_ACT_SILU: x = x / (1.0f + expf(-x)); break;
          case TSB200_ACT_LEAKYRELU: x = x < 0.0f ? 0.01f * x : x; break;
          case TSB200_ACT_GELU: x = 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); break;
          default: break;
        }
        const size_t o = (size_t)row * a.N + col;
        if (a.ep.residual) x += a.ep.residual[o];
        if (a.ep.y32) a.ep.y32[o] = x;
        else reinterpret_cast<__half*>(a.ep.y)[o] = __float2half_rn(x);
      }
    }
  } else {
    const int No = a.N / 2;
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const int col = col0 + j;
      if (col + 1 < a.N) {
        float av = v[j] + (bias ? __half2float(bias[col]) : 0.0f);
        const float gv = v[j + 1] + (bias ? __half2float(bias[col + 1]) : 0.0f);
        if (a.ep.act == TSB200_ACT_SWIGLU) av = av / (1.0f + expf(-av));
        float x = av * gv;
        const size_t o = (size_t)row * No + (col >> 1);
        if (a.ep.residual) x += a.ep.residual[o];
        if (a.ep.y32) a.ep.y32[o] = x;
        else reinterpret_cast<__half*>(a.ep.y)[o] = __float2half_rn(x);
      }
    }
  }
}

// The same epilogue for a full chunk of 32 columns when every pointer is 16-byte aligned and N is a multiple of 32
// (TcArgs::vec_ok): 16-byte loads of bias and residual, 16-byte stores, i.e. whole 32-byte sectors instead of one
// 2-byte store per element (scalar stores made the epilogue longer than the mainloop of a 128 x 256 x 4096 tile).
__device__ __forceinline__ float tc_act(float x, int act) {
  switch (act) {
    case TSB200_ACT_RELU: return x < 0.0f ? 0.0f : x;
    case TSB200_ACT_SILU: return x / (1.0f + expf(-x));
    case TSB200_ACT_LEAKYRELU: return x < 0.0f ? 0.01f * x : x;
    case TSB200_ACT_GELU: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
    default: return x;
  }
}
__device__ __forceinline__ void tc_finish_fast(const TcArgs& a, int row, int col0, const float* v) {
  float b[32];
  if (a.ep.bias) {
    const uint4* bp = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(a.ep.bias) + col0);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 t = bp[q];
      const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        b[q * 8 + 2 * i] = f.x;
        b[q * 8 + 2 * i + 1] = f.y;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) b[j] = 0.0f;
  }
  float x[32];
  int n_out;
  size_t o;
  if (!a.ep.glu) {
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = tc_act(v[j] + b[j], a.ep.act);
    n_out = 32;
    o = (size_t)row * a.N + col0;
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float av = v[2 * j] + b[2 * j];
      const float gv = v[2 * j + 1] + b[2 * j + 1];
      if (a.ep.act == TSB200_ACT_SWIGLU) av = av / (1.0f + expf(-av));
      x[j] = av * gv;
    }
    n_out = 16;
    o = (size_t)row * (a.N / 2) + (col0 >> 1);
  }
  if (a.ep.residual) {
    const float4* rp = reinterpret_cast<const float4*>(a.ep.residual + o);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (q * 4 < n_out) {
        const float4 t = rp[q];
        x[q * 4] += t.x; x[q * 4 + 1] += t.y; x[q * 4 + 2] += t.z; x[q * 4 + 3] += t.w;
      }
    }
  }
  if (a.ep.y32) {
    float4* yp = reinterpret_cast<float4*>(a.ep.y32 + o);
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (q * 4 < n_out) yp[q] = make_float4(x[q * 4], x[q * 4 + 1], x[q * 4 + 2], x[q * 4 + 3]);
  } else {
    uint4* yp = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.ep.y) + o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (q * 8 < n_out) {
        uint4 t;
        __half2* h = reinterpret_cast<__half2*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(x[q * 8 + 2 * i], x[q * 8 + 2 * i + 1]);
        yp[q] = t;
      }
    }
  }
}

__global__ void __launch_bounds__(kTcThreads, 2) gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, TcArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // carve: [stages][A 16K][B 16K] (1024-byte aligned for the 128B swizzle atoms), then barriers
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = smem;
  unsigned char* sB = smem + kTcStages * kABytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kTcStages * (kABytes + kBBytes));
  uint64_t* empty = full + kTcStages;
  uint64_t* acc_ready = empty + kTcStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  __shared__ int s_err;

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y;
  const int k_total = (a.K + kBK - 1) / kBK;
  const int k_per = (k_total + a.ksplit - 1) / a.ksplit;
  const int k_begin = blockIdx.z * k_per;
  const int k_iters = max(0, min(k_total, k_begin + k_per) - k_begin);  // k blocks of this CTA
  __shared__ int s_last;

  if (tid == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      tc_mbar_init(&full[s], 1);
      tc_mbar_init(&empty[s], 1);
    }
    tc_mbar_init(acc_ready, 1);
    s_err = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (w == 2) {  // TMEM allocation: 128 columns of fp32 accumulator (one warp, whole-warp instruction)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_u32(tmem_slot)), "r"(kBN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;

  if (w == 0 && lane == 0) {
    // ---------------- TMA producer
    // B: this CTA's 128 columns are boxes (2p, 2p+1) of column tile ct: 8 KB contiguous in every packed k tile
    const unsigned char* wsrc = a.Wp + ((size_t)(n_tile >> 1) * a.KB) * 16384 + (size_t)(n_tile & 1) * 8192;
    for (int it = 0; it < k_iters; ++it) {
      const int s = it % kTcStages, r = it / kTcStages;
      if (it >= kTcStages && !tc_mbar_wait(&empty[s], (unsigned)((r - 1) & 1))) {
        s_err = 1;
        break;
      }
      const int kb0 = (k_begin + it) * 2;
      const bool two = kb0 + 1 < a.KB;  // the last 64-k block of an odd tile count has one packed tile only
      tc_mbar_expect_tx(&full[s], kABytes + (two ? 16384 : 8192));
      tma_load_2d(sA + s * kABytes, &mapA, (k_begin + it) * kBK, m_tile * kBM, &full[s]);
      tc_bulk_g2s(sB + s * kBBytes, wsrc + (size_t)kb0 * 16384, 8192, &full[s]);
      if (two) tc_bulk_g2s(sB + s * kBBytes + 8192, wsrc + (size_t)(kb0 + 1) * 16384, 8192, &full[s]);
    }
  } else if (w == 1 && lane == 0) {
    // ---------------- MMA issuer
    // instruction descriptor: D fp32, A/B fp16, A K-major, B MN-major, N = 128, M = 128
    const uint32_t idesc = (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (1u << 16) | ((uint32_t)(kBN >> 3) << 17) |
                           ((uint32_t)(kBM >> 4) << 24);
    for (int it = 0; it < k_iters; ++it) {
      const int s = it % kTcStages, r = it / kTcStages;
      if (!tc_mbar_wait(&full[s], (unsigned)(r & 1))) {
        s_err = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_base = s_u32(sA + s * kABytes), b_base = s_u32(sB + s * kBBytes);
      const int kk_end = ((k_begin + it) * 2 + 1 < a.KB) ? 4 : 2;  // no second packed tile: its stage half was not filled
#pragma unroll
      for (int kk = 0; kk < kBK / 16; ++kk) {
        if (kk >= kk_end) break;
        // A (K-major, SW128): rows of 128 B, 8-row atoms 1024 B apart; 16 k = 32 B along the row
        const uint64_t ad = make_desc(a_base + kk * 32, 16, 1024);
        // B (MN-major, SW128), stage = [k tile 2][64-n box 2][32 k][128 B]: k groups of 8 are 1024 B apart (SBO), the
        // second 64-n box is 4096 B away (LBO); 16 k = two groups = 2048 B; the second k tile starts at 8192 B
        const uint64_t bd = make_desc(b_base + (kk >> 1) * 8192 + (kk & 1) * 2048, 4096, 1024);
        umma_f16(tmem_acc, ad, bd, idesc, (it > 0 || kk > 0) ? 1u : 0u);
      }
      umma_commit(&empty[s]);  // frees the stage when these MMAs have read it
    }
    umma_commit(acc_ready);    // accumulator complete
  } else if (w >= 4) {
    // ---------------- epilogue: warp (w - 4) owns TMEM lanes 32*(w-4) .. +31 = rows of the tile
    const int q = w - 4;
    const bool ok = tc_mbar_wait(acc_ready, 0);
    if (!ok) s_err = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int row = m_tile * kBM + q * 32 + lane;
    const int n0 = n_tile * kBN;
    const bool live = ok && row < a.M;
    const size_t Npad = (size_t)gridDim.x * kBN;
#pragma unroll 1
    for (int c = 0; c < kBN; c += 32) {
      uint32_t v[32];
      tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
      if (!live) continue;
      if (a.ksplit == 1) {
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
        if (a.vec_ok && n0 + c + 32 <= a.N) tc_finish_fast(a, row, n0 + c, f);
        else tc_finish(a, row, n0 + c, f);
      } else {
        // raw partial sums of this K slice; the last CTA of the tile adds the slices in a fixed order
        float4* dst = reinterpret_cast<float4*>(a.partials + ((size_t)blockIdx.z * a.M + row) * Npad + n0 + c);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          dst[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                               __uint_as_float(v[4 * j + 3]));
      }
    }
    if (a.ksplit > 1) {
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
      if (w == 4 && lane == 0) {
        const unsigned int tile = blockIdx.y * gridDim.x + blockIdx.x;
        const unsigned int prev = atomicAdd(&a.counters[tile], 1u);
        s_last = (prev == (unsigned int)(a.ksplit - 1));
        if (s_last) a.counters[tile] = 0u;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (s_last && live) {
        __threadfence();
#pragma unroll 1
        for (int c = 0; c < kBN; c += 32) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = 0.0f;
          // two K slices in flight per round trip, added in slice order (bitwise reproducible)
          int z = 0;
          for (; z + 1 < a.ksplit; z += 2) {
            const float4* s0 = reinterpret_cast<const float4*>(a.partials + ((size_t)z * a.M + row) * Npad + n0 + c);
            const float4* s1 = reinterpret_cast<const float4*>(a.partials + ((size_t)(z + 1) * a.M + row) * Npad + n0 + c);
            float4 t0[8], t1[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              t0[j] = __ldcg(s0 + j);
              t1[j] = __ldcg(s1 + j);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              f[4 * j] += t0[j].x; f[4 * j + 1] += t0[j].y; f[4 * j + 2] += t0[j].z; f[4 * j + 3] += t0[j].w;
              f[4 * j] += t1[j].x; f[4 * j + 1] += t1[j].y; f[4 * j + 2] += t1[j].z; f[4 * j + 3] += t1[j].w;
            }
          }
          for (; z < a.ksplit; ++z) {
            const float4* src = reinterpret_cast<const float4*>(a.partials + ((size_t)z * a.M + row) * Npad + n0 + c);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 t = __ldcg(src + j);
              f[4 * j] += t.x; f[4 * j + 1] += t.y; f[4 * j + 2] += t.z; f[4 * j + 3] += t.w;
            }
          }
          if (a.vec_ok && n0 + c + 32 <= a.N) tc_finish_fast(a, row, n0 + c, f);
          else tc_finish(a, row, n0 + c, f);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (w == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(kBN) : "memory");
  }
  if (tid == 0 && s_err) {
    g_tc_error = 1;
    if (a.error_flag) *a.error_flag = 1;
  }
}

// ---- persistent variant for large M ------------------------------------------------------------------------------------
// One CTA per SM walks output tiles of 128 rows x 256 columns (a whole packed column tile: the B stage of a 64-k
// block is two contiguous 16 KB packed tiles, two bulk copies).  Per flop this tile shape needs 0.75x the operand
// bytes of 128x128.  The fp32 accumulator (256 TMEM columns) is double buffered: the four epilogue warps drain tile
// i while the MMA thread is already accumulating tile i+1, and the TMA thread runs ahead through a 4-stage ring
// across tile boundaries.  Tiles are ordered in bands of kBandM row tiles so that the CTAs running at the same
// time share A and B tiles in L2.
constexpr int kP_BN = 256;
constexpr int kP_Stages = 4;
constexpr int kP_ABytes = kBM * kBK * 2;     // 16 KB
constexpr int kP_BBytes = kP_BN * kBK * 2;   // 32 KB = two packed tiles
constexpr int kBandM = 16;

struct TcTile {
  int m_tile, n_tile;
};
__device__ __forceinline__ TcTile tc_tile_of(int t, int m_tiles, int n_tiles) {
  // bands of kBandM row tiles; inside a band column-major (all rows of a column tile are neighbours in time)
  const int band_sz = kBandM * n_tiles;
  const int band = t / band_sz;
  const int rows_in_band = min(kBandM, m_tiles - band * kBandM);
  const int r = t - band * band_sz;
  TcTile o;
  o.n_tile = r / rows_in_band;
  o.m_tile = band * kBandM + r % rows_in_band;
  return o;
}

__global__ void __launch_bounds__(kTcThreads, 1) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap mapA, TcArgs a,
                                                                           int m_tiles, int n_tiles) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = smem;
  unsigned char* sB = smem + kP_Stages * kP_ABytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kP_Stages * (kP_ABytes + kP_BBytes));
  uint64_t* empty = full + kP_Stages;
  uint64_t* acc_full = empty + kP_Stages;   // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  __shared__ int s_err;

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int k_total = (a.K + kBK - 1) / kBK;
  const int n_total = m_tiles * n_tiles;

  if (tid == 0) {
    for (int s = 0; s < kP_Stages; ++s) {
      tc_mbar_init(&full[s], 1);
      tc_mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc_mbar_init(&acc_full[i], 1);
      tc_mbar_init(&acc_empty[i], 4);  // one arrival per epilogue warp
    }
    s_err = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (w == 2) {  // all 512 TMEM columns: two accumulators of 256
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (w == 0 && lane == 0) {
    // ---------------- TMA producer: runs ahead across tiles
    int it_g = 0;  // k blocks issued so far (ring position)
    for (int t = blockIdx.x; t < n_total && !s_err; t += gridDim.x) {
      const TcTile tl = tc_tile_of(t, m_tiles, n_tiles);
      const int it_begin = 0, it_end = k_total;
      const unsigned char* wsrc = a.Wp + ((size_t)tl.n_tile * a.KB) * 16384;
      for (int it = it_begin; it < it_end; ++it, ++it_g) {
        const int s = it_g % kP_Stages, r = it_g / kP_Stages;
        if (it_g >= kP_Stages && !tc_mbar_wait(&empty[s], (unsigned)((r - 1) & 1))) {
          s_err = 1;
          break;
        }
        const int kb0 = it * 2;
        const bool two = kb0 + 1 < a.KB;
        tc_mbar_expect_tx(&full[s], kP_ABytes + (two ? 32768 : 16384));
        tma_load_2d(sA + s * kP_ABytes, &mapA, it * kBK, tl.m_tile * kBM, &full[s]);
        tc_bulk_g2s(sB + s * kP_BBytes, wsrc + (size_t)kb0 * 16384, 16384, &full[s]);
        if (two) tc_bulk_g2s(sB + s * kP_BBytes + 16384, wsrc + (size_t)(kb0 + 1) * 16384, 16384, &full[s]);
      }
    }
  } else if (w == 1 && lane == 0) {
    // ---------------- MMA issuer
    // instruction descriptor: D fp32, A/B fp16, A K-major, B MN-major, N = 256, M = 128
    const uint32_t idesc = (1u << 4) | (1u << 16) | ((uint32_t)(kP_BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
    int it_g = 0, n_done = 0;
    for (int t = blockIdx.x; t < n_total && !s_err; t += gridDim.x, ++n_done) {
      const int buf = n_done & 1;
      if (n_done >= 2 && !tc_mbar_wait(&acc_empty[buf], (unsigned)(((n_done >> 1) - 1) & 1))) {
        s_err = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_acc = tmem_base + buf * kP_BN;
      const int it_begin = 0, it_end = k_total;
      for (int it = it_begin; it < it_end; ++it, ++it_g) {
        const int s = it_g % kP_Stages, r = it_g / kP_Stages;
        if (!tc_mbar_wait(&full[s], (unsigned)(r & 1))) {
          s_err = 1;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_base = s_u32(sA + s * kP_ABytes), b_base = s_u32(sB + s * kP_BBytes);
        const int kk_end = (it * 2 + 1 < a.KB) ? 4 : 2;
#pragma unroll
        for (int kk = 0; kk < kBK / 16; ++kk) {
          if (kk >= kk_end) break;
          const uint64_t ad = make_desc(a_base + kk * 32, 16, 1024);
          // B stage = [k tile 2][64-n box 4][32 k][128 B]: boxes 4096 B apart (LBO), 8-k groups 1024 B apart (SBO),
          // 16 k = 2048 B, the second k tile at 16384 B
          const uint64_t bd = make_desc(b_base + (kk >> 1) * 16384 + (kk & 1) * 2048, 4096, 1024);
          umma_f16(tmem_acc, ad, bd, idesc, (it > it_begin || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);
      }
      if (s_err) break;
      umma_commit(&acc_full[buf]);
    }
  } else if (w >= 4) {
    // ---------------- epilogue: warp (w - 4) owns TMEM lanes 32*(w-4) .. +31 = rows of the tile
    const int q = w - 4;
    int n_done = 0;
    for (int t = blockIdx.x; t < n_total; t += gridDim.x, ++n_done) {
      const TcTile tl = tc_tile_of(t, m_tiles, n_tiles);
      const int buf = n_done & 1;
      if (*(volatile int*)&s_err) break;
      if (!__all_sync(0xffffffffu, tc_mbar_wait(&acc_full[buf], (unsigned)((n_done >> 1) & 1)))) {  // warp-uniform outcome
        s_err = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = tl.m_tile * kBM + q * 32 + lane;
      const int n0 = tl.n_tile * kP_BN;
      const bool live = row < a.M;
#pragma unroll 1
      for (int c = 0; c < kP_BN; c += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * kP_BN + c), v);
        if (!live) continue;
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
        if (a.vec_ok && n0 + c + 32 <= a.N) tc_finish_fast(a, row, n0 + c, f);
        else tc_finish(a, row, n0 + c, f);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_u32(&acc_empty[buf])) : "memory");
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (w == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
  if (tid == 0 && s_err) {
    g_tc_error = 1;
    if (a.error_flag) *a.error_flag = 1;
  }
}

// ---- host side ---------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

int init_tc_attrs(int device) {
  static bool done[kMaxDevices] = {};
  if (done[device]) return 1;
  TSB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                kTcStages * (kABytes + kBBytes) + 1024 + 256));
  TSB_CUDA(cudaFuncSetAttribute(gemm_tc_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                kP_Stages * (kP_ABytes + kP_BBytes) + 1024 + 256));
  done[device] = true;
  return 1;
}

// 1 when a tensor-core GEMM on the current device gave up waiting since the last call (and clears the mark).
int tc_take_error() {
  int e = 0;
  if (cudaMemcpyFromSymbol(&e, g_tc_error, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (e) {
    const int z = 0;
    cudaMemcpyToSymbol(g_tc_error, &z, sizeof(int));
  }
  return e;
}

// Returns 1 ok, 0 error, 2 not handled (caller falls back to the generic kernel).
int64_t gemm_tc_workspace_bytes(int M, int N, int sm_count) {
  const int64_t tiles = (int64_t)((N + kBN - 1) / kBN) * ((M + kBM - 1) / kBM);
  if (tiles >= 2 * sm_count) return 0;
  // split-K partials of the 128 x 128 kernel
  const int64_t ks = (2 * sm_count + tiles - 1) / tiles;
  return 4096 + kWsCounterBytes + ks * M * (int64_t)((N + kBN - 1) / kBN) * kBN * 4;
}

int launch_gemm_tc(int device, DeviceState* st, const void* x, const void* Wp, int M, int K, int N, const Epilogue& ep,
                   int* error_flag, void* ws, int64_t ws_bytes, cudaStream_t s) {
  {
    static int enabled = -1;
    if (enabled < 0) {
      const char* e = getenv("TSB200_TC");  // "0" routes large-M linears to the CUDA-core fallback (A/B measurements)
      enabled = (e && e[0] == '0') ? 0 : 1;
    }
    if (!enabled) return 2;
  }
  if (K % 8 != 0 || ((uintptr_t)x % 16) != 0 || ((uintptr_t)Wp % 16) != 0) return 2;
  EncodeTiledFn enc = get_encode();
  if (!enc) return 2;
  TSB_TRY(init_tc_attrs(device));
  const int KB = (K + 31) / 32;
  CUtensorMap mapA;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBM};
    const cuuint32_t el[2] = {1, 1};
    const CUresult r = enc(&mapA, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, el,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TSB_CHECK(r == CUDA_SUCCESS, "gemm_tc: cuTensorMapEncodeTiled(A) failed with %d", (int)r);
  }
  TcArgs a{};
  a.M = M; a.N = N; a.K = K; a.KB = KB; a.error_flag = error_flag; a.ep = ep;
  a.Wp = reinterpret_cast<const unsigned char*>(Wp);
  {
    const uintptr_t al = (uintptr_t)ep.bias | (uintptr_t)ep.residual | (uintptr_t)ep.y | (uintptr_t)ep.y32;
    a.vec_ok = (N % 32 == 0) && (al % 16 == 0) ? 1 : 0;
  }
  {
    // large M: persistent 128 x 256 tiles with a double-buffered accumulator
    static int pers = -1;
    if (pers < 0) {
      const char* e = getenv("TSB200_TC_PERSISTENT");  // "0": one 128 x 128 tile per CTA for every M (A/B measurements)
      pers = (e && e[0] == '0') ? 0 : 1;
    }
    const int m_tiles = (M + kBM - 1) / kBM, n_tiles = (N + kP_BN - 1) / kP_BN;
    const int tiles = m_tiles * n_tiles;
    if (pers && tiles >= st->sm_count) {
      a.ksplit = 1;
      int g = st->sm_count;
      const size_t smem_p = kP_Stages * (kP_ABytes + kP_BBytes) + 1024 + 256;
      gemm_tc_persistent_kernel<<<g, kTcThreads, smem_p, s>>>(mapA, a, m_tiles, n_tiles);
      count_launch(device);
      return check_launch("gemm_tc_persistent");
    }
  }
  dim3 grid((N + kBN - 1) / kBN, (M + kBM - 1) / kBM, 1);
  TSB_CHECK(grid.y <= 65535, "gemm_tc: too many row tiles");
  // few output tiles (decode-sized M): share each tile's K range among several CTAs so that all SMs stream weights
  a.ksplit = 1;
  {
    const int64_t tiles = (int64_t)grid.x * grid.y;
    const int k_total = (K + kBK - 1) / kBK;
    // Only with a single row tile: from two row tiles on (M > 128) the tiles of a weight column block already share its
    // columns through L2 and the K slices' partial sums cost more than the idle SMs (512 x 4096 x 4096: 59.7 us with two
    // slices, 39.9 us without; 256 x 4096 x 6144: 79.8 against 41.4 us).
    if (tiles < st->sm_count && grid.y == 1 && k_total >= 8 && ws) {
      // about 1.5 CTAs per SM (two fit); every extra K slice costs the last arriver another partial to add
      int ks = (int)((3 * st->sm_count / 2 + tiles - 1) / tiles);
      if (ks > k_total / 4) ks = k_total / 4;
      if (ks > 6) ks = 6;
      if (ks > 1) {
        const int k_per = (k_total + ks - 1) / ks;
        ks = (k_total + k_per - 1) / k_per;  // no empty slice
        const int64_t cnt = kWsCounterBytes;
        const int64_t need = cnt + (int64_t)ks * M * grid.x * kBN * 4;
        if (ks > 1 && ws_bytes >= need) {
          a.ksplit = ks;
          a.counters = reinterpret_cast<unsigned int*>(ws);
          a.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + cnt);
          grid.z = ks;
        }
      }
    }
  }
  const size_t smem = kTcStages * (kABytes + kBBytes) + 1024 + 256;
  gemm_tc_kernel<<<grid, kTcThreads, smem, s>>>(mapA, a);
  count_launch(device);
  return check_launch("gemm_tc");
}

}  // namespace tsb
