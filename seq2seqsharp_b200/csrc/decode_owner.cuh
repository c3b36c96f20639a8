// Owner-partitioned persistent decode step (fp16, one GPU): geometry shared by the host planner, the weight re-packer
// and the kernel.
//
// The layer stack of a decode step is cut so that most dependencies stay inside one CTA or inside a small group of
// CTAs, and every CTA's weights form ONE contiguous byte stream in the order it consumes them:
//
//  * attention block (one grid-wide dependency per layer): the CTAs are divided into one group per KV head.  A group
//    computes the q/k/v columns of its heads (each CTA a range of K, partial sums meet in a group accumulator),
//    runs RoPE + cache append + attention for its heads (each CTA a range of the cached tokens, partial softmax states
//    meet in a group buffer) and multiplies the attention output of its heads with its rows of W0 (each CTA a range
//    of output columns).  Two group-wide waits (18-19 CTAs) replace three grid-wide ones;
//  * FFN block (one grid-wide dependency per layer): every CTA owns a slice of the hidden units: it computes
//    act(x W1 + b1) (.) (x W3 + b3) for its slice over the full K, keeps the slice in shared memory and multiplies it
//    at once with the matching rows of W2;
//  * sums that cross CTAs (group q/k/v accumulator, the residual stream) are accumulated with 64-bit integer atomics
//    on fixed-point values (2^-28 resolution), so the result does not depend on the order of arrival: bitwise
//    reproducible without a fixed-order exchange, and the residual add costs nothing extra;
//  * the LM head is split by columns only.
//
// Weight blocks: a block is the A operand of ONE mma.sync m16n8k16 (16 output columns x 16 k, fp16) stored in
// fragment order: lane l = (g = l / 4, t = l % 4) finds its eight values {W[k0+2t+{0,1}][c0+g], W[..][c0+g+8],
// W[k0+2t+8+{0,1}][c0+g], W[..][c0+g+8]} in 16 consecutive bytes, so a warp loads a block with one conflict-free
// 16-byte shared-memory load per lane.  Eight blocks (one per consumer warp) form a 4 KB row; eight rows a 32 KB tile
// of the TMA ring.  Rows of all jobs of a CTA follow each other without gaps.
//
// Replaces, per decode step, the chain LayerNorm/RMSNorm -> Affine(QKV) -> RoPE -> cache concat -> softmax(QK^T)V ->
// Affine(W0) + residual -> norm -> Affine(W1[,W3]) -> activation/gate -> Affine(W2) + residual of
// Seq2SeqSharp/Layers/MultiHeadAttention.cs:125-240, Layers/GroupQueryAttention.cs:114-233 and
// Layers/PositionwiseFeedForward.cs:72-116, and the LM head of Applications/Decoder.cs:705-716.
#pragma once
#include <stdint.h>

#ifndef __CUDACC__
#ifndef __host__
#define __host__
#define __device__
#define __forceinline__ inline
#endif
#endif

namespace tsb {

constexpr int kOwnBlockBytes = 512;       // one mma A operand (16 columns x 16 k, fp16)
constexpr int kOwnRowBytes = 4096;        // eight blocks, one per consumer warp
constexpr int kOwnTileRows = 8;           // rows per stage of the ring (a power of two)
constexpr int kOwnTileShift = 3;
constexpr int kOwnTileBytes = kOwnTileRows * kOwnRowBytes;   // 32 KB: half as many barrier hand-shakes per byte as 16 KB
constexpr int kOwnKChunk = 8;             // K-split jobs: at most this many strips are accumulated per pass (8 x 4 registers)
constexpr int kOwnMaxSpw = 8;             // strip-split jobs: strips per warp per pass
constexpr int kOwnMaxRows = 4;            // sequences per launch
constexpr int kOwnFixShift = 28;          // fixed point: value * 2^28 in a signed 64-bit integer

enum OwnJobKind { OWN_QKV = 0, OWN_W0 = 1, OWN_UP = 2, OWN_DOWN = 3, OWN_HEAD = 4 };
enum OwnJobMode { OWN_KSPLIT = 0, OWN_SSPLIT = 1 };

// One CTA's share of one linear: `ks` k-steps (of 16) x `ws` strips (of 16 columns) of the matrix.
//  K-split mode: warp w owns k-steps [w*ksw, (w+1)*ksw) of the job and all strips; strips are taken in nchunks passes of
//    nearly equal width (at most kOwnKChunk); rows are ordered (chunk, kk, strip).  The eight warps' sums meet in shared
//    memory.
//  strip-split mode: warp w owns `spw` strips per chunk of 8*spw strips and all k-steps; rows are ordered
//    (chunk, k-step, j).  A warp holds complete sums of its strips.
// In both modes the block of warp w in a row sits at byte w * 512 of the row; blocks outside the job are zero.
struct OwnJob {
  long long row0;     // first row of the job in this CTA's stream
  int kind, mode;
  int ks, ws;         // k-steps and strips of this CTA's share (may be 0)
  int kbase, cbase;   // first k and first column of the share in the source matrix (QKV: column base unused)
  int ksw;            // K-split: k-steps per warp = ceil(ks / 8)
  int spw;            // strip-split: strips per warp per chunk
  int nchunks;
  int nrows;          // rows of the job
  int group;          // attention jobs: KV head of this CTA's group
  int pad;
};

__host__ __device__ __forceinline__ int own_ceil(int a, int b) { return (a + b - 1) / b; }
// K-split jobs take their ws strips in nchunks = ceil(ws / kOwnKChunk) passes of nearly equal width
__host__ __device__ __forceinline__ int own_chunk_width(int ws, int nchunks, int c) { return ws / nchunks + (c < ws % nchunks ? 1 : 0); }
__host__ __device__ __forceinline__ int own_chunk_start(int ws, int nchunks, int c) {
  const int r = ws % nchunks;
  return c * (ws / nchunks) + (c < r ? c : r);
}

// Fills mode-dependent fields of a job whose kind / ks / ws / bases are set.
__host__ __device__ __forceinline__ void own_job_finish(OwnJob& j, int mode) {
  j.mode = mode;
  j.ksw = 0;
  j.spw = 0;
  j.nchunks = 0;
  j.nrows = 0;
  if (j.ks <= 0 || j.ws <= 0) {
    j.ks = j.ws = 0;
    return;
  }
  if (mode == OWN_KSPLIT) {
    j.ksw = own_ceil(j.ks, 8);
    j.nchunks = own_ceil(j.ws, kOwnKChunk);
    j.nrows = j.ksw * j.ws;
  } else {
    j.spw = own_ceil(j.ws, 8);
    if (j.spw > kOwnMaxSpw) j.spw = kOwnMaxSpw;
    j.nchunks = own_ceil(j.ws, 8 * j.spw);
    j.nrows = j.nchunks * j.ks * j.spw;
  }
}

// The (k-step, strip) of the block that warp `w` finds in row `row` of the job (both relative to the job); `live` is
// false for the zero blocks that pad the job to whole rows.
__host__ __device__ __forceinline__ void own_block_coords(const OwnJob& j, int row, int w, int& kstep, int& strip, bool& live) {
  if (j.mode == OWN_KSPLIT) {
    // rows: for chunk c, for kk < ksw, for s < width(c)
    int c = 0, r = row;
    for (;;) {
      const int wc = own_chunk_width(j.ws, j.nchunks, c);
      if (r < j.ksw * wc) {
        const int kk = r / wc, s = r % wc;
        kstep = w * j.ksw + kk;
        strip = own_chunk_start(j.ws, j.nchunks, c) + s;
        break;
      }
      r -= j.ksw * wc;
      ++c;
    }
    live = kstep < j.ks;
  } else {
    const int per_chunk = j.ks * j.spw;
    const int c = row / per_chunk, r = row % per_chunk;
    kstep = r / j.spw;
    strip = c * 8 * j.spw + w * j.spw + (r % j.spw);
    live = strip < j.ws;
  }
}

// Geometry of the q|k|v columns of one KV-head group inside the packed QKV matrix [d, (H + 2 Hkv) hd]: group-local
// column j (0 .. (grp + 2) hd) -> matrix column.
__host__ __device__ __forceinline__ int own_qkv_col(int j, int g, int grp, int hd, int H, int Hkv) {
  if (j < grp * hd) return g * grp * hd + j;
  if (j < (grp + 1) * hd) return H * hd + g * hd + (j - grp * hd);
  return (H + Hkv) * hd + g * hd + (j - (grp + 1) * hd);
}

// Element e (0..7) of lane l of a block <-> (k, column) inside the 16 x 16 block (the mma.m16n8k16 A fragment with the
// output columns as rows).
__host__ __device__ __forceinline__ void own_frag_coords(int lane, int e, int& k, int& c) {
  const int g = lane >> 2, t = lane & 3;
  k = 2 * t + (e & 1) + ((e >> 2) << 3);
  c = g + (((e >> 1) & 1) << 3);
}

// CTA ranges: CTAs [own_group_begin(g), own_group_begin(g+1)) serve KV head g.
__host__ __device__ __forceinline__ int own_group_begin(int g, int G, int Hkv) { return (int)((long long)g * G / Hkv); }
// even split of n items over parts: item range of part i
__host__ __device__ __forceinline__ int own_split(int n, int parts, int i) { return (int)((long long)n * i / parts); }

struct OwnDims {
  int L, d, H, Hkv, hd, F, V, glu;
};

// Jobs of CTA `c` (of G) for layer-independent geometry: fills five jobs (QKV, W0, UP, DOWN of a layer; HEAD).
// row0 fields are left to the caller.
__host__ __device__ inline void own_plan_cta(const OwnDims& D, int G, int c, OwnJob out[5]) {
  const int grp = D.H / D.Hkv;
  int g = 0;
  while (g + 1 < D.Hkv && own_group_begin(g + 1, G, D.Hkv) <= c) ++g;
  const int gb = own_group_begin(g, G, D.Hkv), ge = own_group_begin(g + 1, G, D.Hkv);
  const int gsz = ge - gb, i = c - gb;
  const int KS = D.d / 16, DS = D.d / 16;
  for (int q = 0; q < 5; ++q) {
    out[q] = OwnJob{};
    out[q].kind = q;
    out[q].group = g;
  }
  // q|k|v of the group: a range of K, all (grp + 2) hd columns
  {
    OwnJob& j = out[OWN_QKV];
    const int k0 = own_split(KS, gsz, i), k1 = own_split(KS, gsz, i + 1);
    j.ks = k1 - k0;
    j.ws = (grp + 2) * D.hd / 16;
    j.kbase = k0 * 16;
    j.cbase = 0;
    own_job_finish(j, OWN_SSPLIT);
  }
  // W0 rows of the group's heads, a range of the d output columns
  {
    OwnJob& j = out[OWN_W0];
    const int s0 = own_split(DS, gsz, i), s1 = own_split(DS, gsz, i + 1);
    j.ks = grp * D.hd / 16;
    j.ws = s1 - s0;
    j.kbase = g * grp * D.hd;
    j.cbase = s0 * 16;
    own_job_finish(j, OWN_KSPLIT);
  }
  // FFN: units of 16 hidden columns
  const int units = D.F / 16;
  const int u0 = own_split(units, G, c), u1 = own_split(units, G, c + 1);
  {
    OwnJob& j = out[OWN_UP];
    j.ks = KS;
    j.ws = (u1 - u0) * (D.glu ? 2 : 1);
    j.kbase = 0;
    j.cbase = u0 * 16 * (D.glu ? 2 : 1);
    own_job_finish(j, OWN_KSPLIT);
  }
  {
    OwnJob& j = out[OWN_DOWN];
    j.ks = u1 - u0;
    j.ws = DS;
    j.kbase = u0 * 16;
    j.cbase = 0;
    own_job_finish(j, OWN_SSPLIT);
  }
  {
    OwnJob& j = out[OWN_HEAD];
    const int VS = own_ceil(D.V, 16);
    const int s0 = own_split(VS, G, c), s1 = own_split(VS, G, c + 1);
    j.ks = KS;
    j.ws = s1 - s0;
    j.kbase = 0;
    j.cbase = s0 * 16;
    own_job_finish(j, OWN_KSPLIT);
  }
}

}  // namespace tsb
