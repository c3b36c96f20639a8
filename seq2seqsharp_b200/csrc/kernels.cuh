// Internal launchers shared between the C-ABI entry points and the GPT engine.
#pragma once
#include "common.cuh"

namespace tsb {

struct Epilogue {
  const void* bias;       // [N] in T, may be null
  const float* residual;  // [M, N_out] fp32, may be null
  void* y;                // [M, N_out] in T (when y32 is null)
  float* y32;             // [M, N_out] fp32
  int act;                // TSB200_ACT_*
  int glu;                // 1: columns are interleaved (a_j, g_j) pairs, out_j = act(a_j) * g_j, N_out = N/2
};

int launch_norm_residual(int device, DeviceState* st, int dtype, void* h, float* x, const void* delta, const void* gamma,
                         const void* beta, int norm_type, float eps, int M, int d, cudaStream_t s);
// `packed`: W is in the engine's tiled layout (see gemv_stream.cu) instead of row-major [K,N]
int launch_linear(int device, DeviceState* st, int dtype, const void* x, const void* W, int M, int K, int N,
                  const Epilogue& ep, void* ws, int64_t ws_bytes, cudaStream_t s, bool packed);
// streaming GEMV on packed weights, M <= 4; xmode 0: x is T [M,K]; 1/2: x is the fp32 residual stream and RMSNorm /
// LayerNorm (gamma, beta, eps) is applied as a prologue.  Returns 1 ok, 0 error, 2 shape not handled.
int launch_gemv_stream(int device, DeviceState* st, int dtype, const void* Wp, const void* x, int xmode, const void* gamma,
                       const void* beta, float eps, int M, int K, int N, const Epilogue& ep, int* error_flag, bool pdl, void* ws,
                       int64_t ws_bytes, cudaStream_t s);
int64_t stream_workspace_bytes(int dtype, int M, int K, int N, int sm_count);
// Every linear kernel keeps its (self-resetting, zero between launches) arrival counters in the first kWsCounterBytes
// of the workspace and its partial sums behind them, so that kernels of different shapes sharing one workspace never
// find another kernel's partial sums where they expect zeroed counters.  The stand-alone entry point keeps its error
// word in the last 256 bytes of the counter area.
constexpr int64_t kWsCounterBytes = 65536;

// ---- persistent decode-step kernel (decode_stack.cu): one launch runs a whole list of operations ---------------
struct StackOp {
  int type;               // 0 linear on packed weights, 1 rope + cache append + attention partials
  // linear
  int xmode;              // 0: x is T [M,K]; 1 / 2: RMSNorm / LayerNorm of the fp32 rows x
  const void* Wp;
  const void* x;
  const void* gamma;
  const void* beta;
  float eps;
  int K, N;
  Epilogue ep;
  // attention: q|k|v rows of the current token in `x` (row stride qkv_rs elements), this layer's cache, output
  // rows [M, H*hd] in T at ep.y
  void* cK;
  void* cV;
  // tensor parallelism (row-sharded linears): xsite >= 0: the finished column tiles are partial sums over this rank's
  // share of K; they are stored into every rank's exchange buffer `xsite` (slot = this rank) instead of ep.y32.
  // ssite >= 0 (norm prologue only): the input row is x + the sum over ranks of exchange buffer `ssite`, and CTA 0
  // stores that new residual row to x_out (a different buffer than x: other CTAs are still reading x).
  int xsite, ssite;
  float* x_out;
};
// Device step state of the GPT engine (ints), read by the kernels of a captured decode step:
//   [0] cache length (all sequences), [1] Philox step (all sequences), [2] output slot of this call,
//   [3] 1 when the sequences have their own lengths / steps, [4] where the per-sequence steps start,
//   [kStateLens + b] cache length of sequence b, [state[4] + b] its Philox step.
constexpr int kStateRagged = 3, kStateStepsAt = 4, kStateLens = 8;
#ifdef __CUDACC__
__device__ __forceinline__ int state_len(const int* st, int b, int fallback) {
  if (!st) return fallback;
  return st[kStateRagged] ? st[kStateLens + b] : st[0];
}
__device__ __forceinline__ int state_step(const int* st, int b, int fallback) {
  if (!st) return fallback;
  return st[kStateRagged] ? st[st[kStateStepsAt] + b] : st[1];
}
#endif
// ---- checked build (-DTSB200_CHECKED): device-side index / capacity checks.  A failing check never traps: it records its
// code in the translation unit's check word and SKIPS the access; the engine reads the words after every call
// (TSB200_GptCheckDevice, and together with the wait-limit word after each step) and fails the call with the code.
//   TSB_CHECKED_WORD(tag)            once per .cu that checks: the word and `int chk_take_<tag>()` (returns and clears it)
//   TSB_DEV_CHECK(cond, code, stmt)  inside a kernel: if cond is false, record code and run stmt (continue / return / break)
#ifdef TSB200_CHECKED
#define TSB_CHECKED_WORD(tag)                                                      \
  static __device__ int g_chk_word_##tag;                                          \
  int chk_take_##tag() {                                                           \
    int e = 0;                                                                     \
    if (cudaMemcpyFromSymbol(&e, g_chk_word_##tag, sizeof(int)) != cudaSuccess) {  \
      cudaGetLastError();                                                          \
      return 0;                                                                    \
    }                                                                              \
    if (e) {                                                                       \
      const int z = 0;                                                             \
      cudaMemcpyToSymbol(g_chk_word_##tag, &z, sizeof(int));                       \
    }                                                                              \
    return e;                                                                      \
  }
#define TSB_DEV_CHECK(tag, cond, code, stmt)        \
  if (!(cond)) {                                    \
    atomicCAS(&g_chk_word_##tag, 0, (int)(code));   \
    stmt;                                           \
  }
#else
#define TSB_CHECKED_WORD(tag)
#define TSB_DEV_CHECK(tag, cond, code, stmt)
#endif
int chk_take_engine();
int chk_take_attention();
int chk_take_moe();
int chk_take_sampling();

constexpr int kStackMaxRanks = 8;
constexpr int kStackXchSites = 4;     // exchange buffers: {out-projection, FFN down} x layer parity
constexpr int kStackXchRows = 8;      // rows per exchange slot
struct StackConfig {
  int dtype, M;           // M = sequences (1..4; up to 8 on the fp16 tensor-core kernel)
  int H, Hkv, hd, Tmax, qkv_rs, use_rope;
  const float2* rope_tab; // [Tmax, hd/2] cos/sin
  const int* dT;          // device word holding the cache length before this step
  // tensor parallelism inside the kernel: every rank's exchange region as mapped into this process (own included).
  // Region: [n_ops arrival counters (monotonic, one per operation)] at 0, [epoch word] at 16 KB - 4,
  // [kStackXchSites][ranks][kStackXchRows][d] fp32 from 16 KB.
  int tp_rank, tp_size, d;
  unsigned char* peer[kStackMaxRanks];
  unsigned poll_limit;    // 0: the kernel's default; else acquire-polls of a dependency counter before a CTA gives up
};
constexpr size_t kStackXchHeader = 16384;
// Sizes of the scratch areas launch_decode_stack() needs for a program (host copy of the ops).
void decode_stack_scratch(const StackConfig& c, const StackOp* ops, int n_ops, int sm_count, int64_t* partial_bytes,
                          int64_t* counter_bytes, int64_t* attn_part_bytes);
// 1 ok, 0 error, 2 when the program cannot run on this kernel (caller uses the per-op launches).
int launch_decode_stack(int device, DeviceState* st, const StackConfig& c, const StackOp* ops_dev, const StackOp* ops_host,
                        int n_ops, void* partials, void* counters, void* attn_part, int* error_flag,
                        long long* trace, bool pdl, cudaStream_t s);
int init_stack_attrs(int device);
// ---- owner-partitioned persistent decode step (decode_owner.cu): fp16, one GPU, up to four sequences ------------------
struct OwnDims;
struct OwnerModel;
struct OwnLayerPtrs {  // the engine's buffers of one layer (weights in the packed tile layout)
  const void *n1_g, *n1_b, *wqkv, *bqkv, *wo, *bo, *n2_g, *n2_b, *w1, *b1, *w2, *b2;
  void *cK, *cV;
};
int owner_applicable(const OwnDims& D, int dtype, int sm_count);
int owner_create(int device, DeviceState* st, const OwnDims& D, int norm_type, int act, int use_rope, float eps, int Tmax,
                 const OwnLayerPtrs* layers, const void* nf_g, const void* nf_b, const void* head_w, const void* head_b,
                 OwnerModel** out);
void owner_destroy(OwnerModel* m);
int owner_repack(OwnerModel* m, cudaStream_t s);
bool owner_packed(const OwnerModel* m);
void owner_invalidate(OwnerModel* m);
int owner_reset_counters(OwnerModel* m);
long long owner_stream_bytes(const OwnerModel* m);
// tensor parallelism: every rank's exchange region as mapped here (own included) and the byte offset of this kernel's part
struct OwnTp {
  int rank, size;
  unsigned char* peer[kStackMaxRanks];
  long long offset;
};
long long owner_xch_bytes(const OwnDims& D);   // size of that part
void owner_tp_failed(OwnerModel* m);           // after a failed tensor-parallel step: later launches are refused
int owner_launch(OwnerModel* m, DeviceState* st, int M, const float* x, float* logits, const float2* rope_tab, const int* dT,
                 int* error_flag, unsigned poll_limit, bool pdl, long long* trace, const OwnTp* tp, cudaStream_t s);
int init_owner_attrs();
int64_t packed_bytes(int dtype, int K, int N);
// Element offset of (k, c) inside one packed 16 KB tile (k < 32, c < tile columns).  fp32 tiles are plain
// [32 k][128 columns].  fp16 tiles are stored as the shared-memory image the tensor cores want: four 64-column
// boxes, each [32 k][128 bytes], the eight 16-byte units of a row XOR-ed with k & 7 (the SWIZZLE_128B pattern), so
// that ONE linear 16 KB bulk copy lands a tile ready for ldmatrix / tcgen05 descriptors without bank conflicts.
template <typename T>
__host__ __device__ __forceinline__ int packed_tile_off(int k, int c) {
  if (sizeof(T) == 2) return ((c >> 6) << 11) + (k << 6) + ((((c >> 3) & 7) ^ (k & 7)) << 3) + (c & 7);
  return k * 128 + c;
}
int packed_tile_cols(int dtype);
int launch_pack(int device, DeviceState* st, int dst_dtype, void* dst, int src_dtype, const void* src, int rows, int cols,
                int src_ld, int K, int c0, int cs, cudaStream_t s);
// NCCL binding (comm.cu)
int comm_all_reduce_f32(void* comm, float* buf, int64_t count, cudaStream_t s);
int comm_nranks(void* comm);
// peer-memory all-reduce for small messages (comm.cu)
float* comm_peer_buffer(void* comm, int64_t count);
int comm_peer_reduce(void* comm, float* x, int64_t count, int* error_flag, int sm_count, cudaStream_t s);
int comm_peer_take_error();
int comm_rank(void* comm);
int init_stream_attrs(int device);
// tcgen05/TMEM GEMM on packed fp16 weights (gemm_tc.cu): 1 ok, 0 error, 2 shape not handled
int launch_gemm_tc(int device, DeviceState* st, const void* x, const void* Wp, int M, int K, int N, const Epilogue& ep,
                   int* error_flag, void* ws, int64_t ws_bytes, cudaStream_t s);
int64_t gemm_tc_workspace_bytes(int M, int N, int sm_count);
// stream-K mma.sync GEMM for decode batches of up to 64 rows on packed fp16 weights (gemm_stream_mma.cu)
// mixture-of-experts feed-forward (ops_moe.cu): x32 += sum over the token's experts of score * W2_e act(W1_e h)
int launch_moe_ffn(int device, DeviceState* st, int dtype, float* x32, const void* h, const void* router_w, const void* router_b,
                   const void* W1, const void* W2, void* hidden, int* picks, float* scores, int rows, int d, int E, int k, int act,
                   cudaStream_t s);
// tcgen05 streaming GEMM for 17..64 rows (gemm_stream_tc.cu): the weights are the 128-row operand, the activation rows N
int launch_gemm_stream_tc(int device, DeviceState* st, const void* x, const void* Wp, int M, int K, int N, const Epilogue& ep,
                          int* error_flag, bool pdl, void* ws, int64_t ws_bytes, cudaStream_t s);
int64_t gemm_stream_tc_workspace_bytes(int M, int K, int N, int sm_count);
int stc_take_error();
// The packed q | k | v projection of a decode step (one new position per sequence) with RoPE and the cache append done by
// the linear's epilogue: q columns are rotated and go to the output rows, k columns are rotated and go to the K cache row of
// the sequence's position, v columns go to the V cache row - the arithmetic of rope_append_kernel (the value is rounded to the
// model type first, as when the linear stores it and a second kernel reads it back).
struct RopeFuse {
  void* cK;            // [sequences, Hkv, Tmax, hd]
  void* cV;
  int Hd, KVd, hd, Tmax;
  int use_rope;        // 0: append only
  int T0;              // cache length when `state` is null
  const int* state;    // device step state (per-sequence lengths), may be null
  const float2* tab;   // [Tmax, hd / 2] cos / sin
};
int launch_gemm_stream_mma_norm(int device, DeviceState* st, const float* x32, const void* gamma, const void* beta, int norm_type, float eps,
                                const void* Wp, int M, int K, int N, const Epilogue& ep, int* error_flag, bool pdl, void* ws, int64_t ws_bytes,
                                cudaStream_t s, const RopeFuse* rope = nullptr);
int launch_gemm_stream_mma(int device, DeviceState* st, const void* x, const void* Wp, int M, int K, int N, const Epilogue& ep,
                           int* error_flag, bool pdl, void* ws, int64_t ws_bytes, cudaStream_t s);
int64_t gemm_stream_mma_workspace_bytes(int M, int K, int N, int sm_count);
int gs_take_error();
int init_tc_attrs(int device);
int tc_take_error();
int64_t linear_workspace_bytes(int M, int K, int N);
int launch_attention(int device, DeviceState* st, int dtype, void* out, const void* q, int64_t q_rs, const void* cK,
                     const void* cV, int B, int S, int H, int Hkv, int hd, int T0, const int* dT0, int Tmax, int splits_hint,
                     void* ws, int64_t ws_bytes, cudaStream_t s);
int64_t attn_workspace_bytes(int B, int H, int hd, int T);
int attn_pick_splits(DeviceState* st, int dtype, int B, int H, int Hkv, int hd, int T);
int launch_rope_table(int device, DeviceState* st, float2* tab, int Tmax, int hd, double base, cudaStream_t s);
int launch_rope_append(int device, DeviceState* st, int dtype, void* q, const void* k, const void* v, int64_t q_rs,
                       int64_t kv_rs, void* cK, void* cV, int B, int S, int H, int Hkv, int hd, int T0, const int* dT0,
                       int Tmax, int use_rope, double base, const float2* tab, cudaStream_t s);
int launch_softmax_argmax(int device, DeviceState* st, int* out_ids, float* probs, const float* logits, int B, int V,
                          float temperature, int use_temp, const int* blocked_dev, int n_blocked, cudaStream_t s);
int launch_beam_topk(int device, DeviceState* st, int* out_ids, float* out_p, float* out_logp, float* probs, int rows, int V, int K,
                     cudaStream_t s);
int launch_topp(int device, DeviceState* st, int* out, const float* probs, int rows, int V, float topP, float repeatPenalty,
                const int* history, const int* history_len, int history_stride, const float* u, void* ws, cudaStream_t s);
int launch_philox(int device, float* u, int n, uint64_t seed, uint64_t seq_first, uint32_t step, const int* dstep,
                  cudaStream_t s);
int launch_synthetic(int device, DeviceState* st, void* data, int dtype, int64_t n, uint64_t seed, uint64_t name_hash,
                     float std, cudaStream_t s);
uint64_t fnv1a64(const char* s);
int init_linear_attrs(int device);
int init_topp_attrs(int device);

}  // namespace tsb
