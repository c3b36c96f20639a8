// GPT engine: the token loop of GPT.RunForwardOnSingleDevice / Decoder.GPTDecode / GPTDecoder.Decode
// (Seq2SeqSharp/Applications/GPT.cs:212-335, Applications/Decoder.cs:648-794, Networks/GPTDecoder.cs:153-191)
// on one device, built from the fused kernels of this library.
//
// Differences from the reference's execution model, none of which change results beyond float rounding:
//  * weights are packed at load time: GQA's separate Q/K/V matrices become one [d, (H+2Hkv)hd] matrix (one
//    GEMV/GEMM instead of three), and for the gated FFN W1/W3 are interleaved column-wise so the gate product is
//    an epilogue;
//  * the KV cache is pre-sized and appended in place ([B, Hkv, Tmax, hd], un-expanded for GQA) instead of being
//    re-allocated and re-copied per step (Layers/MultiHeadAttention.cs:173-193);
//  * the residual stream is kept in fp32; matmul inputs/outputs are in the model dtype; accumulation is fp32;
//  * a decode step is one CUDA graph: the cache length and the step counter live in device memory so the same
//    graph is replayed for every token, sampled ids are fed back on the device, and the host reads ids only
//    when asked (every step only if it must test the reference's stop rule, GPT.cs:300-303).
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "decode_owner.cuh"
#include "kernels.cuh"
#include <nvtx3/nvToolsExt.h>   // header-only: ranges cost a pointer test unless a profiler has injected itself

namespace tsb {

// NVTX range for the lifetime of the object: every engine entry point and the phases of a forward pass carry one, so a
// timeline (Nsight Systems) shows prefill / decode / step / cache and beam operations by name.
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

TSB_CHECKED_WORD(engine)
#ifndef TSB200_CHECKED
int chk_take_engine() { return 0; }
#endif

template <typename T>
__global__ void embed_kernel(float* x, const T* E, const T* PE, const int* ids,
                             int rows, int S, int d, int V, float sf, int pe_mode, int pe_rows, int T0_arg,
                             const int* dT0) {
  pdl_trigger();
  pdl_wait();
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    int id = ids[r];
    TSB_DEV_CHECK(engine, id >= 0 && id < V, 0x101, (void)0)          // token id outside the vocabulary (the row is embedded as id 0)
    if (id < 0 || id >= V) id = 0;
    const int s = r % S;
    const int T0 = state_len(dT0, r / S, T0_arg);
    int pos = (pe_mode == 1) ? s : T0 + s;  // pe_mode 1: the reference peeks APE rows [0, S) (PositionEmbedding.cs:30-33)
    TSB_DEV_CHECK(engine, pe_mode == 0 || pos < pe_rows, 0x102, (void)0)   // position beyond the position table (clamped)
    if (pos >= pe_rows) pos = pe_rows - 1;
    const T* e = E + (int64_t)id * d;
    const T* p = (pe_mode != 0) ? PE + (int64_t)pos * d : nullptr;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float v = to_f<T>(e[i]) * sf;
      if (p) v += to_f<T>(p[i]);
      x[(int64_t)r * d + i] = v;
    }
  }
}

// last prompt row of every sequence; `lens` (device, or NULL): prompts of different lengths padded to S columns
__global__ void gather_last_kernel(float* xl, const float* x, int B, int S, int d, const int* lens) {
  for (int b = blockIdx.x; b < B; b += gridDim.x) {
    int last = lens ? lens[b] - 1 : S - 1;
    last = last < 0 ? 0 : (last >= S ? S - 1 : last);
    for (int i = threadIdx.x; i < d; i += blockDim.x) xl[(int64_t)b * d + i] = x[((int64_t)b * S + last) * d + i];
  }
}

// state: the device step state (kernels.cuh).  The per-sequence pointers (ids, history, out) address sequence b0 + b of
// the engine at index b.  stop_fin (sequences with their own lengths only): a sequence whose previous id was </s> (0)
// has finished: it keeps emitting 0 and neither its history nor its cache length nor its Philox step advance.
__global__ void commit_kernel(int* ids_cur, const int* ids_new, int* hist,
                              int* hist_len, int hist_stride, int* out, int B, int* state,
                              int advance_T, int b0, int stop_fin) {
  pdl_trigger();
  pdl_wait();
  const int slot = state[2];
  const bool ragged = state[kStateRagged] != 0;
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    int id = ids_new[b];
    const bool fin = ragged && stop_fin && ids_cur[b] == 0;
    if (fin) id = 0;
    ids_cur[b] = id;
    out[(int64_t)slot * B + b] = id;
    if (fin) continue;
    const int l = hist_len[b];
    TSB_DEV_CHECK(engine, l >= 0 && l < hist_stride, 0x103, (void)0)   // token history full (the id is not recorded)
    if (l < hist_stride) hist[(int64_t)b * hist_stride + l] = id;
    hist_len[b] = l + 1;
    if (ragged) {
      if (advance_T) state[kStateLens + b0 + b] += 1;
      state[state[kStateStepsAt] + b0 + b] += 1;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (advance_T) state[0] += 1;
    state[1] += 1;
    state[2] = slot + 1;
  }
}

// x += delta, after the all-reduce of a row-parallel layer's partial sums (tensor parallelism)
__global__ void residual_add_kernel(float* x, const float* delta, int64_t n) {
  pdl_trigger();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) x[i] += delta[i];
}

template <typename T>
__global__ void fill_const_kernel(T* p, int64_t n, float v) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = from_f<T>(v);
}

struct LayerW {
  void *n1_g = nullptr, *n1_b = nullptr, *wqkv = nullptr, *bqkv = nullptr, *wo = nullptr, *bo = nullptr;
  void *n2_g = nullptr, *n2_b = nullptr, *w1 = nullptr, *b1 = nullptr, *w2 = nullptr, *b2 = nullptr;
  void *cK = nullptr, *cV = nullptr;
  // mixture-of-experts layers (Layers/MoEFeedForward.cs): the layer's LayerNorm, router [d, E] + bias, experts [E, d, 4d] and
  // [E, 4d, d], row-major in the model type.  n2_g / n2_b / w1 / w2 are unused there.
  bool moe = false;
  void *moe_g = nullptr, *moe_b = nullptr, *router_w = nullptr, *router_b = nullptr, *moe_w1 = nullptr, *moe_w2 = nullptr;
  // cross-attention of encoder-decoder models (Layers/MultiHeadAttention.cs:434-527): norm of the query side, Q / K / V / out
  // projections (packed like the other matrices) and the K / V rows of the encoder output [max_batch, H, max_src_tokens, hd]
  void *nx_g = nullptr, *nx_b = nullptr, *xq = nullptr, *xqb = nullptr, *xk = nullptr, *xkb = nullptr, *xv = nullptr, *xvb = nullptr;
  void *xo = nullptr, *xob = nullptr, *xK = nullptr, *xV = nullptr;
};

struct Dest {  // where a logical tensor lives inside the engine's buffers
  void* base = nullptr;
  int64_t rows = 0, cols = 0, row_stride = 0, col_stride = 1;
  // matrices of linear layers live in the tiled layout of gemv_stream.cu: logical column j -> packed column c0 + j*cs
  bool packed = false;
  int64_t c0 = 0, cs = 1;
  // tensor parallelism: the caller hands over the FULL tensor [full_rows, full_cols]; this rank keeps the block that
  // starts at (sr0, sc0).  skip: the tensor belongs to another rank entirely (bias of a row-parallel layer).
  int64_t full_rows = 0, full_cols = 0, sr0 = 0, sc0 = 0;
  bool skip = false;
};

struct GraphKey {
  int B = -1, strategy = -1, splits = -1, n_blocked = -1, ragged = -1, stop_fin = -1;
  float topP = 0, temperature = 0, penalty = 0;
  uint64_t seed = 0, seq_base = 0, blocked_hash = 0;
  bool operator==(const GraphKey& o) const {
    return B == o.B && strategy == o.strategy && splits == o.splits && n_blocked == o.n_blocked && ragged == o.ragged &&
           stop_fin == o.stop_fin && topP == o.topP &&
           temperature == o.temperature && penalty == o.penalty && seed == o.seed && seq_base == o.seq_base &&
           blocked_hash == o.blocked_hash;
  }
};

struct Gpt {
  TSB200GptConfig c;
  DeviceState* st = nullptr;
  cudaStream_t s = nullptr;
  int es = 4;  // element size of the model dtype
  int Nqkv = 0, glu = 0;
  int tp = 1, tp_rank = 0;     // tensor-parallel degree and rank; c.H / c.Hkv / c.F hold this rank's share
  int fullH = 0, fullHkv = 0, fullF = 0;
  void* comm = nullptr;        // communicator for the two all-reduces per layer (TSB200_GptSetComm)
  bool tp_peer = true;         // use the peer-memory all-reduce when the communicator has one (TSB200_TP_PEER=0: NCCL only)
  // exchange region of the persistent decode-step kernel under tensor parallelism (TSB200_GptTpExport / Import)
  unsigned char* xch_region = nullptr;
  size_t xch_bytes = 0;
  unsigned char* xch_peer[kStackMaxRanks] = {};
  bool xch_open[kStackMaxRanks] = {};
  bool xch_ready = false;
  size_t xch_own_off = 0;      // where the owner-partitioned kernel's part of the region starts
  bool lin_syms_used = false;  // a kernel that reports errors through its own symbol ran since the last check
  bool graph_lin_syms = false; // ... and the captured decode step contains such kernels (every replay sets the flag above)
  int last_path = 0;           // how the most recent cached decode step ran: 0 one launch per operation, 1 stream-K persistent kernel, 2 owner-partitioned kernel
  float* x2 = nullptr;         // second residual buffer: a summed residual row is written to the buffer the others do not read
  float* ar_buf = nullptr;     // fp32 [rows, d] partial sums handed to the all-reduce
  void *E = nullptr, *PE = nullptr, *nf_g = nullptr, *nf_b = nullptr, *head_w = nullptr, *head_b = nullptr;
  int pe_rows = 0;
  std::vector<LayerW> L;
  float2* rope_tab = nullptr;
  // activations
  int64_t act_rows = 0;
  float* x = nullptr;
  void *h = nullptr, *qkv = nullptr, *attn = nullptr, *ffn = nullptr;
  float* xl = nullptr;
  void* hl = nullptr;
  // beam search: candidate scratch [max_batch][kMaxBeam] (ids, probabilities, log probabilities), the table of the layers'
  // cache pointers and the (source, destination) pairs of a sequence copy
  int* cross_state = nullptr;     // lengths of the encoder outputs in the layout of the step state (flag at [3], lengths from [8])
  int cross_T = 0;                // longest encoder output of the current call (0: none set)
  int* beam_ids = nullptr;
  float* beam_p = nullptr;
  void** beam_layers = nullptr;   // [2 * L]: K cache, V cache of layer 0, 1, ...
  int* beam_pairs = nullptr;      // [2 * max_batch]
  int* moe_picks = nullptr;      // [rows, experts_per_token] experts chosen by the router, ascending per token
  float* moe_scores = nullptr;   // their router probabilities
  float *logits = nullptr, *probs = nullptr, *u = nullptr;
  int *ids_in = nullptr, *ids_cur = nullptr, *ids_new = nullptr, *hist = nullptr, *hist_len = nullptr, *blocked = nullptr;
  int* state = nullptr;
  int* out_dev = nullptr;
  void *lin_ws = nullptr, *attn_ws = nullptr, *topp_ws = nullptr;
  int64_t lin_ws_bytes = 0, attn_ws_bytes = 0, topp_ws_bytes = 0;
  int n_blocked = 0, blocked_cap = 0;
  int B = 0, T = 0;            // sequences in the cache; cache length (the longest sequence's when they differ)
  uint32_t step = 0;           // Philox step of the next sampled token (the largest when they differ)
  // sequences with their own cache lengths / Philox steps (ragged prompts, refilled slots): host mirrors of the device
  // arrays.  While all sequences agree, `ragged` is false and the kernels read the scalars.
  std::vector<int> Ts, steps_v;
  bool ragged = false;
  bool force_per_seq = false;  // keep the per-sequence state in use even while the sequences agree (TSB200_GptSetPerSequenceState)
  int stop_fin = 0;            // per-sequence stop rule in the captured step (ragged decode with stop_on_eos)
  int seq0 = 0;                // first sequence the per-sequence buffers address (a single-slot prompt run), else 0
  const int* gather_lens = nullptr;   // device prompt lengths of a padded prefill (NULL: every prompt fills its S columns)
  bool probs_valid = false;
  // graph
  cudaGraphExec_t gexec = nullptr;
  GraphKey gkey;
  long long graph_nodes = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  float last_ms = 0.0f;
  long long last_launches = 0;
  // every device buffer of the engine sits between two guard regions of kGuardBytes filled with kGuardByte; a kernel that
  // writes past either end of a buffer changes them, and TSB200_GptCheckGuards finds out
  struct Alloc { void* user; void* base; size_t bytes; };
  std::vector<Alloc> allocs;
  // instrumentation (TSB200_GptProfileDecode): events around every launch group, by kernel class
  bool prof = false;
  std::vector<cudaEvent_t> prof_ev;
  std::vector<int> prof_cls, prof_cnt;   // class and number of launches of every timed run
  bool prof_open = false;
  int prof_open_cls = 0, prof_open_cnt = 0;
  size_t prof_n = 0;
  // per-step events of the last GptDecode (TSB200_GptEnableStepTiming)
  bool step_timing = false;
  std::vector<cudaEvent_t> step_ev;
  int step_ev_n = 0;
  int* pin_ids = nullptr;  // pinned host staging for TSB200_GptStepHost
  int* err_flag = nullptr; // device word raised by a kernel whose bounded wait ran out
  bool pdl = true;         // programmatic dependent launch between the kernels of a decode step
  // persistent decode-step kernel (decode_stack.cu): the program of operations and its scratch
  bool use_stack = true;
  bool fuse_step = true;       // per-operation path, up to eight rows: norm (and RoPE + cache append) inside the linear's launch
                               // (TSB200_FUSED_STEP=0: separate norm / RoPE-append launches, e.g. for a checker engine)
  // Measured crossover on the 7B-class model (ms per step, persistent kernel against one launch per operation with the
  // mma.sync linears): 1 sequence 3.41 / 3.95, 2 sequences 3.79 / 3.92, 3 sequences 4.23 / 3.91, 4 sequences 4.62 / 3.96 --
  // the persistent kernel's dependency chain grows with every row, the per-operation path is flat up to 8 sequences.
  // Tensor-parallel engines keep the persistent kernel (the exchange lives there).
  int stack_cap = -1;          // largest batch the persistent kernels are used for on one GPU (TSB200_STACK_MAXB); -1: fp16 none
                               // (one launch per operation on the tensor-core linears is faster at every batch), fp32 two
  int gemv_rows = -1;          // largest row count of the FMA streaming GEMV in the per-operation path (TSB200_GEMV_MAXROWS);
                               // -1: fp16 none (the tensor-core streaming kernel is faster from one row on), fp32 four
  std::vector<StackOp> stack_host;
  StackOp* stack_dev = nullptr;
  int stack_B = 0;
  const void* stack_key = nullptr;   // activation buffer the program was built for
  void *stack_partials = nullptr, *stack_counters = nullptr, *stack_attn = nullptr;
  int stack_max_B = 4;
  int64_t stack_counter_bytes = 0;
  long long* stack_trace = nullptr;  // optional timestamps (TSB200_GptDebugStackTrace, -DTSB200_TRACE builds)
  unsigned poll_limit = 0;           // 0: default; polls of a dependency counter before a CTA of the persistent kernel gives up
  // owner-partitioned persistent decode step (decode_owner.cu): fp16 engines on one GPU, up to own_cap sequences.  It
  // keeps a second copy of the layer weights, cut into one contiguous stream per CTA (built on first use).
  bool use_owner = true;             // TSB200_OWNER=0: keep the stream-K persistent kernel (saves the second weight copy)
  // Measured on the 7B-class model (same GPU, ms per decode step, kernel only): one sequence 3.10 against 3.20 for the
  // stream-K persistent kernel; two sequences 3.82 against 3.63 (its staging, merges and emissions are per row); on the
  // 1B-class model 1.02 against 1.03.  So it serves single sequences; TSB200_OWNER_MAXB raises the limit (tests do).
  int own_cap = -1;                  // -1: tensor-parallel engines one sequence, one-GPU engines none (TSB200_OWNER_MAXB)
  OwnerModel* own = nullptr;
  int own_B = 0;                     // batch the owner kernel serves for the current program (0: not in use)
};

enum KernelClass { KC_EMBED = 0, KC_NORM = 1, KC_LINEAR = 2, KC_ROPE_APPEND = 3, KC_ATTENTION = 4, KC_SAMPLE = 5, KC_COMMIT = 6, KC_ALLREDUCE = 7, KC_STACK = 8, KC_COUNT = 9 };

// Profiling pass (TSB200_GptProfileDecode): CUDA events around RUNS of consecutive launches of one class.  Inside a run no
// event is recorded between the launches, so they chain exactly as they do in the captured step (an event between two
// launches would serialise them); a run ends when a launch of another class begins, or at prof_flush().
static void prof_close_run(Gpt* g) {
  if (!g->prof_open) return;
  cudaEventRecord(g->prof_ev[2 * g->prof_n + 1], g->s);
  if (g->prof_cls.size() <= g->prof_n) {
    g->prof_cls.resize(g->prof_n + 512);
    g->prof_cnt.resize(g->prof_n + 512);
  }
  g->prof_cls[g->prof_n] = g->prof_open_cls;
  g->prof_cnt[g->prof_n] = g->prof_open_cnt;
  ++g->prof_n;
  g->prof_open = false;
}
static void prof_begin(Gpt* g, int cls) {
  if (!g->prof) return;
  if (g->prof_open && g->prof_open_cls == cls) return;   // the run goes on
  prof_close_run(g);
  if (g->prof_ev.size() < 2 * (g->prof_n + 1)) {
    const size_t old = g->prof_ev.size();
    g->prof_ev.resize(old + 512);
    for (size_t i = old; i < g->prof_ev.size(); ++i) cudaEventCreate(&g->prof_ev[i]);
  }
  cudaEventRecord(g->prof_ev[2 * g->prof_n], g->s);
  g->prof_open = true;
  g->prof_open_cls = cls;
  g->prof_open_cnt = 0;
}
// a launch of class `cls` has been issued (after prof_begin of the same class; a begin whose launch did not happen - a
// kernel that declined the shape - leaves the run open with nothing counted)
static void prof_end(Gpt* g, int cls) {
  if (!g->prof) return;
  if (g->prof_open && g->prof_open_cls == cls) ++g->prof_open_cnt;
}
static void prof_flush(Gpt* g) {
  if (g->prof) prof_close_run(g);
}
#define PROF(cls, call)          \
  do {                           \
    prof_begin(g, cls);          \
    const int _ok = (call);      \
    prof_end(g, cls);            \
    if (!_ok) return 0;          \
  } while (0)

constexpr size_t kGuardBytes = 256;
constexpr int kGuardByte = 0xC5;
constexpr int kMaxBeam = 32;

// Copies whole sequences inside the engine: for every pair (src, dst) the first T cache rows of every (layer, K or V, KV
// head), the token history and the pending id.  grid = (pairs, 2 * L * Hkv); sources and destinations are disjoint.
__global__ void __launch_bounds__(256) seq_copy_kernel(void* const* layers, const int* pairs, int Hkv, int64_t seq_bytes, int64_t head_pitch,
                                                       int64_t head_bytes, int* hist, int* hist_len, int* ids_cur, int hist_stride) {
  const int src = pairs[2 * blockIdx.x], dst = pairs[2 * blockIdx.x + 1];
  TSB_DEV_CHECK(engine, src >= 0 && dst >= 0 && src != dst && head_bytes <= head_pitch, 0x104, return)   // bad pair or rows beyond the cache
  const int lw = blockIdx.y / Hkv, kvh = blockIdx.y % Hkv;
  unsigned char* base = reinterpret_cast<unsigned char*>(layers[lw]);
  const uint4* from = reinterpret_cast<const uint4*>(base + (size_t)src * seq_bytes + (size_t)kvh * head_pitch);
  uint4* to = reinterpret_cast<uint4*>(base + (size_t)dst * seq_bytes + (size_t)kvh * head_pitch);
  for (int64_t i = threadIdx.x; i < head_bytes / 16; i += blockDim.x) to[i] = from[i];
  if (blockIdx.y == 0) {
    const int n = hist_len[src];
    for (int i = threadIdx.x; i < n && i < hist_stride; i += blockDim.x) hist[(size_t)dst * hist_stride + i] = hist[(size_t)src * hist_stride + i];
    if (threadIdx.x == 0) {
      hist_len[dst] = n;
      ids_cur[dst] = ids_cur[src];
    }
  }
}

static int dev_alloc(Gpt* g, void** p, int64_t bytes, bool zero = true) {
  if (bytes <= 0) bytes = 256;
  void* base = nullptr;
  cudaError_t e = cudaMalloc(&base, (size_t)bytes + 2 * kGuardBytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    TSB_FAIL("OOM: cudaMalloc of %lld bytes failed: %s", (long long)bytes, cudaGetErrorString(e));
  }
  *p = (char*)base + kGuardBytes;   // still 256-byte aligned
  TSB_CUDA(cudaMemsetAsync(base, kGuardByte, kGuardBytes, g->s));
  TSB_CUDA(cudaMemsetAsync((char*)*p + bytes, kGuardByte, kGuardBytes, g->s));
  if (zero) TSB_CUDA(cudaMemsetAsync(*p, 0, (size_t)bytes, g->s));
  g->allocs.push_back(Gpt::Alloc{*p, base, (size_t)bytes});
  return 1;
}
static int dev_free(Gpt* g, void* user) {
  for (auto& a : g->allocs)
    if (a.user == user && a.base) {
      TSB_CUDA(cudaFree(a.base));
      a.base = a.user = nullptr;
      return 1;
    }
  TSB_FAIL("engine: freeing a buffer the engine did not allocate");
}

static int fill_const(Gpt* g, void* p, int64_t n, float v) {
  if (g->c.dtype == TSB200_F32) fill_const_kernel<float><<<(int)((n + 255) / 256), 256, 0, g->s>>>((float*)p, n, v);
  else fill_const_kernel<__half><<<(int)((n + 255) / 256), 256, 0, g->s>>>((__half*)p, n, v);
  count_launch(g->c.device);
  return check_launch("fill_const");
}

static bool starts_with(const std::string& s, const char* p) { return s.compare(0, std::strlen(p), p) == 0; }
static bool ends_with(const std::string& s, const char* p) {
  const size_t n = std::strlen(p);
  return s.size() >= n && s.compare(s.size() - n, n, p) == 0;
}

// Maps a reference weight key to its place in the engine's buffers.  g->c holds this rank's LOCAL head and FFN counts;
// the slice of the full tensor that lands here is described by (full_rows, full_cols, sr0, sc0).  The packed MHA
// QKV matrix is sliced in three parts (q, k, v): `part` selects one, *nparts tells how many there are.
static int resolve_local(Gpt* g, const std::string& name, Dest* out);
static int resolve(Gpt* g, const std::string& name, Dest* out, int part = 0, int* nparts = nullptr) {
  if (nparts) *nparts = 1;
  *out = Dest();
  TSB_TRY(resolve_local(g, name, out));
  const TSB200GptConfig& c = g->c;
  const int64_t tp = g->tp, r = g->tp_rank;
  out->full_rows = out->rows;
  out->full_cols = out->cols;
  if (tp <= 1) return 1;
  const int64_t Hd = (int64_t)c.H * c.hd, KVd = (int64_t)c.Hkv * c.hd, F = c.F;
  auto ends = [&](const char* suf) { return ends_with(name, suf); };
  const bool is_vec = out->rows == 1 && !out->packed;
  if (ends(".W0")) { out->full_rows = Hd * tp; out->sr0 = r * Hd; }
  else if (ends("feedForwardLayer2.m_Whd")) { out->full_rows = F * tp; out->sr0 = r * F; }
  else if (ends(".b0") || ends("feedForwardLayer2.m_Bd")) { out->skip = (r != 0); }
  else if (ends(".QKV") || ends(".QKVb")) {
    if (nparts) *nparts = 3;
    out->full_cols = 3 * Hd * tp;
    out->cols = Hd;
    out->sc0 = part * Hd * tp + r * Hd;
    if (out->packed) out->c0 = part * Hd;
    else out->base = (char*)out->base + part * Hd * g->es;
  }
  else if (ends(".Q") || ends(".Qb")) { out->full_cols = Hd * tp; out->sc0 = r * Hd; }
  else if (ends(".K") || ends(".Kb") || ends(".V") || ends(".Vb")) { out->full_cols = KVd * tp; out->sc0 = r * KVd; }
  else if (ends("feedForwardLayer1.m_Whd") || ends("feedForwardLayer1.m_Bd") || ends("feedForwardLayer3.m_Whd") ||
           ends("feedForwardLayer3.m_Bd")) { out->full_cols = F * tp; out->sc0 = r * F; }
  (void)is_vec;
  return 1;
}
static int resolve_local(Gpt* g, const std::string& name, Dest* out) {
  const TSB200GptConfig& c = g->c;
  const int64_t d = c.d, F = c.F, V = c.V, Hd = (int64_t)c.H * c.hd, KVd = (int64_t)c.Hkv * c.hd;
  auto set = [&](void* base, int64_t rows, int64_t cols, int64_t rs, int64_t cs) {
    out->base = base; out->rows = rows; out->cols = cols; out->row_stride = rs; out->col_stride = cs;
    return 1;
  };
  auto off = [&](void* base, int64_t elems) { return (void*)((char*)base + elems * g->es); };
  auto setp = [&](void* base, int64_t rows, int64_t cols, int64_t c0, int64_t cs) {
    out->base = base; out->rows = rows; out->cols = cols; out->packed = true; out->c0 = c0; out->cs = cs;
    return 1;
  };
  out->packed = false;
  if (name == "TgtEmbeddings") return set(g->E, V, d, d, 1);
  if (name == "PosEmbedding") {
    TSB_CHECK(g->PE, "PosEmbedding given but the model's pe_type is not APE");
    return set(g->PE, g->pe_rows, d, d, 1);
  }
  if (name == "GPTDecoder.layerNorm.m_alpha") return set(g->nf_g, 1, d, d, 1);
  if (name == "GPTDecoder.layerNorm.m_beta") return set(g->nf_b, 1, d, d, 1);
  if (name == "FeedForward_Decoder_0.m_Whd") return setp(g->head_w, d, V, 0, 1);
  if (name == "FeedForward_Decoder_0.m_Bd") return set(g->head_b, 1, V, V, 1);
  // the reference names the decoder of its encoder-decoder models "TransformerDecoder" (Applications/Decoder.cs:49)
  const bool dec_prefix = c.cross_attn && starts_with(name, "TransformerDecoder.");
  if (dec_prefix && name == "TransformerDecoder.layerNorm.m_alpha") return set(g->nf_g, 1, d, d, 1);
  if (dec_prefix && name == "TransformerDecoder.layerNorm.m_beta") return set(g->nf_b, 1, d, d, 1);
  if (c.cross_attn && name == "SharedEmbeddings") return set(g->E, V, d, d, 1);   // one table for source and target (BaseSeq2SeqFramework.cs:365)
  TSB_CHECK(starts_with(name, "GPTDecoder.") || dec_prefix, "unknown weight name '%s'", name.c_str());
  const std::string rest = name.substr(dec_prefix ? 19 : 11);
  const size_t us = rest.find('_'), dot = rest.find('.');
  TSB_CHECK(us != std::string::npos && dot != std::string::npos && us < dot, "unknown weight name '%s'", name.c_str());
  const int k = std::atoi(rest.substr(us + 1, dot - us - 1).c_str());
  TSB_CHECK(k >= 0 && k < c.L, "layer index out of range in '%s'", name.c_str());
  LayerW& L = g->L[k];
  const std::string unit = rest.substr(0, us), field = rest.substr(dot + 1);
  const int64_t Nq = g->Nqkv;
  if (unit == "SelfAttn") {
    if (field == "layerNormQ.m_alpha") return set(L.n1_g, 1, d, d, 1);
    if (field == "layerNormQ.m_beta") return set(L.n1_b, 1, d, d, 1);
    if (field == "W0") return setp(L.wo, Hd, d, 0, 1);
    if (field == "b0") return set(L.bo, 1, d, d, 1);
    if (c.attn_type == 0) {
      if (field == "QKV") return setp(L.wqkv, d, Nq, 0, 1);
      if (field == "QKVb") return set(L.bqkv, 1, Nq, Nq, 1);
    } else {
      if (field == "Q") return setp(L.wqkv, d, Hd, 0, 1);
      if (field == "Qb") return set(L.bqkv, 1, Hd, Nq, 1);
      if (field == "K") return setp(L.wqkv, d, KVd, Hd, 1);
      if (field == "Kb") return set(off(L.bqkv, Hd), 1, KVd, Nq, 1);
      if (field == "V") return setp(L.wqkv, d, KVd, Hd + KVd, 1);
      if (field == "Vb") return set(off(L.bqkv, Hd + KVd), 1, KVd, Nq, 1);
    }
  } else if (unit == "EncAttn") {
    TSB_CHECK(c.cross_attn, "'%s': the model has no cross-attention blocks", name.c_str());
    if (field == "layerNormQ.m_alpha") return set(L.nx_g, 1, d, d, 1);
    if (field == "layerNormQ.m_beta") return set(L.nx_b, 1, d, d, 1);
    if (field == "Q") return setp(L.xq, d, Hd, 0, 1);
    if (field == "Qb") return set(L.xqb, 1, Hd, Hd, 1);
    if (field == "K") return setp(L.xk, d, Hd, 0, 1);
    if (field == "Kb") return set(L.xkb, 1, Hd, Hd, 1);
    if (field == "V") return setp(L.xv, d, Hd, 0, 1);
    if (field == "Vb") return set(L.xvb, 1, Hd, Hd, 1);
    if (field == "W0") return setp(L.xo, Hd, d, 0, 1);
    if (field == "b0") return set(L.xob, 1, d, d, 1);
  } else if (unit == "MoEFFN") {
    TSB_CHECK(L.moe, "'%s': layer %d is not a mixture-of-experts layer", name.c_str(), k);
    const int64_t E = c.n_experts, Fh = 4 * d;
    if (field == "layerNorm.m_alpha") return set(L.moe_g, 1, d, d, 1);
    if (field == "layerNorm.m_beta") return set(L.moe_b, 1, d, d, 1);
    if (field == "m_Router") return set(L.router_w, d, E, E, 1);
    if (field == "m_RouterBias") return set(L.router_b, 1, E, E, 1);
    if (field == "m_Whd1") return set(L.moe_w1, E * d, Fh, Fh, 1);      // [E, d, 4d] handed over as [E * d, 4d]
    if (field == "m_Whd2") return set(L.moe_w2, E * Fh, d, d, 1);
  } else if (unit == "PosFFN") {
    TSB_CHECK(!L.moe, "'%s': layer %d is a mixture-of-experts layer", name.c_str(), k);
    if (field == "layerNorm2.m_alpha") return set(L.n2_g, 1, d, d, 1);
    if (field == "layerNorm2.m_beta") return set(L.n2_b, 1, d, d, 1);
    const int64_t w1c = g->glu ? 2 * F : F, cs = g->glu ? 2 : 1;
    if (field == "feedForwardLayer1.m_Whd") return setp(L.w1, d, F, 0, cs);
    if (field == "feedForwardLayer1.m_Bd") return set(L.b1, 1, F, w1c, cs);
    if (g->glu && field == "feedForwardLayer3.m_Whd") return setp(L.w1, d, F, 1, cs);
    if (g->glu && field == "feedForwardLayer3.m_Bd") return set(off(L.b1, 1), 1, F, w1c, cs);
    if (field == "feedForwardLayer2.m_Whd") return setp(L.w2, F, d, 0, 1);
    if (field == "feedForwardLayer2.m_Bd") return set(L.b2, 1, d, d, 1);
  }
  TSB_FAIL("unknown weight name '%s'", name.c_str());
}

// src_dev points at the FULL tensor [dst.full_rows, dst.full_cols]; this rank's block is copied / packed.
static int copy_into(Gpt* g, const Dest& dst, const void* src_dev, int src_dtype) {
  if (dst.skip) return 1;
  const int ses = src_dtype == TSB200_F16 ? 2 : 4;
  const void* src = (const char*)src_dev + (dst.sr0 * dst.full_cols + dst.sc0) * ses;
  if (dst.packed)
    return launch_pack(g->c.device, g->st, g->c.dtype, dst.base, src_dtype, src, (int)dst.rows, (int)dst.cols, (int)dst.full_cols,
                       (int)dst.rows, (int)dst.c0, (int)dst.cs, g->s);
  TSB200Tensor r{}, sv{};
  r.data = dst.base; r.dtype = g->c.dtype; r.ndim = 2;
  r.sizes[0] = dst.rows; r.sizes[1] = dst.cols; r.strides[0] = dst.row_stride; r.strides[1] = dst.col_stride;
  sv.data = const_cast<void*>(src); sv.dtype = src_dtype; sv.ndim = 2;
  sv.sizes[0] = dst.rows; sv.sizes[1] = dst.cols; sv.strides[0] = dst.full_cols; sv.strides[1] = 1;
  return TSB200_Copy(g->c.device, &r, &sv, g->s);
}

static std::vector<std::string> weight_names(const Gpt* g, bool biases, bool norms, bool matrices) {
  const TSB200GptConfig& c = g->c;
  std::vector<std::string> v;
  auto add = [&](bool on, const std::string& s) { if (on) v.push_back(s); };
  add(matrices, "TgtEmbeddings");
  for (int k = 0; k < c.L; ++k) {
    const std::string a = "GPTDecoder.SelfAttn_" + std::to_string(k) + ".", f = "GPTDecoder.PosFFN_" + std::to_string(k) + ".";
    add(norms, a + "layerNormQ.m_alpha");
    if (c.norm_type == 0) add(norms, a + "layerNormQ.m_beta");
    if (c.attn_type == 0) {
      add(matrices, a + "QKV");
      add(biases, a + "QKVb");
    } else {
      add(matrices, a + "Q"); add(biases, a + "Qb");
      add(matrices, a + "K"); add(biases, a + "Kb");
      add(matrices, a + "V"); add(biases, a + "Vb");
    }
    add(matrices, a + "W0");
    add(biases, a + "b0");
    if (c.cross_attn) {
      const std::string e = "GPTDecoder.EncAttn_" + std::to_string(k) + ".";
      add(norms, e + "layerNormQ.m_alpha");
      if (c.norm_type == 0) add(norms, e + "layerNormQ.m_beta");
      add(matrices, e + "Q"); add(biases, e + "Qb");
      add(matrices, e + "K"); add(biases, e + "Kb");
      add(matrices, e + "V"); add(biases, e + "Vb");
      add(matrices, e + "W0"); add(biases, e + "b0");
    }
    if (g->L[k].moe) {
      const std::string m = "GPTDecoder.MoEFFN_" + std::to_string(k) + ".";
      add(norms, m + "layerNorm.m_alpha");
      add(norms, m + "layerNorm.m_beta");
      add(matrices, m + "m_Whd1"); add(matrices, m + "m_Whd2");
      add(matrices, m + "m_Router"); add(biases, m + "m_RouterBias");
      continue;
    }
    add(norms, f + "layerNorm2.m_alpha");
    if (c.norm_type == 0) add(norms, f + "layerNorm2.m_beta");
    add(matrices, f + "feedForwardLayer1.m_Whd"); add(biases, f + "feedForwardLayer1.m_Bd");
    if (g->glu) { add(matrices, f + "feedForwardLayer3.m_Whd"); add(biases, f + "feedForwardLayer3.m_Bd"); }
    add(matrices, f + "feedForwardLayer2.m_Whd"); add(biases, f + "feedForwardLayer2.m_Bd");
  }
  add(norms, "GPTDecoder.layerNorm.m_alpha");
  if (c.norm_type == 0) add(norms, "GPTDecoder.layerNorm.m_beta");
  add(matrices, "FeedForward_Decoder_0.m_Whd");
  add(biases, "FeedForward_Decoder_0.m_Bd");
  return v;
}

static int ensure_act(Gpt* g, int64_t rows) {
  if (rows <= g->act_rows) return 1;
  const TSB200GptConfig& c = g->c;
  TSB_CUDA(cudaStreamSynchronize(g->s));
  // the captured decode step holds the old buffers as kernel arguments
  if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  // ... and so does the program of the persistent decode-step kernel (a new buffer may come back at the old address)
  g->stack_key = nullptr;
  g->stack_B = 0;
  auto re = [&](void** p, int64_t bytes) -> int {
    if (*p) {
      TSB_TRY(dev_free(g, *p));
      *p = nullptr;
    }
    return dev_alloc(g, p, bytes, false);
  };
  const int64_t Hd = (int64_t)c.H * c.hd;
  TSB_TRY(re((void**)&g->x, rows * c.d * 4));
  TSB_TRY(re(&g->h, rows * c.d * g->es));
  TSB_TRY(re(&g->qkv, rows * g->Nqkv * g->es));
  TSB_TRY(re(&g->attn, rows * Hd * g->es));
  {
    // FFN hidden rows; mixture-of-experts layers keep experts_per_token hidden rows of 4 d per token there
    int64_t ffn_elems = rows * c.F;
    if (c.n_experts > 1 && rows * c.experts_per_token * 4 * c.d > ffn_elems) ffn_elems = rows * c.experts_per_token * 4 * c.d;
    TSB_TRY(re(&g->ffn, ffn_elems * g->es));
    if (c.n_experts > 1) {
      TSB_TRY(re((void**)&g->moe_picks, rows * c.experts_per_token * 4));
      TSB_TRY(re((void**)&g->moe_scores, rows * c.experts_per_token * 4));
    }
  }
  if (g->tp > 1) TSB_TRY(re((void**)&g->ar_buf, rows * c.d * 4));
  g->act_rows = rows;
  return 1;
}

static Epilogue make_ep(const void* bias, const float* residual, void* y, float* y32, int act, int glu) {
  Epilogue e{};
  e.bias = bias; e.residual = residual; e.y = y32 ? nullptr : y; e.y32 = y32; e.act = act; e.glu = glu;
  return e;
}

// One linear layer of the engine on packed weights.  With `ng` the input is the fp32 residual stream and the layer's
// LayerNorm / RMSNorm comes first: fused into the streaming GEMV as a prologue for decode-sized row counts, a
// separate launch (into g->h) otherwise.
static int engine_linear(Gpt* g, int rows, const void* x_T, const float* x_resid, const void* ng, const void* nb, void* h_tmp,
                         const void* Wp, int K, int N, const Epilogue& ep) {
  const TSB200GptConfig& c = g->c;
  const int dev = c.device, dt = c.dtype;
  if (rows <= (g->gemv_rows >= 0 ? g->gemv_rows : (dt == TSB200_F16 ? 0 : 4))) {
    prof_begin(g, KC_LINEAR);
    const int r = launch_gemv_stream(dev, g->st, dt, Wp, ng ? (const void*)x_resid : x_T, ng ? (c.norm_type == 0 ? 2 : 1) : 0, ng,
                                     c.norm_type == 0 ? nb : nullptr, c.eps, rows, K, N, ep, g->err_flag, g->pdl, g->lin_ws,
                                     g->lin_ws_bytes, g->s);
    if (r != 2) {
      prof_end(g, KC_LINEAR);
      return r;
    }
  }
  if (ng && dt == TSB200_F16 && rows <= 8 && g->fuse_step) {
    // up to eight rows: the tensor-core streaming kernel norms the rows itself (no norm launch)
    prof_begin(g, KC_LINEAR);
    const int r = launch_gemm_stream_mma_norm(dev, g->st, x_resid, ng, c.norm_type == 0 ? nb : nullptr, c.norm_type, c.eps, Wp, rows, K, N, ep,
                                              g->err_flag, g->pdl, g->lin_ws, g->lin_ws_bytes, g->s);
    if (r != 2) {
      g->lin_syms_used = true;
      prof_end(g, KC_LINEAR);
      return r;
    }
  }
  if (ng) {
    PROF(KC_NORM, launch_norm_residual(dev, g->st, dt, h_tmp, const_cast<float*>(x_resid), nullptr, ng, c.norm_type == 0 ? nb : nullptr,
                                       c.norm_type, c.eps, rows, K, g->s));
    x_T = h_tmp;
  }
  g->lin_syms_used = true;   // these kernels report a wait that ran out through their own error symbols
  PROF(KC_LINEAR, launch_linear(dev, g->st, dt, x_T, Wp, rows, K, N, ep, g->lin_ws, g->lin_ws_bytes, g->s, true));
  return 1;
}

// x += in[rows,K] * Wp[K,d] + bias: the out-projection of attention and the FFN down-projection.  Under tensor
// parallelism each rank holds K/tp rows of the weight, so its product is a partial sum: it goes to a scratch buffer
// (bias only on rank 0), one all-reduce sums it over the ranks, and the residual add follows
// (MultiProcessorNetworkWrapper rework: one all-reduce after the out-projection, one after the down-projection).
static int row_parallel_linear(Gpt* g, int rows, const void* in, const void* Wp, int K, const void* bias) {
  const int d = g->c.d;
  if (g->tp <= 1) return engine_linear(g, rows, in, nullptr, nullptr, nullptr, nullptr, Wp, K, d, make_ep(bias, g->x, nullptr, g->x, TSB200_ACT_NONE, 0));
  TSB_CHECK(g->comm, "tensor parallel engine has no communicator (call TSB200_GptSetComm)");
  if (float* pb = g->tp_peer ? comm_peer_buffer(g->comm, (int64_t)rows * d) : nullptr) {
    // small messages (decode): the partial goes to this rank's peer buffer, one kernel exchanges flags over NVLink,
    // reads every rank's partial from its memory and adds the sum to the residual stream
    TSB_TRY(engine_linear(g, rows, in, nullptr, nullptr, nullptr, nullptr, Wp, K, d, make_ep(bias, nullptr, nullptr, pb, TSB200_ACT_NONE, 0)));
    prof_begin(g, KC_ALLREDUCE);
    const int ok = comm_peer_reduce(g->comm, g->x, (int64_t)rows * d, g->err_flag, g->st->sm_count, g->s);
    count_launch(g->c.device);
    prof_end(g, KC_ALLREDUCE);
    return ok;
  }
  TSB_TRY(engine_linear(g, rows, in, nullptr, nullptr, nullptr, nullptr, Wp, K, d, make_ep(bias, nullptr, nullptr, g->ar_buf, TSB200_ACT_NONE, 0)));
  prof_begin(g, KC_ALLREDUCE);
  int ok = comm_all_reduce_f32(g->comm, g->ar_buf, (int64_t)rows * d, g->s);
  prof_end(g, KC_ALLREDUCE);
  TSB_TRY(ok);
  prof_begin(g, KC_NORM);
  const int64_t n = (int64_t)rows * d;
  int64_t gsz = (n + 255) / 256;
  if (gsz > (int64_t)g->st->sm_count * 8) gsz = (int64_t)g->st->sm_count * 8;
  TSB_CUDA(launch_k(residual_add_kernel, dim3((int)gsz), dim3(256), 0, g->s, g->x, (const float*)g->ar_buf, n));
  count_launch(g->c.device);
  prof_end(g, KC_NORM);
  return check_launch("residual_add");
}

// Builds (or reuses) the operation list of the persistent decode-step kernel for B sequences: per layer QKV (norm
// prologue), attention, out-projection (+residual), FFN up (norm prologue, activation / gate), FFN down (+residual),
// then the LM head behind the final norm.
static int ensure_stack(Gpt* g, int B) {
  const TSB200GptConfig& c = g->c;
  g->stack_max_B = (c.dtype == TSB200_F16) ? 8 : 4;  // fp16: tensor-core consumers take up to 8 rows
  const int cap = g->stack_cap >= 0 ? g->stack_cap : (c.dtype == TSB200_F16 ? 0 : 2);
  if (g->tp == 1 && cap < g->stack_max_B) g->stack_max_B = cap;
  g->own_B = 0;
  if (!g->use_stack || g->ragged) return 1;   // sequences of different lengths: one launch per operation
  if (g->c.n_experts > 1) return 1;           // mixture-of-experts layers exist only as separate launches
  if (g->c.cross_attn) return 1;              // so do the cross-attention blocks
  // tensor-parallel engines: one sequence, and only once the ranks' exchange regions are mapped into each other
  const bool own_tp_ok = g->tp == 1 || (g->xch_ready && g->tp_peer && B == 1 && g->xch_own_off != 0);
  const int own_cap = g->own_cap >= 0 ? g->own_cap : (g->tp > 1 ? 1 : 0);
  if (g->use_owner && own_tp_ok && B <= own_cap && B <= kOwnMaxRows) {
    OwnDims D{};
    D.L = c.L; D.d = c.d; D.H = c.H; D.Hkv = c.Hkv; D.hd = c.hd; D.F = c.F; D.V = c.V; D.glu = g->glu;
    if (owner_applicable(D, c.dtype, g->st->sm_count)) {
      if (!g->own) {
        std::vector<OwnLayerPtrs> lp(c.L);
        for (int k = 0; k < c.L; ++k) {
          const LayerW& L = g->L[k];
          lp[k] = OwnLayerPtrs{L.n1_g, L.n1_b, L.wqkv, L.bqkv, L.wo, L.bo, L.n2_g, L.n2_b, L.w1, L.b1, L.w2, L.b2, L.cK, L.cV};
        }
        TSB_TRY(owner_create(c.device, g->st, D, c.norm_type, c.act, c.pe_type == 2, c.eps, c.max_tokens, lp.data(), g->nf_g, g->nf_b,
                             g->head_w, g->head_b, &g->own));
      }
      if (!owner_packed(g->own)) {
        TSB_TRY(owner_repack(g->own, g->s));
        TSB_CUDA(cudaStreamSynchronize(g->s));
      }
      g->own_B = B;
      return 1;
    }
  }
  if (B > g->stack_max_B) return 1;
  const bool tp = g->tp > 1;
  if (tp && !(g->xch_ready && c.dtype == TSB200_F16 && c.d <= 4096 && c.d % 4 == 0 && g->tp_peer)) return 1;  // per-operation launches + all-reduce
  if (g->stack_dev && g->stack_B == B && g->stack_key == (const void*)g->x) return 1;
  const int d = c.d, Hd = c.H * c.hd;
  const int nmode = c.norm_type == 0 ? 2 : 1;
  std::vector<StackOp> ops;
  auto lin = [&](int xmode, const void* x, const void* ng, const void* nb, const void* Wp, int K, int N, const Epilogue& ep) {
    StackOp o{};
    o.type = 0; o.xmode = xmode; o.Wp = Wp; o.x = x; o.gamma = ng; o.beta = (c.norm_type == 0) ? nb : nullptr; o.eps = c.eps;
    o.K = K; o.N = N; o.ep = ep;
    ops.push_back(o);
  };
  if (!tp) {
    for (int k = 0; k < c.L; ++k) {
      LayerW& L = g->L[k];
      lin(nmode, g->x, L.n1_g, L.n1_b, L.wqkv, d, g->Nqkv, make_ep(L.bqkv, nullptr, g->qkv, nullptr, TSB200_ACT_NONE, 0));
      StackOp at{};
      at.type = 1; at.x = g->qkv; at.cK = L.cK; at.cV = L.cV; at.ep.y = g->attn;
      ops.push_back(at);
      lin(0, g->attn, nullptr, nullptr, L.wo, Hd, d, make_ep(L.bo, g->x, nullptr, g->x, TSB200_ACT_NONE, 0));
      lin(nmode, g->x, L.n2_g, L.n2_b, L.w1, d, g->glu ? 2 * c.F : c.F, make_ep(L.b1, nullptr, g->ffn, nullptr, c.act, g->glu));
      lin(0, g->ffn, nullptr, nullptr, L.w2, c.F, d, make_ep(L.b2, g->x, nullptr, g->x, TSB200_ACT_NONE, 0));
    }
    lin(nmode, g->x, g->nf_g, g->nf_b, g->head_w, d, c.V, make_ep(g->head_b, nullptr, nullptr, g->logits, TSB200_ACT_NONE, 0));
    for (auto& o : ops) { o.xsite = -1; o.ssite = -1; o.x_out = nullptr; }
  } else {
    // Tensor parallel: QKV and FFN-up are column-sharded (local heads / FFN columns), the out-projection and FFN-down
    // are row-sharded: their finished column tiles are partial sums that go to every rank's exchange buffer; the next
    // operation's norm prologue adds them (rank order) to the residual row it reads and CTA 0 stores the new row into
    // the other residual buffer.  Exchange buffers alternate with the layer parity.
    if (!g->x2) TSB_TRY(dev_alloc(g, (void**)&g->x2, (int64_t)c.max_batch * d * 4));
    float* xin = g->x;          // residual rows the next norm prologue reads
    float* xother = g->x2;
    int pending = -1;           // exchange site whose sums the next norm prologue must add
    auto norm_lin = [&](const void* ng, const void* nb, const void* Wp, int N, const Epilogue& ep) {
      lin(nmode, xin, ng, nb, Wp, d, N, ep);
      StackOp& o = ops.back();
      o.xsite = -1; o.ssite = pending; o.x_out = nullptr;
      if (pending >= 0) {
        o.x_out = xother;
        std::swap(xin, xother);
        pending = -1;
      }
    };
    for (int k = 0; k < c.L; ++k) {
      LayerW& L = g->L[k];
      norm_lin(L.n1_g, L.n1_b, L.wqkv, g->Nqkv, make_ep(L.bqkv, nullptr, g->qkv, nullptr, TSB200_ACT_NONE, 0));
      StackOp at{};
      at.type = 1; at.x = g->qkv; at.cK = L.cK; at.cV = L.cV; at.ep.y = g->attn; at.xsite = -1; at.ssite = -1;
      ops.push_back(at);
      lin(0, g->attn, nullptr, nullptr, L.wo, Hd, d, make_ep(L.bo, nullptr, nullptr, g->x2, TSB200_ACT_NONE, 0));
      ops.back().xsite = (k & 1); ops.back().ssite = -1; ops.back().x_out = nullptr;
      pending = (k & 1);
      norm_lin(L.n2_g, L.n2_b, L.w1, g->glu ? 2 * c.F : c.F, make_ep(L.b1, nullptr, g->ffn, nullptr, c.act, g->glu));
      lin(0, g->ffn, nullptr, nullptr, L.w2, c.F, d, make_ep(L.b2, nullptr, nullptr, g->x2, TSB200_ACT_NONE, 0));
      ops.back().xsite = 2 + (k & 1); ops.back().ssite = -1; ops.back().x_out = nullptr;
      pending = 2 + (k & 1);
    }
    norm_lin(g->nf_g, g->nf_b, g->head_w, c.V, make_ep(g->head_b, nullptr, nullptr, g->logits, TSB200_ACT_NONE, 0));
  }
  if (!g->stack_partials) {
    StackConfig sc{};
    sc.dtype = c.dtype; sc.M = c.max_batch < g->stack_max_B ? c.max_batch : g->stack_max_B; sc.H = c.H; sc.Hkv = c.Hkv; sc.hd = c.hd;
    int64_t pb, cb, ab;
    decode_stack_scratch(sc, ops.data(), (int)ops.size(), g->st->sm_count, &pb, &cb, &ab);
    TSB_TRY(dev_alloc(g, &g->stack_partials, pb, false));
    TSB_TRY(dev_alloc(g, &g->stack_counters, cb, true));
    TSB_TRY(dev_alloc(g, &g->stack_attn, ab, false));
    g->stack_counter_bytes = cb;
    void* p = nullptr;
    TSB_TRY(dev_alloc(g, &p, (int64_t)ops.size() * sizeof(StackOp), false));
    g->stack_dev = (StackOp*)p;
  }
  TSB_CUDA(cudaMemcpyAsync(g->stack_dev, ops.data(), ops.size() * sizeof(StackOp), cudaMemcpyHostToDevice, g->s));
  TSB_CUDA(cudaStreamSynchronize(g->s));  // `ops` is pageable host memory
  g->stack_host.swap(ops);
  g->stack_B = B;
  g->stack_key = g->x;
  return 1;
}

// One forward pass over `rows = B*S` new tokens whose ids are in g->ids_in; leaves logits [B,V] in g->logits.
// With use_state the cache length is read from g->state[0] by the kernels (graph replay), else from T0.
static int enqueue_forward(Gpt* g, int B, int S, int T0, bool use_state, int splits) {
  NvtxRange nvtx_(S == 1 ? "tsb200.forward.step" : "tsb200.forward.prompt");
  PdlScope pdl_scope(g->pdl && S == 1);
  const TSB200GptConfig& c = g->c;
  const int dev = c.device, dt = c.dtype, d = c.d, rows = B * S;
  const int* dT = use_state ? g->state : nullptr;
  const int Hd = c.H * c.hd, KVd = c.Hkv * c.hd;
  const int pe_mode = (c.pe_type == 1) ? (c.ape_decode_pos0 ? 1 : 2) : 0;
  const float sf = (float)std::sqrt((double)d);
  {
    prof_begin(g, KC_EMBED);
    const int gsz = rows < g->st->sm_count * 8 ? rows : g->st->sm_count * 8;
    const int* ids = (S == 1 && use_state) ? g->ids_cur : g->ids_in;
    if (dt == TSB200_F32)
      TSB_CUDA(launch_k(embed_kernel<float>, dim3(gsz), dim3(256), 0, g->s, g->x, (const float*)g->E, (const float*)g->PE, ids, rows, S, d, c.V, sf, pe_mode, g->pe_rows, T0, dT));
    else
      TSB_CUDA(launch_k(embed_kernel<__half>, dim3(gsz), dim3(256), 0, g->s, g->x, (const __half*)g->E, (const __half*)g->PE, ids, rows, S, d, c.V, sf, pe_mode, g->pe_rows, T0, dT));
    count_launch(dev);
    prof_end(g, KC_EMBED);
    TSB_TRY(check_launch("embed"));
  }
  if (S == 1 && use_state && g->use_stack && !g->ragged && g->own_B == B && owner_packed(g->own)) {
    prof_begin(g, KC_STACK);
    OwnTp otp{};
    otp.rank = g->tp_rank; otp.size = g->tp; otp.offset = (long long)g->xch_own_off;
    for (int q = 0; q < g->tp && q < kStackMaxRanks; ++q) otp.peer[q] = g->tp > 1 ? g->xch_peer[q] : nullptr;
    const int r = owner_launch(g->own, g->st, B, g->x, g->logits, g->rope_tab, dT, g->err_flag, g->poll_limit, g->pdl, g->stack_trace,
                               g->tp > 1 ? &otp : nullptr, g->s);
    if (r != 2) {
      prof_end(g, KC_STACK);
      g->last_path = 2;
      return r;
    }
  }
  if (S == 1 && use_state) g->last_path = 0;
  if (S == 1 && use_state && g->use_stack && !g->ragged && B <= g->stack_max_B && g->stack_dev && g->stack_B == B && g->stack_key == (const void*)g->x) {
    StackConfig sc{};
    sc.dtype = dt; sc.M = B; sc.H = c.H; sc.Hkv = c.Hkv; sc.hd = c.hd; sc.Tmax = c.max_tokens; sc.qkv_rs = g->Nqkv;
    sc.use_rope = c.pe_type == 2; sc.rope_tab = g->rope_tab; sc.dT = dT;
    sc.tp_rank = g->tp_rank; sc.tp_size = g->tp; sc.d = c.d;
    for (int r = 0; r < g->tp && r < kStackMaxRanks; ++r) sc.peer[r] = g->tp > 1 ? g->xch_peer[r] : nullptr;
    sc.poll_limit = g->poll_limit;
    prof_begin(g, KC_STACK);
    const int r = launch_decode_stack(dev, g->st, sc, g->stack_dev, g->stack_host.data(), (int)g->stack_host.size(),
                                      g->stack_partials, g->stack_counters, g->stack_attn, g->err_flag, g->stack_trace, g->pdl, g->s);
    if (r != 2) {
      prof_end(g, KC_STACK);
      g->last_path = 1;
      return r;
    }
  }
  const int act = c.act;
  for (int k = 0; k < c.L; ++k) {
    LayerW& L = g->L[k];
    void* qp = g->qkv;
    void* kp = (char*)g->qkv + (int64_t)Hd * g->es;
    void* vp = (char*)g->qkv + (int64_t)(Hd + KVd) * g->es;
    bool appended = false;
    if (S == 1 && dt == TSB200_F16 && rows <= 8 && g->fuse_step) {
      // one new position per sequence, up to eight sequences: norm, q | k | v projection, RoPE and the cache append in one launch
      RopeFuse rf{};
      rf.cK = L.cK; rf.cV = L.cV; rf.Hd = Hd; rf.KVd = KVd; rf.hd = c.hd; rf.Tmax = c.max_tokens;
      rf.use_rope = c.pe_type == 2 ? 1 : 0; rf.T0 = T0; rf.state = dT; rf.tab = g->rope_tab;
      prof_begin(g, KC_LINEAR);
      const int r = launch_gemm_stream_mma_norm(dev, g->st, g->x, L.n1_g, c.norm_type == 0 ? L.n1_b : nullptr, c.norm_type, c.eps, L.wqkv, rows, d,
                                                g->Nqkv, make_ep(L.bqkv, nullptr, g->qkv, nullptr, TSB200_ACT_NONE, 0), g->err_flag, g->pdl, g->lin_ws,
                                                g->lin_ws_bytes, g->s, &rf);
      if (r == 0) return 0;
      if (r == 1) {
        g->lin_syms_used = true;
        prof_end(g, KC_LINEAR);
        appended = true;
      }
    }
    if (!appended) {
      TSB_TRY(engine_linear(g, rows, nullptr, g->x, L.n1_g, L.n1_b, g->h, L.wqkv, d, g->Nqkv, make_ep(L.bqkv, nullptr, g->qkv, nullptr, TSB200_ACT_NONE, 0)));
      PROF(KC_ROPE_APPEND, launch_rope_append(dev, g->st, dt, qp, kp, vp, g->Nqkv, g->Nqkv, L.cK, L.cV, B, S, c.H, c.Hkv, c.hd, T0, dT, c.max_tokens, c.pe_type == 2, (double)c.rope_base, g->rope_tab, g->s));
    }
    PROF(KC_ATTENTION, launch_attention(dev, g->st, dt, g->attn, qp, g->Nqkv, L.cK, L.cV, B, S, c.H, c.Hkv, c.hd, T0, dT, c.max_tokens, splits, g->attn_ws, g->attn_ws_bytes, g->s));
    TSB_TRY(row_parallel_linear(g, rows, g->attn, L.wo, Hd, L.bo));
    if (c.cross_attn) {
      // x += W0 (softmax(Q K^T / sqrt(hd)) V) + b0 with Q from the normed stream, K / V the encoder rows prepared by
      // TSB200_GptSetEncoderOutput; every new position sees all source positions of its sequence
      TSB_CHECK(g->cross_T > 0, "decoder step before TSB200_GptSetEncoderOutput");
      TSB_CHECK(S == 1, "cross-attention engines take one new token per sequence and call (got %d)", S);
      TSB_TRY(engine_linear(g, rows, nullptr, g->x, L.nx_g, L.nx_b, g->h, L.xq, d, (int)Hd, make_ep(L.xqb, nullptr, g->qkv, nullptr, TSB200_ACT_NONE, 0)));
      PROF(KC_ATTENTION, launch_attention(dev, g->st, dt, g->attn, g->qkv, Hd, L.xK, L.xV, B, 1, c.H, c.H, c.hd, g->cross_T - 1, g->cross_state,
                                          c.max_src_tokens, attn_pick_splits(g->st, dt, B, c.H, c.H, c.hd, g->cross_T), g->attn_ws, g->attn_ws_bytes, g->s));
      TSB_TRY(row_parallel_linear(g, rows, g->attn, L.xo, Hd, L.xob));
    }
    if (L.moe) {
      // MoEFeedForward.Process: the layer's own LayerNorm (whatever the model's norm type), router, experts, residual add
      PROF(KC_NORM, launch_norm_residual(dev, g->st, dt, g->h, g->x, nullptr, L.moe_g, L.moe_b, 0, c.eps, rows, d, g->s));
      PROF(KC_LINEAR, launch_moe_ffn(dev, g->st, dt, g->x, g->h, L.router_w, L.router_b, L.moe_w1, L.moe_w2, g->ffn, g->moe_picks, g->moe_scores,
                                     rows, d, c.n_experts, c.experts_per_token, act, g->s));
      continue;
    }
    TSB_TRY(engine_linear(g, rows, nullptr, g->x, L.n2_g, L.n2_b, g->h, L.w1, d, g->glu ? 2 * c.F : c.F, make_ep(L.b1, nullptr, g->ffn, nullptr, act, g->glu)));
    TSB_TRY(row_parallel_linear(g, rows, g->ffn, L.w2, c.F, L.b2));
  }
  const float* xlast = g->x;
  if (S > 1) {
    gather_last_kernel<<<B, 256, 0, g->s>>>(g->xl, g->x, B, S, d, g->gather_lens);
    count_launch(dev);
    TSB_TRY(check_launch("gather_last"));
    xlast = g->xl;
  }
  TSB_TRY(engine_linear(g, B, nullptr, xlast, g->nf_g, g->nf_b, g->hl, g->head_w, d, c.V, make_ep(g->head_b, nullptr, nullptr, g->logits, TSB200_ACT_NONE, 0)));
  return 1;
}

// logits -> id (greedy or top-p), then commit: feed back, history, output slot, counters.
static int enqueue_sample(Gpt* g, int B, const TSB200DecodingOptions* opt, bool use_state, bool advance_T) {
  PdlScope pdl_scope(g->pdl && advance_T);
  const TSB200GptConfig& c = g->c;
  const int dev = c.device;
  const bool sampling = opt->strategy == 1;
  const int use_temp = (sampling && opt->temperature != 1.0f) ? 1 : 0;
  PROF(KC_SAMPLE, launch_softmax_argmax(dev, g->st, g->ids_new, sampling ? g->probs : nullptr, g->logits, B, c.V, opt->temperature, use_temp, g->blocked, g->n_blocked, g->s));
  if (sampling) {
    PROF(KC_SAMPLE, launch_philox(dev, g->u, B, opt->seed, opt->seq_base, g->step, use_state ? g->state : nullptr, g->s));
    PROF(KC_SAMPLE, launch_topp(dev, g->st, g->ids_new, g->probs, B, c.V, opt->topP, opt->repeatPenalty, g->hist, g->hist_len, c.max_tokens, g->u, g->topp_ws, g->s));
  }
  prof_begin(g, KC_COMMIT);
  TSB_CUDA(launch_k(commit_kernel, dim3(1), dim3(256), 0, g->s, g->ids_cur, (const int*)g->ids_new, g->hist, g->hist_len, c.max_tokens, g->out_dev, B, g->state, advance_T ? 1 : 0, g->seq0,
                    advance_T ? g->stop_fin : 0));
  count_launch(dev);
  prof_end(g, KC_COMMIT);
  return check_launch("commit");
}

// A kernel whose bounded wait ran out raises the device error word; surface it as a failure of the call.
// `pre`: the two words of the device error flag if the caller has already brought them to the host (in stream order, after
// the step).  The kernels behind launch_linear keep their own error symbols; those are only read when such a kernel ran.
static int check_err_flag(Gpt* g, const int* pre = nullptr) {
  int ew[2] = {0, 0};   // [0] raised, [1] which wait of the owner-partitioned kernel ran out first (0: another kernel)
  if (pre) {
    ew[0] = pre[0];
    ew[1] = pre[1];
  } else {
    TSB_CUDA(cudaMemcpy(ew, g->err_flag, sizeof(ew), cudaMemcpyDeviceToHost));
  }
  int e = ew[0];
  if (g->lin_syms_used) {
    e |= tc_take_error();
    e |= gs_take_error();
    e |= stc_take_error();
    g->lin_syms_used = false;
  }
  if (g->tp > 1) e |= comm_peer_take_error();
#ifdef TSB200_CHECKED
  {
    int c = chk_take_engine();
    if (!c) c = chk_take_attention();
    if (!c) c = chk_take_moe();
    if (!c) c = chk_take_sampling();
    TSB_CHECK(c == 0, "checked build: device-side check 0x%x failed (an index or a capacity was out of range; the access was skipped)", c);
  }
#endif
  if (e) {
    cudaMemset(g->err_flag, 0, 2 * sizeof(int));
    if (g->stack_counters) cudaMemset(g->stack_counters, 0, (size_t)g->stack_counter_bytes);  // a kernel that gave up leaves them mid-count
    owner_reset_counters(g->own);
    if (g->tp > 1) owner_tp_failed(g->own);
    TSB_FAIL("a kernel gave up waiting (a dependency counter or a shared-memory barrier did not arrive within its limit; wait site 0x%x); "
             "the results of this call and the state of its sequences are invalid: reset or restore the cache before the next call", ew[1]);
  }
  return 1;
}

static uint64_t hash_blocked(const int32_t* b, int n) {
  uint64_t h = 0xcbf29ce484222325ull;
  for (int i = 0; i < n; ++i) {
    h ^= (uint32_t)b[i];
    h *= 0x100000001b3ull;
  }
  return h;
}

static int upload_blocked(Gpt* g, const TSB200DecodingOptions* opt) {
  TSB_CHECK(opt->n_blocked >= 0 && (opt->n_blocked == 0 || opt->blocked), "decoding options: blocked list is null");
  if (opt->n_blocked > g->blocked_cap) {
    void* p = nullptr;
    TSB_TRY(dev_alloc(g, &p, (int64_t)opt->n_blocked * 4 + 256, false));
    g->blocked = (int*)p;
    g->blocked_cap = opt->n_blocked + 64;
    if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  }
  if (opt->n_blocked) TSB_CUDA(cudaMemcpyAsync(g->blocked, opt->blocked, (size_t)opt->n_blocked * 4, cudaMemcpyHostToDevice, g->s));
  g->n_blocked = opt->n_blocked;
  return 1;
}

static int state_words(const Gpt* g) { return kStateLens + 2 * g->c.max_batch; }
// host mirrors of the per-sequence lengths / steps follow the scalars while the sequences agree
static void mirror_uniform(Gpt* g) {
  g->Ts.assign(g->c.max_batch, 0);
  g->steps_v.assign(g->c.max_batch, 0);
  for (int b = 0; b < g->B; ++b) {
    g->Ts[b] = g->T;
    g->steps_v[b] = (int)g->step;
  }
  g->ragged = g->force_per_seq;
}
// after a per-sequence change: the scalars hold the largest values, `ragged` says whether the sequences differ
static void refresh_ragged(Gpt* g) {
  int tmax = 0, smax = 0;
  bool differ = false;
  for (int b = 0; b < g->B; ++b) {
    tmax = g->Ts[b] > tmax ? g->Ts[b] : tmax;
    smax = g->steps_v[b] > smax ? g->steps_v[b] : smax;
    differ = differ || g->Ts[b] != g->Ts[0] || g->steps_v[b] != g->steps_v[0];
  }
  g->T = tmax;
  g->step = (uint32_t)smax;
  differ = differ || g->force_per_seq;
  if (differ != g->ragged && g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  g->ragged = differ;
}
static void fill_state(const Gpt* g, int* hst, int out_slot) {
  const int MB = g->c.max_batch;
  for (int i = 0; i < state_words(g); ++i) hst[i] = 0;
  hst[0] = g->T; hst[1] = (int)g->step; hst[2] = out_slot;
  hst[kStateRagged] = g->ragged ? 1 : 0;
  hst[kStateStepsAt] = kStateLens + MB;
  for (int b = 0; b < MB; ++b) {
    const bool have = b < (int)g->Ts.size();
    hst[kStateLens + b] = have ? g->Ts[b] : 0;
    hst[kStateLens + MB + b] = have ? g->steps_v[b] : 0;
  }
}
static int set_state(Gpt* g, int out_slot) {
  std::vector<int> hst(state_words(g));
  fill_state(g, hst.data(), out_slot);
  TSB_CUDA(cudaMemcpyAsync(g->state, hst.data(), hst.size() * sizeof(int), cudaMemcpyHostToDevice, g->s));
  TSB_CUDA(cudaStreamSynchronize(g->s));  // hst is pageable
  return 1;
}
// per-sequence lengths and steps as the device left them (a decode whose sequences advance on their own)
static int read_state(Gpt* g) {
  std::vector<int> hst(state_words(g));
  TSB_CUDA(cudaMemcpy(hst.data(), g->state, hst.size() * sizeof(int), cudaMemcpyDeviceToHost));
  const int MB = g->c.max_batch;
  for (int b = 0; b < g->B; ++b) {
    g->Ts[b] = hst[kStateLens + b];
    g->steps_v[b] = hst[kStateLens + MB + b];
  }
  refresh_ragged(g);
  return 1;
}

// Captures (or reuses) the CUDA graph of one decode step for the current batch and decoding options.
static int ensure_graph(Gpt* g, const TSB200DecodingOptions* opt, int n_steps) {
  const TSB200GptConfig& c = g->c;
  const int B = g->B;
  // split count for the attention kernel: fixed per graph, chosen for the longest cache this call reaches
  int Tp = 256;
  while (Tp < g->T + n_steps) Tp <<= 1;
  TSB_TRY(ensure_stack(g, B));
  GraphKey key;
  key.B = B; key.strategy = opt->strategy; key.splits = attn_pick_splits(g->st, c.dtype, B, c.H, c.Hkv, c.hd, Tp);
  key.n_blocked = opt->n_blocked; key.blocked_hash = hash_blocked(opt->blocked, opt->n_blocked);
  key.topP = opt->topP; key.temperature = opt->temperature; key.penalty = opt->repeatPenalty;
  key.seed = opt->seed; key.seq_base = opt->seq_base;
  key.ragged = g->ragged ? 1 : 0; key.stop_fin = g->stop_fin;
  if (g->gexec && g->gkey == key) return 1;
  if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  cudaGraph_t graph = nullptr;
  const long long l0 = g->st->launches;
  const bool prof = g->prof;
  g->prof = false;
  const bool syms_before = g->lin_syms_used;
  g->lin_syms_used = false;
  TSB_CUDA(cudaStreamBeginCapture(g->s, cudaStreamCaptureModeThreadLocal));
  int ok = enqueue_forward(g, B, 1, g->T, true, key.splits) && enqueue_sample(g, B, opt, true, true);
  cudaError_t e = cudaStreamEndCapture(g->s, &graph);
  g->graph_lin_syms = g->lin_syms_used;
  g->lin_syms_used = syms_before;
  g->prof = prof;
  if (!ok || e != cudaSuccess) {
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    if (ok) set_last_error("gpt_decode: graph capture failed: %s", cudaGetErrorString(e));
    return 0;
  }
  g->graph_nodes = g->st->launches - l0;
  g->st->launches = l0;  // captured launches have not run yet; replays are counted when launched
  e = cudaGraphInstantiate(&g->gexec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    g->gexec = nullptr;
    TSB_FAIL("gpt_decode: cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
  }
  g->gkey = key;
  return 1;
}

}  // namespace tsb

using namespace tsb;

extern "C" {

int TSB200_GptCreate(const TSB200GptConfig* cfg, void** out) {
  TSB_CHECK(cfg && out, "gpt_create: null argument");
  *out = nullptr;
  const TSB200GptConfig& c = *cfg;
  TSB_CHECK(c.L > 0 && c.d > 0 && c.H > 0 && c.hd > 0 && c.F > 0 && c.V > 0, "gpt_create: bad dimensions");
  TSB_CHECK(c.dtype == TSB200_F32 || c.dtype == TSB200_F16, "gpt_create: dtype must be F32 or F16");
  TSB_CHECK(c.norm_type == 0 || c.norm_type == 1, "gpt_create: norm_type must be 0 or 1");
  TSB_CHECK(c.act >= 0 && c.act <= 5, "gpt_create: unknown activation %d", c.act);
  TSB_CHECK(c.pe_type >= 0 && c.pe_type <= 2, "gpt_create: unknown position embedding type");
  TSB_CHECK(c.attn_type == 0 || c.attn_type == 1, "gpt_create: attn_type must be 0 (MHA) or 1 (GQA)");
  const int tp = c.tp_size > 1 ? c.tp_size : 1;
  TSB_CHECK(tp == 1 || (c.tp_rank >= 0 && c.tp_rank < tp), "gpt_create: tp_rank %d out of range for tp_size %d", c.tp_rank, tp);
  {
    const int hkv = c.attn_type == 0 ? c.H : c.Hkv;
    TSB_CHECK(tp == 1 || (c.H % tp == 0 && hkv % tp == 0 && c.F % tp == 0),
              "gpt_create: tensor parallel degree %d must divide the query heads (%d), KV heads (%d) and FFN width (%d)", tp, c.H, hkv, c.F);
  }
  TSB_CHECK(c.max_batch > 0 && c.max_batch <= 1024 && c.max_tokens > 0, "gpt_create: bad cache capacity");
  TSB_CHECK(!c.cross_attn || (c.max_src_tokens > 0 && c.tp_size <= 1 && c.attn_type == 0),
            "gpt_create: cross-attention engines need max_src_tokens > 0, one GPU and the MultiHeadAttention self-attention of TransformerDecoder");
  if (c.n_experts > 1) {
    TSB_CHECK(tp == 1, "gpt_create: mixture-of-experts models are not served tensor-parallel");
    TSB_CHECK(c.experts_per_token >= 1 && c.experts_per_token <= c.n_experts && c.experts_per_token <= 8 && c.n_experts <= 256,
              "gpt_create: %d experts with %d per token is not supported", c.n_experts, c.experts_per_token);
  }
  DeviceState* st;
  TSB_TRY(use_device(c.device, &st));
  Gpt* g = new Gpt();
  g->c = c;
  if (c.attn_type == 0) g->c.Hkv = c.H;
  g->tp = tp;
  g->tp_rank = tp > 1 ? c.tp_rank : 0;
  g->fullH = g->c.H; g->fullHkv = g->c.Hkv; g->fullF = g->c.F;
  g->c.H /= tp; g->c.Hkv /= tp; g->c.F /= tp;  // from here on the config holds this rank's share
  if (g->c.Hkv <= 0 || g->c.H % g->c.Hkv != 0) {
    delete g;
    TSB_FAIL("gpt_create: H must be divisible by Hkv");
  }
  if (g->c.n_experts <= 1) {
    g->c.n_experts = 1;
    g->c.experts_per_token = 1;
  }
  g->st = st;
  g->s = st->stream;
  g->es = c.dtype == TSB200_F16 ? 2 : 4;
  g->glu = (c.act == TSB200_ACT_GLU_NOACT || c.act == TSB200_ACT_SWIGLU) ? 1 : 0;
  {
    const char* e = getenv("TSB200_PDL");  // "0" switches programmatic dependent launch off (A/B measurements)
    g->pdl = !(e && e[0] == '0');
    e = getenv("TSB200_TP_PEER");
    g->tp_peer = !(e && e[0] == '0');
    e = getenv("TSB200_STACK");            // "0": one launch per operation instead of the persistent decode-step kernel
    g->use_stack = !(e && e[0] == '0');
    e = getenv("TSB200_FUSED_STEP");
    g->fuse_step = !(e && e[0] == '0');
    e = getenv("TSB200_STACK_MAXB");       // tuning knobs for the crossover between the three decode paths
    if (e) g->stack_cap = atoi(e);
    e = getenv("TSB200_GEMV_MAXROWS");
    if (e) g->gemv_rows = atoi(e);
    e = getenv("TSB200_OWNER");
    g->use_owner = !(e && e[0] == '0');
    e = getenv("TSB200_OWNER_MAXB");
    if (e) g->own_cap = atoi(e);
  }
  const TSB200GptConfig& cc = g->c;
  const int64_t d = cc.d, F = cc.F, V = cc.V, Hd = (int64_t)cc.H * cc.hd, KVd = (int64_t)cc.Hkv * cc.hd;
  g->Nqkv = (int)(Hd + 2 * KVd);
  const int es = g->es;
  auto fail = [&]() { TSB200_GptDestroy(g); return 0; };
#define G_ALLOC(p, bytes) if (!dev_alloc(g, (void**)&(p), (bytes))) return fail()
  G_ALLOC(g->E, V * d * es);
  if (cc.pe_type == 1) {
    g->pe_rows = cc.max_tokens + 2;  // rows = max length + 2 as in the reference (Applications/GPT.cs:128)
    G_ALLOC(g->PE, (int64_t)g->pe_rows * d * es);
  }
  G_ALLOC(g->nf_g, d * es);
  G_ALLOC(g->nf_b, d * es);
  G_ALLOC(g->head_w, packed_bytes(cc.dtype, (int)d, (int)V));
  G_ALLOC(g->head_b, V * es);
  g->L.resize(cc.L);
  const int64_t cache_elems = (int64_t)cc.max_batch * cc.Hkv * cc.max_tokens * cc.hd;
  for (int k = 0; k < cc.L; ++k) {
    LayerW& L = g->L[k];
    G_ALLOC(L.n1_g, d * es); G_ALLOC(L.n1_b, d * es); G_ALLOC(L.n2_g, d * es); G_ALLOC(L.n2_b, d * es);
    G_ALLOC(L.wqkv, packed_bytes(cc.dtype, (int)d, g->Nqkv)); G_ALLOC(L.bqkv, (int64_t)g->Nqkv * es);
    G_ALLOC(L.wo, packed_bytes(cc.dtype, (int)Hd, (int)d)); G_ALLOC(L.bo, d * es);
    L.moe = cc.n_experts > 1 && k > 1;   // Networks/GPTDecoder.cs:116
    if (L.moe) {
      const int64_t E = cc.n_experts, Fh = 4 * d;
      G_ALLOC(L.moe_g, d * es); G_ALLOC(L.moe_b, d * es);
      G_ALLOC(L.router_w, d * E * es); G_ALLOC(L.router_b, E * es);
      G_ALLOC(L.moe_w1, E * d * Fh * es); G_ALLOC(L.moe_w2, E * Fh * d * es);
      if (!fill_const(g, L.moe_g, d, 1.0f)) return fail();
    } else {
      G_ALLOC(L.w1, packed_bytes(cc.dtype, (int)d, (int)(F * (g->glu ? 2 : 1)))); G_ALLOC(L.b1, F * es * (g->glu ? 2 : 1));
      G_ALLOC(L.w2, packed_bytes(cc.dtype, (int)F, (int)d)); G_ALLOC(L.b2, d * es);
    }
    G_ALLOC(L.cK, cache_elems * es); G_ALLOC(L.cV, cache_elems * es);
    if (cc.cross_attn) {
      G_ALLOC(L.nx_g, d * es); G_ALLOC(L.nx_b, d * es);
      G_ALLOC(L.xq, packed_bytes(cc.dtype, (int)d, (int)Hd)); G_ALLOC(L.xqb, Hd * es);
      G_ALLOC(L.xk, packed_bytes(cc.dtype, (int)d, (int)Hd)); G_ALLOC(L.xkb, Hd * es);
      G_ALLOC(L.xv, packed_bytes(cc.dtype, (int)d, (int)Hd)); G_ALLOC(L.xvb, Hd * es);
      G_ALLOC(L.xo, packed_bytes(cc.dtype, (int)Hd, (int)d)); G_ALLOC(L.xob, d * es);
      const int64_t xe = (int64_t)cc.max_batch * cc.H * cc.max_src_tokens * cc.hd;
      G_ALLOC(L.xK, xe * es); G_ALLOC(L.xV, xe * es);
      if (!fill_const(g, L.nx_g, d, 1.0f)) return fail();
    }
    if (!fill_const(g, L.n1_g, d, 1.0f) || !fill_const(g, L.n2_g, d, 1.0f)) return fail();
  }
  if (!fill_const(g, g->nf_g, d, 1.0f)) return fail();
  if (cc.pe_type == 2) {
    G_ALLOC(g->rope_tab, (int64_t)cc.max_tokens * (cc.hd / 2) * sizeof(float2));
    if (!launch_rope_table(cc.device, st, g->rope_tab, cc.max_tokens, cc.hd, (double)cc.rope_base, g->s)) return fail();
  }
  const int MB = cc.max_batch;
  G_ALLOC(g->xl, (int64_t)MB * d * 4);
  if (tp > 1) G_ALLOC(g->ar_buf, (int64_t)MB * d * 4);
  G_ALLOC(g->hl, (int64_t)MB * d * es);
  G_ALLOC(g->logits, (int64_t)MB * V * 4);
  G_ALLOC(g->probs, (int64_t)MB * V * 4);
  G_ALLOC(g->u, (int64_t)MB * 4);
  G_ALLOC(g->ids_cur, (int64_t)MB * 4);
  G_ALLOC(g->ids_new, (int64_t)MB * 4);
  G_ALLOC(g->hist, (int64_t)MB * cc.max_tokens * 4);
  G_ALLOC(g->hist_len, (int64_t)MB * 4);
  G_ALLOC(g->state, (int64_t)(kStateLens + 2 * cc.max_batch) * 4 + 64);
  if (cc.cross_attn) G_ALLOC(g->cross_state, (int64_t)(kStateLens + 2 * cc.max_batch) * 4 + 64);
  mirror_uniform(g);
  G_ALLOC(g->out_dev, (int64_t)MB * (cc.max_tokens + 1) * 4);
  G_ALLOC(g->blocked, 1024);
  g->blocked_cap = 256;
  int64_t maxN = V > 2 * F ? V : 2 * F;
  if (g->Nqkv > maxN) maxN = g->Nqkv;
  g->lin_ws_bytes = linear_workspace_bytes(8, (int)(F > d ? F : d), (int)maxN);
  {
    const int shapes[5][2] = {{(int)d, g->Nqkv}, {(int)Hd, (int)d}, {(int)d, (int)(F * (g->glu ? 2 : 1))}, {(int)F, (int)d}, {(int)d, (int)V}};
    for (auto& sh : shapes) {
      const int64_t b = stream_workspace_bytes(cc.dtype, 4, sh[0], sh[1], st->sm_count);
      if (b > g->lin_ws_bytes) g->lin_ws_bytes = b;
    }
  }
  if (cc.dtype == TSB200_F16 && g->lin_ws_bytes < (64LL << 20)) g->lin_ws_bytes = 64LL << 20;  // split-K partials of the tensor-core GEMM
  G_ALLOC(g->lin_ws, g->lin_ws_bytes);
  G_ALLOC(g->err_flag, 64);
  g->attn_ws_bytes = attn_workspace_bytes(MB, cc.H, cc.hd, cc.max_tokens);
  G_ALLOC(g->attn_ws, g->attn_ws_bytes);
  g->topp_ws_bytes = TSB200_TopPWorkspaceBytes(MB, cc.V);
  G_ALLOC(g->topp_ws, g->topp_ws_bytes);
#undef G_ALLOC
  if (!init_linear_attrs(cc.device) || !init_topp_attrs(cc.device) || !init_stream_attrs(cc.device) || !init_tc_attrs(cc.device) || !init_stack_attrs(cc.device) || !init_owner_attrs()) return fail();
  if (cudaEventCreate(&g->ev0) != cudaSuccess || cudaEventCreate(&g->ev1) != cudaSuccess) {
    set_last_error("gpt_create: cudaEventCreate failed");
    return fail();
  }
  if (!ensure_act(g, MB)) return fail();
  if (cudaStreamSynchronize(g->s) != cudaSuccess) {
    set_last_error("gpt_create: initialisation failed: %s", cudaGetErrorString(cudaGetLastError()));
    return fail();
  }
  *out = g;
  return 1;
}

int TSB200_GptDestroy(void* h) {
  if (!h) return 1;
  Gpt* g = (Gpt*)h;
  cudaSetDevice(g->c.device);
  if (g->s) cudaStreamSynchronize(g->s);
  if (g->gexec) cudaGraphExecDestroy(g->gexec);
  if (g->ev0) cudaEventDestroy(g->ev0);
  if (g->ev1) cudaEventDestroy(g->ev1);
  for (auto e : g->prof_ev) cudaEventDestroy(e);
  for (auto e : g->step_ev) cudaEventDestroy(e);
  if (g->pin_ids) cudaFreeHost(g->pin_ids);
  for (int r = 0; r < kStackMaxRanks; ++r)
    if (g->xch_open[r]) cudaIpcCloseMemHandle(g->xch_peer[r]);
  if (g->xch_region) cudaFree(g->xch_region);
  owner_destroy(g->own);
  for (auto& a : g->allocs)
    if (a.base) cudaFree(a.base);
  delete g;
  return 1;
}

int TSB200_GptSetWeight(void* h, const char* name, const void* data, int dtype, int64_t rows, int64_t cols, int on_device) {
  NvtxRange nvtx_("tsb200.gpt.set_weight");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && name && data, "gpt_set_weight: null argument");
  TSB_CHECK(dtype == TSB200_F32 || dtype == TSB200_F16, "gpt_set_weight: data must be F32 or F16");
  TSB_TRY(use_device(g->c.device, nullptr));
  Dest dst;
  int nparts = 1;
  TSB_TRY(resolve(g, name, &dst, 0, &nparts));
  TSB_CHECK(rows * cols == dst.full_rows * dst.full_cols && (cols == dst.full_cols || rows * cols == dst.full_cols),
            "gpt_set_weight: '%s' expects the full tensor [%lld, %lld], got [%lld, %lld]", name, (long long)dst.full_rows,
            (long long)dst.full_cols, (long long)rows, (long long)cols);
  const int64_t bytes = rows * cols * (dtype == TSB200_F16 ? 2 : 4);
  const void* src = data;
  void* tmp = nullptr;
  if (!on_device) {
    cudaError_t e = cudaMalloc(&tmp, (size_t)bytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      TSB_FAIL("OOM: staging buffer of %lld bytes: %s", (long long)bytes, cudaGetErrorString(e));
    }
    if (cudaMemcpyAsync(tmp, data, (size_t)bytes, cudaMemcpyHostToDevice, g->s) != cudaSuccess) {
      cudaFree(tmp);
      TSB_FAIL("gpt_set_weight: host to device copy failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    src = tmp;
  }
  int ok = 1;
  for (int part = 0; part < nparts && ok; ++part) {
    ok = resolve(g, name, &dst, part, nullptr) && copy_into(g, dst, src, dtype);
  }
  if (ok && cudaStreamSynchronize(g->s) != cudaSuccess) {
    set_last_error("gpt_set_weight: %s", cudaGetErrorString(cudaGetLastError()));
    ok = 0;
  }
  if (tmp) cudaFree(tmp);
  if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  owner_invalidate(g->own);  // the per-CTA weight streams are rebuilt from the packed matrices on the next decode
  return ok;
}

int TSB200_GptGetWeightPtr(void* h, const char* name, void** ptr, int64_t* rows, int64_t* cols) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && name && ptr, "gpt_get_weight_ptr: null argument");
  Dest dst;
  TSB_TRY(resolve(g, name, &dst));
  TSB_CHECK(!dst.packed && dst.col_stride == 1 && dst.row_stride == dst.cols, "gpt_get_weight_ptr: '%s' is stored in the engine's packed layout", name);
  *ptr = dst.base;
  if (rows) *rows = dst.rows;
  if (cols) *cols = dst.cols;
  return 1;
}

int TSB200_GptFillSynthetic(void* h, uint64_t seed, float std, float bias_std) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g, "gpt_fill_synthetic: null engine");
  TSB_TRY(use_device(g->c.device, nullptr));
  std::vector<std::string> names = weight_names(g, bias_std > 0.0f, false, true);
  if (g->PE) names.push_back("PosEmbedding");
  int64_t max_elems = 0;
  for (auto& n : names) {
    Dest dst;
    TSB_TRY(resolve(g, n, &dst));
    if (dst.full_rows * dst.full_cols > max_elems) max_elems = dst.full_rows * dst.full_cols;
  }
  void* tmp = nullptr;
  cudaError_t e = cudaMalloc(&tmp, (size_t)max_elems * g->es);
  if (e != cudaSuccess) {
    cudaGetLastError();
    TSB_FAIL("OOM: synthetic staging buffer: %s", cudaGetErrorString(e));
  }
  int ok = 1;
  for (auto& n : names) {
    Dest dst;
    int nparts = 1;
    ok = resolve(g, n, &dst, 0, &nparts);
    if (!ok) break;
    const bool is_bias = ends_with(n, "m_Bd") || ends_with(n, "QKVb") || ends_with(n, ".Qb") || ends_with(n, ".Kb") ||
                         ends_with(n, ".Vb") || ends_with(n, ".b0") || ends_with(n, "m_RouterBias");
    // the FULL logical tensor is generated (every rank produces the same values) and this rank's block is kept
    ok = launch_synthetic(g->c.device, g->st, tmp, g->c.dtype, dst.full_rows * dst.full_cols, seed, fnv1a64(n.c_str()),
                          is_bias ? bias_std : std, g->s);
    for (int part = 0; part < nparts && ok; ++part) ok = resolve(g, n, &dst, part, nullptr) && copy_into(g, dst, tmp, g->c.dtype);
    if (!ok) break;
  }
  if (ok && cudaStreamSynchronize(g->s) != cudaSuccess) {
    set_last_error("gpt_fill_synthetic: %s", cudaGetErrorString(cudaGetLastError()));
    ok = 0;
  }
  cudaFree(tmp);
  if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  owner_invalidate(g->own);
  return ok;
}

int TSB200_GptTpExport(void* h, void* handle64) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && handle64, "gpt_tp_export: null argument");
  TSB_CHECK(g->tp > 1 && g->tp <= kStackMaxRanks, "gpt_tp_export: the engine is not tensor parallel (or has more than %d ranks)", kStackMaxRanks);
  TSB_TRY(use_device(g->c.device, nullptr));
  if (!g->xch_region) {
    g->xch_bytes = kStackXchHeader + (size_t)kStackXchSites * g->tp * kStackXchRows * g->c.d * sizeof(float);
    g->xch_bytes = (g->xch_bytes + 255) / 256 * 256;
    {
      // the owner-partitioned kernel's residual buffers and block counters follow (every rank computes the same offset)
      const TSB200GptConfig& c = g->c;
      OwnDims D{};
      D.L = c.L; D.d = c.d; D.H = c.H; D.Hkv = c.Hkv; D.hd = c.hd; D.F = c.F; D.V = c.V; D.glu = g->glu;
      if (owner_applicable(D, c.dtype, g->st->sm_count)) {
        g->xch_own_off = g->xch_bytes;
        g->xch_bytes += (size_t)owner_xch_bytes(D);
      }
    }
    TSB_CUDA(cudaMalloc((void**)&g->xch_region, g->xch_bytes));
    TSB_CUDA(cudaMemset(g->xch_region, 0, g->xch_bytes));
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t hd;
  TSB_CUDA(cudaIpcGetMemHandle(&hd, g->xch_region));
  std::memcpy(handle64, &hd, sizeof(hd));
  return 1;
}

int TSB200_GptTpImport(void* h, const void* handles, int n) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && handles && n == g->tp && g->xch_region, "gpt_tp_import: bad arguments (export first; one 64-byte handle per rank)");
  TSB_TRY(use_device(g->c.device, nullptr));
  for (int r = 0; r < n; ++r) {
    if (r == g->tp_rank) {
      g->xch_peer[r] = g->xch_region;
      continue;
    }
    cudaIpcMemHandle_t hd;
    std::memcpy(&hd, (const unsigned char*)handles + (size_t)r * 64, sizeof(hd));
    void* p = nullptr;
    TSB_CUDA(cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess));
    g->xch_peer[r] = (unsigned char*)p;
    g->xch_open[r] = true;
  }
  g->xch_ready = true;
  if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  g->stack_key = nullptr;  // the program is rebuilt with the exchange
  return 1;
}

// First phase of a collective teardown of a tensor-parallel engine: waits for this device's work, drops the captured
// step and the program that hold the peers' addresses, and unmaps the peers' exchange regions.  Every rank calls it, the
// ranks meet at a host-side barrier, and only then each rank frees its own region (TSB200_GptDestroy).
int TSB200_GptTpClose(void* h) {
  Gpt* g = (Gpt*)h;
  if (!g) return 1;
  TSB_TRY(use_device(g->c.device, nullptr));
  cudaDeviceSynchronize();
  if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  g->stack_key = nullptr;
  g->stack_B = 0;
  g->own_B = 0;
  g->xch_ready = false;
  for (int r = 0; r < kStackMaxRanks; ++r)
    if (g->xch_open[r]) {
      cudaIpcCloseMemHandle(g->xch_peer[r]);
      g->xch_open[r] = false;
      g->xch_peer[r] = nullptr;
    }
  cudaGetLastError();
  return 1;
}

int TSB200_GptSetComm(void* h, void* comm) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g, "gpt_set_comm: null engine");
  TSB_CHECK(!comm || (comm_nranks(comm) == g->tp && comm_rank(comm) == g->tp_rank),
            "gpt_set_comm: communicator is rank %d of %d but the engine is rank %d of %d", comm_rank(comm), comm_nranks(comm), g->tp_rank, g->tp);
  g->comm = comm;
  if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  return 1;
}

int TSB200_GptReset(void* h) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g, "gpt_reset: null engine");
  TSB_TRY(use_device(g->c.device, nullptr));
  g->B = 0;
  g->T = 0;
  g->step = 0;
  g->probs_valid = false;
  if (g->ragged && g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  mirror_uniform(g);
  TSB_CUDA(cudaMemsetAsync(g->hist_len, 0, (size_t)g->c.max_batch * 4, g->s));
  return 1;
}

}  // extern "C"

// Runs S prompt tokens per sequence through the stack on top of T0 = g->T cached positions (0: a fresh prompt;
// > 0: the suffix of a prompt whose first T0 tokens are already cached), samples the next id.
// `plen` (prefill only, or NULL): the prompts' own lengths; shorter prompts are padded to S columns (the pad ids are
// ignored: every sequence continues from its own last token, as if it had been run alone).
static int run_prompt(Gpt* g, const int32_t* ids, int B, int S, const TSB200DecodingOptions* opt, int32_t* out_ids, bool extend,
                      const int32_t* plen = nullptr) {
  const TSB200GptConfig& c = g->c;
  const int T0 = g->T;
  if (extend) {
    TSB_CHECK(T0 > 0 && g->B > 0, "gpt_extend: nothing is cached (prefill or restore a snapshot first)");
    TSB_CHECK(B == g->B, "gpt_extend: batch %d differs from the cached batch %d", B, g->B);
    TSB_CHECK(!g->ragged, "gpt_extend: the sequences have different lengths; extend them one by one (TSB200_GptSlotExtend)");
  } else {
    TSB_CHECK(T0 == 0, "gpt_prefill: the cache is not empty (call TSB200_GptReset first)");
    TSB_CHECK(B > 0 && B <= c.max_batch, "gpt_prefill: batch %d exceeds capacity %d", B, c.max_batch);
  }
  TSB_CHECK(S > 0 && T0 + S < c.max_tokens, "OOM: prompt of %d tokens exceeds the KV-cache capacity %d", T0 + S, c.max_tokens);
  for (int64_t i = 0; i < (int64_t)B * S; ++i) TSB_CHECK(ids[i] >= 0 && ids[i] < c.V, "gpt_prefill: token id %d out of range", ids[i]);
  if (plen) {
    TSB_CHECK(g->tp == 1, "gpt_prefill: prompts of different lengths are not served by tensor-parallel engines");
    for (int b = 0; b < B; ++b) TSB_CHECK(plen[b] >= 1 && plen[b] <= S, "gpt_prefill: prompt length %d of sequence %d is outside [1, %d]", plen[b], b, S);
  }
  TSB_TRY(ensure_act(g, (int64_t)B * S));
  void* ids_dev = nullptr;
  TSB_CUDA(cudaMalloc(&ids_dev, (size_t)B * S * 4));
  g->ids_in = (int*)ids_dev;
  int ok = 1;
  do {
    if (cudaMemcpyAsync(ids_dev, ids, (size_t)B * S * 4, cudaMemcpyHostToDevice, g->s) != cudaSuccess) { ok = 0; set_last_error("gpt_prefill: id upload failed"); break; }
    // history = the prompt (the reference passes the whole sequence as decodedSequence: Decoder.cs:761)
    //  an extension overwrites the pending id at position T0: the caller's tokens are the text from there on
    if (cudaMemcpy2DAsync(g->hist + T0, (size_t)c.max_tokens * 4, ids_dev, (size_t)S * 4, (size_t)S * 4, B, cudaMemcpyDeviceToDevice, g->s) != cudaSuccess) { ok = 0; set_last_error("gpt_prefill: history copy failed"); break; }
    std::vector<int> lens(B, T0 + S);
    if (plen)
      for (int b = 0; b < B; ++b) lens[b] = plen[b];
    if (cudaMemcpyAsync(g->hist_len, lens.data(), (size_t)B * 4, cudaMemcpyHostToDevice, g->s) != cudaSuccess) { ok = 0; set_last_error("gpt_prefill: history length upload failed"); break; }
    cudaStreamSynchronize(g->s);
    g->B = B;
    if (!extend) g->step = 0;
    mirror_uniform(g);
    if (plen) {   // the device state already holds the lengths the prompts END with: the last-row gather reads them
      for (int b = 0; b < B; ++b) g->Ts[b] = plen[b];
      refresh_ragged(g);
      g->T = T0;  // the forward pass below still starts from an empty cache
    }
    if (!(ok = upload_blocked(g, opt))) break;
    if (!(ok = set_state(g, 0))) break;
    const long long l0 = g->st->launches;
    cudaEventRecord(g->ev0, g->s);
    g->gather_lens = plen ? g->state + kStateLens : nullptr;
    ok = enqueue_forward(g, B, S, T0, false, 1);
    g->gather_lens = nullptr;
    if (!ok) break;
    g->T = T0 + S;
    if (plen) refresh_ragged(g);   // T = the longest prompt
    if (!(ok = enqueue_sample(g, B, opt, true, false))) break;
    cudaEventRecord(g->ev1, g->s);
    if (cudaStreamSynchronize(g->s) != cudaSuccess) { ok = 0; set_last_error("gpt_prefill: %s", cudaGetErrorString(cudaGetLastError())); break; }
    cudaEventElapsedTime(&g->last_ms, g->ev0, g->ev1);
    if (!(ok = check_err_flag(g))) break;
    g->last_launches = g->st->launches - l0;
    g->step += 1;
    for (int b = 0; b < B; ++b) {
      g->steps_v[b] += 1;
      if (!plen) g->Ts[b] = g->T;
    }
    g->probs_valid = (opt->strategy == 1);
    if (out_ids && cudaMemcpy(out_ids, g->out_dev, (size_t)B * 4, cudaMemcpyDeviceToHost) != cudaSuccess) { ok = 0; set_last_error("gpt_prefill: id download failed"); break; }
  } while (0);
  g->ids_in = nullptr;
  cudaFree(ids_dev);
  return ok;
}

extern "C" {

int TSB200_GptPrefill(void* h, const int32_t* ids, int B, int S, const TSB200DecodingOptions* opt, int32_t* out_ids) {
  NvtxRange nvtx_("tsb200.gpt.prefill");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && ids && opt, "gpt_prefill: null argument");
  TSB_TRY(use_device(g->c.device, nullptr));
  return run_prompt(g, ids, B, S, opt, out_ids, false);
}

int TSB200_GptPrefillRagged(void* h, const int32_t* ids, const int32_t* lens, int B, int S, const TSB200DecodingOptions* opt,
                            int32_t* out_ids) {
  NvtxRange nvtx_("tsb200.gpt.prefill_ragged");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && ids && lens && opt, "gpt_prefill_ragged: null argument");
  TSB_TRY(use_device(g->c.device, nullptr));
  return run_prompt(g, ids, B, S, opt, out_ids, false, lens);
}

int TSB200_GptExtend(void* h, const int32_t* ids, int B, int S, const TSB200DecodingOptions* opt, int32_t* out_ids) {
  NvtxRange nvtx_("tsb200.gpt.extend");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && ids && opt, "gpt_extend: null argument");
  TSB_TRY(use_device(g->c.device, nullptr));
  return run_prompt(g, ids, B, S, opt, out_ids, true);
}

int TSB200_GptDecode(void* h, int n_steps, const TSB200DecodingOptions* opt, int stop_on_eos, int32_t* out_ids, int* steps_done) {
  NvtxRange nvtx_("tsb200.gpt.decode");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && opt, "gpt_decode: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_CHECK(g->T > 0 && g->B > 0, "gpt_decode: prefill first");
  TSB_CHECK(n_steps >= 0, "gpt_decode: negative step count");
  // the step that generates token n appends position T + n - 1
  TSB_CHECK(g->T + n_steps <= c.max_tokens, "OOM: KV-cache capacity %d exceeded (%d cached + %d steps)", c.max_tokens, g->T, n_steps);
  if (steps_done) *steps_done = 0;
  if (n_steps == 0) return 1;
  const int B = g->B;
  TSB_TRY(upload_blocked(g, opt));
  g->stop_fin = (g->ragged && stop_on_eos) ? 1 : 0;   // sequences with their own lengths stop one by one
  TSB_TRY(set_state(g, 0));
  TSB_TRY(ensure_graph(g, opt, n_steps));
  std::vector<int> last(B);
  int done = 0;
  if (g->step_timing) {
    while ((int)g->step_ev.size() < n_steps + 1) {
      cudaEvent_t e;
      TSB_CUDA(cudaEventCreate(&e));
      g->step_ev.push_back(e);
    }
  }
  g->step_ev_n = 0;
  TSB_CUDA(cudaEventRecord(g->ev0, g->s));
  if (g->step_timing) TSB_CUDA(cudaEventRecord(g->step_ev[0], g->s));
  for (int i = 0; i < n_steps; ++i) {
    TSB_CUDA(cudaGraphLaunch(g->gexec, g->s));
    g->lin_syms_used = g->lin_syms_used || g->graph_lin_syms;
    count_launch(c.device, g->graph_nodes);
    ++done;
    if (g->step_timing) {
      TSB_CUDA(cudaEventRecord(g->step_ev[i + 1], g->s));
      g->step_ev_n = i + 1;
    }
    if (stop_on_eos) {
      // the reference reads the ids back every token to test its stop rule (Decoder.cs:769-782, GPT.cs:300-303)
      TSB_CUDA(cudaMemcpyAsync(last.data(), g->ids_cur, (size_t)B * 4, cudaMemcpyDeviceToHost, g->s));
      TSB_CUDA(cudaStreamSynchronize(g->s));
      bool all_eos = true;
      for (int b = 0; b < B; ++b) all_eos = all_eos && (last[b] == 0);
      if (all_eos) break;
    }
  }
  TSB_CUDA(cudaEventRecord(g->ev1, g->s));
  TSB_CUDA(cudaStreamSynchronize(g->s));
  TSB_CUDA(cudaEventElapsedTime(&g->last_ms, g->ev0, g->ev1));
  TSB_TRY(check_err_flag(g));
  g->last_launches = g->graph_nodes * done;
  if (g->ragged) {
    TSB_TRY(read_state(g));   // finished sequences did not advance
  } else {
    g->T += done;
    g->step += (uint32_t)done;
    for (int b = 0; b < B; ++b) {
      g->Ts[b] = g->T;
      g->steps_v[b] = (int)g->step;
    }
  }
  g->probs_valid = (opt->strategy == 1);
  if (steps_done) *steps_done = done;
  if (out_ids) {
    std::vector<int> tmp((size_t)done * B);
    TSB_CUDA(cudaMemcpy(tmp.data(), g->out_dev, tmp.size() * 4, cudaMemcpyDeviceToHost));
    for (int b = 0; b < B; ++b)
      for (int i = 0; i < n_steps; ++i) out_ids[(int64_t)b * n_steps + i] = i < done ? tmp[(size_t)i * B + b] : 0;
  }
  return 1;
}

int TSB200_GptGetLogits(void* h, float* logits, float* probs) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g, "gpt_get_logits: null engine");
  TSB_TRY(use_device(g->c.device, nullptr));
  TSB_CHECK(g->B > 0, "gpt_get_logits: nothing has run yet");
  const size_t n = (size_t)g->B * g->c.V;
  if (logits) TSB_CUDA(cudaMemcpy(logits, g->logits, n * 4, cudaMemcpyDeviceToHost));
  if (probs) {
    if (!g->probs_valid) {
      TSB_TRY(launch_softmax_argmax(g->c.device, g->st, nullptr, g->probs, g->logits, g->B, g->c.V, 1.0f, 0, g->blocked, g->n_blocked, g->s));
      TSB_CUDA(cudaStreamSynchronize(g->s));
    }
    TSB_CUDA(cudaMemcpy(probs, g->probs, n * 4, cudaMemcpyDeviceToHost));
  }
  return 1;
}

int TSB200_GptCheckGuards(void* h) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g, "gpt_check_guards: null engine");
  TSB_TRY(use_device(g->c.device, nullptr));
  TSB_CUDA(cudaStreamSynchronize(g->s));
  unsigned char host[2 * kGuardBytes];
  int idx = 0;
  for (const auto& a : g->allocs) {
    ++idx;
    if (!a.base) continue;
    TSB_CUDA(cudaMemcpy(host, a.base, kGuardBytes, cudaMemcpyDeviceToHost));
    TSB_CUDA(cudaMemcpy(host + kGuardBytes, (const char*)a.user + a.bytes, kGuardBytes, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < 2 * kGuardBytes; ++i)
      TSB_CHECK(host[i] == (unsigned char)kGuardByte,
                "gpt_check_guards: buffer %d of the engine (%zu bytes) was written out of bounds: guard byte %zu %s it is 0x%02x", idx, a.bytes,
                i % kGuardBytes, i < kGuardBytes ? "before" : "after", host[i]);
  }
  return 1;
}

int TSB200_GptDecodePath(void* h, int* path) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && path, "gpt_decode_path: null argument");
  *path = g->last_path;
  return 1;
}

int TSB200_GptCacheLength(void* h, int* T) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && T, "gpt_cache_length: null argument");
  *T = g->T;
  return 1;
}

int TSB200_GptCacheLengths(void* h, int* lens, int n) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && lens && n >= 0, "gpt_cache_lengths: bad arguments");
  for (int b = 0; b < n; ++b) lens[b] = b < g->B ? g->Ts[b] : 0;
  return 1;
}

}  // extern "C"

// A parked KV cache: rows [0, T) of every layer's K and V for B sequences, compacted, plus what a later call needs
// to continue the text (token history, the pending id, the sampling step counter).
struct GptSnapshot {
  int device = 0, B = 0, T = 0, L = 0, Hkv = 0, hd = 0, es = 0;
  uint32_t step = 0;
  void* kv = nullptr;          // [L][2][B * Hkv][T * hd] elements
  size_t bytes = 0;
  std::vector<int> hist;       // [B][T + 1]: the cached tokens and the pending one
  std::vector<int> pending;    // [B]
};

extern "C" {

int TSB200_GptCacheSnapshot(void* h, void** snap_out) {
  NvtxRange nvtx_("tsb200.gpt.cache_snapshot");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && snap_out, "gpt_cache_snapshot: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_CHECK(g->T > 0 && g->B > 0, "gpt_cache_snapshot: nothing is cached");
  TSB_CHECK(!g->ragged, "gpt_cache_snapshot: the sequences have different lengths; park them one by one (TSB200_GptSlotSnapshot)");
  GptSnapshot* sn = new GptSnapshot();
  sn->device = c.device; sn->B = g->B; sn->T = g->T; sn->L = c.L; sn->Hkv = c.Hkv; sn->hd = c.hd; sn->es = g->es;
  sn->step = g->step;
  const size_t row = (size_t)sn->T * c.hd * g->es, pitch = (size_t)c.max_tokens * c.hd * g->es;
  const size_t rows = (size_t)sn->B * c.Hkv;
  sn->bytes = (size_t)c.L * 2 * rows * row;
  auto fail = [&]() { if (sn->kv) cudaFree(sn->kv); delete sn; return 0; };
  if (cudaMalloc(&sn->kv, sn->bytes) != cudaSuccess) {
    cudaGetLastError();
    set_last_error("OOM: gpt_cache_snapshot could not allocate %zu bytes", sn->bytes);
    return fail();
  }
  for (int k = 0; k < c.L; ++k)
    for (int w = 0; w < 2; ++w) {
      unsigned char* dst = (unsigned char*)sn->kv + ((size_t)k * 2 + w) * rows * row;
      const void* src = w == 0 ? g->L[k].cK : g->L[k].cV;
      if (cudaMemcpy2DAsync(dst, row, src, pitch, row, rows, cudaMemcpyDeviceToDevice, g->s) != cudaSuccess) {
        set_last_error("gpt_cache_snapshot: cache copy failed");
        return fail();
      }
    }
  sn->hist.assign((size_t)sn->B * (sn->T + 1), 0);
  sn->pending.assign(sn->B, 0);
  // a cache decoded to capacity has no history slot for the pending id (it stays in `pending`)
  const size_t hist_w = (size_t)(sn->T + 1 <= c.max_tokens ? sn->T + 1 : c.max_tokens) * 4;
  if (cudaMemcpy2DAsync(sn->hist.data(), (size_t)(sn->T + 1) * 4, g->hist, (size_t)c.max_tokens * 4, hist_w, sn->B,
                        cudaMemcpyDeviceToHost, g->s) != cudaSuccess ||
      cudaMemcpyAsync(sn->pending.data(), g->ids_cur, (size_t)sn->B * 4, cudaMemcpyDeviceToHost, g->s) != cudaSuccess ||
      cudaStreamSynchronize(g->s) != cudaSuccess) {
    set_last_error("gpt_cache_snapshot: %s", cudaGetErrorString(cudaGetLastError()));
    return fail();
  }
  *snap_out = sn;
  return 1;
}

int TSB200_GptCacheSnapshotInfo(void* snap, int* B, int* T, int64_t* bytes, int32_t* tokens) {
  GptSnapshot* sn = (GptSnapshot*)snap;
  TSB_CHECK(sn, "gpt_cache_snapshot_info: null snapshot");
  if (B) *B = sn->B;
  if (T) *T = sn->T;
  if (bytes) *bytes = (int64_t)sn->bytes;
  if (tokens) std::memcpy(tokens, sn->hist.data(), sn->hist.size() * 4);
  return 1;
}

int TSB200_GptCacheSnapshotFree(void* snap) {
  GptSnapshot* sn = (GptSnapshot*)snap;
  if (!sn) return 1;
  TSB_TRY(use_device(sn->device, nullptr));
  if (sn->kv) cudaFree(sn->kv);
  delete sn;
  return 1;
}

int TSB200_GptCacheRestore(void* h, void* snap, int B_new) {
  NvtxRange nvtx_("tsb200.gpt.cache_restore");
  Gpt* g = (Gpt*)h;
  GptSnapshot* sn = (GptSnapshot*)snap;
  TSB_CHECK(g && sn, "gpt_cache_restore: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_CHECK(sn->device == c.device && sn->L == c.L && sn->Hkv == c.Hkv && sn->hd == c.hd && sn->es == g->es,
            "gpt_cache_restore: the snapshot was taken from a different model or device");
  if (B_new <= 0) B_new = sn->B;
  TSB_CHECK(B_new == sn->B || sn->B == 1, "gpt_cache_restore: a snapshot of %d sequences cannot serve %d", sn->B, B_new);
  TSB_CHECK(B_new <= c.max_batch, "gpt_cache_restore: batch %d exceeds capacity %d", B_new, c.max_batch);
  TSB_CHECK(sn->T < c.max_tokens, "OOM: snapshot of %d tokens exceeds the KV-cache capacity %d", sn->T, c.max_tokens);
  const size_t row = (size_t)sn->T * c.hd * g->es, pitch = (size_t)c.max_tokens * c.hd * g->es;
  const size_t rows = (size_t)sn->B * c.Hkv;
  const int copies = (B_new == sn->B) ? 1 : B_new;  // one sequence parked, many served: the rows go to every slot
  for (int k = 0; k < c.L; ++k)
    for (int w = 0; w < 2; ++w) {
      const unsigned char* src = (const unsigned char*)sn->kv + ((size_t)k * 2 + w) * rows * row;
      unsigned char* dst = (unsigned char*)(w == 0 ? g->L[k].cK : g->L[k].cV);
      for (int r = 0; r < copies; ++r)
        TSB_CUDA(cudaMemcpy2DAsync(dst + (size_t)r * c.Hkv * pitch, pitch, src, row, row, rows, cudaMemcpyDeviceToDevice, g->s));
    }
  std::vector<int> lens(B_new, sn->T + 1), pend(B_new);
  for (int b = 0; b < B_new; ++b) {
    const int sb = (B_new == sn->B) ? b : 0;
    pend[b] = sn->pending[sb];
    TSB_CUDA(cudaMemcpyAsync(g->hist + (size_t)b * c.max_tokens, sn->hist.data() + (size_t)sb * (sn->T + 1), (size_t)(sn->T + 1) * 4,
                             cudaMemcpyHostToDevice, g->s));
  }
  TSB_CUDA(cudaMemcpyAsync(g->hist_len, lens.data(), (size_t)B_new * 4, cudaMemcpyHostToDevice, g->s));
  TSB_CUDA(cudaMemcpyAsync(g->ids_cur, pend.data(), (size_t)B_new * 4, cudaMemcpyHostToDevice, g->s));
  TSB_CUDA(cudaStreamSynchronize(g->s));  // lens / pend are on the stack
  if (g->ragged && g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
  g->B = B_new;
  g->T = sn->T;
  g->step = sn->step;
  mirror_uniform(g);
  g->probs_valid = false;
  return 1;
}

// ---- one sequence of the batch at a time: park it, replace it, give it more prompt, while the others keep their state
int TSB200_GptSlotSnapshot(void* h, int slot, void** snap_out) {
  NvtxRange nvtx_("tsb200.gpt.slot_snapshot");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && snap_out, "gpt_slot_snapshot: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_CHECK(slot >= 0 && slot < g->B && g->Ts[slot] > 0, "gpt_slot_snapshot: sequence %d holds nothing", slot);
  GptSnapshot* sn = new GptSnapshot();
  sn->device = c.device; sn->B = 1; sn->T = g->Ts[slot]; sn->L = c.L; sn->Hkv = c.Hkv; sn->hd = c.hd; sn->es = g->es;
  sn->step = (uint32_t)g->steps_v[slot];
  const size_t row = (size_t)sn->T * c.hd * g->es, pitch = (size_t)c.max_tokens * c.hd * g->es;
  const size_t rows = (size_t)c.Hkv;
  sn->bytes = (size_t)c.L * 2 * rows * row;
  auto fail = [&]() { if (sn->kv) cudaFree(sn->kv); delete sn; return 0; };
  if (cudaMalloc(&sn->kv, sn->bytes) != cudaSuccess) {
    cudaGetLastError();
    set_last_error("OOM: gpt_slot_snapshot could not allocate %zu bytes", sn->bytes);
    return fail();
  }
  for (int k = 0; k < c.L; ++k)
    for (int w = 0; w < 2; ++w) {
      unsigned char* dst = (unsigned char*)sn->kv + ((size_t)k * 2 + w) * rows * row;
      const unsigned char* src = (const unsigned char*)(w == 0 ? g->L[k].cK : g->L[k].cV) + (size_t)slot * c.Hkv * pitch;
      if (cudaMemcpy2DAsync(dst, row, src, pitch, row, rows, cudaMemcpyDeviceToDevice, g->s) != cudaSuccess) {
        set_last_error("gpt_slot_snapshot: cache copy failed");
        return fail();
      }
    }
  sn->hist.assign((size_t)sn->T + 1, 0);
  sn->pending.assign(1, 0);
  const size_t hist_w = (size_t)(sn->T + 1 <= c.max_tokens ? sn->T + 1 : c.max_tokens) * 4;
  if (cudaMemcpyAsync(sn->hist.data(), g->hist + (size_t)slot * c.max_tokens, hist_w, cudaMemcpyDeviceToHost, g->s) != cudaSuccess ||
      cudaMemcpyAsync(sn->pending.data(), g->ids_cur + slot, 4, cudaMemcpyDeviceToHost, g->s) != cudaSuccess ||
      cudaStreamSynchronize(g->s) != cudaSuccess) {
    set_last_error("gpt_slot_snapshot: %s", cudaGetErrorString(cudaGetLastError()));
    return fail();
  }
  *snap_out = sn;
  return 1;
}

// slot == the number of sequences: the batch grows by one
static int slot_claim(Gpt* g, int slot, const char* who) {
  TSB_CHECK(g->tp == 1, "%s: tensor-parallel engines serve one set of sequences of equal length", who);
  TSB_CHECK(slot >= 0 && slot <= g->B && slot < g->c.max_batch, "%s: sequence index %d out of range (%d in use, capacity %d)", who, slot, g->B,
            g->c.max_batch);
  if (slot == g->B) {
    if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }
    g->B += 1;
    g->Ts[slot] = 0;
    g->steps_v[slot] = 0;
  }
  return 1;
}

int TSB200_GptSlotReset(void* h, int slot) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g, "gpt_slot_reset: null engine");
  TSB_TRY(use_device(g->c.device, nullptr));
  TSB_TRY(slot_claim(g, slot, "gpt_slot_reset"));
  g->Ts[slot] = 0;
  g->steps_v[slot] = 0;
  TSB_CUDA(cudaMemsetAsync(g->hist_len + slot, 0, 4, g->s));
  TSB_CUDA(cudaMemsetAsync(g->ids_cur + slot, 0, 4, g->s));   // pending id </s>: with stop_on_eos an empty slot stands still
  refresh_ragged(g);
  g->probs_valid = false;
  return 1;
}

int TSB200_GptSetPerSequenceState(void* h, int on) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g, "gpt_set_per_sequence_state: null engine");
  TSB_CHECK(g->tp == 1 || !on, "gpt_set_per_sequence_state: tensor-parallel engines serve sequences of equal length");
  g->force_per_seq = on != 0;
  if (g->Ts.empty()) mirror_uniform(g);
  refresh_ragged(g);
  return 1;
}

int TSB200_GptSlotRestore(void* h, void* snap, int slot) {
  NvtxRange nvtx_("tsb200.gpt.slot_restore");
  Gpt* g = (Gpt*)h;
  GptSnapshot* sn = (GptSnapshot*)snap;
  TSB_CHECK(g && sn, "gpt_slot_restore: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_CHECK(sn->device == c.device && sn->L == c.L && sn->Hkv == c.Hkv && sn->hd == c.hd && sn->es == g->es,
            "gpt_slot_restore: the snapshot was taken from a different model or device");
  TSB_CHECK(sn->B == 1, "gpt_slot_restore: the snapshot holds %d sequences; a slot takes one", sn->B);
  TSB_CHECK(sn->T < c.max_tokens, "OOM: snapshot of %d tokens exceeds the KV-cache capacity %d", sn->T, c.max_tokens);
  TSB_TRY(slot_claim(g, slot, "gpt_slot_restore"));
  const size_t row = (size_t)sn->T * c.hd * g->es, pitch = (size_t)c.max_tokens * c.hd * g->es;
  const size_t rows = (size_t)c.Hkv;
  for (int k = 0; k < c.L; ++k)
    for (int w = 0; w < 2; ++w) {
      const unsigned char* src = (const unsigned char*)sn->kv + ((size_t)k * 2 + w) * rows * row;
      unsigned char* dst = (unsigned char*)(w == 0 ? g->L[k].cK : g->L[k].cV) + (size_t)slot * c.Hkv * pitch;
      TSB_CUDA(cudaMemcpy2DAsync(dst, pitch, src, row, row, rows, cudaMemcpyDeviceToDevice, g->s));
    }
  const int len = sn->T + 1;
  TSB_CUDA(cudaMemcpyAsync(g->hist + (size_t)slot * c.max_tokens, sn->hist.data(), (size_t)len * 4, cudaMemcpyHostToDevice, g->s));
  TSB_CUDA(cudaMemcpyAsync(g->hist_len + slot, &len, 4, cudaMemcpyHostToDevice, g->s));
  TSB_CUDA(cudaMemcpyAsync(g->ids_cur + slot, sn->pending.data(), 4, cudaMemcpyHostToDevice, g->s));
  TSB_CUDA(cudaStreamSynchronize(g->s));  // `len` is on the stack
  g->Ts[slot] = sn->T;
  g->steps_v[slot] = (int)sn->step;
  refresh_ragged(g);
  g->probs_valid = false;
  return 1;
}

// S prompt tokens for ONE sequence on top of what it has cached (nothing after TSB200_GptSlotReset), then its next id.
// The run addresses the sequence's rows of every per-sequence buffer; the other sequences are not touched.
int TSB200_GptSlotExtend(void* h, int slot, const int32_t* ids, int S, const TSB200DecodingOptions* opt, int32_t* out_id) {
  NvtxRange nvtx_("tsb200.gpt.slot_extend");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && ids && opt, "gpt_slot_extend: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_TRY(slot_claim(g, slot, "gpt_slot_extend"));
  const int T0 = g->Ts[slot];
  TSB_CHECK(S > 0 && T0 + S < c.max_tokens, "OOM: prompt of %d tokens exceeds the KV-cache capacity %d", T0 + S, c.max_tokens);
  for (int i = 0; i < S; ++i) TSB_CHECK(ids[i] >= 0 && ids[i] < c.V, "gpt_slot_extend: token id %d out of range", ids[i]);
  TSB_TRY(ensure_act(g, (int64_t)S));
  void* ids_dev = nullptr;
  TSB_CUDA(cudaMalloc(&ids_dev, (size_t)S * 4));
  // the view of one sequence: every per-sequence pointer moves to the sequence's rows
  struct View {
    Gpt* g; int slot; std::vector<std::pair<void*, void*>> kv; int *hist, *hist_len, *ids_cur; uint32_t step;
    View(Gpt* g_, int slot_) : g(g_), slot(slot_), hist(g_->hist), hist_len(g_->hist_len), ids_cur(g_->ids_cur), step(g_->step) {
      const size_t pitch = (size_t)g->c.max_tokens * g->c.hd * g->es * g->c.Hkv;
      for (LayerW& L : g->L) {
        kv.push_back({L.cK, L.cV});
        L.cK = (char*)L.cK + (size_t)slot * pitch;
        L.cV = (char*)L.cV + (size_t)slot * pitch;
      }
      g->hist += (size_t)slot * g->c.max_tokens;
      g->hist_len += slot;
      g->ids_cur += slot;
      g->seq0 = slot;
      g->step = (uint32_t)g->steps_v[slot];
    }
    ~View() {
      for (size_t k = 0; k < kv.size(); ++k) { g->L[k].cK = kv[k].first; g->L[k].cV = kv[k].second; }
      g->hist = hist; g->hist_len = hist_len; g->ids_cur = ids_cur; g->seq0 = 0; g->step = step;
      g->ids_in = nullptr;
    }
  };
  int ok = 1;
  {
    // the device state is set for the whole batch first (the commit kernel counts the sequence's step there)
    if (!upload_blocked(g, opt) || !set_state(g, 0)) { cudaFree(ids_dev); return 0; }
    View view(g, slot);
    g->ids_in = (int*)ids_dev;
    TSB200DecodingOptions o2 = *opt;
    o2.seq_base += (uint64_t)slot;
    const int len = T0 + S;
    do {
      if (cudaMemcpyAsync(ids_dev, ids, (size_t)S * 4, cudaMemcpyHostToDevice, g->s) != cudaSuccess ||
          cudaMemcpyAsync(g->hist + T0, ids_dev, (size_t)S * 4, cudaMemcpyDeviceToDevice, g->s) != cudaSuccess ||
          cudaMemcpyAsync(g->hist_len, &len, 4, cudaMemcpyHostToDevice, g->s) != cudaSuccess ||
          cudaStreamSynchronize(g->s) != cudaSuccess) { ok = 0; set_last_error("gpt_slot_extend: upload failed"); break; }
      const long long l0 = g->st->launches;
      cudaEventRecord(g->ev0, g->s);
      if (!(ok = enqueue_forward(g, 1, S, T0, false, 1))) break;
      if (!(ok = enqueue_sample(g, 1, &o2, false, false))) break;
      // the sequence's logits also go to its own row of the logits buffer
      if (slot != 0) cudaMemcpyAsync(g->logits + (size_t)slot * c.V, g->logits, (size_t)c.V * 4, cudaMemcpyDeviceToDevice, g->s);
      cudaEventRecord(g->ev1, g->s);
      if (cudaStreamSynchronize(g->s) != cudaSuccess) { ok = 0; set_last_error("gpt_slot_extend: %s", cudaGetErrorString(cudaGetLastError())); break; }
      cudaEventElapsedTime(&g->last_ms, g->ev0, g->ev1);
      if (!(ok = check_err_flag(g))) break;
      g->last_launches = g->st->launches - l0;
      if (out_id && cudaMemcpy(out_id, g->out_dev, 4, cudaMemcpyDeviceToHost) != cudaSuccess) { ok = 0; set_last_error("gpt_slot_extend: id download failed"); break; }
    } while (0);
  }
  cudaFree(ids_dev);
  if (!ok) return 0;
  g->Ts[slot] = T0 + S;
  g->steps_v[slot] += 1;
  refresh_ragged(g);
  g->probs_valid = false;
  return 1;
}

int TSB200_GptLastTiming(void* h, float* ms, int64_t* launches) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g, "gpt_last_timing: null engine");
  if (ms) *ms = g->last_ms;
  if (launches) *launches = g->last_launches;
  return 1;
}

int TSB200_GptStream(void* h, void** stream) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && stream, "gpt_stream: null argument");
  *stream = (void*)g->s;
  return 1;
}

int TSB200_GptStepBytes(void* h, int B, int T, int64_t* bytes) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && bytes, "gpt_step_bytes: null argument");
  const TSB200GptConfig& c = g->c;
  const int64_t d = c.d, F = c.F, V = c.V, Hd = (int64_t)c.H * c.hd, KVd = (int64_t)c.Hkv * c.hd, s = g->es;
  const int64_t p_attn = d * (Hd + 2 * KVd) + Hd * d;
  const int64_t p_ffn = (g->glu ? 3 : 2) * d * F;
  const int64_t b_attn = (Hd + 2 * KVd) + d, b_ffn = (g->glu ? 2 : 1) * F + d;
  const int64_t n_norm = (c.norm_type == 0 ? 2 : 1) * d * 2;
  int64_t total = s * (c.L * (p_attn + p_ffn) + d * V);
  total += s * (c.L * (b_attn + b_ffn + n_norm) + V + (c.norm_type == 0 ? 2 : 1) * d);
  total += (int64_t)B * c.L * 2 * KVd * T * s;  // KV read
  total += (int64_t)B * c.L * 2 * KVd * s;      // KV write
  total += (int64_t)B * d * s;                  // embedding rows
  total += (int64_t)B * 4;                      // ids out
  *bytes = total;
  return 1;
}

int TSB200_GptEnableStepTiming(void* h, int enable) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g, "gpt_enable_step_timing: null engine");
  g->step_timing = enable != 0;
  return 1;
}

int TSB200_GptGetStepTimes(void* h, float* ms, int n, int* n_out) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && ms && n_out, "gpt_get_step_times: null argument");
  TSB_TRY(use_device(g->c.device, nullptr));
  const int m = g->step_ev_n < n ? g->step_ev_n : n;
  for (int i = 0; i < m; ++i) TSB_CUDA(cudaEventElapsedTime(&ms[i], g->step_ev[i], g->step_ev[i + 1]));
  *n_out = m;
  return 1;
}

int TSB200_GptStepHost(void* h, const int32_t* last_ids, const TSB200DecodingOptions* opt, int32_t* out_ids) {
  NvtxRange nvtx_("tsb200.gpt.step_host");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && last_ids && opt && out_ids, "gpt_step_host: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_CHECK(g->T > 0 && g->B > 0, "gpt_step_host: prefill first");
  TSB_CHECK(g->T + 1 <= c.max_tokens, "OOM: KV-cache capacity %d exceeded", c.max_tokens);
  const int B = g->B;
  if (!g->pin_ids) TSB_CUDA(cudaHostAlloc((void**)&g->pin_ids, (size_t)(c.max_batch + state_words(g)) * 4 + 64 + 16, cudaHostAllocDefault));
  TSB_TRY(upload_blocked(g, opt));
  g->stop_fin = 0;
  if (!g->gexec) TSB_TRY(set_state(g, 0));
  TSB_TRY(ensure_graph(g, opt, 1));
  for (int b = 0; b < B; ++b) {
    TSB_CHECK(last_ids[b] >= 0 && last_ids[b] < c.V, "gpt_step_host: token id %d out of range", last_ids[b]);
    g->pin_ids[b] = last_ids[b];
  }
  int* pin_state = g->pin_ids + c.max_batch;  // second part of the pinned block
  fill_state(g, pin_state, 0);
  TSB_CUDA(cudaMemcpyAsync(g->ids_cur, g->pin_ids, (size_t)B * 4, cudaMemcpyHostToDevice, g->s));
  // the scalars and the mode flags always; the per-sequence arrays only when the sequences differ
  TSB_CUDA(cudaMemcpyAsync(g->state, pin_state, (size_t)(g->ragged ? state_words(g) : kStateLens) * 4, cudaMemcpyHostToDevice, g->s));
  TSB_CUDA(cudaGraphLaunch(g->gexec, g->s));
  g->lin_syms_used = g->lin_syms_used || g->graph_lin_syms;
  count_launch(c.device, g->graph_nodes);
  TSB_CUDA(cudaMemcpyAsync(g->pin_ids, g->ids_cur, (size_t)B * 4, cudaMemcpyDeviceToHost, g->s));
  int* pin_err = pin_state + state_words(g) + 4;   // the error words travel back with the ids: one synchronisation per step
  TSB_CUDA(cudaMemcpyAsync(pin_err, g->err_flag, 8, cudaMemcpyDeviceToHost, g->s));
  TSB_CUDA(cudaStreamSynchronize(g->s));
  TSB_TRY(check_err_flag(g, pin_err));
  for (int b = 0; b < B; ++b) out_ids[b] = g->pin_ids[b];
  g->T += 1;
  g->step += 1;
  for (int b = 0; b < B; ++b) {
    g->Ts[b] += 1;
    g->steps_v[b] += 1;
  }
  g->probs_valid = (opt->strategy == 1);
  g->last_launches = g->graph_nodes;
  return 1;
}

// K and V rows of the encoder output for every layer's cross-attention block (see the header).
int TSB200_GptSetEncoderOutput(void* h, const void* enc, int dtype, int on_device, const int32_t* src_lens, int B, int S_src, int replicas) {
  NvtxRange nvtx_("tsb200.gpt.set_encoder_output");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && enc, "gpt_set_encoder_output: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_CHECK(c.cross_attn, "gpt_set_encoder_output: the model has no cross-attention blocks");
  TSB_CHECK(dtype == TSB200_F32 || dtype == TSB200_F16, "gpt_set_encoder_output: unsupported dtype %d", dtype);
  if (replicas < 1) replicas = 1;
  TSB_CHECK(B >= 1 && (int64_t)B * replicas <= c.max_batch, "gpt_set_encoder_output: %d sources x %d exceed max_batch %d", B, replicas, c.max_batch);
  TSB_CHECK(S_src >= 1 && S_src <= c.max_src_tokens, "OOM: encoder output of %d positions exceeds max_src_tokens %d", S_src, c.max_src_tokens);
  const int64_t rows = (int64_t)B * S_src, d = c.d, Hd = (int64_t)c.H * c.hd;
  std::vector<int> st((size_t)kStateLens + 2 * c.max_batch, 0);
  st[0] = S_src - 1;
  st[kStateRagged] = 1;
  st[kStateStepsAt] = kStateLens + c.max_batch;
  for (int r = 0; r < replicas; ++r)
    for (int b = 0; b < B; ++b) {
      const int len = src_lens ? src_lens[b] : S_src;
      TSB_CHECK(len >= 1 && len <= S_src, "gpt_set_encoder_output: source length %d of sequence %d outside 1..%d", len, b, S_src);
      st[(size_t)kStateLens + r * B + b] = len - 1;   // the attention kernels read "length before the newest key"
    }
  TSB_TRY(ensure_act(g, rows));
  if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }   // the split count of the captured step follows S_src
  const int64_t bytes = rows * d * (dtype == TSB200_F16 ? 2 : 4);
  const void* src = enc;
  void* tmp = nullptr;
  if (!on_device) {
    cudaError_t e = cudaMalloc(&tmp, (size_t)bytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      TSB_FAIL("OOM: staging buffer of %lld bytes: %s", (long long)bytes, cudaGetErrorString(e));
    }
    if (cudaMemcpyAsync(tmp, enc, (size_t)bytes, cudaMemcpyHostToDevice, g->s) != cudaSuccess) {
      cudaFree(tmp);
      TSB_FAIL("gpt_set_encoder_output: host to device copy failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    src = tmp;
  }
  auto body = [&]() -> int {
    TSB_CUDA(cudaMemcpyAsync(g->cross_state, st.data(), st.size() * 4, cudaMemcpyHostToDevice, g->s));
    Dest dst;
    dst.base = g->h; dst.rows = rows; dst.cols = d; dst.row_stride = d; dst.col_stride = 1; dst.full_rows = rows; dst.full_cols = d;
    TSB_TRY(copy_into(g, dst, src, dtype));   // encoder rows in the model's type
    const int64_t seq_elems = (int64_t)c.H * c.max_src_tokens * c.hd;
    for (int k = 0; k < c.L; ++k) {
      LayerW& L = g->L[k];
      // K = enc Wk + bk, V = enc Wv + bv (the encoder output is not normed here: MultiHeadAttention.cs:453-456)
      TSB_TRY(engine_linear(g, (int)rows, g->h, nullptr, nullptr, nullptr, nullptr, L.xk, (int)d, (int)Hd, make_ep(L.xkb, nullptr, g->qkv, nullptr, TSB200_ACT_NONE, 0)));
      TSB_TRY(engine_linear(g, (int)rows, g->h, nullptr, nullptr, nullptr, nullptr, L.xv, (int)d, (int)Hd, make_ep(L.xvb, nullptr, g->attn, nullptr, TSB200_ACT_NONE, 0)));
      for (int r = 0; r < replicas; ++r) {
        void* dK = (char*)L.xK + (size_t)r * B * seq_elems * g->es;
        void* dV = (char*)L.xV + (size_t)r * B * seq_elems * g->es;
        // no rotation, no query rows: the rows go to positions 0 .. S_src - 1 of the head-major layout the attention kernels read
        TSB_TRY(launch_rope_append(c.device, g->st, c.dtype, nullptr, g->qkv, g->attn, Hd, Hd, dK, dV, B, S_src, 0, c.H, c.hd, 0, nullptr,
                                   c.max_src_tokens, 0, (double)c.rope_base, nullptr, g->s));
      }
    }
    TSB_CUDA(cudaStreamSynchronize(g->s));   // `st` and the staging buffer go away
    return 1;
  };
  const int ok = body();
  if (tmp) cudaFree(tmp);
  if (!ok) return 0;
  g->cross_T = S_src;
  return 1;
}

#ifdef TSB200_CHECKED
__global__ void chk_selftest_kernel(int code) { TSB_DEV_CHECK(engine, code == 0, code, return) }
// Checked builds only: records `code` in the engine's check word the way a failing device-side check would (nothing faults),
// so that a host can see the next engine call report it.
__attribute__((visibility("default"))) int TSB200_DebugCheckedSelfTest(int device, int code) {
  TSB_TRY(use_device(device, nullptr));
  chk_selftest_kernel<<<1, 32>>>(code);
  TSB_CUDA(cudaDeviceSynchronize());
  return 1;
}
#endif

// The K most probable next ids of every sequence after the latest forward (prefill, extend or step), taken as the
// reference takes them in beam search: softmax of the logits, -1 on blocked ids, then K rounds of (first arg-max, zero it)
// (Decoder.cs:447-517 / the same loop in GPTDecode).  ids, probs, log_probs: host arrays [sequences][K].
int TSB200_GptBeamCandidates(void* h, int K, const TSB200DecodingOptions* opt, int32_t* ids, float* probs, float* log_probs) {
  NvtxRange nvtx_("tsb200.gpt.beam_candidates");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && opt && ids && probs && log_probs, "gpt_beam_candidates: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_CHECK(g->B > 0 && g->T > 0, "gpt_beam_candidates: nothing has run yet");
  TSB_CHECK(K >= 1 && K <= kMaxBeam && K <= c.V, "gpt_beam_candidates: %d candidates asked, at most %d", K, kMaxBeam < c.V ? kMaxBeam : c.V);
  if (!g->beam_ids) {
    TSB_TRY(dev_alloc(g, (void**)&g->beam_ids, (int64_t)c.max_batch * kMaxBeam * 4));
    TSB_TRY(dev_alloc(g, (void**)&g->beam_p, (int64_t)c.max_batch * kMaxBeam * 8));
  }
  TSB_TRY(upload_blocked(g, opt));
  const int B = g->B;
  float* logp = g->beam_p + (size_t)c.max_batch * kMaxBeam;
  TSB_TRY(launch_softmax_argmax(c.device, g->st, nullptr, g->probs, g->logits, B, c.V, 1.0f, 0, g->blocked, g->n_blocked, g->s));
  TSB_TRY(launch_beam_topk(c.device, g->st, g->beam_ids, g->beam_p, logp, g->probs, B, c.V, K, g->s));
  g->probs_valid = false;   // the chosen entries of the probabilities are zero now
  TSB_CUDA(cudaMemcpyAsync(ids, g->beam_ids, (size_t)B * K * 4, cudaMemcpyDeviceToHost, g->s));
  TSB_CUDA(cudaMemcpyAsync(probs, g->beam_p, (size_t)B * K * 4, cudaMemcpyDeviceToHost, g->s));
  TSB_CUDA(cudaMemcpyAsync(log_probs, logp, (size_t)B * K * 4, cudaMemcpyDeviceToHost, g->s));
  TSB_CUDA(cudaStreamSynchronize(g->s));
  return 1;
}

// Sequence src[i] is copied over sequence dst[i] (cache rows, history, pending id, length and step), i < n.  A destination
// equal to the number of sequences adds one (destinations in ascending order then).  No destination may also be a source:
// a surviving hypothesis keeps its place, the copies fill the places of the ones that were dropped.
int TSB200_GptBeamCopy(void* h, const int32_t* src, const int32_t* dst, int n) {
  NvtxRange nvtx_("tsb200.gpt.beam_copy");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && (n == 0 || (src && dst)), "gpt_beam_copy: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_CHECK(n >= 0 && n <= c.max_batch, "gpt_beam_copy: %d copies for %d sequences", n, c.max_batch);
  if (n == 0) return 1;
  if (g->Ts.empty()) mirror_uniform(g);
  for (int i = 0; i < n; ++i) {
    TSB_CHECK(src[i] >= 0 && src[i] < g->B, "gpt_beam_copy: source %d is not a sequence in use (%d)", src[i], g->B);
    for (int j = 0; j < n; ++j) TSB_CHECK(dst[j] != src[i], "gpt_beam_copy: sequence %d is both a source and a destination", src[i]);
    for (int j = 0; j < i; ++j) TSB_CHECK(dst[j] != dst[i], "gpt_beam_copy: destination %d named twice", dst[i]);
  }
  if (!g->beam_layers) {
    TSB_TRY(dev_alloc(g, (void**)&g->beam_layers, (int64_t)2 * c.L * sizeof(void*)));
    TSB_TRY(dev_alloc(g, (void**)&g->beam_pairs, (int64_t)2 * c.max_batch * 4));
    std::vector<void*> lp((size_t)2 * c.L);
    for (int k = 0; k < c.L; ++k) {
      lp[2 * k] = g->L[k].cK;
      lp[2 * k + 1] = g->L[k].cV;
    }
    TSB_CUDA(cudaMemcpy(g->beam_layers, lp.data(), lp.size() * sizeof(void*), cudaMemcpyHostToDevice));
  }
  std::vector<int> pairs((size_t)2 * n);
  int Tmax = 0;
  for (int i = 0; i < n; ++i) {
    TSB_TRY(slot_claim(g, dst[i], "gpt_beam_copy"));
    pairs[2 * i] = src[i];
    pairs[2 * i + 1] = dst[i];
    g->Ts[dst[i]] = g->Ts[src[i]];
    g->steps_v[dst[i]] = g->steps_v[src[i]];
    Tmax = g->Ts[src[i]] > Tmax ? g->Ts[src[i]] : Tmax;
  }
  TSB_CUDA(cudaMemcpyAsync(g->beam_pairs, pairs.data(), pairs.size() * 4, cudaMemcpyHostToDevice, g->s));
  const int64_t head_pitch = (int64_t)c.max_tokens * c.hd * g->es;
  const int64_t head_bytes = (((int64_t)Tmax * c.hd * g->es) + 15) / 16 * 16;   // rows of 16-byte multiples (hd * es is one)
  if (Tmax > 0)
    seq_copy_kernel<<<dim3(n, 2 * c.L * c.Hkv), 256, 0, g->s>>>(g->beam_layers, g->beam_pairs, c.Hkv, head_pitch * c.Hkv, head_pitch, head_bytes,
                                                                  g->hist, g->hist_len, g->ids_cur, c.max_tokens);
  count_launch(c.device);
  TSB_TRY(check_launch("seq_copy"));
  TSB_CUDA(cudaStreamSynchronize(g->s));   // `pairs` is pageable
  refresh_ragged(g);
  g->probs_valid = false;
  return 1;
}

#ifdef TSB200_TRACE
int TSB200_GptDebugStackTrace(void* h, void* device_buffer) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g, "gpt_debug_stack_trace: null handle");
  g->stack_trace = reinterpret_cast<long long*>(device_buffer);
  if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }  // the pointer is a kernel argument of the captured step
  return 1;
}
#endif

int TSB200_GptSetWaitLimit(void* h, int polls) {
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && polls >= 0, "gpt_set_wait_limit: bad arguments");
  g->poll_limit = (unsigned)polls;
  if (g->gexec) { cudaGraphExecDestroy(g->gexec); g->gexec = nullptr; }  // the limit is a kernel argument of the captured step
  return 1;
}

int TSB200_GptProfileDecode(void* h, int n_steps, const TSB200DecodingOptions* opt, float* class_ms, int64_t* class_groups,
                            int n_classes) {
  NvtxRange nvtx_("tsb200.gpt.profile_decode");
  Gpt* g = (Gpt*)h;
  TSB_CHECK(g && opt && class_ms && class_groups, "gpt_profile_decode: null argument");
  const TSB200GptConfig& c = g->c;
  TSB_TRY(use_device(c.device, nullptr));
  TSB_CHECK(n_classes >= KC_COUNT, "gpt_profile_decode: need room for %d classes", (int)KC_COUNT);
  TSB_CHECK(g->T > 0 && g->B > 0, "gpt_profile_decode: prefill first");
  TSB_CHECK(g->T + n_steps <= c.max_tokens, "OOM: KV-cache capacity %d exceeded", c.max_tokens);
  for (int i = 0; i < n_classes; ++i) { class_ms[i] = 0.0f; class_groups[i] = 0; }
  TSB_TRY(upload_blocked(g, opt));
  TSB_TRY(set_state(g, 0));
  int Tp = 256;
  while (Tp < g->T + n_steps) Tp <<= 1;
  const int splits = attn_pick_splits(g->st, c.dtype, g->B, c.H, c.Hkv, c.hd, Tp);
  TSB_TRY(ensure_stack(g, g->B));
  g->prof = true;
  g->prof_n = 0;
  int ok = 1;
  for (int i = 0; i < n_steps && ok; ++i) ok = enqueue_forward(g, g->B, 1, g->T, true, splits) && enqueue_sample(g, g->B, opt, true, true);
  prof_flush(g);
  g->prof = false;
  g->prof_open = false;
  cudaError_t e = cudaStreamSynchronize(g->s);
  if (!ok) return 0;
  TSB_CUDA(e);
  TSB_TRY(check_err_flag(g));
  for (size_t i = 0; i < g->prof_n; ++i) {
    float ms = 0.0f;
    TSB_CUDA(cudaEventElapsedTime(&ms, g->prof_ev[2 * i], g->prof_ev[2 * i + 1]));
    class_ms[g->prof_cls[i]] += ms;
    class_groups[g->prof_cls[i]] += g->prof_cnt[i];   // launches, however many of them shared a run
  }
  g->T += n_steps;
  g->step += (uint32_t)n_steps;
  g->probs_valid = (opt->strategy == 1);
  return 1;
}

}  // extern "C"
