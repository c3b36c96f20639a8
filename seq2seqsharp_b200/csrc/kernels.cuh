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
int64_t packed_bytes(int dtype, int K, int N);
int packed_tile_cols(int dtype);
int launch_pack(int device, DeviceState* st, int dst_dtype, void* dst, int src_dtype, const void* src, int rows, int cols,
                int src_ld, int K, int c0, int cs, cudaStream_t s);
// NCCL binding (comm.cu)
int comm_all_reduce_f32(void* comm, float* buf, int64_t count, cudaStream_t s);
int comm_nranks(void* comm);
int comm_rank(void* comm);
int init_stream_attrs(int device);
// tcgen05/TMEM GEMM on packed fp16 weights (gemm_tc.cu): 1 ok, 0 error, 2 shape not handled
int launch_gemm_tc(int device, DeviceState* st, const void* x, const void* Wp, int M, int K, int N, const Epilogue& ep,
                   int* error_flag, void* ws, int64_t ws_bytes, cudaStream_t s);
int64_t gemm_tc_workspace_bytes(int M, int N, int sm_count);
int init_tc_attrs(int device);
int tc_take_error();
int64_t linear_workspace_bytes(int M, int K, int N);
int launch_attention(int device, DeviceState* st, int dtype, void* out, const void* q, int64_t q_rs, const void* cK,
                     const void* cV, int B, int S, int H, int Hkv, int hd, int T0, const int* dT0, int Tmax, int splits_hint,
                     void* ws, int64_t ws_bytes, cudaStream_t s);
int64_t attn_workspace_bytes(int B, int H, int hd, int T);
int attn_pick_splits(DeviceState* st, int B, int H, int Hkv, int T);
int launch_rope_table(int device, DeviceState* st, float2* tab, int Tmax, int hd, double base, cudaStream_t s);
int launch_rope_append(int device, DeviceState* st, int dtype, void* q, const void* k, const void* v, int64_t q_rs,
                       int64_t kv_rs, void* cK, void* cV, int B, int S, int H, int Hkv, int hd, int T0, const int* dT0,
                       int Tmax, int use_rope, double base, const float2* tab, cudaStream_t s);
int launch_softmax_argmax(int device, DeviceState* st, int* out_ids, float* probs, const float* logits, int B, int V,
                          float temperature, int use_temp, const int* blocked_dev, int n_blocked, cudaStream_t s);
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
