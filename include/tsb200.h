/*
 * tsb200.h — C ABI of libtsb200.so: hand-written sm_100a CUDA kernels for Seq2SeqSharp's GPTDecoder
 * autoregressive token loop, reached from C# by P/Invoke behind the TensorSharp backend contract
 * (OpRegistry op names, IAllocator, Storage).
 *
 * Conventions (same as the in-tree native bridge TensorSharp.GGML.Native/ggml_ops.cpp:90-135,4683-4722 and
 * its binding TensorSharp.GGML/GgmlNative.cs:161-331,471-479):
 *   - every function returns int: 1 = success, 0 = failure; nothing throws across the boundary;
 *   - TSB200_GetLastError() returns a thread-local message for the calling thread's last failure;
 *   - plain pointers and sizes only; tensors are described by TSB200Tensor (sizes + element strides, the
 *     fields of TensorSharp.Tensor: TensorSharp/Tensor.cs:42-57);
 *   - every entry point selects its device itself (the reference calls a backend from one thread per device:
 *     Seq2SeqSharp/Tools/BaseSeq2SeqFramework.cs:912) and is safe to call concurrently for different devices;
 *   - `stream` is a cudaStream_t passed as void*; NULL selects the library's own non-blocking stream of the
 *     device.  Nothing runs on the legacy NULL stream;
 *   - there is no CPU fallback: with no usable sm_100 device every compute entry point fails.
 */
#ifndef TSB200_H_
#define TSB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define TSB200_API __declspec(dllexport)
#else
#define TSB200_API __attribute__((visibility("default")))
#endif

/* TensorSharp.DType (TensorSharp/DType.cs:6-13) */
enum { TSB200_F32 = 0, TSB200_F16 = 1, TSB200_F64 = 2, TSB200_I32 = 3, TSB200_U8 = 4 };

/* A strided view over device memory: the (sizes, strides, storage, offset) of TensorSharp.Tensor with the
 * offset already applied to `data`.  Outermost dimension first; strides in elements. */
typedef struct TSB200Tensor {
  void* data;
  int32_t dtype;
  int32_t ndim; /* 1..4 */
  int64_t sizes[4];
  int64_t strides[4];
} TSB200Tensor;

/* ------------------------------------------------------------------------------------------------ lifecycle */
/* replaces TSGgml_GetLastError (TensorSharp.GGML/GgmlNative.cs:171) */
TSB200_API const char* TSB200_GetLastError(void);
/* replaces TSGgml_IsBackendAvailable (GgmlNative.cs:177): 1 when `device` exists and is compute capability 10.x */
TSB200_API int TSB200_IsAvailable(int device);
TSB200_API int TSB200_DeviceCount(int* count);
/* library build facts: "sm_100a;<nvcc version>" */
TSB200_API const char* TSB200_BuildInfo(void);
/* number of kernel launches this library has issued on `device` since load (bench bookkeeping) */
TSB200_API int TSB200_LaunchCount(int device, int64_t* launches);

/* ------------------------------------------------------------------------------------------------ memory
 * IAllocator.Allocate / Storage.Destroy / Storage.CopyToStorage / CopyFromStorage
 * (TensorSharp/IAllocator.cs:13-20, TensorSharp/Storage.cs:32-46; device precedent
 * TensorSharp.CUDA/CudaStorage.cs:10-172).  A failed allocation sets the last error to a message that starts
 * with "OOM:" so the binding can raise OutOfMemoryException (caught at Seq2SeqSharp/Applications/GPT.cs:269). */
TSB200_API int TSB200_Alloc(int device, int64_t bytes, void** ptr);
TSB200_API int TSB200_Free(int device, void* ptr);
TSB200_API int TSB200_MemcpyH2D(int device, void* dst, const void* src, int64_t bytes, void* stream);
TSB200_API int TSB200_MemcpyD2H(int device, void* dst, const void* src, int64_t bytes, void* stream);
TSB200_API int TSB200_MemcpyD2D(int device, void* dst, const void* src, int64_t bytes, void* stream);
/* cross-device copy; replaces cuMemcpyPeer in TensorSharp.CUDA/KernelOps/CopyOps.cs:47-97 */
TSB200_API int TSB200_MemcpyPeer(int dst_device, void* dst, int src_device, const void* src, int64_t bytes);
TSB200_API int TSB200_Synchronize(int device, void* stream);
/* IAllocator.GetAllocatedMemoryRatio (TensorSharp/IAllocator.cs:19) */
TSB200_API int TSB200_MemoryInfo(int device, int64_t* free_bytes, int64_t* total_bytes);

/* ------------------------------------------------------------------------------------------------ unfused ops
 * One entry point per op name the GPT decode path invokes through OpRegistry (the names registered in
 * TensorSharp.CUDA/CudaBasicOps.cs:81-681).  F32 and F16 tensors; strided views where the reference accepts
 * them, contiguous-only where the reference itself requires contiguity. */
/* "copy" (CudaBasicOps.cs:81-163) — same element count, any strides, dtype conversion F32<->F16 allowed */
TSB200_API int TSB200_Copy(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream);
/* "fill" (CudaBasicOps.cs:166) */
TSB200_API int TSB200_Fill(int device, const TSB200Tensor* result, float value, void* stream);
/* "addmm" (CudaBasicOps.cs:195-262): result = beta*src + alpha*m1*m2; src may be a stride-0 broadcast row */
TSB200_API int TSB200_Addmm(int device, const TSB200Tensor* result, float beta, const TSB200Tensor* src, float alpha,
                            const TSB200Tensor* m1, const TSB200Tensor* m2, void* stream);
/* "addmmbatch" (CudaBasicOps.cs:264-328): 3-D, batch outermost */
TSB200_API int TSB200_AddmmBatch(int device, const TSB200Tensor* result, float beta, const TSB200Tensor* src,
                                 float alpha, const TSB200Tensor* m1, const TSB200Tensor* m2, void* stream);
/* "layernorm" / "rmsnorm" (CudaBasicOps.cs:666,673; kernels TensorSharp.CUDA/DeviceCode/AdvFuncKernels.cs:613-685,
 * 791-845): rows = all but the last dimension; beta may be NULL */
TSB200_API int TSB200_LayerNorm(int device, const TSB200Tensor* result, const TSB200Tensor* src,
                                const TSB200Tensor* gamma, const TSB200Tensor* beta, float eps, void* stream);
TSB200_API int TSB200_RMSNorm(int device, const TSB200Tensor* result, const TSB200Tensor* src,
                              const TSB200Tensor* gamma, const TSB200Tensor* beta, float eps, void* stream);
/* "rope" (CudaBasicOps.cs:616; AdvFuncKernels.cs:1245-1279): interleaved pairs, base 500000,
 * position = (row % seqLen) + rowOffset.  TSB200_RoPEEx takes the base as an argument. */
TSB200_API int TSB200_RoPE(int device, const TSB200Tensor* result, const TSB200Tensor* src, int seqLen, int rowOffset,
                           void* stream);
TSB200_API int TSB200_RoPEEx(int device, const TSB200Tensor* result, const TSB200Tensor* src, int seqLen,
                             int rowOffset, float base, void* stream);
/* "softmax" (CudaBasicOps.cs:655; AdvFuncKernels.cs:1534-1600): over the last dimension, fp32 internally */
TSB200_API int TSB200_Softmax(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream);
/* "indexselect" (CudaBasicOps.cs:608; AdvFuncKernels.cs:1214-1243): indices are F32 (or I32), negative = skip row */
TSB200_API int TSB200_IndexSelect(int device, const TSB200Tensor* result, const TSB200Tensor* src,
                                  const TSB200Tensor* indices, int isAdd, void* stream);
/* "addt", "mult" (CudaBasicOps.cs:514,525): broadcasting via stride 0 in either operand */
TSB200_API int TSB200_Add(int device, const TSB200Tensor* result, const TSB200Tensor* lhs, const TSB200Tensor* rhs,
                          void* stream);
TSB200_API int TSB200_Mul(int device, const TSB200Tensor* result, const TSB200Tensor* lhs, const TSB200Tensor* rhs,
                          void* stream);
/* "mulv", "divv" (CudaBasicOps.cs:491,493) */
TSB200_API int TSB200_MulScalar(int device, const TSB200Tensor* result, const TSB200Tensor* src, float value,
                                void* stream);
TSB200_API int TSB200_DivScalar(int device, const TSB200Tensor* result, const TSB200Tensor* src, float value,
                                void* stream);
/* "relu", "SiLU", "LeakyReLU" (CudaBasicOps.cs:416,443,429) */
TSB200_API int TSB200_Relu(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream);
TSB200_API int TSB200_SiLU(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream);
TSB200_API int TSB200_LeakyReLU(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream);
/* "float2half", "half2float" (CudaBasicOps.cs:343,346) */
TSB200_API int TSB200_Float2Half(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream);
TSB200_API int TSB200_Half2Float(int device, const TSB200Tensor* result, const TSB200Tensor* src, void* stream);
/* "argmax" (CudaBasicOps.cs:560; TensorSharp.CUDA/DeviceCode/ReduceDimIndexKernels.cs:25,96-119): along `dim`,
 * lowest index among equal maxima, index stored as a float (or int32 when result is I32) */
TSB200_API int TSB200_Argmax(int device, const TSB200Tensor* result, const TSB200Tensor* src, int dim, void* stream);
/* "buildtrimask" / "buildselftrimask" (CudaBasicOps.cs:645,639; AdvFuncKernels.cs:1414-1437,1383-1412) */
TSB200_API int TSB200_BuildTriMask(int device, const TSB200Tensor* result, float value, float maskedValue,
                                   void* stream);
TSB200_API int TSB200_BuildSelfTriMask(int device, const TSB200Tensor* result, const TSB200Tensor* originalLengths,
                                       int paddedSeqLen, float value, float maskedValue, void* stream);

/* ------------------------------------------------------------------------------------------------ sampling
 * Device replacement for the host loop ComputeGraphTensor.TopPSample
 * (Seq2SeqSharp/Tools/ComputeGraphTensor.cs:2305-2403).  probs [rows, V] F32 contiguous; history [rows,
 * history_stride] I32 with history_len[row] valid ids (the row's decodedSequence), may be NULL; u [rows] F32
 * uniform draws standing in for RandomGenerator.floatRandom (Seq2SeqSharp/Tools/RandomGenerator.cs:41-46);
 * out [rows] I32.  workspace: at least TSB200_TopPWorkspaceBytes(rows, V) bytes of device memory.
 * Same order as the reference: repeat penalty, drop w <= 0, sort (w desc, index asc), sequential fp32 prefix
 * sum stopped at the first acc >= topP, pick the first k with acc[k]/acc >= u. */
TSB200_API int64_t TSB200_TopPWorkspaceBytes(int rows, int V);
TSB200_API int TSB200_TopPSample(int device, int32_t* out, const float* probs, int rows, int V, float topP,
                                 float repeatPenalty, const int32_t* history, const int32_t* history_len,
                                 int history_stride, const float* u, void* workspace, int64_t workspace_bytes,
                                 void* stream);
/* Top-P sampling for callers that must not allocate device memory.  (No counterpart in the reference: its TopPSample
 * runs on the host.)  Some hosts of this library cannot call cudaMalloc on the sampling path: a serving loop that has
 * given all remaining device memory to its own pool (the reference reserves a fixed share of the GPU up front and
 * treats any later allocation failure as out-of-memory), or a per-token loop where the implicit device-wide
 * synchronisation of an allocation would stall every stream.  This variant takes the same inputs and writes the same
 * output as TSB200_TopPSample but sorts inside a 5 MiB scratch block built into the library, so it calls no cudaMalloc,
 * cudaFree or allocating library routine.
 *   - Limit: rows * V <= 262144 (e.g. 4 rows of a 65536-word vocabulary, 8 rows of 32000).  Larger requests fail with a
 *     message naming the limit; use TSB200_TopPSample with your own workspace for those.
 *   - The first call on each device looks up the scratch block's device address and opts the kernel into its shared
 *     memory size; make that first call before starting any stream capture.  With CUDA's lazy module loading that
 *     first call may also be the moment the driver reserves the 5 MiB image of the block, so a host that hands all
 *     free device memory to its own pool should make one call per device (rows = 0 is enough) BEFORE it does so;
 *     otherwise the call that is meant never to allocate can itself report out-of-memory.
 *   - All calls on a device share the one scratch block, which keeps whatever the previous call left in it; nothing
 *     in it needs clearing (the kernel writes every word before reading it), but two calls that overlap on the GPU
 *     (different streams, or different host threads) race on it.  Serialise them. */
TSB200_API int TSB200_TopPSampleStatic(int device, int32_t* out, const float* probs, int rows, int V, float topP,
                                       float repeatPenalty, const int32_t* history, const int32_t* history_len,
                                       int history_stride, const float* u, void* stream);
/* u[i] = Philox4x32-10 uniform in [0,1) for (seed, seq_first + i, step); replaces the process-wide
 * System.Random (RandomGenerator.cs:41-46) with a counter-based stream per sequence */
TSB200_API int TSB200_PhiloxUniform(int device, float* u, int n, uint64_t seed, uint64_t seq_first, uint32_t step,
                                    void* stream);

/* ------------------------------------------------------------------------------------------------ fused ops
 * Building blocks of the fused decode path (additional op names the reworked layers call when the storage is
 * device memory of this backend).  dtype = TSB200_F32 or TSB200_F16 for weights/activations; accumulation is
 * always fp32. */
enum { TSB200_ACT_NONE = -1, TSB200_ACT_RELU = 0, TSB200_ACT_SILU = 1, TSB200_ACT_LEAKYRELU = 2,
       TSB200_ACT_GLU_NOACT = 3 /* the reference's "SwiGLU": (xW1+b1)*(xW3+b3), PositionwiseFeedForward.cs:82-89 */,
       TSB200_ACT_SWIGLU = 4 /* silu(xW1+b1)*(xW3+b3): extension */, TSB200_ACT_GELU = 5 /* erf GELU: extension */ };

/* y[M,N] = act(bias + x[M,K] W[K,N]) (+ residual); W row-major [in,out] as the reference stores it
 * (Seq2SeqSharp/Layers/FeedForwardLayer.cs:43).  x, y in `dtype`; residual and y_f32 optional:
 * when y_f32 != NULL the result (plus residual_f32 when given) is written there in fp32 instead of y.
 * Decode-sized M (<= 16) runs the bandwidth-bound GEMV; larger M the tensor-core GEMM.
 * Replaces Affine = bias copy + cublasGemmEx (TensorSharp.CUDA/MatrixMul/CudaMatrixMulMM.cs:305-362). */
TSB200_API int TSB200_LinearBiasAct(int device, int dtype, void* y, float* y_f32, const void* x, const void* W,
                                    const void* bias, const float* residual_f32, int M, int K, int N, int act,
                                    void* workspace, int64_t workspace_bytes, void* stream);
TSB200_API int64_t TSB200_LinearWorkspaceBytes(int M, int K, int N);

/* The engine's weight layout for decode: contiguous 16 KB tiles [32 rows][256 (F16) or 128 (F32) columns], column-tile
 * major, zero padded, so that a CTA streams one contiguous byte range with TMA bulk copies.  PackWeight converts a
 * row-major [K,N] matrix (F32 or F16 source) into `packed` (PackedWeightBytes bytes). */
TSB200_API int64_t TSB200_PackedWeightBytes(int dtype, int K, int N);
TSB200_API int TSB200_PackWeight(int device, int dtype, void* packed, const void* W, int src_dtype, int K, int N,
                                 void* stream);
/* y = act(bias + prologue(x) Wp) (+ residual) on packed weights.  norm_type -1: x [M,K] in `dtype`; 0 / 1: the input
 * is the fp32 residual stream x_f32 [M,K] and LayerNorm / RMSNorm (gamma, beta, eps) is applied first, fused into the
 * kernel (M <= 4; fp16 models of width 1024 / 2048 / 4096 also for M <= 8 while M * width <= 16384, in the tensor-core
 * streaming kernel).  M <= 4 runs the TMA-fed streaming GEMV; larger M the tensor-core streaming kernels.  Replaces
 * LayerNorm/RMSNorm + Affine + activation/gate/residual of one layer (PositionwiseFeedForward.cs:72-98,
 * MultiHeadAttention.cs:130-137,234-237). */
TSB200_API int64_t TSB200_LinearPackedWorkspaceBytes(int dtype, int M, int K, int N);
TSB200_API int TSB200_LinearPacked(int device, int dtype, void* y, float* y_f32, const void* x, const float* x_f32,
                                   const void* gamma, const void* beta, int norm_type, float eps, const void* Wp,
                                   const void* bias, const float* residual_f32, int M, int K, int N, int act,
                                   void* workspace, int64_t workspace_bytes, void* stream);

/* Fused (residual +) LayerNorm / RMSNorm: x_f32[M,d] (+= delta when given) -> h[M,d] in `dtype`.
 * norm_type 0 = LayerNorm (beta may be NULL), 1 = RMSNorm.  Replaces gLNormalization / RMSNorm
 * (AdvFuncKernels.cs:613-685,791-845) plus the preceding "addt". */
TSB200_API int TSB200_NormResidual(int device, int dtype, void* h, float* x_f32, const void* delta, const void* gamma,
                                   const void* beta, int norm_type, float eps, int M, int d, void* stream);

/* RoPE on q and k for S new positions per sequence starting at cache length T0, then append k, v to the cache.
 * q [B,S,H,hd], k/v [B,S,Hkv,hd] in `dtype` (row strides given in elements), cache K/V [B,Hkv,Tmax,hd].
 * Replaces RoPE x2 + Concat x2 (MultiHeadAttention.cs:141-193, TensorSharp/Core/TensorConcatenation.cs:9-45). */
TSB200_API int TSB200_RopeAppend(int device, int dtype, void* q, const void* k, const void* v, int64_t q_row_stride,
                                 int64_t kv_row_stride, void* cacheK, void* cacheV, int B, int S, int H, int Hkv,
                                 int hd, int T0, int Tmax, int use_rope, float rope_base, void* stream);

/* Split-K flash-decode attention for S = 1: out[B,H,hd] = softmax(q K^T / sqrt(hd)) V over T cached positions,
 * query head h reading KV head h / (H/Hkv) (GroupQueryAttention.cs:156-165).  Replaces MulBatch + Softmax +
 * MulBatch (MultiHeadAttention.cs:195-231).  workspace >= TSB200_FlashDecodeWorkspaceBytes(B,H,hd,T). */
TSB200_API int64_t TSB200_FlashDecodeWorkspaceBytes(int B, int H, int hd, int T);
TSB200_API int TSB200_FlashDecode(int device, int dtype, void* out, const void* q, int64_t q_row_stride,
                                  const void* cacheK, const void* cacheV, int B, int H, int Hkv, int hd, int T,
                                  int Tmax, void* workspace, int64_t workspace_bytes, void* stream);

/* Causal attention for prefill (S query positions on an empty cache or after T0 cached positions).
 * Replaces BuildTriMask + MulBatch + Add + Softmax + MulBatch (Decoder.cs:681-693, MultiHeadAttention.cs:195-231). */
TSB200_API int TSB200_PrefillAttention(int device, int dtype, void* out, const void* q, int64_t q_row_stride,
                                       const void* cacheK, const void* cacheV, int B, int S, int H, int Hkv, int hd,
                                       int T0, int Tmax, void* stream);

/* logits[B,V] F32 -> (optional /temperature) -> softmax -> probs (+= -1 at blocked ids) -> first index of the
 * row maximum.  Replaces Div + Half2Float + Softmax + Scatter/Add + Argmax (Decoder.cs:720-761;
 * ReduceDimIndexKernels.cs:96-119).  probs_out may be NULL. */
TSB200_API int TSB200_SoftmaxArgmax(int device, int32_t* out_ids, float* probs_out, const float* logits, int B, int V,
                                    float temperature, const int32_t* blocked, int n_blocked, void* stream);

/* ------------------------------------------------------------------------------------------------ GPT engine
 * The whole token loop of GPT.RunForwardOnSingleDevice / Decoder.GPTDecode / GPTDecoder.Decode
 * (Seq2SeqSharp/Applications/GPT.cs:212-335, Applications/Decoder.cs:648-794, Networks/GPTDecoder.cs:153-191)
 * on one device: weights by the reference's dictionary names, a pre-sized in-place KV cache, prefill, and
 * CUDA-graph decode steps with on-device ArgMax / Top-P. */
typedef struct TSB200GptConfig {
  int32_t L, d, H, Hkv, hd, F, V;
  int32_t norm_type;       /* 0 LayerNorm, 1 RMSNorm (Seq2SeqSharp/Utils/ArchEnums.cs) */
  int32_t act;             /* TSB200_ACT_* */
  int32_t pe_type;         /* 0 NoPE, 1 APE, 2 RoPE (Seq2SeqSharp/Utils/PositionEmbedding.cs:18-23) */
  int32_t attn_type;       /* 0 MultiHeadAttention (packed QKV [d,3d]), 1 GroupQueryAttention */
  int32_t dtype;           /* TSB200_F32 or TSB200_F16 (weights and activations; accumulation fp32) */
  float eps;               /* reference: 1e-6 */
  float rope_base;         /* reference: 500000 */
  int32_t ape_decode_pos0; /* 1 = reference behaviour: cached decode adds APE row 0 (Decoder.cs:674-677) */
  int32_t max_batch;       /* KV-cache capacity in sequences */
  int32_t max_tokens;      /* KV-cache capacity in positions per sequence */
  int32_t device;
  /* tensor parallelism (MultiProcessorNetworkWrapper rework): H, Hkv, F above are the FULL model's; this rank keeps
   * query heads [H/tp*rank, ..), KV heads [Hkv/tp*rank, ..) and FFN columns [F/tp*rank, ..) and sums the partial
   * results of the out-projection and of the down-projection over the ranks of the communicator given to
   * TSB200_GptSetComm (one all-reduce each per layer).  tp_size <= 1 = off */
  int32_t tp_rank, tp_size;
  /* mixture of experts (Networks/GPTDecoder.cs:114-123, Layers/MoEFeedForward.cs): n_experts > 1 makes layers 2, 3, ... use
   * a router + n_experts feed-forward experts of width 4 d (weights GPTDecoder.MoEFFN_k.{layerNorm.m_alpha, layerNorm.m_beta,
   * m_Router [d,E], m_RouterBias [1,E], m_Whd1 [E*d,4d], m_Whd2 [E*4d,d]}), experts_per_token of them per token.
   * Decoded with one launch per operation; not tensor-parallel.  0 or 1 = off */
  int32_t n_experts, experts_per_token;
  /* encoder-decoder models (Networks/TransformerDecoder.cs:73-120): cross_attn != 0 gives every layer a second attention
   * block between self-attention and feed-forward that reads the encoder's output (weights <prefix>.EncAttn_k.{layerNormQ.*,
   * Q, Qb, K, Kb, V, Vb, W0, b0}, Layers/MultiHeadAttention.cs:434-527); max_src_tokens = capacity of its K/V rows per
   * sequence.  The encoder output arrives through TSB200_GptSetEncoderOutput.  One launch per operation; not tensor-parallel.
   * The layer names may then start with "TransformerDecoder." (the reference's name for this network, Applications/Decoder.cs:49)
 * instead of "GPTDecoder.", and the embedding table may be handed over as "SharedEmbeddings". */
  int32_t cross_attn, max_src_tokens;
} TSB200GptConfig;

typedef struct TSB200DecodingOptions { /* Seq2SeqSharp/Applications/DecodingOptions.cs:16-39 */
  int32_t strategy;        /* 0 GreedySearch, 1 Sampling */
  float topP;
  float temperature;
  float repeatPenalty;
  const int32_t* blocked;  /* host pointer, BlockedTokens */
  int32_t n_blocked;
  uint64_t seed;           /* Philox key of the uniform stream; sequence b draws (seed, seq_base + b, step) */
  uint64_t seq_base;
} TSB200DecodingOptions;

/* Peer-memory all-reduce for the few KB a decode step exchanges (optional; without it the engine uses NCCL for every
 * size).  Each rank exports a 64-byte IPC handle of its exchange region (room for messages of up to max_count floats),
 * the host carries the handles of all ranks to every rank (rank order), and Import maps them.  One process per GPU.
 * The reference has no counterpart (its devices exchange whole tensors with cuMemcpyPeer inside one process,
 * TensorSharp.CUDA/KernelOps/CopyOps.cs:47-97). */
TSB200_API int TSB200_CommPeerExport(void* comm, int64_t max_count, void* handle64);
TSB200_API int TSB200_CommPeerImport(void* comm, const void* handles, int n_ranks);

/* Tensor parallelism inside the persistent decode-step kernel (fp16 models, up to 8 ranks, one process per GPU):
 * the finished column tiles of the row-sharded linears are stored straight into every rank's exchange buffer over
 * NVLink and counted on every rank, and the next operation's norm prologue adds the ranks' partial sums — no
 * collective launch at all in a cached step.  Export returns the 64-byte IPC handle of this rank's exchange region,
 * the host gathers the handles of all ranks (rank order) and hands them to Import.  Optional: without it a tensor-
 * parallel engine runs one launch per operation and all-reduces through the communicator.  No counterpart in the
 * reference. */
TSB200_API int TSB200_GptTpExport(void* gpt, void* handle64);
TSB200_API int TSB200_GptTpImport(void* gpt, const void* handles, int n_ranks);
/* Teardown of peer-mapped memory is collective and has two phases.  Phase 1, on every rank: TSB200_GptTpClose(gpt) and
 * TSB200_CommPeerClose(comm) wait for the device's work and unmap the OTHER ranks' regions.  Then the ranks meet at a
 * host-side barrier (any channel).  Phase 2: TSB200_GptDestroy / TSB200_CommDestroy free this rank's own region.
 * Freeing an exported region while a peer still has it mapped, or while a peer's kernel may still store into it, is
 * undefined behaviour of CUDA IPC and can fault over NVLink; a rank whose call failed must still take part in the
 * barrier before it destroys its handles.  No counterpart in the reference (one process owns all devices there). */
TSB200_API int TSB200_GptTpClose(void* gpt);
TSB200_API int TSB200_CommPeerClose(void* comm);

/* Every device-side wait of the persistent decode-step kernel is bounded: a CTA that polls a dependency counter more
 * than `polls` times raises the engine's error word, walks through the rest of its program without waiting and leaves;
 * the other CTAs see the word and do the same, the call fails with a message, and the engine stays usable (the
 * sequences of the failed call must be reset or restored).  polls = 0 restores the default (2^21, about a second).
 * For hosts that want a tighter bound than a second per step, and for tests that make a wait run out without any
 * fault.  No counterpart in the reference (its kernels never wait on each other). */
TSB200_API int TSB200_GptSetWaitLimit(void* gpt, int polls);
/* Host-only check of the weight layout of the owner-partitioned decode-step kernel (fp16 engines, one GPU, up to four
 * sequences): for a model shape and a number of CTAs it verifies that the CTAs' shares tile every matrix exactly once,
 * that the re-packer places each block where the kernel's consumer loops read it, and that the streams are contiguous.
 * Needs no device.  No counterpart in the reference (its cuBLAS calls read row-major weights,
 * TensorSharp.CUDA/MatrixMul/CudaMatrixMulMM.cs:305-504). */
TSB200_API int TSB200_OwnerLayoutSelfTest(int L, int d, int H, int Hkv, int hd, int F, int V, int glu, int n_ctas);

#ifdef TSB200_TRACE
/* Development builds only (-DTSB200_TRACE): the persistent decode-step kernels stamp %globaltimer per CTA and block of
 * the program into `device_buffer` (NULL switches it off).  The shipped library exports neither of these. */
TSB200_API int TSB200_GptDebugStackTrace(void* gpt, void* device_buffer);
TSB200_API int TSB200_DebugSetGemvTrace(void* device_buffer);
#endif

TSB200_API int TSB200_GptCreate(const TSB200GptConfig* cfg, void** gpt);
TSB200_API int TSB200_GptDestroy(void* gpt);
/* name = the reference's weight key (IModel.AddWeights/GetWeights, Seq2SeqSharp/Tools/WeightTensor.cs:571-604),
 * e.g. "GPTDecoder.SelfAttn_3.QKV", "GPTDecoder.PosFFN_3.feedForwardLayer1.m_Whd", "TgtEmbeddings",
 * "FeedForward_Decoder_0.m_Whd", "PosEmbedding".  data: [rows, cols] row-major FULL (unsharded) tensor in
 * `dtype` (F32 data is converted when the model is F16), host memory (on_device = 0) or memory of the model's
 * device (on_device = 1).  With tp_size > 1 the engine keeps only this rank's slice. */
TSB200_API int TSB200_GptSetWeight(void* gpt, const char* name, const void* data, int dtype, int64_t rows,
                                   int64_t cols, int on_device);
/* device pointer of the engine's copy of a weight (for tests and in-place synthetic fill); NULL name lists nothing */
TSB200_API int TSB200_GptGetWeightPtr(void* gpt, const char* name, void** ptr, int64_t* rows, int64_t* cols);
/* fill every weight with the seeded synthetic N(0, std) generator (norm gains 1, norm betas 0; biases N(0,std)
 * when bias_std > 0 else 0), generated on the device */
TSB200_API int TSB200_GptFillSynthetic(void* gpt, uint64_t seed, float std, float bias_std);
/* communicator for a tensor-parallel engine (one process per GPU): rank 0 creates a 128-byte id, hands it to the
 * other ranks by any host channel, every rank calls CommInitRank.  NCCL over NVLink/NVSwitch, opened at run time.
 * Replaces the cuMemcpyPeer exchanges of TensorSharp.CUDA/KernelOps/CopyOps.cs:47-97 (the reference has no collective). */
TSB200_API int TSB200_CommGetUniqueId(void* id128);
TSB200_API int TSB200_CommInitRank(const void* id128, int rank, int nranks, int device, void** comm);
TSB200_API int TSB200_CommDestroy(void* comm);
TSB200_API int TSB200_AllReduceSumF32(void* comm, float* buf, int64_t count, void* stream);
TSB200_API int TSB200_GptSetComm(void* gpt, void* comm);
/* clear the KV cache and per-sequence histories */
TSB200_API int TSB200_GptReset(void* gpt);
/* Prefill: ids [B,S] host int32 (equal lengths, no padding) -> fills the cache, returns the first generated id
 * per sequence in out_ids [B] (host).  Decoder.GPTDecode with an empty cache (Decoder.cs:679-697). */
TSB200_API int TSB200_GptPrefill(void* gpt, const int32_t* ids, int B, int S, const TSB200DecodingOptions* opt,
                                 int32_t* out_ids);
/* Decode n_steps tokens per sequence, each step feeding back the previous step's id on the device
 * (Decoder.cs:661-678 + GPT.cs:249-304).  out_ids [B, n_steps] host.  stop_on_eos: 1 = stop early once every
 * sequence's last id is 0 (GPT.cs:300-303); *steps_done receives the number of steps run. */
TSB200_API int TSB200_GptDecode(void* gpt, int n_steps, const TSB200DecodingOptions* opt, int stop_on_eos,
                                int32_t* out_ids, int* steps_done);
/* logits [B,V] / probs [B,V] (F32, host) of the most recent step */
TSB200_API int TSB200_GptGetLogits(void* gpt, float* logits, float* probs);
TSB200_API int TSB200_GptCacheLength(void* gpt, int* T);   /* the longest sequence's when they differ */
TSB200_API int TSB200_GptCacheLengths(void* gpt, int* lens, int n);   /* per sequence (n entries) */
/* Every device buffer of the engine (weights, caches, activations, scratch) lies between two 256-byte guard regions with a
 * known pattern.  Returns 0 (message names the buffer) if any guard byte has changed, i.e. if some kernel wrote outside a
 * buffer since the engine was created.  Synchronises the engine's stream; meant for tests and for debugging a new model
 * shape, not for the token loop. */
TSB200_API int TSB200_GptCheckGuards(void* gpt);
/* How the most recent cached decode step was launched (the engine chooses by dtype, batch and parallelism):
 * 0 one launch per operation, 1 the stream-K persistent kernel, 2 the owner-partitioned persistent kernel. */
TSB200_API int TSB200_GptDecodePath(void* gpt, int* path);
/* Prompt suffix on top of a non-empty cache: ids [B,S] host int32 are the text from position T (the cache length)
 * on; they are appended to the cache (causal attention over T + S positions) and the next id per sequence is
 * sampled into out_ids [B].  With S = 1 and the pending id this is Decoder.GPTDecode's cached branch
 * (Decoder.cs:661-678); with S > 1 it serves a request whose prompt starts with an already cached text. */
TSB200_API int TSB200_GptExtend(void* gpt, const int32_t* ids, int B, int S, const TSB200DecodingOptions* opt,
                                int32_t* out_ids);
/* Parking a KV cache between calls (the MemoryCache entries of GPT.cs:236-247 and :312-328, which keep every
 * layer's K/V tensors under the text they belong to): Snapshot copies rows [0,T) of every layer, the token
 * history and the pending id into a compact device buffer; Restore writes them into an engine of the same model
 * (B_new = 0: the parked batch; a snapshot of ONE sequence may serve B_new > 1 slots, e.g. a shared system prompt);
 * Info returns the sizes and, if tokens != NULL, the [B, T+1] token ids (cached text + pending id). */
TSB200_API int TSB200_GptCacheSnapshot(void* gpt, void** snapshot);
TSB200_API int TSB200_GptCacheSnapshotInfo(void* snapshot, int* B, int* T, int64_t* bytes, int32_t* tokens);
TSB200_API int TSB200_GptCacheRestore(void* gpt, void* snapshot, int B_new);
TSB200_API int TSB200_GptCacheSnapshotFree(void* snapshot);

/* ---- sequences with their own lengths ---------------------------------------------------------------------------
 * The reference pads the prompts of a batch to one length and masks the pads (BuildInTokens.PadSentences +
 * BuildSelfTriMask, Applications/Decoder.cs:656,687-692).  Here every sequence keeps its own cache length, RoPE / APE
 * position, append position, Philox step and stop rule, so each one continues exactly as if it had been run alone.
 * Batches whose sequences differ decode with one launch per operation (the persistent kernels serve equal lengths).
 *
 * PrefillRagged: ids [B,S] host int32, prompt b occupies columns [0, lens[b]) (1 <= lens[b] <= S; the rest is padding
 * with any valid id).  out_ids [B]: the next id of every sequence.
 * With stop_on_eos, TSB200_GptDecode then stops the sequences one by one: a sequence whose previous id was </s> (0)
 * keeps emitting 0 and its cache, history and Philox step stand still.
 * SlotSnapshot / SlotRestore / SlotReset / SlotExtend work on ONE sequence while the others keep their state: park a
 * finished sequence, put another parked one (or an empty one) in its place, give it the rest of its prompt.  A slot
 * index equal to the number of sequences adds one.  Snapshots are the handles of TSB200_GptCacheSnapshot (one
 * sequence); SlotExtend runs S >= 1 prompt tokens on top of what the slot holds and returns the slot's next id;
 * uniforms of slot b come from the Philox stream (seed, seq_base + b).  Not for tensor-parallel engines. */
TSB200_API int TSB200_GptPrefillRagged(void* gpt, const int32_t* ids, const int32_t* lens, int B, int S,
                                       const TSB200DecodingOptions* opt, int32_t* out_ids);
TSB200_API int TSB200_GptSlotSnapshot(void* gpt, int slot, void** snapshot);
TSB200_API int TSB200_GptSlotRestore(void* gpt, void* snapshot, int slot);
TSB200_API int TSB200_GptSlotReset(void* gpt, int slot);   /* empties the slot; its pending id becomes </s> */
/* on != 0: the per-sequence state (and with it the per-sequence stop rule of TSB200_GptDecode with stop_on_eos) stays in
 * use even while all sequences happen to have the same length - what a scheduler that refills slots wants. */
TSB200_API int TSB200_GptSetPerSequenceState(void* gpt, int on);
TSB200_API int TSB200_GptSlotExtend(void* gpt, int slot, const int32_t* ids, int S, const TSB200DecodingOptions* opt,
                                    int32_t* out_id);
/* device-timed duration (ms, CUDA events on the engine's stream) of the last GptDecode / GptPrefill call and
 * the number of kernel launches it issued (graph replays count their nodes) */
TSB200_API int TSB200_GptLastTiming(void* gpt, float* ms, int64_t* launches);
/* One decode step with HOST buffers: uploads last_ids [B] (pinned staging), runs the step, downloads the new ids
 * [B].  This is the per-token host round trip the reference makes (ids built on the host each step,
 * TensorUtils.CreateTokensEmbeddings; ids read back, Decoder.cs:769-782): B*4 bytes each way. */
TSB200_API int TSB200_GptStepHost(void* gpt, const int32_t* last_ids, const TSB200DecodingOptions* opt,
                                  int32_t* out_ids);
/* Beam search (DecodingOptions.BeamSearchSize > 1; GPT.cs:236-304, Decoder.cs:447-517, Utils/BeamSearch.cs:36-46).  The
 * reference re-runs every hypothesis from its first token at every step (no KV cache with beams); here every hypothesis is
 * a sequence of the engine with its own cache rows, the host keeps the scores and decides which hypotheses survive:
 *   TSB200_GptBeamCandidates  the K best next ids of every sequence after the latest forward, found as the reference finds
 *                             them (K rounds of first-arg-max and zero-fill on softmax(logits) with -1 on blocked ids), with
 *                             their probabilities and natural logarithms; host arrays [sequences][K];
 *   TSB200_GptBeamCopy        sequence src[i] over sequence dst[i] (cache rows, history, pending id, length): the children
 *                             of a hypothesis beyond the first take the places of dropped hypotheses; dst[i] == number of
 *                             sequences adds a sequence (used once, after the prefill, to open the beams);
 *   TSB200_GptStepHost        then feeds the chosen id of every hypothesis and runs the next step. */
/* Encoder output for the cross-attention blocks (cross_attn engines): enc [B, S_src, d] float32 or float16 (host, or
 * device with on_device != 0), src_lens[B] (host; NULL: all S_src) the unpadded source lengths - keys beyond them are not
 * attended, as under the reference's source/target mask (Decoder.cs:283, BuildSrcTgtMask).  Computes every layer's K and V
 * rows once (the reference caches them after the first step, MultiHeadAttention.cs:462-488).  replicas > 1 serves sequence
 * b + k * B (k < replicas) from source b: the hypotheses of a beam search.  Stays in place (TSB200_GptReset included) until
 * the next call.  Engines with cross-attention take one new position per sequence and call: TSB200_GptPrefill with S = 1
 * (<s>), then TSB200_GptDecode / TSB200_GptStepHost; a longer target prefix is fed through TSB200_GptStepHost. */
TSB200_API int TSB200_GptSetEncoderOutput(void* gpt, const void* enc, int dtype, int on_device, const int32_t* src_lens, int B,
                                          int S_src, int replicas);
TSB200_API int TSB200_GptBeamCandidates(void* gpt, int K, const TSB200DecodingOptions* opt, int32_t* ids, float* probs,
                                        float* log_probs);
TSB200_API int TSB200_GptBeamCopy(void* gpt, const int32_t* src, const int32_t* dst, int n);
/* per-step device durations of the last TSB200_GptDecode call (CUDA events between graph launches) */
TSB200_API int TSB200_GptEnableStepTiming(void* gpt, int enable);
TSB200_API int TSB200_GptGetStepTimes(void* gpt, float* ms, int n, int* n_out);
/* Runs n_steps decode steps un-captured with CUDA events around every launch group and returns, per kernel class
 * (0 embed, 1 norm, 2 linear (GEMV/GEMM), 3 rope+append, 4 attention, 5 sampling, 6 commit), the summed device
 * time in ms and the number of launches.  Consecutive launches of one class are timed as one run (events only at its two
 * ends), so that they chain as they do in the captured step.  n_classes >= 8. */
TSB200_API int TSB200_GptProfileDecode(void* gpt, int n_steps, const TSB200DecodingOptions* opt, float* class_ms,
                                       int64_t* class_groups, int n_classes);
/* the engine's stream (cudaStream_t) */
TSB200_API int TSB200_GptStream(void* gpt, void** stream);
/* algorithmic bytes of one decode step at cache length T for B sequences (weights once + KV read/write +
 * embeddings + ids) */
TSB200_API int TSB200_GptStepBytes(void* gpt, int B, int T, int64_t* bytes);

/* ------------------------------------------------------------------------------------------------ synthetic data
 * Seeded counter-based generator used for weights in tests and benchmarks: element i of tensor `name_hash`
 * = (sum of eight 16-bit fields of two splitmix64 outputs - 262140) * std / 53510.06..., exactly reproducible
 * on host and device. */
TSB200_API int TSB200_FillSynthetic(int device, void* data, int dtype, int64_t n, uint64_t seed, uint64_t name_hash,
                                    float std, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TSB200_H_ */
