// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// CPU restatement (fp32) of Seq2SeqSharp's GPTDecoder autoregressive token loop as the
// reference's TensorSharp.Cpu backend computes it.  It is the checker for the CUDA
// kernels and the timed CPU baseline; nothing in the product library links or calls it.
//
// Parity status: the reference (C#/.NET) cannot be compiled or run in this build
// environment and its test-suite holds no known-answer vector for the assembled GPT
// decode loop, so the assembled loop is "parity unpinned" by the reference's own tests.
// Op-level functions are pinned on the input vectors of the reference's backend
// comparison tests (Tests/Seq2SeqSharp.Tests/GgmlOpsComparison_Tests.cs:419-590) with
// closed-form expectations at that suite's 1e-4 tolerance.
//
// Every function cites the reference file:line it follows.  Arithmetic is kept in the
// reference's order (bias first, then k-sequential axpy accumulation; sequential sums;
// double-precision exp/cos/sin/pow cast to float) and the file is compiled with
// -ffp-contract=off so no FMA contraction changes the rounding.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>
#include <thread>

extern "C" {

struct OrcConfig {
  int32_t L, d, H, Hkv, hd, F, V;
  int32_t norm_type;  // 0 LayerNorm, 1 RMSNorm             (Seq2SeqSharp/Utils/ArchEnums.cs NormEnums)
  int32_t act;        // 0 ReLU, 1 SiLU, 2 LeakyReLU, 3 reference "SwiGLU" (gate, no SiLU), 4 true SwiGLU (extension), 5 GELU-erf (extension)
  int32_t pe_type;    // 0 NoPE, 1 APE, 2 RoPE              (Seq2SeqSharp/Utils/PositionEmbedding.cs:18-23)
  int32_t attn_type;  // 0 MultiHeadAttention (packed QKV), 1 GroupQueryAttention
  float eps;          // 1e-6 in the reference (Layers/LayerNormalization.cs:36, RMSNormalization.cs:26)
  float rope_base;    // 500000 in the reference (TensorSharp/TensorApplyCPU.cs:1162)
  int32_t ape_decode_pos0;  // 1 = reference behaviour: cached decode always adds APE row 0 (Decoder.cs:674-677)
  int32_t max_pos;          // rows of the APE table
  int32_t faithful_cache;   // 1 = grow the cache by allocate+copy each step and keep GQA K/V expanded to H heads, as the reference does
  int32_t threads;          // 1 = as the reference's managed SGEMM; >1 = std::thread workers over output columns / heads
  int32_t n_experts;        // > 1: layers 2.. use MoEFeedForward instead of PositionwiseFeedForward (Networks/GPTDecoder.cs:114-123)
  int32_t experts_per_token;
  int32_t cross_attn;       // 1: TransformerDecoder layers (self-attention, attention over the encoder output, feed-forward: Networks/TransformerDecoder.cs:137-160)
};

}  // extern "C"

namespace {

typedef std::vector<float> vecf;

struct Linear {
  vecf W, b;
  int in = 0, out = 0;
};

struct Layer {
  vecf n1_g, n1_b, n2_g, n2_b;
  Linear qkv, q, k, v, o, w1, w2, w3;
  // cache, reference layout: K [B*Hc, hd, T], V [B*Hc, T, hd]  (MultiHeadAttention.cs:173-193)
  vecf K, Vc;
  int Tcap = 0;
  // MoEFeedForward (Layers/MoEFeedForward.cs:31-52): its own LayerNorm, experts [E, d, 4d] and [E, 4d, d] without bias, router [d, E] + bias
  vecf moe_g, moe_b, moe_w1, moe_w2, router_w, router_b;
  // attention over the encoder output (MultiHeadAttention.Perform with three inputs, Layers/MultiHeadAttention.cs:434-527):
  // its own norm of the query side, Q / K / V / W0, and the projected encoder rows Ks [B*H, hd, Ts], Vs [B*H, Ts, hd]
  vecf nx_g, nx_b, xKs, xVs;
  Linear xq, xk, xv, xo;
};

struct Model {
  OrcConfig c;
  vecf E, PE, nf_g, nf_b;
  Linear head;
  std::vector<Layer> layers;
  int B = 0, T = 0;  // cache batch and length
  int Hc = 0;        // heads held in the cache (H when faithful, Hkv otherwise)
  int xB = 0, xTs = 0;        // encoder output: sequences and (padded) source length
  std::vector<int> src_lens;  // unpadded source lengths
};

// ---------------------------------------------------------------------------------------------
// y[M,N] = bias(broadcast) + x[M,K] * W[K,N]  — ComputeGraphTensor.Affine (Seq2SeqSharp/Tools/
// ComputeGraphTensor.cs:1848-1880): bias copied into the result, then Addmm with beta = 1.
// The managed SGEMM (TensorSharp/Cpu/LinearAlgebra/SGEMM.cs:520-556) runs the row-major product
// as column-major C' = W' * x' in "axpy" form: for each output row, for l = 0..K-1,
// skip when x[m,l] == 0, TEMP = alpha * x[m,l], y[m,:] += TEMP * W[l,:].
// ---------------------------------------------------------------------------------------------
// Static block partition of [0, n) over `threads` workers (per-element arithmetic order is unchanged).
template <class F>
void parallel_for(int n, int threads, F f) {
  if (threads <= 1 || n <= 1) {
    for (int i = 0; i < n; ++i) f(i);
    return;
  }
  const int nt = std::min(threads, n);
  std::vector<std::thread> pool;
  for (int t = 0; t < nt; ++t)
    pool.emplace_back([=, &f]() {
      for (int i = t; i < n; i += nt) f(i);
    });
  for (auto& th : pool) th.join();
}

void gemm_axpy(float* C, const float* A, const float* Bm, int M, int K, int N, float alpha, int threads,
               long lda = -1, long ldb = -1, long ldc = -1) {
  if (lda < 0) lda = K;
  if (ldb < 0) ldb = N;
  if (ldc < 0) ldc = N;
  if (threads > 1 && (long)N * K >= 1 << 16) {
    const int chunk = 256;
    const int nchunks = (N + chunk - 1) / chunk;
    parallel_for(nchunks, threads, [&](int ch) {
      const int n0 = ch * chunk, n1 = std::min(N, n0 + chunk);
      for (int m = 0; m < M; ++m) {
        float* c = C + (long)m * ldc;
        for (int l = 0; l < K; ++l) {
          const float xv = A[(long)m * lda + l];
          if (xv != 0.0f) {
            const float t = alpha * xv;
            const float* w = Bm + (long)l * ldb;
            for (int n = n0; n < n1; ++n) c[n] += t * w[n];
          }
        }
      }
    });
    return;
  }
  for (int m = 0; m < M; ++m) {
    float* c = C + (long)m * ldc;
    for (int l = 0; l < K; ++l) {
      const float xv = A[(long)m * lda + l];
      if (xv != 0.0f) {
        const float t = alpha * xv;
        const float* w = Bm + (long)l * ldb;
        for (int n = 0; n < N; ++n) c[n] += t * w[n];
      }
    }
  }
}

void affine(vecf& y, const vecf& x, const Linear& lin, int M, int threads) {
  y.resize((size_t)M * lin.out);
  for (int m = 0; m < M; ++m) std::memcpy(&y[(size_t)m * lin.out], lin.b.data(), sizeof(float) * lin.out);
  gemm_axpy(y.data(), x.data(), lin.W.data(), M, lin.in, lin.out, 1.0f, threads);
}

// TensorSharp/TensorApplyCPU.cs:1360-1447.  Vector<float>.Count is 8 on x64 .NET 8; the vector
// loops run while i < cols - 8 (strict), the remainder is scalar.  Horizontal adds follow the
// 128-bit-lane dot-product shape ((0+1)+(2+3)) + ((4+5)+(6+7)).
inline float hsum8(const float* v) { return ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7])); }

void layernorm(float* out, const float* in, const float* gamma, const float* beta, float eps, int rows, int cols) {
  const int vs = 8;
  for (int j = 0; j < rows; ++j) {
    float* so = out + (long)j * cols;
    const float* sp = in + (long)j * cols;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (i = 0; i < cols - vs; i += vs)
      for (int l = 0; l < vs; ++l) acc[l] += sp[i + l];
    float sum = hsum8(acc);
    for (; i < cols; ++i) sum += sp[i];
    const float mean = sum / cols;
    float sq = 0.0f;
    for (i = 0; i < cols - vs; i += vs) {
      float e[8];
      for (int l = 0; l < vs; ++l) {
        const float ex = sp[i + l] - mean;
        e[l] = ex * ex;
      }
      sq += hsum8(e);
    }
    for (; i < cols; ++i) {
      const float ex = sp[i] - mean;
      sq += ex * ex;
    }
    const float sigma = (float)std::sqrt((double)(eps + sq / cols));
    for (i = 0; i < cols; ++i) {
      float t = gamma[i] * ((sp[i] - mean) / sigma);
      if (beta) t += beta[i];
      so[i] = t;
    }
  }
}

// TensorSharp/TensorApplyCPU.cs:1451-1496
void rmsnorm(float* out, const float* in, const float* gamma, const float* beta, float eps, int rows, int cols) {
  const float N = (float)cols;
  for (int j = 0; j < rows; ++j) {
    float* y = out + (long)j * cols;
    const float* x = in + (long)j * cols;
    float sq = 0.0f;
    for (int i = 0; i < cols; ++i) sq += x[i] * x[i];
    const float rms = (float)std::sqrt((double)(sq / N + eps));
    for (int i = 0; i < cols; ++i) {
      const float r = x[i] / rms;
      y[i] = gamma[i] * r + (beta ? beta[i] : 0.0f);
    }
  }
}

// TensorSharp/TensorApplyCPU.cs:1230-1268
void softmax(float* out, const float* in, int rows, int cols) {
  for (int j = 0; j < rows; ++j) {
    float* so = out + (long)j * cols;
    const float* sp = in + (long)j * cols;
    float mx = sp[0];
    for (int i = 1; i < cols; ++i) mx = std::max(mx, sp[i]);
    float sum = 0.0f;
    for (int i = 0; i < cols; ++i) {
      const float ex = (float)std::exp((double)(sp[i] - mx));
      so[i] = ex;
      sum += ex;
    }
    for (int i = 0; i < cols; ++i) so[i] /= sum;
  }
}

// TensorSharp/TensorApplyCPU.cs:1148-1178 — interleaved pairs, rows flattened [.., seqLen].
void rope(float* out, const float* in, int rows, int cols, int seqLen, int rowOffset, double base) {
  for (int j = 0; j < rows; ++j) {
    float* r = out + (long)j * cols;
    const float* s = in + (long)j * cols;
    const int m = (j % seqLen) + rowOffset;
    for (int id = 0; id < cols; ++id) {
      const int i = id / 2;
      const float theta = (float)std::pow(base, -2.0 * i / cols);
      const float theta_m = theta * m;
      const float c = (float)std::cos((double)theta_m);
      const float sn = (float)std::sin((double)theta_m);
      if (id % 2 == 0)
        r[id] = s[id] * c - s[id + 1] * sn;
      else
        r[id] = s[id] * c + s[id - 1] * sn;
    }
  }
}

// TensorSharp/TensorApplyCPU.cs:339-360 — strictly-greater scan: lowest index among equal maxima.
void argmax_rows(int* out, const float* p, int rows, int cols) {
  for (int j = 0; j < rows; ++j) {
    const float* s = p + (long)j * cols;
    float v = s[0];
    int idx = 0;
    for (int i = 1; i < cols; ++i)
      if (s[i] > v) {
        v = s[i];
        idx = i;
      }
    out[j] = idx;
  }
}

// Seq2SeqSharp/Tools/ComputeGraphTensor.cs:2305-2403 (one row).  `seq` is the row's full token
// history (prompt + generated so far); `u` stands in for RandomGenerator.floatRandom(0,1).
int topp_row(const float* w_in, int K, float topP, float repeatPenalty, const int* seq, int seqLen, float u,
             int* n_cands = nullptr, float* acc_out = nullptr) {
  std::map<int, int> dist;
  for (int j = 0; j < seqLen; ++j) dist[seq[j]] = seqLen - j;
  std::map<float, std::vector<int>> w2id;
  for (int j = 0; j < K; ++j) {
    float w = w_in[j];
    if (w <= 0.0f) continue;
    auto it = dist.find(j);
    if (it != dist.end()) {
      const float ratio = (float)it->second / (float)seqLen;
      const float rp = (float)std::pow((double)ratio, (double)repeatPenalty);
      w = (float)(w * rp);
    }
    w2id[w].push_back(j);
  }
  float acc = 0.0f;
  std::vector<int> cands;
  std::vector<float> accs;
  for (auto it = w2id.rbegin(); it != w2id.rend(); ++it) {
    const float prob = it->first;
    for (int idx : it->second) {
      acc += prob;
      cands.push_back(idx);
      accs.push_back(acc);
      if (acc >= topP) break;
    }
    if (acc >= topP) break;
  }
  if (n_cands) *n_cands = (int)cands.size();
  if (acc_out) *acc_out = acc;
  for (size_t k = 0; k < accs.size(); ++k)
    if (accs[k] / acc >= u) return cands[k];
  return 0;  // indices[] is zero-initialised in the reference
}

inline float act_fn(int act, float w) {
  switch (act) {
    case 0: return w < 0.0f ? 0.0f : w;                              // relu   TensorApplyCPU.cs:1748-1754
    case 1: return w / (1.0f + (float)std::exp((double)-w));         // SiLU   TensorApplyCPU.cs:1797-1800
    case 2: return w < 0.0f ? 0.01f * w : w;                         // LeakyReLU :1773-1779
    case 3: return w;                                                // "SwiGLU": RunActivateFunction has no branch (PositionwiseFeedForward.cs:100-116)
    case 4: return w / (1.0f + (float)std::exp((double)-w));         // true SwiGLU (extension, not in the reference)
    case 5: return (float)(0.5 * (double)w * (1.0 + std::erf((double)w / std::sqrt(2.0))));  // GELU (extension)
  }
  return w;
}

Linear* find_linear(Model* m, const std::string& name, bool bias) {
  (void)bias;
  if (name == "FeedForward_Decoder_0") return &m->head;
  const char* p = "GPTDecoder.";
  if (name.compare(0, 11, p) != 0) return nullptr;
  std::string rest = name.substr(11);
  auto dot = rest.find('.');
  std::string unit = rest.substr(0, dot), field = rest.substr(dot + 1);
  auto us = unit.find('_');
  int k = std::atoi(unit.substr(us + 1).c_str());
  if (k < 0 || k >= (int)m->layers.size()) return nullptr;
  Layer& L = m->layers[k];
  if (unit.compare(0, 8, "SelfAttn") == 0) {
    if (field == "QKV" || field == "QKVb") return &L.qkv;
    if (field == "Q" || field == "Qb") return &L.q;
    if (field == "K" || field == "Kb") return &L.k;
    if (field == "V" || field == "Vb") return &L.v;
    if (field == "W0" || field == "b0") return &L.o;
  } else if (unit.compare(0, 7, "EncAttn") == 0) {
    if (field == "Q" || field == "Qb") return &L.xq;
    if (field == "K" || field == "Kb") return &L.xk;
    if (field == "V" || field == "Vb") return &L.xv;
    if (field == "W0" || field == "b0") return &L.xo;
  } else if (unit.compare(0, 6, "PosFFN") == 0) {
    if (field.compare(0, 17, "feedForwardLayer1") == 0) return &L.w1;
    if (field.compare(0, 17, "feedForwardLayer2") == 0) return &L.w2;
    if (field.compare(0, 17, "feedForwardLayer3") == 0) return &L.w3;
  }
  return nullptr;
}

bool ends_with(const std::string& s, const char* suf) {
  size_t n = std::strlen(suf);
  return s.size() >= n && s.compare(s.size() - n, n, suf) == 0;
}

void norm_apply(const Model* m, float* out, const float* in, const vecf& g, const vecf& b, int rows) {
  if (m->c.norm_type == 0)
    layernorm(out, in, g.data(), b.empty() ? nullptr : b.data(), m->c.eps, rows, m->c.d);
  else
    rmsnorm(out, in, g.data(), nullptr, m->c.eps, rows, m->c.d);  // RMSNormalization has no beta (RMSNormalization.cs:28-35)
}

// Grow the cache of one layer to hold T1 positions.  faithful: allocate exactly T1 and copy the
// old contents (Ops.Concat = fresh tensor + two copies, TensorSharp/Core/TensorConcatenation.cs:9-45).
void cache_grow(Model* m, Layer& L, int B, int T0, int T1) {
  const int Hc = m->Hc, hd = m->c.hd;
  if (m->c.faithful_cache) {
    vecf K2((size_t)B * Hc * hd * T1), V2((size_t)B * Hc * T1 * hd);
    for (long r = 0; r < (long)B * Hc * hd; ++r)
      for (int t = 0; t < T0; ++t) K2[r * T1 + t] = L.K[r * L.Tcap + t];
    for (long bh = 0; bh < (long)B * Hc; ++bh)
      std::memcpy(&V2[bh * T1 * hd], &L.Vc[bh * L.Tcap * hd], sizeof(float) * (size_t)T0 * hd);
    L.K.swap(K2);
    L.Vc.swap(V2);
    L.Tcap = T1;
  } else if (T1 > L.Tcap) {
    int cap = std::max(T1, std::max(64, L.Tcap * 2));
    vecf K2((size_t)B * Hc * hd * cap), V2((size_t)B * Hc * cap * hd);
    for (long r = 0; r < (long)B * Hc * hd; ++r)
      for (int t = 0; t < T0; ++t) K2[r * cap + t] = L.K[r * L.Tcap + t];
    for (long bh = 0; bh < (long)B * Hc; ++bh)
      if (T0) std::memcpy(&V2[bh * cap * hd], &L.Vc[bh * L.Tcap * hd], sizeof(float) * (size_t)T0 * hd);
    L.K.swap(K2);
    L.Vc.swap(V2);
    L.Tcap = cap;
  }
}

// One attention block: MultiHeadAttention.PerformClassic (Layers/MultiHeadAttention.cs:125-240) or
// GroupQueryAttention.Perform (Layers/GroupQueryAttention.cs:114-233).  x is [B*S, d], updated in place
// with the residual sum.
void attention_block(Model* m, Layer& L, vecf& x, int B, int S, int T0) {
  const OrcConfig& c = m->c;
  const int d = c.d, H = c.H, Hkv = (c.attn_type == 1 ? c.Hkv : c.H), hd = c.hd, Hc = m->Hc;
  const int group = H / Hkv;
  const int M = B * S, T1 = T0 + S;
  vecf h((size_t)M * d);
  norm_apply(m, h.data(), x.data(), L.n1_g, L.n1_b, M);

  // q [B*H, S, hd], k/v [B*Hkv, S, hd] (head-major, as after Transpose(1,2)+AsContiguous)
  vecf q((size_t)B * H * S * hd), kk((size_t)B * Hkv * S * hd), vv((size_t)B * Hkv * S * hd);
  if (c.attn_type == 0) {
    vecf y;
    affine(y, h, L.qkv, M, c.threads);  // columns ordered [3][H][hd] (MultiHeadAttention.cs:133)
    for (int b = 0; b < B; ++b)
      for (int s = 0; s < S; ++s)
        for (int hh = 0; hh < H; ++hh) {
          const float* row = &y[((size_t)b * S + s) * 3 * d];
          std::memcpy(&q[(((size_t)b * H + hh) * S + s) * hd], row + 0 * d + hh * hd, sizeof(float) * hd);
          std::memcpy(&kk[(((size_t)b * H + hh) * S + s) * hd], row + 1 * d + hh * hd, sizeof(float) * hd);
          std::memcpy(&vv[(((size_t)b * H + hh) * S + s) * hd], row + 2 * d + hh * hd, sizeof(float) * hd);
        }
  } else {
    vecf yq, yk, yv;
    affine(yq, h, L.q, M, c.threads);
    affine(yk, h, L.k, M, c.threads);
    affine(yv, h, L.v, M, c.threads);
    for (int b = 0; b < B; ++b)
      for (int s = 0; s < S; ++s) {
        for (int hh = 0; hh < H; ++hh)
          std::memcpy(&q[(((size_t)b * H + hh) * S + s) * hd], &yq[((size_t)b * S + s) * d + hh * hd], sizeof(float) * hd);
        for (int g = 0; g < Hkv; ++g) {
          std::memcpy(&kk[(((size_t)b * Hkv + g) * S + s) * hd], &yk[((size_t)b * S + s) * Hkv * hd + g * hd], sizeof(float) * hd);
          std::memcpy(&vv[(((size_t)b * Hkv + g) * S + s) * hd], &yv[((size_t)b * S + s) * Hkv * hd + g * hd], sizeof(float) * hd);
        }
      }
  }
  if (c.pe_type == 2) {
    vecf t(q.size());
    rope(t.data(), q.data(), B * H * S, hd, S, T0, (double)c.rope_base);
    q.swap(t);
    t.resize(kk.size());
    rope(t.data(), kk.data(), B * Hkv * S, hd, S, T0, (double)c.rope_base);
    kk.swap(t);
  }
  // append to the cache: K [B*Hc, hd, T] (transposed), V [B*Hc, T, hd]
  cache_grow(m, L, B, T0, T1);
  for (int b = 0; b < B; ++b)
    for (int hc = 0; hc < Hc; ++hc) {
      const int g = (Hc == Hkv) ? hc : hc / group;  // expanded order [B, Hkv, group, ...] (GroupQueryAttention.cs:156-165)
      for (int s = 0; s < S; ++s) {
        const float* ks = &kk[(((size_t)b * Hkv + g) * S + s) * hd];
        const float* vs = &vv[(((size_t)b * Hkv + g) * S + s) * hd];
        for (int e = 0; e < hd; ++e) L.K[(((size_t)b * Hc + hc) * hd + e) * L.Tcap + T0 + s] = ks[e];
        std::memcpy(&L.Vc[(((size_t)b * Hc + hc) * L.Tcap + T0 + s) * hd], vs, sizeof(float) * hd);
      }
    }
  // scores = (q K) * scale (+ mask) ; softmax ; P V
  const float scale = 1.0f / (float)std::sqrt((double)hd);
  vecf merged((size_t)M * d);
  // prefill builds the causal mask (Decoder.cs:681-693); cached decode (S = 1) passes none.  S > 1 on a
  // non-empty cache (chunked prefill) does not occur in the reference; the mask is offset by T0 there.
  const bool use_mask = (S > 1);
  parallel_for(B * H, c.threads, [&](int bh) {
    const int b = bh / H, hh = bh % H;
    const int hc = (Hc == H) ? hh : hh / group;
    const float* Kp = &L.K[((size_t)b * Hc + hc) * hd * L.Tcap];
    const float* Vp = &L.Vc[((size_t)b * Hc + hc) * L.Tcap * hd];
    vecf sc((size_t)S * T1, 0.0f), ctx((size_t)S * hd, 0.0f);
    gemm_axpy(sc.data(), &q[(size_t)bh * S * hd], Kp, S, hd, T1, scale, 1, hd, L.Tcap, T1);
    if (use_mask)  // BuildTriMask 0 / -30000 (TensorApplyCPU.cs:1016-1036, ComputeGraphTensor.cs:3932)
      for (int s = 0; s < S; ++s)
        for (int t = 0; t < T1; ++t) sc[(size_t)s * T1 + t] += (t <= T0 + s ? 0.0f : -30000.0f);
    softmax(sc.data(), sc.data(), S, T1);
    gemm_axpy(ctx.data(), sc.data(), Vp, S, T1, hd, 1.0f, 1, T1, hd, hd);
    for (int s = 0; s < S; ++s)
      std::memcpy(&merged[((size_t)b * S + s) * d + hh * hd], &ctx[(size_t)s * hd], sizeof(float) * hd);
  });
  vecf o;
  affine(o, merged, L.o, M, c.threads);
  for (size_t i = 0; i < x.size(); ++i) x[i] = o[i] + x[i];  // graph.Add(finalAttResults, inputQ)
}

// MultiHeadAttention.Perform(inputQ, inputK, inputV, keyMask, ...) (Layers/MultiHeadAttention.cs:434-527) with the projected
// encoder rows taken from the cache the first step leaves (:462-488).  Mask: BuildSrcTgtMask (TensorApplyCPU.cs:1069-1096)
// adds -30000 to source positions beyond a sequence's unpadded length; the reference builds it only for batches of more than
// one sequence (Decoder.cs:283) - with one sequence there is no padding, so the rule below covers both.
void cross_attention_block(Model* m, Layer& L, vecf& x, int B, int S) {
  const OrcConfig& c = m->c;
  const int d = c.d, H = c.H, hd = c.hd, M = B * S, Ts = m->xTs;
  vecf h((size_t)M * d);
  norm_apply(m, h.data(), x.data(), L.nx_g, L.nx_b, M);
  vecf yq;
  affine(yq, h, L.xq, M, c.threads);
  const float scale = 1.0f / (float)std::sqrt((double)hd);
  vecf merged((size_t)M * d);
  parallel_for(B * H, c.threads, [&](int bh) {
    const int b = bh / H, hh = bh % H;
    vecf q((size_t)S * hd), sc((size_t)S * Ts, 0.0f), ctx((size_t)S * hd, 0.0f);
    for (int s = 0; s < S; ++s) std::memcpy(&q[(size_t)s * hd], &yq[((size_t)b * S + s) * d + hh * hd], sizeof(float) * hd);
    gemm_axpy(sc.data(), q.data(), &L.xKs[(size_t)bh * hd * Ts], S, hd, Ts, scale, 1, hd, Ts, Ts);
    for (int s = 0; s < S; ++s)
      for (int t = 0; t < Ts; ++t) sc[(size_t)s * Ts + t] += (t < m->src_lens[b] ? 0.0f : -30000.0f);
    softmax(sc.data(), sc.data(), S, Ts);
    gemm_axpy(ctx.data(), sc.data(), &L.xVs[(size_t)bh * Ts * hd], S, Ts, hd, 1.0f, 1, Ts, hd, hd);
    for (int s = 0; s < S; ++s) std::memcpy(&merged[((size_t)b * S + s) * d + hh * hd], &ctx[(size_t)s * hd], sizeof(float) * hd);
  });
  vecf o;
  affine(o, merged, L.xo, M, c.threads);
  for (size_t i = 0; i < x.size(); ++i) x[i] = o[i] + x[i];
}

// PositionwiseFeedForward.Process (Layers/PositionwiseFeedForward.cs:72-98)
void ffn_block(Model* m, Layer& L, vecf& x, int M) {
  const OrcConfig& c = m->c;
  vecf h((size_t)M * c.d);
  norm_apply(m, h.data(), x.data(), L.n2_g, L.n2_b, M);
  vecf a, g2, o;
  affine(a, h, L.w1, M, c.threads);
  for (auto& v : a) v = act_fn(c.act, v);
  if (c.act == 3 || c.act == 4) {
    affine(g2, h, L.w3, M, c.threads);
    for (size_t i = 0; i < a.size(); ++i) a[i] = a[i] * g2[i];
  }
  affine(o, a, L.w2, M, c.threads);
  for (size_t i = 0; i < x.size(); ++i) x[i] = o[i] + x[i];
}

// TensorApplyCPU.TopK / replace_smaller (TensorSharp/TensorApplyCPU.cs:1097-1146): k best values of a row in descending
// order; a value equal to the current k-th one replaces it (the later index wins at the boundary), equal values further
// up keep their order.
void topk_row(float* val, int* idx, const float* in, int cols, int k) {
  for (int i = 0; i < k; ++i) {
    val[i] = -1.70141e+38f;
    idx[i] = -1;
  }
  for (int i = 0; i < cols; ++i) {
    const float data = in[i];
    if (data < val[k - 1]) continue;
    int j = k - 2;
    for (; j >= 0; --j) {
      if (data > val[j]) {
        val[j + 1] = val[j];
        idx[j + 1] = idx[j];
      } else {
        break;
      }
    }
    val[j + 1] = data;
    idx[j + 1] = i;
  }
}

// MoEFeedForward.Process at inference (Layers/MoEFeedForward.cs:72-160): LayerNorm, router affine, the constant
// -65000 "mask" (its dropout is the identity outside training) added to every router logit - in fp32 that rounds the
// logits to multiples of 2^-7, which is part of the reference's behaviour -, softmax, TopK; then expert by expert (ascending)
// the tokens routed to it: x W1_e, activation, W2_e (no biases), times the token's router probability of that expert,
// accumulated per token in that order (IndexUpdate with accumulate on a zero tensor), and the residual add.
void moe_block(Model* m, Layer& L, vecf& x, int M) {
  const OrcConfig& c = m->c;
  const int d = c.d, E = c.n_experts, k = c.experts_per_token, Fh = 4 * d;
  vecf h((size_t)M * d);
  layernorm(h.data(), x.data(), L.moe_g.data(), L.moe_b.empty() ? nullptr : L.moe_b.data(), c.eps, M, d);
  Linear router;
  router.W = L.router_w;
  router.b = L.router_b;
  router.in = d;
  router.out = E;
  vecf r;
  affine(r, h, router, M, 1);
  for (auto& v : r) v = v + (-65000.0f);
  vecf p((size_t)M * E);
  softmax(p.data(), r.data(), M, E);
  std::vector<int> top((size_t)M * k);
  vecf topv((size_t)M * k);
  for (int i = 0; i < M; ++i) topk_row(&topv[(size_t)i * k], &top[(size_t)i * k], &p[(size_t)i * E], E, k);
  vecf res((size_t)M * d, 0.0f);
  for (int e = 0; e < E; ++e) {
    std::vector<int> rows;
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < k; ++j)
        if (top[(size_t)i * k + j] == e) rows.push_back(i);
    if (rows.empty()) continue;
    const int n = (int)rows.size();
    vecf xe((size_t)n * d), a((size_t)n * Fh, 0.0f), o((size_t)n * d, 0.0f);
    for (int q = 0; q < n; ++q) std::memcpy(&xe[(size_t)q * d], &h[(size_t)rows[q] * d], sizeof(float) * d);
    gemm_axpy(a.data(), xe.data(), &L.moe_w1[(size_t)e * d * Fh], n, d, Fh, 1.0f, c.threads);
    if (c.act == 0 || c.act == 1 || c.act == 2)   // RunActivateFunction has branches for ReLU, SiLU and LeakyReLU only (:162-178)
      for (auto& v : a) v = act_fn(c.act, v);
    gemm_axpy(o.data(), a.data(), &L.moe_w2[(size_t)e * Fh * d], n, Fh, d, 1.0f, c.threads);
    for (int q = 0; q < n; ++q) {
      const float score = p[(size_t)rows[q] * E + e];
      for (int i = 0; i < d; ++i) res[(size_t)rows[q] * d + i] += o[(size_t)q * d + i] * score;
    }
  }
  for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + res[i];
}

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11).
inline void philox4x32_10(uint32_t ctr[4], const uint32_t key_in[2]) {
  uint32_t k0 = key_in[0], k1 = key_in[1];
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * ctr[0];
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * ctr[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ ctr[1] ^ k0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ ctr[3] ^ k1;
    const uint32_t n3 = (uint32_t)p0;
    ctr[0] = n0; ctr[1] = n1; ctr[2] = n2; ctr[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

}  // namespace

extern "C" {

void* orc_create(const OrcConfig* cfg) {
  Model* m = new Model();
  m->c = *cfg;
  m->layers.resize(cfg->L);
  const int Hkv = cfg->attn_type == 1 ? cfg->Hkv : cfg->H;
  m->Hc = cfg->faithful_cache ? cfg->H : Hkv;
  return m;
}

void orc_destroy(void* h) { delete (Model*)h; }

// Names follow the reference's weight dictionary keys ("{unit}.{field}", e.g.
// GPTDecoder.SelfAttn_3.QKV, GPTDecoder.PosFFN_3.feedForwardLayer1.m_Whd, GPTDecoder.layerNorm.m_alpha,
// FeedForward_Decoder_0.m_Whd, TgtEmbeddings, PosEmbedding).  rows/cols give the [in,out] shape.
int orc_set_weight(void* h, const char* name_c, const float* data, int rows, int cols) {
  Model* m = (Model*)h;
  const std::string name(name_c);
  const size_t n = (size_t)rows * cols;
  auto assign = [&](vecf& v) { v.assign(data, data + n); return 1; };
  if (name == "TgtEmbeddings") return assign(m->E);
  if (name == "PosEmbedding") { m->c.max_pos = rows; return assign(m->PE); }
  if (name == "GPTDecoder.layerNorm.m_alpha") return assign(m->nf_g);
  if (name == "GPTDecoder.layerNorm.m_beta") return assign(m->nf_b);
  if (name.find(".layerNormQ.") != std::string::npos || name.find(".layerNorm2.") != std::string::npos) {
    const std::string rest = name.substr(11);
    const int k = std::atoi(rest.substr(rest.find('_') + 1).c_str());
    if (k < 0 || k >= (int)m->layers.size()) return 0;
    Layer& L = m->layers[k];
    const bool first = name.find(".layerNormQ.") != std::string::npos;
    if (rest.compare(0, 7, "EncAttn") == 0) {
      if (ends_with(name, "m_alpha")) return assign(L.nx_g);
      if (ends_with(name, "m_beta")) return assign(L.nx_b);
      return 0;
    }
    if (ends_with(name, "m_alpha")) return assign(first ? L.n1_g : L.n2_g);
    if (ends_with(name, "m_beta")) return assign(first ? L.n1_b : L.n2_b);
    return 0;
  }
  if (name.compare(0, 18, "GPTDecoder.MoEFFN_") == 0) {
    const std::string rest = name.substr(18);
    const int k = std::atoi(rest.c_str());
    if (k < 0 || k >= (int)m->layers.size()) return 0;
    Layer& L = m->layers[k];
    if (ends_with(name, ".layerNorm.m_alpha")) return assign(L.moe_g);
    if (ends_with(name, ".layerNorm.m_beta")) return assign(L.moe_b);
    if (ends_with(name, ".m_Whd1")) return assign(L.moe_w1);
    if (ends_with(name, ".m_Whd2")) return assign(L.moe_w2);
    if (ends_with(name, ".m_RouterBias")) return assign(L.router_b);
    if (ends_with(name, ".m_Router")) return assign(L.router_w);
    return 0;
  }
  size_t dot = name.rfind('.');
  std::string base = name.substr(0, dot), field = name.substr(dot + 1);
  Linear* lin = nullptr;
  bool is_bias = false;
  if (base == "FeedForward_Decoder_0") {
    lin = &m->head;
    is_bias = (field == "m_Bd");
  } else {
    lin = find_linear(m, name, false);
    is_bias = (field == "m_Bd" || field == "QKVb" || field == "Qb" || field == "Kb" || field == "Vb" || field == "b0");
  }
  if (!lin) return 0;
  if (is_bias) {
    lin->b.assign(data, data + n);
  } else {
    lin->W.assign(data, data + n);
    lin->in = rows;
    lin->out = cols;
  }
  return 1;
}

void orc_reset(void* h) {
  Model* m = (Model*)h;
  for (auto& L : m->layers) {
    L.K.clear();
    L.Vc.clear();
    L.Tcap = 0;
  }
  m->B = 0;
  m->T = 0;
}

int orc_cache_len(void* h) { return ((Model*)h)->T; }

// The encoder's output [B, Ts, d] and the unpadded source lengths: every layer's K = Affine(enc, K, Kb) and V likewise,
// laid out as the reference caches them (Ks [B*H, hd, Ts], Vs [B*H, Ts, hd]; MultiHeadAttention.cs:466-485).
int orc_set_encoder_output(void* h, const float* enc, const int* src_lens, int B, int Ts) {
  Model* m = (Model*)h;
  const OrcConfig& c = m->c;
  if (!c.cross_attn || B < 1 || Ts < 1) return 0;
  const int d = c.d, H = c.H, hd = c.hd;
  m->xB = B;
  m->xTs = Ts;
  m->src_lens.assign(B, Ts);
  if (src_lens) m->src_lens.assign(src_lens, src_lens + B);
  vecf e(enc, enc + (size_t)B * Ts * d);
  for (auto& L : m->layers) {
    vecf yk, yv;
    affine(yk, e, L.xk, B * Ts, c.threads);
    affine(yv, e, L.xv, B * Ts, c.threads);
    L.xKs.assign((size_t)B * H * hd * Ts, 0.0f);
    L.xVs.assign((size_t)B * H * Ts * hd, 0.0f);
    for (int b = 0; b < B; ++b)
      for (int t = 0; t < Ts; ++t)
        for (int hh = 0; hh < H; ++hh) {
          const float* kr = &yk[((size_t)b * Ts + t) * d + hh * hd];
          for (int i = 0; i < hd; ++i) L.xKs[(((size_t)b * H + hh) * hd + i) * Ts + t] = kr[i];
          std::memcpy(&L.xVs[(((size_t)b * H + hh) * Ts + t) * hd], &yv[((size_t)b * Ts + t) * d + hh * hd], sizeof(float) * hd);
        }
  }
  return 1;
}

// One forward step — Decoder.GPTDecode (Seq2SeqSharp/Applications/Decoder.cs:648-794) up to the
// probabilities.  ids is [B, S] row-major (prefill: the whole prompt with an empty cache; decode:
// S = 1, the last token).  logits/probs are [B, V]; `blocked` ids get probs += -1 (Decoder.cs:744-752).
// hidden_out (optional) receives the final-norm output of the last row of each sequence, [B, d].
int orc_step(void* h, const int* ids, int B, int S, float temperature, const int* blocked, int n_blocked,
             float* logits_out, float* probs_out, float* hidden_out) {
  Model* m = (Model*)h;
  const OrcConfig& c = m->c;
  if (m->T > 0 && B != m->B) return 0;
  m->B = B;
  const int T0 = m->T, M = B * S, d = c.d;
  vecf x((size_t)M * d);
  const float sf = (float)std::sqrt((double)d);  // scaleFactor (Decoder.cs:673,695)
  for (int r = 0; r < M; ++r) {
    const int id = ids[r];
    if (id < 0 || id >= c.V) return 0;
    for (int i = 0; i < d; ++i) x[(size_t)r * d + i] = m->E[(size_t)id * d + i] * sf;  // IndexSelect then Mul (TensorUtils.cs:135-147)
  }
  if (c.pe_type == 1) {  // PositionEmbedding.AddPositionEmbedding (Utils/PositionEmbedding.cs:28-49): Peek rows [0, S)
    for (int b = 0; b < B; ++b)
      for (int s = 0; s < S; ++s) {
        const int pos = c.ape_decode_pos0 ? s : (T0 + s);
        if (pos >= c.max_pos) return 0;
        for (int i = 0; i < d; ++i) x[((size_t)b * S + s) * d + i] += m->PE[(size_t)pos * d + i];
      }
  }
  for (int k = 0; k < c.L; ++k) {  // GPTDecoder.Decode (Networks/GPTDecoder.cs:153-191)
    attention_block(m, m->layers[k], x, B, S, T0);
    if (c.cross_attn) {   // TransformerDecoder.Decode (Networks/TransformerDecoder.cs:150-158)
      if (m->xB != B || m->xTs <= 0) return 0;
      cross_attention_block(m, m->layers[k], x, B, S);
    }
    if (c.n_experts > 1 && k > 1) moe_block(m, m->layers[k], x, M);   // GPTDecoder.cs:116
    else ffn_block(m, m->layers[k], x, M);
  }
  m->T = T0 + S;
  vecf last((size_t)B * d), hn((size_t)B * d);
  for (int b = 0; b < B; ++b) std::memcpy(&last[(size_t)b * d], &x[((size_t)b * S + S - 1) * d], sizeof(float) * d);
  norm_apply(m, hn.data(), last.data(), m->nf_g, m->nf_b, B);
  if (hidden_out) std::memcpy(hidden_out, hn.data(), sizeof(float) * hn.size());
  vecf z;
  affine(z, hn, m->head, B, c.threads);
  if (temperature != 1.0f)
    for (auto& v : z) v = v / temperature;  // g.Div(ffLayer, Temperature) (Decoder.cs:720-723)
  if (logits_out) std::memcpy(logits_out, z.data(), sizeof(float) * z.size());
  vecf p(z.size());
  softmax(p.data(), z.data(), B, c.V);
  for (int b = 0; b < B; ++b)
    for (int j = 0; j < n_blocked; ++j) p[(size_t)b * c.V + blocked[j]] += -1.0f;
  if (probs_out) std::memcpy(probs_out, p.data(), sizeof(float) * p.size());
  return 1;
}

// ---- op-level exports (used by the op parity tests and golden-vector pins) ----
void orc_layernorm(float* out, const float* in, const float* g, const float* b, float eps, int rows, int cols) { layernorm(out, in, g, b, eps, rows, cols); }
void orc_rmsnorm(float* out, const float* in, const float* g, const float* b, float eps, int rows, int cols) { rmsnorm(out, in, g, b, eps, rows, cols); }
void orc_softmax(float* out, const float* in, int rows, int cols) { softmax(out, in, rows, cols); }
void orc_rope(float* out, const float* in, int rows, int cols, int seqLen, int rowOffset, double base) { rope(out, in, rows, cols, seqLen, rowOffset, base); }
void orc_argmax(int* out, const float* p, int rows, int cols) { argmax_rows(out, p, rows, cols); }
void orc_topk(float* val, int* idx, const float* in, int rows, int cols, int k) {
  for (int r = 0; r < rows; ++r) topk_row(val + (long)r * k, idx + (long)r * k, in + (long)r * cols, cols, k);
}
// C = beta*src + alpha*A*B, row-major (CpuBasicOps.Addmm, TensorSharp/Cpu/CpuBasicOps.cs:49-114)
void orc_addmm(float* C, float beta, const float* src, float alpha, const float* A, const float* Bm, int M, int K, int N) {
  for (long i = 0; i < (long)M * N; ++i) C[i] = (beta == 0.0f) ? 0.0f : (beta == 1.0f ? src[i] : beta * src[i]);
  gemm_axpy(C, A, Bm, M, K, N, alpha, 1);
}
void orc_act(float* out, const float* in, long n, int act) {
  for (long i = 0; i < n; ++i) out[i] = act_fn(act, in[i]);
}
// TensorSharp/TensorApplyCPU.cs:1306-1333 (indices are floats in the reference; negative = skip)
void orc_indexselect(float* out, const float* src, const float* idx, int rows, int cols) {
  for (int j = 0; j < rows; ++j) {
    const int s = (int)idx[j];
    if (s >= 0) std::memcpy(out + (long)j * cols, src + (long)s * cols, sizeof(float) * cols);
  }
}
// seqs is [B, seq_stride] with seq_lens[b] valid entries; u is [B]; out is [B].
void orc_topp(int* out, const float* probs, int B, int V, float topP, float repeatPenalty, const int* seqs,
              const int* seq_lens, int seq_stride, const float* u, int* n_cands, float* acc) {
  for (int b = 0; b < B; ++b)
    out[b] = topp_row(probs + (long)b * V, V, topP, repeatPenalty, seqs ? seqs + (long)b * seq_stride : nullptr,
                      seq_lens ? seq_lens[b] : 0, u[b], n_cands ? n_cands + b : nullptr, acc ? acc + b : nullptr);
}
void orc_philox4x32_10(uint32_t* out4, const uint32_t* ctr4, const uint32_t* key2) {
  uint32_t c[4] = {ctr4[0], ctr4[1], ctr4[2], ctr4[3]};
  philox4x32_10(c, key2);
  std::memcpy(out4, c, sizeof(c));
}
// Uniform draw for (seed, sequence, step): key = (seed lo, seed hi), counter = (step, 0, seq lo, seq hi);
// u = (x0 >> 8) * 2^-24  in [0, 1).
float orc_philox_uniform(uint64_t seed, uint64_t seq, uint32_t step) {
  uint32_t c[4] = {step, 0u, (uint32_t)seq, (uint32_t)(seq >> 32)};
  const uint32_t k[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  philox4x32_10(c, k);
  return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}
int orc_max_threads() {
  const unsigned n = std::thread::hardware_concurrency();
  return n ? (int)n : 1;
}

}  // extern "C"
