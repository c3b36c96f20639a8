"""Host-side mirror of the reference's GPT application for the B200 backend.

Names follow Seq2SeqSharp: `DecodingOptions` (Seq2SeqSharp/Applications/DecodingOptions.cs:16-39),
`GPT.RunForwardOnSingleDevice` (Seq2SeqSharp/Applications/GPT.cs:212-335), weight keys as stored by
IModel.AddWeights (Seq2SeqSharp/Tools/WeightTensor.cs:571-604).  The work is done by the GPT engine of
libtsb200.so through the C ABI; this module only marshals.  There is no CPU path.
"""
import ctypes as C
from dataclasses import dataclass, field
from enum import IntEnum
from typing import Dict, List, Optional

import numpy as np

from . import _native as N
from .synthetic import synth


class DecodingStrategyEnums(IntEnum):  # Seq2SeqSharp/Utils/DecodingStrategyEnums.cs
    GreedySearch = 0
    Sampling = 1


class NormEnums(IntEnum):
    LayerNorm = 0
    RMSNorm = 1


class ActivateFuncEnums(IntEnum):  # Seq2SeqSharp/Utils/ActivateFuncEnums.cs:5-12 (+ two extensions)
    ReLU = 0
    SiLU = 1
    LeakyReLU = 2
    SwiGLU = 3        # the reference's SwiGLU: (xW1+b1) * (xW3+b3), no SiLU (PositionwiseFeedForward.cs:82-116)
    SwiGLU_SiLU = 4   # extension: silu(xW1+b1) * (xW3+b3)
    GELU = 5          # extension: erf GELU


class PositionEmbeddingEnums(IntEnum):  # Seq2SeqSharp/Utils/PositionEmbedding.cs:18-23
    NoPE = 0
    APE = 1
    RoPE = 2


class MultiHeadAttentionTypeEnums(IntEnum):
    MHA = 0
    GQA = 1


@dataclass
class DecodingOptions:
    MaxSrcSentLength: int = 128     # lines of an input file are cut to this many tokens less two (Applications/DecodingOptions.cs:18)
    MaxTgtSentLength: int = 256
    RepeatPenalty: float = 2.0
    BeamSearchSize: int = 1
    Temperature: float = 1.0
    TopP: float = 1.0
    DecodingStrategy: DecodingStrategyEnums = DecodingStrategyEnums.GreedySearch
    BlockedTokens: Optional[List[int]] = None
    # counter-based uniform stream replacing the process-wide System.Random (Tools/RandomGenerator.cs:41-46)
    Seed: int = 0
    SeqBase: int = 0


@dataclass
class GPTConfig:
    """Shape and behaviour switches of GPTDecoder (Seq2SeqSharp/Networks/GPTDecoder.cs:40-133)."""
    L: int
    d: int
    H: int
    hd: int
    F: int
    V: int
    Hkv: int = 0
    norm: NormEnums = NormEnums.LayerNorm
    act: ActivateFuncEnums = ActivateFuncEnums.ReLU
    pe: PositionEmbeddingEnums = PositionEmbeddingEnums.RoPE
    attn: MultiHeadAttentionTypeEnums = MultiHeadAttentionTypeEnums.MHA
    dtype: str = "float32"          # "float32" | "float16"
    eps: float = 1e-6               # Layers/LayerNormalization.cs:36, RMSNormalization.cs:26
    rope_base: float = 500000.0     # TensorSharp/TensorApplyCPU.cs:1162
    ape_decode_pos0: bool = True    # Decoder.cs:674-677 adds APE row 0 in cached decode
    name: str = ""
    expertNum: int = 1              # > 1: layers 2.. use MoEFeedForward (Networks/GPTDecoder.cs:114-123), experts [d, 4d] and [4d, d]
    expertsPerTokenFactor: int = 1  # experts per token (TopK of the router's softmax, Layers/MoEFeedForward.cs:84)
    cross_attn: bool = False        # TransformerDecoder (Networks/TransformerDecoder.cs): every layer also attends to an encoder's output
    max_src_tokens: int = 0         # capacity of the encoder output per sequence (cross_attn models)

    def is_moe_layer(self, k: int) -> bool:
        return self.expertNum > 1 and k > 1

    def kv_heads(self):
        return self.Hkv if (self.attn == MultiHeadAttentionTypeEnums.GQA and self.Hkv) else self.H

    def is_glu(self):
        return self.act in (ActivateFuncEnums.SwiGLU, ActivateFuncEnums.SwiGLU_SiLU)

    def weight_shapes(self, max_pos: int = 0) -> Dict[str, tuple]:
        """Reference weight keys -> [rows, cols] (every linear has a bias; LM head is separate from the embedding)."""
        d, F, V, Hd, KVd = self.d, self.F, self.V, self.H * self.hd, self.kv_heads() * self.hd
        s = {"TgtEmbeddings": (V, d)}
        if self.pe == PositionEmbeddingEnums.APE and max_pos:
            s["PosEmbedding"] = (max_pos, d)
        for k in range(self.L):
            a, f = "GPTDecoder.SelfAttn_%d." % k, "GPTDecoder.PosFFN_%d." % k
            s[a + "layerNormQ.m_alpha"] = (1, d)
            if self.norm == NormEnums.LayerNorm:
                s[a + "layerNormQ.m_beta"] = (1, d)
            if self.attn == MultiHeadAttentionTypeEnums.MHA:
                s[a + "QKV"] = (d, 3 * Hd)
                s[a + "QKVb"] = (1, 3 * Hd)
            else:
                s[a + "Q"], s[a + "Qb"] = (d, Hd), (1, Hd)
                s[a + "K"], s[a + "Kb"] = (d, KVd), (1, KVd)
                s[a + "V"], s[a + "Vb"] = (d, KVd), (1, KVd)
            s[a + "W0"], s[a + "b0"] = (Hd, d), (1, d)
            if self.cross_attn:
                # MultiHeadAttention without shared QKV (TransformerDecoder.cs:86-92, MultiHeadAttention.cs:76-86)
                e = "GPTDecoder.EncAttn_%d." % k
                s[e + "layerNormQ.m_alpha"] = (1, d)
                if self.norm == NormEnums.LayerNorm:
                    s[e + "layerNormQ.m_beta"] = (1, d)
                for n in ("Q", "K", "V"):
                    s[e + n], s[e + n + "b"] = (d, Hd), (1, Hd)
                s[e + "W0"], s[e + "b0"] = (Hd, d), (1, d)
            if self.is_moe_layer(k):
                # MoEFeedForward (Layers/MoEFeedForward.cs:31-52): always LayerNorm; experts without bias; 3-D tensors are
                # handed over as [E * rows, cols]
                m, E = "GPTDecoder.MoEFFN_%d." % k, self.expertNum
                s[m + "layerNorm.m_alpha"], s[m + "layerNorm.m_beta"] = (1, d), (1, d)
                s[m + "m_Whd1"], s[m + "m_Whd2"] = (E * d, 4 * d), (E * 4 * d, d)
                s[m + "m_Router"], s[m + "m_RouterBias"] = (d, E), (1, E)
                continue
            s[f + "layerNorm2.m_alpha"] = (1, d)
            if self.norm == NormEnums.LayerNorm:
                s[f + "layerNorm2.m_beta"] = (1, d)
            s[f + "feedForwardLayer1.m_Whd"], s[f + "feedForwardLayer1.m_Bd"] = (d, F), (1, F)
            if self.is_glu():
                s[f + "feedForwardLayer3.m_Whd"], s[f + "feedForwardLayer3.m_Bd"] = (d, F), (1, F)
            s[f + "feedForwardLayer2.m_Whd"], s[f + "feedForwardLayer2.m_Bd"] = (F, d), (1, d)
        s["GPTDecoder.layerNorm.m_alpha"] = (1, d)
        if self.norm == NormEnums.LayerNorm:
            s["GPTDecoder.layerNorm.m_beta"] = (1, d)
        s["FeedForward_Decoder_0.m_Whd"], s["FeedForward_Decoder_0.m_Bd"] = (d, V), (1, V)
        return s

    def matmul_params(self):
        d, F, V, Hd, KVd = self.d, self.F, self.V, self.H * self.hd, self.kv_heads() * self.hd
        return self.L * (d * (Hd + 2 * KVd) + Hd * d + (3 if self.is_glu() else 2) * d * F) + d * V


def is_bias(name: str) -> bool:
    return name.endswith(("m_Bd", "QKVb", ".Qb", ".Kb", ".Vb", ".b0", "m_RouterBias"))


def is_norm(name: str) -> bool:
    return name.endswith(("m_alpha", "m_beta"))


def synthetic_weights(cfg: GPTConfig, seed: int, std: float = 0.02, bias_std: float = 0.0, max_pos: int = 0):
    """Seeded weights keyed by the reference names: matrices ~ N(0, std); norm gains 1, betas 0; biases 0 (the
    reference default) or N(0, bias_std).  Values are float32; for a float16 model they are rounded to half once
    (round-to-nearest-even) and returned as float32 holding the rounded values, so the oracle sees what the device sees."""
    out = {}
    for name, shape in cfg.weight_shapes(max_pos).items():
        if name.endswith("m_alpha"):
            w = np.ones(shape, dtype=np.float32)
        elif name.endswith("m_beta"):
            w = np.zeros(shape, dtype=np.float32)
        elif is_bias(name):
            w = synth(name, shape, seed, bias_std) if bias_std > 0 else np.zeros(shape, dtype=np.float32)
        else:
            w = synth(name, shape, seed, std)
        if cfg.dtype == "float16":
            w = w.astype(np.float16).astype(np.float32)
        out[name] = w
    return out


def tp_shard_weights(cfg: GPTConfig, weights: Dict[str, np.ndarray], rank: int, n: int) -> Dict[str, np.ndarray]:
    """This rank's share of every weight under n-way tensor parallelism — the same rule the engine applies when it is
    handed full tensors (csrc/engine.cu: resolve): query heads, KV heads and FFN columns are cut into n contiguous blocks;
    Q/K/V/W1/W3 (and their biases) are column blocks, W0/W2 are row blocks, the biases of W0/W2 stay on rank 0 only,
    everything else (embeddings, norms, LM head) is replicated."""
    Hd, KVd, F = cfg.H * cfg.hd, cfg.kv_heads() * cfg.hd, cfg.F
    hq, hk, f = Hd // n, KVd // n, F // n
    out = {}
    for name, w in weights.items():
        w = np.asarray(w)
        if name.endswith(".W0"):
            w = w[rank * hq:(rank + 1) * hq]
        elif name.endswith("feedForwardLayer2.m_Whd"):
            w = w[rank * f:(rank + 1) * f]
        elif name.endswith((".b0", "feedForwardLayer2.m_Bd")):
            w = w if rank == 0 else np.zeros_like(w)
        elif name.endswith((".QKV", ".QKVb")):
            w = np.concatenate([w[:, p * Hd + rank * hq:p * Hd + (rank + 1) * hq] for p in range(3)], axis=1)
        elif name.endswith((".Q", ".Qb")):
            w = w[:, rank * hq:(rank + 1) * hq]
        elif name.endswith((".K", ".Kb", ".V", ".Vb")):
            w = w[:, rank * hk:(rank + 1) * hk]
        elif name.endswith(("feedForwardLayer1.m_Whd", "feedForwardLayer1.m_Bd", "feedForwardLayer3.m_Whd", "feedForwardLayer3.m_Bd")):
            w = w[:, rank * f:(rank + 1) * f]
        out[name] = np.ascontiguousarray(w)
    return out


class GPT:
    """One GPT replica on one device (the reference builds one per device id through
    MultiProcessorNetworkWrapper.GetNetworkOnDevice, Seq2SeqSharp/Applications/GPT.cs:138-146)."""

    def __init__(self, cfg: GPTConfig, device_id: int = 0, max_batch: int = 1, max_tokens: int = 512, tp_rank: int = 0,
                 tp_size: int = 1):
        """tp_size > 1: this process holds rank `tp_rank` of a tensor-parallel group (one process per GPU); weights are
        still handed over as FULL tensors, the engine keeps its share; call InitComm() before running."""
        self.cfg = cfg
        self._comm = C.c_void_p()
        self.device_id = device_id
        self.max_batch = max_batch
        self.max_tokens = max_tokens
        c = N.GptConfig()
        c.L, c.d, c.H, c.Hkv, c.hd, c.F, c.V = cfg.L, cfg.d, cfg.H, cfg.kv_heads(), cfg.hd, cfg.F, cfg.V
        c.norm_type, c.act, c.pe_type, c.attn_type = int(cfg.norm), int(cfg.act), int(cfg.pe), int(cfg.attn)
        c.dtype = N.F16 if cfg.dtype == "float16" else N.F32
        c.eps, c.rope_base = cfg.eps, cfg.rope_base
        c.ape_decode_pos0 = 1 if cfg.ape_decode_pos0 else 0
        c.max_batch, c.max_tokens, c.device = max_batch, max_tokens, device_id
        c.tp_rank, c.tp_size = tp_rank, tp_size
        c.n_experts, c.experts_per_token = cfg.expertNum, cfg.expertsPerTokenFactor
        c.cross_attn, c.max_src_tokens = (1 if cfg.cross_attn else 0), int(cfg.max_src_tokens)
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self._h = C.c_void_p()
        N.call("TSB200_GptCreate", C.byref(c), C.byref(self._h))
        self._keep = None

    def InitComm(self, group=None, peer=True):
        """Creates the NCCL communicator of the tensor-parallel group: rank 0 makes the id, torch.distributed (any
        backend) carries its 128 bytes to the other ranks."""
        import torch.distributed as dist
        buf = (C.c_ubyte * 128)()
        if self.tp_rank == 0:
            N.call("TSB200_CommGetUniqueId", buf)
        box = [bytes(buf)]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        ident = (C.c_ubyte * 128).from_buffer_copy(box[0])
        N.call("TSB200_CommInitRank", ident, self.tp_rank, self.tp_size, self.device_id, C.byref(self._comm))
        # peer-memory all-reduce for decode-sized messages: exchange the IPC handles of the ranks' regions
        if peer and self.tp_size <= 8:
            mine = (C.c_ubyte * 64)()
            N.call("TSB200_CommPeerExport", self._comm, self.max_batch * self.cfg.d, mine)
            allh = [None] * self.tp_size
            dist.all_gather_object(allh, bytes(mine), group=group)
            blob = (C.c_ubyte * (64 * self.tp_size)).from_buffer_copy(b"".join(allh))
            N.call("TSB200_CommPeerImport", self._comm, blob, self.tp_size)
            if self.cfg.dtype == "float16":
                # exchange region of the persistent decode-step kernel (the collective happens inside that kernel)
                N.call("TSB200_GptTpExport", self._h, mine)
                dist.all_gather_object(allh, bytes(mine), group=group)
                blob = (C.c_ubyte * (64 * self.tp_size)).from_buffer_copy(b"".join(allh))
                N.call("TSB200_GptTpImport", self._h, blob, self.tp_size)
        N.call("TSB200_GptSetComm", self._h, self._comm)
        self._group, self._peer_mapped = group, bool(peer and self.tp_size <= 8)

    def close(self, barrier=None):
        """Frees the engine.  A tensor-parallel engine whose ranks mapped each other's memory is torn down in two
        phases: every rank unmaps its peers' regions, the ranks meet at a host barrier (`barrier`, default
        torch.distributed.barrier on the group given to InitComm), then each rank frees its own region."""
        if getattr(self, "_peer_mapped", False) and getattr(self, "_h", None) and self._h.value:
            self._peer_mapped = False
            N.lib().TSB200_GptTpClose(self._h)
            if self._comm.value:
                N.lib().TSB200_CommPeerClose(self._comm)
            if barrier is None:
                def barrier():
                    import torch.distributed as dist
                    if dist.is_available() and dist.is_initialized():
                        dist.barrier(group=self._group)
            barrier()
        if getattr(self, "_h", None) and self._h.value:
            N.lib().TSB200_GptDestroy(self._h)
            self._h = C.c_void_p()
        if getattr(self, "_comm", None) and self._comm.value:
            N.lib().TSB200_CommDestroy(self._comm)
            self._comm = C.c_void_p()

    def __del__(self):
        try:
            self.close(barrier=lambda: None)  # a finalizer cannot take part in a collective: call close() explicitly
        except Exception:
            pass

    @property
    def pos_embedding_rows(self):
        return self.max_tokens + 2

    # ---- weights -----------------------------------------------------------------------------------
    def LoadWeights(self, weights: Dict[str, np.ndarray]):
        """IModel.GetWeights equivalent: full tensors by reference key (float32 or float16 numpy arrays)."""
        for name, w in weights.items():
            w = np.ascontiguousarray(w)
            if w.dtype == np.float16:
                dt = N.F16
            else:
                w = w.astype(np.float32, copy=False)
                dt = N.F32
            rows, cols = (w.shape if w.ndim == 2 else (1, w.size))
            N.call("TSB200_GptSetWeight", self._h, name.encode(), w.ctypes.data_as(C.c_void_p), dt, rows, cols, 0)

    def FillSynthetic(self, seed: int, std: float = 0.02, bias_std: float = 0.0):
        """Same values as synthetic_weights(), generated on the device (for models too large to stage from the host)."""
        N.call("TSB200_GptFillSynthetic", self._h, seed, std, bias_std)

    # ---- token loop --------------------------------------------------------------------------------
    def _opts(self, o: DecodingOptions):
        c = N.DecodingOptionsC()
        c.strategy = int(o.DecodingStrategy)
        c.topP, c.temperature, c.repeatPenalty = o.TopP, o.Temperature, o.RepeatPenalty
        bl = list(o.BlockedTokens or [])
        arr = (C.c_int32 * max(1, len(bl)))(*bl)
        c.blocked = C.cast(arr, C.POINTER(C.c_int32))
        c.n_blocked = len(bl)
        c.seed, c.seq_base = o.Seed, o.SeqBase
        self._keep = arr
        return c

    def Reset(self):
        N.call("TSB200_GptReset", self._h)
        self._B = 0

    def SetWaitLimit(self, polls: int):
        """Bound of the device-side waits of the persistent decode-step kernel (0 = default, about a second)."""
        N.call("TSB200_GptSetWaitLimit", self._h, int(polls))

    def Prefill(self, tokens, opts: DecodingOptions):
        ids = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        if ids.ndim != 2:
            raise ValueError("tokens must be [batch, prompt_len] with equal prompt lengths")
        B, S = ids.shape
        if self.cfg.cross_attn and S > 1:
            # the cross-attention block takes one new position per call: a longer target prefix goes in token by token
            out = self.Prefill(ids[:, :1], opts)
            for s in range(1, S):
                out = self.StepHost(ids[:, s], opts)
            return out
        out = np.zeros(B, dtype=np.int32)
        c = self._opts(opts)
        N.call("TSB200_GptPrefill", self._h, ids.ctypes.data_as(C.c_void_p), B, S, C.byref(c),
               out.ctypes.data_as(C.c_void_p))
        self._B = B
        return out

    def PrefillRagged(self, prompts, opts: DecodingOptions):
        """Prompts of different lengths in one prefill (the reference pads them: BuildInTokens.PadSentences +
        BuildSelfTriMask, Decoder.cs:656,687-692).  `prompts`: a list of id lists.  Every sequence keeps its own cache
        length and continues as if it had been run alone.  Returns the next id of every sequence."""
        lens = np.array([len(p) for p in prompts], dtype=np.int32)
        B, S = len(prompts), int(lens.max())
        ids = np.zeros((B, S), dtype=np.int32)
        for b, p in enumerate(prompts):
            ids[b, :len(p)] = np.asarray(p, dtype=np.int32)
        out = np.zeros(B, dtype=np.int32)
        c = self._opts(opts)
        N.call("TSB200_GptPrefillRagged", self._h, ids.ctypes.data_as(C.c_void_p), lens.ctypes.data_as(C.c_void_p), B, S, C.byref(c),
               out.ctypes.data_as(C.c_void_p))
        self._B = B
        return out

    def Batch(self) -> int:
        """Sequences the engine currently holds."""
        return self._B

    def CacheLengths(self):
        lens = np.zeros(self._B, dtype=np.int32)
        N.call("TSB200_GptCacheLengths", self._h, lens.ctypes.data_as(C.c_void_p), self._B)
        return lens

    # ---- one sequence of the batch at a time (the others keep their state)
    def SlotSnapshot(self, slot: int) -> "KvSnapshot":
        h = C.c_void_p()
        N.call("TSB200_GptSlotSnapshot", self._h, int(slot), C.byref(h))
        return KvSnapshot(h)

    def SlotRestore(self, snap: "KvSnapshot", slot: int):
        N.call("TSB200_GptSlotRestore", self._h, snap._h, int(slot))
        self._B = max(self._B, slot + 1)

    def SlotReset(self, slot: int):
        N.call("TSB200_GptSlotReset", self._h, int(slot))
        self._B = max(self._B, slot + 1)

    def SetPerSequenceState(self, on: bool = True):
        """Keeps the per-sequence lengths / stop rule in use even while the sequences agree (slot schedulers)."""
        N.call("TSB200_GptSetPerSequenceState", self._h, 1 if on else 0)

    def SlotExtend(self, slot: int, tokens, opts: DecodingOptions) -> int:
        """Runs `tokens` (one sequence's prompt, or the rest of it) on top of what the slot holds; returns its next id."""
        ids = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(-1))
        out = np.zeros(1, dtype=np.int32)
        c = self._opts(opts)
        N.call("TSB200_GptSlotExtend", self._h, int(slot), ids.ctypes.data_as(C.c_void_p), int(ids.size), C.byref(c),
               out.ctypes.data_as(C.c_void_p))
        self._B = max(self._B, slot + 1)
        return int(out[0])

    def Decode(self, n_steps: int, opts: DecodingOptions, stop_on_eos: bool = False):
        out = np.zeros((self._B, n_steps), dtype=np.int32)
        done = C.c_int(0)
        c = self._opts(opts)
        N.call("TSB200_GptDecode", self._h, n_steps, C.byref(c), 1 if stop_on_eos else 0,
               out.ctypes.data_as(C.c_void_p), C.byref(done))
        return out[:, :done.value]

    def BeamSearch(self, tokens, decodingOptions: DecodingOptions):
        """tokens [B, promptLen] -> `beam.BeamResult`: the BeamSearchSize hypotheses of every prompt in the reference's beam
        order, each held as a sequence of this engine with its own cache (needs max_batch >= B * BeamSearchSize)."""
        from .beam import beam_search
        return beam_search(self, tokens, decodingOptions)

    def RunForwardOnSingleDevice(self, tokens, decodingOptions: DecodingOptions, stop_on_eos: bool = True):
        """tokens [B, promptLen] -> generated ids [B, n] with n <= MaxTgtSentLength - promptLen: the loop
        `for (i = promptLen; i < MaxTgtSentLength; i++)` with the all-sequences-ended-with-EOS stop rule
        (GPT.cs:249-304).  Raises TSB200OutOfMemory where the reference returns NetworkResultStatus.OOM."""
        if decodingOptions.BeamSearchSize > 1:
            raise ValueError("RunForwardOnSingleDevice returns one hypothesis per prompt; BeamSearch() serves BeamSearchSize > 1")
        ids = np.asarray(tokens, dtype=np.int32)
        B, S = ids.shape
        n_new = decodingOptions.MaxTgtSentLength - S
        if n_new <= 0:
            return np.zeros((B, 0), dtype=np.int32)
        self.Reset()
        first = self.Prefill(ids, decodingOptions)
        if n_new == 1 or (stop_on_eos and bool(np.all(first == 0))):
            return first[:, None]
        rest = self.Decode(n_new - 1, decodingOptions, stop_on_eos=stop_on_eos)
        return np.concatenate([first[:, None], rest], axis=1)

    def Extend(self, tokens, opts: DecodingOptions):
        """tokens [B, S]: the text from the cache length on (the suffix of a prompt whose head is cached).  Appends
        them to the cache and returns the next id per sequence."""
        ids = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        if ids.ndim != 2:
            raise ValueError("tokens must be [batch, suffix_len]")
        B, S = ids.shape
        out = np.zeros(B, dtype=np.int32)
        c = self._opts(opts)
        N.call("TSB200_GptExtend", self._h, ids.ctypes.data_as(C.c_void_p), B, S, C.byref(c),
               out.ctypes.data_as(C.c_void_p))
        return out

    def CacheSnapshot(self) -> "KvSnapshot":
        """Parks the cache (every layer's K/V rows, the token history, the pending id) in a device buffer."""
        h = C.c_void_p()
        N.call("TSB200_GptCacheSnapshot", self._h, C.byref(h))
        return KvSnapshot(h)

    def CacheRestore(self, snap: "KvSnapshot", batch: int = 0):
        """Writes a parked cache back; `batch` > 1 with a one-sequence snapshot serves every slot from it."""
        N.call("TSB200_GptCacheRestore", self._h, snap._h, int(batch))
        self._B = batch if batch > 0 else snap.B

    def StepHost(self, last_ids, opts: DecodingOptions):
        """One decode step with host buffers: ids in -> ids out (what the reference does per token)."""
        ids = np.ascontiguousarray(last_ids, dtype=np.int32)
        out = np.empty_like(ids)
        c = self._opts(opts)
        N.call("TSB200_GptStepHost", self._h, ids.ctypes.data_as(C.c_void_p), C.byref(c), out.ctypes.data_as(C.c_void_p))
        return out

    def SetEncoderOutput(self, enc, src_lens=None, replicas: int = 1):
        """enc [B, S_src, d] (float32 or float16 array): the encoder's output for the sequences to come; src_lens: unpadded
        source lengths (keys beyond them are not attended).  replicas > 1: sequence b + k * B reads source b (beam search).
        Computes every layer's cross-attention K and V rows once; stays until the next call."""
        enc = np.ascontiguousarray(enc)
        if enc.dtype not in (np.float32, np.float16):
            enc = enc.astype(np.float32)
        if enc.ndim != 3 or enc.shape[2] != self.cfg.d:
            raise ValueError("encoder output must be [batch, source_len, %d]" % self.cfg.d)
        B, S = enc.shape[0], enc.shape[1]
        lens = None if src_lens is None else np.ascontiguousarray(src_lens, dtype=np.int32)
        N.call("TSB200_GptSetEncoderOutput", self._h, enc.ctypes.data_as(C.c_void_p), N.F16 if enc.dtype == np.float16 else N.F32, 0,
               lens.ctypes.data_as(C.c_void_p) if lens is not None else None, B, S, int(replicas))

    def BeamCandidates(self, K: int, opts: DecodingOptions):
        """The K best next ids of every sequence after the latest forward, as the reference's beam loop finds them:
        (ids [sequences, K], probabilities, natural logarithms)."""
        B = self._B
        ids = np.zeros((B, K), dtype=np.int32)
        p = np.zeros((B, K), dtype=np.float32)
        lp = np.zeros((B, K), dtype=np.float32)
        c = self._opts(opts)
        N.call("TSB200_GptBeamCandidates", self._h, int(K), C.byref(c), ids.ctypes.data_as(C.c_void_p), p.ctypes.data_as(C.c_void_p),
               lp.ctypes.data_as(C.c_void_p))
        return ids, p, lp

    def BeamCopy(self, src, dst):
        """Sequence src[i] over sequence dst[i]; a destination equal to the number of sequences adds one."""
        src = np.ascontiguousarray(src, dtype=np.int32)
        dst = np.ascontiguousarray(dst, dtype=np.int32)
        if src.size != dst.size:
            raise ValueError("BeamCopy: as many sources as destinations")
        if src.size == 0:
            return
        N.call("TSB200_GptBeamCopy", self._h, src.ctypes.data_as(C.c_void_p), dst.ctypes.data_as(C.c_void_p), int(src.size))
        self._B = max(self._B, int(dst.max()) + 1)

    def EnableStepTiming(self, on=True):
        N.call("TSB200_GptEnableStepTiming", self._h, 1 if on else 0)

    def StepTimes(self, n):
        ms = np.zeros(n, dtype=np.float32)
        got = C.c_int(0)
        N.call("TSB200_GptGetStepTimes", self._h, ms.ctypes.data_as(C.c_void_p), n, C.byref(got))
        return ms[:got.value]

    KERNEL_CLASSES = ("embed", "norm", "linear", "rope_append", "attention", "sampling", "commit", "allreduce", "decode_stack")

    def ProfileDecode(self, n_steps, opts: DecodingOptions):
        """{class: (ms_total, launch_groups)} over n_steps un-captured decode steps (CUDA events per launch group)."""
        n = len(self.KERNEL_CLASSES)
        ms = np.zeros(n, dtype=np.float32)
        groups = np.zeros(n, dtype=np.int64)
        c = self._opts(opts)
        N.call("TSB200_GptProfileDecode", self._h, n_steps, C.byref(c), ms.ctypes.data_as(C.c_void_p),
               groups.ctypes.data_as(C.c_void_p), n)
        return {k: (float(ms[i]), int(groups[i])) for i, k in enumerate(self.KERNEL_CLASSES)}

    # ---- inspection --------------------------------------------------------------------------------
    def Logits(self, want_probs=True):
        B, V = self._B, self.cfg.V
        lg = np.empty((B, V), dtype=np.float32)
        pr = np.empty((B, V), dtype=np.float32) if want_probs else None
        N.call("TSB200_GptGetLogits", self._h, lg.ctypes.data_as(C.c_void_p),
               pr.ctypes.data_as(C.c_void_p) if pr is not None else None)
        return lg, pr

    def CacheLength(self):
        t = C.c_int(0)
        N.call("TSB200_GptCacheLength", self._h, C.byref(t))
        return t.value

    def CheckGuards(self):
        """Raises if any kernel wrote outside one of the engine's device buffers (guard regions around every buffer)."""
        N.call("TSB200_GptCheckGuards", self._h)

    def DecodePath(self):
        """How the most recent cached step ran: 0 per-operation launches, 1 stream-K persistent kernel, 2 owner-partitioned kernel."""
        t = C.c_int(0)
        N.call("TSB200_GptDecodePath", self._h, C.byref(t))
        return t.value

    def LastTiming(self):
        ms, n = C.c_float(0), C.c_int64(0)
        N.call("TSB200_GptLastTiming", self._h, C.byref(ms), C.byref(n))
        return ms.value, n.value

    def StepBytes(self, B, T):
        b = C.c_int64(0)
        N.call("TSB200_GptStepBytes", self._h, B, T, C.byref(b))
        return b.value


class KvSnapshot:
    """Handle of a parked KV cache (device memory); `tokens` [B, T+1] = cached text + the pending id."""

    def __init__(self, handle):
        self._h = handle
        B, T, nbytes = C.c_int(0), C.c_int(0), C.c_int64(0)
        N.call("TSB200_GptCacheSnapshotInfo", self._h, C.byref(B), C.byref(T), C.byref(nbytes), None)
        self.B, self.T, self.nbytes = B.value, T.value, nbytes.value
        self.tokens = np.zeros((self.B, self.T + 1), dtype=np.int32)
        N.call("TSB200_GptCacheSnapshotInfo", self._h, None, None, None, self.tokens.ctypes.data_as(C.c_void_p))

    def close(self):
        if self._h is not None:
            N.call("TSB200_GptCacheSnapshotFree", self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KvCachePool:
    """The reference parks the K/V tensors of a finished call in MemoryCache.Default under the call's text for ten
    minutes and picks them up when the next request's text equals that key (GPT.cs:153-173 key, :236-247 lookup,
    :312-328 store).  Here the key is the token-id text itself (ids 0 = </s> dropped, as GenerateCacheKey drops
    "</s>"), entries are device snapshots, and a lookup also accepts an entry whose cached tokens are a proper
    prefix of the request (the longest one wins), so a shared prompt head is computed once."""

    def __init__(self, ttl_seconds: float = 600.0, max_bytes: int = 8 << 30, clock=None):
        import time
        self._clock = clock or time.monotonic
        self.ttl, self.max_bytes = float(ttl_seconds), int(max_bytes)
        self._entries: Dict[tuple, tuple] = {}  # key -> (snapshot, expiry)
        self.hits = self.misses = 0

    @staticmethod
    def key_of(tokens) -> tuple:
        return tuple(int(t) for t in np.asarray(tokens).reshape(-1) if int(t) != 0)

    def _expire(self):
        now = self._clock()
        for k in [k for k, (_, exp) in self._entries.items() if exp <= now]:
            self._entries.pop(k)[0].close()

    @property
    def nbytes(self):
        return sum(sn.nbytes for sn, _ in self._entries.values())

    def __len__(self):
        self._expire()
        return len(self._entries)

    def put(self, snap: KvSnapshot):
        """Stores a one-sequence snapshot under its text; the oldest entries leave when the byte budget is exceeded."""
        if snap.B != 1:
            raise ValueError("the pool keeps one sequence per entry")
        self._expire()
        key = self.key_of(snap.tokens[0])
        old = self._entries.pop(key, None)
        if old:
            old[0].close()
        self._entries[key] = (snap, self._clock() + self.ttl)
        while self.nbytes > self.max_bytes and len(self._entries) > 1:
            k = min(self._entries, key=lambda k: self._entries[k][1])
            self._entries.pop(k)[0].close()

    def take(self, prompt) -> Optional[KvSnapshot]:
        """Removes and returns the entry that covers the longest head of `prompt` (the reference removes a hit from
        the cache, GPT.cs:245), or None.  An entry qualifies if its T cached tokens equal prompt[:T] and T < len(prompt)."""
        self._expire()
        p = [int(t) for t in np.asarray(prompt).reshape(-1)]
        best = None
        for k, (sn, _) in self._entries.items():
            T = sn.T
            if T < len(p) and [int(t) for t in sn.tokens[0, :T]] == p[:T] and (best is None or T > self._entries[best][0].T):
                best = k
        if best is None:
            self.misses += 1
            return None
        self.hits += 1
        return self._entries.pop(best)[0]

    def clear(self):
        for sn, _ in self._entries.values():
            sn.close()
        self._entries.clear()


def generate_with_pool(gpt: "GPT", pool: KvCachePool, prompt, opts: DecodingOptions, stop_on_eos: bool = True):
    """One request of one sequence through the pool: prompt [S] -> generated ids [n] (n <= MaxTgtSentLength - S),
    the loop of GPT.RunForwardOnSingleDevice (GPT.cs:212-335) with UseKVCache: a parked cache that covers a head of
    the prompt is restored and only the rest of the prompt is run; the cache is parked again afterwards."""
    p = np.asarray(prompt, dtype=np.int32).reshape(-1)
    n_new = opts.MaxTgtSentLength - len(p)
    if n_new <= 0:
        return np.zeros(0, dtype=np.int32)
    gpt.Reset()
    snap = pool.take(p)
    if snap is not None:
        gpt.CacheRestore(snap)
        first = gpt.Extend(p[None, snap.T:], opts)
        snap.close()
    else:
        first = gpt.Prefill(p[None, :], opts)
    out = first[:, None]
    if n_new > 1 and not (stop_on_eos and int(first[0]) == 0):
        out = np.concatenate([out, gpt.Decode(n_new - 1, opts, stop_on_eos=stop_on_eos)], axis=1)
    pool.put(gpt.CacheSnapshot())
    return out[0]
