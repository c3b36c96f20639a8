"""Seeded synthetic weights and prompts (host twin of csrc/synthetic.cu — bit-identical values).

    base     = splitmix64(seed ^ fnv1a64(name))
    a, b     = splitmix64(base + 2i), splitmix64(base + 2i + 1)
    S        = sum of the eight 16-bit fields of a and b
    value(i) = float32((S - 262140) * (float64(float32(std)) / 53509.91992145008))

The distribution is Irwin-Hall(8) scaled to N(0, std) (excess kurtosis -0.15, support +-4.9 sigma); it stands in
for the "seeded N(0, 0.02)" weights of the benchmark configurations and is exactly reproducible on any platform
because only integer arithmetic and one correctly rounded multiply are involved.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)
SIGMA = 53509.91992145008
MEAN = 262140


def fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for ch in name.encode("utf-8"):
        h ^= ch
        h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def splitmix64(x):
    """Vectorised splitmix64 step on uint64 arrays (wrap-around arithmetic)."""
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)).astype(np.uint64)
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)).astype(np.uint64)
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)).astype(np.uint64)
        return z ^ (z >> np.uint64(31))


def synth(name: str, shape, seed: int, std: float = 0.02, dtype=np.float32, offset: int = 0):
    """Values [offset, offset + prod(shape)) of tensor `name`."""
    n = int(np.prod(shape))
    base = splitmix64(np.array([(seed ^ fnv1a64(name)) & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))[0]
    out = np.empty(n, dtype=np.float32)
    scale = np.float64(np.float32(std)) / np.float64(SIGMA)
    step = 1 << 22
    with np.errstate(over="ignore"):
        for s0 in range(0, n, step):
            i = np.arange(s0 + offset, min(n, s0 + step) + offset, dtype=np.uint64)
            a = splitmix64(base + np.uint64(2) * i)
            b = splitmix64(base + np.uint64(2) * i + np.uint64(1))
            s = np.zeros(i.shape, dtype=np.int64)
            for k in range(4):
                sh = np.uint64(16 * k)
                s += ((a >> sh) & np.uint64(0xFFFF)).astype(np.int64)
                s += ((b >> sh) & np.uint64(0xFFFF)).astype(np.int64)
            out[s0:s0 + i.shape[0]] = ((s - MEAN).astype(np.float64) * scale).astype(np.float32)
    out = out.reshape(shape)
    if np.dtype(dtype) == np.float16:
        return out.astype(np.float16)
    return out


def prompt_ids(seed: int, batch: int, length: int, vocab: int, first_id: int = 1):
    """ids uniform in [first_id, vocab) keyed by (seed, sequence, position); id 0 is EOS in the reference
    (Seq2SeqSharp/Utils/Vocab.cs:23-30) and is kept out of prompts."""
    b = np.arange(batch, dtype=np.uint64)[:, None]
    p = np.arange(length, dtype=np.uint64)[None, :]
    with np.errstate(over="ignore"):
        key = splitmix64(np.array([seed & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))[0]
        x = splitmix64(key + (b << np.uint64(32)) + p)
    return (first_id + (x % np.uint64(vocab - first_id))).astype(np.int32)
