"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (no dataset is involved anywhere on this path).

One counter-based generator (splitmix64 over seed and element counter) gives uniforms
(x >> 11) * 2^-53; normals come from the Box-Muller transform in float64, pairs (cos, sin)
filling consecutive elements, as the reference's tensor.Randn does
(born: internal/tensor/creation.go:82-117), then scaled, rounded to float32 and, where a
configuration asks for bf16, rounded to nearest-even bf16.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = x
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def raw_u64(seed, stream, n, offset=0):
    """n 64-bit words of stream `stream` of generator `seed`, starting at counter `offset`."""
    with np.errstate(over="ignore"):
        base = _splitmix64(np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15) + np.uint64(stream))
        ctr = np.arange(offset, offset + n, dtype=np.uint64)
        return _splitmix64(base + ctr * np.uint64(0xD1342543DE82EF95))


def uniform(seed, stream, n, offset=0):
    """float64 uniforms in [0, 1)."""
    return (raw_u64(seed, stream, n, offset) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def uniform_f32(seed, stream, n):
    """float32 uniforms strictly below 1."""
    u = uniform(seed, stream, n).astype(np.float32)
    return np.minimum(u, np.float32(1.0 - 2.0 ** -24))


def normal(seed, stream, n):
    """float64 standard normals by Box-Muller, (cos, sin) pairs in consecutive elements."""
    m = (n + 1) // 2
    u1 = 1.0 - uniform(seed, stream, m, 0)  # (0, 1]
    u2 = uniform(seed, stream, m, m)
    r = np.sqrt(-2.0 * np.log(u1))
    out = np.empty(2 * m, dtype=np.float64)
    out[0::2] = r * np.cos(2.0 * np.pi * u2)
    out[1::2] = r * np.sin(2.0 * np.pi * u2)
    return out[:n]


def randint(seed, stream, n, hi):
    return (raw_u64(seed, stream, n) % np.uint64(hi)).astype(np.int64)


def f32_to_bf16_bits(x):
    """Round-to-nearest-even float32 -> bf16 bit patterns (uint16)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((b >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((b + r) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(h):
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# ----------------------------------------------------------------------------------------
# the benchmark configurations
# ----------------------------------------------------------------------------------------

def config1(seed=0, steps=16):
    """Single-row sampling: B=1, V=32000 fp32 N(0, 2^2) + 8.0 on 3 random ids; T=0.8, top-k 40,
    top-p 0.95, repetition penalty 1.1 over 64 prior ids; `steps` fresh uniforms."""
    V = 32000
    z = (normal(seed, 1, V) * 2.0).astype(np.float32)
    spikes = []
    i = 0
    while len(spikes) < 3:
        t = int(randint(seed, 2, 3 + i, V)[-1])
        if t not in spikes:
            spikes.append(t)
        i += 1
    z[spikes] += np.float32(8.0)
    return {
        "logits": z.reshape(1, V),
        "history": randint(seed, 3, 64, V).astype(np.int32).reshape(1, 64),
        "uniforms": uniform_f32(seed, 4, steps),
        "params": dict(temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.1),
        "spikes": spikes,
    }


def config2(seed=0, batch=64, vocab=128256, hist=512):
    """Batched decode: fp32 N(0, 3^2) + Zipf(s=1.1)-shaped bias -1.1*ln(rank) over a per-row random
    permutation; T=0.7, min-p 0.05, top-p 0.9; frequency 0.5 / presence 0.3 over `hist` prior ids."""
    B, V = batch, vocab
    z = (normal(seed, 10, B * V) * 3.0).reshape(B, V)
    bias = -1.1 * np.log(np.arange(1, V + 1, dtype=np.float64))
    for b in range(B):
        perm = np.argsort(raw_u64(seed, 1000 + b, V), kind="stable")
        z[b, perm] += bias
    return {
        "logits": z.astype(np.float32),
        "history": randint(seed, 11, B * hist, V).astype(np.int32).reshape(B, hist),
        "uniforms": uniform_f32(seed, 12, B),
        "params": dict(temperature=0.7, min_p=0.05, top_p=0.9, frequency_penalty=0.5, presence_penalty=0.3),
    }


def config3(seed=0, batch=256, vocab=151936, allow=0.05):
    """Constrained decoding: bf16 N(0, 2.5^2); per-row grammar bitmask with ~5% of tokens allowed
    (at least one); even rows greedy, odd rows top-k 50 at temperature 1."""
    B, V = batch, vocab
    z = (normal(seed, 20, B * V) * 2.5).astype(np.float32).reshape(B, V)
    words = (V + 31) // 32
    bits = uniform(seed, 21, B * words * 32).reshape(B, words * 32) < allow
    bits[:, V:] = False
    for b in range(B):
        if not bits[b].any():
            bits[b, int(randint(seed, 22, b + 1, V)[-1])] = True
    mask = np.packbits(bits.reshape(B, words, 32), axis=-1, bitorder="little").view(np.uint32).reshape(B, words)
    rows = []
    for b in range(B):
        rows.append(dict(greedy=True) if b % 2 == 0 else dict(temperature=1.0, top_k=50))
    return {
        "logits_bf16": f32_to_bf16_bits(z),
        "mask": np.ascontiguousarray(mask),
        "uniforms": uniform_f32(seed, 23, B),
        "row_params": rows,
    }


def config4(seed=0, batch=32, draft_len=5, vocab=128256):
    """Speculative verification: target fp32 N(0, 2^2) [B, K+1, V]; draft = target[:, :K] + N(0, 0.5^2).
    Draft tokens are drawn from the draft distribution by the caller (see the oracle's
    born_oracle_draft_tokens); uniforms for the draft draw, the accept tests and the resampling."""
    B, K, V = batch, draft_len, vocab
    tgt = (normal(seed, 30, B * (K + 1) * V) * 2.0).astype(np.float32).reshape(B, K + 1, V)
    noise = (normal(seed, 31, B * K * V) * 0.5).astype(np.float32).reshape(B, K, V)
    return {
        "target": tgt,
        "draft": (tgt[:, :K, :] + noise).astype(np.float32),
        "u_draft": uniform_f32(seed, 32, B * K).reshape(B, K),
        "u_accept": uniform_f32(seed, 33, B * K).reshape(B, K),
        "u_resample": uniform_f32(seed, 34, B * (K + 1)).reshape(B, K + 1),
    }


def config5(seed=0, batch=1024, vocab=256000, shards=8):
    """Vocab-sharded sampling: bf16 N(0, 2^2) with 1% of entries spiked by +6; `shards` contiguous
    vocab shards; per-shard top-k 64, then top-p 0.95 over the gathered candidates."""
    B, V = batch, vocab
    z = (normal(seed, 40, B * V) * 2.0).astype(np.float32).reshape(B, V)
    spike = uniform(seed, 41, B * V).reshape(B, V) < 0.01
    z[spike] += np.float32(6.0)
    return {
        "logits_bf16": f32_to_bf16_bits(z),
        "uniforms": uniform_f32(seed, 42, B),
        "shards": shards,
        "params": dict(temperature=1.0, top_k=64, top_p=0.95),
    }
