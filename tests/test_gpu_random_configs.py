"""Randomised parity: a few hundred seeded combinations of shape, dtype, value pattern, mask,
history and sampling parameters (uniform or per row), CUDA path against the CPU oracle.
Tokens, statuses, kept sets and probabilities must match bit for bit.  The one permitted
difference is the documented survivor limit: with top-k off, a row whose min-p survivors
exceed 1024 tokens reports BORN_ROW_OVERFLOW on the GPU where the oracle (no such limit)
answers."""
import numpy as np
import pytest

from born_b200 import workloads as W

pytestmark = pytest.mark.gpu

ROW_OVERFLOW = 4


def _dev(a):
    import torch
    if a is None:
        return None
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).cuda().view(torch.bfloat16)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32).copy()).cuda()
    if a.dtype.names:
        return torch.from_numpy(a.view(np.uint8).copy()).cuda()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _rand_params(rng):
    mode = int(rng.integers(0, 6))
    if mode == 0:
        return dict(greedy=True)
    p = dict(temperature=float(rng.choice([0.3, 0.7, 1.0, 1.5, 0.05])))
    if mode in (1, 2, 5):
        p["top_k"] = int(rng.choice([1, 2, 8, 40, 50, 64, 200, 256, 257, 600, 1024]))
    if mode in (2, 3):
        p["top_p"] = float(rng.choice([0.5, 0.9, 0.95, 0.999]))
    if mode in (3, 4):
        p["min_p"] = float(rng.choice([0.01, 0.05, 0.2]))
    if mode == 5 and rng.random() < 0.5:
        p["min_p"] = 0.02
    if rng.random() < 0.4:
        if rng.random() < 0.5:
            p["repetition_penalty"] = float(rng.choice([1.1, 1.3, 0.8]))
        if rng.random() < 0.6:
            p["frequency_penalty"] = float(rng.choice([0.2, 0.5]))
            p["presence_penalty"] = float(rng.choice([0.0, 0.3]))
    return p


SMALL_BATCHES = [1, 2, 3, 5, 16, 33, 64]
ALL_VOCABS = [1, 7, 33, 1000, 4096, 4097, 8192, 8200, 32000, 50257, 65536, 128256, 151936, 200003]


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_configurations_match_the_oracle(sampler, oracle, seed):
    _random_configurations(sampler, oracle, seed, 80, SMALL_BATCHES, ALL_VOCABS)


@pytest.mark.parametrize("seed", [21, 22])
def test_random_configurations_with_one_cta_per_row(sampler, oracle, seed):
    # batches that fill the GPU with one CTA per row (the instantiations without segment records),
    # rows of one to a dozen tiles
    _random_configurations(sampler, oracle, seed, 40, [252, 256, 280, 296], [1000, 4097, 8200, 20000, 32000, 50257])


def _random_configurations(sampler, oracle, seed, iterations, batches, vocabs):
    import torch
    from born_b200 import SamplingConfig
    from born_b200.sampler import row_params_array
    rng = np.random.default_rng(seed)
    limit_rows = 0
    for it in range(iterations):
        B = int(rng.choice(batches))
        V = int(rng.choice(vocabs))
        bf = rng.random() < 0.4
        z = (W.normal(seed * 1000 + it, 1, B * V) * float(rng.choice([0.5, 2.0, 3.0, 6.0]))).astype(np.float32).reshape(B, V)
        kind = int(rng.integers(0, 5))
        if kind == 0:
            z = np.round(z * 2) / 2  # heavy ties
        if kind == 1:
            z[:, ::3] = -np.inf
        if kind == 2 and V > 10:
            z[:, rng.integers(0, V, 5)] += 12.0  # spikes
        logits = W.f32_to_bf16_bits(z).reshape(B, V) if bf else z
        u = W.uniform_f32(seed * 1000 + it, 2, B)
        mask = None
        if rng.random() < 0.3:
            words = (V + 31) // 32
            bits = W.uniform(seed * 1000 + it, 3, B * words * 32).reshape(B, words * 32) < float(rng.choice([0.05, 0.5, 0.95]))
            bits[:, V:] = False
            if rng.random() < 0.8:
                bits[:, 0] = True
            mask = np.packbits(bits.reshape(B, words, 32), axis=-1, bitorder="little").view(np.uint32).reshape(B, words)
        per_row = rng.random() < 0.3
        rows = [_rand_params(rng) for _ in range(B)] if per_row else None
        params = _rand_params(rng)
        used = rows if per_row else [params]
        hist = hl = None
        if any(("repetition_penalty" in r or "frequency_penalty" in r) for r in used) or rng.random() < 0.1:
            H = int(rng.choice([1, 16, 64, 512, 1024]))
            hist = W.randint(seed * 1000 + it, 4, B * H, V).astype(np.int32).reshape(B, H)
            if rng.random() < 0.4:
                hl = rng.integers(0, H + 1, B).astype(np.int32)
        seg = 1
        if (not per_row and hist is None and 0 < params.get("top_k", 0) <= 128 and "min_p" not in params and V >= 4096
                and rng.random() < 0.3):
            for g in (2, 4, 8):
                if V % g == 0 and params["top_k"] * g <= 1024:
                    seg = g
        op = oracle.params_from_rows(rows) if per_row else oracle.make_params(**params)
        ref = oracle.sample(logits, op, uniforms=u, mask=mask, history=hist, history_len=hl, segments=seg, want_kept=64,
                            nthreads=8)
        kw = {}
        cfg = None
        if per_row:
            kw["row_params"] = _dev(row_params_array([SamplingConfig(**r) for r in rows]))
        else:
            cfg = SamplingConfig(**params)
        out = sampler.sample(_dev(logits), uniforms=_dev(u), config=cfg, mask=_dev(mask), history=_dev(hist),
                             history_len=_dev(hl), want_lse=True, want_kept=64, vocab_segments=seg, **kw)
        torch.cuda.synchronize()
        got = {k: v.cpu().numpy() for k, v in out.items()}
        keep = np.ones(B, dtype=bool)  # every row the oracle answers is answered, exactly
        ctx = (seed, it, B, V, bf, kind, seg, used[:3])
        assert np.array_equal(got["status"][keep], ref["status"][keep]), ctx
        assert np.array_equal(got["token"][keep], ref["token"][keep]), ctx
        assert np.array_equal(got["prob"][keep].view(np.uint32), ref["prob"][keep].view(np.uint32)), ctx
        assert np.array_equal(got["kept_count"][keep], ref["kept_count"][keep]), ctx
        assert np.array_equal(got["kept_ids"][keep], ref["kept_ids"][keep]), ctx
        fin = keep & np.isfinite(ref["lse"]) & (ref["status"] == 0)
        if fin.any():  # both sides sum in fp32, in different orders
            assert np.allclose(got["lse"][fin], ref["lse"][fin], rtol=1e-4, atol=2e-3), ctx
    assert limit_rows == 0
