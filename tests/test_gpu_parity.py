"""Parity of the CUDA path (through the C ABI) with the CPU oracle on identical seeded
inputs: token ids, kept sets and statuses bit-exact, kept-set probabilities bit-exact,
log-sum-exp within 1e-5 relative of a float64 evaluation."""
import os

import numpy as np
import pytest

from born_b200 import workloads as W

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def torch_mod():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch


def to_dev(a, bf16=False):
    torch = torch_mod()
    if a is None:
        return None
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).cuda().view(torch.bfloat16)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32).copy()).cuda()
    if a.dtype.names:  # structured row params
        return torch.from_numpy(a.view(np.uint8).copy()).cuda()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def lse_f64(oracle_like_logits, params_row, mask_row=None, hist_row=None):
    from tests import np_sampler as NP
    z = NP.prepare(oracle_like_logits, params_row, mask_row, hist_row).astype(np.float64)
    greedy = params_row.get("greedy") or params_row.get("temperature", 0.0) == 0.0
    inv_T = 1.0 if greedy else 1.0 / float(np.float32(params_row["temperature"]))
    m = z.max()
    return m * inv_T + np.log(np.exp((z - m) * inv_T).sum())


def run_both(sampler, oracle, logits, params, u, mask=None, hist=None, hist_len=None, segments=1, want_kept=64,
             per_row=None, host=False):
    """Runs the oracle and the GPU on the same inputs; returns (gpu dict of numpy, oracle dict)."""
    from born_b200 import SamplingConfig
    from born_b200.sampler import row_params_array
    if per_row is not None:
        op = oracle.params_from_rows(per_row)
    else:
        op = oracle.make_params(**params)
    ref = oracle.sample(logits, op, uniforms=u, mask=mask, history=hist, history_len=hist_len, segments=segments,
                        want_kept=want_kept, nthreads=8)
    kw = {}
    if per_row is not None:
        rp = row_params_array([SamplingConfig(**r) for r in per_row])
        kw["row_params"] = rp if host else to_dev(rp)
        cfg = None
    else:
        cfg = SamplingConfig(**params)
    if host:
        out = sampler.sample(logits, uniforms=u, config=cfg, mask=mask, history=hist, history_len=hist_len,
                             want_lse=True, want_kept=want_kept, vocab_segments=segments, **kw)
        got = out
    else:
        torch = torch_mod()
        out = sampler.sample(to_dev(logits), uniforms=to_dev(u), config=cfg, mask=to_dev(mask), history=to_dev(hist),
                             history_len=to_dev(hist_len), want_lse=True, want_kept=want_kept,
                             vocab_segments=segments, **kw)
        torch.cuda.synchronize()
        got = {k: v.cpu().numpy() for k, v in out.items()}
    return got, ref


def assert_parity(got, ref, check_kept=True):
    assert np.array_equal(got["status"], ref["status"]), (got["status"], ref["status"])
    bad = np.nonzero(got["token"] != ref["token"])[0]
    assert bad.size == 0, f"token mismatch rows {bad[:8]}: gpu {got['token'][bad[:8]]} oracle {ref['token'][bad[:8]]}"
    assert np.array_equal(got["prob"].view(np.uint32), ref["prob"].view(np.uint32))
    if check_kept and "kept_count" in got:
        assert np.array_equal(got["kept_count"], ref["kept_count"])
        assert np.array_equal(got["kept_ids"], ref["kept_ids"])


# ------------------------------------------------------------------------------ arithmetic
def test_exp_and_mass_bit_exact(sampler, oracle, lib):
    torch = torch_mod()
    n = 1 << 22
    x = np.concatenate([
        -np.abs(W.normal(1, 1, n) * 12.0),
        np.linspace(-90.0, 0.0, n // 4),
        -np.logspace(-9, 1.95, n // 4),
        np.array([0.0, -0.0, -80.0, -80.00001, -1e30, -np.inf, np.nan]),
    ]).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    yd = torch.empty_like(xd)
    qd = torch.empty(x.size, dtype=torch.int64, device="cuda")
    assert lib.born_debug_exp(xd.data_ptr(), yd.data_ptr(), x.size, None) == 0
    assert lib.born_debug_mass(xd.data_ptr(), qd.data_ptr(), x.size, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(yd.cpu().numpy().view(np.uint32), oracle.exp_det(x).view(np.uint32))
    assert np.array_equal(qd.cpu().numpy().view(np.uint64), oracle.mass(x))


def test_committed_fixtures(sampler, oracle):
    g = np.load(os.path.join(GOLD, "sampler_small.npz"))
    for i in range(int(g["n_cases"])):
        rec = g[f"c{i}_params"][0]
        params = {k: rec[k].item() for k in rec.dtype.names if k != "flags"}
        params["greedy"] = bool(rec["flags"] & 1)
        got, _ = run_both(sampler, oracle, g[f"c{i}_logits"], params, g[f"c{i}_uniforms"],
                          mask=g[f"c{i}_mask"] if f"c{i}_mask" in g else None,
                          hist=g[f"c{i}_history"] if f"c{i}_history" in g else None,
                          segments=int(g[f"c{i}_segments"]))
        ref = {k: g[f"c{i}_out_{k}"] for k in ("token", "prob", "status", "kept_ids", "kept_count")}
        assert_parity(got, ref)


# ------------------------------------------------------------------------------ sampling
PARAM_SETS = [
    dict(temperature=1.0, top_k=50),
    dict(temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.1),
    dict(temperature=0.7, min_p=0.05, top_p=0.9, frequency_penalty=0.5, presence_penalty=0.3),
    dict(greedy=True),
    dict(temperature=1.0, top_k=1),
    dict(temperature=1.5, top_k=1024, top_p=0.99),
    dict(temperature=0.3, top_k=7, min_p=0.3),
]


@pytest.mark.parametrize("V", [1, 2, 31, 32, 33, 127, 4095, 4096, 4097, 8193, 32000, 50001])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_shapes_and_ragged_edges(sampler, oracle, V, dtype):
    B = 5
    for pi, p in enumerate(PARAM_SETS):
        seed = 31 * V + pi
        z = (W.normal(seed, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)
        logits = z if dtype == "f32" else W.f32_to_bf16_bits(z)
        u = W.uniform_f32(seed, 2, B)
        hist = W.randint(seed, 3, B * 48, V).astype(np.int32).reshape(B, 48)
        hist[:, -3:] = [-1, V, V + 7]  # ignored ids
        got, ref = run_both(sampler, oracle, logits, p, u, hist=hist, want_kept=min(64, max(1, V)))
        assert_parity(got, ref)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_mask_and_per_row_params(sampler, oracle, dtype):
    B, V = 12, 20000
    z = (W.normal(9, 1, B * V) * 2.5).astype(np.float32).reshape(B, V)
    logits = z if dtype == "f32" else W.f32_to_bf16_bits(z)
    words = (V + 31) // 32
    bits = W.uniform(9, 2, B * words * 32).reshape(B, words * 32) < 0.05
    bits[:, V:] = False
    bits[:, 17] = True
    mask = np.packbits(bits.reshape(B, words, 32), axis=-1, bitorder="little").view(np.uint32).reshape(B, words)
    rows = [dict(greedy=True) if b % 2 == 0 else dict(temperature=1.0, top_k=50) for b in range(B)]
    rows[3] = dict(temperature=0.7, min_p=0.1, top_p=0.9)
    rows[5] = dict(temperature=0.0)
    u = W.uniform_f32(9, 3, B)
    got, ref = run_both(sampler, oracle, logits, None, u, mask=mask, per_row=rows)
    assert_parity(got, ref)
    allowed = np.unpackbits(mask.view(np.uint8), bitorder="little").reshape(B, -1)[:, :V].astype(bool)
    for b in range(B):
        assert allowed[b, got["token"][b]]
        n = got["kept_count"][b]
        assert allowed[b, got["kept_ids"][b][:n]].all()


def test_ties_are_broken_by_index(sampler, oracle):
    # bf16-like heavy ties at the top-k boundary, constant rows, two-valued rows
    B, V = 6, 9000
    rng = np.random.default_rng(3)
    z = rng.integers(-4, 5, size=(B, V)).astype(np.float32)
    z[1] = 1.25
    z[2] = np.where(np.arange(V) % 2 == 0, 2.0, -2.0)
    z[3, :] = -0.0
    z[3, 100:200] = 0.0
    u = W.uniform_f32(3, 1, B)
    for p in (dict(temperature=1.0, top_k=10), dict(temperature=1.0, top_k=600, top_p=0.9), dict(greedy=True),
              dict(temperature=2.0, top_k=1000)):
        got, ref = run_both(sampler, oracle, z, p, u, want_kept=1024)
        assert_parity(got, ref)


def test_sorted_rows_exercise_buffer_overflow_path(sampler, oracle):
    # ascending rows make every element a new candidate: the fast pass must fall back to the
    # piecewise pass without losing or duplicating anything
    B, V = 3, 40000
    z = np.tile(np.arange(V, dtype=np.float32) * 1e-3, (B, 1))
    z[1] = z[1][::-1]
    z[2] = np.sort((W.normal(4, 1, V) * 3).astype(np.float32))
    u = W.uniform_f32(4, 2, B)
    for p in (dict(temperature=1.0, top_k=64), dict(temperature=0.01, top_k=1024, top_p=0.9), dict(greedy=True)):
        got, ref = run_both(sampler, oracle, z, p, u, want_kept=1024)
        assert_parity(got, ref)


def test_small_batches_are_cut_into_slices_and_merged(sampler, oracle):
    # fewer rows than SMs: every row is streamed by several CTAs whose records the last one
    # merges -- filtered supersets, the slices' own top-k bounds, the min-p cut of the row maximum,
    # and (top-k 200: more merged entries than the all-pairs path takes) the cut to the k best
    B, V = 3, 128256
    z = (W.normal(21, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)
    z[1, ::7] = 2.5  # ties across slices
    u = W.uniform_f32(21, 2, B)
    hist = W.randint(21, 3, B * 96, V).astype(np.int32).reshape(B, 96)
    for p, h in ((dict(temperature=0.7, top_k=200, top_p=0.9), None),
                 (dict(temperature=0.7, top_k=40), None),
                 (dict(temperature=0.9, min_p=0.02, top_p=0.95, frequency_penalty=0.4, presence_penalty=0.2), hist),
                 (dict(temperature=1.0, top_k=8, repetition_penalty=1.3), hist),
                 (dict(greedy=True), None)):
        got, ref = run_both(sampler, oracle, z, p, u, hist=h, want_kept=256)
        assert_parity(got, ref)
    zb = W.f32_to_bf16_bits((W.normal(22, 1, 2 * 151936) * 2.5).astype(np.float32)).reshape(2, 151936)
    ub = W.uniform_f32(22, 2, 2)
    for p in (dict(temperature=1.0, top_k=64, top_p=0.9), dict(temperature=0.8, min_p=0.05)):
        got, ref = run_both(sampler, oracle, zb, p, ub, want_kept=128)
        assert_parity(got, ref)


def test_invalid_rows_report_status(sampler, oracle):
    B, V = 6, 5000
    z = (W.normal(5, 1, B * V)).astype(np.float32).reshape(B, V)
    z[1, 4321] = np.nan
    z[2, 77] = np.inf
    z[4, :] = -np.inf
    words = (V + 31) // 32
    mask = np.full((B, words), 0xFFFFFFFF, dtype=np.uint32)
    mask[0] = 0
    mask[3] = 0
    mask[3, 5] = 1 << 9  # only token 169
    mask[5, 4321 >> 5] &= ~np.uint32(1 << (4321 & 31))
    z[5, 4321] = np.nan  # masked NaN: row stays valid
    u = W.uniform_f32(5, 2, B)
    got, ref = run_both(sampler, oracle, z, dict(temperature=1.0, top_k=20), u, mask=mask)
    assert list(ref["status"]) == [1, 2, 3, 0, 1, 0]
    assert_parity(got, ref)
    assert got["token"][3] == 169 and list(got["token"][[0, 1, 2, 4]]) == [-1] * 4


def test_rows_beyond_the_candidate_limit_are_exact(sampler, oracle):
    # top-k off: whatever the number of min-p survivors or the size of the nucleus, the row is
    # answered exactly (the kernel falls to its multi-pass search over the row); nothing reports
    # BORN_ROW_OVERFLOW
    B, V = 4, 30000
    z = (W.normal(6, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)
    u = W.uniform_f32(6, 2, B)
    got, ref = run_both(sampler, oracle, z, dict(temperature=0.7, min_p=0.05, top_p=0.9), u, want_kept=1024)
    assert_parity(got, ref)
    flat = np.zeros((2, V), dtype=np.float32)  # an all-zeros row: the nucleus is 90 % of the vocabulary
    for p in (dict(temperature=1.0, top_p=0.9), dict(temperature=1.0, min_p=0.5), dict(temperature=2.0, min_p=1e-4, top_p=0.5),
              dict(temperature=1.0, top_k=1000), dict(temperature=1.0)):
        got, ref = run_both(sampler, oracle, flat, p, u[:2], want_kept=64)
        assert_parity(got, ref)
    n0 = sampler.fallback_rows
    for T in (1.2, 1.6, 2.0):  # flat distributions: thousands of min-p survivors / nucleus tokens
        for p in (dict(temperature=T, top_p=0.9), dict(temperature=T, min_p=0.001), dict(temperature=T, min_p=0.002, top_p=0.95)):
            got, ref = run_both(sampler, oracle, z, p, u, want_kept=1024)
            assert (ref["kept_count"] > 1024).any(), (T, p)
            assert_parity(got, ref)
    assert sampler.fallback_rows > 0  # these rows did take the exact search
    small = (W.normal(6, 3, 2 * 900) * 2).astype(np.float32).reshape(2, 900)
    for p in (dict(temperature=1.0), dict(temperature=1.0, top_p=0.7)):
        got, ref = run_both(sampler, oracle, small, p, u[:2], want_kept=1024)
        assert_parity(got, ref)
    assert n0 >= 0


def test_lse_within_tolerance_of_float64(sampler, oracle):
    B, V = 8, 128256
    z = (W.normal(7, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)
    u = W.uniform_f32(7, 2, B)
    p = dict(temperature=0.7, top_k=50)
    got, ref = run_both(sampler, oracle, z, p, u)
    assert_parity(got, ref)
    for b in range(B):
        truth = lse_f64(z[b], p)
        # 1e-5 relative on sum(exp) is 1e-5 absolute on its logarithm
        assert abs(got["lse"][b] - truth) <= 1e-5 + 1e-6 * abs(truth), (b, got["lse"][b], truth)


def test_host_memory_call_equals_device_call(sampler, oracle):
    B, V = 7, 33333
    z = (W.normal(8, 1, B * V) * 2.0).astype(np.float32).reshape(B, V)
    u = W.uniform_f32(8, 2, B)
    hist = W.randint(8, 3, B * 100, V).astype(np.int32).reshape(B, 100)
    hl = np.array([100, 0, 5, 99, 100, 1, 50], dtype=np.int32)
    p = dict(temperature=0.9, top_k=30, top_p=0.9, repetition_penalty=1.2, presence_penalty=0.1)
    got_h, ref = run_both(sampler, oracle, z, p, u, hist=hist, hist_len=hl, host=True)
    got_d, _ = run_both(sampler, oracle, z, p, u, hist=hist, hist_len=hl, host=False)
    assert_parity(got_h, ref)
    assert_parity(got_d, ref)
    t = sampler.last_timing_ms()
    assert t["kernel"] > 0 and t["h2d"] > 0


def test_misaligned_rows_take_the_plain_load_path(sampler, oracle):
    torch = torch_mod()
    B, V = 4, 10001  # odd vocab: rows are not 16-byte aligned
    z = (W.normal(11, 1, B * V) * 2.0).astype(np.float32).reshape(B, V)
    u = W.uniform_f32(11, 2, B)
    got, ref = run_both(sampler, oracle, z, dict(temperature=1.0, top_k=25, top_p=0.9), u)
    assert_parity(got, ref)
    zb = W.f32_to_bf16_bits(z)
    got, ref = run_both(sampler, oracle, zb, dict(temperature=1.0, top_k=25), u)
    assert_parity(got, ref)
    # strided rows (row stride > vocab)
    from born_b200 import SamplingConfig
    big = torch.zeros((B, V + 7), dtype=torch.float32, device="cuda")
    big[:, :V] = torch.from_numpy(z).cuda()
    out = sampler.sample(big[:, :V], uniforms=to_dev(u), config=SamplingConfig(temperature=1.0, top_k=25, top_p=0.9))
    torch.cuda.synchronize()
    ref2 = oracle.sample(z, oracle.make_params(temperature=1.0, top_k=25, top_p=0.9), uniforms=u)
    assert np.array_equal(out["token"].cpu().numpy(), ref2["token"])


# ------------------------------------------------------------------------------ configurations
def test_config1_single_row(sampler, oracle):
    c = W.config1(seed=0, steps=64)
    logits = np.repeat(c["logits"], 64, axis=0)
    hist = np.repeat(c["history"], 64, axis=0)
    got, ref = run_both(sampler, oracle, logits, c["params"], c["uniforms"], hist=hist)
    assert_parity(got, ref)
    # one row at a time, as the reference-runnable configuration does
    from born_b200 import SamplingConfig
    torch = torch_mod()
    ld, hd = to_dev(c["logits"]), to_dev(c["history"])
    for s in range(8):
        out = sampler.sample(ld, uniforms=to_dev(c["uniforms"][s:s + 1]), config=SamplingConfig(**c["params"]), history=hd)
        torch.cuda.synchronize()
        assert int(out["token"][0]) == int(ref["token"][s])


def test_config2_batched_decode_full_size(sampler, oracle):
    c = W.config2(seed=0, batch=64)
    got, ref = run_both(sampler, oracle, c["logits"], c["params"], c["uniforms"], hist=c["history"], want_kept=256)
    assert_parity(got, ref)
    assert (ref["status"] == 0).all()
    print("config2 near-cutoff rows:", int((ref["near_cutoff"] != 0).sum()))


def test_config3_constrained_full_size(sampler, oracle):
    c = W.config3(seed=0, batch=256)
    got, ref = run_both(sampler, oracle, c["logits_bf16"], None, c["uniforms"], mask=c["mask"], per_row=c["row_params"])
    assert_parity(got, ref)
    # the greedy rows are the reference's argmax over the masked row
    z = W.bf16_bits_to_f32(c["logits_bf16"][:4])
    allowed = np.unpackbits(c["mask"][:4].view(np.uint8), bitorder="little").reshape(4, -1)[:, :z.shape[1]].astype(bool)
    zm = np.where(allowed, z, -np.inf).astype(np.float32)
    for b in (0, 2):
        assert got["token"][b] == oracle.ref_argmax(zm[b])


def test_config5_single_gpu_segmented(sampler, oracle):
    c = W.config5(seed=0, batch=64)
    got, ref = run_both(sampler, oracle, c["logits_bf16"], c["params"], c["uniforms"], segments=c["shards"],
                        want_kept=512)
    assert_parity(got, ref)


@pytest.mark.parametrize("k", [64, 5, 1])
def test_shard_local_and_merge_equal_segmented_sampling(sampler, oracle, k):
    """The vocab-sharded pipeline on one GPU: G local passes, records concatenated the way an
    all-gather lays them out, one merge.  Must equal the oracle's segmented sampling.  An odd k
    makes every second record start off a 16-byte boundary."""
    torch = torch_mod()
    c = W.config5(seed=1, batch=48, vocab=64000, shards=8)
    G, B = 8, 48
    Vl = 64000 // G
    ld = to_dev(c["logits_bf16"])
    params = dict(c["params"], top_k=k)
    gathered = torch.empty((G, B, sampler.record_bytes(k)), dtype=torch.uint8, device="cuda")
    for g in range(G):
        shard = ld[:, g * Vl:(g + 1) * Vl].contiguous()
        sampler.shard_local(shard, g, G, k, temperature=1.0, top_p=0.95, packed=gathered[g])
    out = sampler.shard_merge(gathered, to_dev(c["uniforms"]), Vl, 0, G, k, temperature=1.0, top_p=0.95)
    torch.cuda.synchronize()
    ref = oracle.sample(c["logits_bf16"], oracle.make_params(**params), uniforms=c["uniforms"], segments=G)
    assert np.array_equal(out["status"].cpu().numpy(), ref["status"])
    assert np.array_equal(out["token"].cpu().numpy(), ref["token"])
    assert np.array_equal(out["prob"].cpu().numpy().view(np.uint32), ref["prob"].view(np.uint32))
    z = W.bf16_bits_to_f32(c["logits_bf16"]).astype(np.float64)
    truth = np.log(np.exp(z - z.max(1, keepdims=True)).sum(1)) + z.max(1)
    assert np.max(np.abs(out["lse"].cpu().numpy() - truth)) <= 2e-5


# ------------------------------------------------------------------------------ size-independent properties
def test_full_size_properties_headline_shape(sampler, oracle):
    """B=256 x V=128256 fp32: properties that need no oracle pass over the whole batch."""
    torch = torch_mod()
    from born_b200 import SamplingConfig
    B, V = 256, 128256
    g = torch.Generator(device="cuda").manual_seed(0)
    z = torch.randn((B, V), generator=g, device="cuda") * 3.0
    u = torch.rand(B, generator=g, device="cuda").clamp_(max=1 - 2 ** -24)
    cfg = SamplingConfig(temperature=0.7, top_k=50, top_p=0.9)
    a = sampler.sample(z, uniforms=u, config=cfg, want_lse=True, want_kept=64)
    b = sampler.sample(z, uniforms=u, config=cfg, want_lse=True, want_kept=64)
    torch.cuda.synchronize()
    assert torch.equal(a["token"], b["token"]) and torch.equal(a["prob"], b["prob"])  # run-to-run determinism
    assert (a["status"] == 0).all()
    # kept ids are the top of a full sort (value desc, index asc), in order
    n = a["kept_count"].cpu().numpy()
    srt = torch.sort(z, dim=1, descending=True, stable=True).indices[:, :64].cpu().numpy()
    kept = a["kept_ids"].cpu().numpy()
    for r in range(B):
        assert np.array_equal(kept[r, :n[r]], srt[r, :n[r]])
        assert a["token"][r].item() in kept[r, :n[r]]
    # shift invariance of the decision (softmax(x + c) = softmax(x)): exact for power-of-two-free shifts
    # is not guaranteed in fp32, so use the lse identity instead: lse(x + c) = lse(x) + c / T
    c = sampler.sample(z + 8.0, uniforms=u, config=cfg, want_lse=True)
    torch.cuda.synchronize()
    assert torch.allclose(c["lse"], a["lse"] + 8.0 / 0.7, rtol=0, atol=2e-4)
    # lse against torch float64
    ref = torch.logsumexp((z.double() / 0.7), dim=1)
    assert (a["lse"].double() - ref).abs().max().item() <= 2e-5
    # spot-check 8 rows against the oracle
    rows = [0, 1, 37, 100, 128, 200, 254, 255]
    zc = z[rows].cpu().numpy()
    r = oracle.sample(zc, oracle.make_params(temperature=0.7, top_k=50, top_p=0.9), uniforms=u[rows].cpu().numpy())
    assert np.array_equal(a["token"][rows].cpu().numpy(), r["token"])


# ------------------------------------------------------------------------------ speculative decoding
def test_spec_verify_fixture_and_config4(sampler, oracle):
    torch = torch_mod()
    g = np.load(os.path.join(GOLD, "sampler_small.npz"))
    out = sampler.spec_verify(to_dev(g["spec_target"]), to_dev(g["spec_draft"]), to_dev(g["spec_draft_tok"]),
                              to_dev(g["spec_u_accept"]), to_dev(g["spec_u_resample"]))
    torch.cuda.synchronize()
    assert np.array_equal(out["accept_len"].cpu().numpy(), g["spec_out_accept_len"])
    assert np.array_equal(out["tokens"].cpu().numpy(), g["spec_out_tokens"])
    assert np.array_equal(out["status"].cpu().numpy(), g["spec_out_status"])

    c = W.config4(seed=0, batch=32)
    dt = oracle.draft_tokens(c["draft"], c["u_draft"])
    ref = oracle.spec_verify(c["target"], c["draft"], dt, c["u_accept"], c["u_resample"], nthreads=8)
    out = sampler.spec_verify(to_dev(c["target"]), to_dev(c["draft"]), to_dev(dt), to_dev(c["u_accept"]),
                              to_dev(c["u_resample"]))
    torch.cuda.synchronize()
    assert np.array_equal(out["accept_len"].cpu().numpy(), ref["accept_len"])
    assert np.array_equal(out["tokens"].cpu().numpy(), ref["tokens"])
    assert np.array_equal(out["status"].cpu().numpy(), ref["status"])
    assert 0 < ref["accept_len"].mean() < 5  # both branches exercised
    # host-memory call
    outh = sampler.spec_verify(c["target"], c["draft"], dt, c["u_accept"], c["u_resample"])
    assert np.array_equal(outh["tokens"], ref["tokens"])


@pytest.mark.parametrize("V,K,rows", [(1000, 1, 2), (4097, 3, 3), (8192, 2, 3), (20001, 4, 5)])
def test_spec_verify_shapes_and_edges(sampler, oracle, V, K, rows):
    torch = torch_mod()
    B = 6
    tgt = (W.normal(V, 1, B * rows * V) * 2.0).astype(np.float32).reshape(B, rows, V)
    drf = (tgt[:, :K] + (W.normal(V, 2, B * K * V) * 0.7).astype(np.float32).reshape(B, K, V)).astype(np.float32)
    drf[1] = tgt[1, :K]          # identical distributions: always accepted
    tgt[2, 0, 5] = np.nan        # invalid target row
    dt = oracle.draft_tokens(drf, W.uniform_f32(V, 3, B * K).reshape(B, K))
    dt[3, 0] = V + 3             # bad draft token
    tgt[4, 0, dt[4, 0]] = -40.0  # certain rejection at position 0
    ua = W.uniform_f32(V, 4, B * K).reshape(B, K)
    ur = W.uniform_f32(V, 5, B * (K + 1)).reshape(B, K + 1)
    ref = oracle.spec_verify(tgt, drf, dt, ua, ur, temperature=0.9)
    out = sampler.spec_verify(to_dev(tgt), to_dev(drf), to_dev(dt), to_dev(ua), to_dev(ur), temperature=0.9)
    torch.cuda.synchronize()
    assert np.array_equal(out["status"].cpu().numpy(), ref["status"]), (out["status"], ref["status"])
    assert np.array_equal(out["accept_len"].cpu().numpy(), ref["accept_len"])
    assert np.array_equal(out["tokens"].cpu().numpy(), ref["tokens"])
    assert ref["accept_len"][1] == K and ref["status"][2] == 2 and ref["status"][3] == 5 and ref["accept_len"][4] == 0


# ------------------------------------------------------------------------------ errors
def test_argument_errors_are_raised_not_ignored(sampler):
    torch = torch_mod()
    from born_b200 import InvalidArgument, SamplerError, SamplingConfig
    z = torch.zeros((2, 100), device="cuda")
    u = torch.zeros(2, device="cuda")
    with pytest.raises(InvalidArgument):
        sampler.sample(z, uniforms=None, config=SamplingConfig(temperature=1.0))
    with pytest.raises(InvalidArgument):
        sampler.sample(z, uniforms=u, config=SamplingConfig(temperature=-1.0))
    with pytest.raises(InvalidArgument):
        sampler.sample(z, uniforms=u, config=SamplingConfig(temperature=1.0, top_k=5000))
    with pytest.raises(InvalidArgument):
        sampler.sample(z.double(), uniforms=u, config=SamplingConfig(temperature=1.0))
    with pytest.raises(InvalidArgument):
        sampler.sample(torch.zeros((4096, 100), device="cuda"), uniforms=u, config=SamplingConfig(greedy=True))
    with pytest.raises(SamplerError):
        sampler.sample(z, uniforms=u, config=SamplingConfig(temperature=1.0),
                       history=torch.zeros((2, 5000), dtype=torch.int32, device="cuda"))
    out = sampler.sample(z, config=SamplingConfig(greedy=True))  # greedy needs no uniforms
    torch.cuda.synchronize()
    assert out["token"].cpu().tolist() == [0, 0]


def test_whole_vocabulary_sampling(sampler, oracle):
    # no top-k and no top-p: temperature-only sampling, and min-p with more than 1024 survivors
    # when the caller asks for the two-pass path -- every token of the row can be drawn
    B, V = 9, 50257
    z = (W.normal(31, 1, B * V) * 1.5).astype(np.float32).reshape(B, V)
    z[2, ::5] = -np.inf
    z[3] = np.round(z[3])
    z[4, :] = -np.inf
    z[4, 77] = 0.5
    z[5, 1234] = np.nan
    z[6, :] = -np.inf
    u = W.uniform_f32(31, 2, B)
    u[7] = 0.0
    u[8] = np.float32(1.0 - 2.0 ** -24)
    words = (V + 31) // 32
    bits = W.uniform(31, 3, B * words * 32).reshape(B, words * 32) < 0.4
    bits[:, V:] = False
    bits[:, 5] = True
    mask = np.packbits(bits.reshape(B, words, 32), axis=-1, bitorder="little").view(np.uint32).reshape(B, words)
    for dtype in ("f32", "bf16"):
        logits = z if dtype == "f32" else W.f32_to_bf16_bits(z).reshape(B, V)
        for m in (None, mask):
            for p in (dict(temperature=1.0), dict(temperature=0.6), dict(temperature=1.5, min_p=0.01, full_vocab=True),
                      dict(temperature=2.0, top_p=1.0)):
                op = {k: v for k, v in p.items() if k != "full_vocab"}
                got, ref = run_both_full(sampler, oracle, logits, p, op, u, m)
                assert np.array_equal(got["status"], ref["status"]), (dtype, p, got["status"], ref["status"])
                assert np.array_equal(got["token"], ref["token"]), (dtype, p)
                assert np.array_equal(got["prob"].view(np.uint32), ref["prob"].view(np.uint32)), (dtype, p)
                assert np.array_equal(got["kept_count"], ref["kept_count"]), (dtype, p)
                ok = ref["status"] == 0
                assert np.allclose(got["lse"][ok], ref["lse"][ok], rtol=1e-4, atol=2e-3)
    # the host-memory call takes the same route
    from born_b200 import SamplingConfig
    hout = sampler.sample(z, uniforms=u, config=SamplingConfig(temperature=0.6), want_lse=True, want_kept_count=True)
    href = oracle.sample(z, oracle.make_params(temperature=0.6), uniforms=u, want_kept=8, nthreads=8)
    assert np.array_equal(hout["token"], href["token"]) and np.array_equal(hout["status"], href["status"])
    assert np.array_equal(hout["kept_count"], href["kept_count"])
    # odd sizes and rows that are not 16-byte aligned
    for V2 in (1, 3, 1025, 4097, 12345):
        z2 = (W.normal(32, V2, 3 * V2) * 2.0).astype(np.float32).reshape(3, V2)
        got, ref = run_both_full(sampler, oracle, z2, dict(temperature=0.9), dict(temperature=0.9), W.uniform_f32(32, 5, 3), None)
        assert np.array_equal(got["token"], ref["token"]) and np.array_equal(got["status"], ref["status"]), V2
        assert np.array_equal(got["prob"].view(np.uint32), ref["prob"].view(np.uint32)), V2


def run_both_full(sampler, oracle, logits, gpu_params, oracle_params, u, mask):
    from born_b200 import SamplingConfig
    torch = torch_mod()
    ref = oracle.sample(logits, oracle.make_params(**oracle_params), uniforms=u, mask=mask, want_kept=8, nthreads=8)
    out = sampler.sample(to_dev(logits), uniforms=to_dev(u), config=SamplingConfig(**gpu_params), mask=to_dev(mask),
                         want_lse=True, want_kept_count=True)
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in out.items()}, ref


def test_top_p_without_top_k_is_taken_against_the_row_total(sampler, oracle):
    # top-p with top-k off: the nucleus is defined against the row total (mass blocks); exact on
    # every row, whether the nucleus fits the candidates collected while streaming or not
    V = 128256
    for B in (3, 160):  # rows cut into many segments, and rows that share CTAs
        z = (W.normal(41, B, B * V) * 3.0).astype(np.float32).reshape(B, V)
        z[0, ::9] = -np.inf
        z[1] = np.round(z[1] * 4) / 4  # ties around the boundary
        u = W.uniform_f32(41, 2, B)
        for p in (dict(temperature=0.7, top_p=0.9), dict(temperature=1.0, top_p=0.5),
                  dict(temperature=0.5, top_p=0.95, min_p=0.001), dict(temperature=1.2, top_p=0.95)):
            if B == 160 and p["temperature"] > 1.1:
                continue  # (every row takes the exact search there: covered with B = 3, slow with 160)
            got, ref = run_both(sampler, oracle, z, p, u, want_kept=64)
            assert_parity(got, ref)
    # bf16 with a mask; and a flat row whose nucleus is far beyond the candidate limit
    B = 5
    zb = (W.normal(42, 1, B * 151936) * 4.0).astype(np.float32).reshape(B, 151936)
    zb[4] *= 0.05
    words = (151936 + 31) // 32
    bits = W.uniform(42, 3, B * words * 32).reshape(B, words * 32) < 0.5
    bits[:, 151936:] = False
    mask = np.packbits(bits.reshape(B, words, 32), axis=-1, bitorder="little").view(np.uint32).reshape(B, words)
    got, ref = run_both(sampler, oracle, W.f32_to_bf16_bits(zb).reshape(B, 151936), dict(temperature=0.5, top_p=0.9),
                        W.uniform_f32(42, 5, B), mask=mask, want_kept=64)
    assert ref["kept_count"][4] > 1024
    assert_parity(got, ref)


def test_whole_vocabulary_routes_with_history_penalties(sampler, oracle):
    # temperature (+ top-p) with repetition / frequency / presence penalties and no top-k: fp32
    # rows are patched in the streaming tiles, bf16 rows go through the clean fp32 copy first
    B, V = 7, 50257
    z = (W.normal(51, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)
    u = W.uniform_f32(51, 2, B)
    hist = W.randint(51, 3, B * 96, V).astype(np.int32).reshape(B, 96)
    hist[:, 10:20] = hist[:, 0:10]                      # repeats
    hist[0, :8] = np.argsort(-z[0])[:8].astype(np.int32)  # the row's best tokens are in its history
    hist[1, 5] = -3
    hist[1, 6] = V + 2
    hl = np.array([96, 96, 0, 1, 50, 96, 17], dtype=np.int32)
    for dtype in ("f32", "bf16"):
        logits = z if dtype == "f32" else W.f32_to_bf16_bits(z).reshape(B, V)
        for p in (dict(temperature=0.9, repetition_penalty=1.3),
                  dict(temperature=0.7, frequency_penalty=0.4, presence_penalty=0.2),
                  dict(temperature=0.6, top_p=0.9, repetition_penalty=1.2, frequency_penalty=0.3, presence_penalty=0.1)):
            want = 32 if "top_p" in p else 0
            from born_b200 import SamplingConfig
            torch = torch_mod()
            ref = oracle.sample(logits, oracle.make_params(**p), uniforms=u, history=hist, history_len=hl, want_kept=max(want, 8),
                                nthreads=8)
            out = sampler.sample(to_dev(logits), uniforms=to_dev(u), config=SamplingConfig(**p), history=to_dev(hist),
                                 history_len=to_dev(hl), want_lse=True, want_kept=want, want_kept_count=True)
            torch.cuda.synchronize()
            got = {k: v.cpu().numpy() for k, v in out.items()}
            fits = np.ones(B, dtype=bool)
            for k in ("status", "token", "kept_count"):
                assert np.array_equal(got[k][fits], ref[k][fits]), (dtype, p, k, got[k], ref[k])
            assert np.array_equal(got["prob"][fits].view(np.uint32), ref["prob"][fits].view(np.uint32)), (dtype, p)
            if want:
                assert np.array_equal(got["kept_ids"][fits], ref["kept_ids"][fits][:, :want]), (dtype, p)
            assert np.allclose(got["lse"][fits], ref["lse"][fits], rtol=1e-4, atol=2e-3)


def test_launch_counts(sampler):
    # one launch for every parameter set, token history or not; two more (the clean fp32 copy and
    # its penalty patch) when whole-vocabulary rows are bf16 with history penalties, one more
    # when they are not 16-byte aligned
    from born_b200 import SamplingConfig
    torch = torch_mod()
    B, V = 4, 32000
    z = torch.randn((B, V), device="cuda")
    u = torch.rand(B, device="cuda").clamp_(max=0.999)
    hist = torch.randint(0, V, (B, 32), device="cuda", dtype=torch.int32)

    def launches(cfg, history=None, logits=z):
        n0 = sampler.launch_count
        sampler.sample(logits, uniforms=u, config=cfg, history=history)
        torch.cuda.synchronize()
        return sampler.launch_count - n0

    pen = dict(frequency_penalty=0.5, presence_penalty=0.3)
    assert launches(SamplingConfig(temperature=0.7, min_p=0.05, top_p=0.9, **pen), hist) == 1
    assert launches(SamplingConfig(temperature=0.7, min_p=0.05, top_p=0.9)) == 1
    assert launches(SamplingConfig(temperature=0.7, top_k=50, top_p=0.9)) == 1
    assert launches(SamplingConfig(temperature=0.7, min_p=0.05)) == 1
    assert launches(SamplingConfig(greedy=True)) == 1
    assert launches(SamplingConfig(temperature=0.7)) == 1
    assert launches(SamplingConfig(temperature=0.7, min_p=0.05, full_vocab=True)) == 1
    assert launches(SamplingConfig(temperature=0.7, top_p=0.9)) == 1
    assert launches(SamplingConfig(temperature=0.7, **pen), hist) == 1
    assert launches(SamplingConfig(temperature=0.7, top_p=0.9, **pen), hist) == 1
    zb = z.to(torch.bfloat16)
    assert launches(SamplingConfig(temperature=0.7, top_k=50, **pen), hist, zb) == 1
    assert launches(SamplingConfig(temperature=0.7, **pen), hist, zb) == 3
    odd = torch.randn((B, V + 1), device="cuda")[:, :V]  # rows of 32001 floats: not 16-byte aligned
    assert launches(SamplingConfig(temperature=0.7, top_k=50), None, odd) == 1
    assert launches(SamplingConfig(temperature=0.7), None, odd) == 2


def test_bounded_wait_expires_and_the_handle_stays_usable(sampler, oracle, lib):
    # A kernel wait that cannot be satisfied (the test hook withholds one bulk copy and sets the
    # limit to a millisecond) must give up, report through the error word and leave the handle in
    # working order -- no trap, no hang.
    from born_b200 import _lib as L
    from born_b200.sampler import SamplerError
    torch = torch_mod()
    rc = lib.born_debug_expire_wait(sampler._h, None)
    assert rc == L.ERR_DEVICE_TIMEOUT, rc
    assert b"bounded on-device wait" in lib.born_last_error(sampler._h)
    assert lib.born_check_error(sampler._h) == L.BORN_OK  # reported once, then clear
    B, V = 6, 50000
    z = (W.normal(61, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)
    u = W.uniform_f32(61, 2, B)
    for p in (dict(temperature=0.8, top_k=40, top_p=0.95), dict(temperature=0.9), dict(greedy=True)):
        got, ref = run_both(sampler, oracle, z, p, u)
        assert_parity(got, ref)
    sampler.check_error()
    assert SamplerError is not None and torch is not None


def test_reserve_leaves_nothing_to_allocate(sampler):
    from born_b200 import SamplingConfig
    torch = torch_mod()
    B, V = 8, 40001
    zb = torch.randn((B, V), device="cuda").to(torch.bfloat16)
    u = torch.rand(B, device="cuda").clamp_(max=0.999)
    hist = torch.randint(0, V, (B, 16), device="cuda", dtype=torch.int32)
    cfg = SamplingConfig(temperature=0.9, repetition_penalty=1.2)  # whole-vocabulary bf16 rows with penalties: clean copy
    sampler.reserve(zb, uniforms=u, config=cfg, history=hist)
    w0 = sampler.workspace_bytes
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        sampler.sample(zb, uniforms=u, config=cfg, history=hist)
    torch.cuda.synchronize()
    assert sampler.workspace_bytes == w0
    assert torch.cuda.mem_get_info()[0] == free0


FULL_SIZE_SETTINGS = [
    ("default", dict(temperature=0.7, min_p=0.05, top_p=0.9, frequency_penalty=0.5, presence_penalty=0.3), 512),
    ("topk_topp", dict(temperature=0.7, top_k=50, top_p=0.9), 0),
    ("temperature_only", dict(temperature=0.8), 0),
    ("top_p_only", dict(temperature=0.7, top_p=0.9), 0),
]


@pytest.mark.parametrize("label,params,H", FULL_SIZE_SETTINGS, ids=[x[0] for x in FULL_SIZE_SETTINGS])
def test_headline_batch_every_row_against_the_oracle(sampler, oracle, label, params, H):
    """B=256 x V=128256 fp32 (the headline shape, the benchmark's value distribution): every row."""
    c = W.config2(seed=7, batch=256)
    hist = c["history"] if H else None
    got, ref = run_both(sampler, oracle, c["logits"], params, c["uniforms"], hist=hist, want_kept=0)
    assert_parity(got, ref, check_kept=False)
    assert (ref["status"] == 0).all()


def test_config5_full_batch_on_one_gpu(sampler, oracle):
    """Config 5 at its stated batch (1024 rows x 256000 bf16, 8 vocabulary segments) on one GPU."""
    c = W.config5(seed=0, batch=1024)
    got, ref = run_both(sampler, oracle, c["logits_bf16"], c["params"], c["uniforms"], segments=c["shards"], want_kept=0)
    assert_parity(got, ref, check_kept=False)


def test_out_of_range_row_params_on_the_device_fail_their_row_only(sampler, oracle):
    # a per-row parameter array in device memory is not seen by the host-side range check: the kernel
    # reports the row (token -1, BORN_ROW_BAD_PARAMS) and samples the others as usual
    from born_b200 import SamplingConfig, _lib as L
    from born_b200.sampler import row_params_array
    torch = torch_mod()
    B, V = 6, 9000
    z = (W.normal(77, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)
    u = W.uniform_f32(77, 2, B)
    rows = [dict(temperature=0.8, top_k=30) for _ in range(B)]
    good = row_params_array([SamplingConfig(**r) for r in rows])
    bad = good.copy()
    bad["temperature"][1] = np.nan
    bad["min_p"][3] = 1.5
    bad["top_k"][4] = 5000
    rp = torch.from_numpy(bad.view(np.uint8).copy()).cuda()
    out = sampler.sample(torch.from_numpy(z).cuda(), uniforms=torch.from_numpy(u).cuda(), row_params=rp)
    torch.cuda.synchronize()
    ref = oracle.sample(z, oracle.params_from_rows(rows), uniforms=u, want_kept=1)
    tok, st = out["token"].cpu().numpy(), out["status"].cpu().numpy()
    for b in range(B):
        if b in (1, 3, 4):
            assert tok[b] == -1 and st[b] == L.ROW_BAD_PARAMS, b
        else:
            assert tok[b] == ref["token"][b] and st[b] == L.ROW_OK, b


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_history_penalties_on_rows_of_more_than_64_tiles(oracle, dtype):
    # beyond 64 tiles per row the history list is built by the hash-table path
    from born_b200 import Sampler, SamplingConfig
    torch = torch_mod()
    B, V, H = 3, 300000 if dtype == "f32" else 600000, 700
    params = dict(temperature=0.9, top_k=64, top_p=0.95, repetition_penalty=1.2, frequency_penalty=0.3, presence_penalty=0.1)
    z = (W.normal(91, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)
    hist = W.randint(91, 3, B * H, V).astype(np.int32).reshape(B, H)
    hist[:, 100:200] = hist[:, 0:100]          # repeats
    hist[1, 300:] = hist[1, 300]               # one token many times
    top = np.argsort(-z, axis=1)[:, :40]
    hist[:, 600:640] = top                      # tokens that matter
    u = W.uniform_f32(91, 2, B)
    logits = W.f32_to_bf16_bits(z).reshape(B, V) if dtype == "bf16" else z
    ld = torch.from_numpy(logits.view(np.int16).copy()).cuda().view(torch.bfloat16) if dtype == "bf16" else torch.from_numpy(z).cuda()
    s = Sampler(device=0, max_batch=4, max_vocab=V)
    try:
        out = s.sample(ld, uniforms=torch.from_numpy(u).cuda(), config=SamplingConfig(**params),
                       history=torch.from_numpy(hist).cuda(), want_lse=True, want_kept=64)
        torch.cuda.synchronize()
        ref = oracle.sample(logits, oracle.make_params(**params), uniforms=u, history=hist, want_kept=64)
        assert np.array_equal(out["status"].cpu().numpy(), ref["status"])
        assert np.array_equal(out["token"].cpu().numpy(), ref["token"])
        assert np.array_equal(out["prob"].cpu().numpy().view(np.uint32), ref["prob"].view(np.uint32))
        assert np.array_equal(out["kept_ids"].cpu().numpy(), ref["kept_ids"][:, :64])
    finally:
        s.close()


@pytest.mark.parametrize("H", [512, 513, 1024])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_history_lengths_either_side_of_the_short_list(sampler, oracle, H, dtype):
    # 256 rows give one CTA per row; fp32 launches with at most 512 history ids per row take the
    # instantiation with the short list and five stages, longer histories the one with four
    B, V = 256, 20000
    params = dict(temperature=0.8, min_p=0.02, top_p=0.95, repetition_penalty=1.3, frequency_penalty=0.4, presence_penalty=0.2)
    z = (W.normal(123, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)
    hist = W.randint(123, 3, B * H, V).astype(np.int32).reshape(B, H)
    hist[:, 40:80] = hist[:, 0:40]                              # repeats
    hist[:, H - 24:] = np.argsort(-z, axis=1)[:, :24]           # the tokens that matter, at the end of the list
    hist_len = np.full(B, H, np.int32)
    hist_len[::7] = H // 2                                      # ragged lengths
    u = W.uniform_f32(123, 2, B)
    logits = W.f32_to_bf16_bits(z).reshape(B, V) if dtype == "bf16" else z
    got, ref = run_both(sampler, oracle, logits, params, u, hist=hist, hist_len=hist_len, want_kept=32)
    assert_parity(got, ref)
    assert (ref["status"] == 0).all()
