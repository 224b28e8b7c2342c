"""The autoregressive loop around the sampler: device-resident history with stop tokens, and the
double-buffered grammar-mask upload -- N steps on synthetic logits against the oracle fed the
history as it grows."""
import ctypes as C

import numpy as np
import pytest

from born_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _dev(a):
    import torch
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32).copy()).cuda()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_history_grows_on_the_device_and_matches_the_oracle(sampler, oracle, dtype):
    import torch
    from born_b200 import SamplingConfig, _lib as L
    B, V, cap, steps, P = 6, 20000, 48, 24, 40   # the ring (48) wraps after 8 steps
    params = dict(temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.3, frequency_penalty=0.4, presence_penalty=0.2)
    cfg, op = SamplingConfig(**params), oracle.make_params(**params)
    prompts = W.randint(7, 1, B * P, V).astype(np.int32).reshape(B, P)
    lens = np.array([40, 0, 17, 40, 3, 25], dtype=np.int32)
    stop = [int(x) for x in W.randint(7, 2, 3, V)]
    sampler.history_create(cap)
    sampler.history_set_stop_tokens(stop)
    sampler.history_reset(_dev(prompts), _dev(lens))
    hist = [list(prompts[b, :lens[b]]) for b in range(B)]   # the oracle's view: everything so far
    finished = np.zeros(B, dtype=bool)
    for t in range(steps):
        z = (W.normal(100 + t, 1, B * V) * 2.5).astype(np.float32).reshape(B, V)
        # make stop tokens likely now and then
        if t % 5 == 4:
            z[t % B, stop[t % 3]] += 30.0
        logits = W.f32_to_bf16_bits(z).reshape(B, V) if dtype == "bf16" else z
        u = W.uniform_f32(100 + t, 2, B)
        ld = torch.from_numpy(logits.view(np.int16).copy()).cuda().view(torch.bfloat16) if dtype == "bf16" else _dev(logits)
        out = sampler.sample_next(ld, uniforms=_dev(u), config=cfg, want_lse=True)
        torch.cuda.synchronize()
        got_tok, got_st = out["token"].cpu().numpy(), out["status"].cpu().numpy()
        # the oracle sees the last `cap` tokens of every row
        H = max(1, max(min(len(h), cap) for h in hist))
        hw = np.zeros((B, H), dtype=np.int32)
        hl = np.zeros(B, dtype=np.int32)
        for b in range(B):
            tail = hist[b][-cap:]
            hw[b, :len(tail)] = tail
            hl[b] = len(tail)
        ref = oracle.sample(logits, op, uniforms=u, history=hw, history_len=hl, want_kept=1)
        for b in range(B):
            if finished[b]:
                assert got_tok[b] == -1 and got_st[b] == L.ROW_FINISHED, (t, b)
                continue
            assert got_tok[b] == ref["token"][b] and got_st[b] == ref["status"][b], (t, b)
            hist[b].append(int(got_tok[b]))
            if int(got_tok[b]) in stop:
                finished[b] = True
    tok, total, fin = sampler.history_read(B, cap)
    assert finished.any() and not finished.all()
    assert np.array_equal(fin.astype(bool), finished)
    for b in range(B):
        assert total[b] == len(hist[b])
        want = np.zeros(cap, dtype=np.int32)
        for i, x in enumerate(hist[b]):
            want[i % cap] = x
        n = min(len(hist[b]), cap)
        assert sorted(tok[b][:n].tolist()) == sorted(hist[b][-cap:]) and np.array_equal(tok[b][:n], want[:n]), b


def test_sample_next_refuses_a_caller_history_and_needs_create(lib):
    import torch
    from born_b200 import _lib as L
    h = C.c_void_p()
    assert lib.born_sampler_create(0, 8, 4096, 0, C.byref(h)) == L.BORN_OK
    try:
        a = L.SampleArgs()
        a.struct_size = C.sizeof(L.SampleArgs)
        assert lib.born_sample_next(h, C.byref(a), None) == L.ERR_INVALID_ARGUMENT       # no history yet
        assert lib.born_history_create(h, 0) == L.ERR_INVALID_ARGUMENT
        assert lib.born_history_create(h, 2000) == L.ERR_INVALID_ARGUMENT
        assert lib.born_history_create(h, 64) == L.BORN_OK
        z = torch.zeros((2, 4096), device="cuda")
        hist = torch.zeros((2, 4), dtype=torch.int32, device="cuda")
        a.memory = L.MEM_DEVICE
        a.batch, a.vocab, a.logits_row_stride = 2, 4096, 4096
        a.logits = z.data_ptr()
        a.history = hist.data_ptr()
        a.history_stride = 4
        assert lib.born_sample_next(h, C.byref(a), None) == L.ERR_INVALID_ARGUMENT       # brings its own history
        assert lib.born_history_set_stop_tokens(h, None, 9) == L.ERR_INVALID_ARGUMENT
    finally:
        lib.born_sampler_destroy(h)


def test_uploaded_masks_alternate_buffers_and_match_a_direct_mask(sampler, oracle):
    import torch
    from born_b200 import SamplingConfig
    B, V = 5, 30000
    words = (V + 31) // 32
    cfg = SamplingConfig(temperature=0.9, top_k=20)
    op = oracle.make_params(temperature=0.9, top_k=20)
    ptrs = []
    for step in range(4):
        z = (W.normal(300 + step, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)
        u = W.uniform_f32(300 + step, 2, B)
        bits = W.uniform(300 + step, 3, B * words * 32).reshape(B, words * 32) < 0.1
        bits[:, V:] = False
        bits[:, step] = True
        mask = np.packbits(bits.reshape(B, words, 32), axis=-1, bitorder="little").view(np.uint32).reshape(B, words)
        buf = sampler.mask_begin(B, words)
        buf[:] = mask
        dptr = sampler.mask_commit()
        ptrs.append(dptr)
        sampler.mask_wait(None)
        out = sampler.sample(_dev(z), uniforms=_dev(u), config=cfg, uploaded_mask=(dptr, words))
        torch.cuda.synchronize()
        ref = oracle.sample(z, op, uniforms=u, mask=mask, want_kept=1)
        assert np.array_equal(out["token"].cpu().numpy(), ref["token"])
        assert np.array_equal(out["status"].cpu().numpy(), ref["status"])
    assert ptrs[0] == ptrs[2] and ptrs[1] == ptrs[3] and ptrs[0] != ptrs[1]


@pytest.mark.parametrize("cap,top_k", [(32, 40), (600, 40), (32, 300)], ids=["short-ring", "long-ring", "exact-search"])
def test_device_history_with_one_cta_per_row(sampler, oracle, cap, top_k):
    # 256 rows: every CTA streams one whole row (the instantiations without segment records), the
    # CTA that finishes a row -- from its candidates or, for top-k above 256, by the exact search --
    # appends the token to the ring; rings of at most 512 ids take the short history list
    import torch
    from born_b200 import SamplingConfig, _lib as L
    B, V, steps, P = 256, 9000, 5, 20
    params = dict(temperature=0.9, top_k=top_k, top_p=0.97, repetition_penalty=1.2, frequency_penalty=0.3, presence_penalty=0.1)
    cfg, op = SamplingConfig(**params), oracle.make_params(**params)
    prompts = W.randint(11, 1, B * P, V).astype(np.int32).reshape(B, P)
    lens = (W.randint(11, 2, B, P + 1)).astype(np.int32)
    stop = [int(x) for x in W.randint(11, 3, 2, V)]
    sampler.history_create(cap)
    sampler.history_set_stop_tokens(stop)
    sampler.history_reset(_dev(prompts), _dev(lens))
    hist = [list(prompts[b, :lens[b]]) for b in range(B)]
    finished = np.zeros(B, dtype=bool)
    for t in range(steps):
        z = (W.normal(500 + t, 1, B * V) * 2.5).astype(np.float32).reshape(B, V)
        z[(7 * t) % B, stop[t % 2]] += 30.0
        u = W.uniform_f32(500 + t, 2, B)
        out = sampler.sample_next(_dev(z), uniforms=_dev(u), config=cfg, want_lse=True)
        torch.cuda.synchronize()
        got_tok, got_st = out["token"].cpu().numpy(), out["status"].cpu().numpy()
        H = max(1, max(min(len(h), cap) for h in hist))
        hw = np.zeros((B, H), dtype=np.int32)
        hl = np.zeros(B, dtype=np.int32)
        for b in range(B):
            tail = hist[b][-cap:]
            hw[b, :len(tail)] = tail
            hl[b] = len(tail)
        ref = oracle.sample(z, op, uniforms=u, history=hw, history_len=hl, want_kept=1, nthreads=8)
        for b in range(B):
            if finished[b]:
                assert got_tok[b] == -1 and got_st[b] == L.ROW_FINISHED, (t, b)
                continue
            assert got_tok[b] == ref["token"][b] and got_st[b] == ref["status"][b], (t, b)
            hist[b].append(int(got_tok[b]))
            if int(got_tok[b]) in stop:
                finished[b] = True
    tok, total, fin = sampler.history_read(B, cap)
    assert finished.any() and not finished.all()
    assert np.array_equal(fin.astype(bool), finished)
    for b in range(B):
        assert total[b] == len(hist[b])
