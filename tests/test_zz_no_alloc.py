"""born_sample_static: the entry point for callers that cannot allocate device memory.

Some hosts of this library run where cudaMalloc is off limits: a serving process whose
memory pool has already claimed the whole GPU, or a decode loop that must not hit the
allocator.  For them the library keeps the kernel's scratch (segment records, mass blocks,
history lists, row tickets) in a fixed device array inside its own image.  This test drives
the entry point through the C ABI twice in a row -- the second call finds the array as the
first one left it -- and holds the results against the regular born_sample entry point and
against the CPU oracle on the same inputs; it also checks that the calls leave the amount of
free device memory unchanged.  It lives in a file of its own that pytest collects last.
"""
import ctypes as C

import numpy as np
import pytest

from born_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _args(L, logits, u, hist, cfg, out, V):
    a = L.SampleArgs()
    a.struct_size = C.sizeof(L.SampleArgs)
    a.memory = L.MEM_DEVICE
    a.batch, a.vocab = int(logits.shape[0]), V
    a.logits_dtype = L.DTYPE_F32
    a.logits_row_stride = int(logits.stride(0))
    a.logits = logits.data_ptr()
    a.history = hist.data_ptr()
    a.history_stride = int(hist.shape[1])
    a.params = cfg.to_struct()
    a.uniforms = u.data_ptr()
    a.out_token = out["token"].data_ptr()
    a.out_prob = out["prob"].data_ptr()
    a.out_lse = out["lse"].data_ptr()
    a.out_status = out["status"].data_ptr()
    return a


@pytest.mark.parametrize("B,params", [
    (12, dict(temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.1)),  # few rows: every row is many segments
    (256, dict(temperature=0.7, min_p=0.05, top_p=0.9, frequency_penalty=0.5, presence_penalty=0.3)),  # the row limit
    (7, dict(temperature=0.9)),               # whole-vocabulary rows: mass blocks in the static array
    (5, dict(temperature=1.6, top_p=0.9)),    # a nucleus beyond the candidates: the exact search, still no allocation
])
def test_static_entry_matches_regular_entry_twice(lib, oracle, B, params):
    import torch
    from born_b200 import Sampler, SamplingConfig, _lib as L
    assert torch.cuda.is_available(), "needs a CUDA device"
    torch.cuda.set_device(0)
    V, H = 128256, 64
    cfg = SamplingConfig(**params)
    with Sampler(device=0, max_batch=B, max_vocab=V) as regular:
        for call in range(2):
            z = torch.from_numpy((W.normal(900 + call, 1, B * V) * 3.0).astype(np.float32).reshape(B, V)).cuda()
            u = torch.from_numpy(W.uniform_f32(900 + call, 2, B)).cuda()
            hist = torch.from_numpy(W.randint(900 + call, 3, B * H, V).astype(np.int32).reshape(B, H)).cuda()
            want = regular.sample(z, uniforms=u, config=cfg, history=hist, want_lse=True)
            got = {"token": torch.full((B,), -7, dtype=torch.int32, device="cuda"),
                   "status": torch.full((B,), -7, dtype=torch.int32, device="cuda"),
                   "prob": torch.zeros(B, dtype=torch.float32, device="cuda"),
                   "lse": torch.zeros(B, dtype=torch.float32, device="cuda")}
            a = _args(L, z, u, hist, cfg, got, V)
            torch.cuda.synchronize()
            free0 = torch.cuda.mem_get_info()[0] if call == 1 else None  # (the first call may load the kernels)
            rc = lib.born_sample_static(C.byref(a), None)
            assert rc == 0, lib.born_last_error(None)
            torch.cuda.synchronize()
            if free0 is not None:
                assert torch.cuda.mem_get_info()[0] == free0
            ref = oracle.sample(z.cpu().numpy(), oracle.make_params(**params), uniforms=u.cpu().numpy(),
                                history=hist.cpu().numpy(), nthreads=8)
            assert np.array_equal(got["token"].cpu().numpy(), ref["token"])
            assert np.array_equal(got["prob"].cpu().numpy().view(np.uint32), ref["prob"].view(np.uint32))
            assert torch.equal(got["status"], want["status"]) and int(got["status"].abs().sum()) == 0
            assert torch.equal(got["token"], want["token"])
            assert torch.equal(got["prob"], want["prob"])  # integer masses: bit-exact
            # same tolerance as the log-sum-exp checks of the parity tests
            assert torch.allclose(got["lse"], want["lse"], rtol=0, atol=1e-5)


def test_static_entry_rejects_what_it_cannot_hold(lib):
    import torch
    from born_b200 import SamplingConfig, _lib as L
    B, V = 257, 1024  # one row more than the static scratch is sized for
    z = torch.zeros((B, V), device="cuda")
    u = torch.zeros(B, device="cuda")
    hist = torch.zeros((B, 1), dtype=torch.int32, device="cuda")
    out = {k: torch.zeros(B, dtype=t, device="cuda") for k, t in
           (("token", torch.int32), ("status", torch.int32), ("prob", torch.float32), ("lse", torch.float32))}
    a = _args(L, z, u, hist, SamplingConfig(temperature=1.0, top_k=5), out, V)
    assert lib.born_sample_static(C.byref(a), None) == L.ERR_UNSUPPORTED
    assert b"static scratch limit" in lib.born_last_error(None)
    a.batch = 4
    a.memory = L.MEM_HOST
    assert lib.born_sample_static(C.byref(a), None) == L.ERR_UNSUPPORTED
    a.memory = L.MEM_DEVICE
    a.vocab_segments = 2
    assert lib.born_sample_static(C.byref(a), None) == L.ERR_UNSUPPORTED  # needs scratch it does not have
    a.vocab_segments = 0
    # whole-vocabulary bf16 rows with history penalties need the clean fp32 copy: refused, not allocated
    zb = torch.zeros((4, V), dtype=torch.bfloat16, device="cuda")
    b = _args(L, zb, u, hist, SamplingConfig(temperature=1.0, repetition_penalty=1.2), out, V)
    b.batch = 4
    b.logits_dtype = L.DTYPE_BF16
    assert lib.born_sample_static(C.byref(b), None) == L.ERR_UNSUPPORTED
    assert b"may not allocate" in lib.born_last_error(None)
    # and the mass-block limit: batch x ceil(vocab / 512) beyond BORN_STATIC_MAX_BLOCKS
    big = _args(L, z, u, hist, SamplingConfig(temperature=1.0, top_k=5), out, V)
    big.batch, big.vocab, big.logits_row_stride = 256, 1 << 20, 1 << 20
    assert lib.born_sample_static(C.byref(big), None) == L.ERR_UNSUPPORTED
    assert b"mass blocks" in lib.born_last_error(None)
