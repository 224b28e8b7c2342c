"""ctypes loader for the CPU oracle (oracle/born_oracle.c).

TEST INFRASTRUCTURE: imported by tests/, by the smoke check and by the CPU-baseline leg of
the benchmark only.  Nothing under born_b200/ imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "libborn_oracle.so")
SRC = os.path.join(HERE, "born_oracle.c")

ROW_PARAMS_DTYPE = np.dtype([
    ("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("top_k", "<i4"),
    ("repetition_penalty", "<f4"), ("frequency_penalty", "<f4"), ("presence_penalty", "<f4"), ("flags", "<u4"),
])

_lib = None


def build(force=False):
    if force or not os.path.exists(SO) or os.path.getmtime(SO) < os.path.getmtime(SRC):
        subprocess.run(["make", "-C", HERE, "-B", "libborn_oracle.so"], check=True, capture_output=True)
    return SO


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(SO):
            build()
        lib = C.CDLL(SO)
        lib.born_oracle_ref_logsoftmax.restype = C.c_float
        lib.born_oracle_ref_logsoftmax.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        lib.born_oracle_ref_softmax.restype = None
        lib.born_oracle_ref_softmax.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        lib.born_oracle_ref_argmax.restype = C.c_int
        lib.born_oracle_ref_argmax.argtypes = [C.c_void_p, C.c_int]
        lib.born_oracle_ref_accuracy.restype = C.c_float
        lib.born_oracle_ref_accuracy.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        lib.born_oracle_exp.restype = None
        lib.born_oracle_exp.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        lib.born_oracle_mass.restype = None
        lib.born_oracle_mass.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        lib.born_oracle_sample.restype = C.c_int
        lib.born_oracle_sample.argtypes = [
            C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_void_p,
            C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
            C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        lib.born_oracle_spec_verify.restype = C.c_int
        lib.born_oracle_spec_verify.argtypes = [
            C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
            C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        lib.born_oracle_draft_tokens.restype = C.c_int
        lib.born_oracle_draft_tokens.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p]
        _lib = lib
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data


def ref_logsoftmax(z):
    z = np.ascontiguousarray(z, dtype=np.float32)
    out = np.empty_like(z)
    lse = load().born_oracle_ref_logsoftmax(_p(z), z.size, _p(out))
    return float(lse), out


def ref_softmax(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    load().born_oracle_ref_softmax(_p(x), _p(out), x.shape[0], x.shape[1])
    return out


def ref_argmax(z):
    z = np.ascontiguousarray(z, dtype=np.float32)
    return int(load().born_oracle_ref_argmax(_p(z), z.size))


def ref_accuracy(logits, targets):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    targets = np.ascontiguousarray(targets, dtype=np.int32)
    return float(load().born_oracle_ref_accuracy(_p(logits), _p(targets), logits.shape[0], logits.shape[1]))


def exp_det(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    load().born_oracle_exp(_p(x), _p(y), x.size)
    return y


def mass(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.empty(x.shape, dtype=np.uint64)
    load().born_oracle_mass(_p(x), _p(q), x.size)
    return q


def make_params(n=None, **kw):
    """One params record (n=None) or an array of n identical records."""
    a = np.zeros(1 if n is None else n, dtype=ROW_PARAMS_DTYPE)
    for k, v in kw.items():
        if k == "greedy":
            a["flags"] = 1 if v else 0
        else:
            a[k] = v
    return a


def params_from_rows(rows):
    a = np.zeros(len(rows), dtype=ROW_PARAMS_DTYPE)
    for i, r in enumerate(rows):
        for k, v in r.items():
            if k == "greedy":
                a["flags"][i] = 1 if v else 0
            else:
                a[k][i] = v
    return a


def sample(logits, params, uniforms=None, mask=None, history=None, history_len=None, segments=1,
           want_kept=0, want_lse=True, nthreads=1):
    """logits: float32 [B, V] or uint16 (bf16 bits) [B, V]; params: structured array of 1 or B records."""
    assert logits.ndim == 2 and logits.flags["C_CONTIGUOUS"]
    B, V = logits.shape
    dtype = 0 if logits.dtype == np.float32 else 1
    assert logits.dtype in (np.float32, np.uint16)
    params = np.ascontiguousarray(params, dtype=ROW_PARAMS_DTYPE)
    rp_stride = 0 if params.size == 1 else 1
    assert params.size in (1, B)
    u = np.zeros(B, dtype=np.float32) if uniforms is None else np.ascontiguousarray(uniforms, dtype=np.float32)
    tok = np.empty(B, dtype=np.int32)
    prob = np.empty(B, dtype=np.float32)
    lse = np.empty(B, dtype=np.float32) if want_lse else None
    status = np.empty(B, dtype=np.int32)
    near = np.zeros(B, dtype=np.int32)
    kept_ids = np.full((B, want_kept), -1, dtype=np.int32) if want_kept else None
    kept_count = np.zeros(B, dtype=np.int32)
    if mask is not None:
        mask = np.ascontiguousarray(mask, dtype=np.uint32)
    if history is not None:
        history = np.ascontiguousarray(history, dtype=np.int32)
    if history_len is not None:
        history_len = np.ascontiguousarray(history_len, dtype=np.int32)
    rc = load().born_oracle_sample(
        B, V, dtype, _p(logits), V, _p(mask), 0 if mask is None else mask.shape[1],
        _p(history), 0 if history is None else history.shape[1], _p(history_len),
        _p(params), rp_stride, _p(u), int(segments), _p(tok), _p(prob), _p(lse), _p(status),
        _p(kept_ids), _p(kept_count), int(want_kept), _p(near), int(nthreads))
    if rc != 0:
        raise MemoryError("oracle allocation failed")
    return {"token": tok, "prob": prob, "lse": lse, "status": status, "kept_ids": kept_ids,
            "kept_count": kept_count, "near_cutoff": near}


def spec_verify(target, draft, draft_tok, u_accept, u_resample, temperature=1.0, nthreads=1):
    target = np.ascontiguousarray(target, dtype=np.float32)
    draft = np.ascontiguousarray(draft, dtype=np.float32)
    B, R, V = target.shape
    K = draft.shape[1]
    draft_tok = np.ascontiguousarray(draft_tok, dtype=np.int32)
    u_accept = np.ascontiguousarray(u_accept, dtype=np.float32)
    u_resample = np.ascontiguousarray(u_resample, dtype=np.float32)
    alen = np.empty(B, dtype=np.int32)
    out = np.empty((B, K + 1), dtype=np.int32)
    status = np.empty(B, dtype=np.int32)
    rc = load().born_oracle_spec_verify(B, K, V, R, _p(target), _p(draft), _p(draft_tok), _p(u_accept),
                                        _p(u_resample), float(temperature), _p(alen), _p(out), _p(status),
                                        int(nthreads))
    if rc != 0:
        raise MemoryError("oracle allocation failed")
    return {"accept_len": alen, "tokens": out, "status": status}


def draft_tokens(draft, u, temperature=1.0):
    draft = np.ascontiguousarray(draft, dtype=np.float32)
    B, K, V = draft.shape
    u = np.ascontiguousarray(u, dtype=np.float32)
    tok = np.empty((B, K), dtype=np.int32)
    load().born_oracle_draft_tokens(B, K, V, _p(draft), _p(u), float(temperature), _p(tok))
    return tok
