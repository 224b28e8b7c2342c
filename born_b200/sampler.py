"""Host-side mirror of the sampling capability, over the C ABI of libborn_sampler.so.

The shape follows the reference's Go idioms (born v0.1.1) so that the tests read like its
own: a plain config struct whose zero values mean "off"/default
(internal/optim/adam.go:59-91), a backend object constructed once and used for many calls
(internal/backend/cpu/backend.go:16-20), programmer errors raised as `InvalidArgument`
(the Go side panics: internal/backend/cpu/backend.go:35-37) and runtime failures as
`SamplerError` (the Go side returns `error`: internal/tensor/raw.go:89-92).  The greedy
path is the reference's `argmax` (internal/nn/cross_entropy.go:241-251).

Buffers may be torch CUDA tensors (device call, asynchronous on the given stream) or numpy
arrays / torch CPU tensors (host call: copy in, run, copy out, synchronous).  There is no
CPU implementation behind this class.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib as L

try:  # torch is only needed for device-resident buffers
    import torch
except Exception:  # pragma: no cover
    torch = None


class SamplerError(RuntimeError):
    """Runtime failure reported by the library (CUDA, NCCL, device timeout, unsupported)."""

    def __init__(self, code, message):
        super().__init__(f"born_sampler error {code}: {message}")
        self.code = code


class InvalidArgument(ValueError):
    """Programmer error: the Go wrapper panics on these."""

    def __init__(self, message):
        super().__init__(message)
        self.code = L.ERR_INVALID_ARGUMENT


def load_library():
    return L.load()


def version():
    return L.load().born_version().decode()


@dataclass
class SamplingConfig:
    """Zero values mean "off"; temperature 0 means greedy (first maximum wins)."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 0.0
    min_p: float = 0.0
    repetition_penalty: float = 0.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    greedy: bool = False
    full_vocab: bool = False  # min-p over the whole vocabulary (no survivor limit); top-k and top-p off

    def flags(self):
        return (L.FLAG_GREEDY if self.greedy else 0) | (L.FLAG_FULL_VOCAB if self.full_vocab else 0)

    def to_struct(self):
        return L.RowParams(self.temperature, self.top_p, self.min_p, int(self.top_k), self.repetition_penalty,
                           self.frequency_penalty, self.presence_penalty, self.flags())


ROW_PARAMS_DTYPE = np.dtype([
    ("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("top_k", "<i4"),
    ("repetition_penalty", "<f4"), ("frequency_penalty", "<f4"), ("presence_penalty", "<f4"), ("flags", "<u4"),
])


def row_params_array(configs):
    """Per-row parameter array (numpy structured, 32 bytes per row) from SamplingConfigs."""
    a = np.zeros(len(configs), dtype=ROW_PARAMS_DTYPE)
    for i, c in enumerate(configs):
        a[i] = (c.temperature, c.top_p, c.min_p, c.top_k, c.repetition_penalty, c.frequency_penalty,
                c.presence_penalty, c.flags())
    return a


def _is_torch(x):
    return torch is not None and isinstance(x, torch.Tensor)


def _on_device(x):
    return _is_torch(x) and x.is_cuda


def _ptr(x):
    if x is None:
        return None
    if _is_torch(x):
        return x.data_ptr()
    return x.ctypes.data


def _check_contig(name, x):
    if x is None:
        return
    ok = x.is_contiguous() if _is_torch(x) else x.flags["C_CONTIGUOUS"]
    if not ok:
        raise InvalidArgument(f"{name} must be contiguous")


def _logits_dtype(x, bf16_hint):
    if _is_torch(x):
        if x.dtype == torch.float32:
            return L.DTYPE_F32
        if x.dtype == torch.bfloat16:
            return L.DTYPE_BF16
        if x.dtype in (torch.uint16, torch.int16) and bf16_hint:
            return L.DTYPE_BF16
    else:
        if x.dtype == np.float32:
            return L.DTYPE_F32
        if x.dtype == np.uint16:
            return L.DTYPE_BF16
    raise InvalidArgument(f"logits dtype {x.dtype} is not float32 or bfloat16 (uint16 bit patterns on the host)")


class PreparedCall:
    """A marshalled `born_sample` call (see `Sampler.prepare`)."""

    def __init__(self, sampler, out):
        self._s = sampler
        self._fn = sampler._lib.born_sample
        self.args = None
        self.out = out

    def set_logits(self, logits):
        self.args.logits = _ptr(logits)
        self._keep = logits

    def run(self, stream=None):
        rc = self._fn(self._s._h, C.byref(self.args), stream)
        if rc != L.BORN_OK:
            self._s._raise(rc)
        return self.out


class Sampler:
    """One handle = one device workspace = one stream of calls."""

    def __init__(self, device=0, max_batch=256, max_vocab=262144, max_k=L.MAX_TOP_K):
        self._lib = L.load()
        h = C.c_void_p()
        rc = self._lib.born_sampler_create(device, max_batch, max_vocab, max_k, C.byref(h))
        if rc != L.BORN_OK:
            msg = self._lib.born_last_error(None).decode()
            if rc == L.ERR_INVALID_ARGUMENT:
                raise InvalidArgument(msg)
            raise SamplerError(rc, msg)
        self._h = h
        self.device = device
        self.max_batch = max_batch
        self.max_vocab = max_vocab

    # -- lifetime -------------------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._lib.born_sampler_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- helpers --------------------------------------------------------------------------
    def _raise(self, rc):
        msg = self._lib.born_last_error(self._h).decode()
        if rc == L.ERR_INVALID_ARGUMENT:
            raise InvalidArgument(msg)
        raise SamplerError(rc, msg)

    def _new(self, like_device, shape, dtype_np, dtype_t):
        if like_device:
            return torch.empty(shape, dtype=dtype_t, device=f"cuda:{self.device}")
        return np.empty(shape, dtype=dtype_np)

    @property
    def workspace_bytes(self):
        return int(self._lib.born_workspace_bytes(self._h))

    @property
    def launch_count(self):
        return int(self._lib.born_launch_count(self._h))

    def last_timing_ms(self):
        out = (C.c_float * 3)()
        self._lib.born_last_timing(self._h, out)
        return {"h2d": out[0], "kernel": out[1], "d2h": out[2]}

    # -- sampling -------------------------------------------------------------------------
    def sample(self, logits, uniforms=None, config=None, row_params=None, mask=None, history=None,
               history_len=None, want_prob=True, want_lse=False, want_kept=0, vocab_segments=0, stream=None,
               bf16=False, out=None, want_kept_count=False, uploaded_mask=None):
        """Sample one token per row of `logits` [batch, vocab].

        row_params: optional per-row array (numpy structured `ROW_PARAMS_DTYPE` on the host, or a
        torch uint8/int32 tensor holding the same 32-byte records on the device).
        Returns a dict with token, status and, when asked, prob, lse, kept_ids, kept_count.
        """
        if logits is None or getattr(logits, "ndim", 0) != 2:
            raise InvalidArgument("Sampler.sample: logits must be 2D [batch, vocab]")
        dev = _on_device(logits)
        for name, x in (("uniforms", uniforms), ("mask", mask), ("history", history), ("history_len", history_len),
                        ("row_params", row_params)):
            if x is not None and _on_device(x) != dev:
                raise InvalidArgument(f"{name} must live on the same side (host/device) as logits")
            _check_contig(name, x)
        B, V = int(logits.shape[0]), int(logits.shape[1])
        stride = int(logits.stride(0)) if _is_torch(logits) else int(logits.strides[0] // logits.itemsize)
        inner = int(logits.stride(1)) if _is_torch(logits) else int(logits.strides[1] // logits.itemsize)
        if inner != 1:
            raise InvalidArgument("logits rows must be contiguous")
        a = L.SampleArgs()
        a.struct_size = C.sizeof(L.SampleArgs)
        a.memory = L.MEM_DEVICE if dev else L.MEM_HOST
        a.batch, a.vocab = B, V
        a.logits_dtype = _logits_dtype(logits, bf16)
        a.logits_row_stride = stride
        a.logits = _ptr(logits)
        if mask is not None:
            if mask.ndim != 2 or int(mask.shape[0]) != B:
                raise InvalidArgument("mask must be [batch, ceil(vocab/32)] uint32")
            a.mask = _ptr(mask)
            a.mask_row_stride = int(mask.shape[1])
        if uploaded_mask is not None:  # (device pointer from mask_commit, words per row)
            if mask is not None or not dev:
                raise InvalidArgument("uploaded_mask goes with device logits and without `mask`")
            a.mask = int(uploaded_mask[0])
            a.mask_row_stride = int(uploaded_mask[1])
        if history is not None:
            if history.ndim != 2 or int(history.shape[0]) != B:
                raise InvalidArgument("history must be [batch, n] int32")
            a.history = _ptr(history)
            a.history_stride = int(history.shape[1])
            a.history_len = _ptr(history_len)
        a.row_params = _ptr(row_params)
        a.params = (config or SamplingConfig()).to_struct()
        a.uniforms = _ptr(uniforms)
        a.vocab_segments = int(vocab_segments)
        res = out if out is not None else {}
        if "token" not in res:
            res["token"] = self._new(dev, (B,), np.int32, torch.int32 if torch else None)
            res["status"] = self._new(dev, (B,), np.int32, torch.int32 if torch else None)
            if want_prob:
                res["prob"] = self._new(dev, (B,), np.float32, torch.float32 if torch else None)
            if want_lse:
                res["lse"] = self._new(dev, (B,), np.float32, torch.float32 if torch else None)
            if want_kept:
                if dev:
                    res["kept_ids"] = torch.full((B, want_kept), -1, dtype=torch.int32, device=f"cuda:{self.device}")
                else:
                    res["kept_ids"] = np.full((B, want_kept), -1, dtype=np.int32)
                res["kept_count"] = self._new(dev, (B,), np.int32, torch.int32 if torch else None)
            elif want_kept_count:  # the size of the kept set without the id list
                res["kept_count"] = self._new(dev, (B,), np.int32, torch.int32 if torch else None)
        a.out_token = _ptr(res["token"])
        a.out_status = _ptr(res["status"])
        a.out_prob = _ptr(res.get("prob"))
        a.out_lse = _ptr(res.get("lse"))
        a.out_kept_ids = _ptr(res.get("kept_ids"))
        a.out_kept_count = _ptr(res.get("kept_count"))
        a.kept_stride = int(res["kept_ids"].shape[1]) if "kept_ids" in res else 0
        if getattr(self, "_marshal", None) is not None:
            self._marshal.args = a
            return res
        entry = self._lib.born_sample_next if getattr(self, "_next", False) else self._lib.born_sample
        rc = entry(self._h, C.byref(a), stream)
        if rc != L.BORN_OK:
            self._raise(rc)
        return res

    # -- the autoregressive loop: device-resident history, stop tokens --------------------------
    def history_create(self, capacity):
        """Allocate the device-resident token history: the last `capacity` tokens of every row."""
        rc = self._lib.born_history_create(self._h, int(capacity))
        if rc != L.BORN_OK:
            self._raise(rc)

    def history_reset(self, tokens, lens=None, stream=None):
        """Load prompts [batch, n] (int32, host or device) with optional per-row lengths; clears the finished flags."""
        dev = _on_device(tokens)
        if lens is not None and _on_device(lens) != dev:
            raise InvalidArgument("lens must live on the same side (host/device) as tokens")
        B, n = int(tokens.shape[0]), int(tokens.shape[1])
        rc = self._lib.born_history_reset(self._h, _ptr(tokens) if n else None, _ptr(lens), B, n,
                                          L.MEM_DEVICE if dev else L.MEM_HOST, stream)
        if rc != L.BORN_OK:
            self._raise(rc)

    def history_set_stop_tokens(self, ids):
        ids = [int(i) for i in ids]
        arr = (C.c_int32 * max(1, len(ids)))(*ids)
        rc = self._lib.born_history_set_stop_tokens(self._h, arr, len(ids))
        if rc != L.BORN_OK:
            self._raise(rc)

    def history_read(self, batch, capacity, stream=None):
        """(tokens [batch, capacity] in ring order, total [batch], finished [batch]) as numpy arrays."""
        tok = np.zeros((batch, capacity), dtype=np.int32)
        total = np.zeros(batch, dtype=np.int32)
        fin = np.zeros(batch, dtype=np.int32)
        rc = self._lib.born_history_read(self._h, tok.ctypes.data, total.ctypes.data, fin.ctypes.data, int(batch), L.MEM_HOST, stream)
        if rc != L.BORN_OK:
            self._raise(rc)
        return tok, total, fin

    def sample_next(self, logits, **kw):
        """`sample` over the device-resident history: the kernel appends every row's token to it."""
        if kw.get("history") is not None or kw.get("history_len") is not None:
            raise InvalidArgument("sample_next reads the sampler's own history")
        self._next = True
        try:
            return self.sample(logits, **kw)
        finally:
            self._next = False

    # -- grammar masks: double-buffered upload ----------------------------------------------------
    def mask_begin(self, batch, words_per_row):
        """The pinned host buffer to fill for the next step, as a numpy uint32 array [batch, words_per_row]."""
        p = C.POINTER(C.c_uint32)()
        rc = self._lib.born_mask_begin(self._h, int(batch), int(words_per_row), C.byref(p))
        if rc != L.BORN_OK:
            self._raise(rc)
        return np.ctypeslib.as_array(p, shape=(int(batch), int(words_per_row)))

    def mask_commit(self):
        """Start the copy of the buffer from `mask_begin` to the device; returns the device pointer."""
        d = C.c_void_p()
        rc = self._lib.born_mask_commit(self._h, C.byref(d))
        if rc != L.BORN_OK:
            self._raise(rc)
        return int(d.value)

    def mask_wait(self, stream=None):
        """Make `stream` wait for the committed mask (no host synchronisation)."""
        rc = self._lib.born_mask_wait(self._h, stream)
        if rc != L.BORN_OK:
            self._raise(rc)

    def prepare(self, logits, **kw):
        """Marshal a `sample` call once and return a `PreparedCall`: `run(stream)` then costs one
        foreign call.  Takes the arguments of `sample`; the buffers must stay alive and in place."""
        kw.pop("stream", None)
        call = PreparedCall(self, kw.get("out"))
        self._marshal = call
        try:
            call.out = self.sample(logits, **kw)
        finally:
            self._marshal = None
        return call

    def reserve(self, logits, **kw):
        """Allocate now whatever scratch a `sample` call with these arguments would allocate on first use."""
        call = self.prepare(logits, **kw)
        rc = self._lib.born_sampler_reserve(self._h, C.byref(call.args))
        if rc != L.BORN_OK:
            self._raise(rc)

    def check_error(self):
        """Raise if a bounded on-device wait gave up in an earlier device-memory call (synchronises)."""
        rc = self._lib.born_check_error(self._h)
        if rc != L.BORN_OK:
            self._raise(rc)

    @property
    def fallback_rows(self):
        """Rows that took the exact multi-pass search since the last read (synchronises)."""
        return int(self._lib.born_fallback_rows(self._h))

    # -- speculative decoding -------------------------------------------------------------
    def spec_verify(self, target_logits, draft_logits, draft_tokens, u_accept, u_resample, temperature=1.0,
                    stream=None):
        """target [B, K or K+1, V], draft [B, K, V] fp32; returns accept_len [B], tokens [B, K+1], status [B]."""
        if getattr(target_logits, "ndim", 0) != 3 or getattr(draft_logits, "ndim", 0) != 3:
            raise InvalidArgument("spec_verify: target and draft logits must be 3D")
        dev = _on_device(target_logits)
        for name, x in (("target_logits", target_logits), ("draft_logits", draft_logits),
                        ("draft_tokens", draft_tokens), ("u_accept", u_accept), ("u_resample", u_resample)):
            if _on_device(x) != dev:
                raise InvalidArgument(f"{name} must live on the same side as target_logits")
            _check_contig(name, x)
        B, R, V = (int(s) for s in target_logits.shape)
        K = int(draft_logits.shape[1])
        a = L.SpecArgs()
        a.struct_size = C.sizeof(L.SpecArgs)
        a.memory = L.MEM_DEVICE if dev else L.MEM_HOST
        a.batch, a.draft_len, a.vocab, a.target_rows = B, K, V, R
        a.target_logits, a.draft_logits = _ptr(target_logits), _ptr(draft_logits)
        a.draft_tokens, a.u_accept, a.u_resample = _ptr(draft_tokens), _ptr(u_accept), _ptr(u_resample)
        a.temperature = float(temperature)
        res = {
            "accept_len": self._new(dev, (B,), np.int32, torch.int32 if torch else None),
            "tokens": self._new(dev, (B, K + 1), np.int32, torch.int32 if torch else None),
            "status": self._new(dev, (B,), np.int32, torch.int32 if torch else None),
        }
        a.out_accept_len, a.out_tokens, a.out_status = _ptr(res["accept_len"]), _ptr(res["tokens"]), _ptr(res["status"])
        rc = self._lib.born_spec_verify(self._h, C.byref(a), stream)
        if rc != L.BORN_OK:
            self._raise(rc)
        return res

    # -- vocab-sharded path ---------------------------------------------------------------
    def record_bytes(self, top_k):
        return int(self._lib.born_shard_record_bytes(int(top_k)))

    @staticmethod
    def nccl_unique_id():
        buf = (C.c_char * 128)()
        rc = L.load().born_shard_unique_id(buf)
        if rc != L.BORN_OK:
            raise SamplerError(rc, L.load().born_last_error(None).decode())
        return bytes(buf)

    def shard_init(self, unique_id, rank, nranks):
        buf = C.create_string_buffer(unique_id, 128)
        rc = self._lib.born_shard_init(self._h, buf, rank, nranks)
        if rc != L.BORN_OK:
            self._raise(rc)

    def _shard_args(self, batch, vocab_local, rank, nranks, top_k, temperature, top_p):
        a = L.ShardArgs()
        a.struct_size = C.sizeof(L.ShardArgs)
        a.memory = L.MEM_DEVICE
        a.batch, a.vocab_local, a.rank, a.nranks, a.top_k = batch, vocab_local, rank, nranks, top_k
        a.temperature, a.top_p = temperature, top_p
        return a

    def shard_local(self, logits, rank, nranks, top_k, temperature=1.0, top_p=0.0, stream=None, packed=None):
        """Local pass over this rank's vocab shard: one packed record per row (device tensor)."""
        if not _on_device(logits) or logits.ndim != 2:
            raise InvalidArgument("shard_local: logits must be a 2D CUDA tensor")
        B, Vl = int(logits.shape[0]), int(logits.shape[1])
        a = self._shard_args(B, Vl, rank, nranks, top_k, temperature, top_p)
        a.logits_dtype = _logits_dtype(logits, False)
        a.logits_row_stride = int(logits.stride(0))
        a.logits = logits.data_ptr()
        if packed is None:
            packed = torch.empty((B, self.record_bytes(top_k)), dtype=torch.uint8, device=logits.device)
        a.packed = packed.data_ptr()
        rc = self._lib.born_shard_local(self._h, C.byref(a), stream)
        if rc != L.BORN_OK:
            self._raise(rc)
        return packed

    def shard_merge(self, gathered, uniforms, vocab_local, rank, nranks, top_k, temperature=1.0, top_p=0.0,
                    want_lse=True, stream=None):
        """Merge the all-gathered records [nranks, batch, record_bytes] and draw the tokens."""
        if not _on_device(gathered) or gathered.ndim != 3:
            raise InvalidArgument("shard_merge: gathered must be a 3D CUDA uint8 tensor")
        B = int(gathered.shape[1])
        a = self._shard_args(B, vocab_local, rank, nranks, top_k, temperature, top_p)
        a.gathered = gathered.data_ptr()
        a.uniforms = uniforms.data_ptr()
        dev = gathered.device
        res = {"token": torch.empty(B, dtype=torch.int32, device=dev),
               "status": torch.empty(B, dtype=torch.int32, device=dev),
               "prob": torch.empty(B, dtype=torch.float32, device=dev)}
        if want_lse:
            res["lse"] = torch.empty(B, dtype=torch.float32, device=dev)
        a.out_token, a.out_status, a.out_prob = res["token"].data_ptr(), res["status"].data_ptr(), res["prob"].data_ptr()
        a.out_lse = res["lse"].data_ptr() if want_lse else None
        rc = self._lib.born_shard_merge(self._h, C.byref(a), stream)
        if rc != L.BORN_OK:
            self._raise(rc)
        return res

    def sample_sharded(self, logits, uniforms, rank, nranks, top_k, temperature=1.0, top_p=0.0, want_lse=True,
                       stream=None, out=None):
        """Local pass + NCCL all-gather + merge in one call (needs shard_init)."""
        if not _on_device(logits) or logits.ndim != 2:
            raise InvalidArgument("sample_sharded: logits must be a 2D CUDA tensor")
        B, Vl = int(logits.shape[0]), int(logits.shape[1])
        a = self._shard_args(B, Vl, rank, nranks, top_k, temperature, top_p)
        a.logits_dtype = _logits_dtype(logits, False)
        a.logits_row_stride = int(logits.stride(0))
        a.logits = logits.data_ptr()
        a.uniforms = uniforms.data_ptr()
        dev = logits.device
        res = out if out is not None else {}
        if "token" not in res:
            res.update({"token": torch.empty(B, dtype=torch.int32, device=dev),
                        "status": torch.empty(B, dtype=torch.int32, device=dev),
                        "prob": torch.empty(B, dtype=torch.float32, device=dev)})
            if want_lse:
                res["lse"] = torch.empty(B, dtype=torch.float32, device=dev)
        a.out_token, a.out_status, a.out_prob = res["token"].data_ptr(), res["status"].data_ptr(), res["prob"].data_ptr()
        a.out_lse = res["lse"].data_ptr() if "lse" in res else None
        rc = self._lib.born_sample_sharded(self._h, C.byref(a), stream)
        if rc != L.BORN_OK:
            self._raise(rc)
        return res
