"""ctypes view of include/born_sampler.h (struct layouts must match the header)."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("BORN_SAMPLER_LIB") or os.path.join(HERE, "libborn_sampler.so")

BORN_OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_CUDA = 2
ERR_NO_DEVICE = 3
ERR_UNSUPPORTED = 4
ERR_NCCL = 5
ERR_DEVICE_TIMEOUT = 6

ROW_OK, ROW_ALL_MASKED, ROW_NAN, ROW_POS_INF, ROW_OVERFLOW, ROW_BAD_TOKEN, ROW_FINISHED, ROW_BAD_PARAMS = range(8)

MAX_TOP_K = 1024
MAX_HISTORY = 1024
MAX_DRAFT = 16
MAX_SHARDS = 16
DTYPE_F32, DTYPE_BF16 = 0, 1
MEM_DEVICE, MEM_HOST = 0, 1
FLAG_GREEDY = 1
FLAG_FULL_VOCAB = 2


class RowParams(C.Structure):
    _fields_ = [
        ("temperature", C.c_float),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("top_k", C.c_int32),
        ("repetition_penalty", C.c_float),
        ("frequency_penalty", C.c_float),
        ("presence_penalty", C.c_float),
        ("flags", C.c_uint32),
    ]


class SampleArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("memory", C.c_uint32),
        ("batch", C.c_int32),
        ("vocab", C.c_int32),
        ("logits_dtype", C.c_int32),
        ("history_stride", C.c_int32),
        ("logits_row_stride", C.c_int64),
        ("logits", C.c_void_p),
        ("mask", C.c_void_p),
        ("mask_row_stride", C.c_int64),
        ("history", C.c_void_p),
        ("history_len", C.c_void_p),
        ("row_params", C.c_void_p),
        ("params", RowParams),
        ("uniforms", C.c_void_p),
        ("out_token", C.c_void_p),
        ("out_prob", C.c_void_p),
        ("out_lse", C.c_void_p),
        ("out_status", C.c_void_p),
        ("out_kept_ids", C.c_void_p),
        ("out_kept_count", C.c_void_p),
        ("kept_stride", C.c_int32),
        ("vocab_segments", C.c_int32),
    ]


class SpecArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("memory", C.c_uint32),
        ("batch", C.c_int32),
        ("draft_len", C.c_int32),
        ("vocab", C.c_int32),
        ("target_rows", C.c_int32),
        ("target_logits", C.c_void_p),
        ("draft_logits", C.c_void_p),
        ("draft_tokens", C.c_void_p),
        ("u_accept", C.c_void_p),
        ("u_resample", C.c_void_p),
        ("temperature", C.c_float),
        ("reserved", C.c_int32),
        ("out_accept_len", C.c_void_p),
        ("out_tokens", C.c_void_p),
        ("out_status", C.c_void_p),
    ]


class ShardArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("memory", C.c_uint32),
        ("batch", C.c_int32),
        ("vocab_local", C.c_int32),
        ("logits_dtype", C.c_int32),
        ("rank", C.c_int32),
        ("nranks", C.c_int32),
        ("top_k", C.c_int32),
        ("logits_row_stride", C.c_int64),
        ("logits", C.c_void_p),
        ("temperature", C.c_float),
        ("top_p", C.c_float),
        ("uniforms", C.c_void_p),
        ("packed", C.c_void_p),
        ("gathered", C.c_void_p),
        ("out_token", C.c_void_p),
        ("out_prob", C.c_void_p),
        ("out_lse", C.c_void_p),
        ("out_status", C.c_void_p),
    ]


# name -> (restype, argtypes); every symbol declared in include/born_sampler.h
SYMBOLS = {
    "born_sampler_create": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "born_sampler_destroy": (C.c_int32, [C.c_void_p]),
    "born_sample": (C.c_int32, [C.c_void_p, C.POINTER(SampleArgs), C.c_void_p]),
    "born_sample_static": (C.c_int32, [C.POINTER(SampleArgs), C.c_void_p]),
    "born_sampler_reserve": (C.c_int32, [C.c_void_p, C.POINTER(SampleArgs)]),
    "born_check_error": (C.c_int32, [C.c_void_p]),
    "born_fallback_rows": (C.c_int64, [C.c_void_p]),
    "born_debug_expire_wait": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "born_history_create": (C.c_int32, [C.c_void_p, C.c_int32]),
    "born_history_reset": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_uint32, C.c_void_p]),
    "born_history_set_stop_tokens": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32), C.c_int32]),
    "born_history_read": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_uint32, C.c_void_p]),
    "born_sample_next": (C.c_int32, [C.c_void_p, C.POINTER(SampleArgs), C.c_void_p]),
    "born_mask_begin": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.POINTER(C.c_uint32))]),
    "born_mask_commit": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "born_mask_wait": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "born_spec_verify": (C.c_int32, [C.c_void_p, C.POINTER(SpecArgs), C.c_void_p]),
    "born_shard_record_bytes": (C.c_int32, [C.c_int32]),
    "born_shard_unique_id": (C.c_int32, [C.c_void_p]),
    "born_shard_init": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32]),
    "born_shard_local": (C.c_int32, [C.c_void_p, C.POINTER(ShardArgs), C.c_void_p]),
    "born_shard_merge": (C.c_int32, [C.c_void_p, C.POINTER(ShardArgs), C.c_void_p]),
    "born_sample_sharded": (C.c_int32, [C.c_void_p, C.POINTER(ShardArgs), C.c_void_p]),
    "born_workspace_bytes": (C.c_int64, [C.c_void_p]),
    "born_launch_count": (C.c_int64, [C.c_void_p]),
    "born_last_timing": (C.c_int32, [C.c_void_p, C.POINTER(C.c_float)]),
    "born_last_error": (C.c_char_p, [C.c_void_p]),
    "born_version": (C.c_char_p, []),
    "born_debug_exp": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "born_debug_mass": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
}

_lib = None


def load():
    """Load libborn_sampler.so and bind every symbol.  Raises if the library is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m born_b200.build` "
            "(there is no CPU fallback for the sampling path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
