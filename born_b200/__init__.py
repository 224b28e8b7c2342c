"""born_b200 -- B200-native token sampling / constrained decoding for born.

The product is libborn_sampler.so (hand-written sm_100a CUDA behind a C ABI, see
include/born_sampler.h).  This package is the thin host-side mirror used by the tests and
the benchmark: ctypes structs (`_lib`), a `Sampler` object with the reference's idioms
(`sampler`), and the synthetic workloads of the benchmark configurations (`workloads`).
There is no CPU fallback: without the built library or without a CUDA device every call
raises.
"""
from .sampler import (  # noqa: F401
    SamplingConfig,
    Sampler,
    SamplerError,
    InvalidArgument,
    load_library,
    version,
)
