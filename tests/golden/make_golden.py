"""Regenerates the committed fixtures of tests/golden/.

    python tests/golden/make_golden.py

reference_kat.json -- the known-answer vectors that the reference's own tests hold for the
    arithmetic on this path (born v0.1.1).  Inputs and tolerances are the ones in those test
    files; expected values are computed here the way those tests compute them (float64
    math.Exp on the inputs), or are the literal constants the tests state:
      softmax [1,2,3], [0,0,0]          internal/autodiff/ops/ops_test.go:651-692   (|d| <= 1e-6)
      softmax [1000,1001,1002]          internal/autodiff/ops/ops_test.go:737-775   (|d| <= 1e-5)
      -logsoftmax([2,1])[0] = 0.313     internal/nn/cross_entropy_test.go:42-57      (|d| <= 1e-2)
      softmax([1,2]) = [0.269, 0.731]   internal/nn/cross_entropy_test.go:124-142    (|d| <= 1e-2)
      argmax rows / accuracy 0.75       internal/nn/cross_entropy_test.go:146-178
      logsoftmax finite [1000,999,998]  internal/nn/cross_entropy_test.go:181-210
sampler_small.npz -- seeded small sampling cases with the outputs of the CPU oracle
    (oracle/born_oracle.c) at the time of generation.  The reference has no sampler, so
    these pin the oracle against accidental change; they are not reference outputs.
"""
import json
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from born_b200 import workloads as W  # noqa: E402
from oracle import born_oracle as O  # noqa: E402


def reference_kat():
    e = [math.exp(1.0), math.exp(2.0), math.exp(3.0)]
    s = sum(e)
    sm123 = [x / s for x in e]
    return {
        "softmax": [
            {"cite": "internal/autodiff/ops/ops_test.go:651-692", "input": [[1.0, 2.0, 3.0], [0.0, 0.0, 0.0]],
             "expected": [sm123, [1.0 / 3.0] * 3], "atol": 1e-6, "rows_sum_to_one_atol": 1e-6},
            {"cite": "internal/autodiff/ops/ops_test.go:737-775", "input": [[1000.0, 1001.0, 1002.0]],
             "expected": [sm123], "atol": 1e-5, "rows_sum_to_one_atol": 1e-5},
            {"cite": "internal/nn/cross_entropy_test.go:124-142", "input": [[1.0, 2.0]],
             "expected": [[0.269, 0.731]], "atol": 1e-2, "rows_sum_to_one_atol": 1e-5},
        ],
        "neg_logsoftmax_at": [
            {"cite": "internal/nn/cross_entropy_test.go:42-57", "input": [2.0, 1.0], "index": 0,
             "expected": 0.313, "atol": 1e-2},
        ],
        "logsoftmax_finite": [
            {"cite": "internal/nn/cross_entropy_test.go:181-210", "input": [1000.0, 999.0, 998.0], "index": 0,
             "neg_at_most": 1.0},
        ],
        "argmax": [
            {"cite": "internal/nn/cross_entropy_test.go:146-178",
             "input": [[1, 2, 3], [3, 1, 2], [2, 3, 1], [1, 1, 3]], "expected": [2, 0, 1, 2],
             "targets": [2, 0, 0, 2], "accuracy": 0.75},
        ],
    }


def small_cases():
    """A dictionary of arrays: for case i, inputs `c{i}_*` and oracle outputs `c{i}_out_*`."""
    out = {}
    specs = [
        # (V, B, dtype, params, mask?, hist, segments)
        (1, 2, "f32", dict(temperature=1.0), False, 0, 1),
        (31, 4, "f32", dict(temperature=0.8, top_k=5), False, 8, 1),
        (33, 4, "bf16", dict(temperature=1.0, top_k=4, top_p=0.9), True, 0, 1),
        (4097, 3, "f32", dict(temperature=0.7, min_p=0.05, top_p=0.9, frequency_penalty=0.5, presence_penalty=0.3), False, 64, 1),
        (5000, 4, "bf16", dict(greedy=True), True, 0, 1),
        (8192, 2, "f32", dict(temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.1), False, 64, 1),
        (8000, 3, "bf16", dict(temperature=1.0, top_k=16, top_p=0.95), False, 0, 4),
    ]
    for i, (V, B, dt, p, use_mask, H, G) in enumerate(specs):
        z = (W.normal(100 + i, 1, B * V) * 2.5).astype(np.float32).reshape(B, V)
        logits = z if dt == "f32" else W.f32_to_bf16_bits(z)
        u = W.uniform_f32(100 + i, 2, B)
        mask = None
        if use_mask:
            words = (V + 31) // 32
            bits = W.uniform(100 + i, 3, B * words * 32).reshape(B, words * 32) < 0.3
            bits[:, V:] = False
            bits[:, 0] = True
            mask = np.packbits(bits.reshape(B, words, 32), axis=-1, bitorder="little").view(np.uint32).reshape(B, words)
        hist = W.randint(100 + i, 4, B * H, V).astype(np.int32).reshape(B, H) if H else None
        r = O.sample(logits, O.make_params(**p), uniforms=u, mask=mask, history=hist, segments=G, want_kept=64)
        out[f"c{i}_logits"] = logits
        out[f"c{i}_params"] = O.make_params(**p)
        out[f"c{i}_uniforms"] = u
        out[f"c{i}_segments"] = np.int32(G)
        if mask is not None:
            out[f"c{i}_mask"] = mask
        if hist is not None:
            out[f"c{i}_history"] = hist
        for k in ("token", "prob", "lse", "status", "kept_ids", "kept_count"):
            out[f"c{i}_out_{k}"] = r[k]
    out["n_cases"] = np.int32(len(specs))
    # deterministic exp / mass on a fixed grid
    x = np.concatenate([np.linspace(-90, 0, 4097), -np.logspace(-8, 1.9, 512)]).astype(np.float32)
    out["exp_x"] = x
    out["exp_y"] = O.exp_det(x)
    out["exp_q"] = O.mass(x)
    # speculative verify, tiny
    B, K, V = 3, 4, 3000
    tgt = (W.normal(200, 1, B * (K + 1) * V) * 2.0).astype(np.float32).reshape(B, K + 1, V)
    drf = (tgt[:, :K] + (W.normal(200, 2, B * K * V) * 0.5).astype(np.float32).reshape(B, K, V)).astype(np.float32)
    ud = W.uniform_f32(200, 3, B * K).reshape(B, K)
    ua = W.uniform_f32(200, 4, B * K).reshape(B, K)
    ur = W.uniform_f32(200, 5, B * (K + 1)).reshape(B, K + 1)
    dt = O.draft_tokens(drf, ud)
    sv = O.spec_verify(tgt, drf, dt, ua, ur)
    out.update(spec_target=tgt, spec_draft=drf, spec_draft_tok=dt, spec_u_accept=ua, spec_u_resample=ur,
               spec_out_accept_len=sv["accept_len"], spec_out_tokens=sv["tokens"], spec_out_status=sv["status"])
    return out


if __name__ == "__main__":
    O.build(force=True)
    with open(os.path.join(HERE, "reference_kat.json"), "w") as f:
        json.dump(reference_kat(), f, indent=1)
    np.savez_compressed(os.path.join(HERE, "sampler_small.npz"), **small_cases())
    print("wrote", os.listdir(HERE))
