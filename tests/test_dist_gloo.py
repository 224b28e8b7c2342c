"""The N>1 host logic on CPU: two gloo ranks.

Rows are partitioned without communication (batch-parallel) and vocab shards exchange one
record per row through a single all-gather (vocab-sharded).  The device kernels are not
involved: ranks build their records with the host-side record encoder, gather them with
gloo, decode them and check that sampling from the merged candidates equals the oracle's
segmented sampling of the full rows -- the property the GPU path relies on."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from born_b200 import parallel as P, workloads as W
    from oracle import born_oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, V, k = 12, 4096, 8
        z = (W.normal(5, 1, B * V) * 2.0).astype(np.float32).reshape(B, V)  # same on every rank
        u = W.uniform_f32(5, 2, B)
        params = O.make_params(temperature=1.0, top_k=k, top_p=0.95)
        want = O.sample(z, params, uniforms=u, segments=world)

        # ---- batch-parallel: own rows only, results concatenated for the check
        lo, hi = P.row_partition(B, rank, world)
        mine = O.sample(np.ascontiguousarray(z[lo:hi]), params, uniforms=u[lo:hi], segments=world)
        parts = [None] * world
        dist.all_gather_object(parts, (lo, hi, mine["token"].tolist()))
        tok = np.full(B, -9, dtype=np.int32)
        for a, b, t in parts:
            tok[a:b] = t
        assert np.array_equal(tok, want["token"])
        assert sorted((a, b) for a, b, _ in parts) == [P.row_partition(B, r, world) for r in range(world)]

        # ---- vocab-sharded: one all-gather of records, every rank merges every row
        c0, c1 = P.shard_range(V, rank, world)
        rec = torch.from_numpy(P.encode_records(z[:, c0:c1], k, idx_offset=c0))
        assert rec.shape == (B, P.record_bytes(k))
        pieces = [torch.empty_like(rec) for _ in range(world)]
        dist.all_gather(pieces, rec)  # the layout NCCL's all-gather produces: [rank, row, bytes]
        gathered = torch.stack(pieces)
        rows = P.decode_records(gathered.numpy())
        merged = np.full((B, V), -np.inf, dtype=np.float32)
        for r, d in enumerate(rows):
            assert len(d["ids"]) == world * k and d["ids"].min() >= 0 and d["ids"].max() < V
            merged[r, d["ids"]] = d["values"]
            assert np.isclose(P.merged_lse(d["parts"]), np.log(np.exp(z[r].astype(np.float64)).sum()), atol=1e-5)
        got = O.sample(merged, O.make_params(temperature=1.0, top_p=0.95), uniforms=u)
        assert np.array_equal(got["token"], want["token"])
        assert np.array_equal(got["prob"].view(np.uint32), want["prob"].view(np.uint32))
        q.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the parent
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def test_two_rank_partitions_and_record_exchange():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_partition_helpers():
    from born_b200 import parallel as P
    for B in (1, 7, 256, 1024):
        for w in (1, 2, 4, 8):
            spans = [P.row_partition(B, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
    assert P.shard_range(256000, 3, 8) == (96000, 128000)
    with pytest.raises(ValueError):
        P.shard_range(1001, 0, 8)
    z = np.array([3.5, -0.0, 0.0, -2.0, np.inf, -np.inf], dtype=np.float32)
    k = P.float_key(z)
    assert k[1] == k[2] and k[3] < k[1] < k[0] < k[4] and k[5] < k[3]
    assert np.array_equal(P.key_to_float(k)[[0, 3, 4, 5]], z[[0, 3, 4, 5]])
