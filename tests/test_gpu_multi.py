"""Vocab-sharded sampling across real GPUs (skipped with fewer than two): every rank runs
born_sample_sharded on its column shard -- local pass, the library's own NCCL all-gather,
merge -- and must produce the tokens the oracle's segmented sampling gives for the full rows."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"  # plain peer transfers: a rank that failed would otherwise fault its peers' links
    import torch
    import torch.distributed as dist
    from born_b200 import Sampler, parallel as P, workloads as W
    from oracle import born_oracle as O
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # set-up only; the data path is the library's NCCL
    s = None
    try:
        B, V, k = 64, 64000, 16
        c = W.config5(seed=3, batch=B, vocab=V, shards=world)
        lo, hi = P.shard_range(V, rank, world)
        bits = np.ascontiguousarray(c["logits_bf16"][:, lo:hi])
        local = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)
        u = torch.from_numpy(c["uniforms"]).cuda()
        s = Sampler(device=rank, max_batch=B, max_vocab=V)
        sh = P.ShardedSampler(s, rank, world, dist)
        for _ in range(2):
            out = sh.sample(local, u, top_k=k, temperature=1.0, top_p=0.95)
            torch.cuda.synchronize()
        ref = O.sample(c["logits_bf16"], O.make_params(temperature=1.0, top_k=k, top_p=0.95), uniforms=c["uniforms"],
                       segments=world)
        assert np.array_equal(out["status"].cpu().numpy(), ref["status"])
        assert np.array_equal(out["token"].cpu().numpy(), ref["token"])
        assert np.array_equal(out["prob"].cpu().numpy().view(np.uint32), ref["prob"].view(np.uint32))
        z = W.bf16_bits_to_f32(c["logits_bf16"]).astype(np.float64)
        truth = np.log(np.exp(z - z.max(1, keepdims=True)).sum(1)) + z.max(1)
        assert np.max(np.abs(out["lse"].cpu().numpy() - truth)) <= 2e-5
        q.put((rank, "ok"))
    except Exception:
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        if s is not None:
            s.close()  # (also on a failed assertion: the communicator is destroyed between steps, nothing in flight)
        dist.destroy_process_group()


def test_sharded_sampling_on_all_visible_gpus():
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
