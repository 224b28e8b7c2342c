#!/usr/bin/env python
"""Benchmark of the sampling hot path: sampled rows/s and achieved HBM GB/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the fused sampling kernel over one batch of synthetic logits.  The
default workload is the batched-decode recipe (fp32 N(0, 3^2) + Zipf-shaped bias,
temperature 0.7, min-p 0.05, top-p 0.9, frequency 0.5 / presence 0.3 over 512 prior ids)
at the headline shape batch 256 x vocab 128256.  With N GPUs every rank samples its own
batch (batch-parallel, no communication): weak scaling.  `--workload c5_sharded` runs the
vocab-sharded path instead (local top-k + one NCCL all-gather + merge).

`value` is device-resident throughput (inputs already in HBM, CUDA events on the launching
stream, max over ranks); `e2e` is the same metric through the host-memory C-ABI call
(pinned host buffers, host<->device copies inside the timed region).  Between timed
iterations the kernel reads a different one of several logits buffers whose total size
exceeds L2, so no launch finds its input cached.  `--impl reference` times the CPU oracle
(the reference's sequential algorithm restated in C, one thread per core over rows) on
this box's host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "sampled_rows_per_s"
UNIT = "rows/s"

WORKLOADS = {
    # name: (batch, vocab, dtype, history, description)
    "c2_batched_decode_b256": dict(B=256, V=128256, dtype="f32", H=512, mask=False,
                                   params=dict(temperature=0.7, min_p=0.05, top_p=0.9, frequency_penalty=0.5,
                                               presence_penalty=0.3)),
    "c2_batched_decode_b64": dict(B=64, V=128256, dtype="f32", H=512, mask=False,
                                  params=dict(temperature=0.7, min_p=0.05, top_p=0.9, frequency_penalty=0.5,
                                              presence_penalty=0.3)),
    "headline_topk_b256": dict(B=256, V=128256, dtype="f32", H=0, mask=False,
                               params=dict(temperature=0.7, top_k=50, top_p=0.9)),
    # nothing narrows the row: the two-pass route over the whole vocabulary
    "temperature_only_b256": dict(B=256, V=128256, dtype="f32", H=0, mask=False, params=dict(temperature=0.8)),
    # top-p without top-k: two whole-vocabulary passes for the survivor total, then the one-pass kernel
    "top_p_only_b256": dict(B=256, V=128256, dtype="f32", H=0, mask=False, params=dict(temperature=0.7, top_p=0.9)),
    "c3_constrained_b256": dict(B=256, V=151936, dtype="bf16", H=0, mask=True, params=None),
    "c5_sharded": dict(B=1024, V=256000, dtype="bf16", H=0, mask=False,
                       params=dict(temperature=1.0, top_k=64, top_p=0.95)),
    # speculative verification: 32 sequences x 5 draft positions (+ bonus row); metric is its own
    "c4_spec_verify": dict(B=32, V=128256, dtype="f32", H=0, mask=False, K=5, params=None),
}


def algorithmic_bytes_per_row(w, V=None):
    V = V or w["V"]
    esz = 4 if w["dtype"] == "f32" else 2
    b = V * esz + 4 * w["H"] + 4 + 8
    if w["mask"]:
        b += 4 * ((V + 31) // 32)
    return b


class ClockSampler(threading.Thread):
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.stop_flag = False

    def run(self):
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                for line in out.strip().splitlines():
                    f = [x.strip() for x in line.split(",")]
                    if len(f) >= 9:
                        self.samples.append(f)
            except Exception:
                pass
            time.sleep(0.1)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no nvidia-smi samples"]}
        sm = sorted(float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit())
        mx = max(float(s[2]) for s in self.samples if s[2].replace(".", "").isdigit())
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            for n, v in zip(names, s[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(self.samples)}


def make_inputs(torch, w, seed, device, nbuf):
    """Seeded synthetic inputs on the device (stand-ins with the configuration's shapes and value
    distributions).  Returns a list of nbuf input dicts that differ in their logits."""
    B, V = w["B"], w["V"]
    g = torch.Generator(device=device).manual_seed(seed)
    bufs = []
    for i in range(nbuf):
        if w["dtype"] == "f32":
            z = torch.randn((B, V), generator=g, device=device) * 3.0
            perm_rank = torch.argsort(torch.rand((B, V), generator=g, device=device), dim=1).float()
            z -= 1.1 * torch.log(perm_rank + 1.0)
            del perm_rank
        elif w["mask"]:
            z = (torch.randn((B, V), generator=g, device=device) * 2.5).to(torch.bfloat16)
        else:
            z = torch.randn((B, V), generator=g, device=device) * 2.0
            z += 6.0 * (torch.rand((B, V), generator=g, device=device) < 0.01)
            z = z.to(torch.bfloat16)
        bufs.append({"logits": z.contiguous()})
    common = {"uniforms": torch.rand(B, generator=g, device=device).clamp_(max=1.0 - 2.0 ** -24)}
    if w["H"]:
        common["history"] = torch.randint(0, V, (B, w["H"]), generator=g, device=device, dtype=torch.int32)
    if w["mask"]:
        words = (V + 31) // 32
        bits = torch.rand((B, words * 32), generator=g, device=device) < 0.05
        bits[:, V:] = False
        bits[:, 0] |= ~bits.any(dim=1)
        weights = (2 ** torch.arange(32, device=device, dtype=torch.int64))
        mask64 = (bits.view(B, words, 32).to(torch.int64) * weights).sum(-1)
        common["mask"] = torch.where(mask64 >= 2 ** 31, mask64 - 2 ** 32, mask64).to(torch.int32).contiguous()
    for b in bufs:
        b.update(common)
    return bufs


def row_params_for(w):
    from born_b200 import SamplingConfig
    from born_b200.sampler import row_params_array
    if w["params"] is not None:
        return SamplingConfig(**w["params"]), None
    rows = [SamplingConfig(greedy=True) if b % 2 == 0 else SamplingConfig(temperature=1.0, top_k=50)
            for b in range(w["B"])]
    return None, row_params_array(rows)


def oracle_params_for(w):
    from oracle import born_oracle as O
    if w["params"] is not None:
        return O.make_params(**w["params"])
    return O.params_from_rows([dict(greedy=True) if b % 2 == 0 else dict(temperature=1.0, top_k=50)
                               for b in range(w["B"])])


def host_copy(torch, buf):
    """numpy views of one input set (bf16 as uint16 bit patterns) for the oracle."""
    out = {}
    z = buf["logits"]
    out["logits"] = (z.view(torch.int16).cpu().numpy().view(np.uint16) if z.dtype == torch.bfloat16
                     else z.cpu().numpy())
    out["uniforms"] = buf["uniforms"].cpu().numpy()
    out["history"] = buf["history"].cpu().numpy() if "history" in buf else None
    out["mask"] = buf["mask"].cpu().numpy().view(np.uint32) if "mask" in buf else None
    return out


def run_reference(args, w, name):
    """CPU arm: the oracle on host cores, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from born_b200 import workloads as W
    from oracle import born_oracle as O
    O.build()
    cores = os.cpu_count() or 1
    B, V = w["B"], w["V"]
    rows = min(B, max(cores, 64))  # bounded sample of the workload
    z = (W.normal(0, 10, rows * V) * 3.0).astype(np.float32).reshape(rows, V)
    if w["dtype"] == "f32":
        bias = -1.1 * np.log(np.arange(1, V + 1, dtype=np.float64))
        for b in range(rows):
            perm = np.argsort(W.raw_u64(0, 1000 + b, V), kind="stable")
            z[b, perm] += bias.astype(np.float32)
        logits = z
    else:
        logits = W.f32_to_bf16_bits(z)
    u = W.uniform_f32(0, 12, rows)
    hist = W.randint(0, 11, rows * w["H"], V).astype(np.int32).reshape(rows, w["H"]) if w["H"] else None
    mask = None
    if w["mask"]:
        words = (V + 31) // 32
        bits = W.uniform(0, 21, rows * words * 32).reshape(rows, words * 32) < 0.05
        bits[:, V:] = False
        bits[:, 0] = True
        mask = np.packbits(bits.reshape(rows, words, 32), axis=-1, bitorder="little").view(np.uint32).reshape(rows, words)
    params = oracle_params_for(w)
    if params.size > 1:
        params = params[:rows]
    seg = 8 if name == "c5_sharded" else 1

    def step():
        O.sample(logits, params, uniforms=u, mask=mask, history=hist, segments=seg, nthreads=cores)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = rows * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": name, "batch": B, "vocab": V, "sample_rows_per_step": rows},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{rows} rows of the workload per step, {args.steps} steps, {cores} threads over rows"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_spec(args, w, name):
    """Speculative verification (born_spec_verify): one step verifies B sequences of K draft
    tokens against K+1 target rows.  Every rank verifies its own batch (no communication)."""
    import torch
    import torch.distributed as dist
    from born_b200 import Sampler, build
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampling path has no CPU fallback")
    build.build()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    B, V, K = w["B"], w["V"], w["K"]
    nbuf = 1 if args.small else 3
    g = torch.Generator(device=device).manual_seed(4321 + rank)
    sets = []
    for _ in range(nbuf):
        tgt = torch.randn((B, K + 1, V), generator=g, device=device) * 2.0
        drf = (tgt[:, :K, :] + 0.5 * torch.randn((B, K, V), generator=g, device=device)).contiguous()
        tok = torch.multinomial(torch.softmax(drf.view(B * K, V), dim=-1), 1, generator=g).view(B, K).to(torch.int32)
        sets.append(dict(target=tgt, draft=drf, tok=tok.contiguous(),
                         ua=torch.rand((B, K), generator=g, device=device),
                         ur=torch.rand((B, K + 1), generator=g, device=device).clamp_(max=1.0 - 2.0 ** -24)))
    sampler = Sampler(device=local, max_batch=B, max_vocab=V)
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream

    def step(i):
        s_ = sets[i % nbuf]
        return sampler.spec_verify(s_["target"], s_["draft"], s_["tok"], s_["ua"], s_["ur"], stream=sp)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    clocks = ClockSampler(local)
    clocks.start()
    l0 = sampler.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = sampler.launch_count - l0
    t_end = time.time() + 0.6
    i = 0
    while time.time() < t_end:
        step(i)
        i += 1
        if i % 16 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    clocks.stop_flag = True
    clocks.join(timeout=3)
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    if rank == 0:
        from oracle import born_oracle as O
        O.build()
        res = step(0)
        torch.cuda.synchronize()
        nchk = min(B, 8)
        s0 = sets[0]
        ref = O.spec_verify(s0["target"][:nchk].cpu().numpy(), s0["draft"][:nchk].cpu().numpy(),
                            s0["tok"][:nchk].cpu().numpy(), s0["ua"][:nchk].cpu().numpy(),
                            s0["ur"][:nchk].cpu().numpy(), nthreads=os.cpu_count() or 1)
        alen = res["accept_len"][:nchk].cpu().numpy()
        toks = res["tokens"][:nchk].cpu().numpy()
        mism = 0
        for b in range(nchk):
            n = int(ref["accept_len"][b]) + 1
            mism += int(alen[b] != ref["accept_len"][b]) + int((toks[b, :n] != ref["tokens"][b, :n]).any())
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            hs = {k: v[:nchk].cpu().numpy() for k, v in s0.items()}
            t0 = time.perf_counter()
            reps = 0
            while time.perf_counter() - t0 < 10.0:
                O.spec_verify(hs["target"], hs["draft"], hs["tok"], hs["ua"], hs["ur"], nthreads=cores)
                reps += 1
            dt = time.perf_counter() - t0
            cpu = {"value": nchk * reps / dt, "unit": "sequences/s", "cores": cores, "kind": "port",
                   "sample": f"{nchk} sequences of the workload x {reps} passes, {cores} threads over sequences"}
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        bytes_launch = B * (2 * K + 1) * V * 4
        kernel_ms = ms / args.steps
        achieved = bytes_launch / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": "spec_verified_sequences_per_s", "value": B * args.steps * world / (ms * 1e-3),
            "unit": "sequences/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": kernel_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "batch_per_gpu": B, "draft_len": K, "vocab": V,
                       "parallelism": "batch-parallel x%d" % world,
                       "l2": f"{nbuf} rotating input sets, {nbuf * bytes_launch / 1e6:.0f} MB > L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": "measured" if peaks else "fallback",
                         "algorithmic_bytes_per_launch": bytes_launch, "frac_of_8TBs": achieved / 8000.0},
            "cpu_baseline": cpu, "e2e": None, "gpu_launches": int(launches), "clocks": clocks.summary(),
            "parity": {"sequences_checked": nchk, "mismatches": mism},
        }
        print(json.dumps(line), flush=True)
    sampler.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", default="c2_batched_decode_b256", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="born_b200", choices=["born_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--small", action="store_true", help="one input buffer, for profiler captures")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    name = args.workload
    if args.impl == "reference":
        if name == "c4_spec_verify":
            raise SystemExit("--impl reference times the sampling workloads; c4_spec_verify reports its own cpu_baseline")
        args.steps = args.steps or 5
        args.warmup = 1 if args.warmup is None else args.warmup
        return run_reference(args, w, name)
    args.steps = args.steps or 200
    args.warmup = 20 if args.warmup is None else args.warmup
    if name == "c4_spec_verify":
        return run_spec(args, w, name)

    import torch
    import torch.distributed as dist
    from born_b200 import Sampler, build

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampling path has no CPU fallback")
    build.build()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    sharded = name == "c5_sharded" and world > 1
    B, V = w["B"], w["V"]
    V_local = V // world if sharded else V

    nbuf = 1 if args.small else max(2, int(np.ceil(400e6 / (B * V_local * (4 if w["dtype"] == "f32" else 2)))) + 1)
    wl = dict(w)
    if sharded:
        wl["V"] = V_local
    bufs = make_inputs(torch, wl, seed=1234 + (0 if sharded else rank), device=device, nbuf=nbuf)
    if sharded:  # uniforms must be identical on every rank
        dist.broadcast(bufs[0]["uniforms"], src=0)
    # the one-GPU form of the sharded workload cuts every row into 8 vocab segments (8 records a row)
    sampler = Sampler(device=local, max_batch=B * (2 if name == "c5_sharded" and not sharded else 1),
                      max_vocab=max(V_local, 1024))
    cfg, rp = row_params_for(w)
    rp_dev = torch.from_numpy(rp.view(np.uint8)).to(device) if rp is not None else None
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream
    if sharded:
        uid = [Sampler.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        sampler.shard_init(uid[0], rank, world)
    out = {}

    def step(i):
        b = bufs[i % nbuf]
        if sharded:
            sampler.sample_sharded(b["logits"], b["uniforms"], rank, world, w["params"]["top_k"],
                                   temperature=w["params"]["temperature"], top_p=w["params"]["top_p"], stream=sp, out=out)
        else:
            sampler.sample(b["logits"], uniforms=b["uniforms"], config=cfg, row_params=rp_dev, mask=b.get("mask"),
                           history=b.get("history"), want_prob=True, want_lse=True, stream=sp, out=out,
                           vocab_segments=8 if name == "c5_sharded" else 0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    clocks = ClockSampler(local)
    clocks.start()
    l0 = sampler.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = sampler.launch_count - l0
    # keep the GPU under the same load a little longer so that the clock sampler sees it
    t_end = time.time() + 0.6
    i = 0
    while time.time() < t_end:
        step(i)
        i += 1
        if i % 64 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    clocks.stop_flag = True
    clocks.join(timeout=3)
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    rows_total = B * args.steps * (1 if sharded else world)
    value = rows_total / (ms * 1e-3)

    # ---- end to end through the host-memory call (pinned host buffers) ----
    e2e = None
    if not args.no_e2e and not sharded:
        hb = {k: (v.cpu().pin_memory() if hasattr(v, "cpu") else v) for k, v in bufs[0].items()}
        hrp = rp
        hout = {}
        esteps = max(3, min(args.steps, 20))

        def estep():
            sampler.sample(hb["logits"], uniforms=hb["uniforms"], config=cfg, row_params=hrp, mask=hb.get("mask"),
                           history=hb.get("history"), want_prob=True, want_lse=True, stream=sp, out=hout,
                           vocab_segments=8 if name == "c5_sharded" else 0)
        for _ in range(3):
            estep()
        barrier()
        e0.record(stream)
        t0 = time.perf_counter()
        for _ in range(esteps):
            estep()
        e1.record(stream)
        barrier()
        wall = time.perf_counter() - t0
        ems = max(e0.elapsed_time(e1), wall * 1e3)
        te = torch.tensor([ems], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        h2d = sum(v.numel() * v.element_size() for k, v in hb.items() if hasattr(v, "numel"))
        if hrp is not None:
            h2d += hrp.nbytes
        d2h = sum(v.nbytes for v in hout.values())
        e2e = {"value": B * esteps * world / (float(te.item()) * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "steps": esteps, "split_ms": sampler.last_timing_ms()}

    # ---- parity spot-check and CPU baseline (rank 0, N == 1 only for the timing) ----
    parity = None
    cpu = None
    if rank == 0 and not sharded:
        from oracle import born_oracle as O
        O.build()
        hc = host_copy(torch, bufs[0])
        nchk = min(B, 32)
        step(0)
        torch.cuda.synchronize()
        params = oracle_params_for(w)
        pr = params if params.size == 1 else params[:nchk]
        ref = O.sample(np.ascontiguousarray(hc["logits"][:nchk]), pr, uniforms=hc["uniforms"][:nchk],
                       mask=None if hc["mask"] is None else np.ascontiguousarray(hc["mask"][:nchk]),
                       history=None if hc["history"] is None else np.ascontiguousarray(hc["history"][:nchk]),
                       segments=8 if name == "c5_sharded" else 1, nthreads=os.cpu_count() or 1)
        tok = out["token"][:nchk].cpu().numpy()
        prob = out["prob"][:nchk].cpu().numpy()
        lse = out["lse"][:nchk].cpu().numpy()
        parity = {"rows_checked": nchk, "token_mismatches": int((tok != ref["token"]).sum()),
                  "prob_bit_mismatches": int((prob.view(np.uint32) != ref["prob"].view(np.uint32)).sum()),
                  "max_abs_lse_diff_vs_sequential_f32": float(np.nanmax(np.abs(lse - ref["lse"]))),
                  "near_cutoff_rows": int((ref["near_cutoff"] != 0).sum()),
                  "row_status_nonzero": int((out["status"].cpu().numpy() != 0).sum())}
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            nrows = min(B, max(cores, 64))
            lg = np.ascontiguousarray(hc["logits"][:nrows])
            pr = params if params.size == 1 else params[:nrows]
            kw = dict(uniforms=hc["uniforms"][:nrows],
                      mask=None if hc["mask"] is None else np.ascontiguousarray(hc["mask"][:nrows]),
                      history=None if hc["history"] is None else np.ascontiguousarray(hc["history"][:nrows]),
                      segments=8 if name == "c5_sharded" else 1)
            O.sample(lg, pr, nthreads=cores, **kw)
            t0 = time.perf_counter()
            reps = 0
            while time.perf_counter() - t0 < 10.0:
                O.sample(lg, pr, nthreads=cores, **kw)
                reps += 1
            dt = time.perf_counter() - t0
            t1 = time.perf_counter()
            O.sample(lg[:8], pr if pr.size == 1 else pr[:8], nthreads=1,
                     **{k: (None if v is None else v[:8]) if k != "segments" else v for k, v in kw.items()})
            single = 8 / (time.perf_counter() - t1)
            cpu = {"value": nrows * reps / dt, "unit": UNIT, "cores": cores, "kind": "port",
                   "sample": f"{nrows} rows of the workload x {reps} passes, {cores} threads over rows",
                   "single_thread_rows_per_s": single}

    if rank == 0:
        bytes_launch = algorithmic_bytes_per_row(w, V_local) * B
        kernel_ms = ms / args.steps
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        achieved = bytes_launch / (kernel_ms * 1e-3) / 1e9
        traffic = None
        try:
            with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
                traffic = json.load(f).get(name)
        except Exception:
            pass
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": kernel_ms, "higher_is_better": True,
            "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": name, "batch_per_gpu": B, "vocab": V, "vocab_per_gpu": V_local,
                       "parallelism": ("vocab-sharded x%d (NCCL all-gather)" % world) if sharded else "batch-parallel x%d" % world,
                       "l2": f"{nbuf} rotating input buffers, {nbuf * B * V_local * (4 if w['dtype'] == 'f32' else 2) / 1e6:.0f} MB > L2",
                       "outputs": "token, prob, lse, status"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": "measured" if peaks else "fallback",
                         "algorithmic_bytes_per_launch": bytes_launch, "frac_of_8TBs": achieved / 8000.0},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks.summary(),
            "parity": parity,
        }
        print(json.dumps(line), flush=True)
    sampler.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
