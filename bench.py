#!/usr/bin/env python
"""Benchmark of the sampling hot path: sampled rows/s and achieved HBM GB/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the sampling kernel over one batch of synthetic logits.  The default
workload is the batched-decode recipe (fp32 N(0, 3^2) + Zipf-shaped bias, temperature 0.7,
min-p 0.05, top-p 0.9, frequency 0.5 / presence 0.3 over 512 prior ids) at the headline shape
batch 256 x vocab 128256.  With N GPUs every rank samples its own batch (batch-parallel, no
communication): weak scaling.

`value` is device-resident throughput: inputs already in HBM, the K timed steps recorded
once into a CUDA graph and replayed between two CUDA events on the launching stream, so that
the figure does not depend on how fast the host issues launches; max over ranks.  Between
timed steps the kernel reads a different one of several logits buffers whose total size
exceeds L2.  `e2e` is the same metric through the host-memory C-ABI call (pinned host
buffers, host<->device copies inside the timed region).  `workloads` holds the other
workloads of the same library (top-k, temperature-only, top-p alone, constrained bf16,
speculative verification; with N > 1 the vocab-sharded path over NCCL), each with its own
time, roofline fraction and a parity block against the CPU oracle over every row.
`--impl reference` times the CPU oracle (the reference's sequential algorithm restated in C,
one thread per core over rows) on the same rows from the same generator.
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
DEFAULT = "c2_batched_decode_b256"

PEN = dict(frequency_penalty=0.5, presence_penalty=0.3)
WORKLOADS = {
    "c2_batched_decode_b256": dict(B=256, V=128256, dtype="f32", H=512, mask=False,
                                   params=dict(temperature=0.7, min_p=0.05, top_p=0.9, **PEN)),
    "c2_batched_decode_b64": dict(B=64, V=128256, dtype="f32", H=512, mask=False,
                                  params=dict(temperature=0.7, min_p=0.05, top_p=0.9, **PEN)),
    "headline_topk_b256": dict(B=256, V=128256, dtype="f32", H=0, mask=False,
                               params=dict(temperature=0.7, top_k=50, top_p=0.9)),
    "temperature_only_b256": dict(B=256, V=128256, dtype="f32", H=0, mask=False, params=dict(temperature=0.8)),
    "top_p_only_b256": dict(B=256, V=128256, dtype="f32", H=0, mask=False, params=dict(temperature=0.7, top_p=0.9)),
    "c3_constrained_b256": dict(B=256, V=151936, dtype="bf16", H=0, mask=True, params=None),
    "c5_sharded": dict(B=1024, V=256000, dtype="bf16", H=0, mask=False,
                       params=dict(temperature=1.0, top_k=64, top_p=0.95)),
    "c4_spec_verify": dict(B=32, V=128256, dtype="f32", H=0, mask=False, K=5, params=None),
}
EXTRA_N1 = ["headline_topk_b256", "temperature_only_b256", "top_p_only_b256", "c3_constrained_b256",
            "c2_batched_decode_b64", "c4_spec_verify"]


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


def read_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except Exception:
        return {}


def roofline(bytes_launch, kernel_ms, name):
    peaks = read_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = bytes_launch / (kernel_ms * 1e-3) / 1e9
    traffic = None
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            traffic = json.load(f).get(name)
    except Exception:
        pass
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": traffic, "peak_source": "measured" if peaks else "fallback",
            "algorithmic_bytes_per_launch": bytes_launch, "frac_of_8TBs": achieved / 8000.0}


def timed_steps(torch, stream, calls, steps, warmup, barrier):
    """Runs warmup steps, then times `steps` steps (calls[i % len(calls)]) between two CUDA events.
    The timed steps are captured once into a CUDA graph and replayed, so the device never waits
    for the host; when capture is not possible they are issued directly.  Returns (ms, how)."""
    n = len(calls)
    sp = stream.cuda_stream
    for i in range(warmup):
        calls[i % n](sp)
    barrier()
    graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            csp = torch.cuda.current_stream().cuda_stream
            for i in range(steps):
                calls[i % n](csp)
        graph.replay()  # one untimed replay: the graph's own first-launch cost
        torch.cuda.synchronize()
    except Exception as e:  # pragma: no cover - capture refused
        sys.stderr.write(f"bench: CUDA graph capture failed ({e!r}); timing direct launches\n")
        graph = None
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    if graph is not None:
        graph.replay()
    else:
        for i in range(steps):
            calls[i % n](sp)
    e1.record(stream)
    barrier()
    return e0.elapsed_time(e1), ("cuda-graph of %d steps" % steps) if graph is not None else "direct launches"


def parity_block(torch, w, name, buf, out, segments=1):
    """GPU outputs of one step on `buf` against the CPU oracle over every row."""
    from oracle import born_oracle as O
    O.build()
    hc = host_copy(torch, buf)
    params = oracle_params_for(w)
    ref = O.sample(hc["logits"], params, uniforms=hc["uniforms"], mask=hc["mask"], history=hc["history"],
                   segments=segments, nthreads=os.cpu_count() or 1)
    tok = out["token"].cpu().numpy()
    prob = out["prob"].cpu().numpy()
    st = out["status"].cpu().numpy()
    res = {"rows_checked": int(tok.size), "token_mismatches": int((tok != ref["token"]).sum()),
           "prob_bit_mismatches": int((prob.view(np.uint32) != ref["prob"].view(np.uint32)).sum()),
           "status_mismatches": int((st != ref["status"]).sum()),
           "near_cutoff_rows": int((ref["near_cutoff"] != 0).sum()),
           "row_status_nonzero": int((st != 0).sum())}
    if "lse" in out:
        lse = out["lse"].cpu().numpy()
        ok = ref["status"] == 0
        res["max_abs_lse_diff_vs_sequential_f32"] = float(np.nanmax(np.abs(lse[ok] - ref["lse"][ok]))) if ok.any() else 0.0
    return res


def run_sampling_workload(torch, dist, sampler, name, w, rank, world, device, steps, warmup, small, barrier):
    """Times one batch-parallel sampling workload; returns a dict with everything the caller reports."""
    B, V = w["B"], w["V"]
    esz = 4 if w["dtype"] == "f32" else 2
    nbuf = 1 if small else max(2, int(np.ceil(400e6 / (B * V * esz))) + 1)
    bufs = make_inputs(torch, w, seed=1234 + rank, device=device, nbuf=nbuf)
    cfg, rp = row_params_for(w)
    rp_dev = torch.from_numpy(rp.view(np.uint8)).to(device) if rp is not None else None
    stream = torch.cuda.current_stream()
    out = {}
    kw = dict(uniforms=bufs[0]["uniforms"], config=cfg, row_params=rp_dev, mask=bufs[0].get("mask"),
              history=bufs[0].get("history"), want_prob=True, want_lse=True, out=out)
    sampler.reserve(bufs[0]["logits"], **kw)
    prepared = [sampler.prepare(b["logits"], **kw) for b in bufs]
    calls = [p.run for p in prepared]
    l0 = sampler.launch_count
    calls[0](stream.cuda_stream)
    per_step = sampler.launch_count - l0
    ms, how = timed_steps(torch, stream, calls, steps, warmup, barrier)
    sampler.check_error()
    fb = sampler.fallback_rows
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    res = {"ms_per_step": ms / steps, "launches_per_step": int(per_step), "timing": how, "nbuf": nbuf,
           "bytes_launch": algorithmic_bytes_per_row(w) * B, "bufs": bufs, "out": out, "prepared": prepared,
           "cfg": cfg, "rp": rp, "fallback_rows_in_timed_steps": fb}
    if rank == 0:
        calls[0](stream.cuda_stream)
        torch.cuda.synchronize()
        res["parity"] = parity_block(torch, w, name, bufs[0], out)
    return res


def run_spec_workload(torch, dist, sampler, w, rank, world, device, steps, warmup, small, barrier, cpu_baseline):
    """Speculative verification (born_spec_verify): one step verifies B sequences of K draft tokens."""
    B, V, K = w["B"], w["V"], w["K"]
    nbuf = 1 if small else 3
    g = torch.Generator(device=device).manual_seed(4321 + rank)
    sets = []
    for _ in range(nbuf):
        tgt = torch.randn((B, K + 1, V), generator=g, device=device) * 2.0
        drf = (tgt[:, :K, :] + 0.5 * torch.randn((B, K, V), generator=g, device=device)).contiguous()
        tok = torch.multinomial(torch.softmax(drf.view(B * K, V), dim=-1), 1, generator=g).view(B, K).to(torch.int32)
        sets.append(dict(target=tgt, draft=drf, tok=tok.contiguous(),
                         ua=torch.rand((B, K), generator=g, device=device),
                         ur=torch.rand((B, K + 1), generator=g, device=device).clamp_(max=1.0 - 2.0 ** -24)))
    stream = torch.cuda.current_stream()
    holder = {}

    def mk(s_):
        def call(sp):
            holder["res"] = sampler.spec_verify(s_["target"], s_["draft"], s_["tok"], s_["ua"], s_["ur"], stream=sp)
        return call
    calls = [mk(s_) for s_ in sets]
    l0 = sampler.launch_count
    calls[0](stream.cuda_stream)
    per_step = sampler.launch_count - l0
    # (spec_verify allocates its outputs per call: direct launches, no graph)
    for i in range(warmup):
        calls[i % nbuf](stream.cuda_stream)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        calls[i % nbuf](stream.cuda_stream)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    res = {"ms_per_step": ms / steps, "launches_per_step": int(per_step), "timing": "direct launches",
           "bytes_launch": B * (2 * K + 1) * V * 4, "sequences": B}
    if rank == 0:
        from oracle import born_oracle as O
        O.build()
        calls[0](stream.cuda_stream)
        torch.cuda.synchronize()
        r = holder["res"]
        s0 = sets[0]
        hs = {k: v.cpu().numpy() for k, v in s0.items()}
        ref = O.spec_verify(hs["target"], hs["draft"], hs["tok"], hs["ua"], hs["ur"], nthreads=os.cpu_count() or 1)
        alen = r["accept_len"].cpu().numpy()
        toks = r["tokens"].cpu().numpy()
        mism = 0
        for b in range(B):
            n = int(ref["accept_len"][b]) + 1
            mism += int(alen[b] != ref["accept_len"][b]) + int((toks[b, :n] != ref["tokens"][b, :n]).any())
        res["parity"] = {"sequences_checked": B, "mismatches": mism}
        if cpu_baseline:
            cores = os.cpu_count() or 1
            t0 = time.perf_counter()
            reps = 0
            while time.perf_counter() - t0 < 5.0:
                O.spec_verify(hs["target"], hs["draft"], hs["tok"], hs["ua"], hs["ur"], nthreads=cores)
                reps += 1
            dt = time.perf_counter() - t0
            res["cpu_baseline"] = {"value": B * reps / dt, "unit": "sequences/s", "cores": cores, "kind": "port",
                                   "sample": f"all {B} sequences of the workload x {reps} passes, {cores} threads over sequences"}
    return res


def run_sharded(torch, dist, sampler, w, rank, world, device, steps, warmup, barrier):
    """Vocab-sharded sampling (local top-k -> NCCL all-gather -> merge) over all ranks, with a
    parity block against the oracle's segmented sampling over every row."""
    from born_b200 import Sampler
    B, V = w["B"], w["V"]
    Vl = V // world
    wl = dict(w)
    wl["V"] = Vl
    esz = 2
    nbuf = max(2, int(np.ceil(400e6 / (B * Vl * esz))) + 1)
    bufs = make_inputs(torch, wl, seed=977 + rank, device=device, nbuf=nbuf)
    dist.broadcast(bufs[0]["uniforms"], src=0)
    uid = [Sampler.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    sampler.shard_init(uid[0], rank, world)
    out = {}
    stream = torch.cuda.current_stream()
    p = w["params"]

    def mk(b):
        def call(sp):
            sampler.sample_sharded(b["logits"], bufs[0]["uniforms"], rank, world, p["top_k"],
                                   temperature=p["temperature"], top_p=p["top_p"], stream=sp, out=out)
        return call
    calls = [mk(b) for b in bufs]
    l0 = sampler.launch_count
    calls[0](stream.cuda_stream)
    per_step = sampler.launch_count - l0
    torch.cuda.synchronize()
    for i in range(warmup):
        calls[i % nbuf](stream.cuda_stream)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        calls[i % nbuf](stream.cuda_stream)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    # parity: rank 0 gathers the shards of buffer 0 once, outside the timed region
    calls[0](stream.cuda_stream)
    torch.cuda.synchronize()
    shard = bufs[0]["logits"].contiguous().view(torch.uint8)  # (bytes: the collective takes no 16-bit integer type)
    gathered = [torch.empty_like(shard) for _ in range(world)] if rank == 0 else None
    dist.gather(shard, gathered, dst=0)
    toks = [torch.empty_like(out["token"]) for _ in range(world)] if rank == 0 else None
    dist.gather(out["token"], toks, dst=0)
    res = None
    if rank == 0:
        from oracle import born_oracle as O
        O.build()
        full = torch.cat([g.view(torch.int16) for g in gathered], dim=1).cpu().numpy().view(np.uint16)
        u = bufs[0]["uniforms"].cpu().numpy()
        ref = O.sample(np.ascontiguousarray(full), O.make_params(**p), uniforms=u, segments=world,
                       nthreads=os.cpu_count() or 1)
        tok = out["token"].cpu().numpy()
        prob = out["prob"].cpu().numpy()
        st = out["status"].cpu().numpy()
        same = all(bool((tk == toks[0]).all().item()) for tk in toks)
        kernel_ms = ms / steps
        bytes_gpu = Vl * esz * B
        res = {"workload": "c5_sharded", "ms_per_step": kernel_ms, "rows_per_s": B / (kernel_ms * 1e-3),
               "launches_per_step": int(per_step), "collective": "one ncclAllGather of %d bytes per rank" % (B * (32 + 8 * p["top_k"])),
               "vocab_per_gpu": Vl, "roofline_per_gpu": roofline(bytes_gpu, kernel_ms, "c5_sharded"),
               "parity": {"rows_checked": int(B), "token_mismatches": int((tok != ref["token"]).sum()),
                          "prob_bit_mismatches": int((prob.view(np.uint32) != ref["prob"].view(np.uint32)).sum()),
                          "status_mismatches": int((st != ref["status"]).sum()),
                          "all_ranks_agree": bool(same)}}
    return res


def reference_inputs(w, rows):
    """The first `rows` rows of the GPU arm's first input buffer (same generator, same seed): made
    on the GPU when there is one, so that both arms see identical rows."""
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl reference needs the GPU box: it samples the rows the GPU arm samples")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    buf = make_inputs(torch, w, seed=1234, device=device, nbuf=1)[0]
    hc = host_copy(torch, buf)
    return {k: (None if v is None else np.ascontiguousarray(v[:rows])) for k, v in hc.items()}


def run_reference(args, w, name):
    """CPU arm: the oracle on host cores, rank 0 only, on the rows the GPU arm samples."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import born_oracle as O
    O.build()
    cores = os.cpu_count() or 1
    B, V = w["B"], w["V"]
    hc = reference_inputs(w, B)
    params = oracle_params_for(w)
    seg = 8 if name == "c5_sharded" else 1

    def step():
        O.sample(hc["logits"], params, uniforms=hc["uniforms"], mask=hc["mask"], history=hc["history"], segments=seg,
                 nthreads=cores)

    for _ in range(args.warmup):
        step()
    # at least `steps` steps and at least 3 s of CPU work
    t0 = time.perf_counter()
    n = 0
    while n < args.steps or time.perf_counter() - t0 < 3.0:
        step()
        n += 1
    dt = time.perf_counter() - t0
    val = B * n / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": n,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / n, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": name, "batch_per_gpu": B, "vocab": V, "same_rows_as_gpu_arm": True},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"all {B} rows of the workload per step, {n} steps, {cores} threads over rows"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="born_b200", choices=["born_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the other workloads of the `workloads` key")
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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = Sampler(device=local, max_batch=1024, max_vocab=262144)
    stream = torch.cuda.current_stream()
    clocks = ClockSampler(local)
    clocks.start()
    spec = name == "c4_spec_verify"
    if spec:
        r = run_spec_workload(torch, dist, sampler, w, rank, world, device, args.steps, args.warmup, args.small, barrier,
                              world == 1 and not args.no_cpu_baseline)
    elif name == "c5_sharded" and world > 1:
        r = None
    else:
        if name == "c5_sharded":
            raise SystemExit("c5_sharded needs --gpus N > 1 (on one GPU its vocab-segment form is covered by the tests)")
        r = run_sampling_workload(torch, dist, sampler, name, w, rank, world, device, args.steps, args.warmup, args.small,
                                  barrier)
        # keep the GPU under the same load a little longer so that the clock sampler sees it
        t_end = time.time() + 0.6
        i = 0
        while time.time() < t_end:
            r["prepared"][i % len(r["prepared"])].run(stream.cuda_stream)
            i += 1
            if i % 64 == 0:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
    clocks.stop_flag = True
    clocks.join(timeout=3)

    # ---- end to end through the host-memory call (pinned host buffers) ----
    e2e = None
    if r is not None and not spec and not args.no_e2e:
        B = w["B"]
        hb = {k: (v.cpu().pin_memory() if hasattr(v, "cpu") else v) for k, v in r["bufs"][0].items()}
        hout = {}
        esteps = max(3, min(args.steps, 20))

        def estep():
            sampler.sample(hb["logits"], uniforms=hb["uniforms"], config=r["cfg"], row_params=r["rp"], mask=hb.get("mask"),
                           history=hb.get("history"), want_prob=True, want_lse=True, stream=stream.cuda_stream, out=hout)
        for _ in range(3):
            estep()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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
        if r["rp"] is not None:
            h2d += r["rp"].nbytes
        d2h = sum(v.nbytes for v in hout.values())
        e2e = {"value": B * esteps * world / (float(te.item()) * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "steps": esteps, "split_ms": sampler.last_timing_ms()}

    # ---- CPU baseline: the oracle on the same rows (rank 0, N == 1) ----
    cpu = None
    if r is not None and not spec and rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import born_oracle as O
        O.build()
        cores = os.cpu_count() or 1
        hc = host_copy(torch, r["bufs"][0])
        params = oracle_params_for(w)
        kw = dict(uniforms=hc["uniforms"], mask=hc["mask"], history=hc["history"])
        O.sample(hc["logits"], params, nthreads=cores, **kw)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            O.sample(hc["logits"], params, nthreads=cores, **kw)
            reps += 1
        dt = time.perf_counter() - t0
        cpu = {"value": w["B"] * reps / dt, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"all {w['B']} rows of the workload x {reps} passes, {cores} threads over rows"}

    # ---- the other workloads of the library, each timed and checked the same way ----
    extra = {}
    if not args.no_extra and not args.small and name == DEFAULT:
        if world == 1:
            for en in EXTRA_N1:
                ew = WORKLOADS[en]
                es, ewm = max(10, min(args.steps, 50)), max(3, min(args.warmup, 5))
                try:
                    if en == "c4_spec_verify":
                        x = run_spec_workload(torch, dist, sampler, ew, rank, world, device, es, ewm, False, barrier, False)
                        extra[en] = {"us_per_step": 1e3 * x["ms_per_step"], "sequences_per_s": x["sequences"] / (x["ms_per_step"] * 1e-3),
                                     "frac_of_measured_peak": roofline(x["bytes_launch"], x["ms_per_step"], en)["frac"],
                                     "launches_per_step": x["launches_per_step"], "parity": x.get("parity")}
                    else:
                        x = run_sampling_workload(torch, dist, sampler, en, ew, rank, world, device, es, ewm, False, barrier)
                        extra[en] = {"us_per_step": 1e3 * x["ms_per_step"], "rows_per_s": ew["B"] / (x["ms_per_step"] * 1e-3),
                                     "frac_of_measured_peak": roofline(x["bytes_launch"], x["ms_per_step"], en)["frac"],
                                     "launches_per_step": x["launches_per_step"], "timing": x["timing"],
                                     "fallback_rows_in_timed_steps": x["fallback_rows_in_timed_steps"],
                                     "parity": x.get("parity")}
                        del x
                    torch.cuda.empty_cache()
                except Exception as e:  # a failing extra must not lose the headline line
                    extra[en] = {"error": repr(e)}
        else:
            try:
                x = run_sharded(torch, dist, sampler, WORKLOADS["c5_sharded"], rank, world, device,
                                max(10, min(args.steps, 50)), max(3, min(args.warmup, 5)), barrier)
                if rank == 0:
                    extra["c5_sharded"] = x
            except Exception as e:
                extra["c5_sharded"] = {"error": repr(e)}
    if name == "c5_sharded" and world > 1:
        x = run_sharded(torch, dist, sampler, w, rank, world, device, args.steps, args.warmup, barrier)
        if rank == 0:
            line = {"metric": METRIC, "value": x["rows_per_s"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": x["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                    "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": {"workload": name, "batch": w["B"], "vocab": w["V"], "vocab_per_gpu": x["vocab_per_gpu"],
                               "parallelism": "vocab-sharded x%d (NCCL all-gather)" % world},
                    "roofline": x["roofline_per_gpu"], "cpu_baseline": None, "e2e": None,
                    "gpu_launches": x["launches_per_step"] * args.steps, "clocks": clocks.summary(), "parity": x["parity"]}
            print(json.dumps(line), flush=True)
    elif rank == 0:
        B, V = w["B"], w["V"]
        kernel_ms = r["ms_per_step"]
        if spec:
            line = {"metric": "spec_verified_sequences_per_s", "value": B * world / (kernel_ms * 1e-3), "unit": "sequences/s",
                    "dtype": "f32", "config": {"workload": name, "batch_per_gpu": B, "draft_len": w["K"], "vocab": V,
                                               "parallelism": "batch-parallel x%d" % world, "timing": r["timing"]},
                    "cpu_baseline": r.get("cpu_baseline")}
        else:
            esz = 4 if w["dtype"] == "f32" else 2
            line = {"metric": METRIC, "value": B * world / (kernel_ms * 1e-3), "unit": UNIT, "dtype": w["dtype"],
                    "config": {"workload": name, "batch_per_gpu": B, "vocab": V, "vocab_per_gpu": V,
                               "parallelism": "batch-parallel x%d" % world,
                               "l2": f"{r['nbuf']} rotating input buffers, {r['nbuf'] * B * V * esz / 1e6:.0f} MB > L2",
                               "timing": r["timing"], "outputs": "token, prob, lse, status"},
                    "cpu_baseline": cpu, "fallback_rows_in_timed_steps": r["fallback_rows_in_timed_steps"]}
        line.update({"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": kernel_ms,
                     "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
                     "roofline": roofline(r["bytes_launch"], kernel_ms, name), "e2e": e2e,
                     "gpu_launches": int(r["launches_per_step"]) * args.steps, "clocks": clocks.summary(),
                     "parity": r.get("parity"), "workloads": extra})
        print(json.dumps(line), flush=True)
    sampler.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
