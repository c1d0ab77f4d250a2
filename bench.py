"""Benchmark of the ring-attention hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default `causal_32k`): bf16 causal self-attention, forward + backward, batch 2,
16 heads, head dim 128, 32768 tokens in total, sharded evenly over the N GPUs of the ring
(strong scaling), Q/K/V/dO ~ N(0,1) from a seeded generator, softmax scale 1/sqrt(128).
One step = one ring forward + one ring backward.  Prints ONE JSON line on rank 0.
Other workloads (`--workload`): `documents_128k` (document mask, causal inside a document),
`alibi_window_64k` (ALiBi bias + causal window of 4096 tokens, head dim 64, forward only),
`causal_1m` (131072 tokens per GPU, weak scaling: 1 Mi tokens at 8 GPUs).

`value` times the C-ABI ring calls with inputs resident in HBM; `e2e` times the public
Python API (`ring_attention` + autograd backward) with inputs in pinned host memory, the
host->device copies of q, k, v, dO and the device->host copies of out, dq, dk, dv of every
step inside the timed region (on copy streams, overlapping the neighbouring steps' compute).  FLOPs are counted exactly: 4d per visible (query, key) pair forward,
10d backward.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: dtype, b, h, d, total tokens, mask
    "causal_32k": dict(dtype="bf16", b=2, h=16, d=128, s=32768, mask="causal"),
    "config1_fp32": dict(dtype="f32", b=1, h=4, d=64, s=1024, mask="causal"),
    "causal_8k": dict(dtype="bf16", b=2, h=16, d=128, s=8192, mask="causal"),
    # documents of seeded lengths U[512, 16384] packed until the sequence is full; a pair is visible
    # inside one document, causally
    "documents_128k": dict(dtype="bf16", b=1, h=32, d=128, s=131072, mask="documents"),
    # ALiBi slopes 2^(-8(h+1)/16), visible iff 0 <= q_pos - kv_pos < 4096; forward only
    "alibi_window_64k": dict(dtype="bf16", b=4, h=16, d=64, s=65536, mask="alibi+window", window=4096, backward=False),
    # the same mask on a quarter of the length: the ncu capture case of the head-dim-64 forward
    "alibi_window_16k": dict(dtype="bf16", b=4, h=16, d=64, s=16384, mask="alibi+window", window=4096, backward=False),
    # 131072 tokens per GPU (1 Mi tokens at 8 GPUs), inputs ~ N(0, 0.5^2)
    "causal_1m": dict(dtype="bf16", b=1, h=8, d=128, s_per_gpu=131072, mask="causal", std=0.5),
}


def metric_name(w):
    return "ring_attention_fwd_bwd_tokens_per_s" if w.get("backward", True) else "ring_attention_fwd_tokens_per_s"


def causal_pairs(s):
    return s * (s + 1) // 2


def document_lengths(s, seed=0):
    """Seeded packing: lengths uniform in [512, 16384] until `s` tokens are filled, the last one cut."""
    import numpy as np

    rng = np.random.default_rng(seed)
    out, left = [], s
    while left > 0:
        n = min(int(rng.integers(512, 16385)), left)
        out.append(n)
        left -= n
    return out


def visible_pairs(w):
    """Exact number of visible (query, key) pairs of one batch element and head."""
    s = w["s"]
    if w["mask"] == "causal":
        return causal_pairs(s)
    if w["mask"] == "documents":
        return sum(causal_pairs(n) for n in document_lengths(s))
    if w["mask"] == "alibi+window":
        win = min(w["window"], s)
        return causal_pairs(win) + (s - win) * win
    raise ValueError(w["mask"])


def flops(w, fwd=True, bwd=True):
    bwd = bwd and w.get("backward", True)
    per_pair = (4 * w["d"] if fwd else 0) + (10 * w["d"] if bwd else 0)
    return w["b"] * w["h"] * visible_pairs(w) * per_pair


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(burst=p["bf16_tflops"], sustained=p["bf16_tflops_sustained"], hbm=p["hbm_gbs"], source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs.

    The sampling runs in a separate `nvidia-smi -lms` process: polling NVML from a thread of
    this process was measured to stretch the timed step (it contends with the launches)."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def __enter__(self):
        import subprocess
        import tempfile

        try:
            fd, self.path = tempfile.mkstemp(prefix="ra_clocks_", suffix=".csv")
            self.out = os.fdopen(fd, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=self.out, stderr=subprocess.DEVNULL)
            # nvidia-smi's start-up (driver queries over every GPU of the box) was seen to stall the
            # device for tens of ms: wait for its first sample before the timed region starts
            t_end = time.time() + 10.0
            while time.time() < t_end and os.path.getsize(self.path) == 0 and self.proc.poll() is None:
                time.sleep(0.05)
            time.sleep(0.1)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()  # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.out.close()

    def summary(self):
        samples, reasons, mx = [], set(), None
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 6 or not f[0].isdigit():
                    continue
                samples.append(int(f[0]))
                mx = int(f[1]) if f[1].isdigit() else mx
                for name, val in zip(self.NAMES, f[2:6]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        s = sorted(samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(s)}


def host_threads():
    """Cores this process may use (its affinity mask), which is what the BLAS pool is set to."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_baseline(w, nranks=4, budget_s=20.0):
    """The reference's algorithm (ring.py:79-211) on the host cores through the oracle port:
    a bounded sample of the workload (one batch element, a few heads, a shorter sequence),
    converted to the metric's unit through the exact FLOP count.  The BLAS thread count is
    set explicitly (a launcher may have exported OMP_NUM_THREADS=1) and the count in use is
    what the line reports."""
    from threadpoolctl import threadpool_info, threadpool_limits

    from oracle import oracle as O

    want = host_threads()
    with threadpool_limits(limits=want):
        used = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
        s, heads = 4096, 4
        sample_flops = O.causal_flops(1, heads, s, w["d"])
        t = O.timed_cpu_ring_causal(1, heads, s, w["d"], nranks)  # warm-up + size probe
        reps = max(1, min(8, int(budget_s / max(t, 1e-3)) - 1))
        ts = [O.timed_cpu_ring_causal(1, heads, s, w["d"], nranks, seed=i + 1) for i in range(reps)]
    best = min(ts + [t])
    flops_per_s = sample_flops / best
    tokens_per_s = w["b"] * w["s"] / (flops(w) / flops_per_s)
    return {
        "value": tokens_per_s, "unit": "tokens/s", "cores": used, "kind": "port",
        "sample": f"oracle port (NumPy float32, BLAS on {used} threads), causal fwd+bwd, b=1 h={heads} "
                  f"S={s} d={w['d']} over {nranks} virtual ranks, best of {len(ts) + 1}: {best:.3f} s = "
                  f"{flops_per_s / 1e9:.1f} GFLOP/s; scaled to the workload by its exact FLOP count",
        "gflops": flops_per_s / 1e9, "extrapolated": True, "sample_seconds": best, "sample_tokens": s,
    }


def cpu_config1():
    """The reference's CPU-runnable configuration, timed for real (nothing extrapolated):
    fp32 causal forward + backward, batch 1, 4 heads, 1024 tokens over 4 virtual ranks, head dim 64."""
    from threadpoolctl import threadpool_limits

    from oracle import oracle as O

    with threadpool_limits(limits=host_threads()):
        O.timed_cpu_ring_causal(1, 4, 1024, 64, 4)
        ts = [O.timed_cpu_ring_causal(1, 4, 1024, 64, 4, seed=i + 1) for i in range(5)]
    best = min(ts)
    return {"workload": "config1: fp32 causal fwd+bwd, b1 h4 S1024 d64, 4 virtual ranks", "seconds": best,
            "tokens_per_s": 1024 / best, "gflops": O.causal_flops(1, 4, 1024, 64) / best / 1e9, "extrapolated": False}


def run_reference(args, w):
    """`--impl reference`: the reference's own CPU algorithm, timed on the host."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(w, budget_s=4.0)
        if i >= args.warmup:
            vals.append(base["value"])
    v = sum(vals) / len(vals)
    base["value"] = v
    ms = w["b"] * w["s"] / v * 1e3
    line = {
        "impl": "reference", "metric": metric_name(w), "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak" if "s_per_gpu" in w else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, w, args.gpus),
        "cpu_baseline": base,
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "extrapolated": True, "sample_seconds": base["sample_seconds"],
        "config1_cpu": cpu_config1(),
        "note": "reference JAX path unavailable on this box (jax not installed, no network); "
                "this is the CPU restatement of its algorithm; every step times a bounded sample "
                "(sample_seconds, measured) and ms_per_step is the workload's time extrapolated from it by "
                "FLOP count, so it does not fit inside this run; config1_cpu is the reference's CPU-runnable "
                "configuration timed for real",
    }
    print(json.dumps(line), flush=True)


def shard_slice(r, t, head, b, c, d, std, dt):
    """Tensor t (0 q, 1 k, 2 v, 3 dO) of rank r's shard, one head: [b, c, d].  Every (rank, tensor,
    head) has a seed of its own, so that any rank can rebuild one head of the whole sequence on
    the host for the parity check without drawing everything."""
    import torch

    g = torch.Generator().manual_seed(1234 + (r * 4 + t) * 4096 + head)
    return (torch.randn((b, c, d), generator=g) * std).to(dt)


def shard_indices(layout, total, r, n):
    """Global token index (= position) of every local token of rank r."""
    import torch

    if layout == "zigzag" and n > 1:
        from ring_attention_b200 import zigzag_indices

        return zigzag_indices(total, r, n)
    c = total // n
    return torch.arange(c) + r * c


def bind_to_gpu_numa(local):
    """Runs this process on the CPUs of the NUMA node its GPU hangs off, so that the pinned host
    buffers allocated afterwards are local to the GPU's PCIe root.  Returns what was found."""
    import torch

    info = {"numa_node": None, "cpus": host_threads()}
    try:
        pr = torch.cuda.get_device_properties(local)
        path = f"/sys/bus/pci/devices/{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0/numa_node"
        node = int(open(path).read().strip())
        info["numa_node"] = node
        if node >= 0:
            cpus = set()
            for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            cpus &= os.sched_getaffinity(0)
            if cpus:
                os.sched_setaffinity(0, cpus)
                info["cpus"] = len(cpus)
    except Exception as e:  # sysfs layout differs, no permission: measure as is
        info["note"] = f"not bound: {type(e).__name__}"
    return info


def parity_check(w, args, rank, N, results, seg_global, slopes, backward):
    """Sampled rows of this rank's results against the CPU oracle on the whole sequence.

    One (batch, head) per rank: the other ranks' shards of that head are rebuilt from their
    seeds, ~16 query rows of this rank's shard give out, L and dQ, and up to 8 of its key rows
    give dK, dV (only key rows whose gradient the oracle can afford: a key at position p of a
    causal sequence needs L and delta of every later query).  Bound: 2e-2 abs + 1e-2 rel."""
    import numpy as np
    import torch
    from threadpoolctl import threadpool_limits

    from oracle import oracle as O

    b, h, d, S = w["b"], w["h"], w["d"], w["s"]
    c = S // N
    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float32
    bb, hh = b - 1, (rank * 5 + 3) % h
    G = [np.zeros((S, d)) for _ in range(4)]
    for r in range(N):
        idx_r = shard_indices(args.layout, S, r, N).numpy()
        for t in range(4 if backward else 3):
            G[t][idx_r] = shard_slice(r, t, hh, b, c, d, w.get("std", 1.0), dt)[bb].to(torch.float64).numpy()
    idx = shard_indices(args.layout, S, rank, N).numpy()
    rng = np.random.default_rng(99 + rank)
    q_loc = np.unique(np.concatenate([[0, c - 1], rng.integers(0, c, 14)]))
    k_loc = np.array([], np.int64)
    if backward:
        if seg_global is not None:
            ok = np.ones(c, bool)  # a key is seen inside its document only
        else:
            p = idx.astype(np.float64)
            ok = (float(S) ** 2 - p ** 2) / 2 * 4 * d <= 3e11
        cand = np.nonzero(ok)[0]
        if cand.size:
            k_loc = np.unique(rng.choice(cand, size=min(8, cand.size), replace=False))
    scale = 1 / math.sqrt(d)
    with threadpool_limits(limits=max(1, host_threads() // N)):
        want = O.sampled_rows(G[0], G[1], G[2], G[3], scale, idx[q_loc], idx[k_loc], seg=seg_global,
                              window=w.get("window", 0), slope=None if slopes is None else float(slopes[hh]),
                              causal=True, score_dtype=np.float32)
    f = lambda t: t.detach().to(torch.float64).cpu().numpy()
    excess = {"out": O.bf16_excess(f(results["out"][bb, q_loc, hh]), want["out"]),
              "L": O.bf16_excess(f(results["lse"][bb, hh, q_loc]), want["L"])}
    if backward:
        excess["dq"] = O.bf16_excess(f(results["dq"][bb, q_loc, hh]), want["dq"])
        if k_loc.size:
            excess["dk"] = O.bf16_excess(f(results["dk"][bb, k_loc, hh]), want["dk"])
            excess["dv"] = O.bf16_excess(f(results["dv"][bb, k_loc, hh]), want["dv"])
    worst = max(excess.values())
    return {"ok": bool(worst <= 0 and all(np.isfinite(v) for v in excess.values())), "max_excess": worst,
            "rows": int(q_loc.size), "key_rows": int(k_loc.size), "head": [int(bb), int(hh)], "excess": excess}


def workload_config(args, w, n):
    what = {"causal": "causal", "documents": "document-masked (causal inside a document)",
            "alibi+window": f"ALiBi + causal window {w.get('window', 0)}"}[w["mask"]]
    return {
        "workload": f"{args.workload}: {w['dtype']} {what} MHA {'fwd+bwd' if w.get('backward', True) else 'fwd'}, "
                    f"batch {w['b']}, heads {w['h']}, head_dim {w['d']}, total seq {w['s']} sharded evenly over {n} GPU(s)",
        "global_batch": w["b"], "seq_len": w["s"], "heads": w["h"], "head_dim": w["d"],
        "parallelism": f"sp{n}", "layout": args.layout if n > 1 else "contiguous", "plan": bool(args.plan and n > 1), "l2": "inputs larger than L2 (each of q,k,v,dO per rank exceeds 126 MB at N<=2; "
                                      "an L2 flush runs between steps otherwise)",
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="causal_32k", choices=list(WORKLOADS))
    ap.add_argument("--block-impl", default="cuda", choices=["cuda", "simt", "tcgen05"])
    ap.add_argument("--layout", default="zigzag", choices=["zigzag", "contiguous"],
                    help="token->rank layout at N>1: zigzag balances causal work, contiguous is the reference tests' layout")
    ap.add_argument("--plan", action="store_true",
                    help="at N>1: leave out the ring steps whose block the mask empties (made once, before the warm-up)")
    ap.add_argument("--timeline", action="store_true",
                    help="rank 0 prints, on stderr, when each block launch and each wait for a transfer of the last timed step ran")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if "s_per_gpu" in w:
        w["s"] = w["s_per_gpu"] * args.gpus
    backward = w.get("backward", True)
    if args.impl == "reference":
        return run_reference(args, w)

    import torch
    import torch.distributed as dist

    import ring_attention_b200 as ra
    from ring_attention_b200 import _lib
    from ring_attention_b200._lib import RaScoreMod, RaShape, RaTensor, check, lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local)
    host_info = bind_to_gpu_numa(local)  # before any pinned allocation
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mesh = ra.Mesh((1, world), ("dp", "sp"))
    ring = mesh.ring("sp")
    ring.set_timing(True)
    N = world
    c = w["s"] // N
    b, h, d = w["b"], w["h"], w["d"]
    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float32
    dcode = _lib.RA_DTYPE_BF16 if w["dtype"] == "bf16" else _lib.RA_DTYPE_F32
    check(lib.ra_set_impl({"cuda": 0, "simt": 1, "tcgen05": 2}[args.block_impl]))

    # synthetic inputs, pinned on the host (e2e) and resident on the device (value)
    host = [torch.stack([shard_slice(rank, t, hd, b, c, d, w.get("std", 1.0), dt) for hd in range(h)], dim=2).pin_memory()
            for t in range(4)]
    q, k, v, do = (t.cuda() for t in host)
    idx = shard_indices(args.layout, w["s"], rank, N)
    pos = idx.to(torch.int32).expand(b, c).contiguous().cuda()
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    lse = torch.empty((b, h, c), dtype=torch.float32, device="cuda")
    mod = RaScoreMod()
    mod.kinds = _lib.RA_MOD_CAUSAL
    mod.q_pos = mod.kv_pos = pos.data_ptr()
    seg = slopes = seg_global = None
    if w["mask"] == "documents":
        lens = torch.tensor(document_lengths(w["s"]))
        seg_global = torch.repeat_interleave(torch.arange(len(lens)), lens)
        seg = seg_global[idx].to(torch.int32).expand(b, c).contiguous().cuda()
        mod.kinds |= _lib.RA_MOD_SEGMENT
        mod.q_seg = mod.kv_seg = seg.data_ptr()
    elif w["mask"] == "alibi+window":
        slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / h) for i in range(h)], dtype=torch.float32, device="cuda")
        mod.kinds |= _lib.RA_MOD_ALIBI | _lib.RA_MOD_WINDOW
        mod.window = w["window"]
        mod.alibi_slopes = slopes.data_ptr()
    sh = RaShape(b, h, c, c, d, d, dcode, 1 / math.sqrt(d))
    tv = lambda t: C.byref(RaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if q.numel() * q.element_size() < (126 << 20) else None

    # the public API's view of the same mask (used by the plan and by the e2e leg)
    qkw = {"q_positions": pos}
    kkw = {"kv_positions": pos}
    if seg is not None:
        qkw["q_segment_ids"] = seg
        kkw["kv_segment_ids"] = seg
    sm = ra.ScoreMod(causal=True, alibi_slopes=slopes, window=w.get("window", 0))
    plan = ra.make_ring_plan(q, k, ring, sm, qkw, kkw) if (args.plan and N > 1) else None
    if plan is not None:
        check(lib.ra_ring_use_plan(ring.handle, plan.handle))

    def step():
        check(lib.ra_ring_fwd(ring.handle, C.byref(sh), tv(q), tv(k), tv(v), C.byref(mod), tv(out), lse.data_ptr(), stream))
        if backward:
            check(lib.ra_ring_bwd(ring.handle, C.byref(sh), tv(q), tv(k), tv(v), tv(out), lse.data_ptr(), tv(do),
                                  C.byref(mod), tv(dq), tv(dk), tv(dv), stream))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    launches0 = lib.ra_launch_count()
    e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush_ms = 0.0
    with ClockSampler(local) as clocks:
        # the device idled while the sampler started (its clocks may have dropped): one more
        # untimed step right before the timed region
        step()
        barrier()
        # K steps back to back with no host synchronisation in between; the device clock brackets them
        e_begin.record()
        for i in range(args.steps):
            if flush is not None:
                flush.fill_(i)
            step()
        e_end.record()
        barrier()
    if flush is not None:  # the L2 flush writes are not part of a step: time them alone and take them out
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for i in range(args.steps):
            flush.fill_(i)
        f1.record()
        torch.cuda.synchronize()
        flush_ms = f0.elapsed_time(f1) / args.steps
    # device times of the last step's block kernels and transfer waits (events recorded inside the timed region)
    # (total device time of this rank's block launches in the last step, number of launches)
    fwd_blocks = ring.last_block_ms(False)
    bwd_blocks = ring.last_block_ms(True) if backward else (0.0, 1)
    exposed_ms = [ring.last_timing(False)[1] + (ring.last_timing(True)[1] if backward else 0.0)]
    launches = lib.ra_launch_count() - launches0
    if args.timeline and rank == 0:
        for name, back in (("forward", False),) + ((("backward", True),) if backward else ()):
            blocks_tl, waits_tl = ring.last_timeline(back)
            tot = ring.last_timing(back)[0]
            print(f"timeline of the last {name} call ({tot:.3f} ms): block launches "
                  + " ".join(f"[{a:.3f},{b_:.3f}]" for a, b_ in blocks_tl) + " | waits for transfers "
                  + " ".join(f"[{a:.3f},{b_:.3f}]" for a, b_ in waits_tl), file=sys.stderr, flush=True)
    step_ms = e_begin.elapsed_time(e_end) / args.steps - flush_ms
    t = torch.tensor([step_ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms = float(t.item())
    exposed_all = [sum(exposed_ms) / len(exposed_ms)]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, exposed_all[0])
        exposed_all = gathered
    impl_used = {1: "simt", 2: "tcgen05"}.get(lib.ra_last_impl(), "?")
    # bytes this rank pushed over NVLink in the last step and the device time of those copies
    push = [ring.last_push(False), ring.last_push(True) if backward else (0.0, 0.0)] if N > 1 else []
    push_bytes, push_ms = sum(x[0] for x in push), sum(x[1] for x in push)
    rotation = {"bytes_per_step": push_bytes, "push_ms": push_ms,
                "gb_per_s_per_direction": (push_bytes / (push_ms * 1e-3) / 1e9) if push_ms > 0 else None}
    # no bounded wait ran out (inside a kernel, or for a peer), and the results are right: sampled rows
    # of this rank's out / L / dq / dk / dv against the CPU oracle, outside every timed region
    status_bits = _lib.device_status()
    verdict = parity_check(w, args, rank, N, {"out": out, "lse": lse, "dq": dq, "dk": dk, "dv": dv},
                           None if seg_global is None else seg_global.numpy(),
                           None if slopes is None else slopes.cpu().numpy(), backward)
    verdict["device_status"] = status_bits
    verdict["ring_aborted"] = bool(ring.aborted)
    verdict["ok"] = verdict["ok"] and status_bits == 0 and not verdict["ring_aborted"]
    per_rank = [{"parity": verdict, "rotation": rotation}]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, per_rank[0])
        per_rank = gathered

    # end to end through the public API, host buffers in and out
    e2e = None
    if not args.no_e2e:
        host_in = host if backward else host[:3]
        host_out = [torch.empty((b, c, h, d), dtype=dt).pin_memory() for _ in range(4 if backward else 1)]
        if plan is not None:
            check(lib.ra_ring_use_plan(ring.handle, None))  # the public API applies the plan per call

        # Every step copies its inputs from pinned host memory and its results back.  The copies
        # run on streams of their own (the host->device and device->host copy engines work next
        # to the SMs), double-buffered on the device, so step i+1's inputs arrive while step i
        # computes and step i-1's results leave: what a training loop that prefetches its next
        # batch does.  The timed region starts before the first copy in and ends after the last
        # copy out.
        main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        dev_in = [[torch.empty((b, c, h, d), dtype=dt, device="cuda") for _ in host_in] for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]  # the compute that read the slot is done
        ev_out = torch.cuda.Event()

        def copy_in(i):
            slot = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_free[slot])
                for dst, src in zip(dev_in[slot], host_in):
                    dst.copy_(src, non_blocking=True)
                ev_in[slot].record(s_in)

        def e2e_run(steps):
            copy_in(0)
            for i in range(steps):
                slot = i & 1
                if i + 1 < steps:
                    copy_in(i + 1)
                main.wait_event(ev_in[slot])
                dev = [t.detach().requires_grad_(backward) for t in dev_in[slot][:3]]
                o = ra.ring_attention(dev[0], dev[1], dev[2], ring, bias_fn=sm, bias_q_kwargs=qkw, bias_kv_kwargs=kkw,
                                      block_impl=args.block_impl, plan=plan)
                if backward:
                    o.backward(dev_in[slot][3])
                ev_free[slot].record(main)
                results = (o.detach(), dev[0].grad, dev[1].grad, dev[2].grad) if backward else (o.detach(),)
                s_out.wait_event(ev_free[slot])
                with torch.cuda.stream(s_out):
                    for dst, src in zip(host_out, results):
                        src.record_stream(s_out)
                        dst.copy_(src, non_blocking=True)
                    ev_out.record(s_out)
            main.wait_event(ev_out)

        # What the host side can deliver: one pinned tensor copied in and one copied out, first by
        # one rank at a time (the others idle), then by all ranks at once.  The second figure is the
        # ceiling of the end-to-end number when the step itself gets short.
        def copy_rate(active):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            a0.record()
            if active:
                for _ in range(3):
                    dev_in[0][0].copy_(host_in[0], non_blocking=True)
                    host_out[0].copy_(dev_in[1][0], non_blocking=True)
            a1.record()
            barrier()
            ms = a0.elapsed_time(a1) / 3
            return (2 * host_in[0].numel() * host_in[0].element_size() / (ms * 1e-3) / 1e9) if active and ms > 0 else 0.0

        copy_rate(True)  # touch the buffers once
        alone = 0.0
        for turn in range(world):
            r_ = copy_rate(turn == rank)
            alone = r_ if turn == rank else alone
        together = copy_rate(True)
        rates_t = torch.tensor([alone, together], device="cuda")
        if world > 1:
            gathered_r = [torch.zeros_like(rates_t) for _ in range(world)]
            dist.all_gather(gathered_r, rates_t)
            rates_all = torch.stack(gathered_r).cpu()
        else:
            rates_all = rates_t.cpu()[None]
        host_probe = {"gb_per_s_one_rank_alone_mean": float(rates_all[:, 0].mean()),
                      "gb_per_s_per_rank_all_copying_mean": float(rates_all[:, 1].mean()),
                      "gb_per_s_all_ranks_together": float(rates_all[:, 1].sum()),
                      "note": "one pinned tensor copied in, then one copied out, per rank (one direction at a time): "
                              "bytes moved / device time"}

        e2e_run(min(args.warmup, 2))
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_run(args.steps)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # the last step's results on the host are the ones the device-resident path produced
        # (dQ is summed by floating-point reductions in no fixed order: equal up to bf16 rounding)
        same = all(torch.allclose(hst.float(), dev_t.cpu().float(), atol=2e-2, rtol=1e-2, equal_nan=True)
                   for hst, dev_t in zip(host_out, (out, dq, dk, dv)))

        # The same step with nothing overlapped: copy in, compute, copy out, one after the other on
        # one stream (the latency of a single call with host buffers, not a throughput).
        def inline_run(steps):
            for _ in range(steps):
                for dst, src in zip(dev_in[0], host_in):
                    dst.copy_(src, non_blocking=True)
                dev = [x.detach().requires_grad_(backward) for x in dev_in[0][:3]]
                o = ra.ring_attention(dev[0], dev[1], dev[2], ring, bias_fn=sm, bias_q_kwargs=qkw, bias_kv_kwargs=kkw,
                                      block_impl=args.block_impl, plan=plan)
                if backward:
                    o.backward(dev_in[0][3])
                results = (o.detach(), dev[0].grad, dev[1].grad, dev[2].grad) if backward else (o.detach(),)
                for dst, src in zip(host_out, results):
                    dst.copy_(src, non_blocking=True)

        inline_run(1)
        barrier()
        i0, i1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        i0.record()
        inline_run(min(args.steps, 3))
        i1.record()
        barrier()
        ti = torch.tensor([i0.elapsed_time(i1) / min(args.steps, 3)], device="cuda")
        if world > 1:
            dist.all_reduce(ti, op=dist.ReduceOp.MAX)
        h2d = sum(x.numel() * x.element_size() for x in host_in)
        d2h = sum(x.numel() * x.element_size() for x in host_out)
        e2e = {"value": b * w["s"] / (float(t.item()) * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": float(t.item()),
               "copies": "own streams, double-buffered on the device, inside the timed region",
               "inline_ms_per_step": float(ti.item()),
               "host_gb_per_s_each_way_all_ranks": world * h2d / (float(t.item()) * 1e-3) / 1e9,
               "matches_device_resident_results": bool(same), "host": host_info, "host_copy_probe": host_probe}

    if rank == 0:
        pk = peaks()
        total_flops = flops(w)
        tflops_gpu = total_flops / N / (step_ms * 1e-3) / 1e12
        # dominant kernel: the backward block kernel.  Algorithmic FLOPs of one launch: this rank's
        # share of the visible pairs, averaged over its block launches of one step (N forward
        # launches; N, or N + 1 with the own block in two parts, backward launches).
        bwd_flops_launch = flops(w, fwd=False) / N / max(bwd_blocks[1], 1)
        fwd_flops_launch = flops(w, bwd=False) / N / max(fwd_blocks[1], 1)
        bwd_ms = bwd_blocks[0] / max(bwd_blocks[1], 1)
        fwd_ms = fwd_blocks[0] / max(fwd_blocks[1], 1)
        # dominant kernel: the backward block where the workload has a backward pass
        dom_ms, dom_flops, dom_name = (bwd_ms, bwd_flops_launch, "backward") if backward else (fwd_ms, fwd_flops_launch, "forward")
        achieved = dom_flops / (dom_ms * 1e-3) / 1e12
        # the step is seconds of back-to-back launches at the power cap: the sustained figure is the
        # denominator at every N; the fraction of the burst figure is printed beside it
        peak = pk["sustained"]
        # DRAM bytes and FLOPs of the ncu capture of the dominant kernel (small causal case), kept next to
        # its summary; traffic of one launch here = capture bytes scaled by the visible-pair count
        capture = None
        cap_path = os.path.join(ROOT, "profiles", "tc_bwd_kernel_causal_8k.json")
        if args.workload in ("causal_32k", "causal_8k") and impl_used == "tcgen05" and os.path.exists(cap_path):
            capture = json.load(open(cap_path))
        parity_all = [x["parity"] for x in per_rank]
        rates = [x["rotation"]["gb_per_s_per_direction"] for x in per_rank if x["rotation"]["gb_per_s_per_direction"]]
        line = {
            "metric": metric_name(w), "value": b * w["s"] / (step_ms * 1e-3), "unit": "tokens/s", "n_gpus": N,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "weak" if "s_per_gpu" in w else "strong", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": workload_config(args, w, N),
            "tflops_per_gpu": tflops_gpu, "pct_bf16_peak": 100 * tflops_gpu / pk["sustained"],
            "block_impl": impl_used,
            "roofline": {
                "bound": "tensor", "kernel": f"{impl_used} {dom_name} block", "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s", "frac": achieved / peak,
                "frac_sustained": achieved / pk["sustained"], "frac_burst": achieved / pk["burst"],
                "traffic": (capture["dram_bytes"] * bwd_flops_launch / capture["flops"]) if capture else None,
                "peak_source": f"{pk['source']} bf16 cuBLAS, sustained ({pk['sustained']}; burst {pk['burst']})",
                "launch_ms": dom_ms, "flops_per_launch": dom_flops,
                "launches_per_step": int(bwd_blocks[1] if backward else fwd_blocks[1]),
                "fwd_block": {"launch_ms": fwd_ms, "achieved": fwd_flops_launch / (fwd_ms * 1e-3) / 1e12},
            },
            # Per rank: time a compute lane waited for a transfer while no block kernel of that rank ran.
            # A rank also waits when a peer is simply slower (the GPUs of a box differ by several per
            # cent at the power cap): the rank that waited least is the one that set the pace, and its
            # figure is what the transfers themselves cost; the largest figure is printed beside it.
            "exposed_comm_ms": min(exposed_all), "exposed_comm_frac": min(exposed_all) / step_ms,
            "exposed_comm_ms_max_over_ranks": max(exposed_all),
            "exposed_comm_ms_per_rank": exposed_all,
            "gpu_launches": int(launches),
            "parity": {"ok": all(x["ok"] for x in parity_all), "max_excess": max(x["max_excess"] for x in parity_all),
                       "rows": sum(x["rows"] for x in parity_all), "key_rows": sum(x["key_rows"] for x in parity_all),
                       "bound": "2e-2 abs + 1e-2 rel against the float64 oracle on the bf16 inputs"
                                if w["dtype"] == "bf16" else "bf16 bound applied to fp32 results",
                       "device_status": [x["device_status"] for x in parity_all], "per_rank": parity_all},
            "rotation": {"transport": ring.transport, "bytes_per_step_per_rank": per_rank[0]["rotation"]["bytes_per_step"],
                         "gb_per_s_per_direction_min": min(rates) if rates else None,
                         "gb_per_s_per_direction_mean": (sum(rates) / len(rates)) if rates else None,
                         "link_peak_gb_per_s": 770.0,
                         "note": "bytes this rank pushed to peers / device time of those peer copies on the transfer "
                                 "stream (events around each copy), last timed step; 770 GB/s is the measured peer-copy "
                                 "rate per direction on this pool"},
            "ring_plan": plan.matrix() if plan is not None else None,
            "clocks": clocks.summary(),
        }
        if e2e is not None:
            line["e2e"] = e2e
        if N == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line), flush=True)
    failed = not all(x["parity"]["ok"] for x in per_rank)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit("parity check failed: see the `parity` object of the JSON line")


if __name__ == "__main__":
    main()
