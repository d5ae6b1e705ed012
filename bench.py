#!/usr/bin/env python
"""Benchmark of the context-parallel attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference_gpu]
                    [--heads H] [--seq S] [--mesh UxR]

One "step" is one non-causal bf16 attention over the whole sequence (B=1, D=128) of the
standalone op sweep: H=24, S=32760 by default (the Wan-2.1-sized row of the sweep; the
largest row that is a single launch of a few ms on one GPU). With N > 1 (torchrun, one rank
per GPU) the sequence is sharded over a ulysses x ring mesh and every step is one call of
``ulysses_attn_func`` / ``ring_attn_func`` / ``UnifiedAttnMode``; total work is fixed, so
scaling is "strong". Prints ONE JSON line (rank 0).

``--impl reference`` times the reference's CPU path on the host cores on a bounded sample of the
same workload (at world size 1 that path is PyTorch's CPU scaled_dot_product_attention in fp32;
the numpy oracle under oracle/ is the parity checker, not the timed baseline); under torchrun
only rank 0 works.

``--impl reference_gpu`` is the comparator on the same GPUs: the reference's own GPU path -
PyTorch's SDPA library kernels (flash and cuDNN backends timed separately), NCCL all-to-alls
for the Ulysses exchange and PyTorch's ring-attention loop - on the same inputs, meshes and
timing harness. With ``--ref DIR`` (a directory holding the ``para_attn`` package) the
reference's functions themselves are called; without it the same sequence of library calls is
issued from this file (the reference adds nothing to them but the orchestration).

Every line of the ``ours`` arm also carries ``parity``: after the timed region 1024 sampled
output rows per rank (512 in each of two heads) are compared with the fp32 numpy oracle over
all keys.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "cp_attention_tflops"
UNIT = "TFLOP/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_gpu"])
    ap.add_argument("--ref", default=None, help="reference_gpu: directory that holds the para_attn package")
    ap.add_argument("--no-parity", action="store_true", help="skip the sampled-row comparison with the oracle")
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--seq", type=int, default=32760)
    ap.add_argument("--mesh", default=None, help="UxR, default Nx1 (all Ulysses)")
    ap.add_argument("--workload", default="attention", choices=["attention", "flux", "wan", "hunyuan", "fbcache"],
                    help="attention = the headline op benchmark; the others time one transformer forward")
    ap.add_argument("--layers", type=int, default=None, help="DiT workloads: override the block count (quick runs)")
    ap.add_argument("--fbcache", type=float, default=0.0, help="DiT workloads: First-Block-Cache threshold (0 = off)")
    ap.add_argument("--causal", action="store_true", help="attention workload: causal mask (FLOPs counted as half)")
    ap.add_argument("--head-dim", type=int, default=128, choices=[64, 128], help="attention workload: head_dim")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


VARIANT = {"D": 128, "causal": False}  # set from --head-dim / --causal; the headline row is D=128 non-causal


def workload_name(H, S):
    kind = "causal" if VARIANT["causal"] else "non-causal"
    return f"attention-op sweep row: bf16 {kind} B=1 H={H} S={S} D={VARIANT['D']}"


def attention_flops(H, S, B=1):
    """4*B*H*S^2*D for the two GEMMs; a causal run is counted as half of that (the visible
    triangle), the usual convention."""
    f = 4.0 * B * H * S * S * VARIANT["D"]
    return f / 2 if VARIANT["causal"] else f


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16_tflops": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


def make_inputs(H, S, seed=0):
    """Sweep inputs: N(0,1)*0.5, q and k RMS-normalised over D per (head, token), bf16; a
    per-tensor generator seeded seed + tensor id. Built on the host."""
    import torch

    outs = []
    for i in range(3):
        g = torch.Generator().manual_seed(seed + i)
        x = torch.randn(1, H, S, VARIANT["D"], generator=g) * 0.5
        if i < 2:
            x = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
        outs.append(x.to(torch.bfloat16))
    return outs


# ------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the oracle on the host cores
# ------------------------------------------------------------------------------------------
def cpu_sample(H, S, budget_s=12.0, ref_dir=None):
    """Time the reference's CPU path for a slab of query rows of one head against all S keys, fp32,
    on all host cores; grow the slab until about budget_s seconds of CPU work were spent. At world
    size 1 that path is one call of PyTorch's CPU scaled_dot_product_attention
    (src/para_attn/para_attn_interface.py:111-119): with the reference package at hand
    (``ref_dir``) its ``ulysses_attn_func`` is called, otherwise the library call it makes.
    Returns (TFLOP/s, sample text, kind)."""
    import torch
    import torch.nn.functional as F

    fn, kind, what = F.scaled_dot_product_attention, "port", "torch CPU SDPA (the call the reference's world-1 path makes)"
    for cand in ([ref_dir] if ref_dir else []) + [str(ROOT / "baseline" / "_ref")]:
        if cand and (Path(cand) / "para_attn" / "__init__.py").exists():
            sys.path.insert(0, str(cand))
            import para_attn

            fn, kind, what = para_attn.ulysses_attn_func, "reference", "para_attn.ulysses_attn_func on CPU tensors"
            break
    g = torch.Generator().manual_seed(0)
    k = torch.randn(1, 1, S, 128, generator=g) * 0.5
    v = torch.randn(1, 1, S, 128, generator=g) * 0.5
    rows, spent, flops = 512, 0.0, 0.0
    with torch.no_grad():
        while spent < budget_s:
            q = torch.randn(1, 1, rows, 128, generator=g) * 0.5
            t0 = time.perf_counter()
            fn(q, k, v)
            dt = time.perf_counter() - t0
            spent += dt
            flops += 4.0 * rows * S * 128
            if dt < 2.0 and rows < 16384:
                rows *= 2
    return (flops / spent / 1e12,
            f"{int(flops / (4.0 * S * 128))} query rows of one head x all {S} keys, fp32, {what}, "
            f"{torch.get_num_threads()} threads, {spent:.1f} s", kind)


def bench_config(H, S, U, R):
    """The `config` object of a bench line: the same for every arm run with the same flags."""
    return {"workload": workload_name(H, S), "mesh": f"{U}x{R} (ulysses x ring)",
            "l2": "256 MB flush between timed iterations", "timing": "CUDA events per step, max over ranks"}


def mesh_of(args, world):
    if args.mesh:
        U, R = (int(x) for x in args.mesh.lower().split("x"))
        return U, R
    return world, 1


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    H, S = args.heads, args.seq
    cores = os.cpu_count() or 1
    vals, sample = [], ""
    kind = "port"
    for _ in range(args.warmup):
        cpu_sample(H, S, budget_s=1.0, ref_dir=args.ref)
    t_all = time.perf_counter()
    for _ in range(args.steps):
        v, sample, kind = cpu_sample(H, S, budget_s=max(2.0, 60.0 / max(args.steps, 1)), ref_dir=args.ref)
        vals.append(v)
    wall = time.perf_counter() - t_all
    value = statistics.mean(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(H, S, *mesh_of(args, max(args.gpus, 1))),
        "note": "the reference's CPU path at world size 1 on the host cores (no GPU work: l2 and timing describe the GPU arm)",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """SM clock and slow-down reasons of one GPU, sampled every few milliseconds through NVML
    from a thread of this process (a timed region of ten 1.6 ms steps is far shorter than
    nvidia-smi's fastest loop); falls back to an `nvidia-smi -lms` child if NVML cannot be
    loaded. Read-only queries."""

    Q = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NVML_REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.samples = []  # (time.time(), sm MHz, reasons bit mask)
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons

            def loop():
                while not self._stop.is_set():
                    try:
                        self.samples.append((time.time(), float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)),
                                             int(reasons(h))))
                    except pynvml.NVMLError:
                        pass
                    time.sleep(0.002)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
            return
        except Exception:  # no NVML binding or no permission: use the command-line tool
            self._thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, t_begin=None, t_end=None):
        """Summarise the samples whose timestamps fall inside [t_begin, t_end] (time.time())."""
        import datetime

        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            inside = [x for x in self.samples if t_begin is None or t_begin - 0.002 <= x[0] <= t_end + 0.002]
            mask = 0
            for x in inside:
                mask |= x[2]
            return {"sm_mhz": statistics.median([x[1] for x in inside]) if inside else None, "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(n for bit, n in self.NVML_REASONS.items() if mask & bit), "samples": len(inside),
                    "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if t_begin is not None and not (t_begin - 0.01 <= ts <= t_end + 0.01):
                    continue
                sm.append(float(parts[1]))
                mx = float(parts[2])
            except ValueError:
                continue
            for n, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    import paraattention_b200 as pa
    from paraattention_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    H, S = args.heads, args.seq
    if args.mesh:
        U, R = (int(x) for x in args.mesh.lower().split("x"))
    else:
        U, R = world, 1
    assert U * R == world and H % U == 0
    S_pad = (S + world - 1) // world * world  # pad to divisibility by the world size
    mesh = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        mesh = dist.init_device_mesh("cuda", (R, U), mesh_dim_names=("ring", "ulysses"))

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # early: nvidia-smi needs a moment before its first sample
    causal = VARIANT["causal"]
    q_h, k_h, v_h = make_inputs(H, S_pad)
    parity_heads = sorted({1 % H, H - 2 if H > 2 else H - 1})
    kv_full = {h: (k_h[0, h].float().numpy().copy(), v_h[0, h].float().numpy().copy()) for h in parity_heads}
    if world > 1:
        q_h, k_h, v_h = (x.chunk(world, dim=-2)[rank].contiguous() for x in (q_h, k_h, v_h))
    q_h, k_h, v_h = q_h.pin_memory(), k_h.pin_memory(), v_h.pin_memory()
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB of L2

    if args.impl == "reference_gpu":
        return run_reference_gpu(args, dict(torch=torch, dist=dist, world=world, rank=rank, dev=dev, mesh=mesh, U=U, R=R,
                                            H=H, S_pad=S_pad, q=q, k=k, v=v, flush=flush, sampler=sampler,
                                            causal=causal))
    if world == 1:
        def step(qq, kk, vv):
            return ops.attention_forward(qq, kk, vv, is_causal=causal)
        launches_per_step = 1  # the attention kernel
    else:
        mode = pa.UnifiedAttnMode(mesh)

        def step(qq, kk, vv):
            with mode:
                return torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=causal)
        # the attention kernel (the exchange rides inside it); Ulysses meshes add the one-warp
        # wait for the output tiles and the hand-out copy; causal runs one more one-warp wait
        launches_per_step = 1 + (2 if U > 1 else 0) + (1 if causal else 0)
    # a launch whose last wave is split (the library decides per shape; never with peers) is two launches
    split = split_plan(torch, dev, ((S_pad // world + 255) // 256) * (H // U) * U,
                       ((S_pad // world + 127) // 128) * world, causal, world > 1)
    if split["k"] > 1 and split["from"] > 0:
        launches_per_step += 1

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def timed(fn, n_warm, n_steps, window=None):
        for _ in range(n_warm):
            fn()
        sync_all()
        if window is not None:
            window["begin"] = time.time()
        evs = []
        for _ in range(n_steps):
            flush.fill_(1)  # evict q/k/v and staging from L2 between timed iterations
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        sync_all()
        if window is not None:
            window["end"] = time.time()
        total_ms = sum(a.elapsed_time(b) for a, b in evs)
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    window = {}
    total_ms = timed(lambda: step(q, k, v), max(args.warmup, 3), args.steps, window)
    clocks = sampler.stop(window.get("begin"), window.get("end")) if rank == 0 else None
    pa.check_device_status()

    # parity, outside the timed region: sampled output rows of this rank against the oracle
    parity = None
    if not args.no_parity and not causal:
        import numpy as np

        from oracle import cp_attention_oracle as O

        out = step(q, k, v)
        torch.cuda.synchronize(dev)
        s_loc = q.shape[2]
        rows = torch.randperm(s_loc, generator=torch.Generator().manual_seed(rank))[:512].sort().values
        max_abs, num, den = 0.0, 0.0, 0.0
        for h in parity_heads:
            got = out[0, h, rows.to(dev)].float().cpu().numpy()
            kf, vf = kv_full[h]
            ref, _ = O.sdpa_with_lse(q[0, h, rows.to(dev)].float().cpu().numpy()[None, None], kf[None, None], vf[None, None])
            ref = ref[0, 0]
            max_abs = max(max_abs, float(np.abs(got - ref).max()))
            num += float(((got - ref) ** 2).sum())
            den += float((ref ** 2).sum())
        stats = torch.tensor([max_abs, num, den], dtype=torch.float64, device=dev)
        if world > 1:
            mx = stats[:1].clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            dist.all_reduce(stats, op=dist.ReduceOp.SUM)
            stats[0] = mx[0]
        max_abs, rel_l2 = float(stats[0]), math.sqrt(float(stats[1]) / max(float(stats[2]), 1e-30))
        parity = {"rows": 512 * len(parity_heads) * world, "heads": parity_heads, "max_abs": max_abs, "rel_l2": rel_l2,
                  "tolerance": {"max_abs": 2e-2, "rel_l2": 5e-3}, "ok": bool(max_abs <= 2e-2 and rel_l2 <= 5e-3),
                  "against": "fp32 numpy oracle over all keys, real peers" if world > 1 else "fp32 numpy oracle over all keys"}

    flops = attention_flops(H, S_pad)
    ms_per_step = total_ms / args.steps
    value = flops / (ms_per_step * 1e-3) / 1e12

    # end to end through the public API with host buffers: H2D of q, k, v and D2H of the result
    e2e = None
    if not args.no_e2e:
        from paraattention_b200.host_io import attention_from_host

        out_h = torch.empty(q_h.shape, dtype=torch.bfloat16).pin_memory()
        cp_kw = {}
        if world > 1:
            cp_kw = dict(ulysses_mesh=mode._ulysses_mesh, ring_mesh=mode._ring_mesh, flat_group=mode._flat_group)

        def e2e_step():
            # the public host-buffer call: H2D of q, k, v, attention and D2H of the result,
            # pipelined over groups of heads
            attention_from_host(q_h, k_h, v_h, out_h, is_causal=causal, device=dev, **cp_kw)

        n_e2e = max(3, min(args.steps, 10))
        e2e_ms = timed(e2e_step, 2, n_e2e) / n_e2e
        e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": int(3 * q_h.numel() * 2), "d2h_bytes_per_step": int(out_h.numel() * 2)}

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    per_gpu_tflops = value / world
    if world == 1:
        roofline = {"bound": "tensor", "achieved": per_gpu_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": per_gpu_tflops / peaks["bf16_tflops"], "traffic": TRAFFIC_BYTES_PER_LAUNCH.get((H, S)) if (VARIANT["D"] == 128 and not causal) else None,
                    "peak_source": f"{peaks['source']} cuBLAS bf16 burst", "kernel": "attn_fwd_kernel",
                    "flops_per_launch": flops}
    else:
        # slower of tensor time and NVLink time at the nominal 900 GB/s per direction per GPU
        hl = H // U
        s_loc = S_pad // world
        sent = ((world - 1) * 2 + (U - 1) * 2) * hl * s_loc * VARIANT["D"] * 2  # K,V to all; Q out + O back
        t_tc = flops / world / (peaks["bf16_tflops"] * 1e12)
        t_nv = sent / NVLINK_GBS / 1e9
        roof = max(t_tc, t_nv)
        roofline = {"bound": "tensor" if t_tc >= t_nv else "nvlink", "achieved": per_gpu_tflops,
                    "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": roof / (ms_per_step * 1e-3),
                    "traffic": None,
                    "peak_source": f"{peaks['source']} cuBLAS bf16 burst; NVLink {NVLINK_GBS:.0f} GB/s per direction (nominal)",
                    "exchanged_bytes_per_gpu": int(sent), "t_tensor_ms": t_tc * 1e3, "t_nvlink_ms": t_nv * 1e3,
                    "nvlink_gbs_if_not_overlapped": sent / (ms_per_step * 1e-3) / 1e9}
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline and not causal and VARIANT["D"] == 128:
        cv, sample, kind = cpu_sample(H, S, budget_s=12.0, ref_dir=args.ref)
        cpu_baseline = {"value": cv, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": kind, "sample": sample}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": bench_config(H, S, U, R), "per_gpu_tflops": per_gpu_tflops, "split_last_wave": split,
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks, "parity": parity,
        "gpu_launches": launches_per_step * args.steps,
    }
    if world == 1 and roofline.get("traffic") is not None and (H, S) != (24, 8192):
        roofline["traffic_scaled_from"] = "ncu capture at H=24 S=8192, scaled by S and heads"
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


NVLINK_GBS = 900.0  # per direction per GPU, NVLink 5 nominal

# dram__bytes_read.sum + dram__bytes_write.sum of one attn_fwd_kernel launch, captured with ncu
# at H=24, S=8192: 151.3 MB read + 33.6 MB written = the q, k, v, out bytes. q, k, v and out
# grow linearly with S while the K/V of one head (16.8 MB at S=32760) still fit the 126 MB L2,
# so the S=32760 rows are that capture scaled by 32760/8192 (and by heads).
_CAPTURED = 184.93e6
TRAFFIC_BYTES_PER_LAUNCH = {
    (24, 8192): _CAPTURED,
    (24, 32760): _CAPTURED * 32760 / 8192,
    (40, 32760): _CAPTURED * 32760 / 8192 * 40 / 24,
}


# ------------------------------------------------------------------------------------------
# comparator: the reference's GPU path (library SDPA + NCCL) on the same GPUs
# ------------------------------------------------------------------------------------------
def split_plan(torch, dev, units, kv_tiles, causal, pushers):
    """What the attention launch of this shape does with its last wave: {"from", "k", "units"}
    (k = 1: one CTA per work unit everywhere)."""
    import ctypes as C
    from paraattention_b200 import _lib as L, config

    lib = L.load()
    ws = int(lib.pa_attn_workspace_bytes()) if config.attention.split_last_wave else 0
    f, k = C.c_int32(units), C.c_int32(1)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    L.check(lib.pa_attn_split_plan(units, sms, kv_tiles, VARIANT["D"], int(causal), int(pushers), ws, C.byref(f),
                                   C.byref(k)))
    return {"units": units, "from": f.value, "k": k.value}


def run_reference_gpu(args, c):
    """Times what the reference runs on GPUs for this step: at world size 1 PyTorch's SDPA; on a
    mesh the Ulysses all-to-alls (src/para_attn/para_attn_interface.py:52-119) around PyTorch's
    ring-attention loop (:162-239; torch/distributed/tensor/experimental/_context_parallel/
    _attention.py) with the library SDPA kernel as its block op (src/para_attn/ops/__init__.py:48-110).
    The flash and cuDNN backends are timed separately; ``value`` is the faster one."""
    torch, dist = c["torch"], c["dist"]
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    world, rank, dev, mesh, U, R, H, S_pad = (c[k] for k in ("world", "rank", "dev", "mesh", "U", "R", "H", "S_pad"))
    q, k, v, flush, causal = c["q"], c["k"], c["v"], c["flush"], c["causal"]
    aten = torch.ops.aten

    ref_pkg = None
    for cand in ([args.ref] if args.ref else []) + [str(ROOT / "baseline" / "_ref")]:
        if cand and (Path(cand) / "para_attn" / "__init__.py").exists():
            sys.path.insert(0, str(cand))
            import para_attn as ref_pkg  # noqa: F811
            break

    def block_op(backend):
        """(out, lse) from the library kernel of one backend, as the reference's custom op returns it."""
        def flash(qq, kk, vv, is_causal=False, dropout_p=0.0, scale=None, **_):
            return aten._scaled_dot_product_flash_attention(qq, kk, vv, dropout_p=dropout_p, is_causal=is_causal,
                                                            scale=scale)[:2]

        def cudnn(qq, kk, vv, is_causal=False, dropout_p=0.0, scale=None, **_):
            return aten._scaled_dot_product_cudnn_attention(qq, kk, vv, attn_bias=None, compute_log_sumexp=True,
                                                            dropout_p=dropout_p, is_causal=is_causal, scale=scale)[:2]
        return flash if backend == "flash" else cudnn

    def a2a(x, pg):
        import torch.distributed._functional_collectives as funcol

        y = funcol.all_to_all_single(x.flatten(), None, None, pg)
        y = y.wait() if isinstance(y, funcol.AsyncCollectiveTensor) else y
        return y.reshape(x.shape)

    def ulysses(qq, kk, vv, pg, inner):
        n = dist.get_world_size(pg)

        def seq_to_heads(x):  # [b, h, s, d] -> [b, h/n, n*s, d]
            b, h, s, d = x.shape
            x = a2a(x.permute(1, 0, 2, 3).contiguous(), pg)
            return x.reshape(n, h // n, b, s, d).permute(2, 1, 0, 3, 4).reshape(b, h // n, n * s, d)

        def heads_to_seq(x):  # [b, h/n, n*s, d] -> [b, h, s, d]
            b, hl, s_all, d = x.shape
            x = a2a(x.permute(2, 0, 1, 3).contiguous(), pg)
            return x.reshape(n, s_all // n, b, hl, d).permute(2, 0, 3, 1, 4).reshape(b, n * hl, s_all // n, d)

        return heads_to_seq(inner(seq_to_heads(qq), seq_to_heads(kk), seq_to_heads(vv)))

    def ring(qq, kk, vv, pg, backend):
        from torch.distributed.tensor.experimental._context_parallel import _attention as A

        opts = A._cp_options
        old = (opts.convert_to_f32, opts.enable_load_balance, opts.rotate_method)
        opts.convert_to_f32, opts.enable_load_balance, opts.rotate_method = True, False, A._RotateMethod.ALL_TO_ALL
        try:
            out = A._templated_ring_attention(pg, 2, block_op(backend), qq, kk, vv, is_causal=causal, dropout_p=0.0,
                                              scale=None)[0]
        finally:
            opts.convert_to_f32, opts.enable_load_balance, opts.rotate_method = old
        return out.to(qq.dtype)

    def make_step(backend):
        sd = SDPBackend.FLASH_ATTENTION if backend == "flash" else SDPBackend.CUDNN_ATTENTION
        if ref_pkg is not None:
            mode = ref_pkg.UnifiedAttnMode(mesh) if world > 1 else None

            def step():
                with sdpa_kernel([sd]):
                    if mode is None:
                        return F.scaled_dot_product_attention(q, k, v, is_causal=causal)
                    with mode:
                        return F.scaled_dot_product_attention(q, k, v, is_causal=causal)
            return step
        ring_pg = mesh["ring"].get_group() if world > 1 else None
        uly_pg = mesh["ulysses"].get_group() if world > 1 else None

        def local(qq, kk, vv):
            with sdpa_kernel([sd]):
                return F.scaled_dot_product_attention(qq, kk, vv, is_causal=causal)

        def inner(qq, kk, vv):
            return ring(qq, kk, vv, ring_pg, backend) if R > 1 else local(qq, kk, vv)

        def step():
            return ulysses(q, k, v, uly_pg, inner) if U > 1 else inner(q, k, v)
        return step

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    flops = attention_flops(H, S_pad)
    backends, errors = {}, {}
    for backend in ("flash", "cudnn"):
        try:
            fn = make_step(backend)
            for _ in range(max(args.warmup, 3)):
                fn()
            sync_all()
            evs = []
            for _ in range(args.steps):
                flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                evs.append((e0, e1))
            sync_all()
            t = torch.tensor([sum(a.elapsed_time(b) for a, b in evs)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            backends[backend] = flops / (float(t.item()) / args.steps * 1e-3) / 1e12
        except Exception as e:  # a backend the library refuses for this shape
            errors[backend] = f"{type(e).__name__}: {str(e)[:160]}"
    c["sampler"].stop()
    if rank == 0:
        if backends:
            best = max(backends, key=backends.get)
            value = backends[best]
            line = {"impl": "reference_gpu", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
                    "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": flops / value / 1e9,
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": bench_config(H, c["S_pad"], U, R), "per_gpu_tflops": value / world,
                    "backends_tflops": backends, "backend_errors": errors, "best_backend": best,
                    "kind": "reference package" if ref_pkg is not None else
                            "the reference's sequence of library calls (torch SDPA, NCCL all_to_all, torch ring loop) issued from bench.py",
                    "gpu_launches": 0}
        else:
            line = {"impl": "reference_gpu", "unavailable": "; ".join(f"{b}: {e}" for b, e in errors.items())[:300]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# second metric: transformer forward latency of the shape-only DiTs under the adapters
# ------------------------------------------------------------------------------------------
def run_dit(args):
    """--workload flux|wan|hunyuan: ms per transformer forward (one denoising step) of the
    shape-only model at full size, random bf16 weights, under parallelize_transformer
    (and apply_cache_on_transformer when --fbcache > 0). Prints one JSON line."""
    import torch
    import torch.distributed as dist

    import paraattention_b200 as pa
    from paraattention_b200.context_parallel import init_context_parallel_mesh
    from paraattention_b200.context_parallel.diffusers_adapters import parallelize_transformer
    from paraattention_b200.first_block_cache import utils as fbc
    from paraattention_b200.first_block_cache.diffusers_adapters import apply_cache_on_transformer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    if not dist.is_initialized():
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    U, R = (int(x) for x in args.mesh.lower().split("x")) if args.mesh else (world, 1)
    mesh = init_context_parallel_mesh("cuda", max_ring_dim_size=R if R > 1 else None)
    dt = torch.bfloat16
    layers = args.layers
    torch.manual_seed(0)
    torch.set_default_dtype(dt)  # build the weights directly in bf16
    with torch.device(dev):
        if args.workload == "flux":
            from paraattention_b200.shape_models import FluxShapedTransformer2DModel

            kw = {} if layers is None else dict(num_layers=max(1, layers // 3), num_single_layers=layers - max(1, layers // 3))
            model = FluxShapedTransformer2DModel(**kw).to(dt)
            n_img, n_txt = 4096, 512
            hw = 64
            ys, xs = torch.meshgrid(torch.arange(hw), torch.arange(hw), indexing="ij")
            inputs = dict(hidden_states=torch.randn(1, n_img, 64).to(dt), encoder_hidden_states=torch.randn(1, n_txt, 4096).to(dt),
                          pooled_projections=torch.randn(1, 768).to(dt), timestep=torch.tensor([500.0]),
                          img_ids=torch.stack([torch.zeros_like(ys), ys, xs], -1).reshape(-1, 3).float(),
                          txt_ids=torch.zeros(n_txt, 3), guidance=torch.tensor([3.5]), return_dict=False)
            call = lambda: model(**inputs)[0]
            desc = "FLUX.1-dev-shaped MMDiT, 512 text + 4096 image tokens"
        elif args.workload == "wan":
            from paraattention_b200.shape_models_video import WanShapedTransformer3DModel

            model = WanShapedTransformer3DModel(**({} if layers is None else dict(num_layers=layers))).to(dt)
            x, enc = torch.randn(1, 16, 21, 60, 104).to(dt), torch.randn(1, 512, 4096).to(dt)
            t = torch.tensor([500.0])
            call = lambda: model(x, t, enc, return_dict=False)[0]
            desc = "Wan 2.1 14B-shaped DiT, 32760 video tokens + 512-token cross-attention"
        else:
            from paraattention_b200.shape_models_hunyuan import HunyuanVideoShapedTransformer3DModel

            kw = {} if layers is None else dict(num_layers=max(1, layers // 3), num_single_layers=layers - max(1, layers // 3))
            model = HunyuanVideoShapedTransformer3DModel(**kw).to(dt)
            x, enc = torch.randn(1, 16, 33, 90, 160).to(dt), torch.randn(1, 256, 4096).to(dt)
            t, mask, pooled, g = torch.tensor([500.0]), torch.ones(1, 256), torch.randn(1, 768).to(dt), torch.tensor([6.0])
            call = lambda: model(x, t, enc, mask, pooled, guidance=g, return_dict=False)[0]
            desc = "HunyuanVideo-shaped DiT, 118800 video + 256 text tokens"
    torch.set_default_dtype(torch.float32)
    n_blocks = sum(1 for _ in model.modules() if type(_).__name__.endswith("Block"))
    parallelize_transformer(model, mesh=mesh)
    if args.fbcache > 0:
        apply_cache_on_transformer(model)
    ctx = fbc.create_cache_context(residual_diff_threshold=args.fbcache)
    times = []
    with torch.no_grad(), fbc.cache_context(ctx):
        for i in range(max(args.warmup, 1) + args.steps):
            torch.cuda.synchronize(dev)
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = call()
            e1.record()
            torch.cuda.synchronize(dev)
            if i >= max(args.warmup, 1):
                t_ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
                dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
                times.append(float(t_ms.item()))
    pa.check_device_status()
    if rank == 0:
        print(json.dumps({
            "metric": "dit_step_latency_ms", "value": statistics.median(times), "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": statistics.mean(times),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": desc, "blocks": n_blocks, "mesh": f"{U}x{R} (ulysses x ring)",
                       "fbcache_threshold": args.fbcache, "weights": "random init", "output_finite": bool(torch.isfinite(out.float()).all())},
        }), flush=True)
    dist.barrier()
    dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# third leg: the HBM-bound cache kernels against the measured copy bandwidth
# ------------------------------------------------------------------------------------------
def run_fbcache_kernels(args):
    """--workload fbcache: GB/s of the First-Block-Cache kernels on a Wan-2.1-sized residual
    (32760 tokens x 5120 channels, bf16: 335 MB per tensor, larger than L2), one JSON line per
    kernel. Algorithmic bytes: decision kernel 3 reads + 1 write; TaylorSeer update (2
    derivatives) 3 reads + 2 writes; TaylorSeer extrapolation + add 4 reads + 1 write."""
    import torch

    from paraattention_b200.first_block_cache import utils as fbc
    from paraattention_b200.first_block_cache.taylorseer import TaylorSeer

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    rows, cols = 32760, 5120
    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda: torch.randn(1, rows, cols, generator=g, device=dev, dtype=torch.float32).bfloat16()  # noqa: E731
    h0, h1, prev = mk(), mk(), mk()
    tensor_bytes = h0.numel() * 2
    seer = TaylorSeer(n_derivatives=2, warmup_steps=100)
    for _ in range(3):  # three computed steps: two derivatives exist from here on
        seer.step(mk())
    y = mk()
    peaks = load_peaks()
    sampler = ClockSampler(0)
    sampler.start()

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        evs = []
        for _ in range(args.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs) / args.steps

    def taylor_update():
        seer.current_step += 1
        seer.update(y)

    legs = [
        ("fbc_residual_diff_kernel", 4, lambda: fbc.fused_residual_diff(h1, h0, prev)),
        ("taylor_update_kernel", 5, taylor_update),
        ("taylor_approx_kernel", 5, lambda: seer.approximate_value(add=h0)),
    ]
    begin = time.time()
    results = [(name, n, timed(fn)) for name, n, fn in legs]
    clocks = sampler.stop(begin, time.time())
    for name, n_tensors, ms in results:
        gbs = n_tensors * tensor_bytes / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "fbcache_kernel_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{name}: residual of {rows} tokens x {cols} channels",
                       "l2": f"{n_tensors} tensors of {tensor_bytes >> 20} MB per launch, larger than L2"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": None, "peak_source": f"{peaks['source']} copy bandwidth",
                         "kernel": name, "bytes_per_launch": n_tensors * tensor_bytes},
            "clocks": clocks, "gpu_launches": args.steps,
        }), flush=True)


if __name__ == "__main__":
    a = parse_args()
    VARIANT["D"], VARIANT["causal"] = a.head_dim, a.causal
    if a.impl == "reference":
        run_reference(a)
    elif a.impl == "reference_gpu" and a.workload != "attention":
        print(json.dumps({"impl": "reference_gpu", "unavailable": "the comparator covers the attention workload only"}))
    elif a.workload == "fbcache":
        run_fbcache_kernels(a)
    elif a.workload != "attention":
        run_dit(a)
    else:
        run_ours(a)
