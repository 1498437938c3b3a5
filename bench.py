#!/usr/bin/env python
"""Benchmark of the Delta Memory hot path: one step = the gated delta-rule forward (chunk
checkpoints every 64 tokens) plus the BPTT backward over one batch of synthetic input.

Workload (the isolated delta op of the baseline configuration list): B=8 sequences, H=16
heads, T=4096 tokens, dh=128, q/k L2-normalised N(0,1), v ~ N(0,1), alpha = sigmoid(N(2,.5)),
beta = sigmoid(N(0,1)), dO ~ N(0,1); seeded synthetic data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype bf16|f32] [--impl ours|reference]

Default mode: bf16 activations (tcgen05 tensor cores, f32 accumulation, f32 recurrent state and
gates; parity tolerance 2e-2). --dtype f32 runs the f32-exact FFMA kernels (tolerance 1e-5).

Under torchrun every rank owns its own batch of B sequences (weak scaling, no collective on the
data path: chains are independent per (sequence, head)). Timing: CUDA events on the launching
stream, barrier + synchronize on both sides, max over ranks. The inputs (4 x 268 MB in f32)
are larger than the 126 MB L2, so no flush is needed between iterations.

`--impl reference` times the reference's own CPU algorithm for the same path (its Rust crate
cannot be built here, so this is the C++ restatement under oracle/) on the host cores, on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

B, H, T, DH, CHUNK = 8, 16, 4096, 128, 64
METRIC = "delta fwd+bwd tok/s"
WORKLOAD = f"isolated gated delta-rule op fwd+BPTT: B{B} H{H} T{T} dh{DH} chunk{CHUNK} per GPU"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle reasons sampled every 2 ms (NVML, read-only) while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index = index
        self.sm, self.mask, self.mx = [], 0, None
        self._stop = threading.Event()
        self._th = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            # CUDA_VISIBLE_DEVICES may renumber devices: match by the UUID torch reports
            import torch

            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            self.h = None
            for i in range(pynvml.nvmlDeviceGetCount()):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                u = pynvml.nvmlDeviceGetUUID(h)
                u = u.decode() if isinstance(u, bytes) else u
                if uuid in u:
                    self.h = h
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.nv = pynvml
            self.mx = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # noqa: BLE001
            self.err = repr(e)
            self.nv = None
            return
        self._th = threading.Thread(target=self._run, daemon=True)
        self._th.start()

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.002)

    def stop(self):
        if self._th is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + getattr(self, "err", "")]}
        self._stop.set()
        self._th.join()
        reasons = sorted(n for bit, n in self.REASONS.items() if self.mask & bit)
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.mx, "reasons": reasons,
                "samples": len(self.sm)}


def make_inputs(seed: int, b: int, t: int, h: int, dh: int):
    """Seeded synthetic inputs with the workload's distributions (numpy, host)."""
    rs = np.random.RandomState(seed)
    n, d = b * t, h * dh
    q = rs.standard_normal((n, h, dh)).astype(np.float32)
    k = rs.standard_normal((n, h, dh)).astype(np.float32)
    qn = np.linalg.norm(q, axis=-1).astype(np.float32)
    kn = np.linalg.norm(k, axis=-1).astype(np.float32)
    q = (q / qn[..., None]).reshape(n, d)
    k = (k / kn[..., None]).reshape(n, d)
    v = rs.standard_normal((n, d)).astype(np.float32)
    d_o = rs.standard_normal((n, d)).astype(np.float32)
    alpha = (1 / (1 + np.exp(-(2 + 0.5 * rs.standard_normal((n, h)))))).astype(np.float32)
    beta = (1 / (1 + np.exp(-rs.standard_normal((n, h))))).astype(np.float32)
    return q, k, v, alpha, beta, qn, kn, d_o


# ------------------------------------------------------------------ reference arm (CPU)
def cpu_sample(threads: int):
    """Bounded sample of the same workload: T tokens of dh=128 chains, one chain per host thread
    (the reference's BPTT partitioning, rust/src/delta.rs:461-475), full sequence length cut to
    keep the run at 10-30 s. Threads are capped at 64: every running chain holds its own
    (T+1)*dh*dh state history (268 MB at T=4096)."""
    import oracle

    oracle.build()
    t_s = T
    h_s = max(threads, 1)
    arrs = make_inputs(1, 2, t_s, h_s, DH)
    return oracle, arrs, (2, t_s, h_s, DH)


def time_cpu(steps: int, warmup: int):
    threads = min(os.cpu_count() or 1, 64)
    oracle, arrs, (b, t, h, dh) = cpu_sample(threads)
    q, k, v, alpha, beta, qn, kn, d_o = arrs

    def step():
        oracle.delta_scan(q, k, v, alpha, beta, b, t, h, dh)
        oracle.delta_bptt(q, k, v, alpha, beta, qn, kn, d_o, b, t, h, dh, max_workers=threads)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    chain_steps = b * t * h
    tok_s = chain_steps / H / dt  # a workload token carries H=16 heads
    sample = (f"{b * h} chains x {t} tokens, dh={dh}, scan + BPTT with per-chain state history, one chain per thread; "
              f"tok/s = chain-steps/s / {H} heads")
    return tok_s, dt * 1e3, threads, sample


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(args.steps, 1), max(args.warmup, 0)
    steps = min(steps, 5)
    tok_s, ms, threads, sample = time_cpu(steps, min(warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": min(warmup, 1), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# dram__bytes_read.sum + dram__bytes_write.sum of one launch at B=2, H=16, T=4096, dh=128 (32 chains), divided by 32:
# traffic is proportional to the number of chains (profiles/delta_tc_bf16_cfg2.md).
NCU_TRAFFIC_PER_CHAIN = {
    ("bf16", "delta_bwd_tc_kernel"): (438.934784e6 + 179.197440e6) / 32,
    ("bf16", "delta_fwd_tc_kernel"): (151.054336e6 + 63.292160e6) / 32,
    ("bf16", "delta_prep_tc_kernel"): (102.092288e6 + 310.865920e6) / 32,
}


# ------------------------------------------------------------------ our arm (GPU)
def run_ours(args):
    import torch
    import torch.distributed as dist

    import asca_b200
    from asca_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    gpu = asca_b200.Gpu(local)
    gpu.use_torch_stream()
    dev = torch.device("cuda", local)
    bf16 = args.dtype == "bf16"
    b, t, h, dh = args.batch, args.seq, H, DH

    host = make_inputs(1234 + rank, b, t, h, dh)
    pin = [torch.from_numpy(a).pin_memory() for a in host]
    q, k, v, alpha, beta, qn, kn, d_o = (x.to(dev) for x in pin)
    if bf16:
        q, k, v, d_o = (x.bfloat16() for x in (q, k, v, d_o))
    n, d = b * t, h * dh
    f32 = dict(dtype=torch.float32, device=dev)
    o = torch.empty_like(q)
    ckpt = torch.empty(ops.delta_ckpt_floats(gpu, b, t, h, dh, CHUNK), **f32)
    d_qkv = torch.empty((n, 3 * d), **f32)
    d_gate = torch.empty((n, 2 * h), **f32)

    def step(ev=None):
        if ev:
            ev[0].record()
        ops.delta_fwd(gpu, q, k, v, alpha, beta, b, t, h, dh, chunk=CHUNK, out=o, ckpt=ckpt)
        if ev:
            ev[1].record()
        ops.delta_bwd(gpu, q, k, v, alpha, beta, qn, kn, d_o, ckpt, b, t, h, dh, chunk=CHUNK, d_qkv=d_qkv,
                      d_gate=d_gate)
        if ev:
            ev[2].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = gpu.launch_count()
    gpu.profile(True)   # CUDA events around every delta kernel launch, on the launching stream
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(evs[i])
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = gpu.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    per_kernel = {}
    for name, ms in gpu.profile_read():
        per_kernel.setdefault(name, []).append(ms)
    gpu.profile(False)
    fwd_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in evs]))
    bwd_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in evs]))
    if world > 1:
        tt = torch.tensor([ms_total], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total = float(tt.item())
    ms_step = ms_total / args.steps
    tok_s = world * b * t / (ms_step * 1e-3)

    # ---- end to end: pinned host buffers in, host results out, every copy inside the timed region
    e2e_steps = max(1, min(args.steps, 3))
    s_io = 2 if bf16 else 4
    if bf16:
        # bf16 mode: the caller holds bf16 activations; device-pointer API + explicit pinned copies
        hp = [x.bfloat16().pin_memory() if i in (0, 1, 2, 7) else x for i, x in enumerate(pin)]
        o_h = torch.empty((n, d), dtype=torch.bfloat16).pin_memory()
        dqkv_h = torch.empty((n, 3 * d), dtype=torch.float32).pin_memory()
        dgate_h = torch.empty((n, 2 * h), dtype=torch.float32).pin_memory()

        pipe = ops.DeltaHostPipeline(gpu, t, h, dh, chunk=CHUNK, dtype=torch.bfloat16)

        def e2e_step():
            pipe.run(hp[0], hp[1], hp[2], hp[3], hp[4], hp[5], hp[6], hp[7], o_h, dqkv_h, dgate_h, b)

        h2d = sum(x.numel() * x.element_size() for x in hp)
        d2h = sum(x.numel() * x.element_size() for x in (o_h, dqkv_h, dgate_h))
        api = "asca_b200.ops.DeltaHostPipeline (device-pointer C ABI; per-sequence copy/compute/copy pipeline from pinned host memory)"
    else:
        # f32 mode: the host-pointer API with the reference's call shape (Gpu.delta_scan + Gpu.delta_bwd_dev)
        hq, hk, hv, ha, hb, hqn, hkn, hdo = (x.numpy() for x in pin)
        o_h = torch.empty((n, d), dtype=torch.float32).pin_memory().numpy()
        dqkv_h = torch.empty((n, 3 * d), dtype=torch.float32).pin_memory().numpy()
        dgate_h = torch.empty((n, 2 * h), dtype=torch.float32).pin_memory().numpy()
        del q, k, v, d_o, o, ckpt, d_qkv, d_gate
        torch.cuda.empty_cache()

        def e2e_step():
            _, dd = gpu.delta_scan(hq, hk, hv, ha, hb, b, t, h, dh, out=o_h)
            gpu.delta_bwd_dev(dd, hdo, hqn, hkn, out=(dqkv_h, dgate_h))
            dd.free()

        h2d = sum(a.nbytes for a in (hq, hk, hv, ha, hb, hdo, hqn, hkn))
        d2h = o_h.nbytes + dqkv_h.nbytes + dgate_h.nbytes
        api = "asca_b200.Gpu.delta_scan + delta_bwd_dev (host-pointer C ABI)"
    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    if world > 1:
        tt = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item())

    if rank == 0:
        peak, which = measured_peaks()
        # algorithmic bytes of the two ops (q,k,v,o / q,k,v,dO,dq,dk,dv + gates), s_io bytes per activation
        bwd_bytes = 4 * n * d * s_io + 3 * n * d * 4 + 6 * n * h * 4
        fwd_bytes = 4 * n * d * s_io + 2 * n * h * 4
        kern_ms = {name: float(np.mean(v)) for name, v in per_kernel.items()}
        kern_n = {name: len(v) for name, v in per_kernel.items()}
        total_k = sum(float(np.sum(v)) for v in per_kernel.values()) or 1.0
        share = {name: float(np.sum(v)) / total_k for name, v in per_kernel.items()}
        top = max(share, key=share.get)
        # the dominant kernel: the backward chain kernel moves the whole backward's algorithmic bytes
        top_bytes = bwd_bytes if "bwd" in top else fwd_bytes
        achieved = top_bytes / (kern_ms[top] * 1e-3) / 1e9
        cpu_tok, cpu_ms, cores, sample = time_cpu(1, 1) if world == 1 and not args.no_cpu else (None, None, 0, "skipped")
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if bf16 else "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD if (b, t) == (B, T) else f"delta fwd+BPTT B{b} H{h} T{t} dh{dh} chunk{CHUNK}",
                       "mode": ("bf16 activations on tcgen05 tensor cores, f32 accumulate, f32 state and gates"
                                if bf16 else "f32 activations and arithmetic (FFMA)"),
                       "l2": "inputs larger than L2 (no flush)", "parallelism": f"dp{world} by sequence, no collective"},
            "ops_ms": {"delta_fwd": fwd_ms, "delta_bwd": bwd_ms},
            "kernels_ms": kern_ms, "kernel_launches_per_step": {k_: v_ / args.steps for k_, v_ in kern_n.items()},
            "kernel_share": share,
            "roofline": {"kernel": top, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": which,
                         "traffic": NCU_TRAFFIC_PER_CHAIN.get((args.dtype, top), 0) * b * h * t / 4096 or None,
                         "algorithmic_bytes": top_bytes,
                         "note": "algorithmic bytes of the op the kernel belongs to / that kernel's mean CUDA-event time; "
                                 "traffic = dram bytes read + written per launch, from one ncu capture at B=2 scaled by the "
                                 "number of (sequence, head) chains (profiles/)"},
            "cpu_baseline": {"value": cpu_tok, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": world * b * t / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "api": api},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bf16", choices=["f32", "bf16"])
    ap.add_argument("--batch", type=int, default=B)
    ap.add_argument("--seq", type=int, default=T)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_ours(args)


if __name__ == "__main__":
    main()
