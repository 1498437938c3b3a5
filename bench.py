#!/usr/bin/env python
"""Benchmark of the Delta Memory + hash-MoE hot path on B200: the training step, batched decode, and the two
isolated ops, each with its roofline, beside the reference's CPU path timed on the host cores of the same box.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--only train,decode,moe,delta]
                    [--transport nccl|ce]   (N > 1: the sharded expert tensors on NCCL kernels, the default, or on the copy engines)
    python bench.py --case gemm_dense|gemm_dense_nt|gemm_dense_tn|moe_fwd|moe_bwd|moe_bwd_8seq|delta_bf16|delta_bf16_dh64|delta_f32|decode|...
                                                                                             (one kernel family, for profiler captures)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        bench.py --gpus N --steps K --warmup W

Headline (the JSON line's top level): **train tok/s** of the 1.3B-class architecture (d 2048, 16 heads of 128, 64
hash experts of 2048 -> 4096 -> 2048, byte vocabulary; bf16 compute, f32 recurrent state, f32 master weights and
AdamW) cut to --layers blocks (24 blocks are 26 B parameters x 18 bytes and fit no GPU; every block costs the same,
so `extrapolated_24_blocks_tok_s` = value x layers / 24). One step = forward + BPTT + optimizer over a FIXED global
batch of 64 sequences x 4096 random bytes ("scaling": "strong"), split by sequence over the ranks, micro-batches of at
most 32 sequences; at N > 1 the gradient exchange (NCCL, inside the library) is queued from inside the backward and the
optimizer is sharded over the ranks. `value` is timed with CUDA events on the launching stream; `e2e` is the same K
steps by the wall clock through the host-pointer entry point (`asca_model_forward_backward_host`: token ids and
targets are host arrays copied in every micro-batch, the loss is copied out) plus the optimizer step.

Sub-records under "records", each with its own roofline / cpu_baseline / e2e / clocks:
  decode      ~125M decode configuration: 256 streams (sharded over ranks), 512-token chunked prefill, 2048 greedy tokens
  moe         isolated hash-MoE layer, 65,536 Zipf tokens, d 1024, 64 experts of 1024 -> 4096 -> 1024, fwd + bwd   (N = 1)
  delta_bf16  isolated gated delta-rule op, B8 H16 T4096 dh128 chunk 64, fwd + BPTT, tensor-core kernels          (N = 1)
  delta_f32   the same op on the f32-exact kernels                                                                (N = 1)

Inputs are synthetic and seeded: token ids come from the reference's xorshift128+ generator
(rust/src/tensor.rs:306-337); weights and float activations are drawn on the device with torch's seeded generator
(the reference's scalar Box-Muller would need minutes for 1e9 numbers). They stand in for the TinyStories bytes the
reference trains on. Timing: >= 3 warm-up steps, CUDA events on the launching stream, barrier + synchronize on both
sides, max over ranks; every workload is far larger than the 126 MB L2, so nothing is flushed between iterations.

`--impl reference` times the reference's own CPU algorithm for the train step (its Rust crate cannot be built here:
the C++ restatement under oracle/) on all host cores, on a bounded slice (one block, one sequence of 512 tokens),
scaled linearly in tokens x blocks to the headline configuration and labelled as that.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "train tok/s (delta+hashMoE)"
TRAIN = dict(V=256, d=2048, H=16, E=64, F=4096, T=4096, global_batch=64, micro=32)
DECODE = dict(V=256, d=768, H=12, L=12, E=16, F=3072, streams=256, prefill=512, tokens=2048)
MOE = dict(n=65536, d=1024, F=4096, E=64)
DELTA = dict(B=8, H=16, T=4096, dh=128, chunk=64)
LR = 3e-4


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm": float(d["hbm_gbs"]), "burst": float(d["bf16_tflops"]), "sustained": float(d["bf16_tflops_sustained"]),
                "source": "measured"}
    return {"hbm": 6650.0, "burst": 1590.0, "sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle reasons sampled every 2 ms (NVML, read-only) while a timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index = index
        self.sm, self.mask, self.mx = [], 0, None
        self._stop = threading.Event()
        self._th = None

    def start(self):
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)   # CUDA_VISIBLE_DEVICES may renumber devices
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
            return self
        self._th = threading.Thread(target=self._run, daemon=True)
        self._th.start()
        return self

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


def reference_ids(seed: int, n: int, below: int = 256) -> np.ndarray:
    """n token ids from the reference's generator (`rng.below`, rust/src/tensor.rs:322-324)."""
    from asca_b200.train import Rng

    r = Rng(seed)
    return np.fromiter((r.below(below) for _ in range(n)), dtype=np.uint32, count=n)


def zipf_ids(seed: int, n: int, s: float = 1.1) -> np.ndarray:
    """Byte ids with Zipf(s) popularity over ranks 1..256 (id = rank - 1), inverse CDF of the reference's `rng.uniform()`."""
    from asca_b200.train import Rng

    w = 1.0 / np.arange(1, 257) ** s
    cdf = np.cumsum(w) / w.sum()
    r = Rng(seed)
    u = np.fromiter((r.uniform() for _ in range(n)), dtype=np.float64, count=n)
    return np.minimum(np.searchsorted(cdf, u), 255).astype(np.uint32)


class Harness:
    """Process-wide plumbing: ranks, the library context, torch.distributed for barriers and max-over-ranks."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        import asca_b200

        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the hot path has no CPU fallback")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.gpu = asca_b200.Gpu(self.local)
        self.gpu.use_torch_stream()
        self.peaks = peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return float(x)
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps, warmup, sample_clocks=True):
        """W untimed calls, then K calls between CUDA events on the launching stream and by the wall clock, barrier +
        synchronize on both sides, max over ranks. Returns (device ms per call, wall ms per call, clocks, launches)."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        self.barrier()
        sampler = ClockSampler(self.local).start() if (sample_clocks and self.rank == 0) else None
        l0 = self.gpu.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        wall = (time.perf_counter() - t0) * 1e3 / steps
        dev_ms = e0.elapsed_time(e1) / steps
        clocks = sampler.stop() if sampler else None
        return self.max_over_ranks(dev_ms), self.max_over_ranks(wall), clocks, self.gpu.launch_count() - l0

    def kernel_table(self, fn):
        """One extra call with the library's per-launch CUDA events on: {kernel: (launches, total ms, total work)}."""
        self.gpu.profile(True)
        fn()
        self.torch.cuda.synchronize()
        tab = {}
        for name, ms, work in self.gpu.profile_read(with_work=True):
            n, t, w = tab.get(name, (0, 0.0, 0.0))
            tab[name] = (n + 1, t + ms, w + work)
        self.gpu.profile(False)
        return tab

    def fill_normal(self, ptr, n, seed, scale=0.02):
        """n f32 numbers N(0, scale) written at device address ptr (seeded, identical on every rank)."""
        from asca_b200 import dp

        torch = self.torch
        g = torch.Generator(device=self.dev).manual_seed(seed)
        t = dp.device_tensor(ptr, n, self.local)
        for lo in range(0, n, 1 << 28):
            hi = min(n, lo + (1 << 28))
            t[lo:hi] = torch.randn(hi - lo, generator=g, dtype=torch.float32, device=self.dev) * scale


# ------------------------------------------------------------------ CPU arm (the oracle as the timed baseline)
def cpu_threads():
    return min(os.cpu_count() or 1, 64)


def cpu_train_slice(steps=1, warmup=0, layers=1, tokens=512):
    """The restated CPU train step (forward + BPTT + AdamW) on one block, one sequence of `tokens` bytes, at the
    training configuration's widths, all host cores. Returns (seconds per step, sample description)."""
    import oracle

    oracle.build()
    oracle.set_threads(0)
    c = TRAIN
    m = oracle.Model(c["V"], c["d"], c["H"], layers, c["E"], c["F"])
    # uniform with the N(0, 0.02) standard deviation: the arithmetic does not depend on the values, and a billion
    # normals would take longer to draw than the step takes
    g = np.random.default_rng(0)
    for lo in range(0, m.n, 1 << 27):
        hi = min(m.n, lo + (1 << 27))
        m.params[lo:hi] = (g.random(hi - lo, dtype=np.float32) - 0.5) * np.float32(0.02 * math.sqrt(12.0))
    ids = reference_ids(1, tokens)
    tg = np.roll(ids, -1).astype(np.uint32)
    grads = np.zeros(m.n, np.float32)
    mo, vo = np.zeros(m.n, np.float32), np.zeros(m.n, np.float32)
    cnt = 0

    def step():
        nonlocal cnt
        grads[:] = 0
        m.forward_backward(ids, tg, 1, grads=grads)
        cnt = m.adamw_step(grads, mo, vo, cnt, LR)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return dt, (f"{layers} block, 1 sequence x {tokens} tokens of the training configuration's widths, f32, forward + BPTT + "
                f"AdamW; scaled linearly in tokens x blocks to the benchmark's step")


def cpu_baseline_train(layers, steps=1, warmup=0):
    dt, sample = cpu_train_slice(steps, warmup, 1, 512)
    tok_s = 512.0 / (dt * layers)          # tokens/s of the `layers`-block model
    return {"value": tok_s, "unit": "tok/s", "cores": cpu_threads(), "kind": "port", "sample": sample,
            "slice_seconds_per_step": dt, "extrapolated": True}


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    steps, warmup = max(1, min(args.steps, 2)), min(max(args.warmup, 0), 1)
    base = cpu_baseline_train(args.layers, steps, warmup)
    c = TRAIN
    n_tok = c["global_batch"] * c["T"]
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tok/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": n_tok / base["value"] * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": train_config(args.layers, 1, "n/a (CPU)"),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference's CPU algorithm (C++ restatement) on a bounded slice, scaled to the configuration; "
                "steps and warm-up are capped so that the run ends within minutes",
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ train step (headline)
def train_config(layers, world, l2):
    c = TRAIN
    return {"workload": (f"ASCA 1.3B-class data-parallel training step, {layers} of 24 blocks: d {c['d']}, {c['H']} heads of "
                         f"{c['d'] // c['H']}, {c['E']} hash experts of {c['d']}->{c['F']}->{c['d']}, byte vocabulary; global batch "
                         f"{c['global_batch']} x {c['T']} random bytes; forward + BPTT + AdamW"),
            "layers": layers, "global_batch": c["global_batch"], "seq_len": c["T"],
            "parallelism": f"dp{world} by sequence; heads and experts local; NCCL gradient exchange overlapped with the backward"
                           + ("; optimizer sharded over the ranks" if world > 1 else ""),
            "l2": l2}


def train_flop_per_token(layers):
    c = TRAIN
    d, H, F, V = c["d"], c["H"], c["F"], c["V"]
    per_layer = d * 3 * d + d * 2 * H + d * d + 2 * d * F          # GEMM parameters a token touches per block
    return 6 * (layers * per_layer + d * V) + 22 * (d // H) ** 2 * H * layers


def run_train(hs: Harness, args):
    import asca_b200
    from asca_b200 import dp

    torch = hs.torch
    c = TRAIN
    L = args.layers
    own = dp.shard_sequences(c["global_batch"], hs.rank, hs.world)
    n_micro = max(1, -(-len(own) // c["micro"]))
    mb = len(own) // n_micro
    assert mb * n_micro == len(own), "the rank's share must be a whole number of micro-batches"
    model = asca_b200.Model(hs.gpu, c["V"], c["d"], c["H"], L, c["E"], c["F"])
    model.set_compute(asca_b200.BF16)
    hs.fill_normal(model.buffers()[0], model.n, seed=0)
    model.params_changed()
    ids_all = reference_ids(1, c["global_batch"] * c["T"]).reshape(c["global_batch"], c["T"])
    ids = torch.from_numpy(ids_all[own.start:own.stop].astype(np.int32)).pin_memory()
    tg = torch.roll(ids, -1, dims=1).contiguous().pin_memory()
    ids_np, tg_np = ids.numpy().view(np.uint32), tg.numpy().view(np.uint32)
    model.set_grad_scale(1.0 / n_micro)
    comm = dp.Comm.from_torch(hs.gpu)
    ov = dp.ShardedOverlap(model, comm, transport=args.transport) if hs.world > 1 else dp.GradOverlap(model, comm)
    last = {"loss": float("nan")}

    def step():
        model.zero_grads()
        loss = 0.0
        for i in range(n_micro):
            rows = slice(i * mb, (i + 1) * mb)
            if i == n_micro - 1:
                with ov:
                    loss += model.forward_backward(ids_np[rows].reshape(-1), tg_np[rows].reshape(-1), mb)
            else:
                loss += model.forward_backward(ids_np[rows].reshape(-1), tg_np[rows].reshape(-1), mb)
        ov.step(LR)
        last["loss"] = loss / n_micro

    first_loss = None
    step()
    torch.cuda.synchronize()
    first_loss = last["loss"]
    dev_ms, wall_ms, clocks, launches = hs.timed(step, args.steps, max(args.warmup - 1, 2))
    # exposed collectives, per step, max over ranks (two more steps; reading the events synchronises)
    tl = {}
    for _ in range(2):
        step()
        t = ov.timeline()
        for k, v in t.items():
            tl[k] = max(tl.get(k, 0.0), hs.max_over_ranks(v))
    free_b, total_b = torch.cuda.mem_get_info()
    table = hs.kernel_table(step)      # every rank: the step holds collectives
    n_tok = c["global_batch"] * c["T"]
    flop_tok = train_flop_per_token(L)
    tf_per_gpu = n_tok * flop_tok / (dev_ms * 1e-3) / 1e12 / hs.world
    rec = None
    if hs.rank == 0:
        pk = hs.peaks
        total_k = sum(t for _, t, _ in table.values()) or 1.0
        kernels = {k: {"launches": n, "ms": round(t, 3), "share_of_profiled": round(t / total_k, 4),
                       **({"TFLOP/s": round(w / (t * 1e-3) / 1e12, 1)} if "gemm_tc" in k and t > 0 else {}),
                       **({"GB/s": round(w / (t * 1e-3) / 1e9, 1)} if "adamw" in k and t > 0 else {})}
                   for k, (n, t, w) in sorted(table.items(), key=lambda kv: -kv[1][1])}
        top = max(table, key=lambda k: table[k][1])
        n_top, t_top, w_top = table[top]
        top_tf = w_top / (t_top * 1e-3) / 1e12 if "gemm_tc" in top else None
        h2d = 2 * len(own) * c["T"] * 4
        rec = {
            "metric": METRIC, "value": n_tok / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": hs.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": train_config(L, hs.world, "activations and weights of a step (tens of GB) far exceed L2; no flush"),
            "extrapolated_24_blocks_tok_s": n_tok / (dev_ms * 1e-3) * L / 24,
            "micro_batches_per_rank": n_micro, "sequences_per_micro_batch": mb, "params": model.n,
            "loss_first_step": first_loss, "loss_last_step": last["loss"],
            "roofline": {"bound": "tensor", "achieved": tf_per_gpu, "peak": pk["sustained"], "unit": "TFLOP/s",
                         "frac": tf_per_gpu / pk["sustained"], "frac_of_burst": tf_per_gpu / pk["burst"], "peak_source": pk["source"],
                         "algorithmic_flop_per_token": flop_tok,
                         # dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel at the captured case
                         # (bench.py --case gemm_dense: 32768 x 6144 x 2048, CTA pairs; profiles/): 224 + 765 MB per launch
                         # against 964 MB algorithmic (A and B once as bf16, C once as f32)
                         "traffic": 989.0e6, "traffic_algorithmic_bytes": 964.7e6, "traffic_case": "bench.py --case gemm_dense",
                         "note": "whole step per GPU: 6 x GEMM parameters a token touches + 22 dh^2 H per block for the recurrence, "
                                 "/ CUDA-event step time / the sustained cuBLAS bf16 figure (a kernel timed inside a long step); "
                                 "dominant kernel below against the burst figure (timed alone by its own events)",
                         "dominant_kernel": {"kernel": top, "launches_per_step": n_top, "ms_per_step": t_top,
                                             "achieved": top_tf, "unit": "TFLOP/s", "peak": pk["burst"],
                                             "frac": (top_tf / pk["burst"]) if top_tf else None}},
            "timeline_ms": {**{k: round(v, 3) for k, v in tl.items()},
                            "note": "per step, max over ranks: how long the end of the backward waited for the gradient exchange, the "
                                    "optimizer update, how long the bf16 weight all-gather ran past the update, and how long the next "
                                    "forward waited for gathered weights; the rest of the step is compute"},
            "kernels_profiled_step": kernels,
            "e2e": {"value": n_tok / (wall_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d * hs.world,
                    "d2h_bytes_per_step": 4 * n_micro * hs.world, "ms_per_step": wall_ms,
                    "api": "asca_model_forward_backward_host (host token ids and targets in, loss out, every micro-batch) + "
                           "asca_model_dp_step; wall clock over the same K steps"},
            "gpu_launches": launches, "clocks": clocks,
            "device_memory_gb": {"used": round((total_b - free_b) / 1e9, 1), "total": round(total_b / 1e9, 1)},
        }
    ov.detach()
    comm.close()
    model.free()
    hs.gpu.lib.asca_ctx_trim(hs.gpu._ctx)
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------ decode
def cpu_baseline_decode():
    """The restated CPU decode (Model::step per stream, f32) on min(cores, 16) streams x 6 tokens, one thread per stream."""
    import oracle

    oracle.build()
    c = DECODE
    m = oracle.Model(c["V"], c["d"], c["H"], c["L"], c["E"], c["F"])
    g = np.random.default_rng(0)
    for lo in range(0, m.n, 1 << 27):
        hi = min(m.n, lo + (1 << 27))
        m.params[lo:hi] = (g.random(hi - lo, dtype=np.float32) - 0.5) * np.float32(0.02 * math.sqrt(12.0))
    n_streams, n_tok = min(cpu_threads(), 16), 6
    oracle.set_threads(1)
    states = [m.new_decode_state() for _ in range(n_streams)]
    toks = reference_ids(3, n_streams * n_tok).reshape(n_streams, n_tok)

    def run(s):
        for t in range(n_tok):
            m.step(int(toks[s, t]), states[s])

    run(0)
    t0 = time.perf_counter()
    ths = [threading.Thread(target=run, args=(s,)) for s in range(n_streams)]
    for th in ths:
        th.start()
    for th in ths:
        th.join()
    dt = time.perf_counter() - t0
    oracle.set_threads(0)
    return {"value": n_streams * n_tok / dt, "unit": "tok/s", "cores": n_streams, "kind": "port",
            "sample": f"{n_streams} streams x {n_tok} tokens, one stream per thread, f32 Model::step of the decode configuration"}


def run_decode(hs: Harness, args):
    import asca_b200
    from asca_b200 import dp

    torch = hs.torch
    c = DECODE
    V, d, H, L, E, F = c["V"], c["d"], c["H"], c["L"], c["E"], c["F"]
    dh = d // H
    own = dp.shard_sequences(c["streams"], hs.rank, hs.world)
    ns = len(own)
    model = asca_b200.Model(hs.gpu, V, d, H, L, E, F)
    model.set_compute(asca_b200.BF16)
    hs.fill_normal(model.buffers()[0], model.n, seed=0)
    model.params_changed()
    prompts = reference_ids(2, c["streams"] * c["prefill"]).reshape(c["streams"], c["prefill"])[own.start:own.stop]
    state = model.new_decode_state(ns)
    # prefill: one chunked call (asca_model_prefill_host) where the reference's decoder steps token by token
    # (rust/src/main.rs:367-371); timed by the wall clock and reported beside the decode figure, not part of it
    prompts = np.ascontiguousarray(prompts)
    model.prefill(model.new_decode_state(ns), prompts[:, :64].copy(), want_logits=False)     # warm-up on a short prompt
    hs.barrier()
    t0 = time.perf_counter()
    _, nxt = model.prefill(state, prompts, want_logits=False)
    torch.cuda.synchronize()
    prefill_ms = hs.max_over_ranks((time.perf_counter() - t0) * 1e3)
    cur = {"ids": nxt}
    chunk = 64

    fed = []      # the ids every timed step consumed (its expert routing decides which weights the step must read)

    def greedy_chunk():
        toks = model.decode_greedy(state, cur["ids"], chunk)
        fed.append(np.concatenate([cur["ids"][None, :], toks[:-1]], axis=0))
        cur["ids"] = toks[-1]

    n_chunks = c["tokens"] // chunk
    dev_ms, wall_ms, clocks, launches = hs.timed(greedy_chunk, n_chunks, 3)
    ms_step, wall_step = dev_ms / chunk, wall_ms / chunk
    table = hs.kernel_table(lambda: model.decode_greedy(state, cur["ids"], 4)) if hs.rank == 0 else None
    rec = None
    if hs.rank == 0:
        pk = hs.peaks
        state_bytes = 2 * L * H * dh * dh * 4 * ns
        # weights a step must read: the dense ones, and W1 / W2 of the experts its tokens route to
        # (hash_route, rust/src/model.rs:69-77) -- counted from the ids the timed steps actually consumed
        ids_fed = np.concatenate(fed[-n_chunks:], axis=0).astype(np.uint64)
        hsh = (ids_fed * 0x9E3779B1) & 0xFFFFFFFF
        hsh ^= hsh >> 15
        hsh = (hsh * 0x85EBCA6B) & 0xFFFFFFFF
        hsh ^= hsh >> 13
        experts_hit = float(np.mean([np.unique(r).size for r in (hsh % E)]))
        weight_bytes_all = (L * (d * 3 * d + d * 2 * H + d * d + 2 * E * d * F) + d * V) * 2
        weight_bytes = int((L * (d * 3 * d + d * 2 * H + d * d + 2 * experts_hit * d * F) + d * V) * 2)
        step_bytes = state_bytes + weight_bytes
        gbs = step_bytes / (ms_step * 1e-3) / 1e9
        total_k = sum(t for _, t, _ in table.values()) or 1.0
        top = max(table, key=lambda k: table[k][1])
        n_top, t_top, w_top = table[top]
        kernels = {k: {"launches": n // 4, "ms_per_step": round(t / 4, 4), "share_of_profiled": round(t / total_k, 4),
                       "GB/s": round(w / (t * 1e-3) / 1e9, 1) if w else None}
                   for k, (n, t, w) in sorted(table.items(), key=lambda kv: -kv[1][1])}
        rec = {
            "metric": "decode tok/s", "value": c["streams"] * 1e3 / ms_step, "unit": "tok/s", "n_gpus": hs.world,
            "steps": c["tokens"], "ms_per_step": ms_step, "scaling": "strong", "dtype": "bf16",
            "config": {"workload": (f"ASCA ~125M greedy decode: {L} blocks, d {d}, {H} heads of {dh}, {E} hash experts of {d}->{F}->{d}, bf16 "
                                    f"weights; {c['streams']} streams sharded over {hs.world} GPU(s), {c['prefill']}-token prefill (chunked, "
                                    f"outside the timed region), {c['tokens']} greedy tokens timed"),
                       "streams_per_gpu": ns, "steps_per_call": chunk,
                       "prefill": f"one chunked asca_model_prefill_host call per rank, {c['prefill']} tokens x {ns} streams",
                       "l2": "a step reads 1.9 GB of weights and 1.2 GB of state: far larger than L2, no flush"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s", "frac": gbs / pk["hbm"],
                         "peak_source": pk["source"], "algorithmic_bytes": step_bytes, "state_bytes": state_bytes,
                         "weight_bytes": weight_bytes, "experts_hit_per_step": experts_hit, "weight_bytes_if_all_experts_hit": weight_bytes_all,
                         "frac_if_all_experts_hit": (state_bytes + weight_bytes_all) / (ms_step * 1e-3) / 1e9 / pk["hbm"], "traffic": None,
                         "note": "per GPU and step: recurrent state read + written once (2 L H dh^2 4 B per stream) + every bf16 weight "
                                 "byte the step needs once (dense weights + W1, W2 of the experts the step's tokens route to, counted from "
                                 "the ids the timed steps consumed) / CUDA-event time of a step",
                         "dominant_kernel": {"kernel": top, "ms_per_step": t_top / 4,
                                             "achieved": (w_top / (t_top * 1e-3) / 1e9) if w_top else None, "unit": "GB/s",
                                             "note": "from a separate pass with per-launch events, which serialises the chain"}},
            "kernels_profiled_step": kernels,
            "e2e": {"value": c["streams"] * 1e3 / wall_step, "unit": "tok/s", "h2d_bytes_per_step": 4 * ns * hs.world / chunk,
                    "d2h_bytes_per_step": 4 * ns * hs.world, "ms_per_step": wall_step,
                    "api": "asca_model_decode_greedy_host: ids in from the host, the chosen tokens of every step back to the host, "
                           f"one call per {chunk} steps; wall clock"},
            "prefill": {"ms": prefill_ms, "tok_s": c["streams"] * c["prefill"] / (prefill_ms * 1e-3),
                        "note": "chunked prefill of all streams (untimed part of the decode record); stepping the same "
                                f"prompt would take {c['prefill']} decode steps"},
            "gpu_launches": launches, "clocks": clocks,
            "cpu_baseline": cpu_baseline_decode() if (hs.world == 1 and not args.no_cpu) else None,
        }
    model.free()
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------ isolated hash-MoE layer
def run_moe(hs: Harness, args):
    from asca_b200 import ops

    torch = hs.torch
    c = MOE
    n, d, F, E = c["n"], c["d"], c["F"], c["E"]
    dev = hs.dev
    f32 = dict(dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)
    ids_h = zipf_ids(4, n)
    ids = torch.from_numpy(ids_h.view(np.int32)).to(dev)
    xn = torch.randn(n, d, generator=g, **f32).bfloat16()
    w1 = (torch.randn(d, E * F, generator=g, **f32) * 0.02).bfloat16()
    w2 = (torch.randn(E * F, d, generator=g, **f32) * 0.02).bfloat16()
    b1, b2 = torch.zeros(E * F, **f32), torch.zeros(d, **f32)
    dout = torch.randn(n, d, generator=g, **f32)
    perm, off = ops.moe_dispatch(hs.gpu, ids, E)
    out, pre_p, hid_p = ops.moe_fwd(hs.gpu, xn, w1, b1, w2, b2, perm, off, F, E)
    grads = ops.moe_bwd(hs.gpu, xn, w1, w2, pre_p, hid_p, dout, perm, off, F, E)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    acc = {"fwd": 0.0, "bwd": 0.0, "n": 0}

    def step():
        ev[0].record()
        ops.moe_dispatch(hs.gpu, ids, E)
        ops.moe_fwd(hs.gpu, xn, w1, b1, w2, b2, perm, off, F, E, out=out, pre_p=pre_p, hid_p=hid_p)
        ev[1].record()
        ops.moe_bwd(hs.gpu, xn, w1, w2, pre_p, hid_p, dout, perm, off, F, E, grads=grads)
        ev[2].record()

    dev_ms, _, clocks, launches = hs.timed(step, 150, 3)
    for _ in range(5):
        step()
        torch.cuda.synchronize()
        acc["fwd"] += ev[0].elapsed_time(ev[1])
        acc["bwd"] += ev[1].elapsed_time(ev[2])
        acc["n"] += 1
    table = hs.kernel_table(step)
    # end to end: host ids, activations and upstream gradient in; outputs and input gradient out (weights stay resident)
    ids_p = torch.from_numpy(ids_h.view(np.int32)).pin_memory()
    xn_p, dout_p = xn.cpu().pin_memory(), dout.cpu().pin_memory()
    out_p, dxn_p = torch.empty((n, d)).pin_memory(), torch.empty((n, d)).pin_memory()

    def e2e_step():
        ids.copy_(ids_p, non_blocking=True)
        xn.copy_(xn_p, non_blocking=True)
        dout.copy_(dout_p, non_blocking=True)
        step()
        out_p.copy_(out, non_blocking=True)
        dxn_p.copy_(grads[4], non_blocking=True)
        torch.cuda.synchronize()

    _, e2e_ms, _, _ = hs.timed(e2e_step, 10, 2, sample_clocks=False)
    pk = hs.peaks
    flop = 12.0 * n * d * F
    tf = flop / (dev_ms * 1e-3) / 1e12
    total_k = sum(t for _, t, _ in table.values()) or 1.0
    top = max(table, key=lambda k: table[k][1])
    n_top, t_top, w_top = table[top]
    cpu = None
    if not args.no_cpu:
        import oracle

        oracle.build()
        oracle.set_threads(0)
        ns = 2048
        sel = np.arange(0, n, n // ns)[:ns]
        t0 = time.perf_counter()
        oracle.moe_forward_backward(xn[sel].float().cpu().numpy(), w1.float().cpu().numpy(), b1.cpu().numpy(), w2.float().cpu().numpy(),
                                    b2.cpu().numpy(), ids_h[sel].copy(), dout[sel].cpu().numpy(), F, E)
        dt = time.perf_counter() - t0
        cpu = {"value": ns / dt, "unit": "tok/s", "cores": cpu_threads(), "kind": "port",
               "sample": f"{ns} of the 65,536 tokens (every 32nd) through the restated f32 HashMoe forward + backward with the full weights"}
    return {
        "metric": "hash-MoE layer fwd+bwd tok/s", "value": n * 1e3 / dev_ms, "unit": "tok/s", "n_gpus": 1, "steps": 150, "ms_per_step": dev_ms,
        "ops_ms": {"dispatch+fwd": acc["fwd"] / acc["n"], "bwd": acc["bwd"] / acc["n"]}, "dtype": "bf16",
        "config": {"workload": f"isolated hash-MoE layer: {n} tokens, byte ids Zipf(1.1), d {d}, {E} experts of {d}->{F}->{d}, bf16 weights "
                               "N(0,0.02), activations N(0,1); dispatch + grouped expert FFN + combine, forward + backward",
                   "l2": "weights 1.07 GB, activations 0.8 GB per pass: larger than L2, no flush"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["sustained"], "unit": "TFLOP/s", "frac": tf / pk["sustained"],
                     "frac_of_burst": tf / pk["burst"], "peak_source": pk["source"], "algorithmic_flop": flop, "traffic": None,
                     "note": "4 N d F forward + 8 N d F backward / CUDA-event time of a pass",
                     "dominant_kernel": {"kernel": top, "launches_per_step": n_top, "ms_per_step": t_top,
                                         "achieved": w_top / (t_top * 1e-3) / 1e12 if w_top else None, "unit": "TFLOP/s",
                                         "peak": pk["burst"], "frac": (w_top / (t_top * 1e-3) / 1e12 / pk["burst"]) if w_top else None}},
        "kernels_profiled_step": {k: {"launches": a, "ms": round(t, 3), "share_of_profiled": round(t / total_k, 4),
                                      "TFLOP/s": round(w / (t * 1e-3) / 1e12, 1) if w else None}
                                  for k, (a, t, w) in sorted(table.items(), key=lambda kv: -kv[1][1])},
        "e2e": {"value": n * 1e3 / e2e_ms, "unit": "tok/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": ids_p.numel() * 4 + xn_p.numel() * 2 + dout_p.numel() * 4,
                "d2h_bytes_per_step": out_p.numel() * 4 + dxn_p.numel() * 4,
                "api": "asca_moe_dispatch + asca_moe_fwd + asca_moe_bwd on device buffers, pinned-host copies of ids, activations, "
                       "upstream gradient in and outputs, input gradient out inside the timed region; weights resident"},
        "gpu_launches": launches, "clocks": clocks, "cpu_baseline": cpu,
    }


# ------------------------------------------------------------------ isolated delta op
# dram__bytes_read.sum + dram__bytes_write.sum of one launch at B=2, H=16, T=4096, dh=128 (32 chains), divided by 32:
# traffic is proportional to the number of chains (profiles/delta_tc_bf16_cfg2.md).
NCU_TRAFFIC_PER_CHAIN = {
    "delta_bwd_tc_kernel": (438.934784e6 + 179.197440e6) / 32,
    "delta_fwd_tc_kernel": (151.054336e6 + 63.292160e6) / 32,
    "delta_prep_tc_kernel": (102.092288e6 + 310.865920e6) / 32,
}


def run_delta(hs: Harness, args, bf16: bool):
    from asca_b200 import ops

    torch = hs.torch
    c = DELTA
    b, h, t, dh, chunk = c["B"], c["H"], c["T"], c["dh"], c["chunk"]
    n, d = b * t, h * dh
    dev = hs.dev
    f32 = dict(dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev).manual_seed(1234)
    q = torch.randn(n, h, dh, generator=g, **f32)
    k = torch.randn(n, h, dh, generator=g, **f32)
    qn, kn = q.norm(dim=-1).contiguous(), k.norm(dim=-1).contiguous()
    q = (q / qn[..., None]).reshape(n, d).contiguous()
    k = (k / kn[..., None]).reshape(n, d).contiguous()
    v = torch.randn(n, d, generator=g, **f32)
    d_o = torch.randn(n, d, generator=g, **f32)
    alpha = torch.sigmoid(2 + 0.5 * torch.randn(n, h, generator=g, **f32))
    beta = torch.sigmoid(torch.randn(n, h, generator=g, **f32))
    host32 = [x.cpu() for x in (q, k, v, alpha, beta, qn, kn, d_o)]
    if bf16:
        q, k, v, d_o = (x.bfloat16() for x in (q, k, v, d_o))
    o = torch.empty_like(q)
    ckpt = torch.empty(ops.delta_ckpt_floats(hs.gpu, b, t, h, dh, chunk), **f32)
    d_qkv = torch.empty((n, 3 * d), **f32)
    d_gate = torch.empty((n, 2 * h), **f32)

    def step():
        ops.delta_fwd(hs.gpu, q, k, v, alpha, beta, b, t, h, dh, chunk=chunk, out=o, ckpt=ckpt)
        ops.delta_bwd(hs.gpu, q, k, v, alpha, beta, qn, kn, d_o, ckpt, b, t, h, dh, chunk=chunk, d_qkv=d_qkv, d_gate=d_gate)

    steps = 600 if bf16 else 50
    dev_ms, _, clocks, launches = hs.timed(step, steps, 3)
    table = hs.kernel_table(lambda: [step() for _ in range(5)])
    s_io = 2 if bf16 else 4
    # algorithmic bytes: q,k,v,o (+ gates) forward; q,k,v,dO in and dq,dk,dv out in the activation dtype
    # (+ gates and their gradients) backward
    fwd_bytes = 4 * n * d * s_io + 2 * n * h * 4
    bwd_bytes = 7 * n * d * s_io + 6 * n * h * 4
    top = max(table, key=lambda kk: table[kk][1])
    n_top, t_top, _ = table[top]
    top_ms = t_top / n_top
    top_bytes = bwd_bytes if "bwd" in top else fwd_bytes
    pk = hs.peaks
    achieved = top_bytes / (top_ms * 1e-3) / 1e9
    # end to end from pinned host buffers
    if bf16:
        hp = [x.bfloat16().pin_memory() if i in (0, 1, 2, 7) else x.pin_memory() for i, x in enumerate(host32)]
        o_h = torch.empty((n, d), dtype=torch.bfloat16).pin_memory()
        dqkv_h = torch.empty((n, 3 * d), dtype=torch.float32).pin_memory()
        dgate_h = torch.empty((n, 2 * h), dtype=torch.float32).pin_memory()
        pipe = ops.DeltaHostPipeline(hs.gpu, t, h, dh, chunk=chunk, dtype=torch.bfloat16)

        def e2e_step():
            pipe.run(hp[0], hp[1], hp[2], hp[3], hp[4], hp[5], hp[6], hp[7], o_h, dqkv_h, dgate_h, b)

        h2d = sum(x.numel() * x.element_size() for x in hp)
        d2h = sum(x.numel() * x.element_size() for x in (o_h, dqkv_h, dgate_h))
        api = "asca_b200.ops.DeltaHostPipeline (device-pointer C ABI; per-sequence copy/compute/copy pipeline from pinned host memory)"
    else:
        hq, hk, hv, ha, hb, hqn, hkn, hdo = (x.pin_memory().numpy() for x in host32)
        o_h = torch.empty((n, d), dtype=torch.float32).pin_memory().numpy()
        dqkv_h = torch.empty((n, 3 * d), dtype=torch.float32).pin_memory().numpy()
        dgate_h = torch.empty((n, 2 * h), dtype=torch.float32).pin_memory().numpy()

        def e2e_step():
            _, dd = hs.gpu.delta_scan(hq, hk, hv, ha, hb, b, t, h, dh, out=o_h)
            hs.gpu.delta_bwd_dev(dd, hdo, hqn, hkn, out=(dqkv_h, dgate_h))
            dd.free()

        h2d = sum(a.nbytes for a in (hq, hk, hv, ha, hb, hdo, hqn, hkn))
        d2h = o_h.nbytes + dqkv_h.nbytes + dgate_h.nbytes
        api = "asca_delta_scan_host + asca_delta_bwd_dev_host (host-pointer C ABI, the reference's call shape)"
    _, e2e_ms, _, _ = hs.timed(e2e_step, 20 if bf16 else 5, 2, sample_clocks=False)
    # CPU leg: the oracle times a bounded sample of the same chains AND checks one chain of what was just timed
    cpu, parity = None, None
    if not args.no_cpu:
        import oracle

        oracle.build()
        oracle.set_threads(0)
        threads = cpu_threads()
        hh = min(h, max(1, threads // 2))
        sl = [x.numpy().reshape(b, t, -1)[:2] for x in host32]

        def heads(a, width):
            return np.ascontiguousarray(a[:, :, : hh * width]).reshape(2 * t, hh * width)

        cq, ck_, cv, cdo = (heads(sl[i], dh) for i in (0, 1, 2, 7))
        ca, cb, cqn, ckn = (heads(sl[i], 1) for i in (3, 4, 5, 6))
        t0 = time.perf_counter()
        o_ref, _ = oracle.delta_scan(cq, ck_, cv, ca, cb, 2, t, hh, dh)
        dqkv_ref, dgate_ref = oracle.delta_bptt(cq, ck_, cv, ca, cb, cqn, ckn, cdo, 2, t, hh, dh, max_workers=threads)
        dt = time.perf_counter() - t0
        cpu = {"value": 2 * t * hh / h / dt, "unit": "tok/s", "cores": threads, "kind": "port",
               "sample": f"{2 * hh} of the {b * h} chains x {t} tokens (2 sequences x {hh} heads), scan + BPTT with per-chain state "
                         f"history, one chain per thread; tok/s = chain-steps/s / {h} heads"}
        # parity of what was just timed: sequence 0, head 0, against the CPU path on the same (unrounded) inputs
        tol = 2e-2 if bf16 else 1e-5
        got_o = o[:t, :dh].float().cpu().numpy()
        got_q = d_qkv[:t].cpu().numpy()
        ref_q = dqkv_ref[:t]

        def rel(a, r):
            return float(np.abs(a.astype(np.float64) - r).max() / max(float(np.abs(r).max()), 1e-9))

        errs = {"o": rel(got_o, o_ref[:t, :dh]), "dq": rel(got_q[:, :dh], ref_q[:, :dh]),
                "dk": rel(got_q[:, d:d + dh], ref_q[:, hh * dh:hh * dh + dh]),
                "dv": rel(got_q[:, 2 * d:2 * d + dh], ref_q[:, 2 * hh * dh:2 * hh * dh + dh]),
                "d_alpha": rel(d_gate[:t, 0].cpu().numpy(), dgate_ref[:t, 0]),
                "d_beta": rel(d_gate[:t, h].cpu().numpy(), dgate_ref[:t, hh])}
        parity = {"chain": "sequence 0, head 0 of the timed batch", "tolerance": tol, "rel_err": errs, "ok": all(e < tol for e in errs.values())}
        assert parity["ok"], f"bench: the timed delta op disagrees with the CPU path: {errs}"
    total_k = sum(tt for _, tt, _ in table.values()) or 1.0
    traffic = NCU_TRAFFIC_PER_CHAIN.get(top) if bf16 else None
    return {
        "metric": "delta fwd+bwd tok/s", "value": b * t * 1e3 / dev_ms, "unit": "tok/s", "n_gpus": 1, "steps": steps, "ms_per_step": dev_ms,
        "dtype": "bf16" if bf16 else "f32",
        "config": {"workload": f"isolated gated delta-rule op fwd+BPTT: B{b} H{h} T{t} dh{dh} chunk{chunk}",
                   "mode": ("bf16 activations on tcgen05 tensor cores, f32 accumulate, f32 state and gates" if bf16
                            else "f32 activations and arithmetic (FFMA)"),
                   "l2": "inputs (4 x 134 MB in bf16) larger than L2, no flush"},
        "kernels_ms": {kk: tt / nn for kk, (nn, tt, _) in table.items()},
        "kernel_share": {kk: tt / total_k for kk, (_, tt, _) in table.items()},
        "roofline": {"kernel": top, "bound": "hbm", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s", "frac": achieved / pk["hbm"],
                     "peak_source": pk["source"], "algorithmic_bytes": top_bytes,
                     "traffic": traffic * b * h if traffic else None,
                     "whole_step": {"algorithmic_bytes": fwd_bytes + bwd_bytes,
                                    "achieved": (fwd_bytes + bwd_bytes) / (dev_ms * 1e-3) / 1e9,
                                    "frac": (fwd_bytes + bwd_bytes) / (dev_ms * 1e-3) / 1e9 / pk["hbm"]},
                     "note": "algorithmic bytes of the op the dominant kernel belongs to (q,k,v,o + gates forward; q,k,v,dO in and "
                             "dq,dk,dv out in the activation dtype + gates backward) / that kernel's mean CUDA-event time; traffic = dram "
                             "bytes of one ncu capture at B=2 scaled by the number of chains"},
        "e2e": {"value": b * t * 1e3 / e2e_ms, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "api": api},
        "gpu_launches": launches, "clocks": clocks, "cpu_baseline": cpu, "parity_of_timed_batch": parity,
    }


# ------------------------------------------------------------------ single-kernel cases (for profiler captures)
def run_case(hs: Harness, args):
    """One small case of one kernel family, a few launches, a few GB on the device at most: what a profiler capture
    should run (`ncu -k regex:... -c 3 python bench.py --case NAME`). Prints one JSON line with the CUDA-event time."""
    import asca_b200
    from asca_b200 import ops

    torch = hs.torch
    dev = hs.dev
    f32 = dict(dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)
    name = args.case
    reps = 3
    if name.startswith("gemm_dense"):
        # the qkv projection of the training configuration at 8 sequences: 32768 x 6144 x 2048 (forward, input gradient,
        # weight gradient forms)
        mode = {"gemm_dense": asca_b200.NN, "gemm_dense_nt": asca_b200.NT, "gemm_dense_tn": asca_b200.TN}[name]
        m_, n_, k_ = {asca_b200.NN: (32768, 6144, 2048), asca_b200.NT: (32768, 2048, 6144), asca_b200.TN: (2048, 6144, 32768)}[mode]
        a = torch.randn((k_, m_) if mode == asca_b200.TN else (m_, k_), generator=g, **f32).bfloat16()
        b = torch.randn((n_, k_) if mode == asca_b200.NT else (k_, n_), generator=g, **f32).bfloat16()
        c = torch.empty(m_, n_, **f32)
        fn = lambda: ops.gemm(hs.gpu, a, b, mode, out=c)  # noqa: E731
        work, unit = 2.0 * m_ * n_ * k_, "TFLOP/s"
    elif name in ("moe_fwd", "moe_bwd", "moe_bwd_8seq"):
        # the expert FFN of the training configuration on one micro-batch of 2 sequences (8192 uniform random bytes);
        # moe_bwd_8seq: 8 sequences, a rank's micro-batch in an 8-GPU run (512 rows per expert)
        n, d, F, E = 32768 if name == "moe_bwd_8seq" else 8192, 2048, 4096, 64
        ids = torch.from_numpy(reference_ids(5, n).view(np.int32)).to(dev)
        xn = torch.randn(n, d, generator=g, **f32).bfloat16()
        w1 = (torch.randn(d, E * F, generator=g, **f32) * 0.02).bfloat16()
        w2 = (torch.randn(E * F, d, generator=g, **f32) * 0.02).bfloat16()
        b1, b2 = torch.zeros(E * F, **f32), torch.zeros(d, **f32)
        dout = torch.randn(n, d, generator=g, **f32)
        perm, off = ops.moe_dispatch(hs.gpu, ids, E)
        out, pre_p, hid_p = ops.moe_fwd(hs.gpu, xn, w1, b1, w2, b2, perm, off, F, E)
        if name == "moe_fwd":
            fn = lambda: ops.moe_fwd(hs.gpu, xn, w1, b1, w2, b2, perm, off, F, E, out=out, pre_p=pre_p, hid_p=hid_p)  # noqa: E731
            work = 4.0 * n * d * F
        else:
            grads = ops.moe_bwd(hs.gpu, xn, w1, w2, pre_p, hid_p, dout, perm, off, F, E)
            fn = lambda: ops.moe_bwd(hs.gpu, xn, w1, w2, pre_p, hid_p, dout, perm, off, F, E, grads=grads)  # noqa: E731
            work = 8.0 * n * d * F
        unit = "TFLOP/s"
    elif name in ("delta_bf16", "delta_f32", "delta_bf16_dh64"):
        # the isolated delta op at B = 2 (32 chains x 4096 tokens): traffic scales with the number of chains;
        # delta_bf16_dh64: heads of 64 (the decode configuration's head size) at the same width, B = 8 (256 chains)
        b, h, t, dh = (8, 32, 4096, 64) if name == "delta_bf16_dh64" else (2, 16, 4096, 128)
        n, d = b * t, h * dh
        q = torch.nn.functional.normalize(torch.randn(n, h, dh, generator=g, **f32), dim=-1).reshape(n, d).contiguous()
        k = torch.nn.functional.normalize(torch.randn(n, h, dh, generator=g, **f32), dim=-1).reshape(n, d).contiguous()
        v, d_o = torch.randn(n, d, generator=g, **f32), torch.randn(n, d, generator=g, **f32)
        alpha = torch.sigmoid(2 + 0.5 * torch.randn(n, h, generator=g, **f32))
        beta = torch.sigmoid(torch.randn(n, h, generator=g, **f32))
        qn, kn = torch.ones(n, h, **f32), torch.ones(n, h, **f32)
        if name != "delta_f32":
            q, k, v, d_o = (x.bfloat16() for x in (q, k, v, d_o))
        o = torch.empty_like(q)
        ckpt = torch.empty(ops.delta_ckpt_floats(hs.gpu, b, t, h, dh, 64), **f32)
        d_qkv, d_gate = torch.empty((n, 3 * d), **f32), torch.empty((n, 2 * h), **f32)

        def fn():
            ops.delta_fwd(hs.gpu, q, k, v, alpha, beta, b, t, h, dh, chunk=64, out=o, ckpt=ckpt)
            ops.delta_bwd(hs.gpu, q, k, v, alpha, beta, qn, kn, d_o, ckpt, b, t, h, dh, chunk=64, d_qkv=d_qkv, d_gate=d_gate)

        s_io = 4 if name == "delta_f32" else 2
        work, unit = 11.0 * n * d * s_io + 8.0 * n * h * 4, "GB/s"
    elif name == "decode":
        # a few greedy steps of the decode configuration (256 streams)
        c = DECODE
        model = asca_b200.Model(hs.gpu, c["V"], c["d"], c["H"], c["L"], c["E"], c["F"])
        model.set_compute(asca_b200.BF16)
        hs.fill_normal(model.buffers()[0], model.n, seed=0)
        model.params_changed()
        state = model.new_decode_state(c["streams"])
        ids0 = reference_ids(2, c["streams"])
        model.decode_greedy(state, ids0, 2)
        fn = lambda: model.decode_greedy(state, ids0, 2)  # noqa: E731
        dh = c["d"] // c["H"]
        work = 2.0 * (2 * c["L"] * c["H"] * dh * dh * 4 * c["streams"]
                      + (c["L"] * (c["d"] * 3 * c["d"] + c["d"] * 2 * c["H"] + c["d"] * c["d"] + 2 * c["E"] * c["d"] * c["F"]) + c["d"] * c["V"]) * 2)
        unit = "GB/s"
        reps = 2
    elif name in ("rmsnorm", "rmsnorm_bwd", "residual_rmsnorm", "adamw", "gather", "dispatch", "delta_step"):
        # the HBM-bound entry points on buffers larger than L2; work = algorithmic bytes per launch
        import ctypes as C

        from asca_b200 import _f, _i64, _p

        unit, reps = "GB/s", 20
        call = lambda nm, *a: hs.gpu._call(nm, hs.gpu._ctx, *a)  # noqa: E731
        rows, cols = 65536, 1024
        if name in ("rmsnorm", "rmsnorm_bwd", "residual_rmsnorm", "gather"):
            xs = [torch.randn(rows, cols, generator=g, **f32) for _ in range(2)]
            y, z = torch.empty(rows, cols, **f32), torch.empty(rows, cols, **f32)
            idx = torch.randperm(rows, device=dev, generator=g).to(torch.int32)
            if name == "rmsnorm":
                fn = lambda: call("asca_rmsnorm_fwd", _p(xs[0]), _p(y), None, _i64(rows), _i64(cols), _f(1e-6))  # noqa: E731
                work = 2.0 * rows * cols * 4
            elif name == "rmsnorm_bwd":
                fn = lambda: call("asca_rmsnorm_bwd", _p(xs[0]), _p(xs[1]), _p(y), _i64(rows), _i64(cols), _f(1e-6))  # noqa: E731
                work = 3.0 * rows * cols * 4
            elif name == "residual_rmsnorm":
                fn = lambda: call("asca_residual_rmsnorm", _p(xs[0]), _p(xs[1]), _p(z), _p(y), _i64(rows), _i64(cols), _f(1e-6))  # noqa: E731
                work = 4.0 * rows * cols * 4
            else:
                fn = lambda: call("asca_gather_rows", _p(xs[0]), _p(idx), _i64(rows), _i64(cols), _p(y))  # noqa: E731
                work = 2.0 * rows * cols * 4
        elif name == "adamw":
            n = 1 << 26
            p_, g_, m_, v_ = (torch.randn(n, generator=g, **f32) * 0.01 for _ in range(4))
            v_.abs_()
            fn = lambda: ops.adamw(hs.gpu, p_, g_, m_, v_, 1e-3, 0.9, 0.95, 1e-8, 1e-5)  # noqa: E731
            work = 7.0 * n * 4
        elif name == "dispatch":
            n = 1 << 22
            ids = torch.from_numpy(zipf_ids(4, 65536).view(np.int32)).to(dev).repeat(n // 65536)
            perm = torch.empty(n, dtype=torch.int32, device=dev)
            off = torch.empty(65, dtype=torch.int32, device=dev)
            fn = lambda: call("asca_moe_dispatch", _p(ids), _i64(n), _i64(64), _p(perm), _p(off), None)  # noqa: E731
            work = 12.0 * n          # ids read twice, perm written
        else:
            ns, H, dh, L = 256, 12, 64, 12   # 12 layers' states rotate: 604 MB > L2
            S = [torch.randn(ns, H, dh, dh, generator=g, **f32) * 0.1 for _ in range(L)]
            d = H * dh
            qkv, gate = torch.randn(ns, 3 * d, generator=g, **f32), torch.randn(ns, 2 * H, generator=g, **f32)
            o = torch.empty(ns, d, **f32)
            it = {"i": 0}

            def fn():
                it["i"] += 1
                ops.delta_step(hs.gpu, qkv, None, None, gate, None, S[it["i"] % L], H, dh, fused=True, out=o)

            work = 2.0 * ns * H * dh * dh * 4 + ns * (4 * d + 2 * H) * 4
            reps = 60
        del C
    else:
        raise SystemExit(f"bench.py: unknown --case {name}")
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    print(json.dumps({"case": name, "ms": ms, "achieved": work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9), "unit": unit,
                      "launches": hs.gpu.launch_count()}))


# ------------------------------------------------------------------ driver
def run_ours(args):
    hs = Harness()
    if args.case:
        run_case(hs, args)
        return
    only = set(filter(None, args.only.split(","))) or {"train", "decode", "moe", "delta"}
    line = run_train(hs, args) if "train" in only else None
    records = {}
    if "decode" in only:
        records["decode"] = run_decode(hs, args)
    if hs.world == 1:        # the isolated ops are per-GPU workloads: measured once, at N = 1
        if "moe" in only:
            records["moe"] = run_moe(hs, args)
        if "delta" in only:
            records["delta_bf16"] = run_delta(hs, args, True)
            hs.gpu.lib.asca_ctx_trim(hs.gpu._ctx)
            hs.torch.cuda.empty_cache()
            records["delta_f32"] = run_delta(hs, args, False)
    if hs.rank == 0:
        if line is None:      # a partial run (--only without train): the first record stands in as the line
            key = next(iter(records))
            line = dict(records.pop(key))
            line.setdefault("warmup", args.warmup)
            line.setdefault("higher_is_better", True)
            line.setdefault("vs_baseline", None)
            line.setdefault("data", "synthetic")
        elif hs.world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline_train(args.layers)
        else:
            line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 0, "kind": "port", "sample": "skipped (rank 0 at N = 1 only)"}
        line["records"] = records
        print(json.dumps(line))
    if hs.world > 1:
        hs.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=4, help="blocks of the 24-block training stack to run (the largest that fits one GPU)")
    ap.add_argument("--transport", default="nccl", choices=["nccl", "ce"],
                    help="N > 1: how the sharded expert tensors travel (NCCL kernels, or copy engines through peer memory)")
    ap.add_argument("--only", default="", help="comma-separated subset of train,decode,moe,delta")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--case", default="", help="run one small single-kernel case instead (for profiler captures): gemm_dense, "
                                               "gemm_dense_nt, gemm_dense_tn, moe_fwd, moe_bwd, moe_bwd_8seq, delta_bf16, delta_bf16_dh64, delta_f32, decode, rmsnorm, rmsnorm_bwd, "
                                               "residual_rmsnorm, adamw, gather, dispatch, delta_step")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_ours(args)


if __name__ == "__main__":
    main()
