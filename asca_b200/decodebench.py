"""Batched greedy decode of the ~125M decode configuration.

    python -m asca_b200.decodebench [--streams 256] [--prefill 512] [--tokens 2048] [--dtype bf16]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m asca_b200.decodebench ...

12 blocks, d 768, 12 heads of 64, 16 hash experts of 768 -> 3072 -> 768, byte vocabulary, weights
N(0, 0.02). --streams concurrent streams are sharded over the ranks (no collective: a stream never
reads another stream's state). Every stream is prefilled with --prefill random bytes by stepping (as
the reference's decoder does), untimed; then --tokens greedy steps are timed (argmax on the device,
lowest index on ties, fed to the next step on the device; the chosen bytes come back to the host
every --chunk steps, which is the only synchronisation). One JSON line from rank 0:
tok/s over all ranks and the HBM roofline of a step -- state read + written once (2 L H dh^2 4 B per
stream) plus every weight byte the step touches once (with 256 streams over 16 experts every expert is
hit, so all of them).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist

import asca_b200
from asca_b200 import dp
from asca_b200.microbench import peaks


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--streams", type=int, default=256)
    ap.add_argument("--prefill", type=int, default=512)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--dtype", default="bf16", choices=["f32", "bf16"])
    ap.add_argument("--chunk", type=int, default=64, help="greedy steps per call (tokens reach the host once per call)")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    gpu = asca_b200.Gpu(local)
    gpu.use_torch_stream()
    V, d, H, L, E, F = 256, 768, 12, 12, 16, 3072
    dh = d // H
    own = dp.shard_sequences(args.streams, rank, world)
    ns = len(own)
    model = asca_b200.Model(gpu, V, d, H, L, E, F)
    if args.dtype == "bf16":
        model.set_compute(asca_b200.BF16)
    g = torch.Generator(device=f"cuda:{local}").manual_seed(0)
    params = dp.device_tensor(model.buffers()[0], model.n, local)
    params[:] = torch.randn(model.n, generator=g, dtype=torch.float32, device=f"cuda:{local}") * 0.02
    model.params_changed()
    prompts = np.random.default_rng(1).integers(0, 256, (args.streams, args.prefill), dtype=np.uint32)[own.start:own.stop]
    state = model.new_decode_state(ns)
    nxt = None
    for t in range(args.prefill):
        _, nxt = model.decode_step(state, prompts[:, t].copy(), want_logits=False)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches0 = gpu.launch_count()
    t0 = time.perf_counter()
    done = 0
    while done < args.tokens:
        n = min(args.chunk, args.tokens - done)
        nxt = model.decode_greedy(state, nxt, n)[-1]
        done += n
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - t0
    if world > 1:
        tt = torch.tensor([wall], device=f"cuda:{local}")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        wall = float(tt.item())
    if rank == 0:
        wbytes = 2 if args.dtype == "bf16" else 4
        state_bytes = 2 * L * H * dh * dh * 4 * ns
        weight_bytes = (L * (d * 3 * d + d * 2 * H + d * d + 2 * E * d * F) + d * V) * wbytes
        step_bytes = state_bytes + weight_bytes
        hbm, _, src = peaks()
        ms = wall / args.tokens * 1e3
        print(json.dumps({
            "case": "greedy decode, ~125M configuration", "dtype": args.dtype, "n_gpus": world, "streams": args.streams,
            "streams_per_gpu": ns, "prefill": args.prefill, "tokens_per_stream": args.tokens, "steps_per_call": args.chunk, "ms_per_step": round(ms, 4),
            "tok_s": round(args.streams * args.tokens / wall, 1), "launches_per_step": (gpu.launch_count() - launches0) / args.tokens,
            "algorithmic_bytes_per_step_per_gpu": step_bytes, "state_bytes": state_bytes, "weight_bytes": weight_bytes,
            "GB/s_per_gpu": round(step_bytes / (ms * 1e-3) / 1e9, 1), "frac_of_hbm_peak": round(step_bytes / (ms * 1e-3) / 1e9 / hbm, 4),
            "peak": src, "roofline_tok_s_per_gpu": round(ns / (step_bytes / (hbm * 1e9)), 1)}), flush=True)
    model.free()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
