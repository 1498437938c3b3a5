"""Data-parallel training step of the 1.3B-class architecture, cut to a few blocks.

    python -m asca_b200.trainbench [--layers 2] [--global-batch 64] [--micro 32] [--steps 3]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m asca_b200.trainbench ...

Architecture of the baseline's largest configuration (d 2048, 16 heads of 128, 64 hash experts of
2048 -> 4096 -> 2048, byte vocabulary) with --layers blocks instead of 24: the full stack does not
fit one GPU replicated (26 B parameters x 16 bytes of f32 master, gradient and moments), and the cost
per block is the same for every block. bf16 compute mode, f32 recurrent state, f32 master weights
and AdamW. The global batch of --global-batch sequences x 4096 uniform random bytes is split by
sequence over the ranks; each rank runs its share as micro-batches of at most --micro sequences with
gradient accumulation (the larger the micro-batch, the fewer passes over the 4.4 GB of expert weight
gradients per block: 8 -> 32 sequences is worth 13 % of the step), the flat gradient buffer is averaged over ranks by NCCL all-reduce queued
block by block from inside the last backward (asca_b200.dp.GradOverlap), then every rank applies the
same AdamW update (--optimizer replicated). Default at N > 1 (--optimizer sharded, dp.ShardedOverlap): the
experts' W1 / W2 gradients are reduce-scattered instead, each rank updates its 1/N chunk of them (and all
small tensors), and the updated bf16 chunks are all-gathered; --verify runs two steps both ways and checks
that the weights are identical. One JSON line from rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

import asca_b200
from asca_b200 import dp
from asca_b200.microbench import peaks


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--global-batch", type=int, default=64)
    ap.add_argument("--micro", type=int, default=32, help="sequences per micro-batch (at most the rank's share)")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--optimizer", default="sharded", choices=["sharded", "replicated"],
                    help="sharded: expert weights reduce-scattered, updated 1/N per rank, bf16 all-gathered (N > 1)")
    ap.add_argument("--verify", action="store_true", help="N > 1: run two steps with both optimizers and compare the weights")
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    gpu = asca_b200.Gpu(local)
    gpu.use_torch_stream()
    V, d, H, L, E, F = 256, 2048, 16, args.layers, 64, 4096
    T = args.seq
    own = dp.shard_sequences(args.global_batch, rank, world)
    n_micro = max(1, len(own) // args.micro)
    mb = len(own) // n_micro
    assert mb * n_micro == len(own), "the rank's share must be a whole number of micro-batches"

    model = asca_b200.Model(gpu, V, d, H, L, E, F)
    model.set_compute(asca_b200.BF16)
    g = torch.Generator(device=f"cuda:{local}").manual_seed(0)          # same weights on every rank
    params = dp.device_tensor(model.buffers()[0], model.n, local)
    for lo in range(0, model.n, 1 << 28):
        hi = min(model.n, lo + (1 << 28))
        params[lo:hi] = torch.randn(hi - lo, generator=g, dtype=torch.float32, device=f"cuda:{local}") * 0.02
    model.params_changed()
    ids_all = torch.randint(0, 256, (args.global_batch, T), generator=torch.Generator().manual_seed(1)).numpy().astype("uint32")
    ids = ids_all[own.start:own.stop]
    tg = ids.copy()
    tg[:, :-1] = ids[:, 1:]
    model.set_grad_scale(1.0 / n_micro)
    sharded = args.optimizer == "sharded" and world > 1
    overlap = dp.ShardedOverlap(model) if sharded else dp.GradOverlap(model)

    def step():
        model.zero_grads()
        t0 = time.perf_counter()
        loss = 0.0
        for i in range(n_micro):
            rows = slice(i * mb, (i + 1) * mb)
            if i == n_micro - 1:
                with overlap:
                    loss += model.forward_backward(ids[rows].reshape(-1), tg[rows].reshape(-1), mb)
            else:
                loss += model.forward_backward(ids[rows].reshape(-1), tg[rows].reshape(-1), mb)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        if sharded:
            overlap.step(3e-4)       # sliced AdamW + all-gather of the bf16 expert chunks
        else:
            model.adamw_step(3e-4)
        gpu.sync()
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        return loss / n_micro, t1 - t0, t2 - t1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.verify and world > 1:
        # the same two steps with the replicated optimizer on a second model: the bf16 weights every rank computes
        # with must be identical, and so must this rank's slices of the f32 master weights
        other = asca_b200.Model(gpu, V, d, H, L, E, F)
        other.set_compute(asca_b200.BF16)
        po = dp.device_tensor(other.buffers()[0], other.n, local)
        po.copy_(params)
        other.params_changed()
        other.set_grad_scale(1.0 / n_micro)
        ov_s, ov_r = dp.ShardedOverlap(model), dp.GradOverlap(other)
        for _ in range(2):
            for mdl, ov in ((model, ov_s), (other, ov_r)):
                mdl.zero_grads()
                for i in range(n_micro):
                    rows = slice(i * mb, (i + 1) * mb)
                    if i == n_micro - 1:
                        with ov:
                            mdl.forward_backward(ids[rows].reshape(-1), tg[rows].reshape(-1), mb)
                    else:
                        mdl.forward_backward(ids[rows].reshape(-1), tg[rows].reshape(-1), mb)
            ov_s.step(3e-4)
            other.adamw_step(3e-4)
        torch.cuda.synchronize()
        a16 = dp.device_tensor_bf16(*model.params16(), local)
        b16 = dp.device_tensor_bf16(*other.params16(), local)
        same16 = bool(torch.equal(a16, b16))
        same32 = all(bool(torch.equal(params[lo:hi], po[lo:hi])) for lo, hi in ov_s.slices)
        ov_s.gather_master()
        same_all = bool(torch.equal(params, po))
        # beyond two ranks a reduce-scatter and an all-reduce add the ranks' gradients in different orders, so the
        # results agree to rounding, not bit for bit: report how far apart they are
        worst, scale, n_diff16 = 0.0, 0.0, 0
        for lo in range(0, model.n, 1 << 28):
            hi = min(model.n, lo + (1 << 28))
            worst = max(worst, float((params[lo:hi] - po[lo:hi]).abs().max()))
            scale = max(scale, float(po[lo:hi].abs().max()))
            n_diff16 += int((a16[lo:hi] != b16[lo:hi]).sum())
        print(json.dumps({"verify": "sharded vs replicated optimizer, 2 steps", "rank": rank, "bf16_weights_equal": same16,
                          "own_master_slices_equal": same32, "master_equal_after_gather": same_all,
                          "max_abs_master_difference": worst, "max_abs_master": scale,
                          "bf16_weights_differing": n_diff16, "of": model.n}), flush=True)
        other.free()
        model.free()
        dist.destroy_process_group()
        return
    step()          # warms the pools and NCCL up
    barrier()
    t_fb = t_opt = 0.0
    t_begin = time.perf_counter()
    for _ in range(args.steps):
        loss, a, b = step()
        t_fb += a
        t_opt += b
    barrier()
    wall = (time.perf_counter() - t_begin) / args.steps
    if world > 1:
        tt = torch.tensor([wall], device=f"cuda:{local}")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        wall = float(tt.item())
    if rank == 0:
        per_layer = d * 3 * d + d * 2 * H + d * d + 2 * d * F          # GEMM parameters a token touches per block
        flop_tok = 6 * (L * per_layer + d * V) + 22 * (d // H) ** 2 * H * L
        n_tok = args.global_batch * T
        _, tf, src = peaks()
        print(json.dumps({
            "case": "train step, 1.3B-class architecture, data parallel by sequence", "n_gpus": world, "layers": L,
            "params": model.n, "global_batch": args.global_batch, "seq": T, "micro_batches_per_rank": n_micro,
            "sequences_per_micro_batch": mb, "loss": round(float(loss), 4), "ms_per_step": round(wall * 1e3, 2),
            "fwd_bwd_allreduce_ms": round(t_fb / args.steps * 1e3, 2), "adamw_ms": round(t_opt / args.steps * 1e3, 2),
            "tok_s": round(n_tok / wall, 1), "algorithmic_flop_per_token": flop_tok,
            "TFLOP/s_per_gpu": round(n_tok * flop_tok / wall / 1e12 / world, 1),
            "frac_of_bf16_peak_per_gpu": round(n_tok * flop_tok / wall / 1e12 / world / tf, 4), "peak": src,
            "optimizer": "sharded" if sharded else "replicated", "scaling": "strong (global batch fixed)"}), flush=True)
    model.free()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
