"""Data parallelism by sequence (one process per GPU).

The hot path shards without any data-path collective: a (sequence, head) chain, a MoE token row
and a decode stream never read another rank's data, and every rank holds the full weights
(heads and experts stay local). Training needs exactly one exchange per step: the sum of the
flat gradient buffer over ranks, scaled by 1/world so that equal per-rank token counts
reproduce the single-process token mean (the property rust/tests/batch_parity.rs pins).
torch.distributed is the plumbing (NCCL over NVLink on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def shard_sequences(n_sequences: int, rank: int, world: int) -> range:
    """Contiguous block of sequence indices owned by `rank` (the first n % world ranks get one more)."""
    base, extra = divmod(n_sequences, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def shard_tokens(ids: np.ndarray, batch: int, rank: int, world: int):
    """Rows (b*T + t) of the sequences owned by `rank`; returns (ids_shard, local_batch)."""
    seq = ids.size // batch
    own = shard_sequences(batch, rank, world)
    return ids.reshape(batch, seq)[own.start:own.stop].reshape(-1).copy(), len(own)


def allreduce_mean_(flat: torch.Tensor, weight: float = 1.0, group=None) -> torch.Tensor:
    """In-place sum over ranks of weight * flat. With weight = local_tokens / global_tokens this is
    the global token mean of per-rank means."""
    if weight != 1.0:
        flat.mul_(weight)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    return flat


class _DevView:
    """Zero-copy torch view of a device buffer owned by the library (CUDA array interface)."""

    def __init__(self, ptr: int, n: int):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def device_tensor(ptr: int, n: int, device: int) -> torch.Tensor:
    return torch.as_tensor(_DevView(ptr, n), device=f"cuda:{device}")


def allreduce_model_grads(model, local_tokens: int, global_tokens: int, group=None) -> None:
    """Average the device-resident flat gradient buffer of an asca_b200.Model over all ranks."""
    grads = device_tensor(model.buffers()[1], model.n, model.gpu.device)
    model.gpu.sync()
    allreduce_mean_(grads, local_tokens / global_tokens, group)


class GradOverlap:
    """All-reduce (average) of an asca_b200.Model's flat gradient buffer, overlapped with its backward.

    The model reports each finished gradient range from inside ``forward_backward`` (one block at a
    time, last block first). For every range this records an event on the compute stream, makes a
    side stream wait for it and queues ``all_reduce(AVG)`` of that slice there, so the exchange of
    block i runs under the backward of blocks i-1 .. 0. ``finish()`` makes the compute stream wait
    for the exchanges; AdamW queued after it sees the averaged gradients.

    With gradient accumulation, arm it only around the last micro-batch (``with overlap:``).
    """

    def __init__(self, model, group=None):
        self.model, self.group = model, group
        dev = model.gpu.device
        self.grads = device_tensor(model.buffers()[1], model.n, dev)
        self.side = torch.cuda.Stream(device=dev)
        self.works = []
        self.ranges = []

    def _ready(self, off, cnt):
        self.ranges.append((off, cnt))
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(self.group) == 1:
            return
        ev = torch.cuda.current_stream().record_event()
        self.side.wait_event(ev)
        with torch.cuda.stream(self.side):
            self.works.append(dist.all_reduce(self.grads[off:off + cnt], op=dist.ReduceOp.AVG, group=self.group, async_op=True))

    def __enter__(self):
        self.ranges = []
        self.model.set_grad_hook(self._ready)
        return self

    def __exit__(self, *exc):
        self.model.set_grad_hook(None)
        self.finish()
        return False

    def finish(self):
        for w in self.works:
            w.wait()          # stream-level wait on the side stream
        self.works = []
        torch.cuda.current_stream().wait_stream(self.side)
