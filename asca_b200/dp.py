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


def device_tensor_bf16(ptr: int, n: int, device: int) -> torch.Tensor:
    """bf16 view of a device buffer of n 2-byte elements."""
    v = _DevView(ptr, n)
    v.__cuda_array_interface__["typestr"] = "<i2"
    return torch.as_tensor(v, device=f"cuda:{device}").view(torch.bfloat16)


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


def shard_plan(cfg, rank: int, world: int):
    """Which parts of the flat parameter buffer `rank` updates under the sharded optimizer.

    The experts' W1 and W2 of every block (98 % of the parameters at the training configuration) are cut into `world`
    equal contiguous chunks, one per rank; every other tensor is updated by every rank. Returns (big, slices):
    big = [(offset, size)] of the sharded tensors in buffer order, slices = the sorted, disjoint (lo, hi) ranges this
    rank updates, adjacent ranges merged. Sizes that `world` x 4 does not divide are not sharded.
    """
    from asca_b200.train import tensor_sizes

    sizes = tensor_sizes(cfg)
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    big, slices = [], []
    for i, n in enumerate(sizes):
        lo = int(offs[i])
        is_expert = i >= 2 and (i - 2) % 10 in (6, 8)      # w1, w2 in the per-block order of tensor_sizes
        if is_expert and world > 1 and n % (4 * world) == 0:
            big.append((lo, int(n)))
            c = n // world
            piece = (lo + rank * c, lo + (rank + 1) * c)
        else:
            piece = (lo, lo + int(n))
        if slices and slices[-1][1] == piece[0]:
            slices[-1] = (slices[-1][0], piece[1])
        else:
            slices.append(piece)
    return big, slices


class ShardedOverlap(GradOverlap):
    """GradOverlap with the optimizer sharded over the ranks for the expert weights (bf16 compute mode).

    For W1 / W2 of every block the gradient exchange is a reduce-scatter (each rank receives the mean of its chunk
    only: half the bytes of an all-reduce), the rank updates its chunk (``finish(lr)`` runs one sliced AdamW over the
    chunks and all small tensors), and the updated bf16 chunks are all-gathered into every rank's bf16 weight copy
    (2 bytes per parameter). The f32 master weights and moments of the other ranks' chunks are never exchanged and
    are stale on this rank: ``gather_master()`` collects them before the parameters are read out.
    """

    def __init__(self, model, group=None):
        super().__init__(model, group)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.big, self.slices = shard_plan(model.cfg, self.rank, self.world)
        # the update is issued tensor group by tensor group, so that the all-gather of a sharded tensor's bf16 chunks
        # runs on the side stream while the next group is being updated: cut the slices at the sharded tensors' ends
        cuts = [lo + n for lo, n in self.big]
        pieces = []
        for a, b in self.slices:
            for c in cuts:
                if a < c < b:
                    pieces.append((a, c))
                    a = c
            pieces.append((a, b))
        self.groups, k = [], 0
        for (lo, n), c in zip(self.big, cuts):
            grp = []
            while k < len(pieces) and pieces[k][1] <= c:
                grp.append(pieces[k])
                k += 1
            self.groups.append((grp, (lo, n)))
        self.groups.append((pieces[k:], None))

    def _ready(self, off, cnt):
        self.ranges.append((off, cnt))
        if self.world == 1:
            return
        ev = torch.cuda.current_stream().record_event()
        self.side.wait_event(ev)
        pieces, pos = [], off
        for lo, n in self.big:                      # cut the range at the sharded tensors inside it
            if lo >= off and lo + n <= off + cnt:
                if lo > pos:
                    pieces.append((pos, lo - pos, False))
                pieces.append((lo, n, True))
                pos = lo + n
        if pos < off + cnt:
            pieces.append((pos, off + cnt - pos, False))
        with torch.cuda.stream(self.side):
            for lo, n, sharded in pieces:
                g = self.grads[lo:lo + n]
                if sharded:
                    c = n // self.world
                    self.works.append(dist.reduce_scatter_tensor(g[self.rank * c:(self.rank + 1) * c], g, op=dist.ReduceOp.AVG,
                                                                 group=self.group, async_op=True))
                else:
                    self.works.append(dist.all_reduce(g, op=dist.ReduceOp.AVG, group=self.group, async_op=True))

    def step(self, lr):
        """After the backward: wait for the exchanges, update this rank's slices, all-gather the bf16 chunks."""
        self.finish()
        if self.world == 1:
            self.model.adamw_step(lr)
            return
        ptr, n16 = self.model.params16()
        p16 = device_tensor_bf16(ptr, n16, self.model.gpu.device)
        last = max(i for i, g in enumerate(self.groups) if g[0])
        for i, (grp, big) in enumerate(self.groups):
            if grp:
                self.model.adamw_slices(lr, grp, advance=(i == last))
            if big is not None:
                lo, n = big
                c = n // self.world
                ev = torch.cuda.current_stream().record_event()
                self.side.wait_event(ev)
                with torch.cuda.stream(self.side):
                    dist.all_gather_into_tensor(p16[lo:lo + n], p16[lo + self.rank * c:lo + (self.rank + 1) * c], group=self.group)
        torch.cuda.current_stream().wait_stream(self.side)

    def gather_master(self):
        """All-gather the f32 master weights and Adam moments of the sharded tensors (before a checkpoint)."""
        if self.world == 1:
            return
        b = self.model.buffers()
        for ptr in (b[0], b[2], b[3]):
            t = device_tensor(ptr, self.model.n, self.model.gpu.device)
            for lo, n in self.big:
                c = n // self.world
                dist.all_gather_into_tensor(t[lo:lo + n], t[lo + self.rank * c:lo + (self.rank + 1) * c], group=self.group)
        torch.cuda.synchronize()
