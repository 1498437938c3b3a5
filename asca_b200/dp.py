"""Data parallelism by sequence (one process per GPU): bindings of the library's exchange.

The hot path shards without any data-path collective: a (sequence, head) chain, a MoE token row
and a decode stream never read another rank's data, and every rank holds the full weights
(heads and experts stay local). Training needs exactly one exchange per step: the mean of the
flat gradient buffer over ranks, which with equal per-rank token counts reproduces the
single-process token mean (the property rust/tests/batch_parity.rs pins).

The exchange itself lives in the library (csrc/dp.cu, behind ``asca_comm_*`` /
``asca_allreduce_grads`` / ``asca_model_dp_*`` of include/asca_b200.h): NCCL collectives on a side
stream owned by the communicator, queued from inside the backward as gradient ranges become final,
ordered against the CONTEXT's stream -- whichever stream that is. This module only binds it.
``torch.distributed`` is used for nothing but handing the 128-byte NCCL id to the other ranks (and,
in CPU tests on gloo, for the host-side helpers at the top).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import AscaError, _f, _i64, _p, load


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


def allreduce_mean_(flat, weight: float = 1.0, group=None):
    """Host-side statement of the exchange on a torch tensor (used by the gloo tests): in-place sum over
    ranks of weight * flat. With weight = local_tokens / global_tokens this is the global token mean."""
    import torch.distributed as dist

    if weight != 1.0:
        flat.mul_(weight)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    return flat


class _DevView:
    """Zero-copy torch view of a device buffer owned by the library (CUDA array interface)."""

    def __init__(self, ptr: int, n: int):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def device_tensor(ptr: int, n: int, device: int):
    import torch

    return torch.as_tensor(_DevView(ptr, n), device=f"cuda:{device}")


def device_tensor_bf16(ptr: int, n: int, device: int):
    """bf16 view of a device buffer of n 2-byte elements."""
    import torch

    v = _DevView(ptr, n)
    v.__cuda_array_interface__["typestr"] = "<i2"
    return torch.as_tensor(v, device=f"cuda:{device}").view(torch.bfloat16)


def shard_plan(cfg, rank: int, world: int):
    """Which parts of the flat parameter buffer `rank` updates under the sharded optimizer
    (``asca_dp_shard_plan``; host arithmetic only, no GPU needed).

    The experts' W1 and W2 of every block (98 % of the parameters at the training configuration) are cut into
    `world` equal contiguous chunks, one per rank; every other tensor is updated by every rank. Returns
    (big, slices): big = [(offset, size)] of the sharded tensors in buffer order, slices = the sorted, disjoint
    (lo, hi) ranges this rank updates, adjacent ranges merged. Sizes that 4 x `world` does not divide are not sharded.
    """
    lib = load()
    vocab, d, H, L, E, F = (int(x) for x in cfg)
    cap = 12 * L + 8
    lo, hi = (C.c_int64 * cap)(), (C.c_int64 * cap)()
    boff, blen = (C.c_int64 * (2 * L))(), (C.c_int64 * (2 * L))()
    ns, nb = C.c_int(), C.c_int()
    rc = lib.asca_dp_shard_plan(_i64(vocab), _i64(d), _i64(H), _i64(L), _i64(E), _i64(F), C.c_int(world), C.c_int(rank),
                                lo, hi, C.c_int(cap), C.byref(ns), boff, blen, C.c_int(2 * L), C.byref(nb))
    if rc != 0:
        raise AscaError(rc, "asca_dp_shard_plan: bad arguments")
    big = [(int(boff[i]), int(blen[i])) for i in range(nb.value)]
    slices = [(int(lo[i]), int(hi[i])) for i in range(ns.value)]
    return big, slices


class Comm:
    """One rank's end of an NCCL communicator owned by the library (``asca_comm_*``)."""

    def __init__(self, gpu, nranks: int, rank: int, unique_id: bytes | None):
        self.gpu, self.nranks, self.rank = gpu, nranks, rank
        h = C.c_void_p()
        buf = C.create_string_buffer(unique_id, 128) if unique_id is not None else None
        gpu._call("asca_comm_init", gpu._ctx, C.c_int(nranks), C.c_int(rank), buf, C.byref(h))
        self._h = h

    @staticmethod
    def unique_id(gpu) -> bytes:
        buf = C.create_string_buffer(128)
        gpu._call("asca_comm_unique_id", gpu._ctx, buf)
        return buf.raw

    @classmethod
    def from_torch(cls, gpu, group=None):
        """Rank 0 of an initialised torch.distributed group draws the id; the group carries it to the others."""
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            return cls(gpu, 1, 0, None)
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [cls.unique_id(gpu) if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls(gpu, world, rank, box[0])

    def allreduce_grads(self, ptr: int, n: int, bucket_off=None):
        """Mean over ranks of the n floats at device address `ptr`, in stream order with the context's stream."""
        if bucket_off is None:
            self.gpu._call("asca_allreduce_grads", self.gpu._ctx, self._h, C.c_void_p(ptr), _i64(n), None, C.c_int(0))
        else:
            off = np.ascontiguousarray(bucket_off, dtype=np.int64)
            self.gpu._call("asca_allreduce_grads", self.gpu._ctx, self._h, C.c_void_p(ptr), _i64(n), _p(off), C.c_int(off.size - 1))

    def close(self):
        if self._h is not None:
            self.gpu.lib.asca_comm_destroy(self.gpu._ctx, self._h)
            self._h = None


def allreduce_model_grads(model, comm: Comm) -> None:
    """Blocking form: average the device-resident flat gradient buffer of an asca_b200.Model over all ranks."""
    comm.allreduce_grads(model.buffers()[1], model.n)


class GradOverlap:
    """The gradient exchange of an asca_b200.Model overlapped with its backward, replicated optimizer.

    ``with overlap:`` arms the model for the backward(s) inside the block (with gradient accumulation, wrap the
    last micro-batch only); the library queues the all-reduce (mean) of every finished gradient range on the
    communicator's side stream from inside ``forward_backward``. ``step(lr)`` waits for the exchanges and applies
    AdamW (use it instead of ``model.adamw_step``). ``ranges`` lists the (offset, count) ranges the last armed
    backward reported, in order. Without a communicator (``comm=None`` and no initialised process group) the
    exchange is a no-op and ``step`` is the plain optimizer step.
    """

    sharded = False

    def __init__(self, model, comm: Comm | None = None, group=None):
        self.model = model
        self.comm = comm if comm is not None else Comm.from_torch(model.gpu, group)
        self.world, self.rank = self.comm.nranks, self.comm.rank
        self.ranges = []
        model.gpu._call("asca_model_dp_attach", model.gpu._ctx, model._h, self.comm._h, C.c_int(1 if self.sharded else 0))

    def _seen(self, off, cnt):
        self.ranges.append((off, cnt))

    def __enter__(self):
        self.ranges = []
        self.model.set_grad_hook(self._seen)
        self.model.gpu._call("asca_model_dp_arm", self.model._h, C.c_int(1))
        return self

    def __exit__(self, *exc):
        self.model.set_grad_hook(None)
        return False

    def step(self, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.01):
        """After the backward: wait for the exchanges, then the optimizer step (this rank's share when sharded)."""
        g = self.model.gpu
        g._call("asca_model_dp_step", g._ctx, self.model._h, _f(lr), _f(beta1), _f(beta2), _f(eps), _f(wd))

    def timeline(self):
        """Milliseconds of the last step: exposed gradient exchange, optimizer update, weight all-gather running
        past the update, and the wait of that step's forward for gathered weights."""
        out = (C.c_float * 4)()
        g = self.model.gpu
        g._call("asca_model_dp_timeline", g._ctx, self.model._h, out)
        return {"exposed_grad_exchange_ms": out[0], "optimizer_ms": out[1], "allgather_past_update_ms": out[2],
                "forward_waited_for_weights_ms": out[3]}

    def gather_master(self):
        """Collect the f32 master weights and moments of the other ranks' chunks (before reading parameters out)."""
        g = self.model.gpu
        g._call("asca_model_dp_gather_master", g._ctx, self.model._h)

    def detach(self):
        g = self.model.gpu
        g._call("asca_model_dp_attach", g._ctx, self.model._h, None, C.c_int(0))


class ShardedOverlap(GradOverlap):
    """GradOverlap with the optimizer sharded over the ranks for the expert weights (bf16 compute mode).

    W1 / W2 of every block are reduce-scattered instead of all-reduced (half the bytes), ``step(lr)`` updates this
    rank's 1/N chunk of them and all small tensors, and the updated bf16 chunks are all-gathered into every rank's
    bf16 weight copy block by block under the next forward. The f32 master weights and moments of the other ranks'
    chunks are then stale on this rank; the library refuses to read them out until ``gather_master()`` has run.
    """

    sharded = True

    def __init__(self, model, comm: Comm | None = None, group=None, transport: str = "nccl", exchange=None):
        """transport "ce": the sharded tensors travel on the copy engines through peer memory mapped with CUDA IPC
        (``asca_model_dp_peer_export`` / ``_open``) instead of NCCL kernels. `exchange` carries one rank's 256-byte
        blob to all ranks and returns the list in rank order; by default the initialised torch.distributed group does."""
        super().__init__(model, comm, group)
        self.big, self.slices = shard_plan(model.cfg, self.rank, self.world) if self.world > 1 else ([], [(0, model.n)])
        self.transport = "nccl"
        if transport == "ce" and self.world > 1 and self.big:
            g = model.gpu
            blob = C.create_string_buffer(256)
            g._call("asca_model_dp_peer_export", g._ctx, model._h, blob)
            if exchange is None:
                import torch.distributed as dist

                def exchange(b):
                    out = [None] * self.world
                    dist.all_gather_object(out, b, group=group)
                    return out
            blobs = exchange(blob.raw)
            assert len(blobs) == self.world and all(len(b) == 256 for b in blobs)
            g._call("asca_model_dp_peer_open", g._ctx, model._h, C.create_string_buffer(b"".join(blobs), 256 * self.world), C.c_int(self.world))
            self.transport = "ce"
