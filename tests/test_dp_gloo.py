"""world_size-2 data parallelism on CPU (gloo): sharding by sequence plus the one gradient
all-reduce reproduce the single-process step. The per-rank compute stand-in is the CPU oracle;
on GPUs the same functions run on the device gradient buffer."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
TINY = (256, 64, 4, 2, 8, 128)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    import oracle
    from asca_b200 import dp

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    oracle.set_threads(2)
    batch, seq = 6, 10
    rng = oracle.Rng(5)
    ids, tg = rng.below(256, batch * seq), rng.below(256, batch * seq)
    model = oracle.Model(*TINY)
    model.init_reference(oracle.Rng(9))
    my_ids, local_b = dp.shard_tokens(ids, batch, rank, world)
    my_tg, _ = dp.shard_tokens(tg, batch, rank, world)
    loss, grads = model.forward_backward(my_ids, my_tg, local_b)
    flat = torch.from_numpy(grads)
    dp.allreduce_mean_(flat, local_b / batch)
    lt = torch.tensor([loss * local_b / batch], dtype=torch.float64)
    dist.all_reduce(lt)
    np.save(Path(out_dir) / f"g{rank}.npy", flat.numpy())
    np.save(Path(out_dir) / f"l{rank}.npy", lt.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_shard_sequences_covers_everything_once():
    from asca_b200 import dp

    for n, w in ((64, 8), (7, 3), (2, 4), (256, 8)):
        seen = [i for r in range(w) for i in dp.shard_sequences(n, r, w)]
        assert seen == list(range(n))
        sizes = [len(dp.shard_sequences(n, r, w)) for r in range(w)]
        assert max(sizes) - min(sizes) <= 1


def test_two_ranks_reproduce_the_single_process_step(tmp_path):
    import torch.multiprocessing as mp

    import oracle

    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    oracle.set_threads(0)
    batch, seq = 6, 10
    rng = oracle.Rng(5)
    ids, tg = rng.below(256, batch * seq), rng.below(256, batch * seq)
    model = oracle.Model(*TINY)
    model.init_reference(oracle.Rng(9))
    loss, grads = model.forward_backward(ids, tg, batch)
    g0, g1 = np.load(tmp_path / "g0.npy"), np.load(tmp_path / "g1.npy")
    assert np.array_equal(g0, g1)                      # every rank ends with the same buffer
    for name in model.names:                           # batch_parity.rs tolerance
        a, b = model.tensor(name, g0), model.tensor(name, grads)
        assert np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-9) <= 2e-4, name
    l0 = float(np.load(tmp_path / "l0.npy")[0])
    assert abs(l0 - loss) / abs(loss) <= 1e-5
