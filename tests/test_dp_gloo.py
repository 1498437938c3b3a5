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


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shard_plan_of_the_library_tiles_the_buffer(world):
    """The sharded optimizer's plan (asca_dp_shard_plan, host arithmetic inside the library; no GPU, no NCCL, no
    process group): over all ranks the expert tensors are covered exactly once, in equal 16-byte-aligned chunks;
    every other tensor is covered by every rank; a rank's ranges are sorted and disjoint. Checked against an
    independent statement built from the tensor sizes."""
    from asca_b200 import dp
    from asca_b200.train import tensor_sizes

    cfg = (256, 2048, 16, 2, 64, 4096)      # two blocks of the 1.3B-class training configuration
    sizes = tensor_sizes(cfg)
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    total = int(offs[-1])
    expert = [i for i in range(len(sizes)) if i >= 2 and (i - 2) % 10 in (6, 8)]
    plans = [dp.shard_plan(cfg, r, world) for r in range(world)]
    want_big = [(int(offs[i]), int(sizes[i])) for i in expert]
    for big, slices in plans:
        assert big == want_big
        assert all(lo < hi for lo, hi in slices)
        assert all(a[1] < b[0] for a, b in zip(slices, slices[1:]))       # sorted, disjoint, merged
        assert slices[0][0] == 0 and slices[-1][1] == total
    # coverage counts at the tensor boundaries and chunk boundaries
    edges = sorted({0, total} | {e for _, sl in plans for s in sl for e in s})
    for a, b in zip(edges, edges[1:]):
        owners = [r for r, (_, sl) in enumerate(plans) if any(lo <= a and b <= hi for lo, hi in sl)]
        in_big = next(((o, n) for o, n in want_big if o <= a and b <= o + n), None)
        if in_big is None:
            assert owners == list(range(world)), (a, b)
        else:
            o, n = in_big
            c = n // world
            assert owners == [(a - o) // c], (a, b)
            assert (a - o) % c == 0 and c % 4 == 0
    # one rank: nothing is sharded
    big1, sl1 = dp.shard_plan(cfg, 0, 1)
    assert big1 == [] and sl1 == [(0, total)]
    # a size that 4 x world does not divide stays whole
    odd = (256, 64, 4, 1, 3, 10)           # 64 * 3 * 10 = 1920 numbers per expert tensor
    big_o, sl_o = dp.shard_plan(odd, 0, 7)
    assert big_o == [] and sl_o == [(0, sum(tensor_sizes(odd)))]
