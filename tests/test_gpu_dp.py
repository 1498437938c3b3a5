"""The data-parallel exchange behind the C ABI (asca_comm_* / asca_allreduce_grads / asca_model_dp_*).

One GPU: the sharded optimizer's slices, applied rank by rank on one model, equal the full step bit for bit;
a one-rank communicator is a no-op that needs no NCCL. Two GPUs (skipped on a single-GPU machine): two ranks as
child processes, NCCL loaded by the library itself, the 128-byte id handed over through a file -- the overlapped
exchange equals a blocking all-reduce of the whole buffer bit for bit, the sharded and the replicated optimizer
give identical weights, and reading stale master weights is refused until they are gathered.
"""
import json
import os
import sys
import time
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
CFG = (256, 512, 4, 2, 4, 256)       # head dim 128, every tensor a multiple of 8 numbers: unpadded bf16 copy


def _tokens(orc, B, T, seed):
    rng = orc.Rng(seed)
    ids = rng.below(256, B * T)
    tg = np.concatenate([ids.reshape(B, T)[:, 1:], rng.below(256, (B, 1))], axis=1).reshape(-1).astype(np.uint32)
    return ids, tg


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_slices_applied_rank_by_rank_equal_the_full_step(orc, gpu, world):
    import torch

    import asca_b200
    from asca_b200 import dp

    ref = orc.Model(*CFG)
    ref.init_reference(orc.Rng(21))
    ids, tg = _tokens(orc, 2, 96, 22)
    models = []
    for _ in range(2):
        m = asca_b200.Model(gpu, *CFG)
        m.set_params(ref.params)
        m.set_compute(asca_b200.BF16)
        models.append(m)
    full, sliced = models
    for step in range(2):
        for m in models:
            m.zero_grads()
            m.forward_backward(ids, tg, 2)
        full.adamw_step(3e-3)
        sliced.params16()
        for r in range(world):
            big, slices = dp.shard_plan(CFG, r, world)
            if r > 0:   # on ONE model the tensors every rank updates must be updated once: keep rank r's chunks only
                slices = [(max(lo, o), min(hi, o + n)) for lo, hi in slices for o, n in big if max(lo, o) < min(hi, o + n)]
            sliced.adamw_slices(3e-3, slices, advance=(r == world - 1))
        assert sliced.adam_counter() == full.adam_counter() == (step + 1) * len(ref.names)
        pa, _ = full.get()
        pb, _ = sliced.get()
        assert np.array_equal(pa, pb)
        for a, b in zip(full.moments(), sliced.moments()):
            assert np.array_equal(a, b)
        a16 = dp.device_tensor_bf16(*full.params16(), 0)
        b16 = dp.device_tensor_bf16(*sliced.params16(), 0)
        assert torch.equal(a16.view(torch.int16), b16.view(torch.int16))
    for m in models:
        m.free()


def test_one_rank_communicator_is_a_no_op(orc, gpu):
    import asca_b200
    from asca_b200 import dp

    ref = orc.Model(*CFG)
    ref.init_reference(orc.Rng(23))
    ids, tg = _tokens(orc, 2, 64, 24)
    a, b = (asca_b200.Model(gpu, *CFG) for _ in range(2))
    for m in (a, b):
        m.set_params(ref.params)
        m.set_compute(asca_b200.BF16)
        m.zero_grads()
    comm = dp.Comm(gpu, 1, 0, None)
    ov = dp.ShardedOverlap(a, comm)
    with ov:
        a.forward_backward(ids, tg, 2)
    b.forward_backward(ids, tg, 2)
    assert sorted(ov.ranges)[0][0] == 0 and sum(n for _, n in ov.ranges) == a.n
    assert len(ov.ranges) == 2 * CFG[3] + 1          # experts and projections of every block, then embedding + head
    comm.allreduce_grads(a.buffers()[1], a.n, [0, a.n // 2, a.n])
    ov.step(3e-3)
    b.adamw_step(3e-3)
    (pa, ga), (pb, gb) = a.get(), b.get()
    assert np.array_equal(pa, pb) and np.array_equal(ga, gb)
    t = ov.timeline()
    assert t["exposed_grad_exchange_ms"] >= 0 and t["optimizer_ms"] > 0
    ov.detach()
    comm.close()
    a.free()
    b.free()


# ------------------------------------------------------------------ two ranks on two GPUs
def _rank_main(rank, world, tmp):
    sys.path.insert(0, str(ROOT))
    import torch

    import asca_b200
    import oracle
    from asca_b200 import dp

    torch.cuda.set_device(rank)
    gpu = asca_b200.Gpu(rank)
    idf = Path(tmp) / "nccl_id"
    if rank == 0:
        raw = dp.Comm.unique_id(gpu)
        (Path(tmp) / "nccl_id.tmp").write_bytes(raw)
        os.replace(Path(tmp) / "nccl_id.tmp", idf)
    else:
        for _ in range(600):
            if idf.exists():
                break
            time.sleep(0.05)
        raw = idf.read_bytes()
    comm = dp.Comm(gpu, world, rank, raw)
    ref = oracle.Model(*CFG)
    ref.init_reference(oracle.Rng(31))
    B, T = 4, 128
    rng = oracle.Rng(32)
    ids = rng.below(256, B * T)
    tg = np.concatenate([ids.reshape(B, T)[:, 1:], rng.below(256, (B, 1))], axis=1).reshape(-1).astype(np.uint32)
    my_ids, lb = dp.shard_tokens(ids, B, rank, world)
    my_tg, _ = dp.shard_tokens(tg, B, rank, world)
    models = {}
    for name in ("sharded", "replicated", "blocking", "ce"):
        m = asca_b200.Model(gpu, *CFG)
        m.set_params(ref.params)
        m.set_compute(asca_b200.BF16)
        models[name] = m
    ov_s = dp.ShardedOverlap(models["sharded"], comm)
    ov_r = dp.GradOverlap(models["replicated"], comm)

    def exchange(blob):   # the 256-byte peer blobs travel through files, like the NCCL id
        (Path(tmp) / f"ce_blob{rank}.tmp").write_bytes(blob)
        os.replace(Path(tmp) / f"ce_blob{rank}.tmp", Path(tmp) / f"ce_blob{rank}")
        blobs = []
        for r in range(world):
            f = Path(tmp) / f"ce_blob{r}"
            for _ in range(600):
                if f.exists():
                    break
                time.sleep(0.05)
            blobs.append(f.read_bytes())
        return blobs

    ov_c = dp.ShardedOverlap(models["ce"], comm, transport="ce", exchange=exchange)
    out = {"rank": rank, "ce_transport": ov_c.transport}
    for step in range(3):
        for name, m in models.items():
            m.zero_grads()
            if name == "sharded":
                with ov_s:
                    m.forward_backward(my_ids, my_tg, lb)
            elif name == "replicated":
                with ov_r:
                    m.forward_backward(my_ids, my_tg, lb)
            elif name == "ce":
                with ov_c:
                    m.forward_backward(my_ids, my_tg, lb)
            else:
                m.forward_backward(my_ids, my_tg, lb)
                dp.allreduce_model_grads(m, comm)
        gpu.sync()
        if step == 0:
            g_r = dp.device_tensor(models["replicated"].buffers()[1], ref.n, rank)
            g_b = dp.device_tensor(models["blocking"].buffers()[1], ref.n, rank)
            g_s = dp.device_tensor(models["sharded"].buffers()[1], ref.n, rank)
            out["overlapped_equals_blocking"] = bool(torch.equal(g_r, g_b))
            own = all(bool(torch.equal(g_s[lo:hi], g_b[lo:hi])) for lo, hi in ov_s.slices)
            out["reduce_scattered_own_slices_equal"] = own
            np.save(Path(tmp) / f"grads{rank}.npy", g_b.cpu().numpy())
        ov_s.step(3e-3)
        ov_r.step(3e-3)
        ov_c.step(3e-3)
        models["blocking"].adamw_step(3e-3)
    w16 = {k: dp.device_tensor_bf16(*m.params16(), rank).view(torch.int16) for k, m in models.items()}
    out["bf16_weights_sharded_equal_replicated"] = bool(torch.equal(w16["sharded"], w16["replicated"]))
    out["bf16_weights_replicated_equal_blocking"] = bool(torch.equal(w16["replicated"], w16["blocking"]))
    # copy-engine transport: at two ranks the sum of two numbers has one order, so it equals the NCCL path bit for bit
    out["bf16_weights_ce_equal_sharded"] = bool(torch.equal(w16["ce"], w16["sharded"]))
    try:
        models["sharded"].get()
        out["stale_master_refused"] = False
    except asca_b200.AscaError as e:
        out["stale_master_refused"] = "gather_master" in str(e)
    ov_s.gather_master()
    ps, _ = models["sharded"].get()
    pr, _ = models["replicated"].get()
    out["master_equal_after_gather"] = bool(np.array_equal(ps, pr))
    out["timeline"] = ov_s.timeline()
    (Path(tmp) / f"out{rank}.json").write_text(json.dumps(out))
    for m in models.values():
        m.free()
    comm.close()


def test_two_ranks_overlapped_exchange_and_sharded_optimizer(orc, tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    env = dict(os.environ)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        mp.spawn(_rank_main, args=(2, str(tmp_path)), nprocs=2, join=True)
    finally:
        os.environ.clear()
        os.environ.update(env)
    outs = [json.loads((tmp_path / f"out{r}.json").read_text()) for r in range(2)]
    for o in outs:
        assert o["overlapped_equals_blocking"], o
        assert o["reduce_scattered_own_slices_equal"], o
        assert o["bf16_weights_sharded_equal_replicated"], o
        assert o["bf16_weights_replicated_equal_blocking"], o
        assert o["ce_transport"] == "ce" and o["bf16_weights_ce_equal_sharded"], o
        assert o["stale_master_refused"], o
        assert o["master_equal_after_gather"], o
    g0, g1 = np.load(tmp_path / "grads0.npy"), np.load(tmp_path / "grads1.npy")
    assert np.array_equal(g0, g1)                      # every rank ends with the same averaged buffer
    # and it is the gradient of the whole batch (bf16 tolerance against the f32 oracle)
    ref = orc.Model(*CFG)
    ref.init_reference(orc.Rng(31))
    ids, tg = _tokens(orc, 4, 128, 32)
    _, g_ref = ref.forward_backward(ids, tg, 4)
    for name in ref.names:
        a, b = ref.tensor(name, g0), ref.tensor(name, g_ref)
        if b.size >= 64 and np.abs(b).max() > 0:
            assert np.abs(a - b).max() / np.abs(b).max() < 2e-2, name
