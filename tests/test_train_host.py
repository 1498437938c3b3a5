"""Host side of training (asca_b200/train.py): checkpoint formats ASCA2CK1 / ASCARSM1, learning-rate
schedule, data windows and the reference generator -- CPU only."""
import os
import struct

import numpy as np
import pytest

from asca_b200 import train

CFG = (256, 16, 2, 2, 4, 32)


def _flat(seed):
    n = sum(train.tensor_sizes(CFG))
    return np.random.default_rng(seed).standard_normal(n).astype(np.float32)


def test_rng_matches_the_oracle_stream(orc):
    for seed in (0, 1, 42, 2**40 + 7):
        a, b = train.Rng(seed), orc.Rng(seed)
        assert [a.below(1 << 32) for _ in range(200)] == [int(x) for x in b.below(1 << 32, 200)]
    a, b = train.Rng(9), orc.Rng(9)
    assert [a.below(977) for _ in range(50)] == [int(x) for x in b.below(977, 50)]


def test_tensor_sizes_follow_the_flat_parameter_order(orc):
    ref = orc.Model(*CFG)
    assert [ref.tensor(n).size for n in ref.names] == train.tensor_sizes(CFG)
    assert sum(train.tensor_sizes((256, 64, 4, 2, 4, 256))) == 331408


def test_weights_only_checkpoint_round_trip(tmp_path):
    p = _flat(1)
    path = tmp_path / "w.bin"
    train.write_checkpoint(path, CFG, p)
    raw = path.read_bytes()
    assert raw[:8] == b"ASCA2CK1" and struct.unpack("<6Q", raw[8:56]) == CFG
    assert struct.unpack("<Q", raw[56:64])[0] == train.tensor_sizes(CFG)[0]        # first tensor: numel then values
    assert np.array_equal(np.frombuffer(raw, "<f4", 4, 64), p[:4])
    assert len(raw) == 56 + 8 * len(train.tensor_sizes(CFG)) + 4 * p.size
    ck = train.read_checkpoint(path)
    assert ck["cfg"] == CFG and ck["step"] == 0 and ck["m"] is None
    assert np.array_equal(ck["params"], p)


def test_resume_checkpoint_round_trip_is_atomic_and_peekable(tmp_path):
    p, m, v = _flat(2), _flat(3), np.abs(_flat(4))
    path = tmp_path / "r.bin"
    train.write_resume(path, CFG, 1234, p, m, v)
    assert not os.path.exists(f"{path}.tmp")
    assert train.peek_resume(path) == (CFG, 1234)
    raw = path.read_bytes()
    n0 = train.tensor_sizes(CFG)[0]
    assert raw[:8] == b"ASCARSM1" and struct.unpack("<Q", raw[56:64])[0] == 1234
    assert struct.unpack("<Q", raw[64:72])[0] == n0
    # per tensor: values, then m, then v
    assert np.array_equal(np.frombuffer(raw, "<f4", n0, 72), p[:n0])
    assert np.array_equal(np.frombuffer(raw, "<f4", n0, 72 + 4 * n0), m[:n0])
    assert np.array_equal(np.frombuffer(raw, "<f4", n0, 72 + 8 * n0), v[:n0])
    ck = train.read_checkpoint(path)
    assert ck["step"] == 1234
    for k, a in (("params", p), ("m", m), ("v", v)):
        assert np.array_equal(ck[k], a)
    # a second save replaces the file in one step
    train.write_resume(path, CFG, 1235, p, m, v)
    assert train.peek_resume(path)[1] == 1235


def test_bad_files_give_readable_errors(tmp_path):
    p = _flat(5)
    path = tmp_path / "t.bin"
    train.write_resume(path, CFG, 7, p, p, p)
    raw = path.read_bytes()
    (tmp_path / "cut.bin").write_bytes(raw[: len(raw) // 2])
    with pytest.raises(ValueError, match="truncated"):
        train.read_checkpoint(tmp_path / "cut.bin")
    (tmp_path / "magic.bin").write_bytes(b"NOTASCA!" + raw[8:])
    with pytest.raises(ValueError, match="not an ASCA"):
        train.read_checkpoint(tmp_path / "magic.bin")
    train.write_checkpoint(tmp_path / "w.bin", CFG, p)
    with pytest.raises(ValueError, match="not a resume"):
        train.peek_resume(tmp_path / "w.bin")
    wrong = bytearray(raw)
    wrong[64:72] = struct.pack("<Q", 3)
    (tmp_path / "size.bin").write_bytes(bytes(wrong))
    with pytest.raises(ValueError, match="does not match"):
        train.read_checkpoint(tmp_path / "size.bin")


def test_lr_schedule_warmup_then_cosine_to_ten_percent():
    lr, warm, steps = 3e-3, 10, 110
    assert train.lr_at(0, lr, warm, steps) == pytest.approx(lr / 10, rel=1e-6)
    assert train.lr_at(9, lr, warm, steps) == pytest.approx(lr, rel=1e-6)
    assert train.lr_at(10, lr, warm, steps) == pytest.approx(lr, rel=1e-6)            # progress 0
    assert train.lr_at(60, lr, warm, steps) == pytest.approx(0.55 * lr, rel=1e-5)      # progress 0.5
    assert train.lr_at(110, lr, warm, steps) == pytest.approx(0.1 * lr, rel=1e-5)      # progress 1
    vals = [train.lr_at(s, lr, warm, steps) for s in range(10, 111)]
    assert all(a >= b for a, b in zip(vals, vals[1:]))
    assert train.lr_at(0, lr, 0, 1) == pytest.approx(lr, rel=1e-6)                     # no warm-up, step 0 of a run


def test_data_windows_use_the_reference_offsets(orc):
    raw = bytes(np.random.default_rng(0).integers(0, 256, 5000, dtype=np.uint8))
    data = train.Data.from_bytes(raw, val_frac=0.1)
    assert data.train_end == 4500
    rng, ref = train.Rng(3), orc.Rng(3)
    ids, tg = data.batch_seqs(rng, 64, 5, "train")
    assert ids.shape == tg.shape == (5 * 64,)
    for b in range(5):
        start = int(ref.below(4500 - 65, 1)[0])
        assert np.array_equal(ids[b * 64:(b + 1) * 64], data.tokens[start:start + 64])
        assert np.array_equal(tg[b * 64:(b + 1) * 64], data.tokens[start + 1:start + 65])
    ids, tg = data.batch(rng, 64, "val")
    start = 4500 + int(ref.below(500 - 65, 1)[0])
    assert np.array_equal(ids, data.tokens[start:start + 64])
    with pytest.raises(ValueError):
        train.Data.from_bytes(b"short")


def test_shard_plan_partitions_the_expert_weights_and_keeps_the_rest_everywhere():
    """dp.shard_plan: over all ranks the chunks of every sharded tensor tile it exactly once, every other element is in
    every rank's slices, slices are sorted, disjoint and start at multiples of 4."""
    from asca_b200.dp import shard_plan
    from asca_b200.train import tensor_sizes

    cfg = (256, 64, 4, 2, 4, 256)
    n = sum(tensor_sizes(cfg))
    for world in (1, 2, 4, 8):
        cover = np.zeros(n, np.int32)
        for rank in range(world):
            big, slices = shard_plan(cfg, rank, world)
            assert all(lo % 4 == 0 and hi > lo for lo, hi in slices)
            assert all(a[1] < b[0] for a, b in zip(slices, slices[1:]))          # sorted, disjoint, merged
            for lo, hi in slices:
                cover[lo:hi] += 1
        sharded = np.zeros(n, bool)
        for lo, size in big:
            sharded[lo:lo + size] = True
        assert (cover[sharded] == 1).all() and (cover[~sharded] == world).all()
        assert len(big) == (0 if world == 1 else 2 * cfg[3])                        # W1 and W2 of every block
