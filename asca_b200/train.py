"""Host side of training around the device model: checkpoint files, learning-rate schedule, data
windows and the step loop, with the reference's semantics so that files and runs are
interchangeable with it.

* Checkpoint formats (rust/src/train.rs:291-542). Both are little-endian:
  ``ASCA2CK1``  magic, 6 x u64 config (vocab, d_model, n_heads, n_layers, n_experts, d_ff), then per
                parameter tensor u64 numel + numel x f32 values;
  ``ASCARSM1``  magic, the same 6 x u64, u64 training step, then per tensor u64 numel + values +
                Adam m + Adam v. Written to ``path.tmp``, flushed to disk, then renamed over
                ``path`` (a reader sees the old file or the new one, never a mixture).
  Tensor order is the flat parameter order of :class:`asca_b200.Model` (embed, head, then per block
  w_qkv, b_qkv, w_gate, b_gate, w_o, b_o, w1, b1, w2, b2; rust/src/model.rs:593-609).
* ``lr_at`` (rust/src/train.rs:201-212): linear warm-up, then cosine to 10 % of the peak, f32.
* ``Data.batch_seqs`` (rust/src/train.rs:128-155): `batch` windows of seq_len + 1 tokens at offsets
  drawn with the reference generator (xorshift128+, rust/src/tensor.rs:306-337); targets are the
  window shifted by one.
* ``Trainer`` (rust/src/train.rs:214-288): per step lr_at, zero grads, one batch, forward + backward,
  AdamW; periodic save through the resume format.
"""
from __future__ import annotations

import math
import os
import struct
from dataclasses import dataclass

import numpy as np

MAGIC = b"ASCA2CK1"
MAGIC_RESUME = b"ASCARSM1"
_M64 = (1 << 64) - 1


class Rng:
    """The reference's xorshift128+ stream (rust/src/tensor.rs:306-337): same seeds, same numbers."""

    def __init__(self, seed: int):
        self.s0 = ((seed * 0x9E3779B97F4A7C15) & _M64) | 1
        self.s1 = (((seed ^ 0xDEADBEEFCAFEF00D) * 0xBF58476D1CE4E5B9) & _M64) | 1

    def next_u64(self) -> int:
        x, y = self.s0, self.s1
        self.s0 = y
        x ^= (x << 23) & _M64
        self.s1 = x ^ y ^ (x >> 17) ^ (y >> 26)
        return (self.s1 + y) & _M64

    def below(self, n: int) -> int:
        return self.next_u64() % n

    def uniform(self) -> float:
        return float(np.float32(self.next_u64() >> 40) / np.float32(1 << 24))


def tensor_sizes(cfg):
    """numel of every parameter tensor in flat order for cfg = (vocab, d, H, L, E, F)."""
    vocab, d, H, L, E, F = cfg
    out = [vocab * d, d * vocab]
    for _ in range(L):
        out += [d * 3 * d, 3 * d, d * 2 * H, 2 * H, d * d, d, d * E * F, E * F, E * F * d, d]
    return out


def _header(magic, cfg):
    return magic + struct.pack("<6Q", *[int(c) for c in cfg])


def write_checkpoint(path, cfg, params):
    """Weights only (``ASCA2CK1``)."""
    params = np.ascontiguousarray(params, dtype="<f4")
    sizes = tensor_sizes(cfg)
    assert params.size == sum(sizes), "parameter count does not match the configuration"
    with open(path, "wb") as f:
        f.write(_header(MAGIC, cfg))
        off = 0
        for n in sizes:
            f.write(struct.pack("<Q", n))
            f.write(params[off:off + n].tobytes())
            off += n


def write_resume(path, cfg, step, params, m, v):
    """Weights, Adam moments and step number (``ASCARSM1``), written atomically."""
    arrs = [np.ascontiguousarray(a, dtype="<f4") for a in (params, m, v)]
    sizes = tensor_sizes(cfg)
    assert all(a.size == sum(sizes) for a in arrs), "buffer size does not match the configuration"
    tmp = f"{path}.tmp"
    with open(tmp, "wb") as f:
        f.write(_header(MAGIC_RESUME, cfg))
        f.write(struct.pack("<Q", int(step)))
        off = 0
        for n in sizes:
            f.write(struct.pack("<Q", n))
            for a in arrs:
                f.write(a[off:off + n].tobytes())
            off += n
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def _need(buf, off, n):
    if off + n > len(buf):
        raise ValueError(f"checkpoint truncated: need {n} bytes at offset {off}, file has {len(buf)}")


def peek_resume(path):
    """(cfg, step) from the 64-byte header of a resume checkpoint, without reading the weights."""
    with open(path, "rb") as f:
        head = f.read(64)
    if len(head) < 64 or head[:8] != MAGIC_RESUME:
        raise ValueError("not a resume checkpoint (no ASCARSM1 header): the step number is unknown")
    nums = struct.unpack("<7Q", head[8:64])
    return tuple(nums[:6]), nums[6]


def read_checkpoint(path):
    """Either format -> dict(cfg, step, params, m, v). A weights-only file gives step 0 and no moments."""
    with open(path, "rb") as f:
        buf = f.read()
    if len(buf) < 56:
        raise ValueError("checkpoint too small")
    magic = buf[:8]
    if magic not in (MAGIC, MAGIC_RESUME):
        raise ValueError("not an ASCA v2 checkpoint")
    resume = magic == MAGIC_RESUME
    cfg = struct.unpack("<6Q", buf[8:56])
    off = 56
    step = 0
    if resume:
        _need(buf, off, 8)
        step = struct.unpack("<Q", buf[off:off + 8])[0]
        off += 8
    sizes = tensor_sizes(cfg)
    total = sum(sizes)
    outs = [np.empty(total, np.float32) for _ in range(3 if resume else 1)]
    pos = 0
    for i, want in enumerate(sizes):
        _need(buf, off, 8)
        n = struct.unpack("<Q", buf[off:off + 8])[0]
        off += 8
        if n != want:
            raise ValueError(f"size of parameter {i} does not match: {n} vs {want}")
        for a in outs:
            _need(buf, off, 4 * n)
            a[pos:pos + n] = np.frombuffer(buf, dtype="<f4", count=n, offset=off)
            off += 4 * n
        pos += n
    return {"cfg": tuple(int(c) for c in cfg), "step": int(step), "params": outs[0],
            "m": outs[1] if resume else None, "v": outs[2] if resume else None}


def save_model(path, model, step=None):
    """Device model -> file. With `step` the resume format (moments included), else weights only."""
    params, _ = model.get()
    if step is None:
        write_checkpoint(path, model.cfg, params)
    else:
        m, v = model.moments()
        write_resume(path, model.cfg, step, params, m, v)


def load_model(gpu, path):
    """File -> (device model, step). Restores the moments and, like the reference's load_resume,
    sets AdamW's counter to the saved training step (rust/src/train.rs:454-455)."""
    import asca_b200

    ck = read_checkpoint(path)
    model = asca_b200.Model(gpu, *ck["cfg"])
    model.set_params(ck["params"])
    if ck["m"] is not None:
        model.set_moments(ck["m"], ck["v"])
        model.adam_counter(ck["step"] & 0xFFFFFFFF)
    return model, ck["step"]


def lr_at(step: int, lr: float, warmup: int, steps: int) -> float:
    """Warm-up then cosine decay to 10 % (f32 arithmetic, rust/src/train.rs:201-212)."""
    f = np.float32
    lr = f(lr)
    if step < warmup:
        return float(lr * (f(step) + f(1.0)) / f(warmup))
    progress = f(step - warmup) / f(max(steps, warmup + 1) - warmup)
    min_lr = lr * f(0.1)
    return float(min_lr + f(0.5) * (lr - min_lr) * (f(1.0) + f(math.cos(float(f(math.pi) * progress)))))


class Data:
    """A token stream with a train / validation split at train_end = floor(len * (1 - val_frac)) in f32."""

    def __init__(self, tokens, val_frac=0.1):
        self.tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        self.train_end = int(np.float32(self.tokens.size) * (np.float32(1.0) - np.float32(val_frac)))

    @classmethod
    def from_bytes(cls, raw: bytes, val_frac=0.1):
        if len(raw) < 1024:
            raise ValueError("file too small")
        return cls(np.frombuffer(raw, dtype=np.uint8).astype(np.uint32), val_frac)

    def batch(self, rng: Rng, seq_len: int, split="train"):
        lo, hi = (0, self.train_end) if split == "train" else (self.train_end, self.tokens.size)
        span = max(max(hi - lo, 0) - (seq_len + 1), 0)
        span = max(span, 1)
        start = lo + rng.below(span)
        return self.tokens[start:start + seq_len], self.tokens[start + 1:start + 1 + seq_len]

    def batch_seqs(self, rng: Rng, seq_len: int, batch: int, split="train"):
        ids, tgts = zip(*(self.batch(rng, seq_len, split) for _ in range(batch)))
        return np.concatenate(ids), np.concatenate(tgts)


@dataclass
class TrainCfg:
    steps: int
    seq_len: int
    batch: int
    lr: float = 3e-3
    warmup: int = 0
    save_every: int = 0


class Trainer:
    """The reference's step loop on the device model (rust/src/train.rs:214-288)."""

    def __init__(self, model, data: Data, cfg: TrainCfg, seed: int, start_step: int = 0):
        self.model, self.data, self.cfg = model, data, cfg
        self.rng = Rng(seed)
        self.step = start_step

    def train_step(self) -> float:
        c = self.cfg
        lr = lr_at(self.step, c.lr, c.warmup, c.steps)
        self.model.zero_grads()
        ids, tgts = self.data.batch_seqs(self.rng, c.seq_len, c.batch, "train")
        loss = self.model.forward_backward(ids, tgts, c.batch)
        self.model.adamw_step(lr)
        self.step += 1
        return loss

    def run(self, save_path=None):
        losses = []
        while self.step < self.cfg.steps:
            losses.append(self.train_step())
            if save_path and self.cfg.save_every and self.step % self.cfg.save_every == 0:
                save_model(save_path, self.model, self.step)
        return losses
