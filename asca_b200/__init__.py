"""asca_b200 -- B200 (sm_100a) backend for ASCA's Delta Memory / hash-MoE hot path.

The product is ``libasca_b200.so`` (hand-written CUDA behind the C ABI of
``include/asca_b200.h``). This package is the thin host side above it:

* :class:`Gpu` mirrors the reference's ``impl Gpu`` (rust/src/cuda/mod.rs): the same method
  names, argument meaning and error behaviour (an exception carrying the library's message
  where the reference returns ``Err(String)``), on host (numpy) arrays.
* :mod:`asca_b200.ops` exposes the device-pointer entry points on torch CUDA tensors, for
  callers that keep activations resident in HBM.

There is no CPU fallback: if the library is missing or no CUDA device is present, creating
a :class:`Gpu` raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
LIB_PATH = _DIR / "libasca_b200.so"

F32, BF16 = 0, 1
NN, TN, NT = 0, 1, 2

_lib = None


class AscaError(RuntimeError):
    """A library call returned a negative ASCA_ERR_* status."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"asca_b200 error {code}: {msg}")
        self.code = code


def load() -> C.CDLL:
    """dlopen the in-tree library (built by ``python -m asca_b200.build``). Never falls back."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m asca_b200.build` "
                "(nvcc, sm_100a). There is no CPU fallback.")
        _lib = C.CDLL(str(LIB_PATH))
        _lib.asca_last_error.restype = C.c_char_p
        _lib.asca_describe.restype = C.c_char_p
        _lib.asca_version.restype = C.c_char_p
        _lib.asca_launch_count.restype = C.c_int64
        _lib.asca_delta_ckpt_floats.restype = C.c_int64
        _lib.asca_delta_ckpt_floats.argtypes = [C.c_int64] * 5
    return _lib


def _p(a):
    """Pointer of a numpy array / torch tensor / raw int / None as c_void_p."""
    if a is None:
        return C.c_void_p(0)
    if isinstance(a, int):
        return C.c_void_p(a)
    if isinstance(a, np.ndarray):
        assert a.flags.c_contiguous, "array must be C-contiguous"
        return C.c_void_p(a.ctypes.data)
    if hasattr(a, "data_ptr"):
        assert a.is_contiguous(), "tensor must be contiguous"
        return C.c_void_p(a.data_ptr())
    raise TypeError(type(a))


def _i64(v):
    return C.c_int64(int(v))


def _f(v):
    return C.c_float(float(v))


def _as_f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class DeltaDev:
    """Device-resident q,k,v,alpha,beta + chunk checkpoints between delta_scan and delta_bwd_dev
    (the reference's DeltaDev, rust/src/cuda/mod.rs:1386-1397)."""

    def __init__(self, gpu, handle, batch, seq, n_heads, dh):
        self._gpu, self._h = gpu, handle
        self.batch, self.seq, self.n_heads, self.dh = batch, seq, n_heads, dh

    def download_states(self):
        """Per-step state history, list of H*B arrays of (seq+1)*dh*dh floats, chain index
        h*B + b (rust/src/cuda/mod.rs:1473-1480). Recomputed on the device; refused when large."""
        n = self.n_heads * self.batch
        out = np.empty((n, (self.seq + 1) * self.dh * self.dh), np.float32)
        self._gpu._call("asca_delta_dev_download_states", self._gpu._ctx, self._h, _p(out))
        return [out[i] for i in range(n)]

    def free(self):
        if self._h is not None:
            self._gpu._call("asca_delta_dev_free", self._gpu._ctx, self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class MoeDev:
    """Device-resident xn, weights, pre/hidden and the dispatch between moe_forward_dev and
    moe_bwd_dev (the reference's MoeDev, rust/src/cuda/mod.rs:1416-1431)."""

    def __init__(self, gpu, handle, t_len, d, d_ff, n_experts):
        self._gpu, self._h = gpu, handle
        self.t_len, self.d, self.d_ff, self.n_experts = t_len, d, d_ff, n_experts

    def download_pre_hidden(self):
        pre = np.empty((self.t_len, self.d_ff), np.float32)
        hid = np.empty((self.t_len, self.d_ff), np.float32)
        self._gpu._call("asca_moe_dev_download_pre_hidden", self._gpu._ctx, self._h, _p(pre), _p(hid))
        return pre, hid

    def free(self):
        if self._h is not None:
            self._gpu._call("asca_moe_dev_free", self._gpu._ctx, self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class MoeBwd:
    """Result of moe_bwd_dev (rust/src/cuda/mod.rs:745-824)."""

    def __init__(self, d_w1, d_b1, d_w2, d_b2, dxn):
        self.d_w1, self.d_b1, self.d_w2, self.d_b2, self.dxn = d_w1, d_b1, d_w2, d_b2, dxn


class Gpu:
    """One context per GPU; host-array methods named after the reference's ``impl Gpu``."""

    def __init__(self, device: int = 0):
        self.lib = load()
        ctx = C.c_void_p()
        rc = self.lib.asca_ctx_create(C.c_int(device), C.byref(ctx))
        if rc != 0 or not ctx:
            raise AscaError(rc, f"cannot create a context on CUDA device {device} (no GPU, or driver missing); "
                                "there is no CPU fallback")
        self._ctx = ctx
        self.device = device

    # ---- plumbing
    def _call(self, name, *args):
        rc = getattr(self.lib, name)(*args)
        if rc != 0:
            raise AscaError(rc, self.lib.asca_last_error(self._ctx).decode())

    def describe(self) -> str:
        return self.lib.asca_describe(self._ctx).decode()

    def launch_count(self) -> int:
        return int(self.lib.asca_launch_count(self._ctx))

    def set_stream(self, cuda_stream: int | None):
        self._call("asca_ctx_set_stream", self._ctx, C.c_void_p(cuda_stream or 0))

    def use_torch_stream(self):
        import torch

        # torch's default stream has handle 0, which the C ABI reads as "the context's own
        # stream"; CUDA's explicit handle for the legacy default stream is 1 (cudaStreamLegacy).
        self.set_stream(torch.cuda.current_stream(self.device).cuda_stream or 1)

    def profile(self, on: bool):
        """Switch per-kernel CUDA-event timing of the delta-rule kernels on or off (clears the record)."""
        self._call("asca_ctx_profile", self._ctx, C.c_int(1 if on else 0))

    def profile_read(self, with_work=False):
        """[(kernel name, milliseconds)] recorded since profile(True); with_work adds the launch's stated
        algorithmic FLOPs or bytes (0 where the launcher states none)."""
        out, i = [], 0
        name, ms, work = C.c_char_p(), C.c_float(), C.c_double()
        while self.lib.asca_ctx_profile_read(self._ctx, C.c_int(i), C.byref(name), C.byref(ms)) == 0:
            if with_work:
                self.lib.asca_ctx_profile_work(self._ctx, C.c_int(i), C.byref(work))
                out.append((name.value.decode(), float(ms.value), float(work.value)))
            else:
                out.append((name.value.decode(), float(ms.value)))
            i += 1
        return out

    def sync(self):
        self._call("asca_ctx_sync", self._ctx)

    def close(self):
        if self._ctx:
            self.lib.asca_ctx_destroy(self._ctx)
            self._ctx = None

    # ---- Gpu::matmul / matmul_ta (rust/src/cuda/mod.rs:286-344)
    def matmul(self, a, b):
        a, b = _as_f32(a), _as_f32(b)
        assert a.shape[1] == b.shape[0], "matmul: inner dims differ"
        c = np.empty((a.shape[0], b.shape[1]), np.float32)
        self._call("asca_matmul_host", self._ctx, _p(a), _p(b), _p(c), _i64(a.shape[0]), _i64(a.shape[1]),
                   _i64(b.shape[1]), C.c_int(NN))
        return c

    def matmul_ta(self, a, b):
        a, b = _as_f32(a), _as_f32(b)
        assert a.shape[0] == b.shape[0], "matmul_ta: row counts differ"
        c = np.empty((a.shape[1], b.shape[1]), np.float32)
        self._call("asca_matmul_host", self._ctx, _p(a), _p(b), _p(c), _i64(a.shape[1]), _i64(a.shape[0]),
                   _i64(b.shape[1]), C.c_int(TN))
        return c

    def matmul_t(self, a, b):
        a, b = _as_f32(a), _as_f32(b)
        assert a.shape[1] == b.shape[1], "matmul_t: inner dims differ"
        c = np.empty((a.shape[0], b.shape[0]), np.float32)
        self._call("asca_matmul_host", self._ctx, _p(a), _p(b), _p(c), _i64(a.shape[0]), _i64(a.shape[1]),
                   _i64(b.shape[0]), C.c_int(NT))
        return c

    # ---- Gpu::rmsnorm / rmsnorm_bwd (rust/src/cuda/mod.rs:911-939, :1122-1153)
    def rmsnorm(self, x, eps=1e-6):
        x = _as_f32(x)
        y = np.empty_like(x)
        inv = np.empty(x.shape[0], np.float32)
        self._call("asca_rmsnorm_fwd_host", self._ctx, _p(x), _p(y), _p(inv), _i64(x.shape[0]), _i64(x.shape[1]), _f(eps))
        return y, inv

    def rmsnorm_bwd(self, x, dy, eps=1e-6):
        x, dy = _as_f32(x), _as_f32(dy)
        dx = np.empty_like(x)
        self._call("asca_rmsnorm_bwd_host", self._ctx, _p(x), _p(dy), _p(dx), _i64(x.shape[0]), _i64(x.shape[1]), _f(eps))
        return dx

    # ---- Gpu::gather_rows / scatter_rows (rust/src/cuda/mod.rs:1156-1221)
    def gather_rows(self, src, idx):
        src = _as_f32(src)
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        dst = np.empty((idx.size, src.shape[1]), np.float32)
        self._call("asca_gather_rows_host", self._ctx, _p(src), _i64(src.shape[0]), _p(idx), _i64(idx.size),
                   _i64(src.shape[1]), _p(dst))
        return dst

    def scatter_rows(self, src, idx, dst):
        src = _as_f32(src)
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        assert dst.dtype == np.float32 and dst.flags.c_contiguous
        self._call("asca_scatter_rows_host", self._ctx, _p(src), _p(idx), _i64(idx.size), _i64(src.shape[1]), _p(dst),
                   _i64(dst.shape[0]))

    # ---- Gpu::adamw_update (rust/src/cuda/mod.rs:1057-1120), CPU-path decay
    def adamw_update(self, val, grad, m, v, lr, beta1, beta2, eps_t, wd):
        for a in (val, grad, m, v):
            assert a.dtype == np.float32 and a.flags.c_contiguous
        self._call("asca_adamw_host", self._ctx, _p(val), _p(grad), _p(m), _p(v), _i64(val.size), _f(lr), _f(beta1),
                   _f(beta2), _f(eps_t), _f(wd))

    # ---- Gpu::delta_scan / delta_bwd_dev (rust/src/cuda/mod.rs:1253-1382)
    def delta_scan(self, q, k, v, alpha, beta, batch, seq, n_heads, dh, keep=True, out=None):
        q, k, v, alpha, beta = map(_as_f32, (q, k, v, alpha, beta))
        assert q.shape == (batch * seq, n_heads * dh), "delta_scan: q rows must be batch*seq"
        o = np.empty_like(q) if out is None else out
        h = C.c_void_p()
        self._call("asca_delta_scan_host", self._ctx, _p(q), _p(k), _p(v), _p(alpha), _p(beta), _i64(batch), _i64(seq),
                   _i64(n_heads), _i64(dh), _p(o), C.byref(h) if keep else None)
        return o, (DeltaDev(self, h, batch, seq, n_heads, dh) if keep else None)

    def delta_bwd_dev(self, dev: DeltaDev, d_o, qnorm, knorm, out=None):
        d_o, qnorm, knorm = map(_as_f32, (d_o, qnorm, knorm))
        n, d = dev.batch * dev.seq, dev.n_heads * dev.dh
        assert d_o.shape == (n, d)
        d_qkv, d_gate = out if out is not None else (np.empty((n, 3 * d), np.float32),
                                                     np.empty((n, 2 * dev.n_heads), np.float32))
        self._call("asca_delta_bwd_dev_host", self._ctx, dev._h, _p(d_o), _p(qnorm), _p(knorm), _p(d_qkv), _p(d_gate))
        return d_qkv, d_gate

    # ---- hash-MoE: dispatch + Gpu::moe_forward_dev / moe_bwd_dev (rust/src/cuda/mod.rs:523-824)
    def moe_dispatch(self, ids, n_experts):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        perm = np.empty(ids.size, np.int32)
        offsets = np.empty(n_experts + 1, np.int32)
        route = np.empty(ids.size, np.int32)
        self._call("asca_moe_dispatch_host", self._ctx, _p(ids), _i64(ids.size), _i64(n_experts), _p(perm), _p(offsets),
                   _p(route))
        return perm, offsets, route

    def moe_forward_dev(self, xn, w1, b1, w2, b2, ids, d_ff, keep=True):
        """`ids` stands where the reference passes host-built `buckets`: the same buckets are
        rebuilt on the device by the counting-sort dispatch."""
        xn, w1, b1, w2, b2 = map(_as_f32, (xn, w1, b1, w2, b2))
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        n, d = xn.shape
        e = w1.shape[1] // d_ff
        out = np.empty((n, d), np.float32)
        h = C.c_void_p()
        self._call("asca_moe_forward_dev_host", self._ctx, _p(xn), _p(w1), _p(b1), _p(w2), _p(b2), _p(ids), _i64(n),
                   _i64(d), _i64(d_ff), _i64(e), _p(out), C.byref(h) if keep else None)
        return out, (MoeDev(self, h, n, d, d_ff, e) if keep else None)

    def moe_bwd_dev(self, dev: MoeDev, dout):
        dout = _as_f32(dout)
        n, d, f, e = dev.t_len, dev.d, dev.d_ff, dev.n_experts
        r = MoeBwd(np.empty((d, e * f), np.float32), np.empty(e * f, np.float32), np.empty((e * f, d), np.float32),
                   np.empty(d, np.float32), np.empty((n, d), np.float32))
        self._call("asca_moe_bwd_dev_host", self._ctx, dev._h, _p(dout), _p(r.d_w1), _p(r.d_b1), _p(r.d_w2), _p(r.d_b2),
                   _p(r.dxn))
        return r


    def moe_forward_dev_buckets(self, xn, w1, b1, w2, b2, buckets, d_ff, keep=True):
        """Gpu::moe_forward_dev with the reference's own argument list (rust/src/cuda/mod.rs:523-532): `buckets` is
        the host-built list of per-expert token-index lists; nothing is sorted on the device."""
        xn, w1, b1, w2, b2 = map(_as_f32, (xn, w1, b1, w2, b2))
        n, d = xn.shape
        e = len(buckets)
        idx = np.ascontiguousarray(np.concatenate([np.asarray(b, np.int32) for b in buckets]), dtype=np.int32)
        off = np.concatenate([[0], np.cumsum([len(b) for b in buckets])]).astype(np.int32)
        out = np.empty((n, d), np.float32)
        h = C.c_void_p()
        self._call("asca_moe_forward_dev_buckets_host", self._ctx, _p(xn), _p(w1), _p(b1), _p(w2), _p(b2), _p(idx), _p(off),
                   _i64(n), _i64(d), _i64(d_ff), _i64(e), _p(out), C.byref(h) if keep else None)
        return out, (MoeDev(self, h, n, d, d_ff, e) if keep else None)

    # ---- head / loss / resident AdamW (rust/src/cuda/mod.rs:828-1055, :1224-1250)
    def head_forward_dev(self, h_final, head):
        h_final, head = _as_f32(h_final), _as_f32(head)
        assert h_final.shape[1] == head.shape[0], "head_forward_dev: head dimension does not match"
        h = C.c_void_p()
        self._call("asca_head_forward_dev_host", self._ctx, _p(h_final), _p(head), _i64(h_final.shape[0]), _i64(h_final.shape[1]),
                   _i64(head.shape[1]), C.byref(h))
        return LogitsDev(self, h, h_final.shape[0], head.shape[1])

    def head_bwd_dev(self, dev, targets, head_t):
        """(loss, d_head (d, V), dh (T, d)); head_t is the head transposed, (V, d), as the reference passes it."""
        head_t = _as_f32(head_t)
        targets = np.ascontiguousarray(targets, dtype=np.uint32)
        assert targets.size == dev.t_len and head_t.shape[0] == dev.vocab
        d = head_t.shape[1]
        loss = C.c_float()
        d_head, dh = np.empty((d, dev.vocab), np.float32), np.empty((dev.t_len, d), np.float32)
        self._call("asca_head_bwd_dev_host", self._ctx, dev._h, _p(targets), _p(head_t), C.byref(loss), _p(d_head), _p(dh))
        return float(loss.value), d_head, dh

    def cross_entropy_bwd(self, logits, targets):
        logits = _as_f32(logits)
        targets = np.ascontiguousarray(targets, dtype=np.uint32)
        assert logits.shape[0] == targets.size
        loss, dl = C.c_float(), np.empty_like(logits)
        self._call("asca_cross_entropy_bwd_host", self._ctx, _p(logits), _p(targets), _i64(logits.shape[0]), _i64(logits.shape[1]),
                   C.byref(loss), _p(dl))
        return float(loss.value), dl

    def adamw_resident(self, key, val, grad, m0, v0, lr, beta1, beta2, eps_t, wd):
        """`key` = (host address of the caller's m buffer, length), as param_key builds it."""
        for a in (val, grad, m0, v0):
            assert a.dtype == np.float32 and a.flags.c_contiguous
        assert key[1] == val.size
        self._call("asca_adamw_resident_host", self._ctx, C.c_void_p(key[0]), _p(val), _p(grad), _p(m0), _p(v0), _i64(val.size),
                   _f(lr), _f(beta1), _f(beta2), _f(eps_t), _f(wd))

    def param_moments(self, key):
        m, v = np.empty(key[1], np.float32), np.empty(key[1], np.float32)
        rc = self.lib.asca_param_moments_host(self._ctx, C.c_void_p(key[0]), _i64(key[1]), _p(m), _p(v))
        if rc == 1:
            return None
        if rc != 0:
            raise AscaError(rc, self.lib.asca_last_error(self._ctx).decode())
        return m, v

    def reset_param_cache(self):
        self._call("asca_reset_param_cache", self._ctx)

    def silu_inplace(self, x):
        assert x.dtype == np.float32 and x.flags.c_contiguous
        self._call("asca_silu_inplace_host", self._ctx, _p(x), _i64(x.size))


def param_key(m: np.ndarray):
    """Cache key of one parameter's moments (rust/src/cuda/mod.rs:57-59): host address and length of its m buffer."""
    return (m.ctypes.data, m.size)


class LogitsDev:
    """Logits and h_final resident on the device between head_forward_dev and head_bwd_dev
    (the reference's LogitsDev, rust/src/cuda/mod.rs:1400-1413)."""

    def __init__(self, gpu, handle, t_len, vocab):
        self._gpu, self._h, self.t_len, self.vocab = gpu, handle, t_len, vocab

    def download(self):
        out = np.empty((self.t_len, self.vocab), np.float32)
        self._gpu._call("asca_logits_dev_download", self._gpu._ctx, self._h, _p(out))
        return out

    def free(self):
        if self._h is not None:
            self._gpu._call("asca_logits_dev_free", self._gpu._ctx, self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Model:
    """Device-resident ASCA model on one flat f32 parameter buffer (reference parameter order,
    rust/src/model.rs:593-609): forward + backward + AdamW and the per-token decode step."""

    def __init__(self, gpu: Gpu, vocab, d, H, L, E, F):
        self.gpu, self.cfg = gpu, (vocab, d, H, L, E, F)
        h = C.c_void_p()
        gpu._call("asca_model_create", gpu._ctx, *[_i64(v) for v in self.cfg], C.byref(h))
        self._h = h
        gpu.lib.asca_model_num_params.restype = C.c_int64
        self.n = int(gpu.lib.asca_model_num_params(h))

    def set_compute(self, dtype):
        """F32 (default) or BF16: tensor-core products on a bf16 copy of the weights, f32 everything else."""
        self.gpu._call("asca_model_set_compute", self.gpu._ctx, self._h, C.c_int(dtype))

    def set_fused_head(self, on: bool):
        """bf16 mode, vocabulary 256: cross-entropy taken in the head product's epilogue where it can be."""
        self.gpu._call("asca_model_set_fused_head", self._h, C.c_int(1 if on else 0))

    def set_fused_qkv(self, on: bool):
        """bf16 mode: q/k normalisation and the bf16 q, k, v written by the qkv product's epilogue where it can."""
        self.gpu._call("asca_model_set_fused_qkv", self._h, C.c_int(1 if on else 0))

    def set_grad_scale(self, scale: float):
        """Scale of dLoss/dlogits (1 / micro-batches when gradients are accumulated over several calls)."""
        self.gpu._call("asca_model_set_grad_scale", self._h, _f(scale))

    def set_grad_hook(self, fn):
        """fn(offset, count) is called from inside forward_backward each time the kernels writing
        grads[offset:offset+count] have all been enqueued (one block at a time, last block first, then
        embedding + head). None removes the hook."""
        if fn is None:
            self._hook = None
            self.gpu._call("asca_model_set_grad_hook", self._h, None, None)
            return
        proto = C.CFUNCTYPE(None, C.c_void_p, C.c_int64, C.c_int64)
        self._hook = proto(lambda _user, off, cnt: fn(int(off), int(cnt)))   # kept alive with the model
        self.gpu._call("asca_model_set_grad_hook", self._h, self._hook, None)

    def adam_counter(self, value=None) -> int:
        """Read (and optionally set) AdamW's per-tensor step counter."""
        got = C.c_uint32()
        setp = C.byref(C.c_uint32(int(value))) if value is not None else None
        self.gpu._call("asca_model_adam_counter", self._h, setp, C.byref(got))
        return int(got.value)

    def moments(self):
        """Host copies of Adam's m and v."""
        m, v = np.empty(self.n, np.float32), np.empty(self.n, np.float32)
        b = self.buffers()
        self.gpu._call("asca_memcpy_d2h", self.gpu._ctx, _p(m), C.c_void_p(b[2]), C.c_size_t(self.n * 4))
        self.gpu._call("asca_memcpy_d2h", self.gpu._ctx, _p(v), C.c_void_p(b[3]), C.c_size_t(self.n * 4))
        return m, v

    def set_moments(self, m, v):
        m, v = _as_f32(m), _as_f32(v)
        assert m.size == self.n and v.size == self.n
        b = self.buffers()
        self.gpu._call("asca_memcpy_h2d", self.gpu._ctx, C.c_void_p(b[2]), _p(m), C.c_size_t(self.n * 4))
        self.gpu._call("asca_memcpy_h2d", self.gpu._ctx, C.c_void_p(b[3]), _p(v), C.c_size_t(self.n * 4))

    def params_changed(self):
        """Tell the model that the flat parameter buffer was written through :meth:`buffers`."""
        self.gpu._call("asca_model_params_changed", self._h)

    def set_params(self, params):
        params = _as_f32(params)
        assert params.size == self.n
        self.gpu._call("asca_model_set_params_host", self.gpu._ctx, self._h, _p(params))

    def get(self):
        p, g = np.empty(self.n, np.float32), np.empty(self.n, np.float32)
        self.gpu._call("asca_model_get_host", self.gpu._ctx, self._h, _p(p), _p(g))
        return p, g

    def zero_grads(self):
        self.gpu._call("asca_model_zero_grads", self.gpu._ctx, self._h)

    def buffers(self):
        """Device addresses (ints) of the flat params, grads, Adam m and Adam v buffers."""
        ptrs = [C.c_void_p() for _ in range(4)]
        self.gpu._call("asca_model_buffers", self._h, *[C.byref(x) for x in ptrs])
        return [x.value for x in ptrs]

    def set_grads(self, grads):
        grads = _as_f32(grads)
        assert grads.size == self.n
        self.gpu._call("asca_memcpy_h2d", self.gpu._ctx, C.c_void_p(self.buffers()[1]), _p(grads), C.c_size_t(self.n * 4))

    def forward_backward(self, ids, targets, batch, want_logits=False):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        targets = np.ascontiguousarray(targets, dtype=np.uint32)
        n = ids.size
        loss = C.c_float()
        logits = np.empty((n, self.cfg[0]), np.float32) if want_logits else None
        self.gpu._call("asca_model_forward_backward_host", self.gpu._ctx, self._h, _p(ids), _p(targets), _i64(batch),
                       _i64(n // batch), C.byref(loss), _p(logits))
        return (loss.value, logits) if want_logits else loss.value

    def adamw_step(self, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.01):
        self.gpu._call("asca_model_adamw_step", self.gpu._ctx, self._h, _f(lr), _f(beta1), _f(beta2), _f(eps), _f(wd))

    def adamw_slices(self, lr, slices, advance=True, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.01):
        """One optimizer step restricted to the sorted, disjoint (lo, hi) slices of the flat buffer (bf16 mode)."""
        lo = np.ascontiguousarray([s[0] for s in slices], dtype=np.int64)
        hi = np.ascontiguousarray([s[1] for s in slices], dtype=np.int64)
        self.gpu._call("asca_model_adamw_slices", self.gpu._ctx, self._h, _f(lr), _f(beta1), _f(beta2), _f(eps), _f(wd), _p(lo), _p(hi),
                       C.c_int(len(slices)), C.c_int(1 if advance else 0))

    def params16(self):
        """(device address, element count) of the bf16 weight copy."""
        ptr, n16 = C.c_void_p(), C.c_int64()
        self.gpu._call("asca_model_params16", self.gpu._ctx, self._h, C.byref(ptr), C.byref(n16))
        return ptr.value, int(n16.value)

    def new_decode_state(self, n_streams):
        import torch

        _, d, H, L, _, _ = self.cfg
        dh = d // H
        return torch.zeros((L, n_streams, H, dh, dh), dtype=torch.float32, device=f"cuda:{self.gpu.device}")

    def decode_step(self, state, ids, want_logits=True):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        ns = ids.size
        logits = np.empty((ns, self.cfg[0]), np.float32) if want_logits else None
        nxt = np.empty(ns, np.uint32)
        self.gpu._call("asca_model_decode_step_host", self.gpu._ctx, self._h, _p(state), _p(ids), _i64(ns), _p(logits),
                       _p(nxt))
        return logits, nxt

    def prefill(self, state, ids, want_logits=True):
        """Chunked prefill of ids (n_streams, T): the recurrent state after the last token lands in `state` (whose
        incoming contents are the initial state); returns (logits of each stream's last token or None, their argmax)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        ns, t = ids.shape
        logits = np.empty((ns, self.cfg[0]), np.float32) if want_logits else None
        nxt = np.empty(ns, np.uint32)
        self.gpu._call("asca_model_prefill_host", self.gpu._ctx, self._h, _p(state), _p(ids), _i64(ns), _i64(t), _p(logits), _p(nxt))
        return logits, nxt

    def decode_greedy(self, state, ids, n_steps):
        """n_steps greedy tokens per stream; the argmax feeds the next step on the device. Returns (n_steps, n_streams)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        toks = np.empty((int(n_steps), ids.size), np.uint32)
        self.gpu._call("asca_model_decode_greedy_host", self.gpu._ctx, self._h, _p(state), _p(ids), _i64(ids.size), _i64(n_steps),
                       _p(toks))
        return toks

    def free(self):
        if self._h is not None:
            self.gpu.lib.asca_model_destroy(self.gpu._ctx, self._h)
            self._h = None


__all__ = ["Gpu", "Model", "DeltaDev", "MoeDev", "MoeBwd", "LogitsDev", "param_key", "AscaError", "load", "LIB_PATH", "F32", "BF16", "NN", "TN", "NT"]
