"""Device-pointer entry points of libasca_b200 on torch CUDA tensors.

torch is used only to own device memory and streams; every function forwards raw pointers
to the C ABI (include/asca_b200.h) and launches the library's own kernels on the stream the
:class:`asca_b200.Gpu` context is bound to (call ``gpu.use_torch_stream()`` to share
torch's current stream).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import BF16, F32, NN, NT, TN, Gpu, _f, _i64, _p  # noqa: F401


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"unsupported dtype {t.dtype}")


def _chk(*ts):
    for t in ts:
        if t is not None:
            assert t.is_cuda and t.is_contiguous(), "expected contiguous CUDA tensors"


def gemm(gpu: Gpu, a, b, mode=NN, bias=None, out=None, accumulate=False):
    """C = op(A) op(B) (+ bias) (+ C). a, b both f32 or both bf16; C f32."""
    _chk(a, b, bias, out)
    if mode == NN:
        m, k, n = a.shape[0], a.shape[1], b.shape[1]
    elif mode == TN:
        m, k, n = a.shape[1], a.shape[0], b.shape[1]
    else:
        m, k, n = a.shape[0], a.shape[1], b.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    gpu._call("asca_gemm", gpu._ctx, C.c_int(mode), _i64(m), _i64(n), _i64(k), _p(a), _i64(a.shape[1]), _p(b),
              _i64(b.shape[1]), _p(out), _i64(n), _p(bias), C.c_int(1 if accumulate else 0), C.c_int(_dt(a)))
    return out


def rmsnorm_fwd(gpu, x, eps=1e-6, want_inv=False):
    _chk(x)
    y = torch.empty_like(x)
    inv = torch.empty(x.shape[0], dtype=torch.float32, device=x.device) if want_inv else None
    gpu._call("asca_rmsnorm_fwd", gpu._ctx, _p(x), _p(y), _p(inv), _i64(x.shape[0]), _i64(x.shape[1]), _f(eps))
    return (y, inv) if want_inv else y


def rmsnorm_bwd(gpu, x, dy, eps=1e-6):
    _chk(x, dy)
    dx = torch.empty_like(x)
    gpu._call("asca_rmsnorm_bwd", gpu._ctx, _p(x), _p(dy), _p(dx), _i64(x.shape[0]), _i64(x.shape[1]), _f(eps))
    return dx


def residual_rmsnorm(gpu, x, y, eps=1e-6, want_norm=True):
    """x_mid = x + y and (optionally) xn = rmsnorm(x_mid) in one pass."""
    _chk(x, y)
    x_mid = torch.empty_like(x)
    xn = torch.empty_like(x) if want_norm else None
    gpu._call("asca_residual_rmsnorm", gpu._ctx, _p(x), _p(y), _p(x_mid), _p(xn), _i64(x.shape[0]), _i64(x.shape[1]),
              _f(eps))
    return x_mid, xn


def gather_rows(gpu, src, idx):
    _chk(src, idx)
    dst = torch.empty((idx.numel(), src.shape[1]), dtype=torch.float32, device=src.device)
    gpu._call("asca_gather_rows", gpu._ctx, _p(src), _p(idx), _i64(idx.numel()), _i64(src.shape[1]), _p(dst))
    return dst


def scatter_rows(gpu, src, idx, dst):
    _chk(src, idx, dst)
    gpu._call("asca_scatter_rows", gpu._ctx, _p(src), _p(idx), _i64(idx.numel()), _i64(src.shape[1]), _p(dst))


def adamw(gpu, p, g, m, v, lr_t, beta1, beta2, eps_t, wd_eff):
    _chk(p, g, m, v)
    gpu._call("asca_adamw", gpu._ctx, _p(p), _p(g), _p(m), _p(v), _i64(p.numel()), _f(lr_t), _f(beta1), _f(beta2),
              _f(eps_t), _f(wd_eff))


def adamw_segmented(gpu, p, g, m, v, seg_off, lr_t, eps_t, beta1, beta2, wd_eff):
    """seg_off: int64 numpy array (n_seg+1); lr_t, eps_t: float32 numpy arrays (n_seg)."""
    import numpy as np

    _chk(p, g, m, v)
    seg_off = np.ascontiguousarray(seg_off, dtype=np.int64)
    lr_t = np.ascontiguousarray(lr_t, dtype=np.float32)
    eps_t = np.ascontiguousarray(eps_t, dtype=np.float32)
    gpu._call("asca_adamw_segmented", gpu._ctx, _p(p), _p(g), _p(m), _p(v), _p(seg_off), _p(lr_t), _p(eps_t),
              C.c_int(lr_t.size), _f(beta1), _f(beta2), _f(wd_eff))


def delta_ckpt_floats(gpu, B, T, H, dh, chunk):
    return int(gpu.lib.asca_delta_ckpt_floats(B, T, H, dh, chunk))


def delta_prep(gpu, qkv, gate, H, dh):
    _chk(qkv, gate)
    n, d = qkv.shape[0], H * dh
    f = dict(dtype=torch.float32, device=qkv.device)
    q, k, v = (torch.empty((n, d), **f) for _ in range(3))
    qn, kn, al, be = (torch.empty((n, H), **f) for _ in range(4))
    gpu._call("asca_delta_prep", gpu._ctx, _p(qkv), _p(gate), _i64(n), _i64(H), _i64(dh), _p(q), _p(k), _p(v), _p(qn),
              _p(kn), _p(al), _p(be))
    return q, k, v, qn, kn, al, be


def delta_fwd(gpu, q, k, v, alpha, beta, B, T, H, dh, chunk=64, s_init=None, want_final=False, want_ckpt=True,
              out=None, ckpt=None):
    _chk(q, k, v, alpha, beta, s_init)
    o = torch.empty_like(q) if out is None else out
    f = dict(dtype=torch.float32, device=q.device)
    s_final = torch.empty((B, H, dh, dh), **f) if want_final else None
    if want_ckpt and ckpt is None:
        ckpt = torch.empty(delta_ckpt_floats(gpu, B, T, H, dh, chunk), **f)
    gpu._call("asca_delta_fwd", gpu._ctx, _p(q), _p(k), _p(v), _p(alpha), _p(beta), _i64(B), _i64(T), _i64(H),
              _i64(dh), _i64(chunk), C.c_int(_dt(q)), _p(o), _p(s_init), _p(s_final), _p(ckpt if want_ckpt else None))
    return o, s_final, (ckpt if want_ckpt else None)


def delta_bwd(gpu, q, k, v, alpha, beta, qnorm, knorm, d_o, ckpt, B, T, H, dh, chunk=64, d_qkv=None, d_gate=None):
    _chk(q, k, v, alpha, beta, qnorm, knorm, d_o, ckpt)
    assert d_o.dtype == q.dtype
    n, d = B * T, H * dh
    f = dict(dtype=torch.float32, device=q.device)
    if d_qkv is None:
        d_qkv = torch.empty((n, 3 * d), **f)
    if d_gate is None:
        d_gate = torch.empty((n, 2 * H), **f)
    gpu._call("asca_delta_bwd", gpu._ctx, _p(q), _p(k), _p(v), _p(alpha), _p(beta), _p(qnorm), _p(knorm), _p(d_o),
              _p(ckpt), _i64(B), _i64(T), _i64(H), _i64(dh), _i64(chunk), C.c_int(_dt(q)), _p(d_qkv), _p(d_gate))
    return d_qkv, d_gate


def delta_step(gpu, q, k, v, alpha, beta, S, H, dh, fused=False, out=None):
    """In-place decode step on S (n_streams, H, dh, dh). fused: q = raw qkv (n, 3d), alpha = raw gate (n, 2H)."""
    _chk(q, k, v, alpha, beta, S)
    n = S.shape[0]
    o = torch.empty((n, H * dh), dtype=torch.float32, device=S.device) if out is None else out
    gpu._call("asca_delta_step", gpu._ctx, _p(q), _p(k), _p(v), _p(alpha), _p(beta), _p(S), _i64(n), _i64(H), _i64(dh),
              C.c_int(1 if fused else 0), _p(o))
    return o


def moe_dispatch(gpu, ids, E, want_route=False):
    _chk(ids)
    assert ids.dtype in (torch.int32, torch.uint32)
    n = ids.numel()
    perm = torch.empty(n, dtype=torch.int32, device=ids.device)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=ids.device)
    route = torch.empty(n, dtype=torch.int32, device=ids.device) if want_route else None
    gpu._call("asca_moe_dispatch", gpu._ctx, _p(ids), _i64(n), _i64(E), _p(perm), _p(offsets), _p(route))
    return (perm, offsets, route) if want_route else (perm, offsets)


def moe_fwd(gpu, xn, w1, b1, w2, b2, perm, offsets, F, E, out=None, pre_p=None, hid_p=None):
    _chk(xn, w1, b1, w2, b2, perm, offsets)
    n, d = xn.shape
    dev = xn.device
    if out is None:
        out = torch.empty((n, d), dtype=torch.float32, device=dev)
    if pre_p is None:
        pre_p = torch.empty((n, F), dtype=torch.float32, device=dev)
    if hid_p is None:
        hid_p = torch.empty((n, F), dtype=xn.dtype, device=dev)
    gpu._call("asca_moe_fwd", gpu._ctx, _p(xn), _p(w1), _p(b1), _p(w2), _p(b2), _p(perm), _p(offsets), _i64(n), _i64(d),
              _i64(F), _i64(E), C.c_int(_dt(xn)), _p(out), _p(pre_p), _p(hid_p))
    return out, pre_p, hid_p


def moe_bwd(gpu, xn, w1, w2, pre_p, hid_p, dout, perm, offsets, F, E, grads=None):
    _chk(xn, w1, w2, pre_p, hid_p, dout, perm, offsets)
    n, d = xn.shape
    f = dict(dtype=torch.float32, device=xn.device)
    if grads is None:
        grads = (torch.empty((d, E * F), **f), torch.empty(E * F, **f), torch.empty((E * F, d), **f),
                 torch.empty(d, **f), torch.empty((n, d), **f))
    d_w1, d_b1, d_w2, d_b2, dxn = grads
    gpu._call("asca_moe_bwd", gpu._ctx, _p(xn), _p(w1), _p(w2), _p(pre_p), _p(hid_p), _p(dout), _p(perm), _p(offsets),
              _i64(n), _i64(d), _i64(F), _i64(E), C.c_int(_dt(xn)), _p(d_w1), _p(d_b1), _p(d_w2), _p(d_b2), _p(dxn))
    return grads


def moe_step(gpu, x, ids, w1, b1, w2, b2, F, E):
    _chk(x, ids, w1, b1, w2, b2)
    out = torch.empty_like(x)
    gpu._call("asca_moe_step", gpu._ctx, _p(x), _p(ids), _p(w1), _p(b1), _p(w2), _p(b2), _i64(x.shape[0]),
              _i64(x.shape[1]), _i64(F), _i64(E), C.c_int(_dt(w1)), _p(out))
    return out


class DeltaHostPipeline:
    """Delta-rule forward + BPTT for sequences that live in pinned host memory.

    The op is independent per sequence, so the step is cut into one stage per sequence and the
    stages are pipelined over three streams: the host->device copy of sequence s+1, the kernels
    of sequence s and the device->host copy of sequence s-1 run at the same time (PCIe is full
    duplex). ``depth`` device slots bound the memory held: each slot has room for one
    sequence's inputs, checkpoints and outputs.

    All host tensors must be pinned; q, k, v, d_o in one dtype (f32 or bf16), the rest f32.
    """

    def __init__(self, gpu: Gpu, T, H, dh, chunk=64, dtype=torch.bfloat16, depth=3):
        self.gpu, self.T, self.H, self.dh, self.chunk, self.depth = gpu, T, H, dh, chunk, depth
        dev = torch.device("cuda", gpu.device)
        self.dev = dev
        d = H * dh
        f = dict(dtype=torch.float32, device=dev)
        a = dict(dtype=dtype, device=dev)
        self.slots = []
        for _ in range(depth):
            self.slots.append(dict(
                q=torch.empty((T, d), **a), k=torch.empty((T, d), **a), v=torch.empty((T, d), **a),
                d_o=torch.empty((T, d), **a), alpha=torch.empty((T, H), **f), beta=torch.empty((T, H), **f),
                qn=torch.empty((T, H), **f), kn=torch.empty((T, H), **f), o=torch.empty((T, d), **a),
                ckpt=torch.empty(delta_ckpt_floats(gpu, 1, T, H, dh, chunk), **f),
                d_qkv=torch.empty((T, 3 * d), **f), d_gate=torch.empty((T, 2 * H), **f),
                computed=torch.cuda.Event(), drained=torch.cuda.Event()))
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))

    def run(self, q, k, v, alpha, beta, qnorm, knorm, d_o, o, d_qkv, d_gate, B):
        """Host in, host out; returns after every result has landed in o, d_qkv, d_gate."""
        T, H, dh, gpu = self.T, self.H, self.dh, self.gpu
        for x in (q, k, v, alpha, beta, qnorm, knorm, d_o, o, d_qkv, d_gate):
            assert not x.is_cuda and x.is_pinned() and x.shape[0] == B * T, "expected pinned host tensors of B*T rows"
        for s in range(B):
            sl = self.slots[s % self.depth]
            rows = slice(s * T, (s + 1) * T)
            with torch.cuda.stream(self.s_in):
                if s >= self.depth:
                    self.s_in.wait_event(sl["computed"])      # the slot's inputs have been consumed
                for name, src in (("q", q), ("k", k), ("v", v), ("alpha", alpha), ("beta", beta), ("qn", qnorm),
                                  ("kn", knorm), ("d_o", d_o)):
                    sl[name].copy_(src[rows], non_blocking=True)
                loaded = self.s_in.record_event()
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(loaded)
                if s >= self.depth:
                    self.s_run.wait_event(sl["drained"])      # the slot's outputs have been copied out
                gpu.use_torch_stream()
                delta_fwd(gpu, sl["q"], sl["k"], sl["v"], sl["alpha"], sl["beta"], 1, T, H, dh, chunk=self.chunk,
                          out=sl["o"], ckpt=sl["ckpt"])
                delta_bwd(gpu, sl["q"], sl["k"], sl["v"], sl["alpha"], sl["beta"], sl["qn"], sl["kn"], sl["d_o"],
                          sl["ckpt"], 1, T, H, dh, chunk=self.chunk, d_qkv=sl["d_qkv"], d_gate=sl["d_gate"])
                sl["computed"].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(sl["computed"])
                o[rows].copy_(sl["o"], non_blocking=True)
                d_qkv[rows].copy_(sl["d_qkv"], non_blocking=True)
                d_gate[rows].copy_(sl["d_gate"], non_blocking=True)
                sl["drained"].record(self.s_out)
        self.s_out.synchronize()
        self.s_run.synchronize()
        gpu.use_torch_stream()   # back on the caller's stream
