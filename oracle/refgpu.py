"""ctypes front-end to oracle/_ref/libasca_ref.so: the reference's own CUDA kernels behind host
launchers (oracle/ref_kernels.cu). TEST INFRASTRUCTURE ONLY -- used to pin the CPU oracle
against outputs of the reference's own code on a GPU."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

SO = Path(__file__).resolve().parent / "_ref" / "libasca_ref.so"
_lib = None


def available() -> bool:
    return SO.exists()


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(SO))
    return _lib


def _f(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _ok(rc, what):
    if rc != 0:
        raise RuntimeError(f"reference kernel {what} failed with CUDA error {rc}")


def matmul(a, b):
    c = np.empty((a.shape[0], b.shape[1]), np.float32)
    _ok(lib().ref_matmul(_f(a), _f(b), _f(c), a.shape[0], a.shape[1], b.shape[1]), "matmul_f32")
    return c


def matmul_ta(a, b):
    c = np.empty((a.shape[1], b.shape[1]), np.float32)
    _ok(lib().ref_matmul_ta(_f(a), _f(b), _f(c), a.shape[1], a.shape[0], b.shape[1]), "matmul_ta_f32")
    return c


def rmsnorm(x, eps=1e-6):
    y, inv = np.empty_like(x), np.empty(x.shape[0], np.float32)
    _ok(lib().ref_rmsnorm(_f(x), _f(y), _f(inv), x.shape[0], x.shape[1], C.c_float(eps)), "rmsnorm_f32")
    return y, inv


def rmsnorm_bwd(x, dy, eps=1e-6):
    dx = np.empty_like(x)
    _ok(lib().ref_rmsnorm_bwd(_f(x), _f(dy), _f(dx), x.shape[0], x.shape[1], C.c_float(eps)), "rmsnorm_bwd_f32")
    return dx


def delta_scan(q, k, v, alpha, beta, B, T, H, dh):
    o = np.empty_like(q)
    states = np.empty((H, B, T + 1, dh, dh), np.float32)
    _ok(lib().ref_delta_scan(_f(q), _f(k), _f(v), _f(alpha), _f(beta), B, T, H, dh, _f(o), _f(states)),
        "delta_fwd_batch_f32")
    return o, states


def delta_fwd_bwd(q, k, v, alpha, beta, qn, kn, d_o, B, T, H, dh):
    n, d = B * T, H * dh
    o = np.empty_like(q)
    d_qkv, d_gate = np.empty((n, 3 * d), np.float32), np.empty((n, 2 * H), np.float32)
    _ok(lib().ref_delta_fwd_bwd(_f(q), _f(k), _f(v), _f(alpha), _f(beta), _f(qn), _f(kn), _f(d_o), B, T, H, dh,
                                _f(o), _f(d_qkv), _f(d_gate)), "delta_fwd_batch_f32 + delta_bwd_f32")
    return o, d_qkv, d_gate


def silu(pre):
    h = np.empty_like(pre)
    _ok(lib().ref_silu(_f(pre), _f(h), pre.size), "silu_out_f32")
    return h


def silu_bwd(dpre, pre):
    g = dpre.copy()
    _ok(lib().ref_silu_bwd(_f(g), _f(pre), pre.size), "silu_bwd_f32")
    return g


def cross_entropy(logits, targets):
    t, v = logits.shape
    dl, ls = np.empty_like(logits), np.empty(t, np.float32)
    tg = np.ascontiguousarray(targets, dtype=np.uint32)
    _ok(lib().ref_cross_entropy(_f(logits), tg.ctypes.data_as(C.POINTER(C.c_uint32)), _f(dl), _f(ls), t, v),
        "cross_entropy_bwd_f32")
    return ls, dl


def _i(a):
    assert a.dtype == np.int32 and a.flags.c_contiguous
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def moe_forward_backward(xn, w1, b1, w2, b2, buckets, dout, F):
    """The reference's moe_forward_dev + moe_bwd_dev launch sequence on host-built buckets (a list of index arrays,
    one per expert). Returns out, pre, hid (token order), d_w1, d_b1, d_w2, d_b2, dxn."""
    t, d = xn.shape
    e = len(buckets)
    idx = np.ascontiguousarray(np.concatenate([np.asarray(b, np.int32) for b in buckets]) if t else np.zeros(0, np.int32))
    off = np.concatenate([[0], np.cumsum([len(b) for b in buckets])]).astype(np.int32)
    out, dxn = np.empty((t, d), np.float32), np.empty((t, d), np.float32)
    pre, hid = np.empty((t, F), np.float32), np.empty((t, F), np.float32)
    d_w1, d_w2 = np.empty_like(w1), np.empty_like(w2)
    d_b1, d_b2 = np.empty(e * F, np.float32), np.empty(d, np.float32)
    _ok(lib().ref_moe_fwd_bwd(_f(xn), _f(w1), _f(b1), _f(w2), _f(b2), _i(idx), _i(off), _f(dout), t, d, F, e, _f(out), _f(pre),
                              _f(hid), _f(d_w1), _f(d_b1), _f(d_w2), _f(d_b2), _f(dxn)), "moe forward + backward sequence")
    return out, pre, hid, d_w1, d_b1, d_w2, d_b2, dxn


def gather_rows(src, idx):
    idx = np.ascontiguousarray(idx, np.int32)
    dst = np.empty((idx.size, src.shape[1]), np.float32)
    _ok(lib().ref_gather_rows(_f(src), src.shape[0], _i(idx), idx.size, src.shape[1], _f(dst)), "gather_rows_f32")
    return dst


def scatter_rows(src, idx, dst):
    idx = np.ascontiguousarray(idx, np.int32)
    _ok(lib().ref_scatter_rows(_f(src), _i(idx), idx.size, src.shape[1], _f(dst), dst.shape[0]), "scatter_rows_f32")
    return dst


def adamw(val, grad, m, v, lr_t, beta1, beta2, eps_t, wd):
    """In place on val, m, v (copies of the caller's arrays are the caller's business)."""
    _ok(lib().ref_adamw(_f(val), _f(grad), _f(m), _f(v), val.size, C.c_float(lr_t), C.c_float(beta1), C.c_float(beta2),
                        C.c_float(eps_t), C.c_float(wd)), "adamw_f32")
