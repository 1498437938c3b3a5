"""CPU oracle for the Delta Memory / hash-MoE hot path (TEST INFRASTRUCTURE ONLY).

A ctypes front-end to ``asca_oracle.cpp``, the C++ restatement of the reference's f32 CPU
path. Only the tests, the smoke check and the benchmark's CPU-baseline leg import this
package; the CUDA library and the ``asca_b200`` package never do.

The reference has no golden vectors for this path and its Rust crate cannot be built where
this runs. The oracle is pinned on a GPU against the reference's own CUDA kernels
(``oracle/build_ref.py``, ``tests/test_reference_pin.py``) and by the reference's own
self-consistency gates restated in ``tests/test_oracle_gates.py``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_SO = _DIR / "libasca_oracle.so"
_SRC = _DIR / "asca_oracle.cpp"
# -mavx2 -mfma rather than -march=native: the library is built on one host and run on another.
_FLAGS = ["-O3", "-mavx2", "-mfma", "-ffp-contract=off", "-std=c++17", "-fPIC", "-shared", "-pthread"]


def build(force: bool = False) -> Path:
    """Compile the oracle into ``oracle/libasca_oracle.so`` (skipped when up to date)."""
    if not force and _SO.exists() and _SO.stat().st_mtime >= _SRC.stat().st_mtime:
        return _SO
    subprocess.check_call(["g++", *_FLAGS, "-o", str(_SO), str(_SRC)])
    return _SO


_lib = None

f32p = C.POINTER(C.c_float)
u32p = C.POINTER(C.c_uint32)
i32p = C.POINTER(C.c_int32)
u64p = C.POINTER(C.c_uint64)
sz = C.c_size_t


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _SO.exists():
            if _SRC.exists() and os.access(_DIR, os.W_OK):
                build()
            else:
                raise RuntimeError(f"{_SO} is missing; run oracle.build()")
        _lib = C.CDLL(str(_SO))
        _lib.orc_model_num_params.restype = sz
        _lib.orc_model_num_params.argtypes = [sz] * 6
        _lib.orc_model_num_tensors.restype = sz
        _lib.orc_model_num_tensors.argtypes = [sz]
        _lib.orc_hash_route.restype = C.c_uint32
        _lib.orc_hash_route.argtypes = [C.c_uint32, C.c_uint32]
        _lib.orc_model_forward_backward.restype = C.c_float
        _lib.orc_model_loss.restype = C.c_float
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_delta_block_forward.restype = C.c_void_p
    return _lib


def _f(a):
    assert a is None or (a.dtype == np.float32 and a.flags.c_contiguous), "need contiguous f32"
    return None if a is None else a.ctypes.data_as(f32p)


def _u(a):
    assert a.dtype == np.uint32 and a.flags.c_contiguous
    return a.ctypes.data_as(u32p)


def _i(a):
    assert a is None or (a.dtype == np.int32 and a.flags.c_contiguous)
    return None if a is None else a.ctypes.data_as(i32p)


def set_threads(n: int) -> None:
    lib().orc_set_threads(C.c_int(n))


def num_threads() -> int:
    return int(lib().orc_num_threads())


class Rng:
    """The reference's xorshift128+ / Box-Muller generator (rust/src/tensor.rs:299-337)."""

    def __init__(self, seed: int):
        self.state = np.zeros(2, dtype=np.uint64)
        lib().orc_rng_new(C.c_uint64(seed), self.state.ctypes.data_as(u64p))

    def _s(self):
        return self.state.ctypes.data_as(u64p)

    def normal(self, shape, scale: float = 1.0) -> np.ndarray:
        out = np.empty(shape, dtype=np.float32)
        lib().orc_rng_normal(self._s(), C.c_float(scale), _f(out), sz(out.size))
        return out

    def uniform(self, shape) -> np.ndarray:
        out = np.empty(shape, dtype=np.float32)
        lib().orc_rng_uniform(self._s(), _f(out), sz(out.size))
        return out

    def below(self, n: int, shape) -> np.ndarray:
        out = np.empty(shape, dtype=np.uint32)
        lib().orc_rng_below(self._s(), C.c_uint64(n), _u(out), sz(out.size))
        return out


# ------------------------------------------------------------------ tensor engine
def matmul(a, b):
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float32)
    lib().orc_matmul(_f(a), _f(b), _f(c), sz(m), sz(k), sz(n))
    return c


def matmul_ta(a, b):
    k, m = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float32)
    lib().orc_matmul_ta(_f(a), _f(b), _f(c), sz(k), sz(m), sz(n))
    return c


def matmul_t(a, b):
    m, k = a.shape
    n = b.shape[0]
    c = np.empty((m, n), np.float32)
    lib().orc_matmul_t(_f(a), _f(b), _f(c), sz(m), sz(k), sz(n))
    return c


def rmsnorm(x, eps=1e-6):
    y = np.empty_like(x)
    inv = np.empty(x.shape[0], np.float32)
    lib().orc_rmsnorm_fwd(_f(x), _f(y), _f(inv), sz(x.shape[0]), sz(x.shape[1]), C.c_float(eps))
    return y, inv


def rmsnorm_bwd(x, dy, eps=1e-6):
    dx = np.empty_like(x)
    lib().orc_rmsnorm_bwd(_f(x), _f(dy), _f(dx), sz(x.shape[0]), sz(x.shape[1]), C.c_float(eps))
    return dx


def adamw_scalars(lr, b1, b2, eps, wd, t):
    a, b, c = C.c_float(), C.c_float(), C.c_float()
    lib().orc_adamw_scalars(C.c_float(lr), C.c_float(b1), C.c_float(b2), C.c_float(eps), C.c_float(wd),
                            C.c_uint32(t), C.byref(a), C.byref(b), C.byref(c))
    return a.value, b.value, c.value


def adamw_apply(p, g, m, v, lr_t, b1, b2, eps_t, wd_eff):
    lib().orc_adamw_apply(_f(p), _f(g), _f(m), _f(v), sz(p.size), C.c_float(lr_t), C.c_float(b1),
                          C.c_float(b2), C.c_float(eps_t), C.c_float(wd_eff))


# ------------------------------------------------------------------ routing
def hash_route(i: int, n_experts: int) -> int:
    return int(lib().orc_hash_route(C.c_uint32(i), C.c_uint32(n_experts)))


def moe_dispatch(ids, n_experts):
    n = ids.size
    perm = np.empty(n, np.int32)
    offsets = np.empty(n_experts + 1, np.int32)
    route = np.empty(n, np.int32)
    lib().orc_moe_dispatch(_u(ids), sz(n), sz(n_experts), _i(perm), _i(offsets), _i(route))
    return perm, offsets, route


# ------------------------------------------------------------------ delta rule
def delta_scan(q, k, v, alpha, beta, B, T, H, dh, want_states=False, per_chain_threads=True):
    o = np.zeros_like(q)
    states = np.zeros((H, B, T + 1, dh, dh), np.float32) if want_states else None
    s_final = np.zeros((B, H, dh, dh), np.float32)
    lib().orc_delta_scan(_f(q), _f(k), _f(v), _f(alpha), _f(beta), sz(B), sz(T), sz(H), sz(dh), _f(o),
                         _f(states), _f(s_final), C.c_int(1 if per_chain_threads else 0))
    return (o, s_final, states) if want_states else (o, s_final)


def delta_scan_scalar(q, k, v, alpha, beta, B, T, H, dh):
    o = np.zeros_like(q)
    lib().orc_delta_scan_scalar(_f(q), _f(k), _f(v), _f(alpha), _f(beta), sz(B), sz(T), sz(H), sz(dh), _f(o))
    return o


def delta_bptt(q, k, v, alpha, beta, qn, kn, d_o, B, T, H, dh, max_workers=None):
    n, d = B * T, H * dh
    d_qkv = np.zeros((n, 3 * d), np.float32)
    d_gate = np.zeros((n, 2 * H), np.float32)
    mw = num_threads() if max_workers is None else max_workers
    lib().orc_delta_bptt(_f(q), _f(k), _f(v), _f(alpha), _f(beta), _f(qn), _f(kn), _f(d_o), sz(B), sz(T),
                         sz(H), sz(dh), _f(d_qkv), _f(d_gate), C.c_int(mw))
    return d_qkv, d_gate


def delta_step_core(q, k, v, alpha, beta, S, H, dh):
    """In-place state update for n_streams independent streams; returns o."""
    ns = q.shape[0]
    o = np.zeros_like(q)
    lib().orc_delta_step_core(_f(q), _f(k), _f(v), _f(alpha), _f(beta), _f(S), sz(ns), sz(H), sz(dh), _f(o))
    return o


class DeltaBlock:
    """The reference's DeltaBlock on six separate parameter arrays (rust/src/delta.rs)."""

    NAMES = ("w_qkv", "b_qkv", "w_gate", "b_gate", "w_o", "b_o")

    def __init__(self, d, H, rng: Rng):
        self.d, self.H = d, H
        s = np.float32(np.sqrt(np.float32(1.0) / np.float32(d)))
        self.w_qkv = rng.normal((d, 3 * d), s)
        self.w_gate = rng.normal((d, 2 * H), s)
        self.w_o = rng.normal((d, d), s)
        self.b_qkv = np.zeros(3 * d, np.float32)
        self.b_gate = np.concatenate([np.full(H, -2.0), np.full(H, -1.0)]).astype(np.float32)
        self.b_o = np.zeros(d, np.float32)

    def params(self):
        return [getattr(self, n) for n in self.NAMES]

    def forward(self, x, batch):
        n = x.shape[0]
        y = np.empty((n, self.d), np.float32)
        h = lib().orc_delta_block_forward(*[_f(p) for p in self.params()], _f(x), sz(n), sz(batch),
                                          sz(self.d), sz(self.H), _f(y))
        return y, C.c_void_p(h)

    def cache_get(self, cache, n):
        d, H = self.d, self.H
        out = {k: np.empty((n, d), np.float32) for k in ("q", "k", "v", "o")}
        out.update({k: np.empty((n, H), np.float32) for k in ("alpha", "beta", "qn", "kn")})
        lib().orc_delta_cache_get(cache, _f(out["q"]), _f(out["k"]), _f(out["v"]), _f(out["alpha"]),
                                  _f(out["beta"]), _f(out["qn"]), _f(out["kn"]), _f(out["o"]))
        return out

    def backward(self, cache, dy):
        n = dy.shape[0]
        grads = [np.zeros_like(p) for p in self.params()]
        dx = np.empty((n, self.d), np.float32)
        lib().orc_delta_block_backward(cache, _f(self.w_qkv), _f(self.w_gate), _f(self.w_o), _f(dy), sz(n),
                                       sz(self.d), sz(self.H), *[_f(g) for g in grads], _f(dx))
        return dx, dict(zip(self.NAMES, grads))

    def free(self, cache):
        lib().orc_delta_cache_free(cache)

    def step(self, x, states):
        y = np.empty((1, self.d), np.float32)
        lib().orc_delta_block_step(*[_f(p) for p in self.params()], _f(x), sz(self.d), sz(self.H),
                                   _f(states), _f(y))
        return y


# ------------------------------------------------------------------ hash MoE
def moe_ffn_forward(xn, w1, b1, w2, b2, ids, F, E, want_cache=False):
    n, d = xn.shape
    out = np.empty((n, d), np.float32)
    pre = np.zeros((n, F), np.float32) if want_cache else None
    hid = np.zeros((n, F), np.float32) if want_cache else None
    lib().orc_moe_ffn_forward(_f(xn), _f(w1), _f(b1), _f(w2), _f(b2), _u(ids), sz(n), sz(d), sz(F), sz(E),
                              _f(out), _f(pre), _f(hid))
    return (out, pre, hid) if want_cache else out


def moe_ffn_backward(xn, w1, w2, pre, hid, ids, dout, F, E):
    n, d = xn.shape
    d_w1 = np.zeros_like(w1)
    d_b1 = np.zeros(E * F, np.float32)
    d_w2 = np.zeros_like(w2)
    d_b2 = np.zeros(d, np.float32)
    dxn = np.empty((n, d), np.float32)
    lib().orc_moe_ffn_backward(_f(xn), _f(w1), _f(w2), _f(pre), _f(hid), _u(ids), _f(dout), sz(n), sz(d),
                               sz(F), sz(E), _f(d_w1), _f(d_b1), _f(d_w2), _f(d_b2), _f(dxn))
    return d_w1, d_b1, d_w2, d_b2, dxn


def moe_forward_backward(x, w1, b1, w2, b2, ids, dout, F, E):
    n, d = x.shape
    out = np.empty((n, d), np.float32)
    d_w1 = np.zeros_like(w1)
    d_b1 = np.zeros(E * F, np.float32)
    d_w2 = np.zeros_like(w2)
    d_b2 = np.zeros(d, np.float32)
    dx = np.empty((n, d), np.float32)
    lib().orc_moe_forward_backward(_f(x), _f(w1), _f(b1), _f(w2), _f(b2), _u(ids), _f(dout), sz(n), sz(d),
                                   sz(F), sz(E), _f(out), _f(d_w1), _f(d_b1), _f(d_w2), _f(d_b2), _f(dx))
    return out, d_w1, d_b1, d_w2, d_b2, dx


def moe_step(x, w1, b1, w2, b2, tok, F, E):
    d = x.shape[-1]
    out = np.empty((1, d), np.float32)
    lib().orc_moe_step(_f(x), _f(w1), _f(b1), _f(w2), _f(b2), C.c_uint32(tok), sz(d), sz(F), sz(E), _f(out))
    return out


# ------------------------------------------------------------------ whole model
class Model:
    """The reference Model on one flat f32 parameter buffer (order rust/src/model.rs:593-609)."""

    def __init__(self, vocab, d, H, L, E, F):
        self.cfg = (vocab, d, H, L, E, F)
        self._c = [sz(v) for v in self.cfg]
        self.n = int(lib().orc_model_num_params(*self._c))
        nt = int(lib().orc_model_num_tensors(sz(L)))
        offs = np.zeros(nt, np.uint64)
        lens = np.zeros(nt, np.uint64)
        lib().orc_model_tensor_table(*self._c, offs.ctypes.data_as(u64p), lens.ctypes.data_as(u64p))
        self.tensor_off = offs.astype(np.int64)
        self.tensor_len = lens.astype(np.int64)
        names = ["embed", "head"]
        for li in range(L):
            names += [f"l{li}.{n}" for n in ("w_qkv", "b_qkv", "w_gate", "b_gate", "w_o", "b_o", "w1", "b1", "w2", "b2")]
        self.names = names
        self.params = np.zeros(self.n, np.float32)

    def init_reference(self, rng: Rng):
        lib().orc_model_init(*self._c, rng._s(), _f(self.params))

    def tensor(self, name, buf=None):
        i = self.names.index(name)
        b = self.params if buf is None else buf
        return b[self.tensor_off[i]: self.tensor_off[i] + self.tensor_len[i]]

    def forward(self, ids, batch):
        logits = np.empty((ids.size, self.cfg[0]), np.float32)
        lib().orc_model_forward(*self._c, _f(self.params), _u(ids), sz(ids.size), sz(batch), _f(logits))
        return logits

    def forward_backward(self, ids, targets, batch, grads=None, want_logits=False):
        if grads is None:
            grads = np.zeros(self.n, np.float32)
        logits = np.empty((ids.size, self.cfg[0]), np.float32) if want_logits else None
        loss = lib().orc_model_forward_backward(*self._c, _f(self.params), _f(grads), _u(ids), _u(targets),
                                                sz(ids.size), sz(batch), _f(logits))
        return (float(loss), grads, logits) if want_logits else (float(loss), grads)

    def loss(self, ids, targets):
        return float(lib().orc_model_loss(*self._c, _f(self.params), _u(ids), _u(targets), sz(ids.size)))

    def new_decode_state(self):
        _, d, H, L, _, _ = self.cfg
        dh = d // H
        return np.zeros((L, H, dh, dh), np.float32)

    def step(self, tok, state):
        logits = np.empty((1, self.cfg[0]), np.float32)
        lib().orc_model_step(*self._c, _f(self.params), C.c_uint32(int(tok)), _f(state), _f(logits))
        return logits

    def adamw_step(self, grads, m, v, counter, lr, b1=0.9, b2=0.95, eps=1e-8, wd=0.01):
        cnt = C.c_uint32(counter)
        lib().orc_model_adamw_step(*self._c, _f(self.params), _f(grads), _f(m), _f(v), C.c_float(lr),
                                   C.c_float(b1), C.c_float(b2), C.c_float(eps), C.c_float(wd), C.byref(cnt))
        return cnt.value
