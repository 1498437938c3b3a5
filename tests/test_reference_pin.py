"""Pins the CPU oracle (and the library) against the REFERENCE'S OWN CUDA kernels.

oracle/_ref/libasca_ref.so is rust/kernels/asca.cu compiled unmodified (oracle/build_ref.py)
behind host launchers that use the reference's launch shapes. The reference documents these
kernels as agreeing with its CPU path to <= 1.2e-6 (docs/CUDA.md:25-34, :254-255); here the
restated CPU path has to agree with them to the same order, which ties the oracle to outputs
of the reference's own code rather than to a restatement alone. Shapes are the ones `asca gpu`
uses (rust/src/main.rs:790-1150) plus dh = 64.
"""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu

PIN_TOL = 5e-6


@pytest.fixture(scope="module")
def ref():
    from oracle import refgpu

    if not refgpu.available():
        pytest.skip("oracle/_ref/libasca_ref.so not built (reference tree absent at build time)")
    return refgpu


def _delta_inputs(orc, seed, B, T, H, dh):
    rng = orc.Rng(seed)
    n, d = B * T, H * dh
    q, k, v, d_o = (rng.normal((n, d)) for _ in range(4))
    qn = np.linalg.norm(q.reshape(n, H, dh), axis=-1).astype(np.float32)
    kn = np.linalg.norm(k.reshape(n, H, dh), axis=-1).astype(np.float32)
    q = (q.reshape(n, H, dh) / qn[..., None]).reshape(n, d).astype(np.float32)
    k = (k.reshape(n, H, dh) / kn[..., None]).reshape(n, d).astype(np.float32)
    alpha = (1 / (1 + np.exp(-(2 + 0.5 * rng.normal((n, H)))))).astype(np.float32)
    beta = (1 / (1 + np.exp(-rng.normal((n, H))))).astype(np.float32)
    return q, k, v, alpha, beta, qn, kn, d_o


@pytest.mark.parametrize("m,k,n", [(64, 64, 192), (128, 64, 512), (37, 53, 91), (256, 256, 256)])
def test_matmul_kernels_pin_oracle(orc, ref, gpu, m, k, n):
    rng = orc.Rng(7)
    a, b, at = rng.normal((m, k), 0.1), rng.normal((k, n), 0.1), rng.normal((k, m), 0.1)
    assert rel_err(orc.matmul(a, b), ref.matmul(a, b)) < PIN_TOL
    assert rel_err(orc.matmul_ta(at, b), ref.matmul_ta(at, b)) < PIN_TOL
    assert rel_err(gpu.matmul(a, b), ref.matmul(a, b)) < PIN_TOL


def test_rmsnorm_kernels_pin_oracle(orc, ref, gpu):
    rng = orc.Rng(3)
    x, dy = rng.normal((300, 192)), rng.normal((300, 192))
    y_ref, inv_ref = ref.rmsnorm(x)
    y, inv = orc.rmsnorm(x)
    assert rel_err(y, y_ref) < PIN_TOL and rel_err(inv, inv_ref) < PIN_TOL
    assert rel_err(orc.rmsnorm_bwd(x, dy), ref.rmsnorm_bwd(x, dy)) < PIN_TOL
    assert rel_err(gpu.rmsnorm(x)[0], y_ref) < PIN_TOL


@pytest.mark.parametrize("B,T,H,dh", [(3, 24, 4, 16), (8, 128, 6, 32), (2, 96, 2, 64)])
def test_delta_kernels_pin_oracle(orc, ref, gpu, B, T, H, dh):
    q, k, v, alpha, beta, qn, kn, d_o = _delta_inputs(orc, 11 + dh, B, T, H, dh)
    o_ref, st_ref = ref.delta_scan(q, k, v, alpha, beta, B, T, H, dh)
    o, _, st = orc.delta_scan(q, k, v, alpha, beta, B, T, H, dh, want_states=True)
    assert rel_err(o, o_ref) < PIN_TOL          # reference reports 1.5e-7 (docs/CUDA.md:27)
    assert rel_err(st, st_ref) < PIN_TOL        # reference reports 1.1e-7
    o2, dqkv_ref, dgate_ref = ref.delta_fwd_bwd(q, k, v, alpha, beta, qn, kn, d_o, B, T, H, dh)
    assert np.array_equal(o2, o_ref)
    d_qkv, d_gate = orc.delta_bptt(q, k, v, alpha, beta, qn, kn, d_o, B, T, H, dh)
    assert rel_err(d_qkv, dqkv_ref) < PIN_TOL   # reference reports <= 8.0e-7
    assert rel_err(d_gate, dgate_ref) < PIN_TOL
    # and the library against the reference's kernels directly
    og, dev = gpu.delta_scan(q, k, v, alpha, beta, B, T, H, dh)
    gq, gg = gpu.delta_bwd_dev(dev, d_o, qn, kn)
    assert rel_err(og, o_ref) < PIN_TOL and rel_err(gq, dqkv_ref) < PIN_TOL and rel_err(gg, dgate_ref) < PIN_TOL


def test_silu_and_cross_entropy_kernels_pin_oracle(orc, ref):
    rng = orc.Rng(5)
    pre, dpre = rng.normal(5000, 2.0), rng.normal(5000)
    want = (pre.astype(np.float64) / (1 + np.exp(-pre.astype(np.float64))))
    assert rel_err(ref.silu(pre), want) < PIN_TOL
    # the oracle's silu / silu' live inside the MoE FFN: compare through a 1-expert, identity-free layer
    n, d, F = 40, 8, 16
    xn = rng.normal((n, d))
    w1, w2 = rng.normal((d, F), 0.5), rng.normal((F, d), 0.5)
    b1, b2 = rng.normal(F, 0.1), np.zeros(d, np.float32)
    ids = np.zeros(n, np.uint32)
    out, p, h = orc.moe_ffn_forward(xn, w1, b1, w2, b2, ids, F, 1, want_cache=True)
    assert rel_err(h, ref.silu(p.reshape(-1)).reshape(n, F)) < PIN_TOL
    dout = rng.normal((n, d))
    g = orc.moe_ffn_backward(xn, w1, w2, p, h, ids, dout, F, 1)
    dpre_oracle_sum = g[1]                                   # d_b1 = column sums of dpre
    dpre_ref = ref.silu_bwd((dout @ w2.T).astype(np.float32).reshape(-1), p.reshape(-1)).reshape(n, F)
    assert rel_err(dpre_oracle_sum, dpre_ref.sum(0)) < 2e-5
    # cross-entropy: reference kernel vs the oracle's model-level loss on the same logits
    t, v = 64, 256
    logits = rng.normal((t, v), 2.0)
    targets = rng.below(v, t)
    losses, dl = ref.cross_entropy(logits, targets)
    lse = np.log(np.exp(logits.astype(np.float64) - logits.max(1, keepdims=True)).sum(1)) + logits.max(1)
    assert rel_err(losses, lse - logits[np.arange(t), targets]) < PIN_TOL
    p_soft = np.exp(logits.astype(np.float64) - lse[:, None]) / t
    p_soft[np.arange(t), targets] -= 1.0 / t
    assert rel_err(dl, p_soft) < PIN_TOL
