"""GPU-vs-oracle parity of every entry point, through the C ABI. Modelled on the reference's own
GPU gate `asca gpu` (rust/src/main.rs:790-1203): same ops, same shapes where it names them,
same error metric max|a-b| / max|ref|.

Tolerances: 1e-5 relative for f32 mode, 2e-2 for bf16 mode; integer results bit-exact.
"""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
BF16_TOL = 2e-2


def _delta_inputs(orc, seed, B, T, H, dh):
    """q,k L2-normalised N(0,1); v N(0,1); alpha = sigmoid(N(2,.5)); beta = sigmoid(N(0,1))."""
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


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("m,k,n", [(64, 64, 192), (128, 64, 512), (37, 53, 91), (256, 256, 256), (1, 64, 192),
                                   (300, 1, 5), (513, 130, 257)])
def test_matmul_and_matmul_ta(orc, gpu, m, k, n):
    rng = orc.Rng(7)
    a, b = rng.normal((m, k), 0.1), rng.normal((k, n), 0.1)
    assert rel_err(gpu.matmul(a, b), orc.matmul(a, b)) < F32_TOL
    at = rng.normal((k, m), 0.1)
    assert rel_err(gpu.matmul_ta(at, b), orc.matmul(np.ascontiguousarray(at.T), b)) < F32_TOL
    bt = rng.normal((n, k), 0.1)
    assert rel_err(gpu.matmul_t(a, bt), orc.matmul_t(a, bt)) < F32_TOL


def test_gemm_bias_accumulate_and_bf16(orc, gpu):
    import torch
    from asca_b200 import ops, NN, TN, NT

    rng = orc.Rng(3)
    m, k, n = 200, 96, 136
    a, b, bias, c0 = rng.normal((m, k)), rng.normal((k, n)), rng.normal(n), rng.normal((m, n))
    ref = a.astype(np.float64) @ b + bias + c0
    ta, tb, tbias = (torch.from_numpy(x).cuda() for x in (a, b, bias))
    out = torch.from_numpy(c0.copy()).cuda()
    ops.gemm(gpu, ta, tb, NN, bias=tbias, out=out, accumulate=True)
    gpu.sync()
    assert rel_err(out.cpu().numpy(), ref) < F32_TOL
    # bf16 operands, f32 accumulate
    a16, b16 = ta.bfloat16(), tb.bfloat16()
    ref16 = a16.float().cpu().numpy().astype(np.float64) @ b16.float().cpu().numpy()
    got = ops.gemm(gpu, a16, b16, NN)
    gpu.sync()
    assert rel_err(got.cpu().numpy(), ref16) < 1e-5  # exact products of the rounded inputs
    got_t = ops.gemm(gpu, a16.t().contiguous(), b16, TN)
    got_nt = ops.gemm(gpu, a16, b16.t().contiguous(), NT)
    gpu.sync()
    assert rel_err(got_t.cpu().numpy(), ref16) < 1e-5 and rel_err(got_nt.cpu().numpy(), ref16) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["NN", "TN", "NT"])
def test_gemm_bf16_large_shapes_take_the_wide_tile_path(gpu, mode):
    """Dense bf16 products big enough for the 128 x 256 tiles (two waves, k >= 4096), with ragged M and N and
    accumulation: sampled output rows against float64 products of the same rounded inputs."""
    import torch
    import asca_b200
    from asca_b200 import ops

    M, N, K = 4200, 5000 + 8, 4096 + 64
    g = torch.Generator(device="cuda").manual_seed(17)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    c0 = torch.randn(M, N, device="cuda", generator=g)
    out = c0.clone()
    if mode == "NN":
        ops.gemm(gpu, a, b, asca_b200.NN, out=out, accumulate=True)
    elif mode == "TN":
        ops.gemm(gpu, a.t().contiguous(), b, asca_b200.TN, out=out, accumulate=True)
    else:
        ops.gemm(gpu, a, b.t().contiguous(), asca_b200.NT, out=out, accumulate=True)
    gpu.sync()
    rows = torch.tensor([0, 1, 127, 128, 2049, 4095, 4096, 4199], device="cuda")
    ref = a[rows].double() @ b.double() + c0[rows].double()
    assert rel_err(out[rows].cpu().numpy(), ref.cpu().numpy()) < 1e-5


# ------------------------------------------------------------------ RMSNorm
@pytest.mark.parametrize("rows,cols", [(1, 64), (257, 64), (100, 192), (33, 1024), (17, 2048), (5, 1000), (9, 7)])
def test_rmsnorm_fwd_bwd(orc, gpu, rows, cols):
    rng = orc.Rng(rows * 31 + cols)
    x, dy = rng.normal((rows, cols)), rng.normal((rows, cols))
    y, inv = gpu.rmsnorm(x, 1e-6)
    y_ref, inv_ref = orc.rmsnorm(x, 1e-6)
    assert rel_err(y, y_ref) < F32_TOL and rel_err(inv, inv_ref) < F32_TOL
    assert rel_err(gpu.rmsnorm_bwd(x, dy, 1e-6), orc.rmsnorm_bwd(x, dy, 1e-6)) < F32_TOL


def test_residual_rmsnorm_fusion(orc, gpu):
    import torch
    from asca_b200 import ops

    rng = orc.Rng(11)
    for rows, cols in ((300, 64), (70, 768), (12, 2048)):
        x, y = rng.normal((rows, cols)), rng.normal((rows, cols))
        x_mid, xn = ops.residual_rmsnorm(gpu, torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda())
        gpu.sync()
        s = (x + np.float32(1.0) * y).astype(np.float32)
        assert np.array_equal(x_mid.cpu().numpy(), s)
        assert rel_err(xn.cpu().numpy(), orc.rmsnorm(s)[0]) < F32_TOL


# ------------------------------------------------------------------ gather / scatter / AdamW
def test_gather_scatter_rows(orc, gpu):
    rng = orc.Rng(5)
    src = rng.normal((100, 48))
    idx = rng.below(100, 37).astype(np.int32)
    assert np.array_equal(gpu.gather_rows(src, idx), src[idx])
    perm = np.random.RandomState(0).permutation(100).astype(np.int32)
    dst = np.full((100, 48), -1.0, np.float32)
    gpu.scatter_rows(src[:60].copy(), perm[:60], dst)
    want = np.full((100, 48), -1.0, np.float32)
    want[perm[:60]] = src[:60]
    assert np.array_equal(dst, want)
    import asca_b200
    with pytest.raises(asca_b200.AscaError):
        gpu.gather_rows(src, np.array([0, 100], np.int32))


def test_adamw_matches_cpu_decay_and_per_tensor_counter(orc, gpu):
    import torch
    from asca_b200 import ops

    rng = orc.Rng(13)
    for n in (1, 7, 1023, 40000):
        p, g = rng.normal(n), rng.normal(n, 0.1)
        m, v = rng.normal(n, 0.01), np.abs(rng.normal(n, 0.01)).astype(np.float32)
        lr_t, eps_t, wd_eff = orc.adamw_scalars(3e-3, 0.9, 0.95, 1e-8, 0.01, 5)
        p2, m2, v2 = p.copy(), m.copy(), v.copy()
        orc.adamw_apply(p2, g, m2, v2, lr_t, 0.9, 0.95, eps_t, wd_eff)
        gpu.adamw_update(p, g, m, v, lr_t, 0.9, 0.95, eps_t, wd_eff)
        assert rel_err(p, p2) < F32_TOL and rel_err(m, m2) < F32_TOL and rel_err(v, v2) < F32_TOL
    # whole model, flat buffer, one segmented launch == the oracle's per-tensor loop
    model = orc.Model(256, 16, 2, 1, 2, 16)
    model.init_reference(orc.Rng(1))
    grads = orc.Rng(2).normal(model.n, 0.1)
    mm, vv = np.zeros(model.n, np.float32), np.zeros(model.n, np.float32)
    tp, tg, tm, tv = (torch.from_numpy(x.copy()).cuda() for x in (model.params, grads, mm, vv))
    counter = 24  # second optimizer step: tensor i uses t = 24 + i + 1
    sc = [orc.adamw_scalars(3e-3, 0.9, 0.95, 1e-8, 0.01, counter + i + 1) for i in range(len(model.names))]
    seg = np.concatenate([model.tensor_off, [model.n]])
    ops.adamw_segmented(gpu, tp, tg, tm, tv, seg, [s[0] for s in sc], [s[1] for s in sc], 0.9, 0.95, sc[0][2])
    gpu.sync()
    assert model.adamw_step(grads, mm, vv, counter, 3e-3) == counter + len(model.names)
    assert rel_err(tp.cpu().numpy(), model.params) < F32_TOL
    assert rel_err(tm.cpu().numpy(), mm) < F32_TOL and rel_err(tv.cpu().numpy(), vv) < F32_TOL


# ------------------------------------------------------------------ dispatch (bit-exact)
def _zipf_ids(orc, seed, n, s=1.1):
    w = 1.0 / np.arange(1, 257) ** s
    cdf = np.cumsum(w) / w.sum()
    u = orc.Rng(seed).uniform(n)
    return np.minimum(np.searchsorted(cdf, u), 255).astype(np.uint32)


@pytest.mark.parametrize("n,e", [(0, 4), (1, 4), (31, 8), (1000, 8), (4097, 16), (65536, 64), (5000, 1), (3000, 300)])
def test_dispatch_bit_exact(orc, gpu, n, e):
    ids = orc.Rng(n + e).below(256 if e < 300 else 100000, max(n, 1))[:n].copy()
    perm, off, route = gpu.moe_dispatch(ids, e)
    p2, o2, r2 = orc.moe_dispatch(ids, e)
    assert np.array_equal(off, o2) and np.array_equal(perm, p2) and np.array_equal(route, r2)


def test_dispatch_bit_exact_zipf_skew_config3(orc, gpu):
    ids = _zipf_ids(orc, 9, 65536)
    perm, off, route = gpu.moe_dispatch(ids, 64)
    p2, o2, r2 = orc.moe_dispatch(ids, 64)
    assert np.array_equal(off, o2) and np.array_equal(perm, p2) and np.array_equal(route, r2)
    load = np.diff(off) / 65536
    assert load.max() > 0.15 and load.min() > 0  # skewed, no empty expert
    # all tokens collide on one expert
    same = np.full(5000, 42, np.uint32)
    perm, off, _ = gpu.moe_dispatch(same, 16)
    assert np.array_equal(perm, np.arange(5000, dtype=np.int32))


# ------------------------------------------------------------------ delta rule
def test_delta_scan_reference_gate_shape(orc, gpu):
    # rust/src/main.rs:853-952: B=3, seq=24, H=4, dh=16, states compared too
    B, T, H, dh = 3, 24, 4, 16
    q, k, v, alpha, beta, *_ = _delta_inputs(orc, 7, B, T, H, dh)
    o_ref, _, st_ref = orc.delta_scan(q, k, v, alpha, beta, B, T, H, dh, want_states=True)
    o, dev = gpu.delta_scan(q, k, v, alpha, beta, B, T, H, dh)
    assert rel_err(o, o_ref) < F32_TOL
    assert rel_err(o, orc.delta_scan_scalar(q, k, v, alpha, beta, B, T, H, dh)) < F32_TOL
    st = np.stack(dev.download_states()).reshape(H, B, T + 1, dh, dh)
    assert rel_err(st, st_ref) < F32_TOL
    # sequence isolation: batch=3 equals three batch=1 launches (rust/src/main.rs:954-981)
    for b in range(B):
        s = slice(b * T, (b + 1) * T)
        ob, _ = gpu.delta_scan(q[s], k[s], v[s], alpha[s], beta[s], 1, T, H, dh, keep=False)
        assert np.array_equal(ob, o[s])


@pytest.mark.parametrize("B,T,H,dh", [(2, 1, 2, 16), (1, 15, 3, 16), (2, 70, 2, 32), (2, 130, 3, 64), (1, 200, 2, 128),
                                      (3, 64, 1, 128)])
def test_delta_fwd_bwd_f32(orc, gpu, B, T, H, dh):
    q, k, v, alpha, beta, qn, kn, d_o = _delta_inputs(orc, 100 + T + dh, B, T, H, dh)
    o_ref, sfin_ref = orc.delta_scan(q, k, v, alpha, beta, B, T, H, dh)
    dqkv_ref, dgate_ref = orc.delta_bptt(q, k, v, alpha, beta, qn, kn, d_o, B, T, H, dh)
    o, dev = gpu.delta_scan(q, k, v, alpha, beta, B, T, H, dh)
    d_qkv, d_gate = gpu.delta_bwd_dev(dev, d_o, qn, kn)
    assert rel_err(o, o_ref) < F32_TOL
    d = H * dh
    for name, sl in (("dq", slice(0, d)), ("dk", slice(d, 2 * d)), ("dv", slice(2 * d, 3 * d))):
        assert rel_err(d_qkv[:, sl], dqkv_ref[:, sl]) < F32_TOL, name
    assert rel_err(d_gate[:, :H], dgate_ref[:, :H]) < F32_TOL
    assert rel_err(d_gate[:, H:], dgate_ref[:, H:]) < F32_TOL


@pytest.mark.parametrize("chunk", [1, 16, 24, 64, 256])
def test_delta_chunk_size_does_not_change_results(orc, gpu, chunk):
    import torch
    from asca_b200 import ops

    B, T, H, dh = 2, 150, 2, 64
    arrs = _delta_inputs(orc, 55, B, T, H, dh)
    q, k, v, alpha, beta, qn, kn, d_o = (torch.from_numpy(a).cuda() for a in arrs)
    o, s_final, ckpt = ops.delta_fwd(gpu, q, k, v, alpha, beta, B, T, H, dh, chunk=chunk, want_final=True)
    d_qkv, d_gate = ops.delta_bwd(gpu, q, k, v, alpha, beta, qn, kn, d_o, ckpt, B, T, H, dh, chunk=chunk)
    gpu.sync()
    o_ref, sfin_ref = orc.delta_scan(*arrs[:5], B, T, H, dh)
    dqkv_ref, dgate_ref = orc.delta_bptt(*arrs[:5], arrs[5], arrs[6], arrs[7], B, T, H, dh)
    assert rel_err(o.cpu().numpy(), o_ref) < F32_TOL
    assert rel_err(s_final.cpu().numpy(), sfin_ref) < F32_TOL
    assert rel_err(d_qkv.cpu().numpy(), dqkv_ref) < F32_TOL
    assert rel_err(d_gate.cpu().numpy(), dgate_ref) < F32_TOL


def test_delta_prefill_continuation_with_initial_state(orc, gpu):
    import torch
    from asca_b200 import ops

    B, T, H, dh = 2, 96, 2, 64
    arrs = _delta_inputs(orc, 77, B, T, H, dh)
    q, k, v, alpha, beta = (torch.from_numpy(a).cuda() for a in arrs[:5])
    o_full, s_full, _ = ops.delta_fwd(gpu, q, k, v, alpha, beta, B, T, H, dh, want_final=True, want_ckpt=False)
    half = T // 2

    def part(x, lo, hi):
        return x.view(B, T, -1)[:, lo:hi].contiguous().view(B * (hi - lo), -1)

    a1 = [part(x, 0, half) for x in (q, k, v, alpha, beta)]
    a2 = [part(x, half, T) for x in (q, k, v, alpha, beta)]
    o1, s1, _ = ops.delta_fwd(gpu, *a1, B, half, H, dh, want_final=True, want_ckpt=False)
    o2, s2, _ = ops.delta_fwd(gpu, *a2, B, T - half, H, dh, s_init=s1, want_final=True, want_ckpt=False)
    gpu.sync()
    assert torch.equal(part(o_full, 0, half), o1) and torch.equal(part(o_full, half, T), o2)
    assert torch.equal(s_full, s2)


def test_delta_bf16_mode(orc, gpu):
    import torch
    from asca_b200 import ops

    B, T, H, dh = 2, 128, 2, 128
    arrs = _delta_inputs(orc, 91, B, T, H, dh)
    q, k, v, alpha, beta, qn, kn, d_o = (torch.from_numpy(a).cuda() for a in arrs)
    q16, k16, v16, do16 = (x.bfloat16() for x in (q, k, v, d_o))
    o, _, ckpt = ops.delta_fwd(gpu, q16, k16, v16, alpha, beta, B, T, H, dh)
    d_qkv, d_gate = ops.delta_bwd(gpu, q16, k16, v16, alpha, beta, qn, kn, do16, ckpt, B, T, H, dh)
    gpu.sync()
    o_ref, _ = orc.delta_scan(*arrs[:5], B, T, H, dh)
    dqkv_ref, dgate_ref = orc.delta_bptt(*arrs[:5], arrs[5], arrs[6], arrs[7], B, T, H, dh)
    assert o.dtype == torch.bfloat16
    assert rel_err(o.float().cpu().numpy(), o_ref) < BF16_TOL
    assert rel_err(d_qkv.cpu().numpy(), dqkv_ref) < BF16_TOL
    assert rel_err(d_gate.cpu().numpy(), dgate_ref) < BF16_TOL


@pytest.mark.parametrize("dh", [128, 64])
@pytest.mark.parametrize("B,T,H", [(1, 64, 1), (2, 128, 2), (2, 200, 3), (1, 1000, 2), (3, 37, 1)])
def test_delta_bf16_tensor_core_forward(orc, gpu, B, T, H, dh):
    """bf16 inputs at dh = 128 (and dh = 64, zero-padded to 128 inside the kernels) take the chunked WY/UT tcgen05
    forward: outputs, final state and every chunk checkpoint against the f32 recurrence on the same (bf16-rounded)
    inputs; ragged last chunk; continuation from an initial state."""
    import torch
    from asca_b200 import ops

    arrs = _delta_inputs(orc, 300 + T, B, T, H, dh)
    q, k, v, alpha, beta = (torch.from_numpy(a).cuda() for a in arrs[:5])
    q16, k16, v16 = q.bfloat16(), k.bfloat16(), v.bfloat16()
    qr, kr, vr = (x.float().cpu().numpy() for x in (q16, k16, v16))
    o_ref, sfin_ref, st_ref = orc.delta_scan(qr, kr, vr, arrs[3], arrs[4], B, T, H, dh, want_states=True)
    o, s_final, ckpt = ops.delta_fwd(gpu, q16, k16, v16, alpha, beta, B, T, H, dh, chunk=64, want_final=True)
    gpu.sync()
    assert o.dtype == torch.bfloat16
    assert rel_err(o.float().cpu().numpy(), o_ref) < BF16_TOL
    assert rel_err(s_final.cpu().numpy(), sfin_ref) < BF16_TOL
    n_ck = (T + 63) // 64
    # tensor-core mode keeps the chunk-start states as bf16 in the first half of the buffer
    ck = ckpt.view(torch.bfloat16)[: B * H * n_ck * dh * dh].view(B, H, n_ck, dh, dh).float().cpu().numpy()
    want = st_ref[:, :, 0:T:64].transpose(1, 0, 2, 3, 4)      # (H,B,..) -> (B,H,n_ck,dh,dh)
    assert ck.shape == want.shape
    assert rel_err(ck, want) < BF16_TOL
    # continuation: second half from the first half's final state
    if T >= 128:
        half = (T // 128) * 64

        def part(x, lo, hi):
            return x.view(B, T, -1)[:, lo:hi].contiguous().view(B * (hi - lo), -1)

        a1 = [part(x, 0, half) for x in (q16, k16, v16, alpha, beta)]
        a2 = [part(x, half, T) for x in (q16, k16, v16, alpha, beta)]
        o1, s1, _ = ops.delta_fwd(gpu, *a1, B, half, H, dh, want_final=True, want_ckpt=False)
        o2, s2, _ = ops.delta_fwd(gpu, *a2, B, T - half, H, dh, s_init=s1, want_final=True, want_ckpt=False)
        gpu.sync()
        assert rel_err(part(o, half, T).float().cpu().numpy(), o2.float().cpu().numpy()) < 1e-2
        assert rel_err(s2.cpu().numpy(), sfin_ref) < BF16_TOL


@pytest.mark.parametrize("dh", [128, 64])
@pytest.mark.parametrize("B,T,H", [(1, 64, 1), (2, 128, 2), (2, 200, 3), (1, 700, 2), (3, 37, 1)])
def test_delta_bf16_tensor_core_backward(orc, gpu, B, T, H, dh):
    """bf16 inputs at dh = 128 or 64, chunk 64: the reverse chunked scan on tcgen05 against the f32 BPTT of
    the oracle on the same (bf16-rounded) inputs; every output block checked separately; the launch list must
    name the tensor-core kernels."""
    import torch
    from asca_b200 import ops

    d = H * dh
    arrs = _delta_inputs(orc, 500 + T, B, T, H, dh)
    q, k, v, alpha, beta, qn, kn, d_o = (torch.from_numpy(a).cuda() for a in arrs)
    q16, k16, v16, do16 = (x.bfloat16() for x in (q, k, v, d_o))
    qr, kr, vr, dor = (x.float().cpu().numpy() for x in (q16, k16, v16, do16))
    dqkv_ref, dgate_ref = orc.delta_bptt(qr, kr, vr, arrs[3], arrs[4], arrs[5], arrs[6], dor, B, T, H, dh)
    gpu.profile(True)
    o, _, ckpt = ops.delta_fwd(gpu, q16, k16, v16, alpha, beta, B, T, H, dh, chunk=64)
    d_qkv, d_gate = ops.delta_bwd(gpu, q16, k16, v16, alpha, beta, qn, kn, do16, ckpt, B, T, H, dh, chunk=64)
    gpu.sync()
    names = {n for n, _ in gpu.profile_read()}
    gpu.profile(False)
    assert {"delta_prep_tc_kernel", "delta_fwd_tc_kernel", "delta_bwd_tc_kernel"} <= names, names
    got, gg = d_qkv.cpu().numpy(), d_gate.cpu().numpy()
    assert rel_err(got[:, 2 * d:], dqkv_ref[:, 2 * d:]) < BF16_TOL, "dv"
    assert rel_err(got[:, :d], dqkv_ref[:, :d]) < BF16_TOL, "dq"
    assert rel_err(got[:, d:2 * d], dqkv_ref[:, d:2 * d]) < BF16_TOL, "dk"
    assert rel_err(gg[:, H:], dgate_ref[:, H:]) < BF16_TOL, "d_gate beta"
    assert rel_err(gg[:, :H], dgate_ref[:, :H]) < BF16_TOL, "d_gate alpha"


@pytest.mark.parametrize("dh", [16, 32, 64, 128])
def test_delta_decode_step(orc, gpu, dh):
    import torch
    from asca_b200 import ops

    ns, H, steps = 5, 3, 6
    d = H * dh
    rng = orc.Rng(dh)
    S_ref = rng.normal((ns, H, dh, dh), 0.1)
    S = torch.from_numpy(S_ref.copy()).cuda()
    for _ in range(steps):
        q, k, v, alpha, beta, *_ = _delta_inputs(orc, int(rng.below(1000, 1)[0]), ns, 1, H, dh)
        o_ref = orc.delta_step_core(q, k, v, alpha, beta, S_ref, H, dh)
        o = ops.delta_step(gpu, *(torch.from_numpy(a).cuda() for a in (q, k, v, alpha, beta)), S, H, dh)
        gpu.sync()
        assert rel_err(o.cpu().numpy(), o_ref) < F32_TOL
        assert rel_err(S.cpu().numpy(), S_ref) < F32_TOL
    # fused prologue: raw qkv + gate logits, compared with the block-level step of the oracle
    blk = orc.DeltaBlock(d, H, orc.Rng(3))
    x = rng.normal((1, d))
    st_ref = rng.normal((H, dh, dh), 0.1)
    st = torch.from_numpy(st_ref.copy()).cuda().view(1, H, dh, dh)
    qkv = orc.matmul(x, blk.w_qkv) + blk.b_qkv
    gate = orc.matmul(x, blk.w_gate) + blk.b_gate
    o = ops.delta_step(gpu, torch.from_numpy(qkv).cuda(), None, None, torch.from_numpy(gate).cuda(), None, st, H, dh,
                       fused=True)
    gpu.sync()
    y = orc.matmul(o.cpu().numpy(), blk.w_o) + blk.b_o
    if dh <= 64 or True:  # the oracle's step uses heap scratch, so dh=128 is checkable too
        y_ref = blk.step(x, st_ref)
        assert rel_err(y, y_ref) < F32_TOL
        assert rel_err(st.cpu().numpy().reshape(H, dh, dh), st_ref) < F32_TOL


def test_delta_block_gradient_gpu_vs_cpu(orc, gpu):
    """rust/src/main.rs:1104-1150: a whole DeltaBlock at B=8, seq=128, d=192, H=6 with the scan and
    the BPTT on the device and the projections through the library's GEMMs."""
    import torch
    from asca_b200 import ops, NN, TN, NT

    B, T, d, H = 8, 128, 192, 6
    dh, n = d // H, B * T
    rng = orc.Rng(42)
    blk = orc.DeltaBlock(d, H, rng)
    x, dy = rng.normal((n, d), 0.5), rng.normal((n, d))
    y_ref, cache = blk.forward(x, B)
    dx_ref, g_ref = blk.backward(cache, dy)
    blk.free(cache)
    t = {nm: torch.from_numpy(getattr(blk, nm)).cuda() for nm in blk.NAMES}
    tx, tdy = torch.from_numpy(x).cuda(), torch.from_numpy(dy).cuda()
    qkv = ops.gemm(gpu, tx, t["w_qkv"], NN, bias=t["b_qkv"])
    gate = ops.gemm(gpu, tx, t["w_gate"], NN, bias=t["b_gate"])
    q, k, v, qn, kn, al, be = ops.delta_prep(gpu, qkv, gate, H, dh)
    o, _, ckpt = ops.delta_fwd(gpu, q, k, v, al, be, B, T, H, dh)
    y = ops.gemm(gpu, o, t["w_o"], NN, bias=t["b_o"])
    d_o = ops.gemm(gpu, tdy, t["w_o"], NT)
    g_w_o = ops.gemm(gpu, o, tdy, TN)
    d_qkv, d_gate = ops.delta_bwd(gpu, q, k, v, al, be, qn, kn, d_o, ckpt, B, T, H, dh)
    g_w_qkv = ops.gemm(gpu, tx, d_qkv, TN)
    g_w_gate = ops.gemm(gpu, tx, d_gate, TN)
    dx = ops.gemm(gpu, d_qkv, t["w_qkv"], NT)
    ops.gemm(gpu, d_gate, t["w_gate"], NT, out=dx, accumulate=True)
    gpu.sync()
    assert rel_err(y.cpu().numpy(), y_ref) < F32_TOL
    assert rel_err(dx.cpu().numpy(), dx_ref) < F32_TOL
    assert rel_err(g_w_o.cpu().numpy(), g_ref["w_o"]) < F32_TOL
    assert rel_err(g_w_qkv.cpu().numpy(), g_ref["w_qkv"]) < F32_TOL
    assert rel_err(g_w_gate.cpu().numpy(), g_ref["w_gate"]) < F32_TOL
    assert rel_err(d_qkv.sum(0).cpu().numpy(), g_ref["b_qkv"]) < 1e-4  # bias grads: column sums
    assert rel_err(d_gate.sum(0).cpu().numpy(), g_ref["b_gate"]) < 1e-4


# ------------------------------------------------------------------ hash MoE
def _moe_params(orc, seed, d, F, E, bias=True):
    rng = orc.Rng(seed)
    w1 = rng.normal((d, E * F), float(np.sqrt(1.0 / d)))
    w2 = rng.normal((E * F, d), float(np.sqrt(1.0 / F)))
    b1 = rng.normal(E * F, 0.1) if bias else np.zeros(E * F, np.float32)
    b2 = rng.normal(d, 0.1) if bias else np.zeros(d, np.float32)
    return w1, b1, w2, b2


@pytest.mark.parametrize("n,d,F,E,vocab", [(1024, 192, 384, 8, 4096), (300, 64, 256, 4, 256), (77, 16, 20, 3, 256),
                                           (2048, 64, 128, 64, 40)])
def test_moe_forward_backward_f32(orc, gpu, n, d, F, E, vocab):
    # first case = rust/src/main.rs:991-1051 (T=1024, d=192, d_ff=384, E=8, ids below 4096);
    # last case leaves many experts empty
    w1, b1, w2, b2 = _moe_params(orc, 77, d, F, E)
    rng = orc.Rng(n)
    x = rng.normal((n, d), 0.5)
    ids = rng.below(vocab, n)
    dout = rng.normal((n, d))
    xn, _ = orc.rmsnorm(x)
    out_ref, pre_ref, hid_ref = orc.moe_ffn_forward(xn, w1, b1, w2, b2, ids, F, E, want_cache=True)
    g_ref = orc.moe_ffn_backward(xn, w1, w2, pre_ref, hid_ref, ids, dout, F, E)
    out, dev = gpu.moe_forward_dev(xn, w1, b1, w2, b2, ids, F)
    pre, hid = dev.download_pre_hidden()
    assert rel_err(out, out_ref) < F32_TOL
    assert rel_err(pre, pre_ref) < F32_TOL and rel_err(hid, hid_ref) < F32_TOL
    r = gpu.moe_bwd_dev(dev, dout)
    for name, got, want in (("d_w1", r.d_w1, g_ref[0]), ("d_b1", r.d_b1, g_ref[1]), ("d_w2", r.d_w2, g_ref[2]),
                            ("d_b2", r.d_b2, g_ref[3]), ("dxn", r.dxn, g_ref[4])):
        assert rel_err(got, want) < F32_TOL, name


def test_moe_bf16_mode(orc, gpu):
    import torch
    from asca_b200 import ops

    n, d, F, E = 600, 128, 256, 8
    w1, b1, w2, b2 = _moe_params(orc, 5, d, F, E, bias=False)
    rng = orc.Rng(8)
    xn = orc.rmsnorm(rng.normal((n, d)))[0]
    ids = rng.below(256, n)
    dout = rng.normal((n, d))
    out_ref, pre_ref, hid_ref = orc.moe_ffn_forward(xn, w1, b1, w2, b2, ids, F, E, want_cache=True)
    g_ref = orc.moe_ffn_backward(xn, w1, w2, pre_ref, hid_ref, ids, dout, F, E)
    c = lambda a: torch.from_numpy(a).cuda()
    perm, offsets = ops.moe_dispatch(gpu, c(ids.view(np.int32)), E)
    txn, tw1, tw2 = c(xn).bfloat16(), c(w1).bfloat16(), c(w2).bfloat16()
    out, pre_p, hid_p = ops.moe_fwd(gpu, txn, tw1, c(b1), tw2, c(b2), perm, offsets, F, E)
    grads = ops.moe_bwd(gpu, txn, tw1, tw2, pre_p, hid_p, c(dout), perm, offsets, F, E)
    gpu.sync()
    assert hid_p.dtype == torch.bfloat16
    assert rel_err(out.cpu().numpy(), out_ref) < BF16_TOL
    for got, want in zip(grads, g_ref):
        assert rel_err(got.cpu().numpy(), want) < BF16_TOL


def test_moe_layer_with_norm_and_decode_step(orc, gpu):
    import torch
    from asca_b200 import ops

    n, d, F, E = 256, 64, 256, 4
    w1, b1, w2, b2 = _moe_params(orc, 21, d, F, E)
    rng = orc.Rng(2)
    x, dout = rng.normal((n, d)), rng.normal((n, d))
    ids = rng.below(256, n)
    ref = orc.moe_forward_backward(x, w1, b1, w2, b2, ids, dout, F, E)
    c = lambda a: torch.from_numpy(a).cuda()
    tx = c(x)
    xn = ops.rmsnorm_fwd(gpu, tx)
    perm, offsets = ops.moe_dispatch(gpu, c(ids.view(np.int32)), E)
    out, pre_p, hid_p = ops.moe_fwd(gpu, xn, c(w1), c(b1), c(w2), c(b2), perm, offsets, F, E)
    d_w1, d_b1, d_w2, d_b2, dxn = ops.moe_bwd(gpu, xn, c(w1), c(w2), pre_p, hid_p, c(dout), perm, offsets, F, E)
    dx = ops.rmsnorm_bwd(gpu, tx, dxn)
    gpu.sync()
    for got, want in zip((out, d_w1, d_b1, d_w2, d_b2, dx), ref):
        assert rel_err(got.cpu().numpy(), want) < F32_TOL
    # decode: one token per stream
    step = ops.moe_step(gpu, tx[:32].contiguous(), c(ids[:32].view(np.int32)), c(w1), c(b1), c(w2), c(b2), F, E)
    gpu.sync()
    want = np.concatenate([orc.moe_step(x[i:i + 1], w1, b1, w2, b2, int(ids[i]), F, E) for i in range(32)])
    assert rel_err(step.cpu().numpy(), want) < F32_TOL
    assert rel_err(step.cpu().numpy(), ref[0][:32]) < F32_TOL  # decode == forward rows


@pytest.mark.parametrize("m,k,n", [(128, 64, 128), (300, 200, 264), (1000, 1032, 520), (129, 72, 8)])
def test_bf16_tensor_core_gemm_all_modes(orc, gpu, m, k, n):
    """bf16 operands go through the tcgen05 kernel (row pitches are multiples of 8): ragged M, N
    and K tails, bias and accumulate, all three modes."""
    import torch
    from asca_b200 import ops, NN, TN, NT

    rng = orc.Rng(m + k + n)
    a, b = rng.normal((m, k)), rng.normal((k, n))
    bias, c0 = rng.normal(n), rng.normal((m, n))
    a16, b16 = torch.from_numpy(a).cuda().bfloat16(), torch.from_numpy(b).cuda().bfloat16()
    ref = a16.float().cpu().numpy().astype(np.float64) @ b16.float().cpu().numpy().astype(np.float64)
    got = ops.gemm(gpu, a16, b16, NN)
    got_tn = ops.gemm(gpu, a16.t().contiguous(), b16, TN) if m % 8 == 0 else None
    got_nt = ops.gemm(gpu, a16, b16.t().contiguous(), NT)
    out = torch.from_numpy(c0.copy()).cuda()
    ops.gemm(gpu, a16, b16, NN, bias=torch.from_numpy(bias).cuda(), out=out, accumulate=True)
    gpu.sync()
    assert rel_err(got.cpu().numpy(), ref) < 1e-5
    assert rel_err(got_nt.cpu().numpy(), ref) < 1e-5
    if got_tn is not None:
        assert rel_err(got_tn.cpu().numpy(), ref) < 1e-5
    assert rel_err(out.cpu().numpy(), ref + bias + c0) < 1e-5


@pytest.mark.parametrize("n,d,F,E,vocab", [(4096, 256, 512, 16, 256), (700, 64, 128, 64, 30), (9000, 128, 192, 8, 256),
                                           (12288, 512, 1024, 16, 256)])
def test_moe_bf16_tensor_core_ragged_experts(orc, gpu, n, d, F, E, vocab):
    """Grouped tcgen05 products: skewed loads, experts with fewer than 64 rows and empty experts; the last case is
    large enough for the 256-row tiles of CTA pairs in all six grouped products (ragged 256-row tiles, ragged k)."""
    import torch
    from asca_b200 import ops

    w1, b1, w2, b2 = _moe_params(orc, 15, d, F, E)
    rng = orc.Rng(n)
    ids = _zipf_ids(orc, n, n) % vocab
    xn = orc.rmsnorm(rng.normal((n, d)))[0]
    dout = rng.normal((n, d))
    c = lambda a: torch.from_numpy(a).cuda()
    txn, tw1, tw2 = c(xn).bfloat16(), c(w1).bfloat16(), c(w2).bfloat16()
    # oracle on the bf16-rounded operands, so only accumulation / intermediate rounding differs
    xr, w1r, w2r = (t.float().cpu().numpy() for t in (txn, tw1, tw2))
    out_ref, pre_ref, hid_ref = orc.moe_ffn_forward(xr, w1r, b1, w2r, b2, ids, F, E, want_cache=True)
    g_ref = orc.moe_ffn_backward(xr, w1r, w2r, pre_ref, hid_ref, ids, dout, F, E)
    perm, offsets = ops.moe_dispatch(gpu, c(ids.view(np.int32)), E)
    out, pre_p, hid_p = ops.moe_fwd(gpu, txn, tw1, c(b1), tw2, c(b2), perm, offsets, F, E)
    grads = ops.moe_bwd(gpu, txn, tw1, tw2, pre_p, hid_p, c(dout), perm, offsets, F, E)
    gpu.sync()
    pre_tok = np.empty_like(pre_ref)
    pre_tok[perm.cpu().numpy()] = pre_p.cpu().numpy()
    assert rel_err(pre_tok, pre_ref) < 1e-5          # f32 accumulate of identical bf16 operands
    assert rel_err(out.cpu().numpy(), out_ref) < BF16_TOL
    for name, got, want in zip(("d_w1", "d_b1", "d_w2", "d_b2", "dxn"), grads, g_ref):
        assert rel_err(got.cpu().numpy(), want) < BF16_TOL, name


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n", [(256, 20000, 32), (128, 16384, 264), (72, 40008, 8)])
def test_bf16_weight_gradient_with_few_tiles_and_long_k(orc, gpu, m, k, n):
    """A^T B over tens of thousands of rows into a narrow output (the gate and head weight gradients): the k range
    is cut into slices and the slices are added in order; plain, and accumulating onto an existing C."""
    import torch
    from asca_b200 import ops, TN

    rng = orc.Rng(m + k + n)
    a, b, c0 = rng.normal((k, m)), rng.normal((k, n)), rng.normal((m, n))
    a16, b16 = torch.from_numpy(a).cuda().bfloat16(), torch.from_numpy(b).cuda().bfloat16()
    ref = a16.float().cpu().numpy().astype(np.float64).T @ b16.float().cpu().numpy().astype(np.float64)
    got = ops.gemm(gpu, a16, b16, TN)
    out = torch.from_numpy(c0.copy()).cuda()
    ops.gemm(gpu, a16, b16, TN, out=out, accumulate=True)
    again = ops.gemm(gpu, a16, b16, TN)
    gpu.sync()
    assert rel_err(got.cpu().numpy(), ref) < 1e-5
    assert rel_err(out.cpu().numpy(), ref + c0) < 1e-5
    assert torch.equal(got, again)      # fixed order of the slices: run-to-run identical


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n", [(1, 64, 128), (17, 768, 2328), (32, 200, 136), (33, 72, 8), (64, 3072, 768), (200, 96, 264),
                                   (256, 768, 768)])
def test_bf16_few_row_gemm(orc, gpu, m, k, n):
    """At most 256 rows: the weight-streaming kernel (output features on the instruction's 128 rows, tokens on its
    N). Ragged rows, features and k; bias and accumulate."""
    import torch
    from asca_b200 import ops, NN

    rng = orc.Rng(7 * m + k + n)
    a, b = rng.normal((m, k)), rng.normal((k, n))
    bias, c0 = rng.normal(n), rng.normal((m, n))
    a16, b16 = torch.from_numpy(a).cuda().bfloat16(), torch.from_numpy(b).cuda().bfloat16()
    ref = a16.float().cpu().numpy().astype(np.float64) @ b16.float().cpu().numpy().astype(np.float64)
    got = ops.gemm(gpu, a16, b16, NN)
    out = torch.from_numpy(c0.copy()).cuda()
    ops.gemm(gpu, a16, b16, NN, bias=torch.from_numpy(bias).cuda(), out=out, accumulate=True)
    gpu.sync()
    assert rel_err(got.cpu().numpy(), ref) < 1e-5
    assert rel_err(out.cpu().numpy(), ref + bias + c0) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("n,d,F,E,vocab", [(256, 128, 256, 16, 256), (100, 64, 128, 8, 5), (500, 192, 384, 8, 256), (1, 64, 128, 4, 256)])
def test_moe_bf16_few_tokens_per_expert(orc, gpu, n, d, F, E, vocab):
    """A decode step's load: a handful of tokens per expert, empty experts, one expert with several token tiles.
    The forward goes through the weight-streaming grouped products and must equal the oracle on the rounded operands."""
    import torch
    from asca_b200 import ops

    w1, b1, w2, b2 = _moe_params(orc, 21, d, F, E)
    rng = orc.Rng(n + E)
    ids = _zipf_ids(orc, n + 1, n) % vocab
    xn = orc.rmsnorm(rng.normal((n, d)))[0]
    c = lambda a: torch.from_numpy(a).cuda()
    txn, tw1, tw2 = c(xn).bfloat16(), c(w1).bfloat16(), c(w2).bfloat16()
    xr, w1r, w2r = (t.float().cpu().numpy() for t in (txn, tw1, tw2))
    out_ref, pre_ref, hid_ref = orc.moe_ffn_forward(xr, w1r, b1, w2r, b2, ids, F, E, want_cache=True)
    perm, offsets = ops.moe_dispatch(gpu, c(ids.view(np.int32)), E)
    out, pre_p, hid_p = ops.moe_fwd(gpu, txn, tw1, c(b1), tw2, c(b2), perm, offsets, F, E)
    gpu.sync()
    pm = perm.cpu().numpy()
    pre_tok = np.empty_like(pre_ref)
    pre_tok[pm] = pre_p.cpu().numpy()
    hid_tok = np.empty_like(hid_ref)
    hid_tok[pm] = hid_p.float().cpu().numpy()
    assert rel_err(pre_tok, pre_ref) < 1e-5
    assert rel_err(hid_tok, hid_ref) < BF16_TOL
    assert rel_err(out.cpu().numpy(), out_ref) < BF16_TOL


# ------------------------------------------------------------------ argument errors (host side, before any launch)
def test_bad_arguments_fail_before_launch(orc, gpu):
    import asca_b200

    q = np.zeros((8, 24), np.float32)
    a = np.zeros((8, 1), np.float32)
    with pytest.raises(asca_b200.AscaError) as e:
        gpu.delta_scan(q, q, q, a, a, 1, 8, 1, 24)  # dh = 24 unsupported
    assert e.value.code == -4
    before = gpu.launch_count()
    with pytest.raises(asca_b200.AscaError):
        gpu._call("asca_rmsnorm_fwd", gpu._ctx, None, None, None, 1, 1, asca_b200._f(1e-6))
    assert gpu.launch_count() == before


@pytest.mark.gpu
def test_delta_host_pipeline_matches_direct_calls(orc, gpu):
    """Per-sequence copy/compute/copy pipeline == one batched call on device tensors (bit-exact)."""
    import torch
    from asca_b200 import ops

    B, T, H, dh = 5, 192, 2, 128
    arrs = _delta_inputs(orc, 977, B, T, H, dh)
    q, k, v, alpha, beta = (torch.from_numpy(a) for a in arrs[:5])
    g = torch.Generator().manual_seed(5)
    d_o = torch.randn(B * T, H * dh, generator=g)
    qn = torch.rand(B * T, H, generator=g) + 0.5
    kn = torch.rand(B * T, H, generator=g) + 0.5
    host = [x.bfloat16().pin_memory() for x in (q, k, v)] + [x.pin_memory() for x in (alpha, beta, qn, kn)] + [d_o.bfloat16().pin_memory()]
    o_h = torch.empty((B * T, H * dh), dtype=torch.bfloat16).pin_memory()
    dqkv_h = torch.empty((B * T, 3 * H * dh)).pin_memory()
    dgate_h = torch.empty((B * T, 2 * H)).pin_memory()
    pipe = ops.DeltaHostPipeline(gpu, T, H, dh, chunk=64, dtype=torch.bfloat16, depth=2)
    pipe.run(*host, o_h, dqkv_h, dgate_h, B)
    dq, dk, dv, da, db, dqn, dkn, ddo = (x.cuda() for x in host)
    o, _, ckpt = ops.delta_fwd(gpu, dq, dk, dv, da, db, B, T, H, dh, chunk=64)
    d_qkv, d_gate = ops.delta_bwd(gpu, dq, dk, dv, da, db, dqn, dkn, ddo, ckpt, B, T, H, dh, chunk=64)
    gpu.sync()
    assert torch.equal(o.cpu(), o_h)
    assert torch.equal(d_qkv.cpu(), dqkv_h)
    assert torch.equal(d_gate.cpu(), dgate_h)


@pytest.mark.gpu
def test_delta_tc_backward_without_kept_tiles_and_with_several_kept(orc, gpu):
    """The tensor-core backward gives the same bits whether it finds the forward's tiles (several
    forwards may be pending, one tile set per checkpoint buffer) or rebuilds them from q, k, v."""
    import torch
    from asca_b200 import ops

    B, T, H, dh = 2, 200, 2, 128
    sets = []
    for seed in (31, 32, 33):
        arrs = _delta_inputs(orc, seed, B, T, H, dh)
        q, k, v, al, be, qn, kn, d_o = (torch.from_numpy(a).cuda() for a in arrs)
        sets.append([q.bfloat16(), k.bfloat16(), v.bfloat16(), al, be, qn, kn, d_o.bfloat16()])
    ckpts = []
    for s in sets:      # three forwards first, as a model does for its blocks
        _, _, ck = ops.delta_fwd(gpu, *s[:5], B, T, H, dh, chunk=64)
        ckpts.append(ck)
    for s, ck in zip(reversed(sets), reversed(ckpts)):
        d1, g1 = ops.delta_bwd(gpu, *s[:5], s[5], s[6], s[7], ck, B, T, H, dh, chunk=64)        # kept tiles
        d2, g2 = ops.delta_bwd(gpu, *s[:5], s[5], s[6], s[7], ck.clone(), B, T, H, dh, chunk=64)  # rebuilt
        gpu.sync()
        assert torch.equal(d1, d2) and torch.equal(g1, g2)


@pytest.mark.gpu
def test_delta_tc_kept_tiles_are_filed_under_the_inputs_too(orc, gpu):
    """A backward that presents the forward's checkpoint buffer but other q/k/v buffers must not pick up the
    forward's tiles: it rebuilds them from what it was given. Trimming the context drops every kept tile."""
    import ctypes

    import torch
    from asca_b200 import ops

    B, T, H, dh = 1, 192, 2, 128
    a1 = [torch.from_numpy(a).cuda() for a in _delta_inputs(orc, 41, B, T, H, dh)]
    a2 = [torch.from_numpy(a).cuda() for a in _delta_inputs(orc, 42, B, T, H, dh)]
    s1 = [a1[0].bfloat16(), a1[1].bfloat16(), a1[2].bfloat16(), a1[3], a1[4], a1[5], a1[6], a1[7].bfloat16()]
    s2 = [a2[0].bfloat16(), a2[1].bfloat16(), a2[2].bfloat16(), a2[3], a2[4], a2[5], a2[6], a2[7].bfloat16()]
    _, _, ck1 = ops.delta_fwd(gpu, *s1[:5], B, T, H, dh, chunk=64)
    want, want_g = ops.delta_bwd(gpu, *s1[:5], s1[5], s1[6], s1[7], ck1, B, T, H, dh, chunk=64)
    # the second problem's forward writes its checkpoints into a fresh buffer; copy them over ck1 and present ck1 with
    # the second problem's inputs: same checkpoint address as the kept tiles, different inputs
    _, _, ck2 = ops.delta_fwd(gpu, *s2[:5], B, T, H, dh, chunk=64)
    ref2, ref2_g = ops.delta_bwd(gpu, *s2[:5], s2[5], s2[6], s2[7], ck2, B, T, H, dh, chunk=64)
    _, _, ck1 = ops.delta_fwd(gpu, *s1[:5], B, T, H, dh, chunk=64, ckpt=ck1)
    ck1.copy_(ck2)
    got2, got2_g = ops.delta_bwd(gpu, *s2[:5], s2[5], s2[6], s2[7], ck1, B, T, H, dh, chunk=64)
    gpu.sync()
    assert torch.equal(got2, ref2) and torch.equal(got2_g, ref2_g)
    assert not torch.equal(got2, want)
    gpu._call("asca_ctx_trim", gpu._ctx)
    gpu._call("asca_ctx_set_tile_cache_bytes", gpu._ctx, ctypes.c_size_t(1 << 30))
    _, _, ck3 = ops.delta_fwd(gpu, *s1[:5], B, T, H, dh, chunk=64)
    again, again_g = ops.delta_bwd(gpu, *s1[:5], s1[5], s1[6], s1[7], ck3, B, T, H, dh, chunk=64)
    gpu.sync()
    assert torch.equal(again, want) and torch.equal(again_g, want_g)
    gpu._call("asca_ctx_set_tile_cache_bytes", gpu._ctx, ctypes.c_size_t(32 << 30))


# ------------------------------------------------------------------ the remaining `impl Gpu` call shapes
@pytest.mark.gpu
def test_moe_forward_dev_with_host_built_buckets(orc, gpu):
    """Gpu::moe_forward_dev as the reference calls it (rust/src/model.rs:159-172): the caller's buckets go in, and the
    result equals the ids form (device dispatch) bit for bit, forward and backward."""
    n, d, F, E = 700, 64, 128, 8
    w1, b1, w2, b2 = _moe_params(orc, 9, d, F, E)
    rng = orc.Rng(10)
    xn = orc.rmsnorm(rng.normal((n, d)))[0]
    ids = rng.below(256, n)
    dout = rng.normal((n, d))
    buckets = [[] for _ in range(E)]
    for t, i in enumerate(ids):
        buckets[orc.hash_route(int(i), E)].append(t)
    out_b, dev_b = gpu.moe_forward_dev_buckets(xn, w1, b1, w2, b2, buckets, F)
    out_i, dev_i = gpu.moe_forward_dev(xn, w1, b1, w2, b2, ids, F)
    assert np.array_equal(out_b, out_i)
    assert rel_err(out_b, orc.moe_ffn_forward(xn, w1, b1, w2, b2, ids, F, E)) < F32_TOL
    rb, ri = gpu.moe_bwd_dev(dev_b, dout), gpu.moe_bwd_dev(dev_i, dout)
    for name in ("d_w1", "d_b1", "d_w2", "d_b2", "dxn"):
        assert np.array_equal(getattr(rb, name), getattr(ri, name)), name
    dev_b.free()
    dev_i.free()
    with pytest.raises(Exception):
        gpu.moe_forward_dev_buckets(xn, w1, b1, w2, b2, [b[:-1] for b in buckets], F)    # a token is missing


@pytest.mark.gpu
def test_head_cross_entropy_and_resident_adamw_host_forms(orc, gpu):
    import asca_b200

    rng = orc.Rng(12)
    T, d, V = 300, 96, 256
    h_final, head = rng.normal((T, d)), rng.normal((d, V), 0.1)
    targets = rng.below(V, T)
    ldev = gpu.head_forward_dev(h_final, head)
    logits = ldev.download()
    assert rel_err(logits, orc.matmul(h_final, head)) < F32_TOL
    loss, d_head, dh = gpu.head_bwd_dev(ldev, targets, np.ascontiguousarray(head.T))
    lg = logits.astype(np.float64)
    lse = np.log(np.exp(lg - lg.max(1, keepdims=True)).sum(1)) + lg.max(1)
    loss_ref = float((lse - lg[np.arange(T), targets]).mean())
    dl_ref = np.exp(lg - lse[:, None]) / T
    dl_ref[np.arange(T), targets] -= 1.0 / T
    assert abs(loss - loss_ref) / loss_ref < F32_TOL
    assert rel_err(d_head, h_final.astype(np.float64).T @ dl_ref) < F32_TOL
    assert rel_err(dh, dl_ref @ head.astype(np.float64).T) < F32_TOL
    loss2, dl = gpu.cross_entropy_bwd(logits, targets)
    assert abs(loss2 - loss_ref) / loss_ref < F32_TOL and rel_err(dl, dl_ref) < F32_TOL
    ldev.free()
    # resident AdamW: the moments stay on the device, keyed by the caller's m buffer
    n = 5000
    p_ref, g1, g2 = rng.normal(n, 0.1), rng.normal(n, 0.01), rng.normal(n, 0.01)
    m_host, v_host = np.zeros(n, np.float32), np.zeros(n, np.float32)     # the caller's (stale) host moments
    key = asca_b200.param_key(m_host)
    gpu.reset_param_cache()
    assert gpu.param_moments(key) is None
    p_dev = p_ref.copy()
    mo, vo = np.zeros(n, np.float32), np.zeros(n, np.float32)
    for t, g in ((1, g1), (2, g2)):
        lr_t, eps_t, wd_eff = orc.adamw_scalars(3e-3, 0.9, 0.95, 1e-8, 0.01, t)
        gpu.adamw_resident(key, p_dev, g, m_host, v_host, lr_t, 0.9, 0.95, eps_t, wd_eff)
        orc.adamw_apply(p_ref, g, mo, vo, lr_t, 0.9, 0.95, eps_t, wd_eff)
    assert rel_err(p_dev, p_ref) < F32_TOL
    m_dev, v_dev = gpu.param_moments(key)
    assert rel_err(m_dev, mo) < F32_TOL and rel_err(v_dev, vo) < F32_TOL and not m_host.any()
    gpu.reset_param_cache()
    assert gpu.param_moments(key) is None
    x = rng.normal(1000, 2.0)
    want = x.astype(np.float64) / (1 + np.exp(-x.astype(np.float64)))
    gpu.silu_inplace(x)
    assert rel_err(x, want) < F32_TOL


@pytest.mark.gpu
def test_a_bounded_wait_that_runs_out_reports_and_leaves_the_context_usable(orc, gpu):
    """The give-up path of the tensor-core kernels (a wait limit passed from the host as 20,000 cycles, on an mbarrier
    nothing arms): the kernel returns by itself, the call answers ASCA_ERR_DEVICE, the TMEM it held is free again (a
    tensor-core product right after allocates all of it) and the next calls work."""
    import ctypes

    import asca_b200
    import torch
    from asca_b200 import NN, ops

    gave_up, seen = ctypes.c_int(), ctypes.c_int()
    rc = gpu.lib.asca_selftest_wait_timeout(gpu._ctx, ctypes.c_int64(20000), ctypes.byref(gave_up), ctypes.byref(seen))
    assert rc == -5 and gave_up.value == 1 and seen.value == 1
    assert b"bounded wait" in gpu.lib.asca_last_error(gpu._ctx)
    gpu.sync()                                                   # the error word was cleared: no stale error
    rng = orc.Rng(1)
    a, b = rng.normal((512, 4096)), rng.normal((4096, 512), 0.1)
    got = ops.gemm(gpu, torch.from_numpy(a).cuda().bfloat16(), torch.from_numpy(b).cuda().bfloat16(), NN)   # 512 TMEM columns
    gpu.sync()
    assert rel_err(got.cpu().numpy(), orc.matmul(a, b)) < BF16_TOL
    with pytest.raises(asca_b200.AscaError):
        gpu._call("asca_selftest_wait_timeout", gpu._ctx, ctypes.c_int64(10 ** 10), None, None)   # limit out of range


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n", [(2304, 520, 2560), (2400, 2048, 2504), (4096, 64, 1288), (2560, 4104, 2304)])
def test_bf16_gemm_cta_pair_tiles(gpu, m, k, n):
    """Dense products large enough for the 256 x 256 tiles of CTA pairs (cta_group::2): all three operand forms,
    ragged edges in M, N and K, bias and accumulate, against an f64 product of the same bf16 operands."""
    import torch
    from asca_b200 import ops, NN, TN, NT

    g = torch.Generator(device="cuda").manual_seed(m + k + n)
    a = torch.randn(m, k, generator=g, device="cuda").bfloat16()
    b = (torch.randn(k, n, generator=g, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(n, generator=g, device="cuda")
    c0 = torch.randn(m, n, generator=g, device="cuda")
    ref = a.double() @ b.double()
    scale = float(ref.abs().max())

    def err(x, r):
        return float((x.double() - r).abs().max()) / scale

    got = ops.gemm(gpu, a, b, NN)
    got_nt = ops.gemm(gpu, a, b.t().contiguous(), NT)
    got_tn = ops.gemm(gpu, a.t().contiguous(), b, TN) if m % 8 == 0 else None
    out = c0.clone()
    ops.gemm(gpu, a, b, NN, bias=bias, out=out, accumulate=True)
    again = ops.gemm(gpu, a, b, NN)
    gpu.sync()
    assert err(got, ref) < 1e-5
    assert err(got_nt, ref) < 1e-5
    if got_tn is not None:
        assert err(got_tn, ref) < 1e-5
    assert err(out, ref + bias.double() + c0.double()) < 1e-5
    assert torch.equal(got, again)
