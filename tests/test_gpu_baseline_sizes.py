"""Parity at the sizes the benchmark quotes speeds for (the baseline configuration list), through the C ABI.

The small-shape tests prove the arithmetic; these prove the code paths that only large shapes reach: 64-chunk
chains, the wide-tile and grouped tensor-core products with a skewed expert load, the 12-block bf16 decode and
the 1.3B-class block. Where the CPU oracle cannot afford the whole workload the device runs it whole and the
oracle checks an exact sub-problem of it (a chain, an expert's rows, a slice of an expert's hidden features --
each independent of the rest by the math, so nothing is approximated).

Tolerances are the contract's: 1e-5 relative in f32 mode, 2e-2 in bf16 mode against the f32 CPU path on the
same, UNROUNDED inputs (error metric max|a-b| / max|ref| per tensor, rust/src/main.rs:814-820); integer results
bit-exact. The bf16 cases also run the oracle on the bf16-rounded inputs: that comparison isolates what the
kernels add (accumulation order, rounded intermediates) from what the input rounding alone costs.
Inputs at these sizes are drawn with numpy's or torch's seeded generators (the reference's scalar generator
would take minutes for 1e9 numbers); both sides see the same arrays.
"""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
BF16_TOL = 2e-2


def _chain_inputs(seed, B, T, H, dh):
    """The isolated-op distributions: q,k L2-normalised N(0,1); v, dO N(0,1); alpha = sigmoid(N(2,.5)); beta = sigmoid(N(0,1))."""
    g = np.random.default_rng(seed)
    n, d = B * T, H * dh
    q = g.standard_normal((n, H, dh), dtype=np.float32)
    k = g.standard_normal((n, H, dh), dtype=np.float32)
    qn = np.linalg.norm(q, axis=-1).astype(np.float32)
    kn = np.linalg.norm(k, axis=-1).astype(np.float32)
    q = (q / qn[..., None]).reshape(n, d).astype(np.float32)
    k = (k / kn[..., None]).reshape(n, d).astype(np.float32)
    v = g.standard_normal((n, d), dtype=np.float32)
    d_o = g.standard_normal((n, d), dtype=np.float32)
    alpha = (1 / (1 + np.exp(-(2 + 0.5 * g.standard_normal((n, H)))))).astype(np.float32)
    beta = (1 / (1 + np.exp(-g.standard_normal((n, H))))).astype(np.float32)
    return q, k, v, alpha, beta, qn, kn, d_o


def _device_normal(seed, n, scale=0.02):
    """n seeded N(0, scale) numbers drawn on the device and brought to the host (a billion of them in a second)."""
    import torch

    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(n, generator=g, device="cuda") * scale).cpu().numpy()


def _blocks(d_qkv, d_gate, d, H):
    return {"dq": d_qkv[:, :d], "dk": d_qkv[:, d:2 * d], "dv": d_qkv[:, 2 * d:], "d_gate alpha": d_gate[:, :H],
            "d_gate beta": d_gate[:, H:]}


# ------------------------------------------------------------------ isolated delta op: T 4096, dh 128, chunk 64
def test_delta_f32_full_length_chains(orc, gpu):
    """f32 mode at the benchmark's sequence length: outputs, final state, every one of the 64 chunk checkpoints and
    all five gradient blocks of two 4096-token chains."""
    import torch
    from asca_b200 import ops

    B, T, H, dh = 1, 4096, 2, 128
    d = H * dh
    arrs = _chain_inputs(21, B, T, H, dh)
    o_ref, sfin_ref, st_ref = orc.delta_scan(*arrs[:5], B, T, H, dh, want_states=True)
    dqkv_ref, dgate_ref = orc.delta_bptt(*arrs, B, T, H, dh)
    q, k, v, alpha, beta, qn, kn, d_o = (torch.from_numpy(a).cuda() for a in arrs)
    o, s_final, ckpt = ops.delta_fwd(gpu, q, k, v, alpha, beta, B, T, H, dh, chunk=64, want_final=True)
    d_qkv, d_gate = ops.delta_bwd(gpu, q, k, v, alpha, beta, qn, kn, d_o, ckpt, B, T, H, dh, chunk=64)
    gpu.sync()
    assert rel_err(o.cpu().numpy(), o_ref) < F32_TOL
    assert rel_err(s_final.cpu().numpy(), sfin_ref) < F32_TOL
    ck = ckpt.view(B, H, T // 64, dh, dh).cpu().numpy()
    want = st_ref[:, :, 0:T:64].transpose(1, 0, 2, 3, 4)
    for c in range(T // 64):
        assert rel_err(ck[:, :, c], want[:, :, c]) < F32_TOL or np.abs(want[:, :, c]).max() == 0, f"checkpoint {c}"
    got = _blocks(d_qkv.cpu().numpy(), d_gate.cpu().numpy(), d, H)
    for name, w in _blocks(dqkv_ref, dgate_ref, d, H).items():
        assert rel_err(got[name], w) < F32_TOL, name


def test_delta_bf16_tensor_core_full_length_chains(orc, gpu):
    """bf16 mode (tcgen05 chunk kernels) at the benchmark's sequence length, against the f32 oracle on the
    unrounded inputs (the contract) and on the rounded inputs (the kernels' own error)."""
    import torch
    from asca_b200 import ops

    B, T, H, dh = 1, 4096, 2, 128
    d = H * dh
    arrs = _chain_inputs(22, B, T, H, dh)
    q, k, v, alpha, beta, qn, kn, d_o = (torch.from_numpy(a).cuda() for a in arrs)
    q16, k16, v16, do16 = (x.bfloat16() for x in (q, k, v, d_o))
    o, s_final, ckpt = ops.delta_fwd(gpu, q16, k16, v16, alpha, beta, B, T, H, dh, chunk=64, want_final=True)
    d_qkv, d_gate = ops.delta_bwd(gpu, q16, k16, v16, alpha, beta, qn, kn, do16, ckpt, B, T, H, dh, chunk=64)
    gpu.sync()
    n_ck = T // 64
    ck = ckpt.view(torch.bfloat16)[: B * H * n_ck * dh * dh].view(B, H, n_ck, dh, dh).float().cpu().numpy()
    got = _blocks(d_qkv.cpu().numpy(), d_gate.cpu().numpy(), d, H)
    rounded = [x.float().cpu().numpy() for x in (q16, k16, v16)] + list(arrs[3:7]) + [do16.float().cpu().numpy()]
    for label, inp in (("unrounded", arrs), ("rounded", rounded)):
        o_ref, sfin_ref, st_ref = orc.delta_scan(*inp[:5], B, T, H, dh, want_states=True)
        dqkv_ref, dgate_ref = orc.delta_bptt(*inp, B, T, H, dh)
        assert rel_err(o.float().cpu().numpy(), o_ref) < BF16_TOL, label
        assert rel_err(s_final.cpu().numpy(), sfin_ref) < BF16_TOL, label
        want = st_ref[:, :, 0:T:64].transpose(1, 0, 2, 3, 4)
        for c in range(1, n_ck):
            assert rel_err(ck[:, :, c], want[:, :, c]) < BF16_TOL, f"{label}: checkpoint {c}"
        assert np.abs(ck[:, :, 0]).max() == 0
        for name, w in _blocks(dqkv_ref, dgate_ref, d, H).items():
            assert rel_err(got[name], w) < BF16_TOL, f"{label}: {name}"


# ------------------------------------------------------------------ isolated hash-MoE layer: 65,536 Zipf tokens, d 1024, F 4096, E 64
def _zipf_ids(seed, n, s=1.1):
    w = 1.0 / np.arange(1, 257) ** s
    cdf = np.cumsum(w) / w.sum()
    u = np.random.default_rng(seed).random(n)
    return np.minimum(np.searchsorted(cdf, u), 255).astype(np.uint32)


def test_moe_layer_at_the_skewed_benchmark_load(orc, gpu):
    """The whole layer runs on the device in bf16 mode (dispatch, both grouped products, combine; the four grouped
    gradient products and the column sums). The dispatch is compared bit for bit over all 65,536 tokens. The FFN is
    compared on the hottest expert (about a fifth of the tokens), the coldest (a few dozen) and two in between:
    outputs and input gradients on rows of each, weight and bias gradients on each expert's own block. For the
    hottest expert the weight gradients are checked on 128 of its 4096 hidden features over ALL its rows (hidden
    features are independent of one another given dout, so the sub-problem is exact)."""
    import torch
    from asca_b200 import ops

    n, d, F, E = 65536, 1024, 4096, 64
    ids = _zipf_ids(3, n)
    c = lambda a: torch.from_numpy(a).cuda()  # noqa: E731
    perm, offsets, route = ops.moe_dispatch(gpu, c(ids.view(np.int32)), E, want_route=True)
    p_ref, o_ref, r_ref = orc.moe_dispatch(ids, E)
    assert np.array_equal(perm.cpu().numpy(), p_ref) and np.array_equal(offsets.cpu().numpy(), o_ref)
    assert np.array_equal(route.cpu().numpy(), r_ref)
    load = np.diff(o_ref)
    assert load.max() > 0.15 * n and load.min() > 0

    g = np.random.default_rng(4)
    x = g.standard_normal((n, d), dtype=np.float32)
    xn = (x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-6)).astype(np.float32)
    del x
    dout = g.standard_normal((n, d), dtype=np.float32)
    gw = torch.Generator(device="cuda").manual_seed(5)
    tw1 = (torch.randn((d, E * F), generator=gw, device="cuda") * 0.02).bfloat16()
    tw2 = (torch.randn((E * F, d), generator=gw, device="cuda") * 0.02).bfloat16()
    b1 = (0.02 * g.standard_normal(E * F)).astype(np.float32)
    b2 = (0.02 * g.standard_normal(d)).astype(np.float32)
    txn = c(xn).bfloat16()
    out, pre_p, hid_p = ops.moe_fwd(gpu, txn, tw1, c(b1), tw2, c(b2), perm, offsets, F, E)
    d_w1, d_b1, d_w2, d_b2, dxn = ops.moe_bwd(gpu, txn, tw1, tw2, pre_p, hid_p, c(dout), perm, offsets, F, E)
    gpu.sync()
    out, dxn = out.cpu().numpy(), dxn.cpu().numpy()

    order = np.argsort(load)
    picks = {"hottest": int(order[-1]), "coldest": int(order[0]), "mid": int(order[E // 2]), "upper": int(order[3 * E // 4])}
    one = np.zeros(1, np.uint32)      # with a single expert every id routes to expert 0
    for label, e in picks.items():
        rows = p_ref[o_ref[e]:o_ref[e + 1]]
        w1e = tw1[:, e * F:(e + 1) * F].float().cpu().numpy().copy()
        w2e = tw2[e * F:(e + 1) * F].float().cpu().numpy().copy()
        b1e = b1[e * F:(e + 1) * F].copy()
        if label == "hottest":
            # (1) all features on a row subset: outputs and input gradients
            sub = rows[:: max(1, len(rows) // 384)]
            ids0 = np.repeat(one, len(sub))
            o_e, pre_e, hid_e = orc.moe_ffn_forward(xn[sub], w1e, b1e, w2e, b2, ids0, F, 1, want_cache=True)
            g_e = orc.moe_ffn_backward(xn[sub], w1e, w2e, pre_e, hid_e, ids0, dout[sub], F, 1)
            assert rel_err(out[sub], o_e) < BF16_TOL, label
            assert rel_err(dxn[sub], g_e[4]) < BF16_TOL, label
            # (2) all rows on a feature subset: weight and bias gradients of those features
            J = np.r_[0:64, F - 64:F]
            ids0 = np.repeat(one, len(rows))
            w1j, w2j, b1j = np.ascontiguousarray(w1e[:, J]), np.ascontiguousarray(w2e[J]), b1e[J].copy()
            _, pre_j, hid_j = orc.moe_ffn_forward(xn[rows], w1j, b1j, w2j, b2, ids0, len(J), 1, want_cache=True)
            gj = orc.moe_ffn_backward(xn[rows], w1j, w2j, pre_j, hid_j, ids0, dout[rows], len(J), 1)
            cols = torch.from_numpy(e * F + J).cuda()
            assert rel_err(d_w1[:, cols].cpu().numpy(), gj[0]) < BF16_TOL, label
            assert rel_err(d_b1[cols].cpu().numpy(), gj[1]) < BF16_TOL, label
            assert rel_err(d_w2[cols].cpu().numpy(), gj[2]) < BF16_TOL, label
            continue
        ids0 = np.repeat(one, len(rows))
        o_e, pre_e, hid_e = orc.moe_ffn_forward(xn[rows], w1e, b1e, w2e, b2, ids0, F, 1, want_cache=True)
        g_e = orc.moe_ffn_backward(xn[rows], w1e, w2e, pre_e, hid_e, ids0, dout[rows], F, 1)
        assert rel_err(out[rows], o_e) < BF16_TOL, label
        assert rel_err(dxn[rows], g_e[4]) < BF16_TOL, label
        assert rel_err(d_w1[:, e * F:(e + 1) * F].cpu().numpy(), g_e[0]) < BF16_TOL, label
        assert rel_err(d_b1[e * F:(e + 1) * F].cpu().numpy(), g_e[1]) < BF16_TOL, label
        assert rel_err(d_w2[e * F:(e + 1) * F].cpu().numpy(), g_e[2]) < BF16_TOL, label
    # the shared output bias gradient is the column sum of dout over every token (rust/src/model.rs:425-431)
    assert rel_err(d_b2.cpu().numpy(), dout.astype(np.float64).sum(axis=0)) < 1e-5


# ------------------------------------------------------------------ ~125M decode configuration, bf16
def test_decode_configuration_teacher_forced_logits(orc, gpu):
    """12 blocks, d 768, 12 heads of 64, 16 experts of 768 -> 3072 -> 768, bf16 weights: 64 streams x 16 steps with
    the tokens forced, logits of every step against the f32 oracle's forward over the same 64 sequences (stepping
    equals the full forward -- rust/tests/decode_parity.rs -- and the oracle passes that gate). Greedy agreement is
    a separate statement: wherever the oracle's best logit leads the runner-up by more than twice the largest
    logit error seen, the device's argmax must be the oracle's."""
    import asca_b200

    cfg = (256, 768, 12, 12, 16, 3072)
    streams, steps = 64, 16
    ref = orc.Model(*cfg)
    ref.params[:] = _device_normal(6, ref.n)
    prompts = np.random.default_rng(7).integers(0, 256, (streams, steps), dtype=np.uint32)
    logits_ref = ref.forward(prompts.reshape(-1).copy(), streams).reshape(streams, steps, 256)
    dev = asca_b200.Model(gpu, *cfg)
    dev.set_params(ref.params)
    dev.set_compute(asca_b200.BF16)
    state = dev.new_decode_state(streams)
    worst_row, worst_abs, agree, decided = 0.0, 0.0, 0, 0
    got_all = np.empty_like(logits_ref)
    nxt_all = np.empty((streams, steps), np.uint32)
    for t in range(steps):
        logits, nxt = dev.decode_step(state, prompts[:, t].copy())
        got_all[:, t], nxt_all[:, t] = logits, nxt
        assert rel_err(logits, logits_ref[:, t]) < BF16_TOL, f"step {t}"
        for s in range(streams):
            worst_row = max(worst_row, rel_err(logits[s], logits_ref[s, t]))
        worst_abs = max(worst_abs, float(np.abs(logits - logits_ref[:, t]).max()))
    assert worst_row < BF16_TOL
    top2 = np.sort(logits_ref, axis=-1)[..., -2:]
    clear = (top2[..., 1] - top2[..., 0]) > 2 * worst_abs
    same = nxt_all == logits_ref.argmax(-1)
    assert clear.sum() > 0 and bool(same[clear].all())
    print(f"decode configuration: worst per-row logit error {worst_row:.2e}; greedy token agreement "
          f"{same.mean():.4f} over {same.size} steps ({int(clear.sum())} with a clear margin, all equal)")
    dev.free()


# ------------------------------------------------------------------ one block of the 1.3B-class training configuration, bf16
def test_training_configuration_block_loss_and_every_gradient(orc, gpu):
    """d 2048, 16 heads of 128, 64 experts of 2048 -> 4096 -> 2048, one block, one sequence of 512 random bytes in
    bf16 compute mode: loss, logits and every gradient tensor (1.09 B numbers) against the f32 oracle."""
    import asca_b200

    cfg = (256, 2048, 16, 1, 64, 4096)
    ref = orc.Model(*cfg)
    ref.params[:] = _device_normal(8, ref.n)
    B, T = 1, 512
    ids = np.random.default_rng(9).integers(0, 256, B * T, dtype=np.uint32)
    tg = np.roll(ids, -1).astype(np.uint32)
    loss_ref, g_ref, logits_ref = ref.forward_backward(ids, tg, B, want_logits=True)
    dev = asca_b200.Model(gpu, *cfg)
    dev.set_params(ref.params)
    dev.set_compute(asca_b200.BF16)
    dev.zero_grads()
    loss, logits = dev.forward_backward(ids, tg, B, want_logits=True)
    _, g = dev.get()
    dev.free()
    assert abs(loss - loss_ref) / abs(loss_ref) < BF16_TOL
    assert rel_err(logits, logits_ref) < BF16_TOL
    errs = {}
    for name in ref.names:
        a, b = ref.tensor(name, g), ref.tensor(name, g_ref)
        if np.abs(b).max() == 0:
            assert np.abs(a).max() == 0, name
        else:
            errs[name] = float(np.abs(a - b).max() / np.abs(b).max())
    print("training configuration block, gradient errors:", {k: f"{v:.2e}" for k, v in errs.items()})
    bad = {k: v for k, v in errs.items() if not v < BF16_TOL}
    assert not bad, bad
