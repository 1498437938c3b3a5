"""The reference's own self-consistency gates, re-run on the CPU oracle (no GPU needed).

The reference ships no golden vectors for this path; these gates are what pins its results:
finite-difference gradcheck of the DeltaBlock (rust/tests/gradcheck.rs) and of the whole model
(rust/tests/gradcheck_model.rs), batch parity (rust/tests/batch_parity.rs), decode parity
(rust/tests/decode_parity.rs), the independent scalar scan of `asca gpu`
(rust/src/main.rs:887-928), and the fp64 recurrent == chunked identity (docs/SPEC_V2.md:63-65).
"""
import numpy as np
import pytest

from conftest import rel_err
import chunkref

TINY = dict(vocab=256, d=64, H=4, L=2, E=8, F=128)  # rust/src/model.rs:32-41


def test_rng_is_deterministic_and_sane(orc):
    a = orc.Rng(7).normal(10000)
    b = orc.Rng(7).normal(10000)
    assert np.array_equal(a, b)
    assert abs(float(a.mean())) < 0.05 and abs(float(a.std()) - 1.0) < 0.05
    u = orc.Rng(1).uniform(10000)
    assert u.min() >= 0.0 and u.max() < 1.0
    # xorshift128+ first outputs for seed 0 follow from the constants in tensor.rs:307-320
    s0 = (0 * 0x9E3779B97F4A7C15) | 1
    s1 = ((0 ^ 0xDEADBEEFCAFEF00D) * 0xBF58476D1CE4E5B9 | 1) & (2**64 - 1)
    x, y = s0, s1
    x ^= (x << 23) & (2**64 - 1)
    n1 = x ^ y ^ (x >> 17) ^ (y >> 26)
    first = (n1 + y) & (2**64 - 1)
    assert int(orc.Rng(0).below(2**32, 1)[0]) == first % 2**32


def test_hash_route_matches_formula_and_load_stats(orc):
    def ref(i, e):
        h = (i * 0x9E3779B1) & 0xFFFFFFFF
        h ^= h >> 15
        h = (h * 0x85EBCA6B) & 0xFFFFFFFF
        h ^= h >> 13
        return h % e

    for e in (1, 2, 3, 4, 8, 16, 64, 100):
        for i in list(range(256)) + [65535, 2**31, 2**32 - 1]:
            assert orc.hash_route(i, e) == ref(i, e)
    # ids per expert over the byte vocabulary: E=4 58-73, E=16 10-20, E=64 1-9, none empty
    for e, lo, hi in ((4, 58, 73), (16, 10, 20), (64, 1, 9)):
        cnt = np.bincount([orc.hash_route(i, e) for i in range(256)], minlength=e)
        assert cnt.min() == lo and cnt.max() == hi


def test_dispatch_is_stable_bucket_concat(orc):
    rng = orc.Rng(2)
    ids = rng.below(256, 1000)
    perm, off, route = orc.moe_dispatch(ids, 8)
    buckets = [[] for _ in range(8)]
    for t, i in enumerate(ids):
        buckets[orc.hash_route(int(i), 8)].append(t)
    assert perm.tolist() == [t for b in buckets for t in b]
    assert off.tolist() == np.concatenate([[0], np.cumsum([len(b) for b in buckets])]).tolist()
    assert all(route[t] == e for e, b in enumerate(buckets) for t in b)


def test_scan_matches_independent_scalar_scan(orc):
    # shapes of `asca gpu` (rust/src/main.rs:853-952)
    B, T, H, dh = 3, 24, 4, 16
    rng = orc.Rng(21)
    q, k, v = (rng.normal((B * T, H * dh)) for _ in range(3))
    alpha = 1 / (1 + np.exp(-rng.normal((B * T, H)))).astype(np.float32)
    beta = 1 / (1 + np.exp(-rng.normal((B * T, H)))).astype(np.float32)
    o, s_final, states = orc.delta_scan(q, k, v, alpha, beta, B, T, H, dh, want_states=True)
    o2 = orc.delta_scan_scalar(q, k, v, alpha, beta, B, T, H, dh)
    assert rel_err(o, o2) < 1e-6
    # one-thread-per-head partitioning gives the same numbers
    o3, _ = orc.delta_scan(q, k, v, alpha, beta, B, T, H, dh, per_chain_threads=False)
    assert np.array_equal(o, o3)
    # sequence isolation: batch=3 equals three batch=1 runs (rust/src/main.rs:954-981)
    for b in range(B):
        s = slice(b * T, (b + 1) * T)
        ob, sf = orc.delta_scan(q[s].copy(), k[s].copy(), v[s].copy(), alpha[s].copy(), beta[s].copy(), 1, T, H, dh)
        assert np.array_equal(ob, o[s])
        assert np.array_equal(sf[0], s_final[b])
    assert np.array_equal(states[:, :, T].transpose(1, 0, 2, 3), s_final)


def test_scan_and_bptt_match_fp64(orc):
    B, T, H, dh = 2, 40, 2, 16
    rng = orc.Rng(5)
    d = H * dh
    q, k, v, d_o = (rng.normal((B * T, d)) for _ in range(4))
    for m in (q, k):
        m4 = m.reshape(B * T, H, dh)
        m4 /= np.linalg.norm(m4, axis=-1, keepdims=True)
    alpha = (1 / (1 + np.exp(-(2 + 0.5 * rng.normal((B * T, H)))))).astype(np.float32)
    beta = (1 / (1 + np.exp(-rng.normal((B * T, H))))).astype(np.float32)
    ones = np.ones((B * T, H), np.float32)
    o, _ = orc.delta_scan(q, k, v, alpha, beta, B, T, H, dh)
    d_qkv, d_gate = orc.delta_bptt(q, k, v, alpha, beta, ones, ones, d_o, B, T, H, dh)
    for b in range(B):
        for h in range(H):
            r, c = slice(b * T, (b + 1) * T), slice(h * dh, (h + 1) * dh)
            a64 = [x.astype(np.float64) for x in (q[r, c], k[r, c], v[r, c], alpha[r, h], beta[r, h])]
            o64, _, _ = chunkref.recurrent_forward(*a64)
            assert rel_err(o[r, c], o64) < 2e-6
            dq, dk, dv, da, db, _ = chunkref.recurrent_backward(*a64, d_o[r, c].astype(np.float64))
            # undo nothing: norms were passed as 1, so d_qkv = (g - y<y,g>) for q,k and dv as is
            qh, kh = a64[0], a64[1]
            dq_n = dq - qh * np.sum(qh * dq, axis=1, keepdims=True)
            dk_n = dk - kh * np.sum(kh * dk, axis=1, keepdims=True)
            assert rel_err(d_qkv[r, c], dq_n) < 2e-5
            assert rel_err(d_qkv[r, d + h * dh: d + (h + 1) * dh], dk_n) < 2e-5
            assert rel_err(d_qkv[r, 2 * d + h * dh: 2 * d + (h + 1) * dh], dv) < 2e-5
            assert rel_err(d_gate[r, h], da * a64[3] * (1 - a64[3])) < 2e-5
            assert rel_err(d_gate[r, H + h], db * a64[4] * (1 - a64[4])) < 2e-5


def test_fp64_chunked_equals_recurrent():
    rs = np.random.RandomState(0)
    T, dh, C = 96, 16, 32
    q, k, v, d_o = (rs.randn(T, dh) for _ in range(4))
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    k /= np.linalg.norm(k, axis=1, keepdims=True)
    alpha = 1 / (1 + np.exp(-(2 + 0.5 * rs.randn(T))))
    beta = 1 / (1 + np.exp(-rs.randn(T)))
    o1, S1, _ = chunkref.recurrent_forward(q, k, v, alpha, beta)
    o2, S2, _ = chunkref.chunked_forward(q, k, v, alpha, beta, C)
    assert np.max(np.abs(o1 - o2)) < 1e-13 and np.max(np.abs(S1 - S2)) < 1e-13
    g1 = chunkref.recurrent_backward(q, k, v, alpha, beta, d_o)[:5]
    g2 = chunkref.chunked_backward(q, k, v, alpha, beta, d_o, C)
    for a, b in zip(g1, g2):
        assert np.max(np.abs(a - b)) / np.max(np.abs(a)) < 1e-11
    # ragged tail (T not a multiple of C)
    o3, S3, _ = chunkref.chunked_forward(q[:70], k[:70], v[:70], alpha[:70], beta[:70], C)
    assert np.max(np.abs(o1[:70] - o3)) < 1e-13


def _loss_of(block, x, dy):
    y, c = block.forward(x, 1)
    block.free(c)
    # serial f32 sum in row-major order (rust/tests/gradcheck.rs:6-15)
    l = np.float32(0)
    for val in (y * dy).ravel():
        l = np.float32(l + val)
    return float(l)


def test_gradcheck_delta_block(orc):
    rng = orc.Rng(7)
    block = orc.DeltaBlock(16, 2, rng)
    T = 12
    x = rng.normal((T, 16))
    dy = rng.normal((T, 16))
    y, cache = block.forward(x, 1)
    dx, grads = block.backward(cache, dy)
    block.free(cache)
    eps = 1e-3
    worst = 0.0
    for name in block.NAMES:
        p = getattr(block, name).reshape(-1)
        g = grads[name].reshape(-1)
        step = max(p.size // 6, 1)
        scale = max(float(np.abs(g).max()), 1e-3)
        for i in range(0, p.size, step):
            orig = p[i]
            p[i] = orig + np.float32(eps)
            lp = _loss_of(block, x, dy)
            p[i] = orig - np.float32(eps)
            lm = _loss_of(block, x, dy)
            p[i] = orig
            num = (lp - lm) / (2 * eps)
            tol = 2e-2 * max(abs(float(g[i])), abs(num)) + 1e-3 * scale
            worst = max(worst, abs(float(g[i]) - num) / tol)
    scale = max(float(np.abs(dx).max()), 1e-3)
    xf = x.reshape(-1)
    for i in range(xf.size):
        orig = xf[i]
        xf[i] = orig + np.float32(eps)
        lp = _loss_of(block, x, dy)
        xf[i] = orig - np.float32(eps)
        lm = _loss_of(block, x, dy)
        xf[i] = orig
        num = (lp - lm) / (2 * eps)
        a = float(dx.reshape(-1)[i])
        tol = 2e-2 * max(abs(a), abs(num)) + 1e-3 * scale
        worst = max(worst, abs(a - num) / tol)
    assert worst <= 1.0, worst


def test_gradcheck_model(orc):
    rng = orc.Rng(11)
    m = orc.Model(256, 16, 2, 1, 2, 16)
    m.init_reference(rng)
    ids = rng.below(256, 10)
    tg = rng.below(256, 10)
    loss, grads = m.forward_backward(ids, tg, 1)
    assert 4.0 < loss < 7.5  # ~ln(256) at init
    eps = 3e-4
    ulp = max(abs(loss), 1.0) * np.finfo(np.float32).eps
    noise = 4.0 * ulp / (2 * eps)
    worst, checked = 0.0, 0
    for name in m.names:
        g = m.tensor(name, grads)
        p = m.tensor(name)
        order = np.argsort(-np.abs(g), kind="stable")[:4]
        for i in order:
            a = float(g[i])
            if abs(a) < 3 * noise:
                continue
            orig = p[i]
            p[i] = orig + np.float32(eps)
            lp = m.loss(ids, tg)
            p[i] = orig - np.float32(eps)
            lm = m.loss(ids, tg)
            p[i] = orig
            num = (lp - lm) / (2 * eps)
            worst = max(worst, abs(a - num) / (0.05 * abs(a) + noise))
            checked += 1
    assert checked >= 10
    assert worst <= 1.0, worst


def test_batch_parity(orc):
    rng = orc.Rng(5)
    batch, seq = 4, 12
    ids = rng.below(256, batch * seq)
    tg = rng.below(256, batch * seq)
    m = orc.Model(**TINY)
    m.init_reference(orc.Rng(9))
    g1 = np.zeros(m.n, np.float32)
    loss1 = 0.0
    for b in range(batch):
        s = slice(b * seq, (b + 1) * seq)
        l, _ = m.forward_backward(ids[s].copy(), tg[s].copy(), 1, grads=g1)
        loss1 += l
    loss1 /= batch
    g1 /= batch
    lossb, gb = m.forward_backward(ids, tg, batch)
    assert abs(loss1 - lossb) / max(abs(loss1), abs(lossb), 1e-6) <= 1e-5
    for name in m.names:
        assert rel_err(m.tensor(name, gb), m.tensor(name, g1)) <= 2e-4, name


def test_decode_parity(orc):
    ids = orc.Rng(3).below(256, 24)
    m = orc.Model(**TINY)
    m.init_reference(orc.Rng(17))
    logits = m.forward(ids, 1)
    st = m.new_decode_state()
    worst = 0.0
    for t, tok in enumerate(ids):
        sl = m.step(int(tok), st)
        worst = max(worst, float(np.abs(sl[0] - logits[t]).max()))
    assert worst / max(float(np.abs(logits).max()), 1e-9) <= 1e-4
    assert st.size == 2 * 4 * 16 * 16  # constant state: L*H*dh*dh floats


def test_param_count_matches_config1(orc):
    # BASELINE config 1: vocab 256, d 64, H 4, L 2, E 4, F 256 -> 331,408 parameters
    assert orc.Model(256, 64, 4, 2, 4, 256).n == 331408
    assert orc.Model(**TINY).n == 331408


def test_adamw_counter_advances_per_tensor(orc):
    m = orc.Model(256, 16, 2, 1, 2, 16)
    m.init_reference(orc.Rng(1))
    g = orc.Rng(2).normal(m.n, 0.1)
    mm = np.zeros(m.n, np.float32)
    vv = np.zeros(m.n, np.float32)
    p0 = m.params.copy()
    cnt = m.adamw_step(g, mm, vv, 0, 3e-3)
    assert cnt == len(m.names) == 12
    # tensor i uses t = i+1 (rust/src/tensor.rs:393): check against a direct numpy statement
    for i, name in enumerate(m.names):
        lr_t, eps_t, wd_eff = orc.adamw_scalars(3e-3, 0.9, 0.95, 1e-8, 0.01, i + 1)
        gi = m.tensor(name, g).astype(np.float32)
        m1 = np.float32(0.1) * gi
        v1 = (np.float32(1) - np.float32(0.95)) * gi * gi
        p = m.tensor(name, p0).copy()
        p -= np.float32(wd_eff) * p
        p -= np.float32(lr_t) * (m1 / (np.sqrt(v1) + np.float32(eps_t)))
        assert rel_err(m.tensor(name), p) < 1e-6, name


def test_moe_ffn_pieces_agree_with_layer(orc):
    rng = orc.Rng(4)
    n, d, F, E = 64, 16, 32, 4
    x = rng.normal((n, d))
    w1 = rng.normal((d, E * F), 0.25)
    b1 = rng.normal(E * F, 0.1)
    w2 = rng.normal((E * F, d), 0.2)
    b2 = rng.normal(d, 0.1)
    ids = rng.below(256, n)
    dout = rng.normal((n, d))
    out, d_w1, d_b1, d_w2, d_b2, dx = orc.moe_forward_backward(x, w1, b1, w2, b2, ids, dout, F, E)
    xn, _ = orc.rmsnorm(x)
    out2, pre, hid = orc.moe_ffn_forward(xn, w1, b1, w2, b2, ids, F, E, want_cache=True)
    assert np.array_equal(out, out2)
    g = orc.moe_ffn_backward(xn, w1, w2, pre, hid, ids, dout, F, E)
    assert np.array_equal(g[0], d_w1) and np.array_equal(g[2], d_w2)
    assert np.array_equal(orc.rmsnorm_bwd(x, g[4]), dx)
    # against a direct fp64 statement
    route = np.array([orc.hash_route(int(i), E) for i in ids])
    ref = np.zeros((n, d))
    for t in range(n):
        e = route[t]
        p = xn[t].astype(np.float64) @ w1[:, e * F:(e + 1) * F] + b1[e * F:(e + 1) * F]
        ref[t] = (p / (1 + np.exp(-p))) @ w2[e * F:(e + 1) * F] + b2
    assert rel_err(out, ref) < 2e-6
