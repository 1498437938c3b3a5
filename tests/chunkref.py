"""fp64 numpy statements of the gated delta rule: the per-step recurrence of the reference
(rust/src/delta.rs:281-315, :485-572) and the chunked WY/UT forms the CUDA kernels use
(forward formulas as in docs/SPEC_V2.md:50-69 of the reference; the chunk backward is derived
from them). Test helper only."""
import numpy as np


def recurrent_forward(q, k, v, alpha, beta, S0=None):
    """One chain. q,k,v: (T, dh); alpha,beta: (T,). Returns o (T, dh), S_T, list of S_t."""
    T, dh = q.shape
    S = np.zeros((dh, dh)) if S0 is None else S0.copy()
    o = np.zeros((T, dh))
    hist = [S.copy()]
    for t in range(T):
        sk = S.T @ k[t]
        u = beta[t] * (v[t] - alpha[t] * sk)
        S = alpha[t] * S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
        hist.append(S.copy())
    return o, S, hist


def recurrent_backward(q, k, v, alpha, beta, d_o, dS_T=None):
    """BPTT of one chain in fp64; returns dq, dk, dv, dalpha, dbeta, dS0."""
    T, dh = q.shape
    _, _, hist = recurrent_forward(q, k, v, alpha, beta)
    dS = np.zeros((dh, dh)) if dS_T is None else dS_T.copy()
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    da = np.zeros(T)
    db = np.zeros(T)
    for t in reversed(range(T)):
        S_t, S_p = hist[t + 1], hist[t]
        dq[t] = S_t @ d_o[t]
        dS = dS + np.outer(q[t], d_o[t])
        sk = S_p.T @ k[t]
        u = beta[t] * (v[t] - alpha[t] * sk)
        du = dS.T @ k[t]
        da[t] = np.sum(dS * S_p) - beta[t] * np.dot(du, sk)
        db[t] = np.dot(du, v[t] - alpha[t] * sk)
        dv[t] = beta[t] * du
        dsk = -beta[t] * alpha[t] * du
        dk[t] = dS @ u + S_p @ dsk
        dS = alpha[t] * dS + np.outer(k[t], dsk)
    return dq, dk, dv, da, db, dS


def chunk_forward(Q, K, V, alpha, beta, S0):
    """One chunk of C steps from state S0. Returns O, S_C and the intermediates."""
    g = np.cumsum(np.log(alpha))
    gam = np.exp(g)
    C = len(g)
    Gam = np.exp(np.minimum(g[:, None] - g[None, :], 0.0)) * (np.arange(C)[:, None] >= np.arange(C)[None, :])
    Kg = gam[:, None] * K
    R = beta[:, None] * (V - Kg @ S0)
    L = np.tril(beta[:, None] * Gam * (K @ K.T), -1)
    U = np.linalg.solve(np.eye(C) + L, R)
    A = np.tril(Gam * (Q @ K.T))
    O = (gam[:, None] * Q) @ S0 + A @ U
    W = np.exp(g[-1] - g)[:, None] * K
    S_C = gam[-1] * S0 + W.T @ U
    return O, S_C, dict(g=g, gam=gam, Gam=Gam, Kg=Kg, R=R, L=L, U=U, A=A, W=W)


def chunked_forward(q, k, v, alpha, beta, C):
    T, dh = q.shape
    S = np.zeros((dh, dh))
    o = np.zeros_like(q)
    bounds = [S.copy()]
    for c0 in range(0, T, C):
        s = slice(c0, min(T, c0 + C))
        o[s], S, _ = chunk_forward(q[s], k[s], v[s], alpha[s], beta[s], S)
        bounds.append(S.copy())
    return o, S, bounds


def chunk_backward(Q, K, V, alpha, beta, S0, dO, dS_C):
    """Backward of one chunk. Returns dQ, dK, dV, dlogalpha-based d_alpha, d_beta, dS0."""
    O, S_C, m = chunk_forward(Q, K, V, alpha, beta, S0)
    g, gam, Gam, Kg, L, U, A, W = m["g"], m["gam"], m["Gam"], m["Kg"], m["L"], m["U"], m["A"], m["W"]
    C = len(g)
    Z = V - Kg @ S0
    dU = A.T @ dO + W @ dS_C
    dR = np.linalg.solve((np.eye(C) + L).T, dU)
    dL = -np.tril(dR @ U.T, -1)
    dV = beta[:, None] * dR
    dZ = dV
    dKg = -dZ @ S0.T
    KK = K @ K.T
    dbeta = np.sum(dR * Z, axis=1) + np.sum(dL * np.tril(Gam * KK, -1), axis=1)
    dA = np.tril(dO @ U.T)
    dAG = dA * Gam
    dQ = (gam[:, None] * dO) @ S0.T + dAG @ K
    M = dL * (beta[:, None] * Gam)
    dW = U @ dS_C.T
    dK = dAG.T @ Q + M @ K + M.T @ K + np.exp(g[-1] - g)[:, None] * dW + gam[:, None] * dKg
    GQ = gam[:, None] * Q
    dS0 = gam[-1] * dS_C + GQ.T @ dO - Kg.T @ dZ
    P = dA * A + dL * L
    dg = P.sum(axis=1) - P.sum(axis=0) + np.sum((GQ @ S0) * dO, axis=1) + np.sum(Kg * dKg, axis=1) \
        - np.sum(W * dW, axis=1)
    dg[-1] += np.sum(W * dW) + gam[-1] * np.sum(S0 * dS_C)
    dlog = np.cumsum(dg[::-1])[::-1]
    dalpha = dlog / alpha
    return dQ, dK, dV, dalpha, dbeta, dS0


def chunked_backward(q, k, v, alpha, beta, d_o, C):
    T, dh = q.shape
    _, _, bounds = chunked_forward(q, k, v, alpha, beta, C)
    dS = np.zeros((dh, dh))
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    da = np.zeros(T)
    db = np.zeros(T)
    starts = list(range(0, T, C))
    for ci in reversed(range(len(starts))):
        s = slice(starts[ci], min(T, starts[ci] + C))
        dq[s], dk[s], dv[s], da[s], db[s], dS = chunk_backward(q[s], k[s], v[s], alpha[s], beta[s],
                                                              bounds[ci], d_o[s], dS)
    return dq, dk, dv, da, db
