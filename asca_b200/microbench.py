"""Per-kernel bandwidth / throughput measurements of the library's entry points.

    python -m asca_b200.microbench [--only name,name] [--reps 20]

Each case times one entry point with CUDA events on the launching stream after warm-up, on
buffers larger than the 126 MB L2 (or a rotation of buffers whose total is), and prints one
JSON line: algorithmic bytes (or FLOPs) per launch, time, achieved GB/s (or TFLOP/s) and the
fraction of the measured peak in MEASURED_PEAKS.json at the repository root when present.
Shapes follow the baseline configurations (decode: 256 streams, 12 heads, dh 64; MoE layer:
65,536 tokens, d 1024, 64 experts, F 4096).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

import asca_b200
from asca_b200 import ops

ROOT = Path(__file__).resolve().parent.parent


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, reps, warmup=3):
    for _ in range(warmup):
        fn(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def report(name, ms, nbytes=None, flops=None, note=""):
    hbm, tf, src = peaks()
    line = {"kernel": name, "ms": round(ms, 5), "note": note}
    if nbytes is not None:
        gbs = nbytes / (ms * 1e-3) / 1e9
        line.update({"bytes": int(nbytes), "GB/s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / hbm, 4), "peak": src})
    if flops is not None:
        t = flops / (ms * 1e-3) / 1e12
        line.update({"flops": int(flops), "TFLOP/s": round(t, 2), "frac_of_bf16_peak": round(t / tf, 4), "peak": src})
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--reps", type=int, default=20)
    args = ap.parse_args()
    only = set(filter(None, args.only.split(",")))
    want = lambda n: not only or n in only  # noqa: E731
    gpu = asca_b200.Gpu(0)
    gpu.use_torch_stream()
    dev = torch.device("cuda", 0)
    f32 = dict(dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)

    if want("delta_step"):
        ns, H, dh, L = 256, 12, 64, 12  # 12 layers' states rotate: 604 MB > L2
        S = [torch.randn(ns, H, dh, dh, generator=g, **f32) * 0.1 for _ in range(L)]
        d = H * dh
        qkv = torch.randn(ns, 3 * d, generator=g, **f32)
        gate = torch.randn(ns, 2 * H, generator=g, **f32)
        o = torch.empty(ns, d, **f32)
        ms = timeit(lambda i: ops.delta_step(gpu, qkv, None, None, gate, None, S[i % L], H, dh, fused=True, out=o), args.reps * 3)
        report("delta_step_kernel<64> fused", ms, 2 * ns * H * dh * dh * 4 + ns * (4 * d + 2 * H) * 4,
               note="256 streams x 12 heads, state read+write per launch")
        ns2, H2, dh2 = 64, 16, 128
        S2 = [torch.randn(ns2, H2, dh2, dh2, generator=g, **f32) * 0.1 for _ in range(4)]
        qkv2 = torch.randn(ns2, 3 * H2 * dh2, generator=g, **f32)
        gate2 = torch.randn(ns2, 2 * H2, generator=g, **f32)
        o2 = torch.empty(ns2, H2 * dh2, **f32)
        ms = timeit(lambda i: ops.delta_step(gpu, qkv2, None, None, gate2, None, S2[i % 4], H2, dh2, fused=True, out=o2), args.reps * 3)
        report("delta_step_kernel<128> fused", ms, 2 * ns2 * H2 * dh2 * dh2 * 4, note="64 streams x 16 heads")
        del S, S2

    if want("rmsnorm"):
        rows, cols = 65536, 1024
        xs = [torch.randn(rows, cols, generator=g, **f32) for _ in range(2)]
        y = torch.empty(rows, cols, **f32)
        ms = timeit(lambda i: gpu._call("asca_rmsnorm_fwd", gpu._ctx, asca_b200._p(xs[i % 2]), asca_b200._p(y), None,
                                        asca_b200._i64(rows), asca_b200._i64(cols), asca_b200._f(1e-6)), args.reps)
        report("rmsnorm_fwd_kernel", ms, 2 * rows * cols * 4, note="65536 x 1024 f32")
        dy = torch.randn(rows, cols, generator=g, **f32)
        ms = timeit(lambda i: gpu._call("asca_rmsnorm_bwd", gpu._ctx, asca_b200._p(xs[i % 2]), asca_b200._p(dy),
                                        asca_b200._p(y), asca_b200._i64(rows), asca_b200._i64(cols), asca_b200._f(1e-6)),
                    args.reps)
        report("rmsnorm_bwd_kernel", ms, 3 * rows * cols * 4, note="65536 x 1024 f32")
        xm = torch.empty(rows, cols, **f32)
        ms = timeit(lambda i: gpu._call("asca_residual_rmsnorm", gpu._ctx, asca_b200._p(xs[0]), asca_b200._p(xs[1]),
                                        asca_b200._p(xm), asca_b200._p(y), asca_b200._i64(rows), asca_b200._i64(cols),
                                        asca_b200._f(1e-6)), args.reps)
        report("residual_rmsnorm (fused)", ms, 4 * rows * cols * 4, note="x + y -> x_mid, xn")
        del xs, y, dy, xm

    if want("dispatch"):
        for n in (65536, 1 << 22):
            w = 1.0 / torch.arange(1, 257, device=dev, dtype=torch.float64) ** 1.1
            ids = torch.multinomial(w.float(), n, replacement=True, generator=g).to(torch.int32)
            perm = torch.empty(n, dtype=torch.int32, device=dev)
            off = torch.empty(65, dtype=torch.int32, device=dev)
            ms = timeit(lambda i: gpu._call("asca_moe_dispatch", gpu._ctx, asca_b200._p(ids), asca_b200._i64(n),
                                            asca_b200._i64(64), asca_b200._p(perm), asca_b200._p(off), None), args.reps)
            report(f"moe_dispatch (3 kernels) N={n}", ms, 2 * 4 * n + 4 * n, note="ids read twice, perm written; Zipf(1.1) ids, E=64")

    if want("adamw"):
        n = 1 << 26
        p, gr, m, v = (torch.randn(n, generator=g, **f32) * 0.01 for _ in range(4))
        v.abs_()
        ms = timeit(lambda i: ops.adamw(gpu, p, gr, m, v, 1e-3, 0.9, 0.95, 1e-8, 1e-5), args.reps)
        report("adamw_kernel", ms, 7 * n * 4, note="2^26 elements: 4 reads + 3 writes")
        del p, gr, m, v

    if want("gather"):
        rows, cols = 65536, 1024
        src = torch.randn(rows, cols, generator=g, **f32)
        idx = torch.randperm(rows, device=dev, generator=g).to(torch.int32)
        dst = torch.empty(rows, cols, **f32)
        ms = timeit(lambda i: gpu._call("asca_gather_rows", gpu._ctx, asca_b200._p(src), asca_b200._p(idx),
                                        asca_b200._i64(rows), asca_b200._i64(cols), asca_b200._p(dst)), args.reps)
        report("gather_rows", ms, 2 * rows * cols * 4, note="random permutation of 65536 x 1024 rows")
        del src, dst

    if want("gemm"):
        for (m_, n_, k_) in ((8192, 8192, 8192), (32768, 6144, 2048)):
            for dt in (torch.float32, torch.bfloat16):
                a = torch.randn(m_, k_, generator=g, **f32).to(dt)
                b = torch.randn(k_, n_, generator=g, **f32).to(dt)
                c = torch.empty(m_, n_, **f32)
                ms = timeit(lambda i: ops.gemm(gpu, a, b, asca_b200.NN, out=c), max(2, args.reps // 5), warmup=1)
                report(f"gemm NN {m_}x{n_}x{k_} {str(dt).split('.')[-1]}", ms, flops=2 * m_ * n_ * k_)
                del a, b, c
        # the transposed forms at the training step's shapes (input gradient and weight gradient of the qkv projection)
        for mode, name, (m_, n_, k_) in ((asca_b200.NT, "NT", (32768, 2048, 6144)), (asca_b200.TN, "TN", (2048, 6144, 32768))):
            a = torch.randn((k_, m_) if mode == asca_b200.TN else (m_, k_), generator=g, **f32).bfloat16()
            b = torch.randn((n_, k_) if mode == asca_b200.NT else (k_, n_), generator=g, **f32).bfloat16()
            c = torch.empty(m_, n_, **f32)
            ms = timeit(lambda i: ops.gemm(gpu, a, b, mode, out=c), max(2, args.reps // 5), warmup=1)
            report(f"gemm {name} {m_}x{n_}x{k_} bfloat16", ms, flops=2 * m_ * n_ * k_)
            del a, b, c

    if want("moe"):
        n, d, F, E = 65536, 1024, 4096, 64
        w = 1.0 / torch.arange(1, 257, device=dev, dtype=torch.float64) ** 1.1
        ids = torch.multinomial(w.float(), n, replacement=True, generator=g).to(torch.int32)
        perm, off = ops.moe_dispatch(gpu, ids, E)
        for dt in (torch.bfloat16,):
            xn = torch.randn(n, d, generator=g, **f32).to(dt)
            w1 = (torch.randn(d, E * F, generator=g, **f32) * 0.02).to(dt)
            w2 = (torch.randn(E * F, d, generator=g, **f32) * 0.02).to(dt)
            b1, b2 = torch.zeros(E * F, **f32), torch.zeros(d, **f32)
            dout = torch.randn(n, d, generator=g, **f32)
            out, pre_p, hid_p = ops.moe_fwd(gpu, xn, w1, b1, w2, b2, perm, off, F, E)
            ms = timeit(lambda i: ops.moe_fwd(gpu, xn, w1, b1, w2, b2, perm, off, F, E, out=out, pre_p=pre_p, hid_p=hid_p),
                        3, warmup=1)
            report(f"moe_fwd {str(dt).split('.')[-1]} (2 grouped GEMMs)", ms, flops=4 * n * d * F, note="config 3, Zipf load")
            grads = ops.moe_bwd(gpu, xn, w1, w2, pre_p, hid_p, dout, perm, off, F, E)
            ms = timeit(lambda i: ops.moe_bwd(gpu, xn, w1, w2, pre_p, hid_p, dout, perm, off, F, E, grads=grads), 3, warmup=1)
            report(f"moe_bwd {str(dt).split('.')[-1]} (4 grouped GEMMs + 2 column sums)", ms, flops=8 * n * d * F,
                   note="config 3, Zipf load")


if __name__ == "__main__":
    main()
