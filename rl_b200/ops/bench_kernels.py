"""Micro-benchmarks of the native kernels against their library twins (cuBLAS through torch, torch eager).

    python -m rl_b200.ops.bench_kernels [--which gemm,norm,...] [--json out.json]

Timing follows the usual hygiene: warm-up, CUDA events on the launching stream, inputs rotated through a
pool larger than L2 so that no iteration starts with its operands cached, and the reported figure is the
mean over the timed iterations. Fractions are against the measured peaks in ``MEASURED_PEAKS.json`` when
that file is present.
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch

from . import functional as F

L2_BYTES = 126 * 1024 * 1024


def _peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


def time_fn(fn, n_pool: int, iters: int = 20, warmup: int = 3) -> float:
    """Mean milliseconds per call of ``fn(i)``; ``i`` cycles over ``n_pool`` operand sets."""
    for i in range(warmup):
        fn(i % n_pool)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(iters):
        fn(i % n_pool)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def bench_gemm(shapes=None):
    peak_tf, _, how = _peaks()
    shapes = shapes or [
        # (M, N, K, a_mn, b_mn): Llama-3.1-8B linear layers at 8192 tokens, forward / dgrad / wgrad
        (8192, 6144, 4096, False, False), (8192, 4096, 4096, False, False), (8192, 28672, 4096, False, False),
        (8192, 4096, 14336, False, False), (8192, 4096, 28672, False, True), (28672, 4096, 8192, True, True),
        (8192, 128256, 4096, False, False), (512, 6144, 4096, False, False), (64, 28672, 4096, False, False),
    ]
    rows = []
    for M, N, K, a_mn, b_mn in shapes:
        bytes_per_set = 2 * (M * K + N * K + M * N)
        n_pool = max(2, min(8, L2_BYTES * 2 // bytes_per_set + 1))
        As = [torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16) for _ in range(n_pool)]
        Bs = [torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16) for _ in range(n_pool)]
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = time_fn(lambda i: F.gemm(As[i], Bs[i], a_mn=a_mn, b_mn=b_mn, out=out), n_pool)

        def lib(i):
            a = As[i].t() if a_mn else As[i]
            b = Bs[i] if b_mn else Bs[i].t()
            torch.matmul(a, b, out=out)

        ms_lib = time_fn(lib, n_pool)
        tf = 2.0 * M * N * K / ms / 1e9
        rows.append(dict(kernel="gemm_bf16", M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, ms=round(ms, 4), tflops=round(tf, 1),
                         frac_of_peak=round(tf / peak_tf, 3), peak=how, cublas_ms=round(ms_lib, 4),
                         vs_cublas=round(ms_lib / ms, 3)))
        print(rows[-1], flush=True)
    return rows


def bench_mxfp8(shapes=None):
    """MXFP8 block-scaled GEMM against the bf16 GEMM of the same shape (dense fp8 peak is 2x the bf16 peak)."""
    from .quant import gemm_mxfp8, quantize_mxfp8, swizzle_mx_scales

    peak_tf, _, how = _peaks()
    shapes = shapes or [(8192, 6144, 4096), (8192, 28672, 4096), (8192, 4096, 14336), (8192, 2048, 768), (8192, 1536, 2048)]
    rows = []
    for M, N, K in shapes:
        n_pool = max(2, min(6, L2_BYTES * 2 // (M * K + N * K + 2 * M * N) + 1))
        As = [torch.randn(M, K, device="cuda", dtype=torch.bfloat16) for _ in range(n_pool)]
        Bs = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(n_pool)]
        qa = [quantize_mxfp8(a) for a in As]
        qb = [quantize_mxfp8(b) for b in Bs]
        sa = [swizzle_mx_scales(s) for _, s in qa]
        sb = [swizzle_mx_scales(s) for _, s in qb]
        ms = time_fn(lambda i: gemm_mxfp8(qa[i][0], sa[i], qb[i][0], sb[i]), n_pool)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms_bf16 = time_fn(lambda i: F.gemm(As[i], Bs[i], out=out), n_pool)
        ms_q = time_fn(lambda i: quantize_mxfp8(As[i]), n_pool)
        tf = 2.0 * M * N * K / ms / 1e9
        rows.append(dict(kernel="gemm_mxfp8", M=M, N=N, K=K, ms=round(ms, 4), tflops=round(tf, 1), frac_of_bf16_peak=round(tf / peak_tf, 3),
                         peak=how, bf16_gemm_ms=round(ms_bf16, 4), vs_bf16_gemm=round(ms_bf16 / ms, 3), quantize_a_ms=round(ms_q, 4)))
        print(rows[-1], flush=True)
    return rows


def bench_grouped():
    """Grouped expert MLP GEMMs (Qwen3-30B-A3B: 16 local experts, d 2048, expert ffn 768) against a per-expert loop of
    library GEMMs (torch.matmul), forward gate_up + down, uneven expert loads."""
    from .moe_ops import ExpertLayout, grouped_linear

    peak_tf, _, how = _peaks()
    rows = []
    E, d, f = 16, 2048, 768
    for total in (16384, 65536):
        g = torch.Generator(device="cuda").manual_seed(0)
        w = torch.rand(E, generator=g, device="cuda") + 0.25
        counts = torch.floor(w / w.sum() * total).to(torch.int64)
        counts[0] += total - counts.sum()
        xs = torch.randn(total, d, device="cuda", dtype=torch.bfloat16)
        gu = torch.randn(E, 2 * f, d, device="cuda", dtype=torch.bfloat16) * 0.02
        dn = torch.randn(E, d, f, device="cuda", dtype=torch.bfloat16) * 0.02
        lay = ExpertLayout(counts, total)
        xp = torch.zeros((lay.mpad, d), dtype=torch.bfloat16, device="cuda").index_copy(0, lay.dest, xs)
        ap = torch.randn(lay.mpad, f, device="cuda", dtype=torch.bfloat16)
        cl = counts.tolist()

        def ours(i):
            with torch.no_grad():
                grouped_linear(xp, gu, lay)
                grouped_linear(ap, dn, lay)

        def lib(i):
            s0 = 0
            for e, c in enumerate(cl):
                torch.matmul(xs[s0 : s0 + c], gu[e].t())
                torch.matmul(ap[s0 : s0 + c], dn[e].t())
                s0 += c

        ms, ms_lib = time_fn(ours, 1), time_fn(lib, 1)
        flops = 2.0 * total * d * 2 * f + 2.0 * total * f * d
        rows.append(dict(kernel="gemm_grouped(gate_up+down)", experts=E, rows=total, d=d, f=f, ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1),
                         frac_of_peak=round(flops / ms / 1e9 / peak_tf, 3), peak=how, per_expert_loop_ms=round(ms_lib, 4),
                         vs_loop=round(ms_lib / ms, 3)))
        print(rows[-1], flush=True)
    return rows


def bench_memory_bound():
    _, hbm, how = _peaks()
    rows = []
    T, d, Fd = 16384, 4096, 14336
    n_pool = 4
    xs = [torch.randn(T, d, device="cuda", dtype=torch.bfloat16) for _ in range(n_pool)]
    w = torch.ones(d, device="cuda", dtype=torch.bfloat16)
    ms = time_fn(lambda i: F.rmsnorm(xs[i], w, 1e-5), n_pool)
    ms_ref = time_fn(lambda i: F._rmsnorm_ref(xs[i], w, 1e-5), n_pool)
    gb = 2 * T * d * 2 / 1e9
    rows.append(dict(kernel="rmsnorm_fwd", ms=round(ms, 4), gbs=round(gb / ms * 1e3, 1), frac_of_hbm=round(gb / ms * 1e3 / hbm, 3),
                     peak=how, torch_eager_ms=round(ms_ref, 4)))
    gus = [torch.randn(T, 2 * Fd, device="cuda", dtype=torch.bfloat16) for _ in range(n_pool)]
    ms = time_fn(lambda i: F.swiglu(gus[i]), n_pool)
    gb = 3 * T * Fd * 2 / 1e9
    rows.append(dict(kernel="swiglu_fwd", ms=round(ms, 4), gbs=round(gb / ms * 1e3, 1), frac_of_hbm=round(gb / ms * 1e3 / hbm, 3), peak=how))
    n = 1 << 28
    p32 = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = time_fn(lambda i: F.adamw_step(pb, None, p32, g, m, v, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, step=i + 1), 1)
    gb = n * (4 + 4 + 4 + 2) * 1.0 / 1e9 + n * (4 + 4 + 4 + 2) / 1e9
    rows.append(dict(kernel="adamw_fp32_master", n=n, ms=round(ms, 4), gbs=round(gb / ms * 1e3, 1), frac_of_hbm=round(gb / ms * 1e3 / hbm, 3), peak=how))
    for r in rows:
        print(r, flush=True)
    return rows


def bench_weight_stream():
    """Decode GEMMs at M = 64 tokens against the ideal time of streaming their weights once at the measured copy bandwidth."""
    _, hbm, how = _peaks()
    rows = []
    for N, K in ((28672, 4096), (4096, 14336), (6144, 4096), (4096, 4096), (128256, 4096)):
        n_pool = max(2, min(8, L2_BYTES * 2 // (N * K * 2) + 1))
        Ws = [torch.randn((N, K), device="cuda", dtype=torch.bfloat16) for _ in range(n_pool)]
        x = torch.randn((64, K), device="cuda", dtype=torch.bfloat16)
        gb = N * K * 2 / 1e9
        ms = time_fn(lambda i: F.gemm(x, Ws[i]), n_pool, iters=30)
        rows.append(dict(kernel="gemm_skinny_M64", N=N, K=K, us=round(ms * 1e3, 2), ideal_us=round(gb / hbm * 1e6, 2),
                         gbs=round(gb / ms * 1e3, 1), frac_of_hbm=round(gb / ms * 1e3 / hbm, 3), peak=how))
        del Ws
        torch.cuda.empty_cache()
    for r in rows:
        print(r, flush=True)
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--which", default="gemm,mem")
    ap.add_argument("--json", default="")
    ap.add_argument("--gemm-shape", default="", help="M,N,K: time only this GEMM shape (small case for profiler captures)")
    a = ap.parse_args(argv)
    out = []
    which = a.which.split(",")
    if "gemm" in which:
        shapes = None
        if a.gemm_shape:
            M, N, K = (int(x) for x in a.gemm_shape.split(","))
            shapes = [(M, N, K, False, False)]
        out += bench_gemm(shapes)
    if "mx" in which:
        out += bench_mxfp8()
    if "grouped" in which:
        out += bench_grouped()
    if "mem" in which:
        out += bench_memory_bound()
    if "stream" in which:
        out += bench_weight_stream()
    if a.json:
        os.makedirs(os.path.dirname(a.json) or ".", exist_ok=True)
        Path(a.json).write_text(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
