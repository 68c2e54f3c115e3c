"""Flash-attention micro-benchmark: causal varlen GQA forward and backward on packed sequences.

    python -m rl_b200.ops.bench_attention --seqs 16 --seq-len 4096 --hq 32 --hkv 8 [--iters 10] [--json out.json]

Times the forward and the forward + backward with CUDA events (warm-up, operands rotated through a pool larger than L2)
and reports TFLOP/s of the causal attention FLOPs (forward 2 x 2 x S^2/2 x Hq x D per sequence, backward 2.5 x that)
against the measured bf16 peak. A small case (``--seqs 2 --seq-len 2048 --iters 1``) suits profiler captures.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import functional as F
from .bench_kernels import L2_BYTES, _peaks


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqs", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    D = 128
    T = a.seqs * a.seq_len
    width = (a.hq + 2 * a.hkv) * D
    pool = max(2, min(6, 2 * L2_BYTES // (T * width * 2) + 1))
    qkvs = [(torch.randn(T, width, device="cuda", dtype=torch.bfloat16) * 0.5).requires_grad_(True) for _ in range(pool)]
    cu = torch.arange(0, T + 1, a.seq_len, device="cuda", dtype=torch.int32)
    dout = torch.randn(T, a.hq * D, device="cuda", dtype=torch.bfloat16)

    def fwd(i):
        with torch.no_grad():
            return F.attention_varlen(qkvs[i % pool], cu, a.seq_len, a.hq, a.hkv, D)

    def fwd_bwd(i):
        q = qkvs[i % pool]
        q.grad = None
        F.attention_varlen(q, cu, a.seq_len, a.hq, a.hkv, D).backward(dout)

    def timed(fn):
        for i in range(min(3, a.iters)):
            fn(i)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(a.iters):
            fn(i)
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / a.iters

    t_f = timed(fwd)
    t_fb = timed(fwd_bwd)
    flops_f = a.seqs * 4 * (a.seq_len ** 2 / 2) * a.hq * D
    peak, _, how = _peaks()
    out = dict(kernel="flash_attention", seqs=a.seqs, seq_len=a.seq_len, hq=a.hq, hkv=a.hkv, fwd_ms=round(t_f, 4), fwd_bwd_ms=round(t_fb, 4),
               fwd_tflops=round(flops_f / t_f / 1e9, 1), bwd_tflops=round(2.5 * flops_f / max(t_fb - t_f, 1e-6) / 1e9, 1),
               fwd_frac_of_peak=round(flops_f / t_f / 1e9 / peak, 3), bwd_frac_of_peak=round(2.5 * flops_f / max(t_fb - t_f, 1e-6) / 1e9 / peak, 3),
               peak=how)
    print(json.dumps(out), flush=True)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(out, f)


if __name__ == "__main__":
    main()
