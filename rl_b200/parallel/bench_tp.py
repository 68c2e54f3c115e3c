"""Benchmarks of the fused tensor-parallel GEMM + collective kernels against their NCCL twins.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 -m rl_b200.parallel.bench_tp [--json out.json] [--tokens 8192]

Shapes are the tensor-parallel linears of Qwen3-32B (hidden 5120, q 8192, kv 1024, ffn 25600) at the job's tensor
parallel size. Every figure is device time from CUDA events, max over ranks, after warm-up; operands rotate through a
pool larger than L2. The roofline of a fused kernel is the slower of (FLOPs / measured GEMM peak) and (bytes that
must cross NVLink per GPU / measured per-direction bandwidth).
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

from rl_b200.ops import functional as F
from rl_b200.parallel.tensor import TPFusedComm, all_gather_rows, reduce_scatter_rows

NVLINK_GBS = 770.0  # measured peer copy, per direction per GPU


def _peak_tflops():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text()).get("bf16_tflops", 1590.0), "measured"
    return 1590.0, "fallback"


def _time(fn, iters=12, warmup=3) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(iters):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--decode-batch", type=int, default=256)
    ap.add_argument("--pushers", type=int, default=12)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    comm = TPFusedComm(None, wait_limit_s=10.0, pushers=args.pushers)
    peak, how = _peak_tflops()
    T, d, tp = args.tokens, 5120, world
    rows = T // tp
    pool = 3
    out = []

    def rnd(*shape):
        return (torch.randn(*shape, device=dev) * 0.05).to(torch.bfloat16)

    # ---------------- all-gather -> column GEMM (qkv: N = (8192 + 2048)/tp, gate_up: N = 51200/tp)
    for name, N in (("qkv", (8192 + 2048) // tp), ("gate_up", 51200 // tp)):
        xs = [rnd(rows, d) for _ in range(pool)]
        ws = [rnd(N, d) for _ in range(pool)]
        fused = _time(lambda i: comm.gather_gemm(xs[i % pool], ws[i % pool]))
        twin = _time(lambda i: F.gemm(all_gather_rows(xs[i % pool], None, world), ws[i % pool]))
        flops = 2.0 * T * N * d
        link_bytes = (tp - 1) * rows * d * 2  # received per GPU
        roof_ms = max(flops / (peak * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        out.append(dict(kernel=f"gather_gemm[{name}]", M=T, N=N, K=d, tp=tp, fused_ms=fused, nccl_twin_ms=twin, roofline_ms=roof_ms,
                        frac_of_roofline=roof_ms / fused, speedup_vs_twin=twin / fused, peaks=how))
    # ---------------- row GEMM -> reduce-scatter (o: K = 8192/tp, down: K = 25600/tp)
    for name, K in (("o_proj", 8192 // tp), ("down", 25600 // tp)):
        as_ = [rnd(T, K) for _ in range(pool)]
        ws = [rnd(d, K) for _ in range(pool)]
        res = rnd(rows, d)
        fused = _time(lambda i: comm.scatter_gemm(as_[i % pool], ws[i % pool], residual=res))
        phases = comm.phase_times_us()
        twin = _time(lambda i: reduce_scatter_rows(F.gemm(as_[i % pool], ws[i % pool]), None, world, rank).add_(res))
        gemm_only = _time(lambda i: F.gemm(as_[i % pool], ws[i % pool]))
        flops = 2.0 * T * d * K
        link_bytes = (tp - 1) * rows * d * 2  # bf16 partials sent per GPU
        roof_ms = max(flops / (peak * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        out.append(dict(kernel=f"scatter_gemm[{name}]", M=T, N=d, K=K, tp=tp, fused_ms=fused, nccl_twin_ms=twin, roofline_ms=roof_ms,
                        plain_gemm_ms=gemm_only, phases_us=dict(zip(("tiles", "grid_sync", "peer_barrier", "reduce"), phases)),
                        frac_of_roofline=roof_ms / fused, speedup_vs_twin=twin / fused, peaks=how))
    # ---------------- decode: row GEMM -> all-reduce (+ residual)
    B = args.decode_batch
    for name, K in (("o_proj", 8192 // tp), ("down", 25600 // tp)):
        as_ = [rnd(B, K) for _ in range(pool)]
        ws = [rnd(d, K) for _ in range(pool)]
        res = rnd(B, d)

        def twin_fn(i):
            y = F.gemm(as_[i % pool], ws[i % pool])
            dist.all_reduce(y)
            return y.add_(res)

        fused = _time(lambda i: comm.scatter_gemm(as_[i % pool], ws[i % pool], residual=res, all_reduce=True), iters=30)
        twin = _time(twin_fn, iters=30)
        hbm_ms = (d * K * 2) / 7.0e12 * 1e3  # weight stream
        link_ms = (tp - 1) * B * d * 2 / (NVLINK_GBS * 1e9) * 1e3
        out.append(dict(kernel=f"gemm_allreduce[{name}]", M=B, N=d, K=K, tp=tp, fused_ms=fused, nccl_twin_ms=twin,
                        roofline_ms=max(hbm_ms, link_ms), frac_of_roofline=max(hbm_ms, link_ms) / fused, speedup_vs_twin=twin / fused, peaks=how))
    torch.cuda.synchronize()
    from rl_b200.ops.lib import check_status

    st = check_status()
    if rank == 0:
        for r in out:
            print(json.dumps(r))
        print(json.dumps({"status": st}))
        if args.json:
            with open(args.json, "w") as f:
                json.dump({"rows": out, "status": st, "world": world}, f, indent=1)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
