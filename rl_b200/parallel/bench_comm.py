"""Micro-benchmarks of the peer-memory communication kernels against their NCCL twins (one process per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P -m rl_b200.parallel.bench_comm [--params 1.2e9]

* the one-kernel optimizer step (gradient reduce-scatter + clipping + AdamW + parameter all-gather over peer memory,
  ``csrc/comm.cu::fused_optim_kernel``) against NCCL reduce-scatter + AdamW kernel + NCCL all-gather, with the bytes that
  cross NVLink per rank and the achieved rate against the measured peer-copy rate (770 GB/s per direction);
* the decode-sized one-shot all-reduce (``p2p_allreduce_rows_kernel``, residual add and RMSNorm fused) against an NCCL
  all-reduce followed by the add and the norm.

Device time with CUDA events on the launching stream, maximum over ranks; rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

PEER_COPY_GBS = 770.0   # measured peer copy, per direction per GPU, on this machine type


def _time(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([t0.elapsed_time(t1) / iters], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)


def bench_optimizer(params: float, iters: int, warmup: int) -> dict:
    from rl_b200.models.config import ModelConfig
    from rl_b200.policy.worker import PolicyWorker

    world, rank = dist.get_world_size(), dist.get_rank()
    # a Llama-shaped model of about `params` parameters (the optimizer only sees the flat buffer)
    d = 2048
    L = max(1, round((params - 2 * 32000 * d) / (12.6 * d * d)))
    mc = ModelConfig(model_type="llama", vocab_size=32000, hidden_size=d, intermediate_size=4 * d, num_hidden_layers=L, num_attention_heads=16,
                     num_key_value_heads=8, head_dim=128)
    out = {}
    for mode in ("fused", "nccl"):
        p = PolicyWorker(dict(precision="bfloat16", train_global_batch_size=world, train_micro_batch_size=1, max_total_sequence_length=128,
                              fused_optimizer=(mode == "fused"), max_grad_norm=1.0,
                              optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-5, weight_decay=0.01))),
                         model_cfg=mc, device=f"cuda:{torch.cuda.current_device()}", init_reference_model=False, seed=1)
        n = p.flat.flat.numel()
        g = p.flat.grad
        g.normal_(0, 1e-3, generator=torch.Generator(device="cuda").manual_seed(rank))

        def step():
            p.optimizer.step(1.0)

        ms = _time(step, iters, warmup)
        link_in = (world - 1) / world * n * (4 + 2)     # fp32 gradient slices pulled + bf16 parameter slices gathered, per rank
        out[mode] = dict(ms=round(ms, 3), params=n, nvlink_bytes_in_per_rank=int(link_in),
                         nvlink_gbs_in=round(link_in / ms / 1e6, 1), fraction_of_peer_copy=round(link_in / ms / 1e6 / PEER_COPY_GBS, 3),
                         path=("one cooperative kernel" if p.fused_comm is not None else "NCCL reduce-scatter + AdamW + NCCL all-gather"))
        del p
        torch.cuda.empty_cache()
    out["speedup"] = round(out["nccl"]["ms"] / out["fused"]["ms"], 3)
    return out


def bench_allreduce_rows(iters: int, warmup: int) -> list[dict]:
    from rl_b200.ops import functional as F
    from rl_b200.parallel.tensor import TPFusedComm

    world = dist.get_world_size()
    comm = TPFusedComm(None)
    rows = []
    for M, N in ((32, 5120), (64, 4096), (256, 8192)):
        part = torch.randn(M, N, device="cuda")
        res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
        w = torch.ones(N, device="cuda", dtype=torch.bfloat16)

        def fused():
            comm.allreduce_rows(part, res, w, 1e-6)

        def twin():
            x = part.to(torch.bfloat16)
            dist.all_reduce(x)
            h = x + res
            F.rmsnorm(h, w, 1e-6)

        a, b = _time(fused, iters, warmup), _time(twin, iters, warmup)
        rows.append(dict(M=M, N=N, fused_us=round(a * 1e3, 1), nccl_twin_us=round(b * 1e3, 1), speedup=round(b / a, 2),
                         bytes_in_per_rank=int((world - 1) * M * N * 4)))
    comm.close()
    return rows


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=float, default=1.2e9)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from rl_b200.ops import lib as L

    L.lib()
    out = dict(n_gpus=dist.get_world_size(), optimizer=bench_optimizer(a.params, a.iters, a.warmup),
               allreduce_rows=bench_allreduce_rows(50, 10), status=L.check_status())
    if dist.get_rank() == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
