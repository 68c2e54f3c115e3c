"""Refit benchmark: time of one trainer -> engine weight synchronisation for a model and a pair of layouts.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 -m rl_b200.refit.bench_refit --model llama3.1-8b \\
        --train-tp 1 --serve-tp 1,2,4,8 [--json out.json]

Weights are uninitialised memory of the right shapes (only bytes move). Times are CUDA-event device times of
``WeightSynchronizer.sync_weights`` (rendezvous + re-shard copy kernel + rendezvous), max over ranks, after warm-up.
"Same layout" rows report the colocated pointer hand-off (no copy at all). The NCCL twin (all-gather every tensor, slice)
is timed the same way.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from rl_b200.models.config import preset
from rl_b200.models.transformer import build_model
from rl_b200.parallel.tensor import TP
from rl_b200.refit.synchronizer import WeightSynchronizer


def _time(fn, iters=5, warmup=2) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3.1-8b")
    ap.add_argument("--train-tp", type=int, default=1)
    ap.add_argument("--serve-tp", default="1,2")
    ap.add_argument("--twin", action="store_true", help="also time the collective twin (all-gather + slice)")
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = preset(a.model)
    tp = TP(None, rank % a.train_tp, a.train_tp)
    train = build_model(cfg, device=f"cuda:{local}", dtype=torch.bfloat16, init=False, tp=tp)
    rows = []
    for ts in [int(x) for x in a.serve_tp.split(",")]:
        if world % ts:
            continue
        ws = WeightSynchronizer(train, cfg, ts)
        ms = _time(ws.sync_weights)
        sent, recv = ws.plan.bytes_over_link(rank)
        local_bytes = ws.last_bytes
        row = dict(model=a.model, world=world, train_tp=a.train_tp, serve_tp=ts, sync_ms=ms, bytes_written_per_rank=local_bytes,
                   nvlink_bytes_sent=sent, nvlink_bytes_received=recv, write_gbs=local_bytes / ms / 1e6)
        if a.twin:
            row["twin_ms"] = _time(ws.twin_sync, iters=2, warmup=1)
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        ws.close()
        del ws
        torch.cuda.empty_cache()
    if rank == 0 and a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f, indent=1)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
