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
    ap.add_argument("--fp8", action="store_true", help="time the quantising refit (block-128 FP8 written on the way) as well")
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
        if a.fp8:
            row["fp8_sync_ms"] = _time(ws.sync_weights_fp8, iters=3, warmup=1)
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


def sweep_main(steps: int = 3, warmup: int = 2, models=("llama3.1-8b", "qwen3-32b"), json_path: str = "") -> int:
    """The refit sweep of ``bench.py --config refit-sweep``: the trainer's layout on all ranks of the node (data parallel,
    resident bf16 parameters) -> serving layouts TP 1 / 2 / 4 / 8, for the 8B and 32B dense architectures, in bf16 and
    with FP8 block-128 quantisation. Rank 0 prints one JSON line whose ``rows`` hold, per case, the device time of one
    refit (max over ranks), the bytes written per rank, the bytes that crossed NVLink and the effective rate."""
    from rl_b200.engine.quantized import quantize_model
    from rl_b200.ops import lib as _L

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _L.lib()
    rows = []
    for name in models:
        cfg = preset(name)
        train = build_model(cfg, device=f"cuda:{local}", dtype=torch.bfloat16, init=False, tp=TP(None, 0, 1))
        for ts in (1, 2, 4, 8):
            if ts > world or world % ts:
                continue
            ws = WeightSynchronizer(train, cfg, ts)
            ms = _time(ws.sync_weights, iters=max(1, steps), warmup=max(1, warmup))
            sent, recv = ws.plan.bytes_over_link(rank)
            row = dict(model=name, world=world, train_layout=f"dp{world} (resident parameters)", serve_tp=ts, precision="bf16",
                       refit_ms=round(ms, 3), bytes_written_per_rank=int(ws.last_bytes), nvlink_bytes_per_rank=int(sent + recv),
                       write_gbs=round(ws.last_bytes / ms / 1e6, 1),
                       colocated_handoff_ms=0.0 if ts == 1 else None)
            rows.append(row)
            # FP8 block-128: the serving copy is quantised as it is refreshed
            fused = getattr(ws, "sync_weights_fp8", None)
            if fused is not None:
                ms8 = _time(fused, iters=max(1, steps), warmup=max(1, warmup))
                how = "one kernel: bf16 tile -> amax -> e4m3 + scale into the serving arena"
            else:
                def two_pass():
                    ws.sync_weights()
                    quantize_model(ws.serving_model, "fp8")
                ms8 = _time(two_pass, iters=max(1, steps), warmup=max(1, warmup))
                how = "two passes: bf16 re-shard copy, then block-128 quantisation of the serving copy"
            rows.append(dict(row, precision="fp8-block128", refit_ms=round(ms8, 3), write_gbs=None, how=how,
                             read_gbs=round(ws.last_bytes / ms8 / 1e6, 1)))
            ws.close()
            del ws
            torch.cuda.empty_cache()
        del train
        torch.cuda.empty_cache()
    status = _L.check_status()
    if rank == 0:
        out = dict(metric="refit_seconds (trainer layout -> serving layout, device time, max over ranks)", unit="ms", n_gpus=world,
                   steps=steps, warmup=warmup, config=dict(name="refit-sweep"), rows=rows, status=status, impl="ours",
                   note="data-parallel training keeps complete bf16 parameters on every rank, so every serving shard is cut from the "
                        "rank's own copy: no byte crosses NVLink and the rate is local HBM traffic")
        print(json.dumps(out), flush=True)
        if json_path:
            with open(json_path, "w") as f:
                json.dump(out, f, indent=1)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    main()
