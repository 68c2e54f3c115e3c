"""Benchmarks of the GRPO step on one node of N GPUs, synthetic prompts, random-init weights.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per GPU by torch.distributed.run)
    python bench.py --config qwen3-32b-tp4dp2 --gpus 8 ...   (other model / layout configurations, see CONFIGS)
    python bench.py --config refit-sweep --gpus 8            (weight re-shard times, trainer layout -> serving layouts)
    python bench.py --impl reference ...                     (the unmodified reference, when it can be installed)

Default (headline) configuration ``llama8b-dp``: one GRPO step (generation + refit + log-probabilities + training) on
the Llama-3.1-8B architecture. Work per step and per GPU is fixed (weak scaling): 8 prompts x 8 generations, prompts of
256 random tokens, 1024 generated tokens each (stop tokens disabled so every response runs to the limit), one optimizer
step over the global batch of 64*N sequences. At N = 8 this is the 64 prompts x 8 generations configuration.

Two timed regions, K steps each:
  * device: the phases called directly, bracketed by CUDA events on the launching stream (max over ranks);
  * e2e:    the same K steps through the public training API (``rl_b200.algorithms.grpo.grpo_train``), wall clock
            between synchronisations, including the data loader, every host->device copy of that step's inputs from
            pinned memory and the device->host reads of sampled tokens, log-probabilities and the loss.
Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


# Named configurations. ``llama8b-dp`` is the headline; the others are the larger model / layout configurations of the
# same benchmark family (one 8-GPU node). Values a flag also sets are defaults that the flag overrides.
CONFIGS = {
    "llama8b-dp": dict(model="llama3.1-8b", tp=1, ep=1, gen_tp=0, prompts_per_gpu=8, generations=8, prompt_len=256, max_new_tokens=1024,
                       train_mb_tokens=5120, logprob_mb_tokens=20480, act_ckpt="off"),
    # Qwen3-32B: TP4 x DP2 training with sequence parallelism, generation TP2 x 4 engines, fused vocabulary-parallel lm_head
    # (4096-token training micro-batches: with 8192 the second step ran out of memory next to the 33 GB serving arena)
    "qwen3-32b-tp4dp2": dict(model="qwen3-32b", tp=4, ep=1, gen_tp=2, prompts_per_gpu=2, generations=8, prompt_len=512, max_new_tokens=3584,
                             train_mb_tokens=4096, logprob_mb_tokens=8192, act_ckpt="on"),
    # Qwen3-30B-A3B: expert parallel over all GPUs, dense parts data parallel
    "qwen3-30b-a3b-ep8": dict(model="qwen3-30b-a3b", tp=1, ep=0, gen_tp=0, prompts_per_gpu=4, generations=8, prompt_len=512, max_new_tokens=2048,
                              train_mb_tokens=8192, logprob_mb_tokens=16384, act_ckpt="on"),
    "refit-sweep": dict(),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="llama8b-dp", choices=sorted(CONFIGS))
    ap.add_argument("--model", default=None)
    ap.add_argument("--prompts-per-gpu", type=int, default=None)
    ap.add_argument("--generations", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--max-new-tokens", type=int, default=None)
    ap.add_argument("--gen-tp", type=int, default=None, help="tensor-parallel size of the generation engines (0: the trainer's)")
    ap.add_argument("--ep", type=int, default=None, help="expert-parallel size (0: all GPUs)")
    ap.add_argument("--logprob-mb-tokens", type=int, default=None)
    ap.add_argument("--sharding", default="optimizer", choices=["optimizer", "full"],
                    help="data-parallel sharding: optimizer state only (resident parameters, the headline) or full (ZeRO-3: "
                         "parameters and gradients sharded too, gathered per layer)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (makes the run invalid as a benchmark)")
    ap.add_argument("--train-mb-tokens", type=int, default=None, help="tokens per training micro-batch (the same at every N)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--tp", type=int, default=None, help="tensor-parallel size of the trainer (with sequence parallelism); "
                    "the headline configuration is --tp 1")
    ap.add_argument("--act-ckpt", default=None, choices=["on", "off"],
                    help="activation checkpointing in training (headline: off, with 5120-token micro-batches the activations of "
                         "Llama-3.1-8B fit next to the unsharded optimizer state even on 1 GPU)")
    args = ap.parse_args()
    for k, v in CONFIGS[args.config].items():   # flags left unset take the configuration's values
        if getattr(args, k, None) is None:
            setattr(args, k, v)
    return args


def reference_arm(args) -> int:
    """The reference (NVIDIA-NeMo/RL) cannot be installed in this image: it requires Python >= 3.13.14 (image: 3.12) and
    its public entry points import ray, omegaconf, hydra, nemo-automodel, nccl4py and pyzmq, none of which is present
    in the image or the offline wheelhouse."""
    why = ("reference not runnable offline: needs Python>=3.13.14 (image has 3.12.3) and ray/omegaconf/hydra/"
           "nemo-automodel/nccl4py/pyzmq, absent from the image and /opt/wheelhouse; "
           "`import nemo_rl.algorithms.grpo` fails with ModuleNotFoundError: ray")
    ref = os.path.join(REPO, "baseline", "_ref")
    try:
        sys.path.insert(0, ref)
        import importlib

        importlib.import_module("nemo_rl.algorithms.grpo")
        why = "reference imported, but no runnable reference arm is wired for this image"
    except Exception as e:  # expected
        why = why if "ray" in str(e) or "nemo_rl" in str(e) else f"reference import failed: {type(e).__name__}: {e}"
    finally:
        if ref in sys.path:
            sys.path.remove(ref)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """Samples SM clock and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.rows: list[list[str]] = []
        self.proc = None

    def start(self):
        try:
            # one sample per second: every query takes driver locks that the decode phase's launches contend for, and a
            # 5 Hz poll was measured to stretch generation by ~15 %
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "1000",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons, power = [], [], set(), []
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                power.append(float(r[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # keep samples taken under load (clock above idle) for the median
        loaded = [c for c, p in zip(sm, power) if p > 300] or sm
        return {"sm_mhz": statistics.median(loaded) if loaded else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(power) if power else None}


def main() -> int:
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    if args.config == "refit-sweep":
        from rl_b200.refit.bench_refit import sweep_main

        return sweep_main(steps=args.steps, warmup=args.warmup)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and rank == 0:
        print(f"[bench] note: --gpus {args.gpus} but WORLD_SIZE={world}; using WORLD_SIZE", file=sys.stderr)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if os.environ.get("RLB_BIND_NUMA", "1") == "1":
        # keep every rank's host loop (scheduler, table uploads) on the cores and memory next to its GPU
        try:
            from rl_b200.distributed.numa import bind_to_gpu_numa_node

            bind_to_gpu_numa_node(local_rank)
        except Exception:
            pass
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from rl_b200.csrc.build import build_all
    from rl_b200.ops import lib as L

    if not L.available():
        if rank == 0:
            build_all()
        if world > 1:
            dist.barrier()
    L.lib()

    from rl_b200.algorithms import grpo as G
    from rl_b200.algorithms.loss.loss_functions import ClippedPGLossFn
    from rl_b200.data.collate import rl_collate_fn
    from rl_b200.data.datasets.synthetic import RandomTokenPromptDataset
    from rl_b200.environments.synthetic import HashParityEnv
    from rl_b200.models.config import preset

    mc = preset(args.model)
    if args.layers:
        mc.num_hidden_layers = args.layers
    n_prompts = args.prompts_per_gpu * world
    n_gen = args.generations
    seqs_per_gpu = args.prompts_per_gpu * n_gen
    max_len = args.prompt_len + args.max_new_tokens
    steps_needed = args.warmup + 2 * args.steps + 2
    mb_tokens = args.train_mb_tokens
    gen_tp = args.gen_tp or args.tp   # every engine of gen_tp ranks serves the sequences of gen_tp GPUs
    cfg = {
        "grpo": dict(num_prompts_per_step=n_prompts, num_generations_per_prompt=n_gen, max_num_steps=10**9, val_period=0, seed=0,
                     normalize_rewards=True, use_leave_one_out_baseline=True),
        "loss_fn": dict(reference_policy_kl_penalty=0.01, ratio_clip_min=0.2, ratio_clip_max=0.2),
        "policy": dict(
            model_name=None, precision="bfloat16", train_global_batch_size=seqs_per_gpu * world, train_micro_batch_size=4,
            parallel=dict(tensor_parallel_size=args.tp, sequence_parallel=args.tp > 1, data_parallel_sharding=args.sharding,
                          expert_parallel_size=(world if args.ep == 0 else args.ep) if mc.is_moe else 1),
            logprob_batch_size=8, max_total_sequence_length=max_len, max_grad_norm=1.0,
            activation_checkpointing=(args.act_ckpt == "on"), grad_dtype="float32",
            sequence_packing=dict(enabled=True, train_mb_tokens=mb_tokens, logprob_mb_tokens=args.logprob_mb_tokens,
                                  algorithm="modified_first_fit_decreasing"),
            optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=3e-7, weight_decay=0.01, betas=[0.9, 0.999], eps=1e-8)),
            generation=dict(max_new_tokens=args.max_new_tokens, temperature=1.0, top_p=1.0, top_k=None, stop_token_ids=[],
                            kv_cache_tokens=seqs_per_gpu * gen_tp * (max_len + 64), block_size=64, max_running=max(64, seqs_per_gpu * gen_tp),
                            max_prefill_tokens=16384, free_kv_cache_on_sleep=False,
                            **({"native_cfg": {"tensor_parallel_size": gen_tp}} if gen_tp != args.tp else {})),
        ),
        "logger": dict(log_dir=tempfile.mkdtemp(prefix="rlb_bench_logs_")),
        "checkpointing": dict(enabled=False),
        "data": dict(shuffle=False),
    }
    ds = RandomTokenPromptDataset(n_prompts * steps_needed, args.prompt_len, args.prompt_len, mc.vocab_size, seed=1, task_name="synthetic")
    env = {"synthetic": HashParityEnv()}
    policy, gen, loader, _, loss_fn, logger, ck, save_state, cfg = G.setup(cfg, None, ds, None, env, model_cfg=mc)
    adv_est = G.create_advantage_estimator(cfg["grpo"], cfg["loss_fn"])
    it = iter(loader)

    def barrier_sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    phase_ms = {"generation": 0.0, "refit": 0.0, "logprobs": 0.0, "training": 0.0}
    tokens_per_step = []

    def one_step(timed: bool):
        """The GRPO step with its phases called directly; CUDA events bracket each phase when ``timed``."""
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        batch = next(it)
        repeated = batch.repeat_interleave(n_gen)
        repeated["message_log"] = [[dict(m) for m in log] for log in repeated["message_log"]]
        pf, _ = G.batched_message_log_to_flat_message(repeated["message_log"], {"token_ids": 0})
        prompt_ids = pf["token_ids"]
        ev[0].record()
        G.refit_policy_generation(policy, gen)
        ev[1].record()
        repeated, rm = G.run_multi_turn_rollout(gen, repeated, None, env, max_len, 1, greedy=False, pad_token_id=0)
        gen.finish_generation()
        ev[2].record()
        rewards = repeated["total_reward"].float()
        train_data = G.build_train_data(repeated, 0)
        train_data["rewards"] = rewards
        policy.prepare_for_lp_inference()
        train_data["prev_logprobs"] = policy.get_logprobs(train_data)["logprobs"]
        train_data["reference_policy_logprobs"] = policy.get_reference_policy_logprobs(train_data)["reference_logprobs"]
        ev[3].record()
        train_data["advantages"] = adv_est.compute_advantage(prompt_ids, rewards, train_data["token_mask"],
                                                             valid_mask=torch.ones_like(rewards))
        policy.prepare_for_training()
        res = policy.train(train_data, loss_fn, gbs=cfg["policy"]["train_global_batch_size"], mbs=4)
        ev[4].record()
        torch.cuda.synchronize()
        if rank == 0:   # progress on stderr: a run that is cut short still leaves the phases of the steps it finished
            print("[bench] step done (%s): " % ("timed" if timed else "warm-up") +
                  ", ".join("%s %.0f ms" % (n, ev[a].elapsed_time(ev[b])) for n, a, b in
                            (("refit", 0, 1), ("generation", 1, 2), ("logprobs", 2, 3), ("training", 3, 4))) +
                  ", tokens %d, status %d" % (int(train_data["input_lengths"].sum()), L.check_status()), file=sys.stderr, flush=True)
        if timed:
            for name, a, b in (("refit", 0, 1), ("generation", 1, 2), ("logprobs", 2, 3), ("training", 3, 4)):
                phase_ms[name] += ev[a].elapsed_time(ev[b])
            tokens_per_step.append(int(train_data["input_lengths"].sum()))
        return res, train_data

    # ---------------------------------------------------------------- warm-up
    for _ in range(args.warmup):
        res, td = one_step(False)
    mult_prob_err = float(sum(res["all_mb_metrics"].get("token_mult_prob_error", [0.0])))

    # ---------------------------------------------------------------- device-timed region
    sampler = ClockSampler(local_rank)
    sampler.start()
    L.Counters.reset()
    for k in gen.engine.stats:
        gen.engine.stats[k] = 0
    barrier_sync()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        one_step(True)
    t1.record()
    barrier_sync()
    dev_ms = t0.elapsed_time(t1)
    launches = L.Counters.launches
    eng = dict(gen.engine.stats)
    clocks = sampler.stop()

    # ---------------------------------------------------------------- end-to-end region (public API)
    e2e = None
    if not args.skip_e2e:
        L.Counters.reset()
        cfg["grpo"]["max_num_steps"] = args.steps
        save_state.update(current_step=0, total_steps=0)
        barrier_sync()
        w0 = time.perf_counter()
        G.grpo_train(policy, gen, loader, None, None, loss_fn, env, env, None, ck, save_state, cfg)
        barrier_sync()
        e2e_s = time.perf_counter() - w0
        e2e = dict(seconds=e2e_s, h2d=L.Counters.h2d_bytes // args.steps, d2h=L.Counters.d2h_bytes // args.steps)

    # ---------------------------------------------------------------- reduce over ranks
    status = L.check_status()
    stats = torch.tensor([dev_ms, e2e["seconds"] if e2e else 0.0, float(sum(tokens_per_step)), float(launches), mult_prob_err] +
                         [phase_ms[k] for k in ("generation", "refit", "logprobs", "training")], dtype=torch.float64, device=dev)
    PH = 5  # index of the first phase entry
    mx = stats.clone()
    sm = stats.clone()
    mn = stats.clone()
    st_all = torch.tensor([float(status)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        dist.all_reduce(st_all, op=dist.ReduceOp.MAX)
    dev_ms_max, e2e_s_max = float(mx[0]), float(mx[1])
    total_tokens = float(sm[2]) / args.tp  # all data-parallel ranks, all timed steps (the ranks of a tensor-parallel group share their data)
    ms_per_step = dev_ms_max / args.steps
    value = total_tokens / (dev_ms_max / 1e3)
    if rank == 0:
        out = {
            "metric": "grpo_tokens_per_sec (generation+refit+logprobs+training, prompt+response tokens, all GPUs)",
            "value": round(value, 1),
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 2),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic (uniform-random token prompts, random-init weights, hash-parity reward)",
            "config": {
                "model": args.model + (f"[layers={args.layers}: INVALID as benchmark]" if args.layers else ""),
                "global_batch": seqs_per_gpu * world, "seq_len": max_len,
                "prompts_per_step": n_prompts, "generations_per_prompt": n_gen, "prompt_len": args.prompt_len,
                "max_new_tokens": args.max_new_tokens,
                "name": args.config,
                "parallelism": (f"ep{world if args.ep == 0 else args.ep} experts, dense parts dp{world} (fused peer-memory dispatch / combine, generation colocated)" if mc.is_moe else
                                f"dp{world} (resident bf16 params, optimizer state sharded {world}-way, generation TP1 colocated)" if args.tp == 1 else
                                f"tp{args.tp} x dp{world // args.tp} (sequence parallel, fused peer-memory TP kernels, generation TP{gen_tp} x {world // gen_tp} engines colocated)"),
                "train_mb_tokens": mb_tokens, "data_parallel_sharding": args.sharding,
                "l2": "inputs larger than L2 (16 GB of weights streamed every pass)",
            },
            "tokens_per_sec_per_gpu": round(value / world, 1),
            "step_split_ms": {k: round(float(mx[PH + i]) / args.steps, 2) for i, k in enumerate(("generation", "refit", "logprobs", "training"))},
            # per-rank partial means sum to the global mean; the ranks of a tensor-parallel group hold the same data
            "token_mult_prob_error": round(float(sm[4]) / args.tp, 5),
            "generation_ms_per_rank": {"min": round(float(mn[PH]) / args.steps, 2), "max": round(float(mx[PH]) / args.steps, 2)},
            "optimizer_path": "fused_peer" if getattr(policy, "fused_comm", None) is not None and world // args.tp > 1 else ("local" if world // args.tp == 1 else "nccl"),
            "status": int(st_all[0]),
            "engine_rank0": {"decode_ms_per_step": round(1e3 * eng["decode_s"] / max(1, eng["decode_steps"]), 3),
                             "decode_steps": int(eng["decode_steps"]) // args.steps, "prefill_ms": round(1e3 * eng["prefill_s"] / args.steps, 1),
                             "decode_window": gen.engine.decode_window, "captured_graphs": len(gen.engine._graphs)},
            "clocks": clocks,
            "gpu_launches": int(float(mx[3])),
            "impl": "ours",
        }
        if e2e:
            out["e2e"] = {"value": round(total_tokens / e2e_s_max, 1), "unit": "tokens/s", "seconds_per_step": round(e2e_s_max / args.steps, 3),
                          "h2d_bytes_per_step": int(e2e["h2d"]), "d2h_bytes_per_step": int(e2e["d2h"])}
        print(json.dumps(out), flush=True)
    if world > 1:
        try:
            gen.shutdown()   # drops the captured decode graphs before the communicators go away
        except Exception:
            pass
        import gc

        gc.collect()   # captured graphs are gone before the communicators are
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
