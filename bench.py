"""Headline benchmark: one GRPO step (generation + refit + log-probabilities + training) on the Llama-3.1-8B
architecture, N GPUs of one node, synthetic prompts, random-init weights.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per GPU by torch.distributed.run)
    python bench.py --impl reference ...                     (the unmodified reference, when it can be installed)

Work per step and per GPU is fixed (weak scaling): 8 prompts x 8 generations, prompts of 256 random tokens, 1024
generated tokens each (stop tokens disabled so every response runs to the limit), one optimizer step over the global
batch of 64*N sequences. At N = 8 this is the 64 prompts x 8 generations configuration.

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


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3.1-8b")
    ap.add_argument("--prompts-per-gpu", type=int, default=8)
    ap.add_argument("--generations", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--max-new-tokens", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (makes the run invalid as a benchmark)")
    ap.add_argument("--train-mb-tokens", type=int, default=5120, help="tokens per training micro-batch (the same at every N)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size of the trainer and the engine (with sequence parallelism); "
                    "the headline configuration is --tp 1")
    ap.add_argument("--act-ckpt", default="auto", choices=["auto", "on", "off"],
                    help="activation checkpointing in training (auto = off: with 5120-token micro-batches the activations of "
                         "Llama-3.1-8B fit next to the unsharded optimizer state even on 1 GPU)")
    return ap.parse_args()


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
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
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
    cfg = {
        "grpo": dict(num_prompts_per_step=n_prompts, num_generations_per_prompt=n_gen, max_num_steps=10**9, val_period=0, seed=0,
                     normalize_rewards=True, use_leave_one_out_baseline=True),
        "loss_fn": dict(reference_policy_kl_penalty=0.01, ratio_clip_min=0.2, ratio_clip_max=0.2),
        "policy": dict(
            model_name=None, precision="bfloat16", train_global_batch_size=seqs_per_gpu * world, train_micro_batch_size=4,
            parallel=dict(tensor_parallel_size=args.tp, sequence_parallel=args.tp > 1),
            logprob_batch_size=8, max_total_sequence_length=max_len, max_grad_norm=1.0,
            activation_checkpointing=(args.act_ckpt == "on"), grad_dtype="float32",
            sequence_packing=dict(enabled=True, train_mb_tokens=mb_tokens, logprob_mb_tokens=20480,
                                  algorithm="modified_first_fit_decreasing"),
            optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=3e-7, weight_decay=0.01, betas=[0.9, 0.999], eps=1e-8)),
            generation=dict(max_new_tokens=args.max_new_tokens, temperature=1.0, top_p=1.0, top_k=None, stop_token_ids=[],
                            kv_cache_tokens=seqs_per_gpu * args.tp * (max_len + 64), block_size=64, max_running=max(64, seqs_per_gpu * args.tp),
                            max_prefill_tokens=16384, free_kv_cache_on_sleep=False),
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
    barrier_sync()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        one_step(True)
    t1.record()
    barrier_sync()
    dev_ms = t0.elapsed_time(t1)
    launches = L.Counters.launches
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
    stats = torch.tensor([dev_ms, e2e["seconds"] if e2e else 0.0, float(sum(tokens_per_step)), float(launches), mult_prob_err] +
                         [phase_ms[k] for k in ("generation", "refit", "logprobs", "training")], dtype=torch.float64, device=dev)
    PH = 5  # index of the first phase entry
    mx = stats.clone()
    sm = stats.clone()
    if world > 1:
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
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
                "parallelism": (f"dp{world} (resident bf16 params, optimizer state sharded {world}-way, generation TP1 colocated)" if args.tp == 1 else
                                f"tp{args.tp} x dp{world // args.tp} (sequence parallel, fused peer-memory TP kernels, generation TP{args.tp} colocated)"),
                "l2": "inputs larger than L2 (16 GB of weights streamed every pass)",
            },
            "tokens_per_sec_per_gpu": round(value / world, 1),
            "step_split_ms": {k: round(float(mx[PH + i]) / args.steps, 2) for i, k in enumerate(("generation", "refit", "logprobs", "training"))},
            "token_mult_prob_error": round(float(sm[4]), 5),  # per-rank partial means sum to the global mean
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
        torch.cuda.synchronize()
        dist.barrier()
        if args.tp > 1:
            # a tensor-parallel engine captures NCCL broadcasts in its decode graphs; tearing the process groups down after
            # that was seen to stall in the NCCL watchdog, so these ranks leave without the teardown (all work is complete)
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
