"""CPU/gloo end-to-end oracle: tiny Llama-architecture policy (4 layers, d 256, 4 heads, SwiGLU 688, vocab 2048, fp32,
seed 0), 16 prompts x 4 generations of 32 tokens at temperature 1, reward = fraction of generated tokens equal to id 7,
ClippedPG with KL 0.01, 2 steps. The run must (a) make the engine and the trainer agree on the log-probabilities of
the sampled tokens and (b) give the same losses and gradient norms on one rank and on two gloo ranks, which exercises
the prompt sharding, the global-token loss normalisation and the sharded optimizer."""

import json
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(rank, world, port, out_path, tp=1, pp=1, cp=1):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(2)
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from rl_b200.algorithms.grpo import grpo_train, setup
    from rl_b200.data.datasets.synthetic import RandomTokenPromptDataset
    from rl_b200.environments.synthetic import TokenFractionEnv
    from rl_b200.models.config import preset

    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    cfg = {
        "grpo": dict(num_prompts_per_step=16, num_generations_per_prompt=4, max_num_steps=2, val_period=0, seed=0),
        "loss_fn": dict(reference_policy_kl_penalty=0.01),
        "policy": dict(precision="float32", train_global_batch_size=64, train_micro_batch_size=8, logprob_batch_size=16,
                       max_total_sequence_length=128, max_grad_norm=1.0, parallel=dict(tensor_parallel_size=tp, pipeline_parallel_size=pp, context_parallel_size=cp),
                       optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3, weight_decay=0.01)),
                       generation=dict(max_new_tokens=32, temperature=1.0, stop_token_ids=[], kv_cache_tokens=8192, block_size=16, max_running=64)),
        "logger": dict(log_dir=os.path.join(os.path.dirname(out_path), f"logs_w{world}")),
        "checkpointing": dict(enabled=False),
        "data": dict(shuffle=False),
    }
    ds = RandomTokenPromptDataset(64, 16, 64, 2048, seed=0)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}
    policy, gen, dl, vdl, loss_fn, logger, ck, ss, cfg = setup(cfg, None, ds, None, env, model_cfg=mc)
    hist = []
    grpo_train(policy, gen, dl, vdl, None, loss_fn, env, env, logger, ck, ss, cfg,
               step_callback=lambda s, m: hist.append({k: m["train"][k] for k in ("loss", "grad_norm", "reward", "token_mult_prob_error", "kl_penalty")}))
    if rank == 0:
        json.dump(hist, open(out_path, "w"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def test_grpo_oracle_one_vs_two_ranks(tmp_path):
    p1, p2 = str(tmp_path / "w1.json"), str(tmp_path / "w2.json")
    mp.spawn(_run, args=(1, _free_port(), p1), nprocs=1, join=True)
    mp.spawn(_run, args=(2, _free_port(), p2), nprocs=2, join=True)
    a, b = json.load(open(p1)), json.load(open(p2))
    assert len(a) == len(b) == 2
    for x, y in zip(a, b):
        assert x["token_mult_prob_error"] == pytest.approx(1.0, abs=1e-4)
        assert y["token_mult_prob_error"] == pytest.approx(1.0, abs=1e-4)
        assert x["reward"] == pytest.approx(y["reward"], abs=1e-9)
        assert x["loss"] == pytest.approx(y["loss"], rel=1e-4, abs=1e-6)
        assert x["grad_norm"] == pytest.approx(y["grad_norm"], rel=1e-3)
    assert a[0]["kl_penalty"] == pytest.approx(0.0, abs=1e-6)  # policy equals the reference before the first update
    assert a[1]["kl_penalty"] > 0


def test_grpo_oracle_tensor_parallel(tmp_path):
    """Two gloo ranks forming one tensor-parallel (sequence-parallel) replica reproduce the single-rank run: same
    samples (identical logits -> identical Gumbel-max draws), same loss and gradient norm."""
    p1, p2 = str(tmp_path / "w1.json"), str(tmp_path / "tp2.json")
    mp.spawn(_run, args=(1, _free_port(), p1), nprocs=1, join=True)
    mp.spawn(_run, args=(2, _free_port(), p2, 2), nprocs=2, join=True)
    a, b = json.load(open(p1)), json.load(open(p2))
    assert len(a) == len(b) == 2
    for x, y in zip(a, b):
        assert y["token_mult_prob_error"] == pytest.approx(1.0, abs=1e-4)
        assert x["reward"] == pytest.approx(y["reward"], abs=1e-9)
        assert x["loss"] == pytest.approx(y["loss"], rel=1e-3, abs=1e-6)
        assert x["grad_norm"] == pytest.approx(y["grad_norm"], rel=2e-3)


@pytest.mark.parametrize("pp,cp,tp", [(2, 1, 1), (1, 2, 1), (2, 1, 2)])
def test_grpo_oracle_pipeline_and_context_parallel(tmp_path, pp, cp, tp):
    """GRPO end to end with a pipeline- or context-parallel trainer: the stages (ranks) of the replica share the rollout
    work, every rank serves a complete copy of the weights, and the run reproduces the single-rank numbers."""
    p1, p2 = str(tmp_path / "w1.json"), str(tmp_path / "w2.json")
    mp.spawn(_run, args=(1, _free_port(), p1), nprocs=1, join=True)
    world = pp * cp * tp
    mp.spawn(_run, args=(world, _free_port(), p2, tp, pp, cp), nprocs=world, join=True)
    a, b = json.load(open(p1)), json.load(open(p2))
    assert len(a) == len(b) == 2
    for x, y in zip(a, b):
        assert y["token_mult_prob_error"] == pytest.approx(1.0, abs=1e-4)
        assert x["reward"] == pytest.approx(y["reward"], abs=1e-9)
        assert x["loss"] == pytest.approx(y["loss"], rel=1e-3, abs=1e-6)
        assert x["grad_norm"] == pytest.approx(y["grad_norm"], rel=5e-3)
