"""Asynchronous GRPO on split rank sets (gloo, 2 training + 2 generation ranks on CPU): generation ranks produce
trajectories while training ranks train; weights travel trainer -> generation ranks over the sync communicator;
trajectory ages stay within ``max_trajectory_age_steps``; both sets are busy at the same time."""

import os
import socket
import sys
import time

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cfg(max_age, in_flight, steps):
    return {
        "grpo": dict(num_prompts_per_step=4, num_generations_per_prompt=2, max_num_steps=steps, seed=3, val_period=0,
                     async_grpo=dict(enabled=True, max_trajectory_age_steps=max_age, in_flight_weight_updates=in_flight)),
        "loss_fn": dict(reference_policy_kl_penalty=0.0, use_importance_sampling_correction=True),
        "policy": dict(model_name=None, precision="float32", train_global_batch_size=8, train_micro_batch_size=2, max_total_sequence_length=48,
                       optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=5e-3, weight_decay=0.0)),
                       generation=dict(max_new_tokens=8, temperature=1.0, stop_token_ids=[], kv_cache_tokens=2048, block_size=16, max_running=8,
                                       colocated=dict(enabled=False, resources=dict(gpus_per_node=2, num_nodes=1)))),
        "checkpointing": dict(enabled=False), "logger": dict(log_dir=os.path.join("/tmp", f"rlb_nc_logs_{os.getpid()}")), "data": dict(shuffle=False),
    }


def _entry(rank, world, port, max_age, in_flight, steps, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    torch.manual_seed(0)
    torch.set_num_threads(2)
    import torch.distributed as dist

    from rl_b200.algorithms import grpo, noncolocated as nc
    from rl_b200.data.datasets.synthetic import RandomTokenPromptDataset
    from rl_b200.distributed.roles import init_roles
    from rl_b200.environments.synthetic import HashParityEnv
    from rl_b200.models.config import preset

    cfg = _cfg(max_age, in_flight, steps)
    layout = init_roles(cfg, backend="gloo")
    assert (layout.role, layout.role_world) == (("train", 2) if rank < 2 else ("generation", 2))
    assert dist.get_world_size() == 2    # every set has its own default group
    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    ds = RandomTokenPromptDataset(4 * (steps + 2), 6, 10, mc.vocab_size, seed=1, task_name="synthetic")
    env = {"synthetic": HashParityEnv()}
    out = {"role": layout.role}
    if layout.role == "generation":
        gen = nc.build_generation_rank(cfg, None, mc, layout.device)
        w0 = next(gen.engine.model.parameters()).detach().clone()
        busy = []
        stats = nc.generation_service(layout, cfg, gen, ds, None, env, step_callback=lambda s, t, v: busy.append((time.time(), s, t, v)))
        out.update(stats=stats, busy=busy, weights_moved=bool((next(gen.engine.model.parameters()) - w0).abs().max() > 0))
    else:
        policy, _, _, _, loss_fn, logger, ck, save_state, cfg = grpo.setup(cfg, None, ds, None, env, model_cfg=mc, build_generation=False)
        steps_seen = []
        last = nc.noncolocated_grpo_train(policy, layout, loss_fn, None, ck, save_state, cfg, None,
                                          step_callback=lambda s, m: steps_seen.append((time.time(), s, m["train"]["trajectory_age"], m["train"]["loss"])))
        out.update(steps=steps_seen, first_param=float(next(policy.model.parameters()).flatten()[0]))
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()


def _run(max_age, in_flight, steps=4):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_entry, args=(r, 4, port, max_age, in_flight, steps, q)) for r in range(4)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    res = {}
    while not q.empty():
        r, v = q.get()
        res[r] = v
    for p in procs:
        assert p.exitcode == 0, res
    return res


@pytest.mark.parametrize("max_age,in_flight", [(1, False), (2, True)])
def test_split_job_trains_while_generating(max_age, in_flight):
    steps = 4
    res = _run(max_age, in_flight, steps)
    trainers, gens = [res[0], res[1]], [res[2], res[3]]
    for t in trainers:
        assert [s for _, s, _, _ in t["steps"]] == list(range(1, steps + 1))
        assert all(0 <= age <= max_age for _, _, age, _ in t["steps"]), t["steps"]
        assert all(torch.isfinite(torch.tensor(l)) for *_, l in t["steps"])
    assert trainers[0]["first_param"] == trainers[1]["first_param"]            # the training set stays in sync
    shards = sum(g["stats"]["shards"] for g in gens)
    assert shards >= steps * 2                                                  # two trainer shards per step
    for g in gens:
        assert g["weights_moved"] and g["stats"]["weight_updates"] >= 2         # initial weights + at least one refit
        assert g["stats"]["final_version"] == steps + 1
    # overlap: some shard was generated after the first optimizer step finished and before the last one did
    t_first, t_last = trainers[0]["steps"][0][0], trainers[0]["steps"][-1][0]
    assert any(t_first < ts < t_last for g in gens for ts, *_ in g["busy"])
    # trajectories of step >= 2 were produced with refitted weights (version > 1)
    assert any(v > 1 for g in gens for _, s, _, v in g["busy"] if s >= 2)


def test_generation_ranks_from_config():
    from rl_b200.distributed.roles import generation_ranks_from_config

    assert generation_ranks_from_config({"policy": {"generation": {"colocated": {"enabled": True}}}}, 8) == 0
    assert generation_ranks_from_config({"policy": {"generation": {"colocated": {"enabled": False, "resources": {"gpus_per_node": 3}}}}}, 8) == 3
    assert generation_ranks_from_config({"policy": {"generation": {"colocated": {"enabled": False}}}}, 8) == 4
    assert generation_ranks_from_config({"grpo": {"async_grpo": {"generation_ranks": 2}}}, 8) == 2
    with pytest.raises(ValueError):
        generation_ranks_from_config({"grpo": {"async_grpo": {"generation_ranks": 8}}}, 8)
