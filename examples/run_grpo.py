"""GRPO / DAPO / GSPO / Reinforce++ entrypoint.

    python examples/run_grpo.py --config examples/configs/grpo_math_1B.yaml grpo.max_num_steps=10
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/run_grpo.py --config examples/configs/grpo_math_8B.yaml

Same flow as the reference driver (examples/run_grpo.py:71-254): config -> tokenizer -> data + environments -> ``setup``
-> synchronous or asynchronous trainer. One process per GPU replaces the Ray cluster.
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms import grpo  # noqa: E402
from rl_b200.data.datasets.registry import setup_response_data  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "grpo_math_1B.yaml"), argv)
    dataset, val_dataset, task_to_env, val_task_to_env = setup_response_data(tokenizer, cfg["data"], cfg.get("env"))
    from rl_b200.distributed.roles import current_layout

    layout = current_layout()
    if layout is not None and layout.role != "colocated":
        # split job (policy.generation.colocated.enabled: false): generation ranks serve, training ranks train, concurrently
        return _run_split(cfg, layout, tokenizer, dataset, task_to_env, val_task_to_env)
    policy, generation, loader, val_loader, loss_fn, logger, checkpointer, save_state, cfg = grpo.setup(
        cfg, tokenizer, dataset, val_dataset, task_to_env, val_task_to_env, model_cfg=model_cfg_for_tokenizer(cfg, tokenizer))
    try:
        if (cfg["grpo"].get("async_grpo") or {}).get("enabled"):
            from rl_b200.algorithms.async_grpo import async_grpo_train

            async_grpo_train(policy, generation, loader, tokenizer, loss_fn, task_to_env, logger, checkpointer, save_state, cfg)
        elif (cfg.get("data_plane") or {}).get("enabled"):
            # samples travel through the data plane between rollout and optimizer step (the reference picks its
            # TransferQueue-mediated trainer by the same key)
            from rl_b200.algorithms.grpo_sync import grpo_train_sync

            grpo_train_sync(policy, generation, loader, val_loader, tokenizer, loss_fn, task_to_env, val_task_to_env, logger,
                            checkpointer, save_state, cfg)
        else:
            grpo.grpo_train(policy, generation, loader, val_loader, tokenizer, loss_fn, task_to_env, val_task_to_env, logger,
                            checkpointer, save_state, cfg)
    finally:
        for env in {id(e): e for e in list(task_to_env.values()) + list(val_task_to_env.values())}.values():
            env.shutdown()
        shutdown_distributed()


def _run_split(cfg, layout, tokenizer, dataset, task_to_env, val_task_to_env):
    from rl_b200.algorithms import noncolocated as nc

    mc = model_cfg_for_tokenizer(cfg, tokenizer)
    try:
        if layout.role == "generation":
            generation = nc.build_generation_rank(cfg, tokenizer, mc, layout.device)
            stats = nc.generation_service(layout, cfg, generation, dataset, tokenizer, task_to_env)
            print(f"[generation rank {layout.role_rank}] {stats}", flush=True)
        else:
            policy, _, _, _, loss_fn, logger, checkpointer, save_state, cfg = grpo.setup(
                cfg, tokenizer, dataset, None, task_to_env, val_task_to_env, model_cfg=mc, build_generation=False)
            nc.noncolocated_grpo_train(policy, layout, loss_fn, logger, checkpointer, save_state, cfg, tokenizer)
    finally:
        for env in {id(e): e for e in list(task_to_env.values()) + list(val_task_to_env.values())}.values():
            env.shutdown()
        shutdown_distributed()


if __name__ == "__main__":
    main()
