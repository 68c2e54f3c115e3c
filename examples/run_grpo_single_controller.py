"""GRPO driven by the single controller: rollout pump and train pump over the data plane.

    python examples/run_grpo_single_controller.py --config examples/configs/grpo_single_controller.yaml grpo.max_num_steps=10

Counterpart of the reference's examples/run_grpo_single_controller.py (controller: algorithms/single_controller.py:92).
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms import grpo  # noqa: E402
from rl_b200.algorithms.single_controller import SingleController  # noqa: E402
from rl_b200.data.datasets.registry import setup_response_data  # noqa: E402
from rl_b200.data_plane import create_data_plane  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "grpo_single_controller.yaml"), argv)
    dataset, val_dataset, task_to_env, val_task_to_env = setup_response_data(tokenizer, cfg["data"], cfg.get("env"))
    policy, generation, loader, _, loss_fn, logger, checkpointer, save_state, cfg = grpo.setup(
        cfg, tokenizer, dataset, val_dataset, task_to_env, val_task_to_env, model_cfg=model_cfg_for_tokenizer(cfg, tokenizer))
    if world > 1:
        (cfg.setdefault("single_controller", {}))["pump_mode"] = "interleaved"   # all ranks must enter collectives in one order
    controller = SingleController(policy, generation, loader, tokenizer, loss_fn, task_to_env, cfg,
                                  data_plane=create_data_plane(cfg.get("data_plane")), logger=logger, checkpointer=checkpointer,
                                  save_state=save_state)
    try:
        return controller.run()
    finally:
        for env in {id(e): e for e in list(task_to_env.values()) + list(val_task_to_env.values())}.values():
            env.shutdown()
        shutdown_distributed()


if __name__ == "__main__":
    main()
