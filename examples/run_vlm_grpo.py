"""GRPO on a vision-language task (reference: examples/run_vlm_grpo.py): the prompts carry images, the engine and the
trainer both see them, the environment checks the answer.

    python examples/run_vlm_grpo.py --config examples/configs/vlm_grpo_offline.yaml grpo.max_num_steps=10
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms import grpo  # noqa: E402
from rl_b200.data.datasets.vlm import setup_vlm_data  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.environments.registry import create_env  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "vlm_grpo_offline.yaml"), argv)
    mc = model_cfg_for_tokenizer(cfg, tokenizer)
    train, val = setup_vlm_data(tokenizer, cfg["data"], mc, with_answer=False)
    envs = {"vlm": create_env("vlm", (cfg.get("env") or {}).get("vlm"))}
    policy, generation, loader, val_loader, loss_fn, logger, checkpointer, save_state, cfg = grpo.setup(
        cfg, tokenizer, train, val, envs, envs, model_cfg=mc)
    try:
        grpo.grpo_train(policy, generation, loader, val_loader, tokenizer, loss_fn, envs, envs, logger, checkpointer, save_state, cfg)
    finally:
        shutdown_distributed()


if __name__ == "__main__":
    main()
