"""PPO (policy + learned critic, GAE / VAPO) entrypoint (reference: examples/run_ppo.py).

    python examples/run_ppo.py --config examples/configs/ppo_math_1B.yaml ppo.max_num_steps=10
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms import ppo  # noqa: E402
from rl_b200.data.datasets.registry import setup_response_data  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "ppo_math_1B.yaml"), argv)
    dataset, val_dataset, task_to_env, _ = setup_response_data(tokenizer, cfg["data"], cfg.get("env"))
    mc = model_cfg_for_tokenizer(cfg, tokenizer)
    policy, value, generation, loader, ploss, vloss, logger, ck, save_state, cfg = ppo.setup(cfg, tokenizer, dataset, val_dataset, task_to_env,
                                                                                           model_cfg=mc)
    try:
        trainer = ppo.async_ppo_train if (cfg["ppo"].get("async_ppo") or {}).get("enabled") else ppo.ppo_train
        trainer(policy, value, generation, loader, tokenizer, ploss, vloss, task_to_env, logger, ck, save_state, cfg)
    finally:
        for env in task_to_env.values():
            env.shutdown()
        shutdown_distributed()


if __name__ == "__main__":
    main()
