"""GRPO driven by ONE controller process over a group of worker processes (the reference's driver / worker-group shape):

    python examples/run_grpo_controller.py --config examples/configs/grpo_arithmetic_offline.yaml cluster.gpus_per_node=2

The controller loads the recipe, the data and the environments, builds a virtual cluster of ``cluster.gpus_per_node x
cluster.num_nodes`` bundles, starts one policy worker per bundle (``rl_b200/policy/lm_policy.py::Policy`` over
``rl_b200/distributed/worker_groups.py``) and runs the ordinary GRPO loop against that facade: batches are sharded over the
data-parallel workers, results are gathered back. ``torchrun examples/run_grpo.py`` (every rank its own driver) is the faster
path for plain training; this one is for jobs that want a single point of control.
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms import grpo  # noqa: E402
from rl_b200.algorithms.utils import get_tokenizer  # noqa: E402
from rl_b200.data.datasets.registry import setup_response_data  # noqa: E402
from rl_b200.distributed.virtual_cluster import cluster_from_config  # noqa: E402
from rl_b200.policy.lm_policy import Policy  # noqa: E402
from rl_b200.utils.cli import apply_env_vars, model_cfg_for_tokenizer, parse_args_and_overrides, validate_recipe  # noqa: E402
from rl_b200.utils.config import load_config  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    from dataclasses import asdict

    path, overrides = parse_args_and_overrides(argv)
    cfg = load_config(path or os.path.join(HERE, "configs", "grpo_math_1B.yaml"), overrides)
    apply_env_vars(cfg)
    validate_recipe(cfg)
    tokenizer = get_tokenizer((cfg.get("policy") or {}).get("tokenizer") or {"name": "byte"})
    dataset, val_dataset, task_to_env, val_task_to_env = setup_response_data(tokenizer, cfg["data"], cfg.get("env"))
    cluster = cluster_from_config(cfg.get("cluster") or {}, colocated_groups=1, name="grpo")
    mc = model_cfg_for_tokenizer(cfg, tokenizer)
    needs_ref = (cfg.get("loss_fn") or {}).get("reference_policy_kl_penalty", 0.01) != 0
    policy = Policy(cluster, cfg["policy"], tokenizer_cfg=(cfg.get("policy") or {}).get("tokenizer"), init_reference_model=needs_ref,
                    model_cfg=asdict(mc) if mc is not None else None, seed=int((cfg.get("grpo") or {}).get("seed", 42)),
                    backend=(cfg.get("cluster") or {}).get("backend"))
    try:
        policy_, generation, loader, val_loader, loss_fn, logger, checkpointer, save_state, cfg = grpo.setup(
            cfg, tokenizer, dataset, val_dataset, task_to_env, val_task_to_env, policy=policy)
        grpo.grpo_train(policy, generation, loader, val_loader, tokenizer, loss_fn, task_to_env, val_task_to_env, logger, checkpointer,
                        save_state, cfg)
    finally:
        for env in {id(e): e for e in list(task_to_env.values()) + list(val_task_to_env.values())}.values():
            env.shutdown()
        policy.shutdown()
        cluster.shutdown()


if __name__ == "__main__":
    main()
