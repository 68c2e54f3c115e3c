"""pass@k / cons@k evaluation of a model on a verifiable dataset (reference: examples/run_eval.py, nemo_rl/evals/eval.py).

    python examples/run_eval.py --config examples/configs/evals/eval.yaml eval.num_tests_per_prompt=8 eval.k_value=4
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms.grpo import _ShardedPromptLoader  # noqa: E402
from rl_b200.data.collate import rl_collate_fn  # noqa: E402
from rl_b200.data.datasets.registry import setup_response_data  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.evals.eval import run_env_eval  # noqa: E402
from rl_b200.policy.worker import PolicyWorker  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "evals", "eval.yaml"), argv)
    _, val, _, envs = setup_response_data(tokenizer, {**cfg["data"], "train": None}, cfg.get("env"), is_eval=True)
    policy = PolicyWorker(cfg["policy"], model_cfg=model_cfg_for_tokenizer(cfg, tokenizer), tokenizer=tokenizer, init_optimizer=False,
                          init_reference_model=False, seed=(cfg.get("eval") or {}).get("seed", 42))
    generation = policy.build_generation(cfg["policy"].get("generation"))
    bs = max(world, (min(int((cfg.get("eval") or {}).get("batch_size", 64)), len(val)) // world) * world)
    loader = _ShardedPromptLoader(val, bs, rl_collate_fn, False, 0, rank, world)
    try:
        out = run_env_eval(generation, loader, tokenizer, envs, cfg)
        if rank == 0:
            print("=" * 60)
            print(f"model={cfg['policy']['model_name']} dataset={cfg['data']['validation'].get('dataset_name')}")
            print(f"{out['metric']}={out['score']:.4f} over {out['num_prompts']} prompts x {out['num_tests_per_prompt']} samples")
            print("=" * 60)
    finally:
        for env in envs.values():
            env.shutdown()
        shutdown_distributed()


if __name__ == "__main__":
    main()
