"""On-policy distillation entrypoint: student rollouts scored by a teacher's top-k logits (reference:
examples/run_distillation.py, nemo_rl/algorithms/distillation.py:677).

    python examples/run_distillation.py --config examples/configs/distillation_math.yaml
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms import distillation  # noqa: E402
from rl_b200.data.datasets.registry import setup_response_data  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "distillation_math.yaml"), argv)
    dataset, val_dataset, task_to_env, _ = setup_response_data(tokenizer, cfg["data"], cfg.get("env"))
    student_cfg = model_cfg_for_tokenizer(cfg, tokenizer)
    teacher_cfg = model_cfg_for_tokenizer({"policy": cfg.get("teacher") or cfg["policy"]}, tokenizer)
    student, teacher, generation, loader, loss_fn, logger, ck, save_state, cfg = distillation.setup(
        cfg, tokenizer, dataset, val_dataset, task_to_env, student_cfg=student_cfg, teacher_cfg=teacher_cfg)
    try:
        distillation.distillation_train(student, teacher, generation, loader, tokenizer, loss_fn, task_to_env, logger, ck, save_state, cfg)
    finally:
        for env in task_to_env.values():
            env.shutdown()
        shutdown_distributed()


if __name__ == "__main__":
    main()
