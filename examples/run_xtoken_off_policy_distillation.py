"""Off-policy distillation between a teacher and a student that use different tokenizers.

    python examples/run_xtoken_off_policy_distillation.py --config examples/configs/xtoken_distillation_offline.yaml

Counterpart of the reference's examples/run_xtoken_off_policy_distillation.py.
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms import xtoken_off_policy_distillation as xt  # noqa: E402
from rl_b200.algorithms.utils import get_tokenizer  # noqa: E402
from rl_b200.data.datasets.registry import load_text_corpus  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "xtoken_distillation_offline.yaml"), argv)
    teacher_tok = get_tokenizer(cfg["teacher"]["tokenizer"])
    dataset = load_text_corpus(cfg["data"])
    student_cfg = model_cfg_for_tokenizer(cfg, tokenizer)
    teacher_cfg = model_cfg_for_tokenizer({"policy": cfg["teacher"]}, teacher_tok)
    parts = xt.setup(cfg, tokenizer, teacher_tok, dataset, student_cfg=student_cfg, teacher_cfg=teacher_cfg)
    try:
        return xt.xtoken_distillation_train(*parts)
    finally:
        shutdown_distributed()


if __name__ == "__main__":
    main()
