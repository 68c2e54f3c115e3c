"""Supervised fine-tuning of a vision-language model (reference: examples/run_vlm_sft.py).

    python examples/run_vlm_sft.py --config examples/configs/vlm_sft_offline.yaml sft.max_num_steps=20
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms import sft  # noqa: E402
from rl_b200.data.datasets.vlm import setup_vlm_data  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "vlm_sft_offline.yaml"), argv)
    mc = model_cfg_for_tokenizer(cfg, tokenizer)
    train, val = setup_vlm_data(tokenizer, cfg["data"], mc, with_answer=True)
    policy, loader, val_loader, loss_fn, logger, ck, save_state, cfg = sft.setup_sft(cfg, tokenizer, train, val, model_cfg=mc)
    try:
        sft.sft_train(policy, loader, val_loader, tokenizer, loss_fn, logger, ck, save_state, cfg)
    finally:
        shutdown_distributed()


if __name__ == "__main__":
    main()
