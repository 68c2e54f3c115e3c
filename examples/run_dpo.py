"""DPO entrypoint on preference data (reference: examples/run_dpo.py).

    python examples/run_dpo.py --config examples/configs/dpo.yaml dpo.max_num_steps=20
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from examples.run_sft import setup_data  # noqa: E402
from rl_b200.algorithms import sft  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "dpo.yaml"), argv)
    train, val = setup_data(tokenizer, cfg["data"], default_processor="preference_processor")
    policy, loader, val_loader, loss_fn, logger, ck, save_state, cfg = sft.setup_dpo(cfg, tokenizer, train, val,
                                                                                    model_cfg=model_cfg_for_tokenizer(cfg, tokenizer))
    try:
        sft.dpo_train(policy, loader, val_loader, tokenizer, loss_fn, logger, ck, save_state, cfg)
    finally:
        shutdown_distributed()


if __name__ == "__main__":
    main()
