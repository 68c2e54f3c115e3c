"""Supervised fine-tuning entrypoint (reference: examples/run_sft.py:57-229).

    python examples/run_sft.py --config examples/configs/sft.yaml sft.max_num_steps=20
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms import sft  # noqa: E402
from rl_b200.data.datasets.registry import ProcessedDataset, load_raw_dataset  # noqa: E402
from rl_b200.data.interfaces import TaskDataSpec  # noqa: E402
from rl_b200.data.processors import get_processor  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def setup_data(tokenizer, data_cfg: dict, default_processor: str = "sft_processor"):
    """``data.train`` / ``data.validation`` dataset specs -> processed train / validation datasets."""
    max_len = data_cfg.get("max_input_seq_length")
    default = data_cfg.get("default") or {}

    def build(spec, split):
        if spec is None:
            return None
        spec = {**default, **spec}
        if spec.get("dataset_name") == "random_sft":
            from rl_b200.data.datasets.preference import RandomSFTDataset

            return RandomSFTDataset(spec.get("num_samples", 256) if split == "train" else spec.get("num_val_samples", 32),
                                    spec.get("vocab_size", 256), seed=spec.get("seed", 0) + (split != "train"))
        if spec.get("dataset_name") == "random_preference":
            from rl_b200.data.datasets.preference import RandomPreferenceDataset

            return RandomPreferenceDataset(spec.get("num_samples", 256) if split == "train" else spec.get("num_val_samples", 32),
                                           spec.get("vocab_size", 256), seed=spec.get("seed", 0) + (split != "train"))
        recs, proc = load_raw_dataset(spec, split)
        if recs is None:
            return None
        ts = TaskDataSpec(task_name=spec.get("task_name", "sft"), prompt_file=spec.get("prompt_file"),
                          system_prompt_file=spec.get("system_prompt_file"), prompt=spec.get("prompt"))
        name = spec.get("processor") or (proc if proc in ("sft_processor", "preference_processor") else default_processor)
        return ProcessedDataset(recs, tokenizer, ts, get_processor(name), max_len)

    return build(data_cfg.get("train"), "train"), build(data_cfg.get("validation") or data_cfg.get("train"), "validation")


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "sft.yaml"), argv)
    train, val = setup_data(tokenizer, cfg["data"])
    policy, loader, val_loader, loss_fn, logger, ck, save_state, cfg = sft.setup_sft(cfg, tokenizer, train, val,
                                                                                   model_cfg=model_cfg_for_tokenizer(cfg, tokenizer))
    try:
        sft.sft_train(policy, loader, val_loader, tokenizer, loss_fn, logger, ck, save_state, cfg)
    finally:
        shutdown_distributed()


if __name__ == "__main__":
    main()
