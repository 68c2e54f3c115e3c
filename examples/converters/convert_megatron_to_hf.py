"""Converts a Megatron-core distributed checkpoint into a HuggingFace safetensors directory (reference:
examples/converters/convert_megatron_to_hf.py), without a Megatron installation.

    python examples/converters/convert_megatron_to_hf.py --megatron-ckpt-path results/step_10/policy/weights/iter_0000000 \\
        --hf-config meta-llama/Llama-3.1-8B-Instruct --hf-ckpt-path out/hf

``--hf-config``: a directory (or file) with the model's HuggingFace ``config.json``, or a preset name of this framework.
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from rl_b200.checkpoint.megatron_names import convert_megatron_to_hf  # noqa: E402
from rl_b200.models.config import PRESETS, ModelConfig, preset  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--megatron-ckpt-path", required=True)
    ap.add_argument("--hf-config", required=True)
    ap.add_argument("--hf-ckpt-path", required=True)
    a = ap.parse_args(argv)
    if a.hf_config in PRESETS:
        cfg = preset(a.hf_config)
    else:
        cfg = ModelConfig.from_pretrained(a.hf_config if os.path.isdir(a.hf_config) else os.path.dirname(a.hf_config))
    print("saved", convert_megatron_to_hf(a.megatron_ckpt_path, a.hf_ckpt_path, cfg))


if __name__ == "__main__":
    main()
