"""Converts a training checkpoint (sharded flat-buffer DCP directory) into a HuggingFace safetensors directory
(reference: examples/converters/convert_dcp_to_hf.py).

    python examples/converters/convert_dcp_to_hf.py --dcp-ckpt-path results/grpo/step_10/policy/weights --hf-ckpt-path out/hf
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from rl_b200.checkpoint.io import convert_dcp_to_hf  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--dcp-ckpt-path", required=True)
    ap.add_argument("--hf-ckpt-path", required=True)
    args = ap.parse_args(argv)
    print("saved", convert_dcp_to_hf(args.dcp_ckpt_path, args.hf_ckpt_path))


if __name__ == "__main__":
    main()
