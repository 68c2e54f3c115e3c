"""Exports the quantised deployment form of a policy trained with ``policy.quant_cfg`` (reference:
examples/modelopt/export_quantized_to_hf.py): packed NVFP4 weights, E4M3 block scales, fp32 tensor scales, calibrated input
scales and ``hf_quant_config.json``.

    python examples/converters/export_quantized_to_hf.py --ckpt results/qa-grpo/step_10/policy/weights \\
        --quant-cfg NVFP4_DEFAULT_CFG --out out/nvfp4

``--ckpt`` is a weights directory written by the trainer (HF safetensors layout; ``quantizers.pt`` beside it holds the
calibrated input ranges) or any HF model directory (ranges then stay dynamic and no input scales are written).
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

from rl_b200.models.hf_io import load_pretrained  # noqa: E402
from rl_b200.policy import qat  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--quant-cfg", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    model = load_pretrained(args.ckpt, device=args.device)
    quantizers = qat.attach(model, qat.resolve_quant_cfg(args.quant_cfg))
    ranges = os.path.join(os.path.dirname(os.path.abspath(args.ckpt)), "quantizers.pt")
    if os.path.exists(ranges):
        qat.load_state_dict(quantizers, torch.load(ranges))
    meta = qat.export_quantized(model, quantizers, args.out)
    print("saved", args.out, meta["quantization"]["quant_algo"], f"{len(quantizers)} quantised parameters")
    return meta


if __name__ == "__main__":
    main()
