"""Merges a LoRA adapter into its base model and writes a plain HuggingFace checkpoint
(reference: examples/converters/convert_lora_to_hf.py).

    python examples/converters/convert_lora_to_hf.py --base-ckpt path/to/base_hf --adapter path/to/adapter_dir --out merged_hf
"""

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from rl_b200.models.hf_io import load_lora_adapter, load_pretrained, merge_lora, save_pretrained  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-ckpt", required=True)
    ap.add_argument("--adapter", required=True)
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    ac = json.load(open(os.path.join(a.adapter, "adapter_config.json")))
    lora = {"enabled": True, "dim": ac["r"], "alpha": ac["lora_alpha"], "target_modules": ac.get("target_modules")}
    model = load_pretrained(a.base_ckpt, lora=lora)
    load_lora_adapter(model, a.adapter)
    merge_lora(model)
    model.lora_cfg = None
    for layer in model.layers:  # drop the (now zero) adapters so that only HF tensors are written
        layer.self_attn.qkv_lora = layer.self_attn.o_lora = None
        layer.mlp.gate_up_lora = layer.mlp.down_lora = None
    save_pretrained(model, a.out)
    print("saved", a.out)


if __name__ == "__main__":
    main()
