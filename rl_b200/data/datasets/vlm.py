"""Vision-language data: a processor that turns ``{image, question, answer}`` records into message logs carrying image
patch rows, and a synthetic image dataset for runs without network access.

The user turn's text contains the literal ``<image>`` once per image; after the chat template is applied, every such
marker becomes ``n_patches`` copies of the model's image placeholder token, and the patches travel with the message as
``pixel_patches`` ([n_patches, C * p * p]) and ``image_sizes``. Counterpart of the VLM processors in
nemo_rl/data/processors.py and the clevr / geometry VLM datasets.
"""

from __future__ import annotations

import random
from typing import Optional

import torch

from rl_b200.data.interfaces import DatumSpec, TaskDataSpec
from rl_b200.data.llm_message_utils import get_formatted_message_log
from rl_b200.data.multimodal_utils import patchify

IMAGE_MARK = "<image>"
COLOURS = {"red": (0.9, 0.1, 0.1), "green": (0.1, 0.8, 0.1), "blue": (0.1, 0.1, 0.9), "white": (0.95, 0.95, 0.95), "black": (0.05, 0.05, 0.05),
           "yellow": (0.9, 0.9, 0.1)}


class SyntheticColourDataset:
    """Images of one dominant colour (with noise and a darker border) and the question which colour it is."""

    def __init__(self, num_samples: int = 512, image_size: int = 16, colours: Optional[list[str]] = None, noise: float = 0.05, seed: int = 0):
        rng = random.Random(seed)
        g = torch.Generator().manual_seed(seed)
        names = colours or list(COLOURS)
        self.records = []
        for _ in range(num_samples):
            name = rng.choice(names)
            img = torch.tensor(COLOURS[name]).view(3, 1, 1).expand(3, image_size, image_size).clone()
            img += noise * torch.randn(img.shape, generator=g)
            img[:, 0, :] *= 0.5
            img[:, :, 0] *= 0.5
            self.records.append({"image": img.clamp(0, 1), "question": "What colour is this?", "answer": name, "task_name": "vlm"})

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        return self.records[i]


def _splice_image_tokens(log, tokenizer, images, patch: int, image_token_id: int):
    """Re-tokenises messages whose text holds ``<image>`` markers: marker k -> one placeholder token per patch of image k."""
    k = 0
    for m in log:
        if IMAGE_MARK not in m["content"]:
            continue
        parts = m["content"].split(IMAGE_MARK)
        ids, rows, sizes = [], [], []
        for j, part in enumerate(parts):
            if part:
                ids += tokenizer(part, add_special_tokens=False)["input_ids"]
            if j + 1 < len(parts):
                p = patchify(images[k], patch)
                k += 1
                ids += [image_token_id] * p.shape[0]
                rows.append(p)
                sizes.append(p.shape[0])
        m["token_ids"] = torch.tensor(ids, dtype=torch.long)
        m["pixel_patches"] = torch.cat(rows)
        m["image_sizes"] = sizes
    assert k == len(images), f"{len(images)} images for {k} <image> markers"
    return log


def make_vlm_processor(patch: int, image_token_id: int, with_answer: bool):
    """Processor factory: ``with_answer`` appends the reference answer as the assistant turn (SFT); without it the log ends
    at the generation prompt and the answer goes to the environment (RL)."""

    def proc(rec: dict, spec: TaskDataSpec, tokenizer, max_seq_length: Optional[int], idx: int) -> DatumSpec:
        images = rec["images"] if "images" in rec else [rec["image"]]
        q = rec["question"] if IMAGE_MARK in rec["question"] else IMAGE_MARK * len(images) + rec["question"]
        msgs = [{"role": "user", "content": spec.prompt.format(q) if (spec is not None and spec.prompt) else q}]
        if with_answer:
            msgs.append({"role": "assistant", "content": str(rec["answer"])})
            log = get_formatted_message_log(msgs, tokenizer)
        else:
            log = get_formatted_message_log(msgs, tokenizer, add_eos_token=False, add_generation_prompt=True)
        log = _splice_image_tokens(log, tokenizer, images, patch, image_token_id)
        length = sum(int(m["token_ids"].numel()) for m in log)
        mult = 1.0 if max_seq_length is None or length <= max_seq_length else 0.0
        return {"message_log": log, "length": length, "extra_env_info": {"ground_truth": str(rec["answer"])}, "loss_multiplier": mult,
                "idx": idx, "task_name": rec.get("task_name", "vlm")}

    return proc


class ProcessedVLMDataset:
    def __init__(self, raw, tokenizer, patch: int, image_token_id: int, with_answer: bool, max_seq_length: Optional[int] = None, spec=None):
        self.raw, self.tok, self.max_len, self.spec = raw, tokenizer, max_seq_length, spec
        self.proc = make_vlm_processor(patch, image_token_id, with_answer)

    def __len__(self):
        return len(self.raw)

    def __getitem__(self, i):
        return self.proc(self.raw[i], self.spec, self.tok, self.max_len, i)


def setup_vlm_data(tokenizer, data_cfg: dict, model_cfg, with_answer: bool):
    """``data.train`` / ``data.validation`` -> processed datasets. ``dataset_name``: ``synthetic_colours`` (offline) or
    ``jsonl`` (``path``; records ``{image_path | image (nested lists), question, answer}``)."""
    from rl_b200.models.vision import vision_config

    patch = vision_config(model_cfg)["patch_size"]

    def build(spec, split):
        if spec is None:
            return None
        name = spec.get("dataset_name", "synthetic_colours")
        if name == "synthetic_colours":
            n = spec.get("num_samples", 512) if split == "train" else spec.get("num_val_samples", 64)
            raw = SyntheticColourDataset(n, int(spec.get("image_size", 16)), spec.get("colours"), seed=int(spec.get("seed", 0)) + (split != "train"))
        elif name == "jsonl":
            from rl_b200.data.datasets.registry import JsonlRecords

            raw = []
            for r in JsonlRecords(spec["path"]).records:
                img = torch.tensor(r["image"], dtype=torch.float32) if "image" in r else torch.load(r["image_path"])
                raw.append({**r, "image": img})
        else:
            raise ValueError(f"unknown VLM dataset {name!r}")
        return ProcessedVLMDataset(raw, tokenizer, patch, model_cfg.image_token_id, with_answer, data_cfg.get("max_input_seq_length"))

    return build(data_cfg.get("train"), "train"), build(data_cfg.get("validation"), "validation")
