"""Synthetic prompt datasets: uniform-random token prompts for benchmarks and the CPU oracle (no tokenizer, no files)."""

from __future__ import annotations

import torch


class RandomTokenPromptDataset:
    """``num_prompts`` prompts of uniform-random token ids with lengths uniform in [min_len, max_len].

    Deterministic in ``seed``; token ids avoid ``reserved_ids`` (e.g. pad / eos) so that stop conditions stay under the
    caller's control."""

    def __init__(self, num_prompts: int, min_len: int, max_len: int, vocab_size: int, seed: int = 0,
                 task_name: str = "synthetic", reserved_ids: tuple[int, ...] = ()):
        g = torch.Generator().manual_seed(seed)
        self.items = []
        for i in range(num_prompts):
            L = int(torch.randint(min_len, max_len + 1, (1,), generator=g))
            ids = torch.randint(0, vocab_size, (L,), generator=g)
            for r in reserved_ids:
                ids[ids == r] = (r + 1) % vocab_size
            self.items.append({
                "message_log": [{"role": "user", "content": "", "token_ids": ids}],
                "length": L, "extra_env_info": {"idx": i}, "loss_multiplier": 1.0, "idx": i, "task_name": task_name,
            })

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        it = self.items[i]
        return {**it, "message_log": [dict(m) for m in it["message_log"]]}
