"""Synthetic supervised / preference datasets (token-level, tokenizer-free) for tests and smoke runs, plus JSONL
loaders for chat-format SFT and preference data."""

from __future__ import annotations

import json
from typing import Optional

import torch


def _chain(first, n, vocab_size):
    out, cur = [], int(first)
    for _ in range(n):
        cur = (cur * 7 + 3) % vocab_size
        out.append(cur)
    return torch.tensor(out, dtype=torch.long)


def _msg(role, ids):
    return {"role": role, "content": "", "token_ids": ids}


class RandomSFTDataset:
    """Prompt + response token sequences; every response token is a fixed function of the token before it (a bigram
    rule), so a small model learns the task in a few dozen steps."""

    def __init__(self, n: int, vocab_size: int, prompt_len: int = 8, response_len: int = 8, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.items = []
        for i in range(n):
            p = torch.randint(2, vocab_size, (prompt_len,), generator=g)
            r = _chain(p[-1], response_len, vocab_size)
            self.items.append({"message_log": [_msg("user", p), _msg("assistant", r)], "length": prompt_len + response_len,
                               "loss_multiplier": 1.0, "idx": i, "task_name": "sft"})

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        it = self.items[i]
        return {**it, "message_log": [dict(m) for m in it["message_log"]]}


class RandomPreferenceDataset:
    """Pairs (chosen, rejected): the chosen response follows the rule of ``RandomSFTDataset``, the rejected is noise."""

    def __init__(self, n: int, vocab_size: int, prompt_len: int = 8, response_len: int = 8, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.items = []
        for i in range(n):
            p = torch.randint(2, vocab_size, (prompt_len,), generator=g)
            good = _chain(p[-1], response_len, vocab_size)
            bad = torch.randint(2, vocab_size, (response_len,), generator=g)
            self.items.append({"message_log_chosen": [_msg("user", p), _msg("assistant", good)],
                               "message_log_rejected": [_msg("user", p.clone()), _msg("assistant", bad)],
                               "length_chosen": prompt_len + response_len, "length_rejected": prompt_len + response_len,
                               "loss_multiplier": 1.0, "idx": i, "task_name": "preference"})

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        it = self.items[i]
        return {**it, "message_log_chosen": [dict(m) for m in it["message_log_chosen"]],
                "message_log_rejected": [dict(m) for m in it["message_log_rejected"]]}


class JsonlChatDataset:
    """One JSON object per line with a ``messages`` list ([{role, content}, ...]); tokenised with the chat template."""

    def __init__(self, path: str, tokenizer, max_seq_length: Optional[int] = None, messages_key: str = "messages"):
        from rl_b200.data.llm_message_utils import get_formatted_message_log

        self.items = []
        with open(path) as f:
            for i, line in enumerate(f):
                if not line.strip():
                    continue
                rec = json.loads(line)
                log = get_formatted_message_log(rec[messages_key], tokenizer)
                length = sum(int(m["token_ids"].numel()) for m in log)
                mult = 1.0
                if max_seq_length is not None and length > max_seq_length:
                    for m in log:  # keep a stub so that batch shapes stay bounded; the sample is masked out
                        m["token_ids"] = m["token_ids"][: max(1, max_seq_length // len(log))]
                    length = sum(int(m["token_ids"].numel()) for m in log)
                    mult = 0.0
                self.items.append({"message_log": log, "length": length, "loss_multiplier": mult, "idx": i, "task_name": "sft"})

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]


class JsonlPreferenceDataset:
    """Lines of {prompt | context, chosen, rejected} (strings or message lists)."""

    def __init__(self, path: str, tokenizer, max_seq_length: Optional[int] = None):
        from rl_b200.data.llm_message_utils import get_formatted_message_log

        def as_msgs(x, role):
            return x if isinstance(x, list) else [{"role": role, "content": x}]

        self.items = []
        with open(path) as f:
            for i, line in enumerate(f):
                if not line.strip():
                    continue
                rec = json.loads(line)
                ctx = as_msgs(rec.get("prompt", rec.get("context", "")), "user")
                ch = get_formatted_message_log(ctx + as_msgs(rec["chosen"], "assistant"), tokenizer)
                rj = get_formatted_message_log(ctx + as_msgs(rec["rejected"], "assistant"), tokenizer)
                lc = sum(int(m["token_ids"].numel()) for m in ch)
                lr = sum(int(m["token_ids"].numel()) for m in rj)
                mult = 0.0 if (max_seq_length is not None and max(lc, lr) > max_seq_length) else 1.0
                self.items.append({"message_log_chosen": ch, "message_log_rejected": rj, "length_chosen": lc, "length_rejected": lr,
                                   "loss_multiplier": mult, "idx": i, "task_name": "preference"})

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]
