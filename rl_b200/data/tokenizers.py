"""Offline tokenizers. ``ByteTokenizer`` is a self-contained byte-level tokenizer with a minimal chat template, used
when no tokenizer files are available (air-gapped runs, tests, benchmarks); it implements the subset of the
HuggingFace tokenizer API the framework touches (``__call__``, ``encode``, ``decode``, ``batch_decode``,
``apply_chat_template``, ``pad_token_id`` / ``eos_token_id`` / ``bos_token_id``)."""

from __future__ import annotations

from typing import Sequence

import torch


class ByteTokenizer:
    """ids 0..255 are bytes; 256 = <bos>, 257 = <eos>, 258 = <pad>, 259.. = role markers."""

    SPECIALS = ["<bos>", "<eos>", "<pad>", "<|system|>", "<|user|>", "<|assistant|>", "<|environment|>", "<|end|>"]

    def __init__(self, vocab_size: int = 512):
        assert vocab_size >= 256 + len(self.SPECIALS)
        self.vocab_size = vocab_size
        self._sp = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self._inv = {v: k for k, v in self._sp.items()}
        self.bos_token, self.eos_token, self.pad_token = "<bos>", "<eos>", "<pad>"
        self.bos_token_id, self.eos_token_id, self.pad_token_id = 256, 257, 258
        self.chat_template = "byte"
        self.name_or_path = "byte"

    def __len__(self):
        return self.vocab_size

    # ------------------------------------------------------------------ encode / decode
    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids: list[int] = [self.bos_token_id] if add_special_tokens else []
        i = 0
        while i < len(text):
            if text[i] == "<":
                hit = next((s for s in self.SPECIALS if text.startswith(s, i)), None)
                if hit is not None:
                    ids.append(self._sp[hit])
                    i += len(hit)
                    continue
            ids.extend(text[i].encode("utf-8"))
            i += 1
        return ids

    def __call__(self, text, add_special_tokens: bool = False, return_tensors=None, **_):
        batch = [text] if isinstance(text, str) else list(text)
        enc = [self.encode(t, add_special_tokens) for t in batch]
        if return_tensors == "pt":
            L = max((len(e) for e in enc), default=0)
            out = torch.full((len(enc), L), self.pad_token_id, dtype=torch.long)
            for i, e in enumerate(enc):
                out[i, : len(e)] = torch.tensor(e, dtype=torch.long)
            return {"input_ids": out}
        return {"input_ids": enc[0] if isinstance(text, str) else enc}

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        if isinstance(ids, torch.Tensor):
            ids = ids.tolist()
        out, buf = [], bytearray()
        for t in ids:
            if 0 <= t < 256:
                buf.append(t)
                continue
            if buf:
                out.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
            if not skip_special_tokens and t in self._inv:
                out.append(self._inv[t])
        if buf:
            out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    def batch_decode(self, seqs: Sequence, skip_special_tokens: bool = False) -> list[str]:
        return [self.decode(s, skip_special_tokens) for s in seqs]

    # ------------------------------------------------------------------ chat
    def apply_chat_template(self, messages, tokenize: bool = False, add_generation_prompt: bool = False, **_):
        parts = ["<bos>"]
        for m in messages:
            role = m["role"] if f"<|{m['role']}|>" in self._sp else "user"
            parts.append(f"<|{role}|>{m['content']}<|end|>")
        if add_generation_prompt:
            parts.append("<|assistant|>")
        text = "".join(parts)
        return self.encode(text) if tokenize else text


class PairTokenizer(ByteTokenizer):
    """Byte tokenizer with one merge rule: two adjacent lowercase ASCII letters form one token (ids from ``pair_base``
    on, 26 x 26 of them). A second offline tokenisation of the same text with different boundaries, which is what
    cross-tokenizer distillation needs to be exercised without tokenizer files."""

    def __init__(self, vocab_size: int = 1024):
        super().__init__(vocab_size)
        self.pair_base = 256 + len(self.SPECIALS)
        assert vocab_size >= self.pair_base + 26 * 26
        self.name_or_path = "pair"

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids: list[int] = [self.bos_token_id] if add_special_tokens else []
        i = 0
        while i < len(text):
            if text[i] == "<":
                hit = next((s for s in self.SPECIALS if text.startswith(s, i)), None)
                if hit is not None:
                    ids.append(self._sp[hit])
                    i += len(hit)
                    continue
            a = text[i]
            b = text[i + 1] if i + 1 < len(text) else ""
            if "a" <= a <= "z" and b and "a" <= b <= "z":
                ids.append(self.pair_base + (ord(a) - 97) * 26 + (ord(b) - 97))
                i += 2
                continue
            ids.extend(a.encode("utf-8"))
            i += 1
        return ids

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        if isinstance(ids, torch.Tensor):
            ids = ids.tolist()
        flat: list[int] = []
        for t in ids:
            if self.pair_base <= t < self.pair_base + 676:
                p = t - self.pair_base
                flat += [97 + p // 26, 97 + p % 26]
            else:
                flat.append(t)
        return super().decode(flat, skip_special_tokens)
