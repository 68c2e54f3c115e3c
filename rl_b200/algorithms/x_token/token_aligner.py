"""Alignment of two tokenisations of one text, and the vocabulary projection between their tokenizers.

Teacher and student may cut the same string differently. Both token sequences are mapped to character spans; walking
the two span lists in step gives *chunks*: minimal groups of consecutive student tokens and teacher tokens that cover
the same characters. At every chunk start both models are conditioned on exactly the same text, so their next-token
distributions are comparable wherever the vocabularies share a token string (``build_vocab_projection``); over a whole
chunk the product of token probabilities is the probability of the same piece of text under either model. This is the
method of nemo_rl/algorithms/x_token/token_aligner.py:242 in a span-based form.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch


@dataclass
class Chunk:
    s_lo: int   # student tokens [s_lo, s_hi)
    s_hi: int
    t_lo: int   # teacher tokens [t_lo, t_hi)
    t_hi: int
    c_lo: int   # characters [c_lo, c_hi)
    c_hi: int

    @property
    def one_to_one(self) -> bool:
        return self.s_hi - self.s_lo == 1 and self.t_hi - self.t_lo == 1


def token_spans(tokenizer, ids: Sequence[int], text: Optional[str] = None) -> list[tuple[int, int]]:
    """Character span of every token. Uses the tokenizer's offset mapping when it has one; otherwise decodes growing
    prefixes (exact for byte-level vocabularies, where a token may end inside a multi-byte character: such a token gets
    an empty span and the character is attributed to the token that completes it)."""
    if text is not None and getattr(tokenizer, "is_fast", False):
        enc = tokenizer(text, add_special_tokens=False, return_offsets_mapping=True)
        if list(enc["input_ids"]) == list(ids):
            return [tuple(o) for o in enc["offset_mapping"]]
    spans, prev = [], 0
    ids = list(ids)
    for i in range(len(ids)):
        s = tokenizer.decode(ids[: i + 1])
        n = len(s) - (1 if s.endswith("�") else 0)   # an incomplete UTF-8 tail decodes to U+FFFD
        n = max(n, prev)
        spans.append((prev, n))
        prev = n
    return spans


class TokenAligner:
    def __init__(self, student_tokenizer, teacher_tokenizer):
        self.s_tok, self.t_tok = student_tokenizer, teacher_tokenizer

    def align_spans(self, s_spans: Sequence[tuple[int, int]], t_spans: Sequence[tuple[int, int]]) -> list[Chunk]:
        chunks: list[Chunk] = []
        i = j = 0
        ns, nt = len(s_spans), len(t_spans)
        while i < ns and j < nt:
            i0, j0 = i, j
            c0 = min(s_spans[i][0], t_spans[j][0])
            se, te = s_spans[i][1], t_spans[j][1]
            i += 1
            j += 1
            # extend the side that ends first until both end on the same character; a chunk never closes on a token
            # that ends inside a multi-byte character (zero width so far), the completing token belongs to it as well
            ok = True
            while se != te or se == c0:
                if se < te or (se == te and i < ns and (j >= nt or s_spans[i][1] <= t_spans[j][1])):
                    if i >= ns:
                        ok = False
                        break
                    se = s_spans[i][1]
                    i += 1
                else:
                    if j >= nt:
                        ok = False
                        break
                    te = t_spans[j][1]
                    j += 1
            if not ok:
                break   # the texts differ from here on (one side was truncated): nothing more can be aligned
            chunks.append(Chunk(i0, i, j0, j, c0, se))
        return chunks

    def align(self, text: str, s_ids: Optional[Sequence[int]] = None, t_ids: Optional[Sequence[int]] = None):
        """Returns (student ids, teacher ids, chunks) for ``text``."""
        s_ids = list(s_ids) if s_ids is not None else list(self.s_tok.encode(text))
        t_ids = list(t_ids) if t_ids is not None else list(self.t_tok.encode(text))
        return s_ids, t_ids, self.align_spans(token_spans(self.s_tok, s_ids, text), token_spans(self.t_tok, t_ids, text))


def build_vocab_projection(student_tokenizer, teacher_tokenizer, student_vocab: Optional[int] = None,
                           teacher_vocab: Optional[int] = None) -> torch.Tensor:
    """``proj[t]`` = id of the student token with the same string as teacher token ``t``, or -1. A sparse one-to-one
    map: probability mass of teacher tokens without a twin is left out of the comparison."""
    sv = student_vocab or len(student_tokenizer)
    tv = teacher_vocab or len(teacher_tokenizer)
    by_text: dict[str, int] = {}
    for i in range(sv):
        s = student_tokenizer.decode([i])
        if s and "�" not in s and s not in by_text:
            by_text[s] = i
    proj = torch.full((tv,), -1, dtype=torch.long)
    for t in range(tv):
        s = teacher_tokenizer.decode([t])
        if s and "�" not in s:
            proj[t] = by_text.get(s, -1)
    return proj
