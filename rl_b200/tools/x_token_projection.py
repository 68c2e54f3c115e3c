"""Sparse projection maps between two tokenizers' vocabularies for cross-tokenizer distillation: which student tokens stand for
a teacher token, with what weight (role of tools/x_token/minimal_projection_generator.py, sort_and_cut_projection_matrix.py,
reapply_exact_map.py and utils.py: ``project_token_likelihoods``, ``sinkhorn_one_dim``).

    python -m rl_b200.tools.x_token_projection --student byte --teacher pair --top-k 4 --out proj.pt

A map is ``{"indices": [Vt, k] student ids (-1 unused), "values": [Vt, k] weights (rows sum to 1 or 0), "student_vocab": Vs}``.
A teacher token whose text is also a student token maps to it alone (weight 1). Any other teacher token is spelled by the
student tokenizer as a short sequence; the FIRST student token of that spelling is what the student must emit at the position
where the teacher emits its token, so it gets the largest weight, later pieces geometrically less (``decay``), at most ``top_k``
of them. Teacher tokens that cannot be spelled (specials, broken bytes) map to nothing.
"""

from __future__ import annotations

import argparse
import json
from typing import Optional

import torch


def _text_of(tok, i: int) -> str:
    try:
        s = tok.decode([i])
    except Exception:
        return ""
    return "" if ("�" in s) else s


def build_sparse_projection(student_tok, teacher_tok, student_vocab: Optional[int] = None, teacher_vocab: Optional[int] = None, top_k: int = 4,
                            exact_only: bool = False, decay: float = 0.5) -> dict:
    sv, tv = student_vocab or len(student_tok), teacher_vocab or len(teacher_tok)
    by_text: dict[str, int] = {}
    for i in range(sv):
        s = _text_of(student_tok, i)
        if s and s not in by_text:
            by_text[s] = i
    idx = torch.full((tv, top_k), -1, dtype=torch.long)
    val = torch.zeros((tv, top_k), dtype=torch.float32)
    exact = torch.zeros(tv, dtype=torch.bool)
    for t in range(tv):
        s = _text_of(teacher_tok, t)
        if not s:
            continue
        if s in by_text:
            idx[t, 0], val[t, 0], exact[t] = by_text[s], 1.0, True
            continue
        if exact_only:
            continue
        pieces = [int(p) for p in student_tok.encode(s) if 0 <= int(p) < sv]
        if not pieces or student_tok.decode(pieces) != s:
            continue       # the student cannot spell this text exactly
        seen: dict[int, float] = {}
        for j, p in enumerate(pieces[:top_k]):
            seen[p] = seen.get(p, 0.0) + decay ** j
        for j, (p, w) in enumerate(sorted(seen.items(), key=lambda kv: -kv[1])[:top_k]):
            idx[t, j], val[t, j] = p, w
    proj = {"indices": idx, "values": val, "student_vocab": sv, "exact": exact}
    return sinkhorn_one_dim(proj)


def sinkhorn_one_dim(proj: dict, iters: int = 1) -> dict:
    """Normalises every non-empty row to sum 1 (the one-sided Sinkhorn step: teacher probability mass is conserved)."""
    v = proj["values"].clone()
    for _ in range(max(1, iters)):
        s = v.sum(-1, keepdim=True)
        v = torch.where(s > 0, v / s.clamp(min=1e-30), v)
    return dict(proj, values=v)


def sort_and_cut(proj: dict, k: int) -> dict:
    """Keeps the ``k`` heaviest targets of every row (sorted by weight) and renormalises."""
    v, order = proj["values"].sort(-1, descending=True)
    i = proj["indices"].gather(-1, order)
    v, i = v[:, :k].clone(), i[:, :k].clone()
    i[v <= 0] = -1
    return sinkhorn_one_dim(dict(proj, indices=i, values=v))


def reapply_exact_map(proj: dict) -> dict:
    """After a map was edited or learned: teacher tokens that have an identical student token go back to that token alone."""
    base_i, base_v = proj["indices"].clone(), proj["values"].clone()
    ex = proj.get("exact")
    if ex is None:
        return proj
    first = base_i[:, 0]
    base_i[ex, 1:], base_v[ex, 1:] = -1, 0.0
    base_i[ex, 0], base_v[ex, 0] = first[ex], 1.0
    return dict(proj, indices=base_i, values=base_v)


def project_token_likelihoods(teacher_probs: torch.Tensor, proj: dict) -> torch.Tensor:
    """[..., Vt] teacher probabilities -> [..., Vs] on the student's vocabulary (mass of unmapped teacher tokens is dropped)."""
    i, v = proj["indices"].to(teacher_probs.device), proj["values"].to(teacher_probs.device, teacher_probs.dtype)
    out = teacher_probs.new_zeros(teacher_probs.shape[:-1] + (int(proj["student_vocab"]),))
    flat = teacher_probs.reshape(-1, teacher_probs.shape[-1])
    o = out.reshape(-1, out.shape[-1])
    for j in range(i.shape[1]):
        ok = i[:, j] >= 0
        o.index_add_(1, i[ok, j], flat[:, ok] * v[ok, j])
    return out


def as_one_to_one(proj: dict) -> torch.Tensor:
    """[Vt] the heaviest student target of every teacher token (-1: none): the form the distillation batch preparation takes."""
    v, j = proj["values"].max(-1)
    first = proj["indices"].gather(-1, j[:, None])[:, 0]
    return torch.where(v > 0, first, torch.full_like(first, -1))


def coverage(proj: dict) -> dict:
    mapped = (proj["values"].sum(-1) > 0)
    ex = proj.get("exact", torch.zeros_like(mapped))
    return dict(teacher_vocab=int(mapped.numel()), mapped=int(mapped.sum()), exact=int(ex.sum()), spelled=int((mapped & ~ex).sum()),
                unmapped=int((~mapped).sum()), mean_targets=float((proj["indices"] >= 0).sum(-1)[mapped].float().mean()) if mapped.any() else 0.0)


def main(argv=None) -> int:
    from rl_b200.algorithms.utils import get_tokenizer

    ap = argparse.ArgumentParser()
    ap.add_argument("--student", required=True)
    ap.add_argument("--teacher", required=True)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--exact-only", action="store_true")
    ap.add_argument("--decay", type=float, default=0.5)
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    proj = build_sparse_projection(get_tokenizer({"name": a.student}), get_tokenizer({"name": a.teacher}), top_k=a.top_k, exact_only=a.exact_only,
                                   decay=a.decay)
    torch.save(proj, a.out)
    print(json.dumps(coverage(proj)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
