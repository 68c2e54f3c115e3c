"""Cross-tokenizer distillation loss and the batch preparation that feeds it.

Two terms, both defined on the chunks of :mod:`token_aligner`:

* next-token term — at the first token of every chunk teacher and student see the same text prefix; the teacher's top-k
  next-token distribution is projected to the student's vocabulary (tokens with identical strings) and compared with
  the student's distribution on that shared support (forward KL, both renormalised over it);
* chunk term — the log-probability of the chunk's text, i.e. the sum of the token log-probabilities inside it, should
  agree between student and teacher whatever the number of tokens on either side (squared difference).

Role of ``CrossTokenizerDistillationLossFn`` (nemo_rl/algorithms/loss/loss_functions.py:1463-2667) and
x_token/loss_utils.py:69,228 in the reference.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from rl_b200.algorithms.loss.interfaces import LossInputType, LossType
from rl_b200.distributed.batched_data_dict import BatchedDataDict

from .token_aligner import TokenAligner


class CrossTokenizerDistillationLossFn:
    loss_type = LossType.TOKEN_LEVEL
    input_type = LossInputType.LOGIT

    def __init__(self, cfg: Optional[dict] = None):
        c = dict(next_token_weight=1.0, chunk_weight=0.1, chunk_loss="squared")
        c.update(cfg or {})
        assert c["chunk_loss"] in ("squared", "abs")
        self.cfg = c

    def __call__(self, logits, data, global_valid_seqs, global_valid_toks):
        c = self.cfg
        logp = torch.log_softmax(logits[:, :-1].float(), dim=-1)                 # row r predicts token r + 1
        B, R, _ = logp.shape
        sm = data["sample_mask"].to(logp.dtype)
        norm = global_valid_toks + 1e-8
        # ---- next-token term on the aligned positions
        pos = data["xt_student_pos"].long().clamp(max=R - 1)                      # [B, A]
        amask = data["xt_align_mask"].to(logp.dtype) * sm[:, None]               # [B, A]
        sid = data["xt_student_ids"].long()                                      # [B, A, k] (0 where invalid)
        valid = data["xt_valid"].bool()                                          # [B, A, k]
        rows = logp.gather(1, pos[:, :, None].expand(-1, -1, logp.shape[-1]))    # [B, A, V]
        s = rows.gather(-1, sid).masked_fill(~valid, float("-inf"))
        t = data["xt_teacher_topk_logits"].float().masked_fill(~valid, float("-inf"))
        has = valid.any(-1)
        s = torch.where(has[..., None], s, torch.zeros_like(s))                  # rows without support contribute 0
        t = torch.where(has[..., None], t, torch.zeros_like(t))
        s = s - torch.logsumexp(s, -1, keepdim=True)
        t = t - torch.logsumexp(t, -1, keepdim=True)
        kl = torch.where(valid & has[..., None], t.exp() * (t - s), torch.zeros_like(s)).sum(-1)
        nt_loss = (kl * amask * has).sum() / norm
        # ---- chunk term
        tok_lp = logp.gather(-1, data["xt_next_ids"].long()[:, :R, None])[..., 0]    # [B, R] log p(token r+1)
        cid = data["xt_chunk_id"].long()[:, :R]                                   # [B, R], -1 outside chunks
        C = data["xt_teacher_chunk_lp"].shape[1]
        inside = (cid >= 0).to(logp.dtype)
        s_chunk = torch.zeros(B, C, dtype=logp.dtype, device=logp.device).scatter_add_(1, cid.clamp(min=0), tok_lp * inside)
        cmask = data["xt_chunk_mask"].to(logp.dtype) * sm[:, None]
        diff = s_chunk - data["xt_teacher_chunk_lp"].to(logp.dtype)
        per = diff * diff if c["chunk_loss"] == "squared" else diff.abs()
        ch_loss = (per * cmask).sum() / norm
        loss = c["next_token_weight"] * nt_loss + c["chunk_weight"] * ch_loss
        return loss, {"loss": loss.item(), "next_token_kl": nt_loss.item(), "chunk_loss": ch_loss.item(),
                      "num_valid_samples": sm.sum().item(), "aligned_positions": (amask * has).sum().item()}


def prepare_xtoken_batch(texts: Sequence[str], aligner: TokenAligner, proj: torch.Tensor, teacher, k: int, max_len: int,
                         logprob_batch_size: Optional[int] = None) -> BatchedDataDict:
    """Tokenises ``texts`` for both models, runs the teacher (top-k next-token logits and token log-probabilities) and
    lays out what the loss needs, padded per batch. ``teacher``: a policy worker built on the teacher's tokenizer."""
    if isinstance(proj, dict):      # a sparse map from rl_b200/tools/x_token_projection.py: every teacher token's heaviest student target
        from rl_b200.tools.x_token_projection import as_one_to_one

        proj = as_one_to_one(proj)
    s_tok, t_tok = aligner.s_tok, aligner.t_tok
    n = len(texts)
    S_ids, T_ids, CH = [], [], []
    for text in texts:
        s_ids, t_ids, chunks = aligner.align(text)
        s_ids, t_ids = [s_tok.bos_token_id] + s_ids, [t_tok.bos_token_id] + t_ids       # shared first context
        chunks = [ch for ch in chunks if ch.s_hi + 1 <= max_len and ch.t_hi + 1 <= max_len]
        s_end = (chunks[-1].s_hi + 1) if chunks else 1
        t_end = (chunks[-1].t_hi + 1) if chunks else 1
        S_ids.append(s_ids[:s_end])
        T_ids.append(t_ids[:t_end])
        CH.append(chunks)
    Ls, Lt = max(len(x) for x in S_ids), max(len(x) for x in T_ids)
    Ls, Lt = max(Ls, 2), max(Lt, 2)
    A = max(1, max(len(c) for c in CH))
    spad = s_tok.pad_token_id if s_tok.pad_token_id is not None else 0
    tpad = t_tok.pad_token_id if t_tok.pad_token_id is not None else 0
    t_data = BatchedDataDict(input_ids=torch.full((n, Lt), tpad, dtype=torch.long), input_lengths=torch.tensor([len(x) for x in T_ids]))
    for i, x in enumerate(T_ids):
        t_data["input_ids"][i, : len(x)] = torch.tensor(x)
    topk = teacher.get_topk_logits(t_data, k, logprob_batch_size)
    t_lp = teacher.get_logprobs(t_data, logprob_batch_size)["logprobs"]                  # [n, Lt], entry j = log p(t_j | t_<j)
    out = BatchedDataDict(
        input_ids=torch.full((n, Ls), spad, dtype=torch.long), input_lengths=torch.tensor([len(x) for x in S_ids]),
        token_mask=torch.zeros(n, Ls), sample_mask=torch.ones(n),
        xt_student_pos=torch.zeros(n, A, dtype=torch.long), xt_align_mask=torch.zeros(n, A),
        xt_student_ids=torch.zeros(n, A, k, dtype=torch.long), xt_valid=torch.zeros(n, A, k, dtype=torch.bool),
        xt_teacher_topk_logits=torch.zeros(n, A, k), xt_next_ids=torch.zeros(n, Ls, dtype=torch.long),
        xt_chunk_id=torch.full((n, Ls), -1, dtype=torch.long), xt_teacher_chunk_lp=torch.zeros(n, A), xt_chunk_mask=torch.zeros(n, A))
    for i in range(n):
        s = torch.tensor(S_ids[i])
        out["input_ids"][i, : len(s)] = s
        out["xt_next_ids"][i, : len(s) - 1] = s[1:]
        if not CH[i]:
            out["sample_mask"][i] = 0.0
        for c, ch in enumerate(CH[i]):
            s_lo, s_hi, t_lo, t_hi = ch.s_lo + 1, ch.s_hi + 1, ch.t_lo + 1, ch.t_hi + 1   # shifted by the leading bos
            out["token_mask"][i, s_lo:s_hi] = 1.0
            out["xt_chunk_id"][i, s_lo - 1 : s_hi - 1] = c
            out["xt_teacher_chunk_lp"][i, c] = t_lp[i, t_lo:t_hi].sum()
            out["xt_chunk_mask"][i, c] = 1.0
            out["xt_student_pos"][i, c] = s_lo - 1
            tid = topk["topk_indices"][i, t_lo - 1]
            sid = proj[tid]
            out["xt_valid"][i, c] = sid >= 0
            out["xt_student_ids"][i, c] = sid.clamp(min=0)
            out["xt_teacher_topk_logits"][i, c] = topk["topk_logits"][i, t_lo - 1]
            out["xt_align_mask"][i, c] = 1.0
    return out
