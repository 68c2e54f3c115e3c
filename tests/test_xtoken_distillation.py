"""Cross-tokenizer distillation: token alignment, vocabulary projection, loss against a hand computation, training loop."""

import random

import pytest
import torch

from rl_b200.algorithms import xtoken_off_policy_distillation as xt
from rl_b200.algorithms.x_token import CrossTokenizerDistillationLossFn, TokenAligner, build_vocab_projection
from rl_b200.data.tokenizers import ByteTokenizer, PairTokenizer
from rl_b200.models.config import ModelConfig


def test_alignment_covers_text_with_equal_strings_per_chunk():
    s, t = ByteTokenizer(512), PairTokenizer(1024)
    al = TokenAligner(s, t)
    rng = random.Random(0)
    alphabet = "abcdefgh XYZ01 é日<|end|>"
    for _ in range(20):
        text = "".join(rng.choice(["ab", "c", " ", "Q", "é", "日", "<|end|>", "xyz", "7"]) for _ in range(rng.randint(1, 30)))
        si, ti, chunks = al.align(text)
        assert chunks[0].s_lo == 0 and chunks[0].t_lo == 0 and chunks[-1].s_hi == len(si) and chunks[-1].t_hi == len(ti)
        for a, b in zip(chunks, chunks[1:]):
            assert a.s_hi == b.s_lo and a.t_hi == b.t_lo and a.c_hi == b.c_lo
        for c in chunks:
            assert s.decode(si[c.s_lo : c.s_hi]) == t.decode(ti[c.t_lo : c.t_hi]) == text[c.c_lo : c.c_hi] != ""
    assert alphabet  # silence linters
    # a truncated side ends the alignment instead of mis-aligning
    si, ti, chunks = al.align("hello world", t_ids=t.encode("hello world")[:3])
    assert chunks and chunks[-1].t_hi <= 3


def test_vocab_projection_maps_equal_strings_only():
    s, t = ByteTokenizer(512), PairTokenizer(1024)
    proj = build_vocab_projection(s, t)
    assert proj[ord("a")] == ord("a") and proj[t.eos_token_id] == s.eos_token_id
    assert (proj[t.pair_base : t.pair_base + 676] == -1).all()        # merged pairs have no single student token
    back = build_vocab_projection(t, s)
    assert back[ord("z")] == ord("z") and (back[:128] >= 0).sum() >= 95


def test_loss_matches_hand_computation_and_vanishes_for_equal_models():
    torch.manual_seed(0)
    B, S, V, A, k = 2, 6, 11, 3, 4
    logits = torch.randn(B, S, V, dtype=torch.float64, requires_grad=True)
    logp = torch.log_softmax(logits[:, :-1], -1)
    data = dict(sample_mask=torch.ones(B), xt_student_pos=torch.tensor([[0, 2, 4], [1, 3, 0]]), xt_align_mask=torch.tensor([[1., 1, 1], [1, 1, 0]]),
                xt_student_ids=torch.randint(0, V, (B, A, k)), xt_valid=torch.rand(B, A, k) > 0.3,
                xt_teacher_topk_logits=torch.randn(B, A, k), xt_next_ids=torch.randint(0, V, (B, S)),
                xt_chunk_id=torch.tensor([[0, 0, 1, 1, 2, -1], [-1, 0, 0, 1, -1, -1]]),
                xt_teacher_chunk_lp=torch.randn(B, A), xt_chunk_mask=torch.tensor([[1., 1, 1], [1, 1, 0]]))
    data["xt_valid"][0, 1] = False                                   # a position without shared support contributes nothing
    fn = CrossTokenizerDistillationLossFn(dict(next_token_weight=1.0, chunk_weight=0.5))
    ntok = torch.tensor(9.0)
    loss, m = fn(logits, data, torch.tensor(2.0), ntok)
    want_kl = 0.0
    for b in range(B):
        for a in range(A):
            v = data["xt_valid"][b, a]
            if data["xt_align_mask"][b, a] == 0 or not v.any():
                continue
            sl = logp[b, data["xt_student_pos"][b, a], data["xt_student_ids"][b, a][v]]
            tl = data["xt_teacher_topk_logits"][b, a][v].double()
            sl, tl = sl - torch.logsumexp(sl, 0), tl - torch.logsumexp(tl, 0)
            want_kl = want_kl + (tl.exp() * (tl - sl)).sum()
    want_ch = 0.0
    for b in range(B):
        for c in range(A):
            if data["xt_chunk_mask"][b, c] == 0:
                continue
            rows = (data["xt_chunk_id"][b, : S - 1] == c).nonzero()[:, 0]
            slp = sum(logp[b, r, data["xt_next_ids"][b, r]] for r in rows)
            want_ch = want_ch + (slp - data["xt_teacher_chunk_lp"][b, c].double()) ** 2
    want = (want_kl + 0.5 * want_ch) / ntok
    assert loss.item() == pytest.approx(float(want.detach()), rel=1e-6)
    loss.backward()
    assert torch.isfinite(logits.grad).all() and logits.grad.abs().sum() > 0
    assert m["aligned_positions"] == 4


def _mc(vocab):
    return ModelConfig(vocab_size=vocab, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=8, torch_dtype="float32")


def test_training_loop_pulls_student_towards_teacher(tmp_path):
    s_tok, t_tok = ByteTokenizer(512), PairTokenizer(1024)
    rng = random.Random(1)
    words = ["alpha", "beta", "gamma", "delta", "x1", "y22", "Zed"]
    ds = [{"text": " ".join(rng.choice(words) for _ in range(rng.randint(2, 5)))} for _ in range(64)]
    cfg = {"distillation": dict(max_num_steps=10, max_num_epochs=3, topk_logits_k=8, seed=0), "loss_fn": dict(next_token_weight=1.0, chunk_weight=0.05),
           "policy": dict(precision="float32", train_global_batch_size=16, train_micro_batch_size=8, logprob_batch_size=16, max_total_sequence_length=48,
                          max_grad_norm=1.0, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-2, weight_decay=0.0))),
           "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False), "data": dict(shuffle=False)}
    student, teacher, loader, aligner, proj, loss_fn, logger, ck, ss, cfg = xt.setup(cfg, s_tok, t_tok, ds, student_cfg=_mc(512), teacher_cfg=_mc(1024))
    hist = []
    xt.xtoken_distillation_train(student, teacher, loader, aligner, proj, loss_fn, logger, ck, ss, cfg,
                                 step_callback=lambda s, m: hist.append(m["train"]))
    assert len(hist) == 10
    assert hist[-1]["loss"] < 0.5 * hist[0]["loss"] and hist[-1]["chunk_loss"] < hist[0]["chunk_loss"]
    assert all(h["aligned_positions"] > 0 and h["next_token_kl"] >= 0 for h in hist)


def test_sparse_vocabulary_projection_between_tokenizers(tmp_path):
    """Student = byte tokenizer, teacher = byte pairs: a teacher pair token has no twin in the student's vocabulary and is spelled
    by two byte tokens (first one heavier); single bytes map one to one; specials map to nothing."""
    from rl_b200.data.tokenizers import ByteTokenizer, PairTokenizer
    from rl_b200.tools import x_token_projection as X

    s_tok, t_tok = ByteTokenizer(vocab_size=512), PairTokenizer(vocab_size=1024)
    proj = X.build_sparse_projection(s_tok, t_tok, top_k=3)
    assert proj["indices"].shape == (1024, 3) and proj["student_vocab"] == 512
    a = t_tok.encode("a")[0]
    assert proj["indices"][a].tolist() == [s_tok.encode("a")[0], -1, -1] and proj["values"][a, 0] == 1.0 and bool(proj["exact"][a])
    th = t_tok.encode("th")
    assert len(th) == 1
    row_i, row_v = proj["indices"][th[0]], proj["values"][th[0]]
    assert row_i[:2].tolist() == [s_tok.encode("t")[0], s_tok.encode("h")[0]] and row_v[:2].tolist() == pytest.approx([2 / 3, 1 / 3])
    assert not bool(proj["exact"][th[0]])
    aa = t_tok.encode("aa")[0]                                  # the same student token twice: one target, all the weight
    assert proj["indices"][aa].tolist() == [s_tok.encode("a")[0], -1, -1] and float(proj["values"][aa, 0]) == pytest.approx(1.0)
    cov = X.coverage(proj)
    assert cov["exact"] >= 128 and cov["spelled"] == 676 and cov["mapped"] + cov["unmapped"] == 1024
    # teacher probabilities land on the student's vocabulary with their mass conserved on mapped tokens
    p = torch.zeros(2, 1024)
    p[0, th[0]], p[0, a], p[1, aa] = 0.6, 0.4, 1.0
    q = X.project_token_likelihoods(p, proj)
    assert q.shape == (2, 512) and q.sum(-1).tolist() == pytest.approx([1.0, 1.0])
    assert float(q[0, s_tok.encode("t")[0]]) == pytest.approx(0.4) and float(q[0, s_tok.encode("a")[0]]) == pytest.approx(0.4)
    # cut to the single heaviest target, the form the distillation batch takes
    one = X.as_one_to_one(X.sort_and_cut(proj, 1))
    assert int(one[th[0]]) == s_tok.encode("t")[0] and int(one[a]) == s_tok.encode("a")[0]
    # an edited map gets its exact rows back
    bent = dict(proj, values=proj["values"].clone(), indices=proj["indices"].clone())
    bent["indices"][a, 1], bent["values"][a] = 5, torch.tensor([0.5, 0.5, 0.0])
    fixed = X.reapply_exact_map(bent)
    assert fixed["indices"][a].tolist() == proj["indices"][a].tolist() and fixed["values"][a].tolist() == [1.0, 0.0, 0.0]
    exact_only = X.build_sparse_projection(s_tok, t_tok, top_k=2, exact_only=True)
    assert float(exact_only["values"][th[0]].sum()) == 0.0
    assert X.main(["--student", "byte", "--teacher", "pair", "--top-k", "2", "--out", str(tmp_path / "p.pt")]) == 0
    assert torch.load(tmp_path / "p.pt", weights_only=False)["indices"].shape[1] == 2
