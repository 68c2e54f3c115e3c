"""Loss family and advantage estimators against hand-computed values (CPU)."""

import math

import pytest
import torch

from rl_b200.algorithms.advantage_estimator import GAEAdvantageEstimator, GRPOAdvantageEstimator, create_advantage_estimator
from rl_b200.algorithms.loss.loss_functions import ClippedPGLossFn, DPOLossFn, MseValueLossFn, NLLLossFn, PreferenceLossFn
from rl_b200.algorithms.reward_functions import apply_reward_shaping, scale_rewards
from rl_b200.algorithms.utils import calculate_baseline_and_std_per_prompt, calculate_kl, masked_mean
from rl_b200.distributed.batched_data_dict import BatchedDataDict


def _pg_data(B=3, S=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    tm = torch.ones(B, S)
    tm[:, :2] = 0
    return BatchedDataDict(
        token_mask=tm, sample_mask=torch.tensor([1.0, 1.0, 0.0][:B]), advantages=torch.randn(B, S, generator=g),
        prev_logprobs=-torch.rand(B, S, generator=g), generation_logprobs=-torch.rand(B, S, generator=g),
        reference_policy_logprobs=-torch.rand(B, S, generator=g))


def test_kl_estimators():
    a, b = torch.tensor([-1.0]), torch.tensor([-1.5])
    logr = -0.5
    assert calculate_kl(a, b, "k1").item() == pytest.approx(0.5)
    assert calculate_kl(a, b, "k2").item() == pytest.approx(0.125)
    assert calculate_kl(a, b, "k3").item() == pytest.approx(math.exp(logr) - 1 - logr)
    assert calculate_kl(torch.tensor([0.0]), torch.tensor([100.0]), "k3").item() == pytest.approx(10.0)  # output clamp


def test_clipped_pg_matches_manual():
    d = _pg_data()
    curr = (d["prev_logprobs"][:, 1:] + 0.3 * torch.randn(3, 5, generator=torch.Generator().manual_seed(1))).requires_grad_()
    fn = ClippedPGLossFn(dict(reference_policy_kl_penalty=0.1, ratio_clip_min=0.2, ratio_clip_max=0.3))
    mask = d["token_mask"][:, 1:] * d["sample_mask"][:, None]
    N = mask.sum()
    loss, m = fn(curr, d, torch.tensor(2.0), N)
    ratio = (curr - d["prev_logprobs"][:, 1:]).exp()
    A = d["advantages"][:, 1:]
    pg = torch.max(-A * ratio, -A * ratio.clamp(0.8, 1.3))
    logr = d["reference_policy_logprobs"][:, 1:] - curr
    kl = logr.exp() - 1 - logr
    want = ((pg + 0.1 * kl) * mask).sum() / (N + 1e-8)
    assert loss.item() == pytest.approx(want.item(), rel=1e-5)
    assert m["probs_ratio"] == pytest.approx(((ratio * mask).sum() / N).item(), rel=1e-5)
    assert m["num_valid_samples"] == 2
    loss.backward()
    assert curr.grad[2].abs().sum() == 0  # masked sample gets no gradient


def test_clipped_pg_variants_run_and_differ():
    d = _pg_data()
    curr = d["prev_logprobs"][:, 1:] + 0.5
    N = (d["token_mask"][:, 1:] * d["sample_mask"][:, None]).sum()
    base, _ = ClippedPGLossFn({})(curr, d, torch.tensor(2.0), N)
    dual, _ = ClippedPGLossFn({"ratio_clip_c": 3.0})(curr, d, torch.tensor(2.0), N)
    cispo, _ = ClippedPGLossFn({"use_cispo": True})(curr, d, torch.tensor(2.0), N)
    seq, ms = ClippedPGLossFn({"token_level_loss": False, "sequence_level_importance_ratios": True})(curr, d, torch.tensor(2.0), N)
    tis, mt = ClippedPGLossFn({"use_importance_sampling_correction": True, "truncated_importance_sampling_ratio": 1.1})(curr, d, torch.tensor(2.0), N)
    ice, mi = ClippedPGLossFn({"use_importance_sampling_correction": True, "truncated_importance_sampling_ratio": 1.5,
                               "truncated_importance_sampling_ratio_min": 0.8, "truncated_importance_sampling_type": "icepop"})(curr, d, torch.tensor(2.0), N)
    smt, _ = ClippedPGLossFn({"use_importance_sampling_correction": True, "truncated_importance_sampling_ratio": 1.002,
                              "truncated_importance_sampling_ratio_min": 0.999, "truncated_importance_sampling_type": "seq-mask-tis"})(curr, d, torch.tensor(2.0), N)
    onp, mo = ClippedPGLossFn({"force_on_policy_ratio": True})(curr, d, torch.tensor(2.0), N)
    assert mo["probs_ratio"] == pytest.approx(1.0)
    assert "is_oob_ratio" in mt and "is_oob_ratio" in mi
    assert dual.item() <= base.item() + 1e-6
    assert len({round(x.item(), 6) for x in (base, cispo, seq, tis, ice)}) >= 4


def test_nll_preference_dpo_value():
    B, S = 4, 5
    lp = -torch.rand(B, S - 1)
    d = BatchedDataDict(token_mask=torch.ones(B, S), sample_mask=torch.ones(B), reference_policy_logprobs=torch.zeros(B, S))
    loss, m = NLLLossFn()(lp, d, torch.tensor(4.0), torch.tensor(16.0))
    assert loss.item() == pytest.approx(-lp.mean().item(), rel=1e-5) and m["num_unmasked_tokens"] == 16
    scores = torch.tensor([2.0, 0.0, -1.0, 1.0])
    pl, pm = PreferenceLossFn()(scores, d, torch.tensor(4.0), torch.tensor(16.0))
    want = -(torch.nn.functional.logsigmoid(torch.tensor(2.0)) + torch.nn.functional.logsigmoid(torch.tensor(-2.0))) / 2
    assert pl.item() == pytest.approx(want.item(), rel=1e-5) and pm["accuracy"] == pytest.approx(0.5)
    dl, dm = DPOLossFn({"reference_policy_kl_penalty": 0.1, "sft_loss_weight": 0.5})(lp, d, torch.tensor(4.0), torch.tensor(16.0))
    r = lp.sum(-1)
    want = -(torch.nn.functional.logsigmoid(0.1 * (r[0] - r[1])) + torch.nn.functional.logsigmoid(0.1 * (r[2] - r[3]))) / 2
    assert dm["preference_loss"] == pytest.approx(want.item(), rel=1e-4) and dm["sft_loss"] > 0
    v = torch.randn(B, S)
    dv = BatchedDataDict(token_mask=torch.ones(B, S), sample_mask=torch.ones(B), returns=torch.zeros(B, S), old_values=v + 1.0)
    vl, vm = MseValueLossFn({"value_clip": 0.2})(v, dv, torch.tensor(4.0), torch.tensor(20.0))
    assert vl.item() >= 0.5 * (v ** 2).mean().item() - 1e-6


def test_baseline_leave_one_out_and_grpo_advantage():
    prompts = torch.tensor([[1, 2], [1, 2], [1, 2], [3, 4], [3, 4], [5, 6]])
    r = torch.tensor([1.0, 0.0, 1.0, 2.0, 4.0, 7.0])
    base, std = calculate_baseline_and_std_per_prompt(prompts, r, torch.ones(6), True)
    assert base.tolist() == pytest.approx([0.5, 1.0, 0.5, 4.0, 2.0, 7.0])
    assert std[5] == 0 and std[3] == 0  # a single other sample has no spread
    assert std[1].item() == pytest.approx(0.0) and std[0].item() == pytest.approx(math.sqrt(0.5))
    adv = GRPOAdvantageEstimator({"normalize_rewards": True}).compute_advantage(prompts, r, torch.ones(6, 3))
    assert adv[5].abs().sum() == 0 and adv.shape == (6, 3)
    assert adv[0, 0].item() == pytest.approx(0.5 / (math.sqrt(0.5) + 1e-6))
    assert adv[1, 0].item() == pytest.approx(-1.0)  # std 0: not divided
    est = create_advantage_estimator({"adv_estimator": {"name": "reinforce_plus_plus"}}, {})
    a2 = est.compute_advantage(prompts, r, torch.ones(6, 3))
    assert abs(a2.mean().item()) < 1e-5


def test_gae_matches_reference_scan():
    est = GAEAdvantageEstimator({"gamma": 0.9, "lambda": 0.8, "normalize_advantages": False})
    values = torch.tensor([[0.1, 0.2, 0.3, 0.4]])
    mask = torch.tensor([[0.0, 1.0, 1.0, 1.0]])
    adv, ret = est.compute_advantage(None, torch.tensor([1.0]), mask, values=values)
    d3 = 1.0 - 0.4
    d2 = 0.9 * 0.4 - 0.3
    d1 = 0.9 * 0.3 - 0.2
    a3 = d3
    a2 = d2 + 0.72 * a3
    a1 = d1 + 0.72 * a2
    assert adv[0].tolist() == pytest.approx([0.0, a1, a2, a3], abs=1e-6)
    assert ret[0, 3].item() == pytest.approx(a3 + 0.4)


def test_reward_shaping_and_scaling():
    b = BatchedDataDict(total_reward=torch.tensor([1.0, 1.0, 1.0]), generation_lengths=torch.tensor([50, 90, 100]), truncated=torch.tensor([False, False, True]))
    out = apply_reward_shaping(b, dict(enabled=True, overlong_buffer_length=20, overlong_buffer_penalty=1.0, max_response_length=100))
    assert out["total_reward"].tolist() == pytest.approx([1.0, 0.5, 0.0])
    b2 = BatchedDataDict(total_reward=torch.tensor([1.0, 2.0]), generation_lengths=torch.tensor([1, 1]), truncated=torch.tensor([True, False]))
    assert apply_reward_shaping(b2, dict(enabled=True, stop_properly_penalty_coef=0.0))["total_reward"].tolist() == [0.0, 2.0]
    b3 = BatchedDataDict(total_reward=torch.tensor([-1.0, 0.5, 3.0]))
    assert scale_rewards(b3, dict(enabled=True, source_min=0, source_max=1, target_min=-1, target_max=1))["total_reward"].tolist() == pytest.approx([-1.0, 0.0, 1.0])


def test_per_sequence_wrapper_equals_the_batched_loss_and_draft_wrapper_adds_up():
    from rl_b200.algorithms.loss.loss_functions import ClippedPGLossFn, DraftCrossEntropyLossFn
    from rl_b200.algorithms.loss.wrapper import DraftLossWrapper, PerSequenceLossWrapper, merge_metrics
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    torch.manual_seed(0)
    B, S, V = 3, 10, 7
    lens = torch.tensor([10, 6, 8])
    tm = (torch.arange(S)[None] < lens[:, None]).float()
    tm[:, :2] = 0
    data = BatchedDataDict(input_ids=torch.randint(0, V, (B, S)), input_lengths=lens, token_mask=tm, sample_mask=torch.tensor([1.0, 1.0, 0.5]),
                           advantages=torch.randn(B, S), prev_logprobs=-torch.rand(B, S), generation_logprobs=-torch.rand(B, S),
                           reference_policy_logprobs=-torch.rand(B, S))
    lp = (-torch.rand(B, S - 1)).requires_grad_()
    fn = ClippedPGLossFn(dict(reference_policy_kl_penalty=0.05))
    toks = (tm[:, 1:] * data["sample_mask"][:, None]).sum()
    seqs = data["sample_mask"].sum()
    kw = dict(data=data, global_valid_seqs=seqs, global_valid_toks=toks)
    full, m_full = fn(next_token_logprobs=lp, **kw)
    per, m_per = PerSequenceLossWrapper(fn)(next_token_logprobs=lp, **kw)
    assert torch.allclose(full, per, atol=1e-6) and m_per["num_valid_samples"] == pytest.approx(m_full["num_valid_samples"])
    g1 = torch.autograd.grad(full, lp, retain_graph=True)[0]
    g2 = torch.autograd.grad(per, lp)[0]
    assert torch.allclose(g1, g2, atol=1e-6)
    assert merge_metrics({"probs_ratio_min": 0.5, "x": 1}, {"probs_ratio_min": 0.2, "probs_ratio_max": float("inf"), "x": 2}) == {"probs_ratio_min": 0.2, "x": 3}
    draft = torch.randn(B, S - 1, V, requires_grad=True)
    target = torch.randn(B, S - 1, V)
    w = DraftLossWrapper(fn, draft_weight=0.5)
    both, m = w(draft_logits=draft, target_logits=target, next_token_logprobs=lp.detach().requires_grad_(), **kw)
    d_only, dm = DraftCrossEntropyLossFn()(draft, target, data, seqs, toks)
    assert torch.allclose(both, full.detach() + 0.5 * d_only, atol=1e-6) and m["draft_accuracy"] == dm["draft_accuracy"] and m["policy_loss"] == m_full["loss"]
    assert w(next_token_logprobs=lp, **kw)[0].item() == pytest.approx(full.item())      # no draft head: the policy loss alone
