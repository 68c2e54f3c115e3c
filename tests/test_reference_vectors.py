"""Numeric cases of the reference's own unit tests, restated as inputs and expected values for this framework's
classes: ClippedPG in its PPO / REINFORCE / CISPO / dual-clip / KL / importance-sampling forms, the KL estimators with
their clamps and gradients, the OPD advantage, reward scaling and shaping. The inputs and the hand-computed expectations
come from tests/unit/algorithms/test_loss_functions.py, test_advantage_estimator.py and test_reward_functions.py of
NVIDIA-NeMo/RL; passing them pins the semantics, not just self-consistency."""

import math

import pytest
import torch

from rl_b200.algorithms.advantage_estimator import OPDAdvantageEstimator
from rl_b200.algorithms.loss.loss_functions import ClippedPGLossFn
from rl_b200.algorithms.reward_functions import apply_reward_shaping, scale_rewards
from rl_b200.algorithms.utils import calculate_kl
from rl_b200.distributed.batched_data_dict import BatchedDataDict


def _data(adv, prev, gen=None, ref=None, B=1, S=4):
    """One sequence of 4 tokens, the first masked: the reference's mock batch."""
    tm = torch.ones(B, S)
    tm[:, 0] = 0
    z = lambda: torch.zeros(B, S)
    d = BatchedDataDict(token_mask=tm, sample_mask=torch.ones(B), advantages=z(), prev_logprobs=z(), generation_logprobs=z(),
                        reference_policy_logprobs=z())
    d["advantages"][0, 1:] = torch.tensor(adv)
    d["prev_logprobs"][0, 1:] = torch.tensor(prev)
    d["generation_logprobs"][0, 1:] = torch.tensor(gen if gen is not None else prev)
    if ref is not None:
        d["reference_policy_logprobs"][0, 1:] = torch.tensor(ref)
    return d


def _loss(cfg, curr, data):
    fn = ClippedPGLossFn(cfg)
    mask = data["token_mask"][:, 1:] * data["sample_mask"][:, None]
    return fn(torch.tensor([curr]), data, data["sample_mask"].sum(), mask.sum())


RATIO_CASE = dict(adv=[1.0, -1.0, 2.0], prev=[-1.0, -1.0, -1.0], curr=[-1.69315, -1.0, -0.59453])   # ratios 0.5, 1.0, 1.5


def test_ppo_clipping_vector():
    # max(-A r, -A clip(r, 0.8, 1.2)) = [-0.5, 1.0, -2.4]; mean = -0.6333
    loss, _ = _loss(dict(reference_policy_kl_penalty=0.0), RATIO_CASE["curr"], _data(RATIO_CASE["adv"], RATIO_CASE["prev"]))
    assert loss.item() == pytest.approx(-1.9 / 3, rel=1e-3)


def test_reinforce_mode_vector():
    # disable_ppo_ratio: loss = -A * logprob = [0.5, -1.0, 3.0]; mean = 0.8333
    loss, _ = _loss(dict(reference_policy_kl_penalty=0.0, disable_ppo_ratio=True, ratio_clip_min=0.0, ratio_clip_max=0.0),
                    [-0.5, -1.0, -1.5], _data([1.0, -1.0, 2.0], [0.0, 0.0, 0.0]))
    assert loss.item() == pytest.approx(2.5 / 3, rel=1e-4)


def test_cispo_vector():
    # -A * clip(r).detach() * logprob with clip(r) = [0.8, 1.0, 1.2]
    c = RATIO_CASE
    want = sum(-a * r * lp for a, r, lp in zip(c["adv"], [0.8, 1.0, 1.2], c["curr"])) / 3
    loss, _ = _loss(dict(reference_policy_kl_penalty=0.0, use_cispo=True), c["curr"], _data(c["adv"], c["prev"]))
    assert loss.item() == pytest.approx(want, rel=1e-3)


def test_dual_clip_vector():
    # ratios [0.5, 1, 10], A = [1, -1, -4], c = 3: clip loss [-0.5, 1.0, 12.0] (40 capped at 12); mean = 4.1667
    loss, _ = _loss(dict(reference_policy_kl_penalty=0.0, ratio_clip_c=3.0), [-1.69315, -1.0, -0.69741],
                    _data([1.0, -1.0, -4.0], [-1.0, -1.0, -3.0]))
    assert loss.item() == pytest.approx(12.5 / 3, rel=1e-3)


def test_kl_penalty_vector():
    # zero advantages: loss = 0.1 * mean(exp(r) - r - 1), r = ref - curr = [-1, 0, 1] -> [0.368, 0, 0.718] -> 0.0362
    loss, m = _loss(dict(reference_policy_kl_penalty=0.1), [0.0, -1.0, -2.0], _data([0.0, 0.0, 0.0], [0.0, 0.0, 0.0], ref=[-1.0, -1.0, -1.0]))
    want = 0.1 * ((math.exp(-1) + 1 - 1) + 0.0 + (math.exp(1) - 1 - 1)) / 3
    assert loss.item() == pytest.approx(want, rel=1e-4) and loss.item() == pytest.approx(0.0362, rel=2e-3)


def test_icepop_vector():
    # on-policy ratios, IS weights exp(prev - gen) = [0.6065, 12.18, 0.8187]; [0.5, 5] keeps the first and third
    prev, gen, adv = [-1.0, -1.0, -1.0], [-0.5, -3.5, -0.8], [1.0, -1.0, 2.0]
    cfg = dict(reference_policy_kl_penalty=0.0, use_importance_sampling_correction=True, truncated_importance_sampling_type="icepop",
               truncated_importance_sampling_ratio=5.0, truncated_importance_sampling_ratio_min=0.5)
    loss, _ = _loss(cfg, prev, _data(adv, prev, gen=gen))
    want = (math.exp(-0.5) * -1.0 + 0.0 + math.exp(-0.2) * -2.0) / 3
    assert loss.item() == pytest.approx(want, rel=1e-3)


def test_tis_out_of_bounds_ratio_vector():
    cfg = dict(reference_policy_kl_penalty=0.0, use_importance_sampling_correction=True, truncated_importance_sampling_type="tis",
               truncated_importance_sampling_ratio=2.0)
    d = _data([1.0, 1.0, 1.0], [math.log(1.0), math.log(3.0), math.log(0.5)], gen=[0.0, 0.0, 0.0])
    _, m = _loss(cfg, [0.0, 0.0, 0.0], d)
    assert m["is_oob_ratio"] == pytest.approx(1.0 / 3.0)


@pytest.mark.parametrize("kl_type,plain,clamped", [
    ("k1", [-1.0, 14.0, 29.0], [-1.0, 10.0, 10.0]),
    ("k2", [0.5, 98.0, 420.5], [0.5, 10.0, 10.0]),
    ("k3", [0.7183, 13.0, 28.0], [0.7183, 10.0, 10.0]),
])
def test_kl_estimator_vectors(kl_type, plain, clamped):
    lp, ref = torch.tensor([[-1.0, -1.0, -1.0]]), torch.tensor([[-0.0, -15.0, -30.0]])
    assert torch.allclose(calculate_kl(lp, ref, kl_type, None, None), torch.tensor([plain]), rtol=1e-3)
    assert torch.allclose(calculate_kl(lp, ref, kl_type, 20.0, 10.0), torch.tensor([clamped]), rtol=1e-3)


def test_kl_input_clamp_detaches_the_sampling_weight():
    lp = torch.tensor([[-3.0, -1.0]], requires_grad=True)
    w = torch.exp(lp - lp.detach())
    kl = calculate_kl(lp, torch.zeros_like(lp), "k3", 2.0, None, importance_sampling_weights=w)
    torch.testing.assert_close(kl.detach(), torch.tensor([[4.389056, 0.7182818]]))
    kl.sum().backward()
    torch.testing.assert_close(lp.grad, torch.tensor([[0.0, -1.0]]), atol=1e-6, rtol=1e-6)


def test_kl_output_clamp_applies_after_the_weight_and_blocks_its_gradient():
    lp = torch.tensor([[-1.0]], requires_grad=True)
    w = 100.0 * torch.exp(lp - lp.detach())
    kl = calculate_kl(lp, torch.zeros_like(lp), "k3", None, 1.0, importance_sampling_weights=w)
    torch.testing.assert_close(kl.detach(), torch.tensor([[1.0]]))
    kl.sum().backward()
    torch.testing.assert_close(lp.grad, torch.zeros_like(lp), atol=1e-6, rtol=1e-6)


def test_opd_advantage_vectors():
    est = OPDAdvantageEstimator({"name": "opd"}, {})
    B, S = 2, 4
    t, s_ = torch.zeros(B, S), torch.full((B, S), -1.0)
    adv = est.compute_advantage(torch.arange(B), torch.zeros(B), torch.ones(B, S), teacher_logprobs=t, prev_logprobs=s_)
    assert adv.shape == (B, S) and (adv > 0).all()
    assert est.last_metrics["on_policy_distillation/teacher_student_logprob_gap_mean"] == pytest.approx(1.0)
    assert est.last_metrics["on_policy_distillation/adv_mean"] == pytest.approx(1.0)
    assert est.last_metrics["on_policy_distillation/adv_std"] == pytest.approx(0.0, abs=1e-5)
    lp = torch.randn(B, S)
    torch.testing.assert_close(est.compute_advantage(torch.arange(B), torch.zeros(B), torch.ones(B, S), teacher_logprobs=lp, prev_logprobs=lp),
                               torch.zeros(B, S))
    mask = torch.tensor([[1, 1, 1, 0, 0, 0]], dtype=torch.float32)
    adv = est.compute_advantage(torch.arange(1), torch.zeros(1), mask, teacher_logprobs=torch.zeros(1, 6), prev_logprobs=torch.full((1, 6), -1.0))
    assert (adv[:, 3:] == 0).all() and (adv[:, :3] > 0).all()


def _reward_batch(lengths, rewards, **extra):
    return BatchedDataDict(total_reward=torch.tensor(rewards), generation_lengths=torch.tensor(lengths), **extra)


def test_reward_scaling_vectors():
    b = scale_rewards(_reward_batch([10, 20, 30], [1.0, 0.5, 0.8]), dict(enabled=True, source_min=0.0, source_max=1.0, target_min=0.0, target_max=0.7))
    assert torch.allclose(b["total_reward"], torch.tensor([0.7, 0.35, 0.56]))
    b = scale_rewards(_reward_batch([10] * 5, [1.0, 0.0, 0.0, 1.0, 0.0]), dict(enabled=True, source_min=0.0, source_max=1.0, target_min=-1.0, target_max=1.0))
    assert torch.allclose(b["total_reward"], torch.tensor([1.0, -1.0, -1.0, 1.0, -1.0]))
    b = scale_rewards(_reward_batch([10] * 6, [-2.8, -0.25, 1.5, 0.5, 2.0, 2.5]),
                      dict(enabled=True, source_min=-2.0, source_max=2.0, target_min=-1.0, target_max=1.0))
    assert torch.allclose(b["total_reward"], torch.tensor([-1.0, -0.125, 0.75, 0.25, 1.0, 1.0]))
    orig = _reward_batch([10, 20, 30], [1.0, 0.5, 0.8])
    assert scale_rewards(orig, dict(enabled=False)) is orig


def test_overlong_shaping_vectors():
    # max 25, buffer 5 -> expected 20; lengths 10 / 22 / 25 / 30 lose 0 / 0.2 / 0.5 / 1.0
    b = apply_reward_shaping(_reward_batch([10, 22, 25, 30], [1.0, 0.8, 0.6, 0.4]),
                             dict(enabled=True, overlong_buffer_length=5, overlong_buffer_penalty=0.5, max_response_length=25))
    assert torch.allclose(b["total_reward"], torch.tensor([1.0, 0.6, 0.1, -0.6]), atol=1e-6)
    assert torch.allclose(b["unshaped_reward"], torch.tensor([1.0, 0.8, 0.6, 0.4]))


def test_stop_properly_penalty_vectors():
    b = apply_reward_shaping(_reward_batch([10, 20, 30, 40], [1.0, 0.8, 0.6, 0.4], truncated=torch.tensor([False, True, False, True])),
                             dict(enabled=True, stop_properly_penalty_coef=0.5))
    assert torch.allclose(b["total_reward"], torch.tensor([1.0, 0.4, 0.6, 0.2]), atol=1e-6)
    b = apply_reward_shaping(_reward_batch([10, 20], [1.0, 0.5], truncated=torch.tensor([True, True])), dict(enabled=True, stop_properly_penalty_coef=0.0))
    assert torch.allclose(b["total_reward"], torch.tensor([0.0, 0.0]))
