"""Advantage estimators: GRPO (group-relative, leave-one-out), GDPO (per-component normalisation of multi-reward
signals), Reinforce++ (global batch normalisation, optional per-prompt baseline), raw rewards, GAE (with VAPO's
decoupled / length-adaptive lambda), and OPD (teacher-minus-student log-ratio for on-policy distillation).

Semantics follow nemo_rl/algorithms/advantage_estimator.py:57-627. Every estimator returns a ``[B, S]`` tensor
aligned to token positions (the per-sample advantage broadcast over tokens for the outcome-reward estimators).
"""

from __future__ import annotations

from typing import Optional

import torch

from rl_b200.algorithms.utils import calculate_baseline_and_std_per_prompt, masked_mean, masked_var


class GRPOAdvantageEstimator:
    """A_i = (r_i - baseline_i) / (std_i + 1e-6); baseline / std over the responses of the same prompt."""

    def __init__(self, cfg: dict, loss_cfg: Optional[dict] = None):
        self.use_leave_one_out_baseline = cfg.get("use_leave_one_out_baseline", True)
        self.normalize_rewards = cfg.get("normalize_rewards", True)

    def compute_advantage(self, prompt_ids, rewards, mask, **kw) -> torch.Tensor:
        valid = kw.get("valid_mask", torch.ones_like(rewards))
        baseline, std = calculate_baseline_and_std_per_prompt(prompt_ids, rewards, valid, self.use_leave_one_out_baseline)
        adv = (rewards - baseline).unsqueeze(-1)
        if self.normalize_rewards:
            std = std.unsqueeze(-1)
            nz = std > 0
            adv = torch.where(nz, adv / (std + 1e-6), adv)
        return adv.expand(mask.shape).clone()


class GDPOAdvantageEstimator:
    """Multi-reward GRPO: every reward component is normalised per prompt on its own, the normalised components are
    combined with ``reward_weights`` and the sum is normalised over the batch."""

    def __init__(self, cfg: dict, loss_cfg: Optional[dict] = None):
        self.use_leave_one_out_baseline = cfg.get("use_leave_one_out_baseline", True)
        self.normalize_rewards = cfg.get("normalize_rewards", True)
        self.reward_weights = cfg.get("reward_weights")

    def compute_advantage(self, prompt_ids, rewards, mask, reward_components: Optional[torch.Tensor] = None, **kw):
        comps = reward_components if reward_components is not None else rewards.unsqueeze(-1)
        valid = kw.get("valid_mask", torch.ones(comps.shape[0], device=comps.device, dtype=comps.dtype))
        K = comps.shape[1]
        w = torch.tensor(self.reward_weights or [1.0] * K, device=comps.device, dtype=comps.dtype)
        total = torch.zeros(comps.shape[0], device=comps.device, dtype=comps.dtype)
        for k in range(K):
            base, std = calculate_baseline_and_std_per_prompt(prompt_ids, comps[:, k], valid, self.use_leave_one_out_baseline)
            a = comps[:, k] - base
            if self.normalize_rewards:
                a = torch.where(std > 0, a / (std + 1e-6), a)
            total = total + w[k] * a
        if self.normalize_rewards and total.numel() > 1:
            # batch statistics over every data-parallel rank's samples (unbiased std, as torch.std)
            mean, var, n = _global_masked_moments(total, torch.ones_like(total), kw.get("dp_group"))
            std = (var * n / max(n - 1.0, 1.0)).sqrt()
            total = (total - mean) / (std + 1e-6)
        return total.unsqueeze(-1).expand(mask.shape).clone()


def _global_masked_moments(x: torch.Tensor, mask: torch.Tensor, group=None):
    """Mean and biased variance of ``x`` over the masked entries of EVERY data-parallel rank (one all-reduce of
    sum / sum of squares / count), so that whitening does not depend on how the batch is split over ranks."""
    import torch.distributed as dist

    m = mask.to(torch.float64)
    xd = x.to(torch.float64)
    stats = torch.stack([(xd * m).sum(), (xd * xd * m).sum(), m.sum()])
    if group != "self" and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        buf = stats.cuda() if dist.get_backend(group) == "nccl" else stats.cpu()
        dist.all_reduce(buf, group=group)
        stats = buf.to(x.device)
    n = stats[2].clamp(min=1.0)
    mean = stats[0] / n
    var = (stats[1] / n - mean * mean).clamp(min=0.0)
    return mean.to(x.dtype), var.to(x.dtype), float(stats[2])


class ReinforcePlusPlusAdvantageEstimator:
    """Reinforce++: optional per-prompt mean baseline, a per-token KL penalty subtracted from the reward
    (``use_kl_in_reward``), then whitening over all valid tokens of the global batch with the biased variance
    clamped at 1e-8 (nemo_rl/algorithms/advantage_estimator.py:233-265). ``kl_reward_to_go: true`` (off by default, an
    extension) charges each token with the penalties of the tokens after it as well."""

    def __init__(self, cfg: dict, loss_cfg: Optional[dict] = None):
        self.minus_baseline = cfg.get("minus_baseline", True)
        self.reward_to_go = bool(cfg.get("kl_reward_to_go", False))
        self.loss_cfg = loss_cfg or {}

    def compute_advantage(self, prompt_ids, rewards, mask, logprobs_policy=None, logprobs_reference=None, **kw):
        valid = kw.get("valid_mask", torch.ones_like(rewards))
        r = rewards
        if self.minus_baseline:
            base, _ = calculate_baseline_and_std_per_prompt(prompt_ids, rewards, valid, leave_one_out_baseline=False)
            r = rewards - base
        adv = r.unsqueeze(-1).expand(mask.shape).clone()
        if self.loss_cfg.get("use_kl_in_reward") and logprobs_policy is not None and logprobs_reference is not None:
            from rl_b200.algorithms.utils import calculate_kl

            kl = calculate_kl(logprobs_policy, logprobs_reference, self.loss_cfg.get("reference_policy_kl_type", "k3"))
            beta = self.loss_cfg.get("reference_policy_kl_penalty", 0.0)
            pen = beta * kl
            if self.reward_to_go:
                pen = (pen * mask).flip(-1).cumsum(-1).flip(-1)
            adv = adv - pen
        mean, var, _ = _global_masked_moments(adv, mask, kw.get("dp_group"))
        return (adv - mean) * var.clamp(min=1e-8).rsqrt()


class RawAdvantageEstimator:
    """Advantage = reward, broadcast over tokens."""

    def __init__(self, cfg: dict, loss_cfg: Optional[dict] = None):
        pass

    def compute_advantage(self, prompt_ids, rewards, mask, **kw):
        return rewards.unsqueeze(-1).expand(mask.shape).clone()


class GAEAdvantageEstimator:
    """Generalised advantage estimation over response tokens with a terminal outcome reward.

    delta_t = r_t + gamma V_{t+1} - V_t,  A_t = delta_t + gamma lambda A_{t+1} (reverse scan over the masked span).
    VAPO options: ``lambda_policy`` decoupled from the critic's lambda, and a length-adaptive
    lambda = 1 - 1 / (alpha * L) per sequence. Returns (advantages, returns); returns = A(lambda_critic) + V.
    """

    def __init__(self, cfg: dict, loss_cfg: Optional[dict] = None):
        self.gamma = cfg.get("gamma", 1.0)
        self.lam = cfg.get("lambda", cfg.get("gae_lambda", 0.95))
        self.lam_critic = cfg.get("lambda_critic", self.lam)
        self.length_adaptive_alpha = cfg.get("length_adaptive_alpha")
        self.normalize = cfg.get("normalize_advantages", True)

    def _scan(self, token_rewards, values, mask, lam):
        B, S = values.shape
        adv = torch.zeros_like(values)
        last = torch.zeros(B, device=values.device, dtype=values.dtype)
        next_v = torch.zeros(B, device=values.device, dtype=values.dtype)
        lam_t = lam if isinstance(lam, torch.Tensor) else torch.full((B,), float(lam), device=values.device, dtype=values.dtype)
        for t in range(S - 1, -1, -1):
            m = mask[:, t]
            delta = token_rewards[:, t] + self.gamma * next_v - values[:, t]
            cur = delta + self.gamma * lam_t * last
            last = torch.where(m > 0, cur, last)
            next_v = torch.where(m > 0, values[:, t], next_v)
            adv[:, t] = cur * m
        return adv

    def compute_advantage(self, prompt_ids, rewards, mask, values: Optional[torch.Tensor] = None,
                          token_rewards: Optional[torch.Tensor] = None, **kw):
        assert values is not None, "GAE needs value predictions"
        m = mask.to(values.dtype)
        if token_rewards is None:
            # outcome reward on the last valid token of every sequence
            token_rewards = torch.zeros_like(values)
            idx = (m * torch.arange(m.shape[1], device=m.device)).argmax(-1)
            has = m.sum(-1) > 0
            token_rewards[torch.arange(m.shape[0], device=m.device)[has], idx[has]] = rewards[has].to(values.dtype)
        lam_pol = self.lam
        if self.length_adaptive_alpha:
            L = m.sum(-1).clamp(min=1)
            lam_pol = (1.0 - 1.0 / (self.length_adaptive_alpha * L)).clamp(0.0, 1.0)
        adv = self._scan(token_rewards, values, m, lam_pol)
        adv_c = adv if (self.lam_critic == self.lam and not self.length_adaptive_alpha) else self._scan(token_rewards, values, m, self.lam_critic)
        returns = (adv_c + values) * m
        if self.normalize:
            mean = masked_mean(adv, m)
            var = masked_var(adv, m)
            adv = (adv - mean) * torch.rsqrt(var + 1e-8) * m
        return adv, returns


class OPDAdvantageEstimator:
    """On-policy distillation signal: per-token advantage = teacher logprob - student logprob of the sampled token
    (a reverse-KL gradient estimate), optionally added to the outcome-reward advantage."""

    def __init__(self, cfg: dict, loss_cfg: Optional[dict] = None):
        self.coef = cfg.get("opd_coef", 1.0)
        self.reward_coef = cfg.get("reward_coef", 0.0)
        self.inner = GRPOAdvantageEstimator(cfg) if self.reward_coef else None

    def compute_advantage(self, prompt_ids, rewards, mask, teacher_logprobs=None, logprobs_policy=None, prev_logprobs=None, **kw):
        student = logprobs_policy if logprobs_policy is not None else prev_logprobs
        assert teacher_logprobs is not None and student is not None
        gap = (teacher_logprobs - student).detach()
        adv = self.coef * gap * mask
        n = mask.sum().clamp(min=1)
        mean = (adv * mask).sum() / n
        self.last_metrics = {
            "on_policy_distillation/teacher_student_logprob_gap_mean": float((gap * mask).sum() / n),
            "on_policy_distillation/adv_mean": float(mean),
            "on_policy_distillation/adv_std": float((((adv - mean) ** 2 * mask).sum() / n).sqrt()),
        }
        if self.inner is not None:
            adv = adv + self.reward_coef * self.inner.compute_advantage(prompt_ids, rewards, mask, **kw)
        return adv


_ESTIMATORS = {
    "grpo": GRPOAdvantageEstimator,
    "gdpo": GDPOAdvantageEstimator,
    "reinforce_plus_plus": ReinforcePlusPlusAdvantageEstimator,
    "raw": RawAdvantageEstimator,
    "gae": GAEAdvantageEstimator,
    "opd": OPDAdvantageEstimator,
}


def create_advantage_estimator(grpo_cfg: dict, loss_cfg: Optional[dict] = None):
    """Builds the estimator named by ``grpo.adv_estimator.name`` (default: grpo with the top-level
    ``normalize_rewards`` / ``use_leave_one_out_baseline`` switches)."""
    est = dict(grpo_cfg.get("adv_estimator") or {})
    name = est.get("name", "grpo")
    est.setdefault("normalize_rewards", grpo_cfg.get("normalize_rewards", True))
    est.setdefault("use_leave_one_out_baseline", grpo_cfg.get("use_leave_one_out_baseline", True))
    if name not in _ESTIMATORS:
        raise ValueError(f"unknown advantage estimator '{name}' ({sorted(_ESTIMATORS)})")
    return _ESTIMATORS[name](est, loss_cfg)
