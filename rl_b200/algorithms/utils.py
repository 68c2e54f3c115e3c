"""Numeric helpers shared by the algorithms: KL estimators, masked statistics, per-prompt baselines, seeding and
the performance metrics printed after each step.

Semantics follow nemo_rl/algorithms/utils.py:42-224 and :519-915 (tokens/s/GPU definitions at :791-822).
"""

from __future__ import annotations

import os
import random
from typing import Optional

import numpy as np
import torch


def calculate_kl(logprobs: torch.Tensor, logprobs_reference: torch.Tensor, kl_type: str = "k3",
                 input_clamp_value: Optional[float] = 20.0, output_clamp_value: Optional[float] = 10.0,
                 importance_sampling_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-token KL estimate between two log-probability tensors (Schulman's k1 / k2 / k3 estimators).

    ``logr = ref - logprobs`` is clamped to +-``input_clamp_value``; where the clamp bites, the importance weight
    stops carrying gradient too. The weighted estimate is clamped to +-``output_clamp_value``.
    """
    logr = logprobs_reference - logprobs
    w = importance_sampling_weights
    if input_clamp_value is not None:
        clamped = logr.clamp(-input_clamp_value, input_clamp_value)
        if w is not None:
            w = torch.where(logr == clamped, w, w.detach())
        logr = clamped
    if kl_type == "k1":
        kl = -logr
    elif kl_type == "k2":
        kl = 0.5 * logr * logr
    elif kl_type == "k3":
        kl = torch.expm1(logr) - logr
    else:
        raise ValueError(f"unknown KL estimator '{kl_type}' (k1, k2 or k3)")
    if w is not None:
        kl = w * kl
    if output_clamp_value is not None:
        kl = kl.clamp(-output_clamp_value, output_clamp_value)
    return kl


def masked_mean(values: torch.Tensor, mask: torch.Tensor, dim: Optional[int] = None,
                global_normalization_factor=None) -> torch.Tensor:
    """sum(values * mask) / (N + 1e-8), with N the mask sum or a caller-supplied global count."""
    denom = mask.sum(dim=dim) if global_normalization_factor is None else global_normalization_factor
    return (values * mask).sum(dim=dim) / (denom + 1e-8)


def masked_var(values: torch.Tensor, mask: torch.Tensor, unbiased: bool = True) -> torch.Tensor:
    mean = masked_mean(values, mask)
    var = masked_mean((values - mean) ** 2, mask)
    if unbiased:
        n = mask.sum()
        var = var * n / (n - 1).clamp(min=1)
    return var


def mask_out_neg_inf_logprobs(logprobs: torch.Tensor, mask: torch.Tensor, name: str = "logprobs"):
    """Tokens whose training-side logprob is -inf (they fell outside the trainer's top-k/top-p set) leave the loss."""
    bad = torch.isinf(logprobs)
    n_bad = int((bad & mask.bool()).sum())
    if n_bad:
        print(f"[warning] {n_bad}/{int(mask.sum())} valid tokens have -inf in {name}; masked out")
    mask = mask * (~bad).to(mask.dtype)
    return torch.where(mask.bool(), logprobs, torch.zeros_like(logprobs)), mask


def calculate_baseline_and_std_per_prompt(prompts: torch.Tensor, rewards: torch.Tensor, valid_mask: torch.Tensor,
                                          leave_one_out_baseline: bool = True,
                                          std_rewards: Optional[torch.Tensor] = None):
    """Per-sample baseline and standard deviation over the responses of the same prompt.

    Prompts are grouped by exact token equality. With ``leave_one_out_baseline`` the baseline of a response is the
    mean reward of the *other* valid responses to its prompt (RLOO). Groups with at most one valid response get
    baseline = reward (zero advantage). The std uses the same (leave-one-out) sample with Bessel's correction.
    Vectorised: one ``unique`` plus scatter-adds instead of a loop over prompts.
    """
    if std_rewards is None:
        std_rewards = rewards
    dev = rewards.device
    _, inv = torch.unique(prompts.to(dev), dim=0, return_inverse=True)
    G = int(inv.max().item()) + 1 if inv.numel() else 0
    vm = valid_mask.to(rewards.dtype)
    cnt = torch.zeros(G, device=dev, dtype=rewards.dtype).index_add_(0, inv, vm)
    s1 = torch.zeros(G, device=dev, dtype=rewards.dtype).index_add_(0, inv, rewards * vm)
    t1 = torch.zeros(G, device=dev, dtype=rewards.dtype).index_add_(0, inv, std_rewards * vm)
    t2 = torch.zeros(G, device=dev, dtype=rewards.dtype).index_add_(0, inv, std_rewards * std_rewards * vm)
    n_g, s_g, t1_g, t2_g = cnt[inv], s1[inv], t1[inv], t2[inv]
    if leave_one_out_baseline:
        # the left-out element is the sample itself whether or not it is valid (its masked value is removed)
        num_valid = n_g - 1
        base_sum = s_g - rewards * vm
        m1 = t1_g - std_rewards * vm
        m2 = t2_g - std_rewards * std_rewards * vm
    else:
        num_valid, base_sum, m1, m2 = n_g, s_g, t1_g, t2_g
    safe = num_valid.clamp(min=1)
    baseline = base_sum / safe
    mean = m1 / safe
    var = (m2 / safe - mean * mean) * (num_valid / (num_valid - 1))
    std = var.clamp(min=0).sqrt().nan_to_num(0.0, posinf=0.0, neginf=0.0)
    degenerate = n_g <= 1
    baseline = torch.where(degenerate, rewards, baseline)
    std = torch.where(degenerate, torch.zeros_like(std), std)
    return baseline, std


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def get_tokenizer(tokenizer_config: dict):
    """Loads a HF tokenizer by name; applies chat template overrides and makes sure a pad token exists."""
    if str(tokenizer_config.get("name", "")).lower() in ("byte", "bytes"):
        from rl_b200.data.tokenizers import ByteTokenizer

        return ByteTokenizer(int(tokenizer_config.get("vocab_size", 512)))
    if str(tokenizer_config.get("name", "")).lower() == "pair":
        from rl_b200.data.tokenizers import PairTokenizer

        return PairTokenizer(int(tokenizer_config.get("vocab_size", 1024)))
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(tokenizer_config["name"], trust_remote_code=True)
    tmpl = tokenizer_config.get("chat_template")
    if tmpl is not None:
        if str(tmpl).lower() == "default":
            pass
        elif os.path.exists(str(tmpl)):
            tok.chat_template = open(tmpl).read()
        else:
            tok.chat_template = tmpl
    if tok.pad_token is None:
        tok.pad_token = tok.eos_token
    return tok


def compute_performance_metrics(timing: dict, *, num_gpus: int, total_tokens: int, generated_tokens: int,
                                train_tokens: Optional[int] = None, logprob_tokens: Optional[int] = None) -> dict:
    """tokens/s/GPU = tokens / (stage time x #GPUs) for the whole step and per stage."""
    out = {}
    step = timing.get("total_step_time", 0.0)
    if step > 0:
        out["tokens_per_sec_per_gpu"] = total_tokens / step / num_gpus
    gen = timing.get("generation", 0.0)
    if gen > 0:
        out["generation_tokens_per_sec_per_gpu"] = generated_tokens / gen / num_gpus
    tr = timing.get("policy_training", 0.0)
    if tr > 0:
        out["policy_training_tokens_per_sec_per_gpu"] = (train_tokens or total_tokens) / tr / num_gpus
    lp = timing.get("policy_and_reference_logprobs", 0.0)
    if lp > 0:
        out["policy_and_reference_logprobs_tokens_per_sec_per_gpu"] = (logprob_tokens or total_tokens) / lp / num_gpus
    return out
