"""Loss family: ClippedPG (PPO / GRPO / DAPO / GSPO / CISPO / dual-clip / truncated-IS variants), NLL, preference
(Bradley-Terry), DPO, distillation KL, value MSE and draft cross-entropy.

Behaviour follows nemo_rl/algorithms/loss/loss_functions.py (ClippedPG :180-788, NLL :791-842, Preference
:853-946, DPO :966-1106, Distillation :1124-1206, MSE value :1218-1341, draft CE :66-108). All ``[B, S]`` inputs are
aligned to token positions; next-token quantities use ``[:, 1:]``.

On CUDA, the common token-level ClippedPG configuration runs as one fused kernel (loss terms, analytic gradient
and every metric partial sum in a single pass); every other configuration, and CPU, uses the PyTorch statement of
the same math below, which is also the oracle the kernel is tested against.
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from rl_b200.algorithms.utils import calculate_kl, masked_mean
from rl_b200.ops import lib as _L

from .interfaces import LossInputType, LossType

CLIPPED_PG_DEFAULTS = dict(
    disable_ppo_ratio=False,
    token_level_loss=True,
    sequence_level_importance_ratios=False,
    ratio_clip_min=0.2,
    ratio_clip_max=0.2,
    ratio_clip_c=None,
    reference_policy_kl_penalty=0.01,
    reference_policy_kl_type="k3",
    kl_input_clamp_value=20.0,
    kl_output_clamp_value=10.0,
    use_kl_in_reward=False,
    use_importance_sampling_correction=False,
    truncated_importance_sampling_type="tis",
    truncated_importance_sampling_ratio=None,
    truncated_importance_sampling_ratio_min=None,
    use_on_policy_kl_approximation=False,
    force_on_policy_ratio=False,
    use_cispo=False,
    positive_example_nll_weight=0.0,
)


def _nan_to_zero(x: torch.Tensor) -> torch.Tensor:
    return torch.nan_to_num(x, nan=0.0, posinf=0.0, neginf=0.0)


class _FusedPG(torch.autograd.Function):
    """Loss value and d loss / d curr_logprobs from the fused kernel."""

    @staticmethod
    def forward(ctx, curr, prev, gen, ref, adv, mask, cfg, inv_norm):
        T = curr.numel()
        dev = curr.device
        sums = torch.empty(16, dtype=torch.float32, device=dev)
        dcurr = torch.empty(T, dtype=torch.float32, device=dev)
        kl_type = {"k1": 1, "k2": 2, "k3": 3}[cfg["reference_policy_kl_type"]]
        tis_ratio = cfg["truncated_importance_sampling_ratio"]
        tis_type = 0
        if tis_ratio is not None:
            tis_type = {"tis": 1, "icepop": 2}[cfg["truncated_importance_sampling_type"]]
        tis_min = cfg["truncated_importance_sampling_ratio_min"]
        _L.call(
            "rlb_clipped_pg", _L.ptr(curr), _L.ptr(prev), _L.ptr(gen), _L.ptr(ref), _L.ptr(adv), _L.ptr(mask), T,
            float(cfg["ratio_clip_min"]), float(cfg["ratio_clip_max"]),
            float(cfg["ratio_clip_c"]) if cfg["ratio_clip_c"] is not None else -1.0,
            float(cfg["reference_policy_kl_penalty"]) if ref is not None else 0.0, kl_type,
            float(cfg["kl_input_clamp_value"] if cfg["kl_input_clamp_value"] is not None else 3e38),
            float(cfg["kl_output_clamp_value"] if cfg["kl_output_clamp_value"] is not None else 3e38),
            int(cfg["use_importance_sampling_correction"]), tis_type,
            float(tis_ratio) if tis_ratio is not None else 3e38, float(tis_min) if tis_min is not None else 0.0,
            int(cfg["force_on_policy_ratio"]), int(cfg["use_cispo"]), int(cfg["use_on_policy_kl_approximation"]),
            float(inv_norm), _L.ptr(sums), _L.ptr(dcurr), _L.stream_ptr(),
        )
        ctx.save_for_backward(dcurr)
        ctx.shape = curr.shape
        beta = float(cfg["reference_policy_kl_penalty"]) if ref is not None else 0.0
        loss = (sums[0] + beta * sums[1]) * inv_norm
        ctx.mark_non_differentiable(sums)
        return loss, sums

    @staticmethod
    def backward(ctx, dloss, _dsums):
        (dcurr,) = ctx.saved_tensors  # already carries mask / global-token normalisation
        return (dcurr * dloss).view(ctx.shape), None, None, None, None, None, None, None


class ClippedPGLossFn:
    """Clipped policy-gradient loss with optional KL penalty against a reference policy.

    ``loss = actor_loss + beta * KL(curr || ref) + mu * NLL(correct samples)`` where ``actor_loss`` is the masked mean
    of ``w_is * max(-A r, -A clip(r, 1-eps_lo, 1+eps_hi))`` (token-level: over all valid tokens of the global batch;
    sequence-level: mean over tokens then over samples).
    """

    input_type = LossInputType.LOGPROB

    def __init__(self, cfg: Optional[dict] = None):
        c = dict(CLIPPED_PG_DEFAULTS)
        c.update(cfg or {})
        self.cfg = c
        self.loss_type = LossType.TOKEN_LEVEL if c["token_level_loss"] else LossType.SEQUENCE_LEVEL
        if c["sequence_level_importance_ratios"]:
            assert self.loss_type == LossType.SEQUENCE_LEVEL, "sequence-level importance ratios need token_level_loss=false"
        if c["ratio_clip_c"] is not None:
            assert c["ratio_clip_c"] > 1, "ratio_clip_c is a lower bound on the ratio and must exceed 1"
        if c["truncated_importance_sampling_ratio"] is not None:
            assert c["use_importance_sampling_correction"], "truncated importance sampling needs the IS correction on"
            assert c["truncated_importance_sampling_type"] in ("tis", "icepop", "seq-mask-tis")
        for k, v in c.items():
            setattr(self, k, v)

    # ---- fused path applicability
    def _can_fuse(self, curr: torch.Tensor, data) -> bool:
        c = self.cfg
        return (
            curr.is_cuda and _L.use_native(curr) and self.loss_type == LossType.TOKEN_LEVEL
            and not c["disable_ppo_ratio"] and not c["sequence_level_importance_ratios"]
            and c["truncated_importance_sampling_type"] != "seq-mask-tis"
            and c["positive_example_nll_weight"] == 0 and "curr_logprobs_unfiltered" not in data
            and c["reference_policy_kl_type"] in ("k1", "k2", "k3")
        )

    def __call__(self, next_token_logprobs: torch.Tensor, data, global_valid_seqs, global_valid_toks):
        c = self.cfg
        curr = next_token_logprobs
        token_mask = data["token_mask"][:, 1:].to(curr.dtype)
        sample_mask = data["sample_mask"].to(curr.dtype)
        adv = data["advantages"][:, 1:]
        gen = data["generation_logprobs"][:, 1:]
        prev = curr.detach() if c["force_on_policy_ratio"] else data["prev_logprobs"][:, 1:]
        beta = c["reference_policy_kl_penalty"]
        ref = data["reference_policy_logprobs"][:, 1:] if beta != 0 else None
        mask = token_mask * sample_mask.unsqueeze(-1)
        if self._can_fuse(curr, data):
            return self._fused(curr, prev, gen, ref, adv, mask, sample_mask, global_valid_toks)
        return self._reference(curr, prev, gen, ref, adv, token_mask, sample_mask, mask, data, global_valid_seqs,
                               global_valid_toks)

    # ---- fused CUDA path
    def _fused(self, curr, prev, gen, ref, adv, mask, sample_mask, global_valid_toks):
        c = self.cfg
        beta = c["reference_policy_kl_penalty"]
        inv_norm = 1.0 / (float(global_valid_toks) + 1e-8)
        f = lambda t: None if t is None else t.float().contiguous()
        loss, sums = _FusedPG.apply(f(curr), f(prev), f(gen), f(ref), f(adv), f(mask), c, inv_norm)
        s = (sums.detach() * inv_norm).tolist()
        raw = sums.detach()
        rmin, rmax, cmin, cmax = raw[10].item(), raw[11].item(), raw[12].item(), raw[13].item()
        if raw[5].item() == 0:
            rmin, rmax, cmin, cmax = float("inf"), float("-inf"), float("inf"), float("-inf")
        metrics = {
            "loss": loss.item(),
            "probs_ratio": s[2],
            "probs_ratio_clamped": s[3],
            "probs_ratio_min": rmin,
            "probs_ratio_max": rmax,
            "probs_ratio_clamped_min": cmin,
            "probs_ratio_clamped_max": cmax,
            "kl_penalty": s[1] if beta != 0 else 0,
            "token_mult_prob_error": s[4],
            "gen_kl_error": s[6],
            "policy_kl_error": s[7],
            "js_divergence_error": s[14],
            "sampling_importance_ratio": s[8],
            "num_valid_samples": sample_mask.sum().item(),
            "approx_entropy": s[9],
            "positive_nll_loss": 0.0,
        }
        if c["truncated_importance_sampling_ratio"] is not None:
            metrics["is_oob_ratio"] = s[15]
        return loss, metrics

    # ---- PyTorch statement of the same math (CPU path, oracle, and every non-fused configuration)
    def _reference(self, curr, prev, gen, ref, adv, token_mask, sample_mask, mask, data, gvs, gvt):
        c = self.cfg
        beta = c["reference_policy_kl_penalty"]
        token_level = self.loss_type == LossType.TOKEN_LEVEL

        def reduce(x):
            if token_level:
                return masked_mean(x, mask, global_normalization_factor=gvt)
            return masked_mean(masked_mean(x, token_mask, dim=-1), sample_mask, global_normalization_factor=gvs)

        with torch.no_grad():
            mult_prob_error = masked_mean(torch.exp((gen - prev).abs() * mask), mask, global_normalization_factor=gvt).item()
            kt = c["reference_policy_kl_type"]
            gen_kl = masked_mean(calculate_kl(gen, prev, kt, None, None), mask, global_normalization_factor=gvt).item()
            pol_kl = masked_mean(calculate_kl(prev, gen, kt, None, None), mask, global_normalization_factor=gvt).item()
            log_mix = torch.log(0.5 * prev.exp() + 0.5 * gen.exp())
            k3 = lambda d: torch.expm1(d) - d
            js = masked_mean(0.5 * k3(prev - log_mix) + 0.5 * k3(gen - log_mix), mask, global_normalization_factor=gvt).item()

        if beta != 0:
            curr_unf = data.get("curr_logprobs_unfiltered", curr)
            if c["use_on_policy_kl_approximation"]:
                kw = torch.exp(curr_unf - gen)
            else:
                kw = torch.exp(curr_unf - curr_unf.detach())
            kw = _nan_to_zero(kw)
            kl_tok = calculate_kl(curr_unf, ref, c["reference_policy_kl_type"], c["kl_input_clamp_value"],
                                  c["kl_output_clamp_value"], importance_sampling_weights=kw)
            kl = beta * reduce(kl_tok)
        else:
            kl = torch.zeros((), device=curr.device)

        if c["force_on_policy_ratio"]:
            ratios = (curr - curr.detach()).exp()
            ratios_clamped = ratios
        elif not c["disable_ppo_ratio"]:
            log_ratios = curr - prev
            if c["sequence_level_importance_ratios"]:
                seq = masked_mean(log_ratios, token_mask, dim=-1).unsqueeze(-1).exp()
                ratios = seq.expand(-1, adv.shape[1])
            else:
                ratios = log_ratios.exp()
            ratios_clamped = ratios.clamp(1.0 - c["ratio_clip_min"], 1.0 + c["ratio_clip_max"])
        else:
            ratios = curr
            ratios_clamped = curr

        if c["use_cispo"]:
            clip_loss = -adv * ratios_clamped.detach() * curr
        else:
            clip_loss = torch.max(-adv * ratios, -adv * ratios_clamped)
        if c["ratio_clip_c"] is not None:
            clip_loss = torch.where(adv < 0, torch.min(clip_loss, -adv * c["ratio_clip_c"]), clip_loss)

        # importance weights between the trainer's and the generator's probabilities of the sampled tokens
        extra: dict[str, Any] = {}
        if c["sequence_level_importance_ratios"]:
            w = _nan_to_zero(torch.exp(((prev - gen) * mask).sum(-1)).detach()).unsqueeze(-1)
        else:
            w = _nan_to_zero(torch.exp(prev - gen))
        tr = c["truncated_importance_sampling_ratio"]
        if tr is not None:
            kind = c["truncated_importance_sampling_type"]
            tmin = c["truncated_importance_sampling_ratio_min"]
            if kind == "tis":
                tmin = 0.0 if tmin is None else tmin
                oob = (w > tr) | (w < tmin)
                extra["is_oob_ratio"] = masked_mean(oob.float().expand_as(mask), mask, global_normalization_factor=gvt).item()
                w = w.clamp(tmin, tr)
            elif kind == "icepop":
                keep = (w >= tmin) & (w <= tr)
                extra["is_oob_ratio"] = masked_mean((~keep).float().expand_as(mask), mask, global_normalization_factor=gvt).item()
                w = torch.where(keep, w, torch.zeros_like(w))
            else:  # seq-mask-tis: drop whole sequences whose geometric-mean IS ratio leaves [min, max]
                geo = masked_mean(_nan_to_zero(prev - gen), token_mask, dim=-1).exp().detach()
                keep = ((geo >= tmin) & (geo <= tr)).float()
                extra["is_oob_ratio"] = masked_mean(1.0 - keep, sample_mask, global_normalization_factor=gvs).item()
                w = w * keep.unsqueeze(-1)
        w_used = w if c["use_importance_sampling_correction"] else torch.ones_like(prev)
        actor_loss = reduce(w_used * clip_loss)

        if c["sequence_level_importance_ratios"]:
            sir = masked_mean(w.squeeze(-1), sample_mask, global_normalization_factor=gvs)
        else:
            sir = masked_mean(w, mask, global_normalization_factor=gvt)
        with torch.no_grad():
            approx_entropy = -masked_mean(torch.exp(curr - gen) * curr, mask, global_normalization_factor=gvt)

        nll = torch.zeros((), device=curr.device)
        mu = c["positive_example_nll_weight"]
        if mu > 0 and "rewards" in data:
            cm = mask * (data["rewards"] > 0).to(mask.dtype).unsqueeze(-1)
            n = cm.sum()
            if n > 0:
                nll = masked_mean(-curr, cm, global_normalization_factor=n)

        loss = actor_loss + kl + mu * nll
        with torch.no_grad():
            pr = masked_mean(ratios.detach().expand_as(mask), mask, global_normalization_factor=gvt).item()
            prc = masked_mean(ratios_clamped.detach().expand_as(mask), mask, global_normalization_factor=gvt).item()
            sel = mask.bool()
            mr, mrc = ratios.detach().expand_as(mask)[sel], ratios_clamped.detach().expand_as(mask)[sel]
            if mr.numel():
                rmin, rmax, cmin, cmax = mr.min().item(), mr.max().item(), mrc.min().item(), mrc.max().item()
            else:
                rmin, rmax, cmin, cmax = float("inf"), float("-inf"), float("inf"), float("-inf")
        metrics = {
            "loss": loss.item(),
            "probs_ratio": pr,
            "probs_ratio_clamped": prc,
            "probs_ratio_min": rmin,
            "probs_ratio_max": rmax,
            "probs_ratio_clamped_min": cmin,
            "probs_ratio_clamped_max": cmax,
            "kl_penalty": kl.item() / beta if beta != 0 else 0,
            "token_mult_prob_error": mult_prob_error,
            "gen_kl_error": gen_kl,
            "policy_kl_error": pol_kl,
            "js_divergence_error": js,
            "sampling_importance_ratio": sir.item(),
            "num_valid_samples": sample_mask.sum().item(),
            "approx_entropy": approx_entropy.item(),
            **extra,
            "positive_nll_loss": nll.item(),
        }
        return loss, metrics


class NLLLossFn:
    """Teacher-forced negative log-likelihood over masked tokens (SFT)."""

    loss_type = LossType.TOKEN_LEVEL
    input_type = LossInputType.LOGPROB

    def __call__(self, next_token_logprobs, data, global_valid_seqs, global_valid_toks, dpo_loss: bool = False,
                 dpo_average_log_probs: bool = False):
        token_mask = data["token_mask"][:, 1:].to(next_token_logprobs.dtype)
        sample_mask = data["sample_mask"].to(next_token_logprobs.dtype)
        mask = token_mask * sample_mask.unsqueeze(-1)
        if dpo_loss:
            # per-sample (optionally length-averaged) NLL, averaged over valid sequences
            per = -(next_token_logprobs * mask).sum(-1)
            if dpo_average_log_probs:
                per = per / mask.sum(-1).clamp(min=1)
            num_unmasked = sample_mask.sum()
            loss = (per * sample_mask).sum() / (global_valid_seqs + 1e-8)
        else:
            num_unmasked = mask.sum()
            loss = -masked_mean(next_token_logprobs, mask, global_normalization_factor=global_valid_toks)
        return loss, {"loss": loss.item() if loss.dim() == 0 else loss,
                      "num_unmasked_tokens": num_unmasked.item(), "num_valid_samples": sample_mask.sum().item()}


class PreferenceLossFn:
    """Bradley-Terry loss on reward-model scores; rows alternate chosen, rejected, chosen, rejected..."""

    loss_type = LossType.SEQUENCE_LEVEL
    input_type = LossInputType.LOGIT
    requires_pairs = True  # rows 2i / 2i+1 belong together: micro-batches must not separate or reorder them

    @staticmethod
    def split(t: torch.Tensor):
        return t[0::2], t[1::2]

    def _preference_loss(self, rewards: torch.Tensor, sample_mask: torch.Tensor, global_valid_seqs, beta: float = 1.0):
        rc, rr = self.split(rewards)
        m = sample_mask[0::2]
        diff = beta * (rc - rr)
        gv = global_valid_seqs / 2
        per = -torch.nn.functional.logsigmoid(diff)
        loss = masked_mean(per, m, global_normalization_factor=gv)
        acc = masked_mean((diff > 0).float(), m, global_normalization_factor=gv)
        rc_mean = masked_mean(rc, m, global_normalization_factor=gv)
        rr_mean = masked_mean(rr, m, global_normalization_factor=gv)
        return loss, acc, rc_mean, rr_mean

    def __call__(self, logits, data, global_valid_seqs, global_valid_toks):
        rewards = logits.squeeze(-1) if logits.dim() > 1 else logits
        sample_mask = data["sample_mask"].to(rewards.dtype)
        loss, acc, rc, rr = self._preference_loss(rewards.float(), sample_mask, global_valid_seqs)
        n = sample_mask.sum() / 2
        return loss, {"loss": loss.item(), "accuracy": acc.item(), "rewards_chosen_mean": rc.item(),
                      "rewards_rejected_mean": rr.item(), "num_valid_samples": n.item()}


DPO_DEFAULTS = dict(reference_policy_kl_penalty=0.05, preference_loss_weight=1.0, sft_loss_weight=0.0,
                    preference_average_log_probs=False, sft_average_log_probs=False)


class DPOLossFn(PreferenceLossFn):
    """Direct preference optimisation: -log sigmoid(beta * ((pi_c - ref_c) - (pi_r - ref_r))) plus an optional SFT
    term on the chosen responses."""

    loss_type = LossType.SEQUENCE_LEVEL
    input_type = LossInputType.LOGPROB

    def __init__(self, cfg: Optional[dict] = None):
        c = dict(DPO_DEFAULTS)
        c.update(cfg or {})
        self.cfg = c
        self.sft = NLLLossFn()

    def __call__(self, next_token_logprobs, data, global_valid_seqs, global_valid_toks):
        c = self.cfg
        token_mask = data["token_mask"][:, 1:].to(next_token_logprobs.dtype)
        sample_mask = data["sample_mask"].to(next_token_logprobs.dtype)
        ref = data["reference_policy_logprobs"][:, 1:]
        diff = (next_token_logprobs - ref) * token_mask
        rewards = diff.sum(-1)
        if c["preference_average_log_probs"]:
            rewards = rewards / token_mask.sum(-1).clamp(min=1)
        pref, acc, rc, rr = self._preference_loss(rewards, sample_mask, global_valid_seqs, beta=c["reference_policy_kl_penalty"])
        sft = torch.zeros((), device=rewards.device)
        if c["sft_loss_weight"] > 0:
            sft_all, _ = self.sft(next_token_logprobs, data, global_valid_seqs, global_valid_toks, dpo_loss=True,
                                  dpo_average_log_probs=c["sft_average_log_probs"])
            # only the chosen rows carry the SFT term; recompute on them
            per = -(next_token_logprobs * token_mask).sum(-1)
            if c["sft_average_log_probs"]:
                per = per / token_mask.sum(-1).clamp(min=1)
            sft = masked_mean(per[0::2], sample_mask[0::2], global_normalization_factor=global_valid_seqs / 2)
        loss = c["preference_loss_weight"] * pref + c["sft_loss_weight"] * sft
        n = sample_mask.sum() / 2
        return loss, {"loss": loss.item(), "sft_loss": sft.item(), "preference_loss": pref.item(), "accuracy": acc.item(),
                      "rewards_chosen_mean": rc.item(), "rewards_rejected_mean": rr.item(), "num_valid_samples": n.item()}


class DistillationLossFn:
    """KL between teacher and student over the teacher's top-k vocabulary entries.

    ``kl_type``: forward KL(teacher || student), reverse KL(student || teacher), or ``mixed`` = weighted sum.
    ``zero_outside_topk`` renormalises both distributions over the top-k set before comparing.
    """

    loss_type = LossType.TOKEN_LEVEL
    input_type = LossInputType.DISTILLATION

    def __init__(self, cfg: Optional[dict] = None):
        c = dict(kl_type="mixed", mixed_kl_weight=0.5, zero_outside_topk=False)
        c.update(cfg or {})
        assert c["kl_type"] in ("forward", "reverse", "mixed")
        self.cfg = c

    def __call__(self, student_topk_logprobs, teacher_topk_logprobs, data, global_valid_seqs, global_valid_toks, H_all=None):
        c = self.cfg
        token_mask = data["token_mask"][:, 1:].to(student_topk_logprobs.dtype)
        sample_mask = data["sample_mask"].to(student_topk_logprobs.dtype)
        mask = token_mask * sample_mask.unsqueeze(-1)
        s, t = student_topk_logprobs, teacher_topk_logprobs
        if c["zero_outside_topk"]:
            s = s - torch.logsumexp(s, -1, keepdim=True)
            t = t - torch.logsumexp(t, -1, keepdim=True)
        fwd = (t.exp() * (t - s)).sum(-1)
        rev = (s.exp() * (s - t)).sum(-1)
        if c["kl_type"] == "forward":
            per = fwd
        elif c["kl_type"] == "reverse":
            per = rev
        else:
            per = c["mixed_kl_weight"] * fwd + (1 - c["mixed_kl_weight"]) * rev
        per = per[:, : mask.shape[1]]
        loss = masked_mean(per, mask, global_normalization_factor=global_valid_toks)
        return loss, {"loss": loss.item(), "num_valid_samples": sample_mask.sum().item()}


class MseValueLossFn:
    """Clipped value-function regression for PPO critics: 0.5 * max((v - R)^2, (clip(v, v_old +- eps) - R)^2)."""

    loss_type = LossType.TOKEN_LEVEL
    input_type = LossInputType.VALUE

    def __init__(self, cfg: Optional[dict] = None):
        c = dict(value_clip=None)
        c.update(cfg or {})
        self.cfg = c

    def __call__(self, values, data, global_valid_seqs, global_valid_toks):
        token_mask = data["token_mask"].to(values.dtype)
        sample_mask = data["sample_mask"].to(values.dtype)
        mask = token_mask * sample_mask.unsqueeze(-1)
        returns = data["returns"]
        err = (values - returns) ** 2
        clip_frac = torch.zeros((), device=values.device)
        eps = self.cfg["value_clip"]
        if eps is not None and "old_values" in data:
            old = data["old_values"]
            vclip = old + (values - old).clamp(-eps, eps)
            err_clip = (vclip - returns) ** 2
            clip_frac = masked_mean((err_clip > err).float(), mask, global_normalization_factor=global_valid_toks)
            err = torch.max(err, err_clip)
        loss = 0.5 * masked_mean(err, mask, global_normalization_factor=global_valid_toks)
        with torch.no_grad():
            vmean = masked_mean(values, mask, global_normalization_factor=global_valid_toks)
        return loss, {"loss": loss.item(), "value_mean": vmean.item(), "value_clip_frac": clip_frac.item(),
                      "num_valid_samples": sample_mask.sum().item()}


class DraftCrossEntropyLossFn:
    """Soft-target cross-entropy between a draft head's logits and the policy's (detached) distribution, used to
    train speculative-decoding draft heads alongside the policy."""

    loss_type = LossType.TOKEN_LEVEL
    input_type = LossInputType.DRAFT

    def __call__(self, draft_logits, target_logits, data, global_valid_seqs, global_valid_toks, token_mask=None):
        """``token_mask`` [B, S - 1]: which predictions count, when they are not the plain next-token ones (a draft that reads
        the following token's embedding predicts one position further, so its mask is shifted once more)."""
        token_mask = (data["token_mask"][:, 1:] if token_mask is None else token_mask).to(torch.float32)
        sample_mask = data["sample_mask"].to(torch.float32)
        mask = token_mask * sample_mask.unsqueeze(-1)
        tgt = torch.softmax(target_logits.float().detach(), dim=-1)
        logp = torch.log_softmax(draft_logits.float(), dim=-1)
        per = -(tgt * logp).sum(-1)[:, : mask.shape[1]]
        loss = masked_mean(per, mask, global_normalization_factor=global_valid_toks)
        with torch.no_grad():
            agree = (draft_logits.argmax(-1) == target_logits.argmax(-1)).float()[:, : mask.shape[1]]
            acc = masked_mean(agree, mask, global_normalization_factor=global_valid_toks)
        return loss, {"loss": loss.item(), "draft_accuracy": acc.item(), "num_valid_samples": sample_mask.sum().item()}
