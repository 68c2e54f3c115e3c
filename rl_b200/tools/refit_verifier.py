"""Refit verifier: after a weight hand-over, the serving engine must score a batch exactly like the trainer does.

    python -m rl_b200.tools.refit_verifier --model tiny-llama-oracle --steps 2

Builds a policy and its engine, perturbs the trainer's weights (an optimizer step on random data), refits, generates, and
compares the engine's log-probabilities of the sampled tokens with the trainer's on the same tokens. Prints the maximum
absolute difference and ``token_mult_prob_error``; non-zero exit status when they exceed the tolerance. Role of the
reference's tools/refit_verifier.py.
"""

from __future__ import annotations

import argparse
import json
import sys

import torch


def verify(model: str = "tiny-llama-oracle", steps: int = 2, batch: int = 8, prompt_len: int = 16, new_tokens: int = 16, tol: float = 5e-2,
           device: str = "cpu") -> dict:
    from rl_b200.algorithms.grpo import refit_policy_generation
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import preset
    from rl_b200.policy.worker import PolicyWorker

    mc = preset(model, torch_dtype="float32" if device == "cpu" else "bfloat16")
    cfg = dict(precision="float32" if device == "cpu" else "bfloat16", train_global_batch_size=batch, train_micro_batch_size=batch,
               logprob_batch_size=batch, max_total_sequence_length=prompt_len + new_tokens + 8,
               optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-2)),
               generation=dict(max_new_tokens=new_tokens, temperature=1.0, stop_token_ids=[], kv_cache_tokens=batch * (prompt_len + new_tokens + 64),
                               block_size=16, max_running=max(8, batch)))
    policy = PolicyWorker(cfg, model_cfg=mc, init_reference_model=False, seed=0)
    gen = policy.build_generation(cfg["generation"])
    g = torch.Generator().manual_seed(0)
    out = {"steps": []}
    for s in range(steps):
        ids = torch.randint(0, mc.vocab_size, (batch, prompt_len), generator=g)
        data = BatchedDataDict(input_ids=ids, input_lengths=torch.full((batch,), prompt_len), token_mask=torch.ones(batch, prompt_len), sample_mask=torch.ones(batch))
        policy.prepare_for_training()
        policy.train(data, NLLLossFn(), gbs=batch, mbs=batch)      # weights move
        refit_policy_generation(policy, gen, None)
        res = gen.generate(data)
        gen.finish_generation()
        seq = BatchedDataDict(input_ids=res["output_ids"], input_lengths=res["unpadded_sequence_lengths"])
        policy.prepare_for_lp_inference()
        lp = policy.get_logprobs(seq)["logprobs"]
        mask = (res["logprobs"] != 0).float()
        diff = ((lp - res["logprobs"]).abs() * mask)
        err = float(torch.exp(diff.sum() / mask.sum().clamp(min=1)))
        out["steps"].append(dict(step=s + 1, max_abs_diff=float(diff.max()), token_mult_prob_error=err))
    out["ok"] = all(x["max_abs_diff"] <= tol for x in out["steps"])
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-llama-oracle")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--tol", type=float, default=5e-2)
    a = ap.parse_args(argv)
    res = verify(a.model, a.steps, tol=a.tol, device=a.device)
    print(json.dumps(res))
    return 0 if res["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
