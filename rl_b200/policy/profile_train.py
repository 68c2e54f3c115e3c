"""Training-phase profiler: one log-prob pass and one optimizer step of the policy worker on synthetic packed batches.

    python -m rl_b200.policy.profile_train --model llama3.1-8b --layers 4 --seqs 8 --seq-len 1280 --mb-tokens 5120

Prints CUDA-event times of the log-prob pass, of forward + backward and of the optimizer step, with the model FLOPs they
stand for. With ``--layers 4`` and one micro-batch it is small enough to list every kernel under
``ncu --metrics gpu__time_duration.sum``.
"""

from __future__ import annotations

import argparse
import json

import torch

from rl_b200.algorithms.loss.loss_functions import ClippedPGLossFn
from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.models.config import preset
from rl_b200.policy.worker import PolicyWorker


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3.1-8b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=1280)
    ap.add_argument("--mb-tokens", type=int, default=5120)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    mc = preset(a.model)
    if a.layers:
        mc.num_hidden_layers = a.layers
    cfg = dict(precision="bfloat16", train_global_batch_size=a.seqs, train_micro_batch_size=4, logprob_batch_size=8,
               max_total_sequence_length=a.seq_len, max_grad_norm=1.0, grad_dtype="float32",
               sequence_packing=dict(enabled=True, train_mb_tokens=a.mb_tokens, logprob_mb_tokens=4 * a.mb_tokens),
               optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=3e-7, weight_decay=0.01)))
    w = PolicyWorker(cfg, model_cfg=mc, init_reference_model=False, seed=0)
    g = torch.Generator().manual_seed(0)
    n, S = a.seqs, a.seq_len
    data = BatchedDataDict(input_ids=torch.randint(0, mc.vocab_size, (n, S), generator=g), input_lengths=torch.full((n,), S),
                           token_mask=torch.cat([torch.zeros(n, S // 5), torch.ones(n, S - S // 5)], 1), sample_mask=torch.ones(n),
                           advantages=torch.randn(n, S, generator=g), generation_logprobs=-torch.rand(n, S, generator=g))
    loss_fn = ClippedPGLossFn(dict(reference_policy_kl_penalty=0.01))
    times = {"logprobs": [], "train": []}
    for it in range(a.iters):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        torch.cuda.synchronize()
        ev[0].record()
        w.prepare_for_lp_inference()
        lp = w.get_logprobs(data)["logprobs"]
        ev[1].record()
        data["prev_logprobs"], data["reference_policy_logprobs"] = lp, lp
        w.prepare_for_training()
        w.train(data, loss_fn, gbs=n, mbs=4)
        ev[2].record()
        torch.cuda.synchronize()
        times["logprobs"].append(ev[0].elapsed_time(ev[1]))
        times["train"].append(ev[1].elapsed_time(ev[2]))
    tokens = n * S
    params = mc.num_parameters() - mc.vocab_size * mc.hidden_size   # the input embedding is a lookup
    attn = 4 * mc.num_hidden_layers * mc.q_size * S / 2               # causal QK^T + PV FLOPs per token (forward)
    fwd = tokens * (2 * params + attn)
    out = dict(model=a.model, layers=mc.num_hidden_layers, tokens=tokens, logprob_ms=round(min(times["logprobs"]), 2),
               train_ms=round(min(times["train"]), 2), logprob_tflops=round(fwd / min(times["logprobs"]) / 1e9, 1),
               train_tflops=round(3 * fwd / min(times["train"]) / 1e9, 1))
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
