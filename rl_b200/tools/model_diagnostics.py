"""Model diagnostics (the checks of the reference's tools/model_diagnostics/*.py as sub-commands of one tool).

    python -m rl_b200.tools.model_diagnostics decode-vs-prefill --model tiny-llama-oracle
    python -m rl_b200.tools.model_diagnostics max-len --model tiny-llama-oracle
    python -m rl_b200.tools.model_diagnostics embeddings --path /ckpt/hf_dir

``decode-vs-prefill``  long generation, then the same tokens scored in one prefill pass: the incremental (paged-KV decode)
                       and the full-sequence log-probabilities must agree; drift here is what makes
                       ``token_mult_prob_error`` grow with response length.
``max-len``            the engine never returns more than ``max_model_len`` tokens per sequence and marks cut responses.
``embeddings``         rows of the embedding / output matrices that were never trained (all-zero or exactly at their
                       initial scale) — special tokens added after pre-training show up here.
"""

from __future__ import annotations

import argparse
import json
import sys

import torch


def _engine(model_name: str, device: str, max_model_len: int, layers: int = 0):
    from rl_b200.engine.engine import GenerationEngine
    from rl_b200.models.config import preset
    from rl_b200.models.transformer import build_model

    dt = torch.float32 if device == "cpu" else torch.bfloat16
    mc = preset(model_name, torch_dtype="float32" if device == "cpu" else "bfloat16")
    if layers:
        mc.num_hidden_layers = layers
    model = build_model(mc, device=device, dtype=dt, seed=0)
    eng = GenerationEngine(model, block_size=16, kv_cache_tokens=8 * (max_model_len + 64), max_running=8, max_model_len=max_model_len,
                           use_cuda_graphs=device != "cpu")
    return mc, model, eng


def decode_vs_prefill(model_name: str, device: str, prompt_len: int = 32, new_tokens: int = 256, layers: int = 0) -> dict:
    from rl_b200.engine.engine import SamplingParams
    from rl_b200.models.transformer import PackedBatch

    mc, model, eng = _engine(model_name, device, prompt_len + new_tokens + 8, layers)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, mc.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(4)]
    recs = eng.generate(prompts, SamplingParams(max_new_tokens=new_tokens, stop_token_ids=[], seed=1))
    worst, mean, by_quarter = 0.0, 0.0, [0.0] * 4
    for r in recs:
        seq = torch.tensor([r.prompt + r.out_tokens], device=device)
        b = PackedBatch.from_padded(seq, torch.tensor([seq.shape[1]], device=device))
        if device != "cpu":
            b.input_ids = b.input_ids.to(torch.int32)
        with torch.no_grad():
            lp, _ = model.next_token_logprobs(b)
        gap = (lp[len(r.prompt):].float().cpu() - torch.tensor(r.out_logprobs)).abs()
        worst, mean = max(worst, float(gap.max())), mean + float(gap.mean()) / len(recs)
        q = max(1, gap.numel() // 4)
        for i in range(4):
            by_quarter[i] += float(gap[i * q : (i + 1) * q].mean()) / len(recs)
    tol = 1e-4 if device == "cpu" else 0.05
    return dict(check="decode-vs-prefill", mean_abs_gap=mean, max_abs_gap=worst, mean_gap_by_response_quarter=by_quarter, ok=mean < tol)


def max_len(model_name: str, device: str, layers: int = 0) -> dict:
    from rl_b200.engine.engine import SamplingParams

    mc, model, eng = _engine(model_name, device, 48, layers)
    prompts = [[1] * 40, [2] * 10]
    recs = eng.generate(prompts, SamplingParams(max_new_tokens=64, stop_token_ids=[], seed=1))
    lens = [len(r.prompt) + len(r.out_tokens) for r in recs]
    return dict(check="max-len", total_lengths=lens, truncated=[bool(r.truncated) for r in recs], ok=all(n <= 48 for n in lens) and all(r.truncated for r in recs))


def embeddings(path: str) -> dict:
    from rl_b200.models import hf_io

    model = hf_io.load_pretrained(path, dtype=torch.float32)
    out = {"check": "embeddings"}
    for name, w in (("embed_tokens", model.embed_tokens), ("lm_head", model.lm_head)):
        if w is None:
            continue
        w = w.detach().float()
        norms = w.norm(dim=1)
        med = float(norms.median())
        zero = (norms == 0).nonzero()[:, 0].tolist()
        tiny = ((norms > 0) & (norms < 0.1 * med)).nonzero()[:, 0].tolist()
        out[name] = dict(rows=w.shape[0], median_norm=med, zero_rows=zero[:32], num_zero=len(zero), far_below_median=tiny[:32], num_far_below=len(tiny))
    out["ok"] = all(v.get("num_zero", 0) == 0 for v in out.values() if isinstance(v, dict))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("decode-vs-prefill", "max-len"):
        p = sub.add_parser(name)
        p.add_argument("--model", default="tiny-llama-oracle")
        p.add_argument("--layers", type=int, default=0)
        p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    sub.choices["decode-vs-prefill"].add_argument("--new-tokens", type=int, default=256)
    p = sub.add_parser("embeddings")
    p.add_argument("--path", required=True)
    a = ap.parse_args(argv)
    if a.cmd == "decode-vs-prefill":
        res = decode_vs_prefill(a.model, a.device, new_tokens=a.new_tokens, layers=a.layers)
    elif a.cmd == "max-len":
        res = max_len(a.model, a.device, a.layers)
    else:
        res = embeddings(a.path)
    print(json.dumps(res))
    return 0 if res["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
