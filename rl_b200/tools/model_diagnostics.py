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
``precision``          engine against trainer on the same samples with and without captured graphs: the
                       ``token_mult_prob_error`` the perf suite gates on (< 1.1), per mode.
``prefix-caching``     the same prompts with the prefix cache and chunked prefill on and off: equal tokens under greedy
                       decoding, finite log-probabilities, and the second pass served from cached blocks.
``routed-experts``     a mixture-of-experts model records the experts of every token in every MoE layer of a rollout
                       (what router replay and expert-load traces rely on).
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


def precision(model_name: str, device: str, layers: int = 0, new_tokens: int = 64) -> dict:
    import math

    from rl_b200.engine.engine import GenerationEngine, SamplingParams
    from rl_b200.models.transformer import PackedBatch

    mc, model, _ = _engine(model_name, device, 32 + new_tokens + 8, layers)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, mc.vocab_size, (32,), generator=g).tolist() for _ in range(8)]
    out = {"check": "precision"}
    for graphs in ((True, False) if device != "cpu" else (False,)):
        eng = GenerationEngine(model, block_size=16, kv_cache_tokens=8 * (new_tokens + 96), max_running=8, max_model_len=32 + new_tokens + 8,
                               use_cuda_graphs=graphs)
        recs = eng.generate(prompts, SamplingParams(max_new_tokens=new_tokens, stop_token_ids=[], seed=2))
        tot, n = 0.0, 0
        for r in recs:
            seq = torch.tensor([r.prompt + r.out_tokens], device=device)
            b = PackedBatch.from_padded(seq, torch.tensor([seq.shape[1]], device=device))
            if device != "cpu":
                b.input_ids = b.input_ids.to(torch.int32)
            with torch.no_grad():
                lp, _ = model.next_token_logprobs(b)
            gap = (lp[len(r.prompt):].float().cpu() - torch.tensor(r.out_logprobs)).abs()
            tot, n = tot + float(gap.sum()), n + gap.numel()
        out["graphs" if graphs else "eager"] = math.exp(tot / max(1, n))
    out["ok"] = all(v < 1.1 for k, v in out.items() if k in ("graphs", "eager"))
    return out


def prefix_caching(model_name: str, device: str, layers: int = 0) -> dict:
    from rl_b200.engine.engine import GenerationEngine, SamplingParams

    mc, model, _ = _engine(model_name, device, 160, layers)
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(0, mc.vocab_size, (64,), generator=g).tolist()
    prompts = [shared + torch.randint(0, mc.vocab_size, (8 + i,), generator=g).tolist() for i in range(4)]
    sp = SamplingParams(max_new_tokens=16, stop_token_ids=[], greedy=True)
    res = {}
    for on in (False, True):
        eng = GenerationEngine(model, block_size=16, kv_cache_tokens=8 * 256, max_running=8, max_model_len=160, use_cuda_graphs=False,
                               enable_prefix_caching=on, max_prefill_tokens=48 if on else 0)
        first = eng.generate(prompts, sp, share_prefixes=False)
        second = eng.generate(prompts, sp, share_prefixes=False) if on else first
        res[on] = (first, second, dict(eng.stats))
    same = all(a.out_tokens == b.out_tokens for a, b in zip(res[False][0], res[True][0])) and \
        all(a.out_tokens == b.out_tokens for a, b in zip(res[True][0], res[True][1]))
    finite = all(all(x == x and abs(x) < 1e4 for x in r.out_logprobs) for r in res[True][1])
    cached = int(res[True][2].get("cached_prefix_tokens", 0))
    return dict(check="prefix-caching", same_tokens=same, finite_logprobs=finite, cached_prefix_tokens=cached, ok=same and finite and cached > 0)


def routed_experts(device: str) -> dict:
    from rl_b200.engine.engine import GenerationEngine, SamplingParams
    from rl_b200.models.config import preset
    from rl_b200.models.transformer import PackedBatch, build_model
    from rl_b200.utils import routing_trace as R

    dt = torch.float32 if device == "cpu" else torch.bfloat16
    mc = preset("tiny-llama-oracle", torch_dtype="float32" if device == "cpu" else "bfloat16", num_experts=8, num_experts_per_tok=2,
                moe_intermediate_size=128, hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128)
    model = build_model(mc, device=device, dtype=dt, seed=0)
    eng = GenerationEngine(model, block_size=16, kv_cache_tokens=2048, max_running=8, max_model_len=96, use_cuda_graphs=False)
    recs = eng.generate([[1, 2, 3, 4, 5, 6], [7, 8, 9]], SamplingParams(max_new_tokens=8, stop_token_ids=[], seed=1))
    seqs = [r.prompt + r.out_tokens for r in recs]
    S = max(len(x) for x in seqs)
    ids = torch.zeros((len(seqs), S), dtype=torch.long, device=device)
    for i, x in enumerate(seqs):
        ids[i, : len(x)] = torch.tensor(x)
    b = PackedBatch.from_padded(ids, torch.tensor([len(x) for x in seqs], device=device))
    if device != "cpu":
        b.input_ids = b.input_ids.to(torch.int32)
    with torch.no_grad():
        model.hidden_states(b)
    tr = R.capture(model)
    T = sum(len(x) for x in seqs)
    complete = len(tr) == mc.num_hidden_layers and all(t.shape == (T, mc.num_experts_per_tok) for t in tr.values())
    in_range = all(int(t.min()) >= 0 and int(t.max()) < mc.num_experts for t in tr.values())
    return dict(check="routed-experts", layers=len(tr), tokens=T, ok=complete and in_range)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("decode-vs-prefill", "max-len", "precision", "prefix-caching"):
        p = sub.add_parser(name)
        p.add_argument("--model", default="tiny-llama-oracle")
        p.add_argument("--layers", type=int, default=0)
        p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    sub.choices["decode-vs-prefill"].add_argument("--new-tokens", type=int, default=256)
    p = sub.add_parser("embeddings")
    p.add_argument("--path", required=True)
    p = sub.add_parser("routed-experts")
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    if a.cmd == "precision":
        res = precision(a.model, a.device, a.layers)
    elif a.cmd == "prefix-caching":
        res = prefix_caching(a.model, a.device, a.layers)
    elif a.cmd == "routed-experts":
        res = routed_experts(a.device)
    elif a.cmd == "decode-vs-prefill":
        res = decode_vs_prefill(a.model, a.device, new_tokens=a.new_tokens, layers=a.layers)
    elif a.cmd == "max-len":
        res = max_len(a.model, a.device, a.layers)
    else:
        res = embeddings(a.path)
    print(json.dumps(res))
    return 0 if res["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
