"""Encode / decode / chat-template throughput of a tokenizer on synthetic or file text (role of tools/benchmark_fastokens.py:
deciding whether tokenisation can keep up with the data loader).

    python -m rl_b200.tools.benchmark_tokenizer --tokenizer byte [--file corpus.txt] [--docs 2000] [--batch 64]
"""

from __future__ import annotations

import argparse
import json
import random
import time


def synthetic_docs(n: int, words: int = 200, seed: int = 0) -> list[str]:
    rng = random.Random(seed)
    vocab = ["the", "of", "and", "to", "in", "is", "that", "for", "x", "y", "=", "+", "1", "2", "3", "\\frac{a}{b}", "therefore", "solve", "answer"]
    return [" ".join(rng.choice(vocab) for _ in range(words)) for _ in range(n)]


def benchmark(tokenizer, docs: list[str], batch: int = 64) -> dict:
    t0 = time.perf_counter()
    enc = [tokenizer.encode(d) for d in docs]
    t_enc = time.perf_counter() - t0
    ntok = sum(len(e) for e in enc)
    t0 = time.perf_counter()
    for e in enc[: max(1, len(enc) // 4)]:
        tokenizer.decode(e)
    t_dec = time.perf_counter() - t0
    out = dict(docs=len(docs), tokens=ntok, chars=sum(len(d) for d in docs), encode_tokens_per_s=ntok / max(t_enc, 1e-9),
               decode_tokens_per_s=sum(len(e) for e in enc[: max(1, len(enc) // 4)]) / max(t_dec, 1e-9), chars_per_token=sum(len(d) for d in docs) / max(1, ntok))
    if hasattr(tokenizer, "apply_chat_template"):
        t0 = time.perf_counter()
        for d in docs[:batch]:
            tokenizer.apply_chat_template([{"role": "user", "content": d}], tokenize=False, add_generation_prompt=True)
        out["chat_templates_per_s"] = min(batch, len(docs)) / max(time.perf_counter() - t0, 1e-9)
    return out


def main(argv=None) -> int:
    from rl_b200.algorithms.utils import get_tokenizer

    ap = argparse.ArgumentParser()
    ap.add_argument("--tokenizer", default="byte")
    ap.add_argument("--file")
    ap.add_argument("--docs", type=int, default=2000)
    ap.add_argument("--batch", type=int, default=64)
    a = ap.parse_args(argv)
    tok = get_tokenizer({"name": a.tokenizer})
    if a.file:
        with open(a.file) as f:
            docs = [l.strip() for l in f if l.strip()][: a.docs]
    else:
        docs = synthetic_docs(a.docs)
    print(json.dumps(benchmark(tok, docs, a.batch)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
