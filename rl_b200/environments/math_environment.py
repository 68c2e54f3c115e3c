"""Math answer verification environment (single turn).

The reference scores responses with HF ``math-verify`` inside Ray worker actors
(nemo_rl/environments/math_environment.py:87-555). Here verification is a self-contained normaliser: it extracts the
last ``\\boxed{...}`` (or the text after "answer is" / the last number), canonicalises LaTeX fractions, units, thousands
separators and surrounding text, and compares numerically (relative 1e-6) or symbolically through ``sympy`` when that
package is importable. Workers are a thread pool (verification is CPU-light).
"""

from __future__ import annotations

import re
from concurrent.futures import ThreadPoolExecutor
from fractions import Fraction
from typing import Optional

import torch

from .interfaces import EnvironmentReturn


def extract_boxed(text: str) -> Optional[str]:
    """Content of the last balanced ``\\boxed{...}`` / ``\\fbox{...}``."""
    idx = max(text.rfind("\\boxed"), text.rfind("\\fbox"))
    if idx < 0:
        return None
    i = text.find("{", idx)
    if i < 0:
        rest = text[idx:].split()
        return rest[1] if len(rest) > 1 else None
    depth, j = 0, i
    while j < len(text):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[i + 1 : j]
        j += 1
    return None


def extract_answer(text: str) -> Optional[str]:
    b = extract_boxed(text)
    if b is not None:
        return b
    m = re.findall(r"(?:final answer|answer)\s*(?:is|:|=)\s*\$?([^\n$]+)", text, flags=re.I)
    if m:
        return m[-1].strip().rstrip(".")
    nums = re.findall(r"-?\d[\d,]*\.?\d*(?:/\d+)?", text)
    return nums[-1] if nums else None


_FRAC = re.compile(r"\\[dt]?frac\s*\{([^{}]+)\}\s*\{([^{}]+)\}")


def normalize_answer(s: str) -> str:
    s = s.strip().strip("$").strip()
    s = re.sub(r"\\text\s*\{[^{}]*\}", "", s)
    s = re.sub(r"\\(?:left|right|!|,|;|:| )", "", s)
    s = s.replace("\\%", "").replace("%", "").replace("^\\circ", "").replace("^{\\circ}", "").replace("°", "")
    s = s.replace("\\$", "").replace("$", "")
    for _ in range(4):
        s2 = _FRAC.sub(r"(\1)/(\2)", s)
        if s2 == s:
            break
        s = s2
    s = re.sub(r"\\sqrt\s*\{([^{}]+)\}", r"sqrt(\1)", s)
    s = s.replace("\\cdot", "*").replace("\\times", "*").replace("\\pi", "pi")
    s = re.sub(r"(?<=\d),(?=\d{3}\b)", "", s)
    s = re.sub(r"^[a-zA-Z]\s*=\s*", "", s)
    s = s.replace(" ", "").rstrip(".")
    if s.startswith("(") and s.endswith(")") and s.count("(") == 1:
        s = s[1:-1]
    return s


def _to_number(s: str) -> Optional[float]:
    try:
        if re.fullmatch(r"-?\(?-?\d+\)?/\(?-?\d+\)?", s):
            a, b = s.replace("(", "").replace(")", "").split("/")
            return float(Fraction(int(a), int(b)))
        return float(s)
    except Exception:
        return None


def answers_match(pred: Optional[str], truth: str) -> bool:
    if pred is None:
        return False
    p, t = normalize_answer(pred), normalize_answer(str(truth))
    if p == t:
        return True
    a, b = _to_number(p), _to_number(t)
    if a is not None and b is not None:
        return abs(a - b) <= 1e-6 * max(1.0, abs(b))
    try:
        import sympy
        from sympy.parsing.sympy_parser import parse_expr

        return bool(sympy.simplify(parse_expr(p.replace("^", "**")) - parse_expr(t.replace("^", "**"))) == 0)
    except Exception:
        return False


class MathEnvironment:
    def __init__(self, cfg: Optional[dict] = None):
        cfg = cfg or {}
        self.pool = ThreadPoolExecutor(max_workers=int(cfg.get("num_workers", 4)))
        self.stop_strings = cfg.get("stop_strings")

    @staticmethod
    def _score(args) -> tuple[float, Optional[str]]:
        response, truth = args
        pred = extract_answer(response)
        return (1.0 if answers_match(pred, truth) else 0.0), pred

    def step(self, message_log_batch, metadata) -> EnvironmentReturn:
        responses = ["".join(str(m["content"]) for m in log if m["role"] == "assistant") for log in message_log_batch]
        truths = [(md or {}).get("ground_truth", "") for md in metadata]
        results = list(self.pool.map(self._score, zip(responses, truths)))
        rewards = torch.tensor([r for r, _ in results], dtype=torch.float32)
        n = len(responses)
        obs = [{"role": "environment", "content": "Environment: " + ("correct" if r else "incorrect")} for r, _ in results]
        return EnvironmentReturn(obs, list(metadata), [None] * n, rewards, torch.ones(n, dtype=torch.bool), [p for _, p in results])

    def global_post_process_and_metrics(self, batch):
        r = batch["total_reward"].float() if "total_reward" in batch else batch["rewards"].float()
        metrics = {"accuracy": float(r.mean()) if len(r) else 0.0}
        if "generation_lengths" in batch:
            gl = batch["generation_lengths"].float()
            metrics["generation_lengths"] = float(gl.mean())
            if "truncated" in batch:
                metrics["fraction_of_samples_properly_ended"] = float(1.0 - batch["truncated"].float().mean())
        # pass@k over the generations of each prompt, when the prompt grouping is known
        if "prompt_group" in batch:
            groups = batch["prompt_group"]
            solved = {}
            for g, x in zip(groups.tolist(), r.tolist()):
                solved[g] = max(solved.get(g, 0.0), x)
            metrics["pass@samples_per_prompt"] = sum(solved.values()) / max(1, len(solved))
        return batch, metrics

    def shutdown(self):
        self.pool.shutdown(wait=False)
