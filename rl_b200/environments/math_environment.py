"""Math and multiple-choice answer verification environments (single turn).

The reference scores responses with HF ``math-verify`` (or the DAPO verifier) inside Ray worker actors, has English and
multilingual multiple-choice verifiers and a multi-reward variant for GDPO (nemo_rl/environments/math_environment.py:87-555,
:555-640). Here:

* ``math_verify_impl: hf_math_verify`` uses the ``math_verify`` package when it is importable and otherwise the built-in
  grader: it extracts the last ``\\boxed{...}`` (or the text after "answer is" / the last number), canonicalises LaTeX
  fractions, roots, units, percent signs, thousands separators, mixed numbers and scientific notation, compares tuples /
  sets / intervals element-wise, numbers to relative 1e-6 and everything else symbolically through ``sympy`` (under a
  time limit) when that package is importable.
* ``math_verify_impl: dapo_math_verify``: the DAPO rule (the last ``\\boxed{}`` inside the final 300 characters, string
  equality after normalisation, reward +1 / -1 mapped to 1 / 0 here like the reference's wrapper does).
* ``verifier_type: english_multichoice | multilingual_multichoice``: ``Answer: X`` extraction.
* :class:`MathMultiRewardEnvironment`: per-sample reward components (correctness, integer answer, think/answer format).

Workers are a thread pool (verification is CPU-light); a verification that runs out of time scores 0.
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


# ------------------------------------------------------------------------------------------------ structured answers
def _split_top_level(s: str, sep: str = ",") -> list[str]:
    out, depth, cur = [], 0, []
    for ch in s:
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == sep and depth == 0:
            out.append("".join(cur))
            cur = []
        else:
            cur.append(ch)
    out.append("".join(cur))
    return [x for x in (y.strip() for y in out)]


def _mixed_number(s: str) -> str:
    m = re.fullmatch(r"(-?\d+)\s+(\d+)/(\d+)", s.strip())
    if not m:
        return s
    whole, a, b = int(m.group(1)), int(m.group(2)), int(m.group(3))
    sign = -1 if whole < 0 else 1
    return f"{whole * b + sign * a}/{b}"


def _sci(s: str) -> str:
    return re.sub(r"(\d(?:\.\d+)?)\s*(?:\\times|\\cdot|\*|x)\s*10\^\{?(-?\d+)\}?", lambda m: f"{m.group(1)}e{m.group(2)}", s)


def answers_match_structured(pred: Optional[str], truth: str) -> bool:
    """Scalars through :func:`answers_match`; tuples, intervals and sets element by element (sets regardless of order;
    interval brackets must agree)."""
    if pred is None:
        return False
    p, t = _sci(_mixed_number(pred.strip().strip("$"))), _sci(_mixed_number(str(truth).strip().strip("$")))
    p, t = p.replace("\\{", "{").replace("\\}", "}"), t.replace("\\{", "{").replace("\\}", "}")
    p, t = re.sub(r"\\(?:left|right)", "", p), re.sub(r"\\(?:left|right)", "", t)
    if answers_match(p, t):
        return True
    if len(p) >= 2 and len(t) >= 2 and p[0] in "([{" and t[0] in "([{" and p[-1] in ")]}" and t[-1] in ")]}":
        pe, te = _split_top_level(p[1:-1]), _split_top_level(t[1:-1])
        if len(pe) != len(te):
            return False
        if p[0] == "{" and t[0] == "{":
            rest = list(te)
            for x in pe:
                hit = next((y for y in rest if answers_match(x, y)), None)
                if hit is None:
                    return False
                rest.remove(hit)
            return True
        return p[0] == t[0] and p[-1] == t[-1] and all(answers_match(x, y) for x, y in zip(pe, te))
    pe, te = _split_top_level(p), _split_top_level(t)
    if len(pe) == len(te) > 1:     # an unbracketed list: "3, 5" against "3,5"
        return all(answers_match(x, y) for x, y in zip(pe, te))
    return False


def dapo_math_verify(response: str, truth: str) -> tuple[float, Optional[str]]:
    """The DAPO rule: only the last 300 characters count, the answer is the last ``\\boxed{}`` there, and it must equal the
    ground truth as a normalised string (no numeric or symbolic leniency)."""
    pred = extract_boxed(response[-300:])
    if pred is None:
        return 0.0, None

    def norm(x: str) -> str:
        x = x.split("=")[-1]
        for a in ("\\$", "$", "\\%", "%", " ", "\\!", "\\,", "\\left", "\\right", "^\\circ", "^{\\circ}", "dollars", "units"):
            x = x.replace(a, "")
        x = re.sub(r"\\text\s*\{([^{}]*)\}", r"\1", x)
        x = re.sub(r"\\[dt]frac", r"\\frac", x)
        x = re.sub(r"(?<=\d),(?=\d{3}\b)", "", x)
        return x.rstrip(".").strip()

    return (1.0 if norm(pred) == norm(str(truth)) else 0.0), pred


_HF_VERIFY = None


def _hf_math_verify():
    """``(parse, verify, gold config, prediction config)`` of the ``math_verify`` package set up like the reference's worker
    (gold: LaTeX; prediction: expression or LaTeX), or False when the package is not installed. Its own time limits use
    signals, which only work on a process's main thread; they are switched off and the caller's limit applies instead."""
    global _HF_VERIFY
    if _HF_VERIFY is None:
        try:
            import logging

            from math_verify import parse, verify
            from math_verify.parser import ExprExtractionConfig, LatexExtractionConfig

            for name in ("math_verify", "math_verify.parser", "math_verify.grader", "math_verify.utils"):
                logging.getLogger(name).setLevel(logging.CRITICAL)
            _HF_VERIFY = (parse, verify, (LatexExtractionConfig(),), (ExprExtractionConfig(), LatexExtractionConfig()))
        except Exception:
            _HF_VERIFY = False
    return _HF_VERIFY


# multiple choice ("Answer: X"), English and other scripts (role of nemo_rl/evals/answer_parsing.py)
_ANSWER_WORDS = ["Answer", "Respuesta", "Réponse", "Antwort", "Risposta", "Resposta", "Ответ", "答案", "答え", "回答", "정답", "답",
                 "الإجابة", "উত্তর", "उत्तर", "Jawaban", "Jibu", "Ìdáhùn", "Cevap"]
_LETTER_MAP = {"أ": "A", "ب": "B", "ج": "C", "د": "D", "অ": "A", "ব": "B", "ড": "C", "ঢ": "D", "Ａ": "A", "Ｂ": "B", "Ｃ": "C", "Ｄ": "D"}


def _normalize_mc_response(text: str) -> str:
    for a in ("**", "$\\boxed{", "}$", "\\$", "$\\text{", "$", "\\mathrm{", "\\{", "\\text", "\\(", "\\mathbf{", "{", "\\boxed"):
        text = text.replace(a, "")
    return text


def extract_multichoice(response: str, multilingual: bool = False) -> Optional[str]:
    text = _normalize_mc_response(response)
    words = _ANSWER_WORDS if multilingual else ["Answer"]
    letters = "A-Z" + "".join(_LETTER_MAP)
    for w in words:
        m = re.search(rf"(?i){re.escape(w)}\s*[:：][ \t]*\(?([{letters}])", text)
        if m:
            c = m.group(1)
            return _LETTER_MAP.get(c, c).upper().strip()
    return None


def _with_time_limit(fn, seconds: float, default):
    """Runs ``fn()`` on a helper thread and gives up after ``seconds`` (a runaway symbolic simplification scores 0)."""
    import threading

    box = [default]

    def run():
        try:
            box[0] = fn()
        except Exception:
            box[0] = default

    t = threading.Thread(target=run, daemon=True)
    t.start()
    t.join(seconds)
    return box[0] if not t.is_alive() else default


class MathEnvironment:
    def __init__(self, cfg: Optional[dict] = None):
        cfg = cfg or {}
        self.cfg = cfg
        self.pool = ThreadPoolExecutor(max_workers=int(cfg.get("num_workers", 4)))
        self.stop_strings = cfg.get("stop_strings")
        self.verifier_type = cfg.get("verifier_type") or "math"
        self.impl = cfg.get("math_verify_impl") or "hf_math_verify"
        self.time_limit_s = float(cfg.get("verify_timeout_s", 5.0))
        if self.verifier_type not in ("math", "english_multichoice", "multilingual_multichoice"):
            raise ValueError(f"unknown verifier_type '{self.verifier_type}'")
        if self.impl not in ("hf_math_verify", "dapo_math_verify"):
            raise ValueError(f"unknown math_verify_impl '{self.impl}' (hf_math_verify | dapo_math_verify)")

    def _score(self, args) -> tuple[float, Optional[str]]:
        response, truth = args
        if self.verifier_type != "math":
            pred = extract_multichoice(response, multilingual=self.verifier_type == "multilingual_multichoice")
            want = _normalize_mc_response(str(truth)).strip().upper() if self.verifier_type == "english_multichoice" else str(truth)
            return (1.0 if pred is not None and pred == want else 0.0), pred
        if self.impl == "dapo_math_verify":
            return dapo_math_verify(response, truth)
        hf = _hf_math_verify()
        if hf:
            parse, verify, gold_cfg, pred_cfg = hf

            def run():
                gold = parse("\\boxed{" + str(truth) + "}", extraction_config=gold_cfg, parsing_timeout=None)
                pred = parse(response, extraction_config=pred_cfg, parsing_timeout=None)
                shown = str(pred[-1]) if pred else None
                return (1.0 if (gold and pred and verify(gold, pred, timeout_seconds=None)) else 0.0), shown

            return _with_time_limit(run, self.time_limit_s, (0.0, None))
        pred = extract_answer(response)
        ok = _with_time_limit(lambda: answers_match_structured(pred, truth), self.time_limit_s, False)
        return (1.0 if ok else 0.0), pred

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


class MathMultiRewardEnvironment(MathEnvironment):
    """Several reward components per sample, for estimators that normalise them separately (GDPO): whether the answer inside
    ``<answer>...</answer>`` equals the ground truth, whether it is an integer, and whether the response has the
    ``<think>...</think>\\n<answer>...</answer>`` shape (nemo_rl/environments/math_environment.py:260-367, :555-640).
    ``rewards`` is ``[B, 3]`` in the order of :attr:`REWARD_NAMES`."""

    REWARD_NAMES = ["reward/correctness", "reward/integer", "reward/format"]
    _FORMAT = re.compile(r"^<think>.*?</think>\n<answer>.*?</answer>$", re.DOTALL)

    @staticmethod
    def _xml_answer(text: str) -> str:
        return text.split("<answer>")[-1].split("</answer>")[0].strip()

    def _components(self, args) -> tuple[list[float], Optional[str]]:
        response, truth = args
        ans = self._xml_answer(response)
        fmt = bool(self._FORMAT.search(response)) and response.count("<answer>") == 1 and response.count("</answer>") == 1
        return [1.0 if ans == str(truth) else 0.0, 1.0 if ans.isdigit() else 0.0, 1.0 if fmt else 0.0], ans

    def step(self, message_log_batch, metadata) -> EnvironmentReturn:
        responses = ["".join(str(m["content"]) for m in log if m["role"] == "assistant") for log in message_log_batch]
        truths = [(md or {}).get("ground_truth", "") for md in metadata]
        results = list(self.pool.map(self._components, zip(responses, truths)))
        rewards = torch.tensor([r for r, _ in results], dtype=torch.float32).reshape(len(responses), len(self.REWARD_NAMES))
        n = len(responses)
        obs = [{"role": "environment", "content": "Environment: " + ("correct" if r[0] else "incorrect")} for r, _ in results]
        return EnvironmentReturn(obs, list(metadata), [None] * n, rewards, torch.ones(n, dtype=torch.bool), [a for _, a in results])
