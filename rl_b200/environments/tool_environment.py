"""Multi-turn tool-use environment: the policy calls tools by writing ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``,
the environment runs the tool and answers with a ``<tool_response>`` observation; the episode ends when the policy gives a final
answer (no tool call), which is scored against the ground truth. Built-in tools: ``calculator`` (safe arithmetic) and
``retrieve`` (keyword retrieval over a small document list from the config or the sample's metadata), the role of the
reference's retriever / tool environments (nemo_rl/environments/tools/retriever.py).
"""

from __future__ import annotations

import ast
import json
import operator
import re
from typing import Any, Callable, Optional

import torch

from .interfaces import EnvironmentReturn

_CALL = re.compile(r"<tool_call>(.*?)</tool_call>", re.S)
_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv, ast.FloorDiv: operator.floordiv,
        ast.Mod: operator.mod, ast.Pow: operator.pow, ast.USub: operator.neg, ast.UAdd: operator.pos}


def safe_eval(expr: str) -> float:
    """Arithmetic on numbers only (no names, calls or attribute access); exponents are bounded."""
    def ev(n):
        if isinstance(n, ast.Constant) and isinstance(n.value, (int, float)):
            return n.value
        if isinstance(n, ast.BinOp) and type(n.op) in _OPS:
            a, b = ev(n.left), ev(n.right)
            if isinstance(n.op, ast.Pow) and (abs(b) > 64 or abs(a) > 1e6):
                raise ValueError("exponent out of range")
            return _OPS[type(n.op)](a, b)
        if isinstance(n, ast.UnaryOp) and type(n.op) in _OPS:
            return _OPS[type(n.op)](ev(n.operand))
        raise ValueError("unsupported expression")
    return ev(ast.parse(expr.strip(), mode="eval").body)


def keyword_retrieve(query: str, docs: list[str], k: int = 1) -> list[str]:
    q = set(re.findall(r"\w+", query.lower()))
    scored = sorted(((len(q & set(re.findall(r"\w+", d.lower()))), -i, d) for i, d in enumerate(docs)), reverse=True)
    return [d for s, _, d in scored[:k] if s > 0]


class ToolEnvironment:
    def __init__(self, cfg: Optional[dict] = None, tools: Optional[dict[str, Callable[..., Any]]] = None):
        c = dict(max_tool_calls=4, documents=[], tool_call_penalty=0.0, answer_pattern=r"\\boxed\{([^}]*)\}")
        c.update(cfg or {})
        self.cfg = c
        self.tools: dict[str, Callable[..., Any]] = {"calculator": lambda expression: safe_eval(str(expression))}
        self.tools.update(tools or {})

    def _run(self, call_text: str, meta: dict) -> str:
        try:
            call = json.loads(call_text)
            name, args = call["name"], call.get("arguments") or {}
            if name == "retrieve":
                docs = (meta or {}).get("documents") or self.cfg["documents"]
                return json.dumps({"documents": keyword_retrieve(str(args.get("query", "")), docs, int(args.get("k", 1)))})
            if name not in self.tools:
                return json.dumps({"error": f"unknown tool {name!r}"})
            return json.dumps({"result": self.tools[name](**args)})
        except Exception as e:   # a malformed call is the policy's mistake: it gets the error text back, not an exception
            return json.dumps({"error": f"{type(e).__name__}: {e}"})

    def step(self, message_log_batch, metadata) -> EnvironmentReturn:
        obs, metas, rewards, term, answers = [], [], [], [], []
        for log, meta in zip(message_log_batch, metadata):
            meta = dict(meta or {})
            resp = next((m["content"] for m in reversed(log) if m["role"] == "assistant"), "")
            calls = _CALL.findall(resp)
            used = int(meta.get("tool_calls", 0))
            if calls and used < int(self.cfg["max_tool_calls"]):
                meta["tool_calls"] = used + 1
                out = self._run(calls[0], meta)
                obs.append({"role": "environment", "content": f"<tool_response>{out}</tool_response>"})
                rewards.append(-float(self.cfg["tool_call_penalty"]))
                term.append(False)
                answers.append(None)
            else:
                m = re.search(self.cfg["answer_pattern"], resp, flags=re.S)
                ans = (m.group(1) if m else resp).strip()
                gt = str(meta.get("ground_truth", "")).strip()
                ok = False
                if gt:
                    try:
                        ok = abs(float(ans) - float(gt)) < 1e-6
                    except ValueError:
                        ok = ans.lower() == gt.lower()
                obs.append({"role": "environment", "content": ""})
                rewards.append(float(ok))
                term.append(True)
                answers.append(ans)
            metas.append(meta)
        n = len(message_log_batch)
        return EnvironmentReturn(obs, metas, [None] * n, torch.tensor(rewards, dtype=torch.float32), torch.tensor(term, dtype=torch.bool), answers)

    def global_post_process_and_metrics(self, batch):
        r = batch["total_reward"] if "total_reward" in batch else batch["rewards"]
        return batch, {"accuracy": float((r >= 1.0).float().mean()) if len(r) else 0.0}

    def shutdown(self) -> None:
        pass
