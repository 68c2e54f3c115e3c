"""Code environments.

``CodeEnvironment`` executes the last fenced ``python`` block of a response in a child interpreter with a time and
memory limit and scores it against unit tests (``extra_env_info = {"tests": [...asserts...]}``) or an expected stdout
(``{"expected_output": ...}``), the role of nemo_rl/environments/code_environment.py. ``CodeJaccardEnvironment`` scores
a response by token Jaccard similarity with a reference solution (no execution).
"""

from __future__ import annotations

import os
import re
import subprocess
import sys
import tempfile
from concurrent.futures import ThreadPoolExecutor
from typing import Optional

import torch

from rl_b200.environments.interfaces import EnvironmentReturn

_FENCE = re.compile(r"```(?:python|py)?\s*\n(.*?)```", re.S)


def extract_code(text: str) -> Optional[str]:
    blocks = _FENCE.findall(text)
    return blocks[-1] if blocks else None


def run_sandboxed(code: str, timeout_s: float = 5.0, memory_mb: int = 512) -> tuple[int, str, str]:
    """Runs ``code`` in ``python -I`` with resource limits. Returns (exit code, stdout, stderr)."""
    prelude = (f"import resource\nresource.setrlimit(resource.RLIMIT_AS, ({memory_mb} << 20, {memory_mb} << 20))\n"
               f"resource.setrlimit(resource.RLIMIT_CPU, ({int(timeout_s) + 1}, {int(timeout_s) + 1}))\n")
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "prog.py")
        with open(path, "w") as f:
            f.write(prelude + code)
        try:
            r = subprocess.run([sys.executable, "-I", path], capture_output=True, text=True, timeout=timeout_s, cwd=d,
                               env={"PATH": os.environ.get("PATH", "")})
            return r.returncode, r.stdout, r.stderr
        except subprocess.TimeoutExpired:
            return 124, "", "timeout"


class CodeEnvironment:
    def __init__(self, cfg: Optional[dict] = None):
        cfg = cfg or {}
        self.timeout_s = float(cfg.get("timeout_s", 5.0))
        self.memory_mb = int(cfg.get("memory_mb", 512))
        self.pool = ThreadPoolExecutor(max_workers=int(cfg.get("num_workers", 4)))

    def _score(self, args) -> tuple[float, str]:
        text, md = args
        code = extract_code(text)
        if code is None:
            return 0.0, "no code block"
        md = md or {}
        if md.get("tests"):
            prog = code + "\n\n" + "\n".join(md["tests"]) + "\nprint('__ALL_TESTS_PASSED__')\n"
            rc, out, err = run_sandboxed(prog, self.timeout_s, self.memory_mb)
            ok = rc == 0 and "__ALL_TESTS_PASSED__" in out
            return (1.0 if ok else 0.0), ("passed" if ok else (err.strip().splitlines() or ["failed"])[-1][:200])
        rc, out, err = run_sandboxed(code, self.timeout_s, self.memory_mb)
        exp = md.get("expected_output")
        ok = rc == 0 and (exp is None or out.strip() == str(exp).strip())
        return (1.0 if ok else 0.0), (out.strip()[:200] if rc == 0 else (err.strip().splitlines() or ["error"])[-1][:200])

    def step(self, message_log_batch, metadata) -> EnvironmentReturn:
        texts = ["".join(str(m["content"]) for m in log if m["role"] == "assistant") for log in message_log_batch]
        res = list(self.pool.map(self._score, zip(texts, metadata)))
        n = len(texts)
        return EnvironmentReturn([{"role": "environment", "content": f"Execution: {msg}"} for _, msg in res], list(metadata), [None] * n,
                                 torch.tensor([r for r, _ in res], dtype=torch.float32), torch.ones(n, dtype=torch.bool), [m for _, m in res])

    def global_post_process_and_metrics(self, batch):
        r = batch["total_reward"].float()
        return batch, {"pass_rate": float(r.mean()) if len(r) else 0.0}

    def shutdown(self):
        self.pool.shutdown(wait=False)


class CodeJaccardEnvironment:
    def __init__(self, cfg: Optional[dict] = None):
        pass

    @staticmethod
    def _tokens(s: str) -> set:
        return set(re.findall(r"[A-Za-z_]\w*|\d+|\S", s))

    def step(self, message_log_batch, metadata) -> EnvironmentReturn:
        n = len(message_log_batch)
        rewards = torch.zeros(n)
        for i, (log, md) in enumerate(zip(message_log_batch, metadata)):
            text = "".join(str(m["content"]) for m in log if m["role"] == "assistant")
            a, b = self._tokens(extract_code(text) or text), self._tokens((md or {}).get("ground_truth", ""))
            rewards[i] = len(a & b) / max(1, len(a | b))
        return EnvironmentReturn([{"role": "environment", "content": ""}] * n, list(metadata), [None] * n, rewards,
                                 torch.ones(n, dtype=torch.bool), [None] * n)

    def global_post_process_and_metrics(self, batch):
        return batch, {"mean_jaccard": float(batch["total_reward"].float().mean())}

    def shutdown(self):
        pass
