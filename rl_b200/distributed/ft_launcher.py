"""Job-level fault tolerance: run a training command under a supervisor that watches a heartbeat and restarts the job.

    python -m rl_b200.distributed.ft_launcher --max-restarts 3 --step-timeout 1800 -- \\
        torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/run_grpo.py --config ...

The training loops touch the file named by ``RLB_FT_HEARTBEAT`` after every step (``beat()``); the supervisor kills and
restarts the job when the process exits with an error, or when the heartbeat is older than ``--step-timeout`` (a hang).
Recovery is checkpoint resume: the algorithms load the latest ``step_N`` directory on start. This is the role of
``ft_launcher`` from nvidia-resiliency-ext in the reference (docs/guides/ft-launcher-guide.md, examples/ft_launcher/).
Only the process group the supervisor itself started is ever signalled.
"""

from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import tempfile
import time
from dataclasses import dataclass, field
from typing import Optional, Sequence

ENV = "RLB_FT_HEARTBEAT"


def beat(step: Optional[int] = None) -> None:
    """Called by the training loops after every step; no-op unless the job runs under the supervisor."""
    path = os.environ.get(ENV)
    if not path:
        return
    try:
        with open(path, "w") as f:
            f.write(f"{time.time()} {'' if step is None else step}\n")
    except OSError:
        pass


@dataclass
class FTResult:
    returncode: int
    restarts: int
    reasons: list = field(default_factory=list)


def run_with_restarts(cmd: Sequence[str], max_restarts: int = 3, initial_timeout_s: float = 3600.0, step_timeout_s: float = 1800.0,
                      poll_s: float = 1.0, grace_s: float = 10.0, env: Optional[dict] = None, heartbeat_path: Optional[str] = None,
                      log=print) -> FTResult:
    hb = heartbeat_path or os.path.join(tempfile.mkdtemp(prefix="rlb_ft_"), "heartbeat")
    reasons: list[str] = []
    attempt = 0
    while True:
        if os.path.exists(hb):
            os.remove(hb)
        child_env = dict(os.environ if env is None else env)
        child_env[ENV] = hb
        child_env["RLB_FT_ATTEMPT"] = str(attempt)
        proc = subprocess.Popen(list(cmd), env=child_env, start_new_session=True)   # its own process group
        started = time.time()
        reason = None
        while True:
            rc = proc.poll()
            if rc is not None:
                if rc == 0:
                    return FTResult(0, attempt, reasons)
                reason = f"exit code {rc}"
                break
            now = time.time()
            if os.path.exists(hb):
                age = now - os.path.getmtime(hb)
                if age > step_timeout_s:
                    reason = f"no heartbeat for {age:.0f} s"
            elif now - started > initial_timeout_s:
                reason = f"no first heartbeat within {initial_timeout_s:.0f} s"
            if reason:
                _stop_group(proc, grace_s)
                break
            time.sleep(poll_s)
        reasons.append(reason)
        log(f"[ft_launcher] attempt {attempt} failed: {reason}")
        if attempt >= max_restarts:
            return FTResult(proc.returncode if proc.returncode not in (None, 0) else 1, attempt, reasons)
        attempt += 1
        log(f"[ft_launcher] restarting ({attempt}/{max_restarts}); the job resumes from its latest checkpoint")


def _stop_group(proc: subprocess.Popen, grace_s: float) -> None:
    """SIGTERM, then SIGKILL, to the process group this supervisor created for the child (and to nothing else)."""
    try:
        pgid = os.getpgid(proc.pid)
    except ProcessLookupError:
        return
    for sig, wait in ((signal.SIGTERM, grace_s), (signal.SIGKILL, 5.0)):
        try:
            os.killpg(pgid, sig)
        except ProcessLookupError:
            return
        try:
            proc.wait(timeout=wait)
            return
        except subprocess.TimeoutExpired:
            continue


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--max-restarts", type=int, default=3)
    ap.add_argument("--initial-timeout", type=float, default=3600.0)
    ap.add_argument("--step-timeout", type=float, default=1800.0)
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.cmd[1:] if a.cmd and a.cmd[0] == "--" else a.cmd
    if not cmd:
        ap.error("no command given")
    res = run_with_restarts(cmd, a.max_restarts, a.initial_timeout, a.step_timeout)
    return res.returncode


if __name__ == "__main__":
    sys.exit(main())
