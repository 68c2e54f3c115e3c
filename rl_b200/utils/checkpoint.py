"""Checkpoint directory manager: atomic step directories, top-k retention by a metric, resume lookup.

Layout kept from the reference (nemo_rl/utils/checkpoint.py:142-619):

    <checkpoint_dir>/step_<N>/{training_info.json, config.yaml, train_dataloader.pt, policy/{weights, optimizer, tokenizer}}

A save writes into ``tmp_step_<N>`` and renames to ``step_<N>`` once everything is on disk, so a killed job never
leaves a half-written ``step_*`` directory. Retention keeps the best ``keep_top_k`` by ``metric_name`` (always
including the latest), or, with ``ft_keep_latest_k``, additionally the most recent k for fault-tolerant restarts.
"""

from __future__ import annotations

import json
import os
import re
import shutil
import threading
from pathlib import Path
from typing import Any, Callable, Optional

import yaml

CHECKPOINTING_DEFAULTS = dict(
    enabled=False,
    checkpoint_dir="results/checkpoints",
    metric_name=None,
    higher_is_better=True,
    keep_top_k=None,
    save_period=10,
    checkpoint_must_save_by=None,
    model_save_format="safetensors",
    save_consolidated=False,
    save_optimizer=True,
    ft_save_period=None,
    ft_keep_latest_k=None,
)

_STEP_RE = re.compile(r"^step_(\d+)$")


def _jsonable(x: Any) -> Any:
    try:
        import numpy as np
        import torch

        if isinstance(x, torch.Tensor):
            return x.item() if x.numel() == 1 else x.tolist()
        if isinstance(x, np.generic):
            return x.item()
        if isinstance(x, np.ndarray):
            return x.tolist()
    except Exception:
        pass
    if isinstance(x, dict):
        return {k: _jsonable(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_jsonable(v) for v in x]
    return x


class CheckpointManager:
    def __init__(self, cfg: Optional[dict] = None):
        c = dict(CHECKPOINTING_DEFAULTS)
        c.update(cfg or {})
        self.cfg = c
        self.dir = Path(c["checkpoint_dir"])
        self.enabled = bool(c["enabled"])
        self._finalizer: Optional[threading.Thread] = None
        if self.enabled:
            self.dir.mkdir(parents=True, exist_ok=True)

    # context-manager form: `with checkpointer: train(...)` waits for a background finalisation on exit
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.wait()
        return False

    # ------------------------------------------------------------------ save
    def init_tmp_checkpoint(self, step: int, training_info: dict, run_config: Optional[dict] = None) -> Path:
        """Creates ``tmp_step_<N>`` with ``training_info.json`` (+ ``config.yaml``) and returns its path."""
        self.wait()
        tmp = self.dir / f"tmp_step_{step}"
        if tmp.exists():
            shutil.rmtree(tmp)
        tmp.mkdir(parents=True)
        with open(tmp / "training_info.json", "w") as f:
            json.dump(_jsonable(training_info), f, indent=2)
        if run_config is not None:
            with open(tmp / "config.yaml", "w") as f:
                yaml.safe_dump(_jsonable(run_config), f)
        return tmp

    def finalize_checkpoint(self, tmp_path: os.PathLike) -> Path:
        """Atomically renames ``tmp_step_<N>`` to ``step_<N>`` and applies retention."""
        tmp = Path(tmp_path)
        final = tmp.parent / tmp.name[len("tmp_") :]
        if final.exists():
            shutil.rmtree(final)
        os.replace(tmp, final)
        self.remove_old_checkpoints()
        return final

    def begin_finalization(self, tmp_path: os.PathLike, wait_for: Optional[Callable[[], None]] = None) -> None:
        """Finalises in a background thread, after ``wait_for()`` (e.g. asynchronous tensor writes) returns."""

        def run():
            if wait_for is not None:
                wait_for()
            self.finalize_checkpoint(tmp_path)

        self.wait()
        self._finalizer = threading.Thread(target=run, daemon=True)
        self._finalizer.start()

    def wait(self) -> None:
        if self._finalizer is not None:
            self._finalizer.join()
            self._finalizer = None

    # ------------------------------------------------------------------ retention
    def _steps(self) -> list[tuple[int, Path]]:
        if not self.dir.exists():
            return []
        out = []
        for p in self.dir.iterdir():
            m = _STEP_RE.match(p.name)
            if m and p.is_dir():
                out.append((int(m.group(1)), p))
        return sorted(out)

    def _metric_of(self, path: Path) -> Optional[float]:
        name = self.cfg["metric_name"]
        if not name:
            return None
        try:
            info = json.load(open(path / "training_info.json"))
        except Exception:
            return None
        # "val:accuracy" style keys address nested dicts; plain keys address the top level
        if ":" in name:
            prefix, key = name.split(":", 1)
            for cand in (info.get(prefix), info.get(f"{prefix}_metrics"), info):
                if isinstance(cand, dict) and key in cand:
                    return float(cand[key])
            flat = f"{prefix}_{key}"
            return float(info[flat]) if flat in info else (float(info[name]) if name in info else None)
        return float(info[name]) if name in info else None

    def remove_old_checkpoints(self, exclude_latest: bool = True) -> None:
        k = self.cfg["keep_top_k"]
        if k is None:
            return
        steps = self._steps()
        if len(steps) <= k:
            return
        latest = steps[-1][0]
        keep: set[int] = set()
        ftk = self.cfg.get("ft_keep_latest_k")
        if ftk:
            keep.update(s for s, _ in steps[-int(ftk):])
        scored = [(self._metric_of(p), s) for s, p in steps]
        if self.cfg["metric_name"] and all(m is not None for m, _ in scored):
            hib = self.cfg["higher_is_better"]
            # best metric first; ties resolved toward the more recent step
            ranked = sorted(scored, key=lambda t: ((-t[0]) if hib else t[0], -t[1]))
        else:
            ranked = sorted(scored, key=lambda t: -t[1])
        keep.update(s for _, s in ranked[:k])
        if exclude_latest:
            keep.add(latest)
        for s, p in steps:
            if s not in keep:
                shutil.rmtree(p, ignore_errors=True)

    # ------------------------------------------------------------------ resume
    def get_latest_checkpoint_path(self) -> Optional[str]:
        steps = self._steps()
        return str(steps[-1][1]) if steps else None

    def get_best_checkpoint_path(self) -> Optional[str]:
        steps = self._steps()
        if not steps:
            return None
        scored = [(self._metric_of(p), s, p) for s, p in steps]
        if not self.cfg["metric_name"] or any(m is None for m, _, _ in scored):
            return str(steps[-1][1])
        hib = self.cfg["higher_is_better"]
        return str(sorted(scored, key=lambda t: ((-t[0]) if hib else t[0], -t[1]))[0][2])

    def load_training_info(self, path: Optional[str] = None) -> Optional[dict]:
        path = path or self.get_latest_checkpoint_path()
        if path is None:
            return None
        with open(Path(path) / "training_info.json") as f:
            return json.load(f)

    def get_resume_paths(self, path: Optional[str] = None) -> Optional[dict[str, Optional[str]]]:
        """Paths of the pieces of a checkpoint (None for pieces that were not saved)."""
        path = path or self.get_latest_checkpoint_path()
        if path is None:
            return None
        p = Path(path)
        def ex(q):
            return str(q) if q.exists() else None
        return {
            "root": str(p),
            "weights": ex(p / "policy" / "weights"),
            "optimizer": ex(p / "policy" / "optimizer"),
            "tokenizer": ex(p / "policy" / "tokenizer"),
            "dataloader": ex(p / "train_dataloader.pt"),
            "value_weights": ex(p / "value" / "weights"),
            "value_optimizer": ex(p / "value" / "optimizer"),
            "replay_buffer": ex(p / "replay_buffer.pt"),
        }
