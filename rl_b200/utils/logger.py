"""Metric logging fan-out: console, JSONL (always available), TensorBoard, Weights & Biases, MLflow, SwanLab, plus a
background GPU monitor (NVML) and per-step train-data dumps.

``Logger.log_metrics(metrics, step, prefix=...)`` keeps the prefixes the reference uses (``train/``, ``validation/``,
``timing/train/``, ``performance/``, ``refit/``; nemo_rl/utils/logger.py:964-1071, algorithms/grpo.py:3757-3772).
Back-ends whose package is not installed are skipped with a notice instead of failing the run.
"""

from __future__ import annotations

import glob
import json
import os
import re
import threading
import time
from typing import Any, Mapping, Optional

import torch

LOGGER_DEFAULTS = dict(
    log_dir="logs",
    wandb_enabled=False,
    tensorboard_enabled=False,
    mlflow_enabled=False,
    swanlab_enabled=False,
    monitor_gpus=False,
    num_val_samples_to_print=0,
    gpu_monitoring=dict(collection_interval=10, flush_interval=10),
)


def flatten_dict(d: Mapping[str, Any], sep: str = ".") -> dict[str, Any]:
    out: dict[str, Any] = {}
    for k, v in d.items():
        if isinstance(v, Mapping):
            for k2, v2 in flatten_dict(v, sep).items():
                out[f"{k}{sep}{k2}"] = v2
        elif isinstance(v, (list, tuple)):
            for i, x in enumerate(v):
                if isinstance(x, Mapping):
                    for k2, v2 in flatten_dict(x, sep).items():
                        out[f"{k}{sep}{i}{sep}{k2}"] = v2
                else:
                    out[f"{k}{sep}{i}"] = x
        else:
            out[k] = v
    return out


def _scalar(v: Any) -> Optional[float]:
    if isinstance(v, torch.Tensor):
        return float(v.float().mean()) if v.numel() else None
    if isinstance(v, (int, float, bool)):
        return float(v)
    try:
        import numpy as np

        if isinstance(v, (np.generic, np.ndarray)):
            return float(np.mean(v))
    except Exception:
        pass
    return None


def get_next_experiment_dir(base: str) -> str:
    """``base/exp_001``, ``exp_002``...: the next unused experiment directory."""
    os.makedirs(base, exist_ok=True)
    nums = [int(m.group(1)) for p in glob.glob(os.path.join(base, "exp_*")) if (m := re.search(r"exp_(\d+)$", p))]
    path = os.path.join(base, f"exp_{(max(nums) + 1 if nums else 1):03d}")
    os.makedirs(path, exist_ok=True)
    return path


class _Backend:
    def log(self, metrics: dict[str, float], step: int) -> None: ...
    def log_hyperparams(self, params: dict) -> None: ...
    def close(self) -> None: ...


class JsonlBackend(_Backend):
    def __init__(self, log_dir: str):
        os.makedirs(log_dir, exist_ok=True)
        self.path = os.path.join(log_dir, "metrics.jsonl")
        self._f = open(self.path, "a")

    def log(self, metrics, step):
        self._f.write(json.dumps({"step": step, **metrics}) + "\n")
        self._f.flush()

    def log_hyperparams(self, params):
        with open(os.path.join(os.path.dirname(self.path), "hparams.json"), "w") as f:
            json.dump(params, f, indent=1, default=str)

    def close(self):
        self._f.close()


class TensorboardBackend(_Backend):
    def __init__(self, log_dir: str, **kw):
        from torch.utils.tensorboard import SummaryWriter

        self.w = SummaryWriter(log_dir=os.path.join(log_dir, "tensorboard"))

    def log(self, metrics, step):
        for k, v in metrics.items():
            self.w.add_scalar(k, v, step)

    def log_hyperparams(self, params):
        self.w.add_text("hparams", json.dumps(params, default=str))

    def close(self):
        self.w.close()


class WandbBackend(_Backend):
    def __init__(self, log_dir: str, **kw):
        import wandb

        self.run = wandb.init(dir=log_dir, **kw)

    def log(self, metrics, step):
        self.run.log(metrics, step=step)

    def log_hyperparams(self, params):
        self.run.config.update(params, allow_val_change=True)

    def close(self):
        self.run.finish()


class MlflowBackend(_Backend):
    def __init__(self, log_dir: str, experiment_name: str = "rl_b200", run_name: Optional[str] = None, tracking_uri: Optional[str] = None, **kw):
        import mlflow

        self.mlflow = mlflow
        if tracking_uri:
            mlflow.set_tracking_uri(tracking_uri)
        mlflow.set_experiment(experiment_name)
        self.run = mlflow.start_run(run_name=run_name)

    def log(self, metrics, step):
        self.mlflow.log_metrics({k.replace("@", "_at_"): v for k, v in metrics.items()}, step=step)

    def log_hyperparams(self, params):
        self.mlflow.log_params({k: str(v)[:250] for k, v in flatten_dict(params).items()})

    def close(self):
        self.mlflow.end_run()


class SwanlabBackend(_Backend):
    def __init__(self, log_dir: str, **kw):
        import swanlab

        self.swanlab = swanlab
        self.run = swanlab.init(logdir=log_dir, **kw)

    def log(self, metrics, step):
        self.swanlab.log(metrics, step=step)

    def log_hyperparams(self, params):
        self.swanlab.config.update(params)

    def close(self):
        self.swanlab.finish()


class GpuMonitor:
    """Samples memory / utilisation / clocks / power of the visible GPUs through NVML on a background thread."""

    def __init__(self, logger: "Logger", collection_interval: float = 10, flush_interval: float = 10):
        self.logger, self.interval = logger, collection_interval
        self._stop = threading.Event()
        self._t: Optional[threading.Thread] = None
        self._step = 0

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
        except Exception as e:  # no NVML on this machine
            print(f"[logger] GPU monitor disabled: {e}")
            return
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def sample(self) -> dict[str, float]:
        n = self.nvml
        out = {}
        for i in range(n.nvmlDeviceGetCount()):
            h = n.nvmlDeviceGetHandleByIndex(i)
            mem = n.nvmlDeviceGetMemoryInfo(h)
            util = n.nvmlDeviceGetUtilizationRates(h)
            out[f"gpu.{i}.memory_used_gb"] = mem.used / 1e9
            out[f"gpu.{i}.util"] = float(util.gpu)
            try:
                out[f"gpu.{i}.sm_mhz"] = float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM))
                out[f"gpu.{i}.power_w"] = n.nvmlDeviceGetPowerUsage(h) / 1000.0
            except Exception:
                pass
        return out

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self.logger.log_metrics(self.sample(), self._step, prefix="ray")
                self._step += 1
            except Exception:
                pass

    def stop(self):
        self._stop.set()


class Logger:
    def __init__(self, cfg: Optional[dict] = None, is_main: bool = True):
        c = dict(LOGGER_DEFAULTS)
        c.update(cfg or {})
        self.cfg = c
        self.is_main = is_main
        self.backends: list[_Backend] = []
        self.log_dir = c["log_dir"]
        if not is_main:
            return
        os.makedirs(self.log_dir, exist_ok=True)
        self.backends.append(JsonlBackend(self.log_dir))
        for key, cls, sub in (("tensorboard_enabled", TensorboardBackend, "tensorboard"), ("wandb_enabled", WandbBackend, "wandb"),
                              ("mlflow_enabled", MlflowBackend, "mlflow"), ("swanlab_enabled", SwanlabBackend, "swanlab")):
            if c.get(key):
                try:
                    self.backends.append(cls(self.log_dir, **(c.get(sub) or {})))
                except Exception as e:
                    print(f"[logger] {sub} back-end unavailable ({type(e).__name__}: {e}); skipping")
        self.monitor: Optional[GpuMonitor] = None
        if c.get("monitor_gpus"):
            gm = c.get("gpu_monitoring") or {}
            self.monitor = GpuMonitor(self, gm.get("collection_interval", 10), gm.get("flush_interval", 10))
            self.monitor.start()

    def log_metrics(self, metrics: Mapping[str, Any], step: int, prefix: str = "", step_metric: Optional[str] = None) -> None:
        if not self.is_main:
            return
        flat = {}
        for k, v in flatten_dict(metrics).items():
            s = _scalar(v)
            if s is not None:
                flat[f"{prefix}/{k}" if prefix else k] = s
        for b in self.backends:
            try:
                b.log(flat, step)
            except Exception as e:
                print(f"[logger] {type(b).__name__} failed: {e}")

    def log_hyperparams(self, params: Mapping[str, Any]) -> None:
        if not self.is_main:
            return
        for b in self.backends:
            try:
                b.log_hyperparams(dict(params))
            except Exception as e:
                print(f"[logger] {type(b).__name__} failed: {e}")

    def log_batched_dict_as_jsonl(self, data: Mapping[str, Any], filename: str) -> None:
        """One JSON line per sample of a batch (tensors become lists), for offline inspection of train data."""
        if not self.is_main:
            return
        path = os.path.join(self.log_dir, filename)
        n = None
        for v in data.values():
            if isinstance(v, (torch.Tensor, list)):
                n = len(v)
                break
        with open(path, "w") as f:
            for i in range(n or 0):
                row = {}
                for k, v in data.items():
                    if isinstance(v, torch.Tensor):
                        row[k] = v[i].tolist()
                    elif isinstance(v, list):
                        row[k] = v[i] if isinstance(v[i], (int, float, str, list, dict, type(None))) else str(v[i])
                f.write(json.dumps(row) + "\n")

    def log_plot_token_mult_prob_error(self, data: Mapping[str, Any], step: int, name: str = "token_mult_prob_error") -> None:
        """Writes the per-token |trainer - generator| log-prob gap of the worst sample as a PNG when matplotlib exists."""
        if not self.is_main:
            return
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
        except Exception:
            return
        gen, prev, mask = data["generation_logprobs"], data["prev_logprobs"], data["token_mask"]
        err = ((gen - prev).abs() * mask).float()
        i = int(err.sum(-1).argmax())
        fig, ax = plt.subplots(figsize=(8, 3))
        ax.plot(err[i].tolist())
        ax.set_title(f"|logp_train - logp_gen| per token (sample {i}, step {step})")
        fig.savefig(os.path.join(self.log_dir, f"{name}_step{step}.png"), dpi=80)
        plt.close(fig)

    def close(self) -> None:
        if getattr(self, "monitor", None):
            self.monitor.stop()
        for b in self.backends:
            try:
                b.close()
            except Exception:
                pass


def print_message_log_samples(samples: list[str], rewards: list[float], num_samples: int = 2, step: int = 0) -> None:
    """Console preview of a few validation generations with their rewards."""
    n = min(num_samples, len(samples))
    if n == 0:
        return
    print(f"--- samples at step {step} ---")
    for i in range(n):
        print(f"[{i}] reward={rewards[i]:.4f}\n{samples[i]}\n")
