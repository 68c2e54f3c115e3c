"""Refit time model: how long moving a model's weights from the training layout to the serving layout takes, given
bytes per rank and link bandwidth (reference: tools/refit_bandwidth_calculator.py:26-43).

On one NVSwitch node every GPU reaches every peer at full NVLink bandwidth, so a reshard's time is bounded by the
largest per-GPU send or receive volume over the per-direction bandwidth, plus a launch/synchronisation floor:

    t = max_r(max(bytes_out[r], bytes_in[r])) / bw_per_direction + latency

Colocated same-layout refit moves zero bytes (the engine reads the trainer's buffers).

    python -m rl_b200.tools.refit_bandwidth_calculator --params 8.03e9 --train dp8 --serve tp8
"""

from __future__ import annotations

import argparse
import re

NVLINK_MEASURED_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU on a B200 NVSwitch node
NVLINK_NOMINAL_GBS = 900.0


def parse_layout(s: str) -> dict[str, int]:
    out = {"dp": 1, "tp": 1, "pp": 1, "ep": 1}
    for name, n in re.findall(r"([a-z]+)(\d+)", s.lower()):
        out[name] = int(n)
    return out


def bytes_held(total_bytes: float, layout: dict[str, int], expert_fraction: float = 0.0) -> float:
    """Bytes of weights one rank holds: dense part split by tp*pp, expert part also by ep."""
    dense = total_bytes * (1 - expert_fraction) / (layout["tp"] * layout["pp"])
    experts = total_bytes * expert_fraction / (layout["tp"] * layout["pp"] * layout["ep"])
    return dense + experts


def refit_seconds(total_bytes: float, train: dict[str, int], serve: dict[str, int], world: int, bw_gbs: float = NVLINK_MEASURED_GBS,
                  latency_s: float = 50e-6, expert_fraction: float = 0.0, colocated_same_layout_free: bool = True) -> dict:
    """Every serving rank must receive the bytes it holds under ``serve`` that it does not already hold under ``train``.
    With ZeRO-style training replicas (full parameters resident on every dp rank) a serving shard is always a local
    slice: zero bytes cross the link."""
    hold_t = bytes_held(total_bytes, train, expert_fraction)
    hold_s = bytes_held(total_bytes, serve, expert_fraction)
    if colocated_same_layout_free and all(train[k] == serve[k] for k in ("tp", "pp", "ep")):
        recv = 0.0
    elif train["tp"] * train["pp"] * train["ep"] == 1:
        recv = 0.0  # trainer holds everything locally
    else:
        overlap = min(hold_t, hold_s)  # shard boundaries nest when both sizes are powers of two and ranks are aligned
        recv = max(0.0, hold_s - overlap)
    t = recv / (bw_gbs * 1e9) + (latency_s if recv else 0.0)
    return {"bytes_per_rank_train": hold_t, "bytes_per_rank_serve": hold_s, "recv_bytes_per_rank": recv, "seconds": t,
            "effective_gbs": (recv / t / 1e9) if t else float("inf")}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=float, required=True, help="parameter count")
    ap.add_argument("--bytes-per-param", type=float, default=2.0)
    ap.add_argument("--train", default="dp8")
    ap.add_argument("--serve", default="tp8")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--bw-gbs", type=float, default=NVLINK_MEASURED_GBS)
    ap.add_argument("--expert-fraction", type=float, default=0.0)
    a = ap.parse_args(argv)
    r = refit_seconds(a.params * a.bytes_per_param, parse_layout(a.train), parse_layout(a.serve), a.world, a.bw_gbs,
                      expert_fraction=a.expert_fraction)
    print(f"train {a.train}: {r['bytes_per_rank_train'] / 1e9:.2f} GB/rank; serve {a.serve}: {r['bytes_per_rank_serve'] / 1e9:.2f} GB/rank")
    print(f"receive {r['recv_bytes_per_rank'] / 1e9:.2f} GB/rank -> {r['seconds'] * 1e3:.2f} ms at {a.bw_gbs:.0f} GB/s per direction")


if __name__ == "__main__":
    main()
