"""Lists the runs of TCP ports on this host that nothing listens on (to choose ``port_range_low`` / ``port_range_high`` for
rendezvous and serving ports; role of tools/find_available_port_ranges.py).

    python -m rl_b200.tools.find_available_port_ranges [--low 1024] [--high 65535] [--min-size 16]
"""

from __future__ import annotations

import argparse
import socket


def is_free(port: int, host: str = "127.0.0.1") -> bool:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.settimeout(0.05)
        return s.connect_ex((host, port)) != 0


def free_ranges(low: int = 1024, high: int = 65535, host: str = "127.0.0.1", probe=is_free) -> list[tuple[int, int]]:
    """Inclusive (first, last) runs of free ports, in order."""
    out, start = [], None
    for p in range(low, high + 1):
        if probe(p, host):
            start = p if start is None else start
        elif start is not None:
            out.append((start, p - 1))
            start = None
    if start is not None:
        out.append((start, high))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--low", type=int, default=1024)
    ap.add_argument("--high", type=int, default=65535)
    ap.add_argument("--min-size", type=int, default=1)
    a = ap.parse_args(argv)
    print("size\trange")
    for lo, hi in free_ranges(a.low, a.high):
        if hi - lo + 1 >= a.min_size:
            print(f"{hi - lo + 1}\t{lo}" + (f"-{hi}" if hi > lo else ""))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
