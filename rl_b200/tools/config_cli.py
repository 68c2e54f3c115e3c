"""Config utility: expand (resolve inheritance + interpolation), compare and minimise recipe YAMLs
(reference: tools/config_cli.py).

    python -m rl_b200.tools.config_cli expand examples/configs/grpo_math_8B.yaml [k=v ...]
    python -m rl_b200.tools.config_cli compare a.yaml b.yaml
    python -m rl_b200.tools.config_cli minimize base.yaml child.yaml     # child as a minimal diff on top of base
"""

from __future__ import annotations

import argparse
import sys
from typing import Any

import yaml

from rl_b200.utils.config import load_config

_MISSING = object()


def flatten(node: Any, prefix: str = "") -> dict[str, Any]:
    if isinstance(node, dict) and node:
        out: dict[str, Any] = {}
        for k, v in node.items():
            out.update(flatten(v, f"{prefix}.{k}" if prefix else str(k)))
        return out
    return {prefix: node}


def compare(a: dict, b: dict) -> list[tuple[str, Any, Any]]:
    fa, fb = flatten(a), flatten(b)
    return [(k, fa.get(k, _MISSING), fb.get(k, _MISSING)) for k in sorted(set(fa) | set(fb)) if fa.get(k, _MISSING) != fb.get(k, _MISSING)]


def minimize(base: Any, child: Any) -> Any:
    """The smallest tree that, deep-merged over ``base``, reproduces ``child`` (keys the child drops are not expressible)."""
    if isinstance(base, dict) and isinstance(child, dict):
        out = {}
        for k, v in child.items():
            if k not in base:
                out[k] = v
            else:
                d = minimize(base[k], v)
                if d is not _MISSING:
                    out[k] = d
        return out if out else _MISSING
    return _MISSING if base == child else child


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="config_cli")
    sub = ap.add_subparsers(dest="cmd", required=True)
    e = sub.add_parser("expand")
    e.add_argument("config")
    e.add_argument("overrides", nargs="*")
    e.add_argument("--no-resolve", action="store_true")
    c = sub.add_parser("compare")
    c.add_argument("a")
    c.add_argument("b")
    m = sub.add_parser("minimize")
    m.add_argument("base")
    m.add_argument("child")
    args = ap.parse_args(argv)
    if args.cmd == "expand":
        yaml.safe_dump(load_config(args.config, args.overrides, do_resolve=not args.no_resolve), sys.stdout, sort_keys=False)
    elif args.cmd == "compare":
        diffs = compare(load_config(args.a, do_resolve=False), load_config(args.b, do_resolve=False))
        for k, va, vb in diffs:
            fmt = lambda v: "<missing>" if v is _MISSING else repr(v)  # noqa: E731
            print(f"{k}: {fmt(va)} -> {fmt(vb)}")
        return 1 if diffs else 0
    else:
        d = minimize(load_config(args.base, do_resolve=False), load_config(args.child, do_resolve=False))
        out = {"defaults": args.base, **({} if d is _MISSING else d)}
        yaml.safe_dump(out, sys.stdout, sort_keys=False)
    return 0


if __name__ == "__main__":
    sys.exit(main())
