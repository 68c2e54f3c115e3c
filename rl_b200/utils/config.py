"""YAML configuration: ``defaults:`` inheritance, ``_override_`` replace-not-merge, ``${...}`` interpolation with
arithmetic resolvers, and Hydra-style command-line overrides.

The grammar matches what the reference accepts (nemo_rl/utils/config.py:30-204) so that its recipe files load
unchanged, but the implementation is self-contained (no OmegaConf / Hydra dependency):

* ``defaults: parent.yaml`` or a list of parents, resolved relative to the child file, merged depth-first with the
  child winning. A dict carrying ``_override_: true`` replaces the parent's dict instead of merging into it.
* ``${a.b.c}`` refers to another key of the merged tree; ``${mul:${a},2}``, ``${add:..}``, ``${div:..}``, ``${max:..}``,
  ``${min:..}``, ``${sub:..}`` evaluate arithmetic; ``${oc.env:NAME,default}`` reads the environment.
* Overrides: ``a.b=3`` sets, ``+a.b=3`` adds a new key, ``~a.b`` deletes, ``++a.b=3`` sets or adds. Values are parsed
  as YAML scalars / flow collections (``[1,2]``, ``{k: v}``, ``null``, ``true``).
"""

from __future__ import annotations

import copy
import os
import re
from pathlib import Path
from typing import Any, Callable, Iterable, Mapping

import yaml

OVERRIDE_KEY = "_override_"


class ConfigError(ValueError):
    pass


# ------------------------------------------------------------------------------------------ merge / load
def deep_merge(base: Any, new: Any) -> Any:
    """Returns ``new`` merged over ``base``: dicts merge key-wise, everything else is replaced by ``new``."""
    if isinstance(base, dict) and isinstance(new, dict):
        if new.get(OVERRIDE_KEY, False):
            out = {k: copy.deepcopy(v) for k, v in new.items() if k != OVERRIDE_KEY}
            return out
        out = dict(base)
        for k, v in new.items():
            if k == OVERRIDE_KEY:
                continue
            out[k] = deep_merge(base[k], v) if k in base else _strip_override(copy.deepcopy(v))
        return out
    return _strip_override(copy.deepcopy(new))


def _strip_override(node: Any) -> Any:
    if isinstance(node, dict):
        return {k: _strip_override(v) for k, v in node.items() if k != OVERRIDE_KEY}
    if isinstance(node, list):
        return [_strip_override(v) for v in node]
    return node


def _load_yaml(path: Path) -> dict:
    with open(path, "r") as f:
        data = yaml.safe_load(f)
    if data is None:
        return {}
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be a mapping")
    return data


def load_config_with_inheritance(path: str | os.PathLike, _seen: tuple = ()) -> dict:
    """Loads ``path`` and every file named by its ``defaults:`` key (recursively), child over parent."""
    path = Path(path).resolve()
    if path in _seen:
        raise ConfigError(f"circular defaults: {' -> '.join(map(str, _seen + (path,)))}")
    cfg = _load_yaml(path)
    parents = cfg.pop("defaults", None)
    if parents is None:
        return _strip_override(cfg)
    if isinstance(parents, (str, os.PathLike)):
        parents = [parents]
    merged: dict = {}
    for p in parents:
        ppath = Path(p)
        if not ppath.is_absolute():
            ppath = path.parent / ppath
        merged = deep_merge(merged, load_config_with_inheritance(ppath, _seen + (path,)))
    return deep_merge(merged, cfg)


# ------------------------------------------------------------------------------------------ interpolation
def _num(x: Any) -> float | int:
    if isinstance(x, bool):
        return int(x)
    if isinstance(x, (int, float)):
        return x
    s = str(x).strip()
    try:
        return int(s)
    except ValueError:
        return float(s)


def _int_if_whole(v):
    if isinstance(v, float) and v.is_integer() and abs(v) < 2**53:
        return int(v)
    return v


RESOLVERS: dict[str, Callable[..., Any]] = {
    "add": lambda *a: _int_if_whole(sum(_num(x) for x in a)),
    "sub": lambda a, b: _int_if_whole(_num(a) - _num(b)),
    "mul": lambda *a: _int_if_whole(__import__("math").prod(_num(x) for x in a)),
    "div": lambda a, b: _int_if_whole(_num(a) / _num(b)),
    "max": lambda *a: max(_num(x) for x in a),
    "min": lambda *a: min(_num(x) for x in a),
    "oc.env": lambda name, default=None: os.environ.get(str(name), default),
}


def register_resolver(name: str, fn: Callable[..., Any]) -> None:
    RESOLVERS[name] = fn


def _get_path(root: Mapping, dotted: str) -> Any:
    node: Any = root
    for part in dotted.split("."):
        if isinstance(node, list):
            node = node[int(part)]
        elif isinstance(node, Mapping) and part in node:
            node = node[part]
        else:
            raise ConfigError(f"interpolation key '{dotted}' not found")
    return node


def _split_args(s: str) -> list[str]:
    args, depth, cur = [], 0, []
    for ch in s:
        if ch == "," and depth == 0:
            args.append("".join(cur).strip())
            cur = []
            continue
        if ch in "{[":
            depth += 1
        elif ch in "}]":
            depth -= 1
        cur.append(ch)
    args.append("".join(cur).strip())
    return args


def _find_innermost(s: str):
    """Returns (start, end) of an innermost ``${...}`` span of ``s`` or None."""
    end = s.find("}")
    while end != -1:
        start = s.rfind("${", 0, end)
        if start != -1:
            return start, end + 1
        end = s.find("}", end + 1)
    return None


def _absolute_key(expr: str, here: tuple) -> str:
    """``.key`` names a sibling of the value being resolved, ``..key`` a key of the parent container, and so on."""
    if not expr.startswith("."):
        return expr
    up = len(expr) - len(expr.lstrip("."))
    base = here[: len(here) - (up - 1)] if up - 1 <= len(here) else ()
    return ".".join([*map(str, base), expr[up:]])


def _resolve_str(s: str, root: Mapping, stack: tuple, here: tuple = ()) -> Any:
    while True:
        span = _find_innermost(s)
        if span is None:
            return s
        a, b = span
        expr = s[a + 2 : b - 1].strip()
        if ":" in expr and re.match(r"^[A-Za-z_][\w.]*:", expr):
            name, argstr = expr.split(":", 1)
            if name not in RESOLVERS:
                raise ConfigError(f"unknown resolver '{name}' in '{s}'")
            args = [yaml.safe_load(x) if x != "" else "" for x in _split_args(argstr)]
            val = RESOLVERS[name](*args)
        else:
            expr = _absolute_key(expr, here)
            if expr in stack:
                raise ConfigError(f"interpolation cycle through '{expr}'")
            val = _resolve_node(_get_path(root, expr), root, stack + (expr,), tuple(expr.split(".")[:-1]))
        if a == 0 and b == len(s):
            return val
        s = s[:a] + str(val) + s[b:]


def _resolve_node(node: Any, root: Mapping, stack: tuple = (), here: tuple = ()) -> Any:
    """``here`` is the path of the container that holds ``node`` (for relative ``${.key}`` interpolation)."""
    if isinstance(node, str) and "${" in node:
        return _resolve_str(node, root, stack, here)
    if isinstance(node, dict):
        return {k: (_resolve_node(v, root, stack, here + (k,)) if isinstance(v, (dict, list)) else _resolve_node(v, root, stack, here))
                for k, v in node.items()}
    if isinstance(node, list):
        return [(_resolve_node(v, root, stack, here + (i,)) if isinstance(v, (dict, list)) else _resolve_node(v, root, stack, here))
                for i, v in enumerate(node)]
    return node


def resolve(cfg: dict) -> dict:
    """Evaluates every ``${...}`` in the tree against the tree itself."""
    return _resolve_node(cfg, cfg)


# ------------------------------------------------------------------------------------------ overrides
def _parse_value(text: str) -> Any:
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def _set_path(cfg: dict, dotted: str, value: Any, must_exist: bool | None) -> None:
    parts = dotted.split(".")
    node: Any = cfg
    for p in parts[:-1]:
        if isinstance(node, list):
            node = node[int(p)]
            continue
        if p not in node or node[p] is None:
            if must_exist:
                raise ConfigError(f"override '{dotted}': key '{p}' does not exist (use +{dotted}=... to add)")
            node[p] = {}
        node = node[p]
    last = parts[-1]
    if isinstance(node, list):
        node[int(last)] = value
        return
    exists = last in node
    if must_exist is True and not exists:
        raise ConfigError(f"override '{dotted}': key does not exist (use +{dotted}=... to add)")
    if must_exist is False and exists:
        raise ConfigError(f"override '+{dotted}': key already exists (use {dotted}=... or ++{dotted}=...)")
    node[last] = value


def _del_path(cfg: dict, dotted: str) -> None:
    parts = dotted.split(".")
    node: Any = cfg
    for p in parts[:-1]:
        node = node[int(p)] if isinstance(node, list) else node[p]
    if isinstance(node, list):
        del node[int(parts[-1])]
    else:
        if parts[-1] not in node:
            raise ConfigError(f"override '~{dotted}': key does not exist")
        del node[parts[-1]]


def apply_overrides(cfg: dict, overrides: Iterable[str]) -> dict:
    """Applies Hydra-syntax overrides (``k=v``, ``+k=v``, ``++k=v``, ``~k``) to a copy of ``cfg``."""
    out = copy.deepcopy(cfg)
    for ov in overrides:
        ov = ov.strip()
        if not ov:
            continue
        if ov.startswith("~"):
            _del_path(out, ov[1:].split("=", 1)[0])
            continue
        if "=" not in ov:
            raise ConfigError(f"cannot parse override '{ov}'")
        key, val = ov.split("=", 1)
        if key.startswith("++"):
            _set_path(out, key[2:], _parse_value(val), None)
        elif key.startswith("+"):
            _set_path(out, key[1:], _parse_value(val), False)
        else:
            _set_path(out, key, _parse_value(val), True)
    return out


def load_config(path: str | os.PathLike, overrides: Iterable[str] = (), do_resolve: bool = True) -> dict:
    """File -> inheritance -> overrides -> interpolation. Returns a plain nested dict."""
    cfg = load_config_with_inheritance(path)
    cfg = apply_overrides(cfg, overrides)
    return resolve(cfg) if do_resolve else cfg


def parse_args_and_overrides(argv: list[str] | None = None):
    """Splits ``--config file.yaml k=v ...`` into (config path or None, overrides)."""
    import argparse

    ap = argparse.ArgumentParser(add_help=True)
    ap.add_argument("--config", type=str, default=None)
    args, rest = ap.parse_known_args(argv)
    return args.config, rest


class AttrDict(dict):
    """dict with attribute access, used for config sub-trees in code paths that prefer ``cfg.a.b``."""

    def __getattr__(self, k):
        try:
            v = self[k]
        except KeyError as e:
            raise AttributeError(k) from e
        return v

    __setattr__ = dict.__setitem__

    @staticmethod
    def wrap(node: Any) -> Any:
        if isinstance(node, dict):
            return AttrDict({k: AttrDict.wrap(v) for k, v in node.items()})
        if isinstance(node, list):
            return [AttrDict.wrap(v) for v in node]
        return node
