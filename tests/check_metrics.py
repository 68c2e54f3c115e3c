"""Asserts expressions over a run's logged metrics (the role of the reference's tests/check_metrics.py):

    python tests/check_metrics.py metrics.json 'max(data["train/token_mult_prob_error"]) < 1.05' 'mean(data["train/loss"], 1, 3) < 5'

``data[metric]`` is ``{step: value}``. Helpers accept such a mapping: ``min`` / ``max`` / ``mean(d, first_step=None,
last_step=None)`` / ``last(d)`` / ``ratio_above(d, bound)`` (fraction of steps above ``bound``). Every expression must be true;
the exit code is the number of expressions that are not.
"""

import json
import statistics
import sys


def _vals(d, lo=None, hi=None):
    if not isinstance(d, dict):
        return list(d)
    items = sorted(((int(k), v) for k, v in d.items()))
    return [v for k, v in items if (lo is None or k >= lo) and (hi is None or k <= hi)]


def helpers():
    import builtins

    return {
        "min": lambda d, *a: builtins.min(_vals(d, *a)) if isinstance(d, (dict, list, tuple)) else builtins.min(d, *a),
        "max": lambda d, *a: builtins.max(_vals(d, *a)) if isinstance(d, (dict, list, tuple)) else builtins.max(d, *a),
        "mean": lambda d, lo=None, hi=None: statistics.fmean(_vals(d, lo, hi)),
        "median": lambda d, lo=None, hi=None: statistics.median(_vals(d, lo, hi)),
        "last": lambda d: _vals(d)[-1],
        "first": lambda d: _vals(d)[0],
        "ratio_above": lambda d, bound: sum(1 for v in _vals(d) if v > bound) / max(1, len(_vals(d))),
        "len": lambda d: len(d),
        "abs": abs,
    }


def evaluate(data: dict, expr: str):
    return eval(expr, {"__builtins__": {}}, dict(helpers(), data=data))   # noqa: S307 (expressions come from the test scripts)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) < 2:
        print(__doc__)
        return 2
    with open(argv[0]) as f:
        data = json.load(f)
    failed = 0
    for expr in argv[1:]:
        try:
            ok = bool(evaluate(data, expr))
            note = ""
        except Exception as e:      # a missing metric is a failed check, not a crash
            ok, note = False, f"  ({type(e).__name__}: {e})"
        print(("PASS  " if ok else "FAIL  ") + expr + note)
        failed += 0 if ok else 1
    return failed


if __name__ == "__main__":
    raise SystemExit(main())
