"""Environment fingerprint: what has to match between the machine that produced a number and the one that reproduces it
(package versions, CUDA / driver, GPU model, the hash of the native library's sources). The reference checks a
container fingerprint at import (nemo_rl/__init__.py:98-229); this tool prints and compares one.

    python -m rl_b200.tools.fingerprint [--compare other.json]
"""

from __future__ import annotations

import argparse
import glob
import hashlib
import json
import os
import platform
import sys


def source_hash() -> str:
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
    h = hashlib.sha256()
    for p in sorted(glob.glob(os.path.join(root, "*.cu")) + glob.glob(os.path.join(root, "*.cuh")) + glob.glob(os.path.join(root, "*.cpp")) + glob.glob(os.path.join(root, "*.h"))):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def fingerprint() -> dict:
    import torch

    out = dict(python=platform.python_version(), torch=torch.__version__, cuda=torch.version.cuda, native_sources=source_hash())
    for mod in ("numpy", "transformers", "safetensors"):
        try:
            out[mod] = __import__(mod).__version__
        except Exception:
            out[mod] = None
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        out.update(gpu=p.name, sm=f"{p.major}{p.minor}", sms=p.multi_processor_count, gpu_mem_gib=round(p.total_memory / 2**30, 1),
                   nccl=".".join(map(str, torch.cuda.nccl.version())))
    return out


def compare(a: dict, b: dict) -> dict:
    return {k: (a.get(k), b.get(k)) for k in sorted(set(a) | set(b)) if a.get(k) != b.get(k)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--compare")
    a = ap.parse_args(argv)
    fp = fingerprint()
    if a.compare:
        diff = compare(fp, json.load(open(a.compare)))
        print(json.dumps({"differences": diff}, indent=1))
        return 1 if diff else 0
    print(json.dumps(fp, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
