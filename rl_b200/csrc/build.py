"""Builds the native library (CUDA kernels + C++ runtime) in-tree with nvcc for sm_100a.

One shared object, ``rl_b200/_C.so``, holds every kernel and the C++ engine runtime behind a plain C ABI
that :mod:`rl_b200.ops.lib` binds with ctypes. Sources are compiled in parallel, each to an object file
under ``rl_b200/csrc/build/``, and relinked only when something changed.

    python -m rl_b200.csrc.build [--force] [--verbose]
"""

from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
BUILD = CSRC / "build"
LIB = PKG / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--use_fast_math",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return exe


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _digest(path: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(path.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _compile_one(src: Path, verbose: bool, ptxas_v: bool) -> tuple[Path, str]:
    obj = BUILD / (src.name + ".o")
    stamp = BUILD / (src.name + ".sha")
    if src.suffix == ".cu":
        flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_v else [])
        cmd = [_nvcc(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    else:
        flags = list(CXX_FLAGS)
        cmd = [shutil.which("g++") or "g++", *flags, "-I", str(CSRC), "-I", "/usr/local/cuda/include", "-c", str(src), "-o", str(obj)]
    dig = _digest(src, flags)
    if obj.exists() and stamp.exists() and stamp.read_text() == dig and not ptxas_v:
        return obj, ""
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    stamp.write_text(dig)
    return obj, (res.stdout + res.stderr) if (verbose or ptxas_v) else ""


def build_all(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> Path:
    """Compiles every source for sm_100a and links ``rl_b200/_C.so``. Returns the library path."""
    BUILD.mkdir(exist_ok=True)
    if force:
        for f in BUILD.glob("*"):
            f.unlink()
    srcs = sources()
    objs: list[Path] = []
    relink = force or not LIB.exists()
    before = {p: (BUILD / (p.name + ".o")).stat().st_mtime if (BUILD / (p.name + ".o")).exists() else None for p in srcs}
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        for obj, log in ex.map(lambda s: _compile_one(s, verbose, ptxas_v), srcs):
            objs.append(obj)
            if log:
                print(log)
    for p in srcs:
        o = BUILD / (p.name + ".o")
        if before[p] is None or o.stat().st_mtime != before[p]:
            relink = True
    if relink:
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-lcudart", "-lpthread"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    try:      # what the library was built from, so that a stale library can be told from its sources at load time
        from rl_b200.tools.fingerprint import source_hash

        Path(str(LIB) + ".sources").write_text(source_hash())
    except Exception:
        pass
    return LIB


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-v", action="store_true", help="print registers / spills / shared memory per kernel")
    a = ap.parse_args(argv)
    lib = build_all(a.force, a.verbose, a.ptxas_v)
    print(lib)
    return 0


if __name__ == "__main__":
    sys.exit(main())
