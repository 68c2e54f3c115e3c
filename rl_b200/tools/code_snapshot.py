"""Copies the source files a run depends on into a snapshot directory and runs from there, so that editing the working tree
does not change a queued or running job (role of tools/code_snapshot.sh).

    python -m rl_b200.tools.code_snapshot --name my-experiment [--root .] [--dest code_snapshots]

Tracked files (``git ls-files``) are copied when the root is a git work tree, else every source-like file; the built native
library travels too. Prints the snapshot path; a second call with the same name re-uses the existing snapshot.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess

SOURCE_SUFFIXES = (".py", ".yaml", ".yml", ".json", ".cu", ".cuh", ".cpp", ".h", ".sub", ".md", ".toml", ".txt", ".jinja")


def list_files(root: str) -> list[str]:
    try:
        out = subprocess.run(["git", "-C", root, "ls-files"], check=True, capture_output=True, text=True).stdout.splitlines()
        files = [f for f in out if os.path.isfile(os.path.join(root, f))]
        if files:
            return files
    except (subprocess.CalledProcessError, FileNotFoundError):
        pass
    files = []
    for d, dirs, fs in os.walk(root):
        dirs[:] = [x for x in dirs if not x.startswith(".") and x not in ("code_snapshots", "__pycache__", "results", "logs", "build")]
        files += [os.path.relpath(os.path.join(d, f), root) for f in fs if f.endswith(SOURCE_SUFFIXES)]
    return files


def snapshot(name: str, root: str = ".", dest: str = "code_snapshots") -> str:
    root = os.path.abspath(root)
    target = os.path.join(root, dest, name)
    if os.path.isdir(target):
        return target
    files = list_files(root)
    lib = os.path.join("rl_b200", "_C.so")
    if os.path.exists(os.path.join(root, lib)) and lib not in files:
        files.append(lib)
    for f in files:
        if f.startswith(dest + os.sep):
            continue
        os.makedirs(os.path.dirname(os.path.join(target, f)) or target, exist_ok=True)
        shutil.copy2(os.path.join(root, f), os.path.join(target, f))
    return target


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--name", required=True)
    ap.add_argument("--root", default=".")
    ap.add_argument("--dest", default="code_snapshots")
    a = ap.parse_args(argv)
    print(snapshot(a.name, a.root, a.dest))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
