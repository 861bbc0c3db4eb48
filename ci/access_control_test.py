#!/usr/bin/env python
"""Change-driven test gate: decide from the list of changed files which test tiers have to run, then run them.

Tiers
* ``skip``  -- only prose, pictures, launch examples or profiler summaries changed: nothing runs;
* ``cpu``   -- only CPU test files changed: the device-free suite (``pytest -m "not gpu"``);
* ``build`` -- anything else: compile every CUDA extension for sm_100a, then the device-free suite,
  then -- when a GPU is visible -- the GPU suite (``pytest -m gpu``).

The changed files come from ``--files-from`` (one path per line; default ``modify.txt`` beside the
working directory when it exists) or from ``git diff --name-only <base>``.  Exit status is that of the
first failing tier.

Reference behaviour: ``ci/access_control_test.py:156-185`` (skip for docs-only changes, unit tests only
when only unit tests changed, unit then system tests otherwise).
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from typing import Iterable, List, Sequence

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROSE_SUFFIXES = (".md", ".txt", ".png", ".jpg", ".jpeg", ".svg")
PROSE_PREFIXES = ("examples/", "profiles/", "docs/", "LICENSE", "OWNERS")
GPU_TEST_FILES = ("tests/test_gpu_", "tests/multi_gpu_cases.py", "tests/test_zz_no_alloc.py")


def is_prose(path: str) -> bool:
    return path.endswith(PROSE_SUFFIXES) or path.startswith(PROSE_PREFIXES)


def is_cpu_test(path: str) -> bool:
    return path.startswith("tests/") and not path.startswith(GPU_TEST_FILES)


def choose_tier(files: Iterable[str]) -> str:
    files = [f.strip() for f in files if f.strip()]
    if not files:
        return "build"                       # no information: run everything
    if all(is_prose(f) for f in files):
        return "skip"
    if all(is_prose(f) or is_cpu_test(f) for f in files):
        return "cpu"
    return "build"


def commands_for(tier: str, gpu: bool) -> List[List[str]]:
    py = sys.executable
    cpu = [py, "-m", "pytest", "tests/", "-x", "-q", "-m", "not gpu"]
    if tier == "skip":
        return []
    if tier == "cpu":
        return [cpu]
    out = [[py, "-c", "import __graft_entry__ as g; g.build()"], cpu]
    if gpu:
        out.append([py, "-m", "pytest", "tests/", "-x", "-q", "-m", "gpu"])
    return out


def changed_files(files_from: str | None, base: str | None) -> List[str]:
    if files_from and os.path.exists(files_from):
        with open(files_from) as f:
            return [line.strip() for line in f]
    if base:
        res = subprocess.run(["git", "diff", "--name-only", base], cwd=ROOT, capture_output=True, text=True)
        if res.returncode == 0:
            return res.stdout.splitlines()
    return []


def gpu_visible() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def main(argv: Sequence[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--files-from", default=os.path.join(ROOT, "modify.txt"))
    ap.add_argument("--base", default=None, help="git revision to diff against when no file list is given")
    ap.add_argument("--dry-run", action="store_true", help="print the tier and its commands, run nothing")
    args = ap.parse_args(argv)
    tier = choose_tier(changed_files(args.files_from, args.base))
    cmds = commands_for(tier, gpu_visible() if not args.dry_run else False)
    print(f"[gate] tier: {tier}")
    for cmd in cmds:
        print("[gate] run:", " ".join(cmd))
        if args.dry_run:
            continue
        rc = subprocess.run(cmd, cwd=ROOT).returncode
        if rc != 0:
            print(f"[gate] failed with status {rc}")
            return rc
    return 0


if __name__ == "__main__":
    sys.exit(main())
