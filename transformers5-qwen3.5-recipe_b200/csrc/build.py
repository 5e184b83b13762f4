"""Build libb2g.so (sm_100a) in-tree with nvcc.  Usage: python build.py [--force] [--verbose]."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCES = ["b2g_api.cu", "b2g_dequant.cu", "b2g_routing.cu", "b2g_lora.cu", "b2g_qgemm.cu", "b2g_ep.cu", "b2g_loss.cu"]
HEADERS = ["b2g_common.cuh", "b2g_formats.cuh", "../../include/b2g.h"]
LIB = HERE / "libb2g.so"
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    hdrs = [HERE / h for h in HEADERS] + [Path(__file__)]
    jobs = []
    for src in SOURCES:
        obj = objdir / (src[:-3] + ".o")
        if force or _stale(obj, [HERE / src] + hdrs):
            cmd = [nvcc, *FLAGS, "-c", str(HERE / src), "-o", str(obj)]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {cmd[-3]}")

    with ThreadPoolExecutor(max_workers=min(5, max(1, len(jobs)))) as ex:
        list(ex.map(run, jobs))
    objs = [objdir / (s[:-3] + ".o") for s in SOURCES]
    if jobs or force or _stale(LIB, objs):
        run([nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-Xcompiler", "-fvisibility=hidden"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
