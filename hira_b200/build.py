"""Builds libhira_b200.so (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

Run as ``python -m hira_b200.build`` or call :func:`build_library`.  The library
is written next to this file so that it travels with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libhira_b200.so"
PROFILE_LIB_PATH = PKG_DIR / "libhira_b200_profile.so"   # the same library with phase time stamps in search_q8.cu
OBJ_DIR = CSRC / "build"

SOURCES = ["api.cu", "search.cu", "search_q8.cu", "attention.cu", "append.cu", "threshold.cu", "build.cu", "assign_tc.cu", "exchange.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr", "--extended-lambda",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or install the CUDA toolkit)")


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    headers = [CSRC / "common.cuh", CSRC / "search_common.cuh", CSRC / "tc_common.cuh", CSRC / "merge_row.cuh", PKG_DIR.parent / "include" / "hira_b200.h"]
    sources = list(SOURCES)
    jobs = []
    for src in sources:
        obj = OBJ_DIR / (src + ".o")
        if force or _stale(obj, [CSRC / src, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(run, jobs):
            if verbose or ptxas_info or r.returncode != 0:
                sys.stderr.write(f"[nvcc {src}]\n{r.stdout}{r.stderr}\n")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
    objs = [str(OBJ_DIR / (s + ".o")) for s in sources]
    if force or jobs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("linking libhira_b200.so failed")
    return LIB_PATH


def build_profile_library() -> Path:
    """A second library whose int8 pre-filter search kernel writes globaltimer stamps at its phase
    boundaries (-DHIRA_Q8_PROFILE); read back by `python bench.py --phase-profile`.  Never loaded by
    the package itself."""
    nvcc = _nvcc()
    build_library()
    obj = OBJ_DIR / "search_q8.profile.o"
    r = subprocess.run([nvcc, *NVCC_FLAGS, "-DHIRA_Q8_PROFILE", "-c", str(CSRC / "search_q8.cu"), "-o", str(obj)],
                       capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("nvcc failed on search_q8.cu (profile build)")
    objs = [str(OBJ_DIR / (s + ".o")) for s in SOURCES if s != "search_q8.cu"] + [str(obj)]
    r = subprocess.run([nvcc, "-shared", "-o", str(PROFILE_LIB_PATH), *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("linking the profile library failed")
    return PROFILE_LIB_PATH


if __name__ == "__main__":
    if "--profile" in sys.argv:
        print(build_profile_library())
    else:
        p = build_library(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
        print(p)
