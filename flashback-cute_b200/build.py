"""Build libflashback_b200.so in-tree with nvcc for sm_100a.

    python flashback-cute_b200/build.py [--force] [--verbose]

Sources: csrc/*.cu. Output: flashback_cute/libflashback_b200.so (next to the Python host
code that loads it with ctypes). Object files go to build/ (git-ignored). The CUDA runtime is
linked statically and the driver API is resolved at run time, so the library loads on a
machine without a GPU driver (compute entry points then return an error status).
"""

from __future__ import annotations

import argparse
import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "flashback_cute" / "libflashback_b200.so"
OBJ = HERE / "build"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-DFB_BUILDING_LIBRARY",
]


def _newer(a: Path, deps) -> bool:
    return a.exists() and all(a.stat().st_mtime >= d.stat().st_mtime for d in deps)


def build(force: bool = False, verbose: bool = False, profile: bool = False, defines=()) -> Path:
    """profile=True builds the variant with the kernels' cycle / timeline instrumentation compiled in
    (-DFB_PROFILE) as libflashback_b200_prof.so; select it at run time with FLASHBACK_LIB=<path>."""
    global OBJ, OUT
    flags = list(FLAGS) + [f"-D{d}" for d in defines]
    if defines:  # an experimental variant: its own objects and library name
        tag = "_".join(d.replace("=", "") for d in defines).lower()
        OBJ, OUT = HERE / f"build_{tag}", HERE / "flashback_cute" / f"libflashback_b200_{tag}.so"
    if profile:
        OBJ, OUT = HERE / "build_prof", HERE / "flashback_cute" / "libflashback_b200_prof.so"
        flags.append("-DFB_PROFILE")
    srcs = sorted(CSRC.glob("*.cu"))
    hdrs = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted((HERE.parent / "include").glob("*.h"))
    OBJ.mkdir(exist_ok=True)
    jobs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if force or not _newer(o, [s, *hdrs]):
            cmd = [NVCC, *flags, "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            for cmd, res in zip(jobs, ex.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs)):
                if verbose or res.returncode:
                    sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
                if res.returncode:
                    raise RuntimeError(f"nvcc failed: {' '.join(cmd)}")
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if force or jobs or not _newer(OUT, objs):
        cmd = [NVCC, "-shared", "-o", str(OUT), *map(str, objs), "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--profile", action="store_true", help="build the instrumented variant (libflashback_b200_prof.so)")
    ap.add_argument("-D", dest="defines", action="append", default=[], help="extra macro for an experimental variant, e.g. -D FB_EXP2_POLY=4")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.profile, a.defines))
