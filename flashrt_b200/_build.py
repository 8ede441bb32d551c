"""In-tree build of the sm_100a CUDA library (``libflashrt_b200.so``) with nvcc.

The library is a plain C-ABI shared object: no torch, no pybind.  nvcc
cross-compiles for sm_100a without a GPU, so this also runs on a CPU-only box.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libflashrt_b200.so")
OBJ = os.path.join(CSRC, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    n = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(n):
        raise RuntimeError("nvcc not found; the sm_100a library cannot be built")
    return n


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_native(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``csrc/*.cu`` and link ``libflashrt_b200.so``.  Returns its path.

    ``FRT_NVCC_EXTRA`` (environment, space separated) appends compiler flags, e.g. ``-DFRT_PHASE_STAMPS`` for the
    device-timer phase stamps that ``bench.py --workload timeline`` reads through ``frt_b200_phase_stamps_read`` (use
    ``--force`` when switching it on or off: the objects do not depend on the environment)."""
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    extra = os.environ.get("FRT_NVCC_EXTRA", "").split()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "flashrt_b200.h"))
    headers = [h for h in headers if os.path.exists(h)]
    jobs = []
    objs = []
    for s in sources():
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + NVCC_FLAGS + extra + ["-I", os.path.join(os.path.dirname(HERE), "include"), "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            logs = list(ex.map(run, jobs))
        if verbose:
            print("\n".join(logs))
    if jobs or force or _stale(LIB, objs):
        run([nvcc, "-shared", "-o", LIB] + objs)
    return LIB


if __name__ == "__main__":
    import sys
    print(build_native(force="--force" in sys.argv, verbose="-v" in sys.argv))
