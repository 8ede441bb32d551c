"""Generates ``sf_layout.npz``: NVFP4 scale-factor byte offsets taken from CUTLASS's own layout object
(``Sm1xxBlockScaledConfig<16>::tile_atom_to_shape_SFA / _SFB``), the layout the reference writes.

Needs nvcc and a CUTLASS header tree (any site-packages copy will do); run it where those exist:
    python tests/golden/make_sf_layout_golden.py
The fixture pins the closed-form offset used by the oracle and the kernels.
"""
import glob
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [(130, 192, 0), (50, 1024, 0), (300, 2048, 1), (129, 80, 0), (257, 4096, 1), (10, 1024, 0)]


def cutlass_include() -> str:
    for pat in ("flashinfer/data/cutlass/include", "tilelang/3rdparty/cutlass/include"):
        for sp in sys.path:
            hit = glob.glob(os.path.join(sp, pat))
            if hit:
                return hit[0]
    raise RuntimeError("no CUTLASS header tree found")


def main():
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "sf_layout_table")
        subprocess.check_call(["nvcc", "-std=c++17", "-w", "-I", cutlass_include(), "-o", exe,
                               os.path.join(HERE, "sf_layout_table.cu")])
        out = {}
        for rows, K, is_b in CASES:
            txt = subprocess.run([exe, str(rows), str(K), str(is_b)], capture_output=True, text=True, check=True).stdout
            vals = np.array(txt.split(), dtype=np.int64)
            out[f"size_{rows}_{K}_{is_b}"] = vals[:1]
            out[f"offs_{rows}_{K}_{is_b}"] = vals[1:].reshape(rows, K // 16).astype(np.int32)
        np.savez_compressed(os.path.join(HERE, "sf_layout.npz"), **out)
        print("wrote sf_layout.npz with", len(CASES), "cases")


if __name__ == "__main__":
    main()
