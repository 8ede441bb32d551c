"""Generates ``nvfp4_fake_quant.npz``: outputs of the reference's own torch NVFP4 reference on seeded inputs.

The reference keeps a CPU-runnable statement of its NVFP4 quantise + dequantise (block of 16, RN-even E4M3 block
scale of amax / 6, e2m1 levels chosen with ``torch.bucketize`` so that a tie goes to the smaller magnitude) in
``tests/test_fp4_integration_meta.py`` (``E2M1_LEVELS``, ``E2M1_MIDS``, ``fake_nvfp4``; "same algorithm as
csrc/quantize/quantize_fp4_dynamic.cu").  That module imports the CUDA extensions at import time, so it cannot be
imported on a CPU box; this script reads the file, takes exactly those three definitions out of its syntax tree and
executes them unchanged -- the numbers below are produced by the reference's code, not by a restatement.

Run where the reference tree is present:
    python tests/golden/make_nvfp4_golden.py [/path/to/reference]
"""
import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
WANTED = {"E2M1_LEVELS", "E2M1_MIDS", "fake_nvfp4"}


def load_reference(ref_root: str):
    path = os.path.join(ref_root, "tests", "test_fp4_integration_meta.py")
    tree = ast.parse(open(path).read())
    keep = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in WANTED:
            keep.append(node)
        elif isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id in WANTED for t in node.targets):
            keep.append(node)
    assert {getattr(n, "name", None) or n.targets[0].id for n in keep} == WANTED, "reference file changed"
    ns = {"torch": torch}
    exec(compile(ast.Module(body=keep, type_ignores=[]), path, "exec"), ns)
    return ns["fake_nvfp4"]


def inputs():
    g = torch.Generator().manual_seed(1234)
    cases = {}
    cases["normal_50x1024"] = (torch.randn(50, 1024, generator=g)).to(torch.bfloat16).float()
    cases["small_33x272"] = (torch.randn(33, 272, generator=g) * 0.02).to(torch.bfloat16).float()
    cases["wide_7x4096"] = (torch.randn(7, 4096, generator=g) * 3.0).to(torch.bfloat16).float()
    edge = torch.randn(8, 64, generator=g).to(torch.bfloat16).float()
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    edge[0, :16] = 0.0                   # all-zero block
    edge[1, 16:32] = ties                # amax 6 -> scale 1: every element sits on a threshold
    edge[2, 32:48] = ties * 0.5
    edge[3, 0:16] *= 1e-6                # scale rounds to zero
    edge[4, 16:32] *= 300.0
    cases["edge_8x64"] = edge
    return cases


def main():
    if len(sys.argv) < 2 and "FLASHRT_REFERENCE" not in os.environ:
        raise SystemExit("usage: make_nvfp4_golden.py <path to a FlashRT checkout>  (or FLASHRT_REFERENCE=<path>)")
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ["FLASHRT_REFERENCE"]
    fake_nvfp4 = load_reference(ref_root)
    out = {}
    for name, x in inputs().items():
        out["in_" + name] = x.numpy()
        out["out_" + name] = fake_nvfp4(x).numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "nvfp4_fake_quant.npz"), **out)
    print("wrote nvfp4_fake_quant.npz:", ", ".join(f"{k} {v.shape}" for k, v in out.items() if k.startswith("out_")))


if __name__ == "__main__":
    main()
