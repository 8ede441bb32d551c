"""Generates ``reference_surface.json``: for the pybind entry points of the reference that the denoise path calls,
the keyword names in binding order, read from the reference's own binding sources
(``csrc/bindings.cpp``, ``csrc/fa2_bindings.cpp``, ``csrc/fp4_bindings.cpp``: the ``py::arg("...")`` lists).

    python tests/golden/make_surface_golden.py [/path/to/reference]

The CPU test ``tests/test_abi_cpu.py`` checks that the stand-in modules of this package accept the same names in the
same order, so that reference call sites (positional or keyword) bind unchanged.
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

WANTED = {
    "flash_rt_kernels": ("csrc/bindings.cpp", [
        "rms_norm", "rms_norm_fp8", "ada_rms_norm_style", "ada_rms_norm_style_fp8", "residual_add_rms_norm",
        "residual_add_rms_norm_fp8", "gate_residual_ada_norm_fp8", "gate_geglu_merged", "gate_geglu_merged_fp8",
        "qkv_split_rope", "qkv_split_rope_devpos", "quantize_fp8_static", "quantize_fp8_device",
        "fp8_accumulate_scale_max", "residual_add", "bias_residual", "gate_mul_residual", "gpu_copy",
        "cfg_combine_into_residual", "fp8_gemm_descale_bf16out", "layer_norm", "bias_gelu_quantize_fp8_static_bf16",
        "bias_gate_mul_residual_bf16", "add_bias_bf16", "adaln_modulation6_bf16", "quantize_bf16_to_nvfp4_swizzled",
        "rms_norm_to_nvfp4_swizzled_bf16", "residual_add_rms_norm_to_nvfp4_swizzled_bf16"]),
    "flash_rt_fa2": ("csrc/fa2_bindings.cpp", ["fwd_bf16", "fwd_bf16_seqused", "fwd_bf16_seqused_splitkv"]),
    "flash_rt_fp4": ("csrc/fp4_bindings.cpp", [
        "quantize_fp4_dynamic_sfa_fp16", "quantize_fp4_dynamic_sfa_fp16_vec", "quantize_fp4_dynamic_sfa_bf16_vec",
        "sfa_size_bytes", "cutlass_fp4_gemm_variant", "cutlass_fp4_sq_fp16", "cutlass_fp4_gemm_bias_bf16",
        "pi05_adarms_fp4_sfa_fp16", "pi05_gate_res_adarms_fp4_sfa_fp16", "pi05_adarms_fp4_sfa_native_fp16",
        "pi05_gate_res_adarms_fp4_sfa_native_fp16", "gate_geglu_fp4_sfa_fp16", "gate_geglu_fp4_sfa_v2_fp16",
        "gate_geglu_fp4_sfa_vec_fp16", "rms_norm_fp4_sfa_fp16", "residual_add_rms_norm_fp4_sfa_fp16",
        "residual_add_rms_norm_fp4_sfa_v2_fp16"]),
}


def args_of(text: str, name: str):
    """py::arg names of the ``m.def("name", ...)`` statement (up to the next m.def / class_ / end of module)."""
    m = re.search(r'\.def\(\s*"%s"' % re.escape(name), text)
    if not m:
        return None
    rest = text[m.end():]
    nxt = re.search(r'\bm\.def\(|\.def\(\s*"|py::class_|PYBIND11_MODULE', rest)
    body = rest[:nxt.start()] if nxt else rest
    return re.findall(r'py::arg\("(\w+)"\)', body)


def main():
    if len(sys.argv) < 2 and "FLASHRT_REFERENCE" not in os.environ:
        raise SystemExit("usage: make_surface_golden.py <path to a FlashRT checkout>  (or FLASHRT_REFERENCE=<path>)")
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ["FLASHRT_REFERENCE"]
    out = {}
    for module, (path, names) in WANTED.items():
        text = open(os.path.join(ref, path)).read()
        out[module] = {}
        for n in names:
            a = args_of(text, n)
            assert a is not None, f"{path}: no binding named {n}"
            out[module][n] = a
    # GemmRunner methods are class members in the same file
    text = open(os.path.join(ref, "csrc/bindings.cpp")).read()
    out["GemmRunner"] = {n: args_of(text, n) for n in ("bf16_nn", "fp8_nn_dev", "fp8_nt_dev")}
    with open(os.path.join(HERE, "reference_surface.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print({k: len(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
