"""CPU suite: the C-ABI shared library loads and exports every symbol the public header declares
(no compute call is made: there is no GPU here)."""
import ctypes
import os
import re

from flashrt_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_declares_only_plain_c_types():
    protos = _lib.parse_header()
    assert len(protos) >= 15
    for name, types in protos.items():
        assert name.startswith("frt_b200_")
        for t in types:
            assert t in ("ptr", "int", "long long", "float"), (name, t)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in _lib.parse_header():
        assert hasattr(lib, name), name


def test_every_exported_entry_point_is_declared():
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    exported = set(re.findall(r"\bT (frt_b200_\w+)", out))
    assert exported == set(_lib.parse_header())


def test_header_cites_the_reference_for_every_entry_point():
    text = open(_lib.HEADER_PATH).read()
    # each prototype is preceded by a comment block naming a reference file:line (or says it has none)
    blocks = re.split(r"\bint\s+frt_b200_\w+\s*\(", text)
    for b in blocks[:-1]:
        tail = b[-2500:]
        assert re.search(r"csrc/[\w/]+\.(cpp|cu|cuh|h):\d+", tail) or "no counterpart in the reference" in tail \
            or "Status word" in tail or "status word" in tail or "grid sizing" in tail


def test_shim_mirrors_reference_binding_names():
    from flashrt_b200 import flash_rt_fa2, flash_rt_kernels as fvk
    for n in ("rms_norm", "rms_norm_fp8", "ada_rms_norm_style", "ada_rms_norm_style_fp8", "residual_add_rms_norm",
              "residual_add_rms_norm_fp8", "gate_residual_ada_norm_fp8", "gate_geglu_merged", "gate_geglu_merged_fp8",
              "qkv_split_rope", "qkv_split_rope_devpos", "gate_mul_residual", "bias_residual", "residual_add",
              "gpu_copy", "quantize_fp8_static", "quantize_fp8_device", "fp8_accumulate_scale_max",
              "fp8_gemm_descale_bf16out", "GemmRunner", "has_cutlass_sm100", "get_sm_version"):
        assert callable(getattr(fvk, n)), n
    for n in ("fp8_nt_dev", "fp8_nn_dev", "bf16_nn", "autotune_fp8_nn_dev", "autotune_bf16_nn"):
        assert callable(getattr(fvk.GemmRunner, n)), n
    for n in ("fwd_bf16", "fwd_bf16_seqused", "fwd_bf16_seqused_splitkv"):
        assert callable(getattr(flash_rt_fa2, n)), n
    assert not hasattr(fvk, "silu_mul_split_fp8_fp16")        # outside the path: refused, not faked
    import pytest
    with pytest.raises(fvk.NotBuilt):
        fvk.GemmRunner().bf16_nn(0, 0, 0, 128, 128, 128)      # only the 32 <-> 1024 action projections are on the path


def test_stand_in_modules_accept_the_reference_binding_signatures():
    """Every reference entry point of the path (names and keyword order read from the reference's pybind sources into
    tests/golden/reference_surface.json) exists in the stand-in modules with the same parameter names in the same
    order, so that positional and keyword call sites of the reference bind unchanged.  Extra parameters of the
    stand-ins are keyword-only."""
    import inspect
    import json
    import os
    from flashrt_b200 import flash_rt_fa2, flash_rt_fp4, flash_rt_kernels
    surface = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_surface.json")))
    mods = {"flash_rt_kernels": flash_rt_kernels, "flash_rt_fa2": flash_rt_fa2, "flash_rt_fp4": flash_rt_fp4,
            "GemmRunner": flash_rt_kernels.GemmRunner}
    problems = []
    for mod_name, entries in surface.items():
        for name, ref_args in entries.items():
            fn = getattr(mods[mod_name], name, None)
            if fn is None:
                problems.append(f"{mod_name}.{name}: missing")
                continue
            params = list(inspect.signature(fn).parameters.values())
            if params and params[0].name == "self":
                params = params[1:]
            positional = [p.name for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
            if positional != ref_args:
                problems.append(f"{mod_name}.{name}: {positional} != reference {ref_args}")
    assert not problems, "\n".join(problems)


def test_expert_loop_args_struct_matches_the_header():
    """The ctypes mirror of ``frt_b200_expert_loop_args`` has the header's members in the header's order, and the
    size a C compiler gives the struct."""
    import subprocess
    import tempfile
    from flashrt_b200.pi05_decoder import ExpertLoopArgs
    text = open(_lib.HEADER_PATH).read()
    body = re.search(r"typedef struct frt_b200_expert_loop_args \{(.*?)\} frt_b200_expert_loop_args;", text, re.S).group(1)
    names = []
    for decl in body.split(";"):
        decl = decl.strip()
        if decl:
            names += [n.strip().lstrip("*") for n in re.sub(r"^(const\s+)?(void|long long|int)\s*", "", decl).split(",")]
    assert names == [f[0] for f in ExpertLoopArgs._fields_]
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "s.c")
        open(src, "w").write('#include <stdio.h>\n#include "flashrt_b200.h"\n'
                             'int main(void){printf("%zu", sizeof(frt_b200_expert_loop_args));return 0;}\n')
        exe = os.path.join(d, "s")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), src, "-o", exe], check=True)
        size = int(subprocess.run([exe], capture_output=True, text=True, check=True).stdout)
    assert size == ctypes.sizeof(ExpertLoopArgs)


def test_expert_loop_schedule_covers_every_unit_once():
    """Host evaluation of the persistent kernel's static schedule: in every phase of every block each unit has exactly
    one owner, no CTA owns two units of a phase, attention CTAs own no QKV unit of the same block, and over the whole
    loop every CTA streams the same number of weight units to within one."""
    lib = _lib.load()
    G, att_units, blocks = 148, 52, 180
    counts = {0: 20, 1: 16, 2: 64, 3: 32, 4: att_units}
    out = ctypes.c_int(0)
    per_cta = [0] * G
    for gl in list(range(0, 40)) + [blocks - 1]:
        owners = {}
        for ph, n in counts.items():
            seen = {}
            for cta in range(G):
                assert lib.frt_b200_expert_loop_schedule(G, cta, gl, ph, att_units, ctypes.addressof(out)) == 0
                u = out.value
                assert -1 <= u < n
                if u >= 0:
                    assert u not in seen
                    seen[u] = cta
                    if ph < 4 and gl < 37:           # 37 blocks x 132 units = 33 full rounds of 148
                        per_cta[cta] += 1
            assert sorted(seen) == list(range(n)), (gl, ph)
            owners[ph] = set(seen.values())
        assert not (owners[0] & owners[4])
    assert max(per_cta) - min(per_cta) <= 1
    assert lib.frt_b200_expert_loop_schedule(G, G, 0, 0, att_units, ctypes.addressof(out)) == -1


def test_expert_loop_entry_points_validate_before_touching_the_device():
    """Argument checks of the single-launch loop run on the host: no GPU is needed to be refused."""
    from flashrt_b200.pi05_decoder import ExpertLoopArgs
    lib = _lib.load()
    n = ctypes.c_longlong(0)
    assert lib.frt_b200_expert_loop_workspace_bytes(50, 768, ctypes.addressof(n)) == 0
    # sync words + FP8 / bf16 activations + split-K partials + 4 x 13 attention units of 128 x 256 bf16 + their lse
    assert n.value == 256 + 64 * 1024 + 64 * 2048 * 2 + 64 * 2048 + 64 * 4096 + 4 * 64 * 1024 * 4 + 52 * 128 * 256 * 2 \
        + 52 * 128 * 4
    assert lib.frt_b200_expert_loop_workspace_bytes(65, 768, ctypes.addressof(n)) == -2      # more than 64 tokens
    assert lib.frt_b200_expert_loop_workspace_bytes(50, 768, None) == -1
    a = ExpertLoopArgs()
    assert lib.frt_b200_expert_loop_fp8(None, ctypes.sizeof(a), None) == -1
    assert lib.frt_b200_expert_loop_fp8(ctypes.addressof(a), ctypes.sizeof(a) - 8, None) == -1   # struct size mismatch
    assert lib.frt_b200_expert_loop_fp8(ctypes.addressof(a), ctypes.sizeof(a), None) == -1       # null pointers


def test_fp16_named_fp4_entries_refuse_without_a_stated_dtype():
    """The reference's ``*_fp16`` bindings take fp16 buffers; here the 16-bit type is bf16 and a pointer carries no type,
    so those names refuse unless the caller states that its buffers hold bf16."""
    import pytest
    from flashrt_b200 import flash_rt_fp4 as fp4
    from flashrt_b200.flash_rt_kernels import NotBuilt
    assert fp4.STREAM_DTYPE == "bfloat16"
    for name in ("pi05_adarms_fp4_sfa_fp16", "quantize_fp4_dynamic_sfa_fp16", "rms_norm_fp4_sfa_fp16",
                 "residual_add_rms_norm_fp4_sfa_v2_fp16", "gate_geglu_fp4_sfa_fp16", "cutlass_fp4_sq_fp16"):
        with pytest.raises(NotBuilt, match="bf16"):
            getattr(fp4, name)(0, 0, 0, 0, 0, 0, 0, 0, 0)
