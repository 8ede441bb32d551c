"""Generates ``precision_spec_reference.json`` with the reference's OWN classes: a small ``ModelPrecisionSpec`` holding
one entry per group (the shapes its Pi0.5 frontend snapshots at calibration time), written by its ``to_json``.

    python tests/golden/make_precision_spec_golden.py /path/to/reference

The CPU test ``tests/test_formats_cpu.py`` loads that file with this package's mirror, checks every field, and checks
that writing it again gives the same JSON document -- so a spec file written by either side loads on the other.
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    path = os.path.join(sys.argv[1], "flash_rt", "core", "precision_spec.py")
    spec = importlib.util.spec_from_file_location("ref_precision_spec", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_precision_spec"] = mod          # dataclasses resolve annotations through sys.modules
    spec.loader.exec_module(mod)
    P, M = mod.PrecisionSpec, mod.ModelPrecisionSpec
    m = M(source="calibration")
    common = dict(dtype="fp8_e4m3", granularity="per_tensor", scheme="symmetric", scale_source="calibration",
                  calibration_method="percentile", calibration_samples=8, calibration_percentile=99.9)
    m.decoder_layer_specs["decoder_attn_qkv_w_3__step_7"] = P(scale=np.array([0.0123], np.float32), **common)
    m.encoder_layer_specs["encoder_ffn_down_w_0"] = P(scale=np.array([0.5], np.float32), **common)
    m.activation_specs["vision_patch"] = P(scale=np.array([1.25], np.float32), **common)
    m.weight_specs["decoder_ffn_down_w_1"] = P(dtype="fp8_e4m3", scale_source="manual", scale=np.array([3.0e-4], np.float32))
    m.validate()
    m.to_json(os.path.join(HERE, "precision_spec_reference.json"))


if __name__ == "__main__":
    main()
