"""Quantisation descriptors of a loaded model: which format every quantised tensor has and where its scale came from.

Mirrors the record the reference's frontends expose as ``model.precision_spec`` (``flash_rt/core/precision_spec.py:46-159``,
filled by ``Pi05TorchFrontendRtx._snapshot_precision_spec``, ``flash_rt/frontends/torch/pi05_rtx.py:1480-1541``): the same
field names and the same JSON layout, so a file written by either side loads on the other.  Pure data and validation: no
kernel is chosen here.

What ``validate`` accepts is what this library's kernels compute:
  * ``fp8_e4m3``, per tensor, symmetric (static scale = amax / 448) -- every FP8 GEMM operand;
  * ``nvfp4``, per group of 16, symmetric (unsigned-E4M3 block scale, optional fp32 tensor scale) -- the NVFP4 GEMMs.
Everything else raises ``NotImplementedError``, as the reference's table does for what its kernels lack.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, fields
from typing import Any, Dict, Optional

import numpy as np

DTYPES = ("fp32", "fp16", "bf16", "fp8_e4m3", "fp8_e5m2", "nvfp4", "int8", "int4")
GRANULARITIES = ("per_tensor", "per_channel", "per_group")
SCHEMES = ("symmetric", "asymmetric")
SCALE_SOURCES = ("calibration", "qat_checkpoint", "runtime_dynamic", "manual")

# (dtype, granularity, group_size) combinations with a kernel behind them
SUPPORTED = {("fp8_e4m3", "per_tensor", None), ("nvfp4", "per_group", 16)}


def _as_list(a):
    return None if a is None else np.asarray(a).tolist()


@dataclass
class PrecisionSpec:
    """One quantised tensor (an activation site or a weight)."""
    dtype: str = "fp8_e4m3"
    granularity: str = "per_tensor"
    scheme: str = "symmetric"
    group_size: Optional[int] = None
    scale_source: str = "calibration"
    scale: Optional[np.ndarray] = None
    zero_point: Optional[np.ndarray] = None
    calibration_method: Optional[str] = None
    calibration_samples: Optional[int] = None
    calibration_percentile: Optional[float] = None

    def validate(self) -> None:
        for value, allowed, what in ((self.dtype, DTYPES, "dtype"), (self.granularity, GRANULARITIES, "granularity"),
                                     (self.scheme, SCHEMES, "scheme"), (self.scale_source, SCALE_SOURCES, "scale_source")):
            if value not in allowed:
                raise ValueError(f"{what}={value!r} is not one of {allowed}")
        if self.group_size is not None and self.granularity != "per_group":
            raise ValueError("group_size is only valid for per_group granularity")
        if self.granularity == "per_group" and self.group_size is None:
            raise ValueError("per_group granularity requires group_size")
        if self.scheme == "asymmetric" and self.zero_point is None:
            raise ValueError("asymmetric scheme requires zero_point")
        if self.scheme != "symmetric" or (self.dtype, self.granularity, self.group_size) not in SUPPORTED:
            raise NotImplementedError(
                f"no kernel of this library computes dtype={self.dtype!r}, granularity={self.granularity!r}, "
                f"group_size={self.group_size!r}, scheme={self.scheme!r}; built: {sorted(SUPPORTED, key=str)} symmetric")

    def to_dict(self) -> Dict[str, Any]:
        d = {f.name: getattr(self, f.name) for f in fields(self)}
        d["scale"], d["zero_point"] = _as_list(self.scale), _as_list(self.zero_point)
        return d

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PrecisionSpec":
        d = dict(d)
        if d.get("scale") is not None:
            d["scale"] = np.asarray(d["scale"], dtype=np.float32)
        if d.get("zero_point") is not None:
            d["zero_point"] = np.asarray(d["zero_point"])
        return cls(**d)


_GROUPS = ("encoder_layer_specs", "decoder_layer_specs", "weight_specs", "activation_specs")


@dataclass
class ModelPrecisionSpec:
    """All quantised tensors of a model, keyed by name inside four groups (the reference's grouping)."""
    encoder_layer_specs: Dict[str, PrecisionSpec] = field(default_factory=dict)
    decoder_layer_specs: Dict[str, PrecisionSpec] = field(default_factory=dict)
    weight_specs: Dict[str, PrecisionSpec] = field(default_factory=dict)
    activation_specs: Dict[str, PrecisionSpec] = field(default_factory=dict)
    source: str = "calibration"

    def validate(self) -> None:
        for g in _GROUPS:
            for spec in getattr(self, g).values():
                spec.validate()

    def to_json(self, path: str) -> None:
        payload = {"source": self.source}
        for g in _GROUPS:
            payload[g] = {k: v.to_dict() for k, v in getattr(self, g).items()}
        with open(path, "w", encoding="utf-8") as f:
            json.dump(payload, f, indent=2)

    @classmethod
    def from_json(cls, path: str) -> "ModelPrecisionSpec":
        with open(path, encoding="utf-8") as f:
            payload = json.load(f)
        return cls(source=payload.get("source", "calibration"),
                   **{g: {k: PrecisionSpec.from_dict(v) for k, v in payload.get(g, {}).items()} for g in _GROUPS})


# names of the decoder's GEMM-input sites, as the reference names their scale buffers
# (flash_rt/models/pi05/pipeline_rtx.py:649-660: "<weight name>_<layer>__step_<step>")
DECODER_SITE_NAMES = {"qkv": "decoder_attn_qkv_w", "o": "decoder_attn_o_w", "gu": "decoder_ffn_gate_up_w",
                      "d": "decoder_ffn_down_w"}


def snapshot_decoder(act_scale, sites, weight_scales: Dict[str, Any], *, precision: str, method: str, samples: int,
                     percentile: Optional[float], raw_scale=None) -> ModelPrecisionSpec:
    """The record of a calibrated action-expert decoder.  ``act_scale`` (steps, layers, len(sites)) static activation
    scales; ``weight_scales`` name -> per-layer weight scales; ``raw_scale`` (steps, layers, 2): scales of the
    un-normalised operands of the deferred-row-scale loop (sites "qkv_raw", "gu_raw")."""
    spec = ModelPrecisionSpec(source="calibration")
    if precision == "nvfp4":
        for name in weight_scales:
            e = PrecisionSpec(dtype="nvfp4", granularity="per_group", group_size=16, scale_source="runtime_dynamic")
            e.validate()
            spec.weight_specs[name] = e
        return spec
    a = np.asarray(act_scale, dtype=np.float32)
    common = dict(dtype="fp8_e4m3", granularity="per_tensor", scheme="symmetric", scale_source="calibration",
                  calibration_method=method, calibration_samples=samples, calibration_percentile=percentile)
    for s in range(a.shape[0]):
        for i in range(a.shape[1]):
            for k, site in enumerate(sites):
                e = PrecisionSpec(scale=a[s, i, k:k + 1].copy(), **common)
                e.validate()
                spec.decoder_layer_specs[f"{DECODER_SITE_NAMES[site]}_{i}__step_{s}"] = e
            if raw_scale is not None:
                r = np.asarray(raw_scale, dtype=np.float32)
                for k, site in enumerate(("qkv", "gu")):
                    e = PrecisionSpec(scale=r[s, i, k:k + 1].copy(), **common)
                    spec.decoder_layer_specs[f"{DECODER_SITE_NAMES[site]}_{i}__step_{s}__unnormalised"] = e
    for name, scales in weight_scales.items():
        for i, v in enumerate(np.asarray(scales, dtype=np.float32).reshape(-1)):
            e = PrecisionSpec(dtype="fp8_e4m3", scale_source="manual", scale=np.array([v], np.float32))
            spec.weight_specs[f"{name}_{i}"] = e
    return spec
