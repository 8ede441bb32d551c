"""Architecture detection and the (config, framework, arch) -> frontend dispatch table.

Mirror of the reference's ``flash_rt/hardware/__init__.py``: ``detect_arch()`` (:32-67), ``_PIPELINE_MAP`` (:74-226)
and ``resolve_pipeline_class`` (:241-273).  The reference accepts compute capabilities 8.7, 8.9, 11.0 and 12.x and
raises for 10.0; this package adds the one arch it is written for, ``"b200_sm100"``.  External packages extend
the map the same way the reference documents (``docs/plugin_model_template.md:14-24``): add a row at import.
"""
from __future__ import annotations

import importlib

ARCH_B200 = "b200_sm100"

# (config, framework, arch) -> (module, class)
_PIPELINE_MAP: dict[tuple[str, str, str], tuple[str, str]] = {
    ("pi05", "torch", ARCH_B200): ("flashrt_b200.pi05_decoder", "Pi05DecoderB200"),
    ("pi05_decoder", "torch", ARCH_B200): ("flashrt_b200.pi05_decoder", "Pi05DecoderB200"),
    ("pi05_prefix_encoder", "torch", ARCH_B200): ("flashrt_b200.pi05_prefix", "Pi05PrefixEncoderB200"),
}


def detect_arch() -> str:
    """``"b200_sm100"`` on a compute-capability 10.0 device; anything else is refused (one target, no dispatch)."""
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: flashrt_b200 has no CPU path")
    major, minor = torch.cuda.get_device_capability()
    if (major, minor) == (10, 0):
        return ARCH_B200
    raise RuntimeError(f"unsupported GPU compute capability {major}.{minor}: flashrt_b200 targets sm_100a (B200) only")


def resolve_pipeline_class(config: str, framework: str, arch: str):
    key = (config, framework, arch)
    if key not in _PIPELINE_MAP:
        known = ", ".join(sorted({f"{c}/{f}/{a}" for c, f, a in _PIPELINE_MAP}))
        raise ValueError(f"no pipeline registered for config={config!r} framework={framework!r} arch={arch!r}; "
                         f"known: {known}")
    mod, cls = _PIPELINE_MAP[key]
    return getattr(importlib.import_module(mod), cls)
