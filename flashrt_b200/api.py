"""Public API: ``load_model(...)`` -> ``VLAModel`` with ``predict`` / ``infer`` / ``calibrate``.

Mirror of the reference's ``flash_rt/api.py`` (``load_model`` :317-359, ``VLAModel`` :34-315) for the decoder-only
path: constructor keyword arguments the frontend does not declare are dropped after inspection of its
signature (as at ``api.py:926-1027``), the frontend is found through ``hardware._PIPELINE_MAP``, and the model
object exposes the same verbs.  ``set_prompt`` is replaced by ``set_prefix`` because the prompt / vision prefix
producer is outside this package: the caller hands over the per-layer prefix keys and values.
"""
from __future__ import annotations

import inspect

import numpy as np

from . import hardware

_FRAMEWORKS = ("torch",)


class VLAModel:
    def __init__(self, frontend, config: str, arch: str):
        self._fe = frontend
        self.config = config
        self.arch = arch

    @property
    def frontend(self):
        return self._fe

    @property
    def calibrated(self) -> bool:
        return bool(getattr(self._fe, "calibrated", False))

    @property
    def precision_spec(self):
        """The frontend's quantisation record (``flash_rt/api.py:286-290``), ``None`` if it keeps none yet."""
        return getattr(self._fe, "precision_spec", None)

    def set_prefix(self, prefix_k, prefix_v) -> None:
        self._fe.set_prefix(prefix_k, prefix_v)

    def set_prefix_from_encoder(self, encoder, embeds, slot: int = 0) -> int:
        """Run the prefix producer (``flashrt_b200.pi05_prefix.Pi05PrefixEncoderB200``) on ``embeds`` (seq, 2048) and
        let it write the per-layer keys / values straight into this model's cache rows [0, seq) of batch ``slot``
        -- the part of the reference's ``set_prompt`` + encoder forward that precedes the denoise loop."""
        fe = self._fe
        if encoder.layers != fe.layers:
            raise ValueError(f"encoder has {encoder.layers} layers, the action expert {fe.layers}")
        seq = encoder.encode(embeds, fe.k_cache[:, slot], fe.v_cache[:, slot])
        if seq != fe.prefix_len and not getattr(fe, "fixed_shape", False):
            raise ValueError(f"prefix of {seq} tokens, model built for {fe.prefix_len} (use fixed_shape=True)")
        if getattr(fe, "fixed_shape", False):
            fe.set_valid_prefix_len(seq)
        return seq

    def calibrate(self, noises, percentile: float | None = None, **kw) -> None:
        self._fe.calibrate(noises, percentile=percentile, **kw)

    def infer(self, obs: dict) -> dict:
        return self._fe.infer(obs)

    def predict(self, noise=None, **obs) -> np.ndarray:
        """One denoise loop.  ``noise``: host array (chunk, 32); returns the actions as a host array."""
        o = dict(obs)
        if noise is not None:
            o["noise"] = noise
        return self._fe.infer(o)["actions"]


def load_model(checkpoint, framework: str = "torch", config: str = "pi05", hardware_arch: str = "auto", **kwargs):
    """checkpoint: path to a ``.safetensors`` file, a ``{key: tensor}`` dict with the HF key names, or
    ``"synthetic[:seed]"`` for random-init weights of the right shapes."""
    if framework not in _FRAMEWORKS:
        raise ValueError(f"framework must be one of {_FRAMEWORKS}, got {framework!r}")
    arch = hardware.detect_arch() if hardware_arch in ("auto", None) else hardware_arch
    cls = hardware.resolve_pipeline_class(config, framework, arch)
    params = inspect.signature(cls.__init__).parameters
    accepted = {k: v for k, v in kwargs.items() if k in params}
    dropped = sorted(set(kwargs) - set(accepted))
    if dropped and not any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values()):
        raise TypeError(f"{cls.__name__} does not accept: {', '.join(dropped)}")
    return VLAModel(cls(checkpoint, **accepted), config, arch)
