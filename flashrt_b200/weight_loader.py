"""Declarative weight loading: the ``WEIGHT_SPEC`` plugin contract of the reference
(``flash_rt/executors/weight_loader.py:89-264`` and ``flash_rt/executors/torch_weights.py``).

A frontend declares ``WEIGHT_SPEC = ModelWeightSpec(framework, blocks=[LayerBlock(prefix_fmt, num_layers,
items=[Item(name, key | FusedQKV | FusedGateUp, transforms=[...], sink=..., scale_into=...)])])`` and loads with
``WeightLoader(source, target=self, spec=self.WEIGHT_SPEC).run()``.  Names and argument meaning follow the
reference so that a spec written for it reads the same here; the implementation is this package's own.

Differences that matter on B200: ``Quant()`` produces FP8 E4M3 with the per-tensor scale
``max(amax / 448, 1e-12)`` (``flash_rt/frontends/torch/pi05_rtx.py:344-350``), and FP8 GEMM weights are kept
(N, K) K-contiguous (the reference's ``fp8_layout == "nk"`` form) because that is what the tcgen05 GEMM reads —
so decoder specs here use ``Quant()`` without the ``tT()`` the (K, N) cuBLASLt path needed.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Protocol, runtime_checkable

import torch

FP8 = torch.float8_e4m3fn


# ------------------------------------------------------------------ sources
@runtime_checkable
class WeightSource(Protocol):
    def get(self, key: str) -> torch.Tensor: ...
    def has(self, key: str) -> bool: ...


class DictSource:
    """Checkpoint held as a ``{key: tensor}`` mapping."""

    def __init__(self, tensors: dict):
        self._t = tensors

    def get(self, key: str) -> torch.Tensor:
        try:
            return self._t[key]
        except KeyError as e:
            raise KeyError(f"checkpoint has no tensor {key!r}") from e

    def has(self, key: str) -> bool:
        return key in self._t


class SafetensorsSource:
    """Lazy reader of a ``.safetensors`` file."""

    def __init__(self, path: str):
        from safetensors import safe_open
        self._f = safe_open(path, framework="pt", device="cpu")
        self._keys = set(self._f.keys())

    def get(self, key: str) -> torch.Tensor:
        if key not in self._keys:
            raise KeyError(f"checkpoint has no tensor {key!r}")
        return self._f.get_tensor(key)

    def has(self, key: str) -> bool:
        return key in self._keys


# ------------------------------------------------------------------ spec
@dataclass
class Item:
    name: str
    key: Any
    transforms: list = field(default_factory=list)
    sink: Any = None
    scale_into: str | None = None


@dataclass
class LayerBlock:
    prefix_fmt: str
    num_layers: int
    items: list
    name: str = ""


@dataclass
class ModelWeightSpec:
    framework: str
    blocks: list = field(default_factory=list)
    singletons: list = field(default_factory=list)
    dims: dict = field(default_factory=dict)


@dataclass
class LoaderContext:
    source: Any
    target: Any
    prefix: str = ""
    layer_idx: int = -1
    scales: dict = field(default_factory=dict)
    pending_scale: float | None = None

    def subkey(self, template: str) -> str:
        return template.format(prefix=self.prefix, i=self.layer_idx) if "{" in template else template


# ------------------------------------------------------------------ composite keys
def _interleave_rows(w: torch.Tensor, heads: int) -> torch.Tensor:
    """(out, in): within each head move row j of the first half to 2j and row j of the second half to 2j+1,
    which turns rotate-half RoPE into rotation of adjacent pairs (pi05_rtx.py:70-79)."""
    out_dim, in_dim = w.shape
    hd = out_dim // heads
    return w.reshape(heads, 2, hd // 2, in_dim).permute(0, 2, 1, 3).reshape(out_dim, in_dim)


@dataclass
class FusedQKV:
    """q | k | v projection weights, each (out, in), concatenated along ``out``."""
    q: str
    k: str
    v: str
    interleave_q_heads: int = 0
    interleave_k_heads: int = 0

    def resolve(self, source, ctx: LoaderContext) -> torch.Tensor:
        q = source.get(ctx.subkey(self.q)).float()
        k = source.get(ctx.subkey(self.k)).float()
        v = source.get(ctx.subkey(self.v)).float()
        if self.interleave_q_heads:
            q = _interleave_rows(q, self.interleave_q_heads)
        if self.interleave_k_heads:
            k = _interleave_rows(k, self.interleave_k_heads)
        return torch.cat([q, k, v], dim=0)


@dataclass
class FoldNorm:
    """Wrap a (composite) weight key: multiply every input column of the (out, in) weight by ``1 + norm_weight``,
    in fp32, so that the RMSNorm in front of the projection runs with unit weight (pi05_rtx.py:180-206; folding in
    bf16 would round 1 + w to 0 for weights near -1)."""
    inner: Any
    norm: str

    def resolve(self, source, ctx: LoaderContext) -> torch.Tensor:
        w = self.inner.resolve(source, ctx) if hasattr(self.inner, "resolve") else source.get(ctx.subkey(self.inner))
        return w.float() * (1.0 + source.get(ctx.subkey(self.norm)).float()).unsqueeze(0)


@dataclass
class FusedGateUp:
    """gate | up projection weights, each (out, in), concatenated along ``out`` (merged [gate | up] layout)."""
    gate: str
    up: str

    def resolve(self, source, ctx: LoaderContext) -> torch.Tensor:
        return torch.cat([source.get(ctx.subkey(self.gate)).float(), source.get(ctx.subkey(self.up)).float()], dim=0)


# ------------------------------------------------------------------ transforms
class tT:
    """Transpose the last two dims and make contiguous."""

    def apply(self, t, ctx):
        return t.transpose(-1, -2).contiguous()


class ToBf16:
    def apply(self, t, ctx):
        return t.to(torch.bfloat16)


class Scale:
    """Multiply by a constant (e.g. the -1/N folded into the action out-projection)."""

    def __init__(self, factor: float):
        self.factor = factor

    def apply(self, t, ctx):
        return t.float() * self.factor


class Quant:
    """Per-tensor symmetric FP8 E4M3: scale = max(amax / 448, 1e-12); codes = e4m3(clamp(w / scale)).
    The weight is first rounded to bf16, the precision the reference quantises from."""

    def apply(self, t, ctx):
        w = t.to(torch.bfloat16).float()
        amax = float(w.abs().max())
        scale = max(amax / 448.0, 1e-12)
        ctx.pending_scale = scale
        return (w / scale).clamp(-448.0, 448.0).to(FP8)


# ------------------------------------------------------------------ sinks
class Attr:
    def __init__(self, name: str):
        self.name = name

    def reset(self, target):
        pass

    def store(self, target, tensor, scale=None):
        setattr(target, self.name, tensor)

    def finalize(self, target):
        pass


class TensorList:
    def __init__(self, name: str):
        self.name = name

    def reset(self, target):
        setattr(target, self.name, [])

    def store(self, target, tensor, scale=None):
        getattr(target, self.name).append(tensor)

    def finalize(self, target):
        pass


class FlatCat:
    """Collect per-layer tensors and stack them into one (layers, ...) tensor at the end."""

    def __init__(self, name: str):
        self.name = name
        self._parts: list = []

    def reset(self, target):
        self._parts = []

    def store(self, target, tensor, scale=None):
        self._parts.append(tensor)

    def finalize(self, target):
        if self._parts:
            setattr(target, self.name, torch.stack(self._parts, dim=0).contiguous())
        self._parts = []


# ------------------------------------------------------------------ runner
class WeightLoader:
    def __init__(self, source, *, target, spec: ModelWeightSpec):
        if not isinstance(source, WeightSource):
            raise TypeError(f"WeightLoader: source must implement get/has (got {type(source).__name__})")
        if not isinstance(spec, ModelWeightSpec):
            raise TypeError(f"WeightLoader: spec must be ModelWeightSpec (got {type(spec).__name__})")
        self.source, self.target, self.spec = source, target, spec

    def _items(self):
        for it in self.spec.singletons:
            yield it
        for b in self.spec.blocks:
            for it in b.items:
                yield it

    def _run_item(self, item: Item, ctx: LoaderContext):
        try:
            if hasattr(item.key, "resolve"):
                t = item.key.resolve(self.source, ctx)
            else:
                t = self.source.get(ctx.subkey(item.key))
            ctx.pending_scale = None
            for tr in item.transforms:
                t = tr.apply(t, ctx)
        except Exception as e:
            raise type(e)(f"weight item {item.name!r} (layer {ctx.layer_idx}): {e}") from e
        if ctx.pending_scale is not None and item.scale_into:
            ctx.scales.setdefault(item.scale_into, []).append(ctx.pending_scale)
        if item.sink is not None:
            item.sink.store(self.target, t, scale=ctx.pending_scale)

    def run(self) -> LoaderContext:
        ctx = LoaderContext(source=self.source, target=self.target)
        seen = set()
        for it in self._items():
            if it.sink is not None and id(it.sink) not in seen:
                it.sink.reset(self.target)
                seen.add(id(it.sink))
        for it in self.spec.singletons:
            ctx.prefix, ctx.layer_idx = "", -1
            self._run_item(it, ctx)
        for b in self.spec.blocks:
            for i in range(b.num_layers):
                ctx.prefix, ctx.layer_idx = b.prefix_fmt.format(i=i), i
                for it in b.items:
                    self._run_item(it, ctx)
        seen = set()
        for it in self._items():
            if it.sink is not None and id(it.sink) not in seen:
                it.sink.finalize(self.target)
                seen.add(id(it.sink))
        for name, values in ctx.scales.items():
            setattr(self.target, name, values)
        return ctx
