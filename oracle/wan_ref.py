"""TEST INFRASTRUCTURE ONLY — fp32 torch restatement (CPU) of a Wan2.2-shape video-DiT block.

PINNING.  Building blocks: pinned against the reference's own catalog ground truth -- ``_rms`` + ``_rope``
(full-width q/k RMSNorm, complex-pair RoPE) against ``qk_norm_rope_ref``, affine LayerNorm against
``norm_fused_ref``, modulated affine-free LayerNorm -> projections against ``modnorm_qkv_chain_ref``, LN -> fc1 ->
GELU(tanh) -> fc2 + x against ``vision_ffn_ref``, attention against ``attention_core_ref``
(``flash_rt/structures/catalog/*/reference.py``; fixtures ``tests/golden/wan_parts.npz`` by
``tests/golden/make_wan_golden.py``, checked in ``tests/test_oracle_cpu.py``).  Composition of the block (order of
the sub-layers, which of the six modulation vectors goes where): PARITY UNPINNED -- that arithmetic lives in the
external ``wan`` package (``wan.modules.model``, imported at flash_rt/frontends/torch/wan22_rtx.py:78-113), which
is not vendored in the reference tree, carries no pinned version there and is not installed here; the reference's
tests at that boundary are structural only.  The composition is restated from BASELINE configuration 4 and from the kernel call sites
the reference does contain: the six-way modulation and its use (flash_rt/models/motus/_modulate_fuse_swap.py:1-33,
csrc/kernels/elementwise.cu:603-645), the q/k RMSNorm over the full model width and the complex-pair 3-D RoPE
(csrc/quantize/qkv_split_norm_rope_bf16.cuh:22-41), affine-free LayerNorm with eps 1e-6
(csrc/quantize/ada_layer_norm_fp8.cu:58-147), GELU-tanh FFN (csrc/quantize/bias_gelu_quantize_fp8.cu:18-23).
"""
from __future__ import annotations

import torch


def _ln(x, eps=1e-6):
    return (x - x.mean(-1, keepdim=True)) * torch.rsqrt(x.var(-1, keepdim=True, unbiased=False) + eps)


def _rms(x, w, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, cos, sin):
    """x (B, L, H, hd); complex pairs (2c, 2c+1) times (cos + i sin)[t, c]."""
    B, L, H, hd = x.shape
    xr = x.reshape(B, L, H, hd // 2, 2)
    re, im = xr[..., 0], xr[..., 1]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.stack([re * c - im * s, re * s + im * c], dim=-1).reshape(B, L, H, hd)


def _attn(q, k, v):
    """q (B, Lq, H, hd), k / v (B, Lk, H, hd) -> (B, Lq, H*hd); bidirectional."""
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) * q.shape[-1] ** -0.5
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), v).reshape(q.shape[0], q.shape[1], -1)


def block(x, bw: dict, time_proj, context, cos, sin, head_dim: int):
    """x (B, L, D) fp32; bw: one entry of ``synthetic_wan_state()['blocks']`` (matrices (out, in));
    time_proj (B, 6, D); context (B, T, text_dim)."""
    B, L, D = x.shape
    H = D // head_dim
    f = lambda t: t.float()  # noqa: E731
    e = f(bw["modulation"])[None] + time_proj.float()                     # (B, 6, D)
    e = [e[:, j:j + 1, :] for j in range(6)]
    h = _ln(x) * (1 + e[1]) + e[0]
    q = _rms(h @ f(bw["q"]).t() + f(bw["q_b"]), f(bw["norm_q"])).reshape(B, L, H, head_dim)
    k = _rms(h @ f(bw["k"]).t() + f(bw["k_b"]), f(bw["norm_k"])).reshape(B, L, H, head_dim)
    v = (h @ f(bw["v"]).t() + f(bw["v_b"])).reshape(B, L, H, head_dim)
    a = _attn(_rope(q, cos, sin), _rope(k, cos, sin), v)
    x = x + (a @ f(bw["o"]).t() + f(bw["o_b"])) * e[2]
    hc = _ln(x) * f(bw["norm3_w"]) + f(bw["norm3_b"])
    cq = _rms(hc @ f(bw["cq"]).t() + f(bw["cq_b"]), f(bw["norm_cq"])).reshape(B, L, H, head_dim)
    T = context.shape[1]
    ck = _rms(context.float() @ f(bw["ck"]).t() + f(bw["ck_b"]), f(bw["norm_ck"])).reshape(B, T, H, head_dim)
    cv = (context.float() @ f(bw["cv"]).t() + f(bw["cv_b"])).reshape(B, T, H, head_dim)
    x = x + (_attn(cq, ck, cv) @ f(bw["co"]).t() + f(bw["co_b"]))
    h2 = _ln(x) * (1 + e[4]) + e[3]
    ff = torch.nn.functional.gelu(h2 @ f(bw["ffn1"]).t() + f(bw["ffn1_b"]), approximate="tanh")
    return x + (ff @ f(bw["ffn2"]).t() + f(bw["ffn2_b"])) * e[5]


def step(x, state: dict, time_proj, context, cos, sin):
    for bw in state["blocks"]:
        x = block(x, bw, time_proj, context, cos, sin, state["head_dim"])
    return x
