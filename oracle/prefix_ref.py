"""TEST INFRASTRUCTURE ONLY — fp32 torch restatement (CPU) of the Gemma-2B encoder layers that produce the prefix
keys / values of the action expert.

Only ``tests/`` import this module.  It follows
  * layer dataflow ........ training/_vendor/openpi_pi0_pytorch/gemma_pytorch.py:158-238 (pre-norm attention and GeGLU
                            MLP with residuals; RMSNorm scales by 1 + weight) and the kernel sequence of
                            flash_rt/models/pi05/pipeline_rtx.py:1209-1435 (the last layer stops after K / V)
  * weight preparation .... flash_rt/frontends/torch/pi05_rtx.py:178-214 (1 + w folded into the next projection in
                            fp32, q / k rows interleaved so that RoPE rotates adjacent pairs)
  * attention / RoPE ...... the functions of ``block_ref`` (pinned against the reference's catalog functions by
                            tests/golden/cfg0_block.npz); the composition of the layer itself is restated from the
                            source text and is not pinned by a reference fixture ("parity unpinned" for that part).
"""
from __future__ import annotations

import numpy as np
import torch

from . import block_ref as R

ENC_D, ENC_H, ENC_NH, ENC_NKV, ENC_HD = 2048, 16384, 8, 1, 256
EP = "paligemma_with_expert.paligemma.model.language_model.layers.{i}"


def rms(x, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def _fq(t: torch.Tensor, scale: float) -> torch.Tensor:
    """Per-tensor FP8 E4M3 fake quantisation: e4m3(clamp(t / scale, +-448)) * scale (torch's cast is bit-identical to
    the oracle's and the kernels', checked in tests/test_oracle_cpu.py)."""
    return (t / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() * scale


def _wq(w: torch.Tensor) -> torch.Tensor:
    """Weight as the loader stores it: rounded to bf16, then per-tensor E4M3 with scale amax / 448."""
    w = w.to(torch.bfloat16).float()
    return _fq(w, max(float(w.abs().max()) / 448.0, 1e-12))


def encoder_kv(embeds: torch.Tensor, sd: dict, layers: int, act_scales=None):
    """embeds (seq, 2048) fp32 -> lists K[i], V[i] of (seq, 256): K with RoPE at positions 0..seq-1, in the
    interleaved feature order of the kernel layout.  ``act_scales`` (layers, 4) [qkv, o, gu, d]: restate the FP8
    arithmetic of the device path (quantised weights with the norm scale folded in, GEMM inputs quantised with the
    given static scales, bf16 GEMM outputs); None = plain fp32."""
    if act_scales is not None:
        return _encoder_kv_fp8(embeds, sd, layers, act_scales)
    f = lambda k: sd[k].float()  # noqa: E731
    seq = embeds.shape[0]
    tab = R.rope_table(np.arange(seq)).to(torch.bfloat16).float()
    x = embeds.float().clone()
    Ks, Vs = [], []
    for i in range(layers):
        p = EP.format(i=i)
        h = rms(x) * (1.0 + f(f"{p}.input_layernorm.weight"))
        q = h @ R.interleave_qk_rows(f(f"{p}.self_attn.q_proj.weight"), ENC_NH).t()
        k = h @ R.interleave_qk_rows(f(f"{p}.self_attn.k_proj.weight"), ENC_NKV).t()
        v = h @ f(f"{p}.self_attn.v_proj.weight").t()
        q = R.rope_adjacent_pairs(q.reshape(seq, ENC_NH, ENC_HD), tab)
        k = R.rope_adjacent_pairs(k.reshape(seq, ENC_NKV, ENC_HD), tab)
        v = v.reshape(seq, ENC_NKV, ENC_HD)
        Ks.append(k.reshape(seq, ENC_HD))
        Vs.append(v.reshape(seq, ENC_HD))
        if i == layers - 1:
            break
        a = R.attention(q, k, v, ENC_HD ** -0.5).reshape(seq, ENC_NH * ENC_HD)
        x = x + a @ f(f"{p}.self_attn.o_proj.weight").t()
        h2 = rms(x) * (1.0 + f(f"{p}.post_attention_layernorm.weight"))
        hidden = R.gelu_tanh(h2 @ f(f"{p}.mlp.gate_proj.weight").t()) * (h2 @ f(f"{p}.mlp.up_proj.weight").t())
        x = x + hidden @ f(f"{p}.mlp.down_proj.weight").t()
    return Ks, Vs


def _encoder_kv_fp8(embeds, sd, layers, act_scales):
    f = lambda k: sd[k].float()  # noqa: E731
    bf = lambda t: t.to(torch.bfloat16).float()  # noqa: E731
    seq = embeds.shape[0]
    tab = R.rope_table(np.arange(seq)).to(torch.bfloat16).float()
    x = bf(embeds.float())
    Ks, Vs = [], []
    for i in range(layers):
        p = EP.format(i=i)
        sc = [float(v) for v in act_scales[i]]
        fold_a = (1.0 + f(f"{p}.input_layernorm.weight")).unsqueeze(0)
        wqkv = _wq(torch.cat([R.interleave_qk_rows(f(f"{p}.self_attn.q_proj.weight"), ENC_NH),
                              R.interleave_qk_rows(f(f"{p}.self_attn.k_proj.weight"), ENC_NKV),
                              f(f"{p}.self_attn.v_proj.weight")], dim=0) * fold_a)
        qkv = bf(_fq(rms(x), sc[0]) @ wqkv.t())
        q = bf(R.rope_adjacent_pairs(qkv[:, :2048].reshape(seq, ENC_NH, ENC_HD), tab))
        k = bf(R.rope_adjacent_pairs(qkv[:, 2048:2304].reshape(seq, ENC_NKV, ENC_HD), tab))
        v = qkv[:, 2304:].reshape(seq, ENC_NKV, ENC_HD)
        Ks.append(k.reshape(seq, ENC_HD))
        Vs.append(v.reshape(seq, ENC_HD))
        if i == layers - 1:
            break
        a = bf(R.attention(q, k, v, ENC_HD ** -0.5).reshape(seq, ENC_NH * ENC_HD))
        x = bf(x + bf(_fq(a, sc[1]) @ _wq(f(f"{p}.self_attn.o_proj.weight")).t()))
        fold_f = (1.0 + f(f"{p}.post_attention_layernorm.weight")).unsqueeze(0)
        wgu = _wq(torch.cat([f(f"{p}.mlp.gate_proj.weight"), f(f"{p}.mlp.up_proj.weight")], dim=0) * fold_f)
        gu = bf(_fq(rms(x), sc[2]) @ wgu.t())
        hidden = R.gelu_tanh(gu[:, :ENC_H]) * gu[:, ENC_H:]
        x = bf(x + bf(_fq(hidden, sc[3]) @ _wq(f(f"{p}.mlp.down_proj.weight")).t()))
    return Ks, Vs
