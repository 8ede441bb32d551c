"""TEST INFRASTRUCTURE ONLY — fp32 torch restatement (CPU) of the reference's action-expert
denoise step: adaRMS block, MQA attention over prefix + fresh keys, GeGLU MLP, gated residuals,
time conditioning, and the Euler flow-matching loop.

Only ``tests/``, the smoke check and the benchmark's CPU-baseline leg import this module.

What each function follows (paths inside the FlashRT tree):
  * block dataflow ............ training/_vendor/openpi_pi0_pytorch/gemma_pytorch.py:158-238,
                                flash_rt/structures/catalog/decoder_block/reference.py:10-38
  * adaRMS + gate ............. flash_rt/structures/catalog/adaln_producer/reference.py:8-40
  * GeGLU MLP + gated residual  flash_rt/structures/catalog/decoder_ffn/reference.py:20-64
  * attention ................. flash_rt/structures/catalog/attention_core/reference.py:8-36
  * RoPE ...................... flash_rt/structures/catalog/qkv_rope/reference.py:8-39 (rotate-half) and the
                                adjacent-pair kernel form, csrc/kernels/rope.cu:135-208, related by the row
                                interleave of flash_rt/frontends/torch/pi05_rtx.py:70-79
  * rope table ................ flash_rt/models/pi05/pipeline_rtx.py:473-505
  * time embedding / styles ... flash_rt/frontends/torch/pi05_rtx.py:394-437
  * Euler loop ................ flash_rt/models/pi05/pipeline_rtx.py:1451-1504 (out-projection pre-scaled by
                                -1/N, flash_rt/frontends/torch/pi05_rtx.py:587-593)

Pinning: ``tests/golden/cfg0_block.npz`` holds outputs of the reference's own catalog functions (imported
from the reference tree by ``tests/golden/make_golden.py``) on the seeded configuration-0 inputs;
``tests/test_oracle_cpu.py`` checks this module against them.

Weight dictionary ("kernel layout", what the reference's converter produces, pi05_rtx.py:216-283):
  decoder_attn_qkv_w (L, D, 2560)  [K, N], Q and K output columns interleaved for adjacent-pair RoPE
  decoder_attn_o_w (L, 2048, D), decoder_ffn_gate_w / decoder_ffn_up_w (L, D, H), decoder_ffn_down_w (L, H, D)
  decoder_pre_attn_norm_mod_w (L, D, 3D) / _b (L, 3D), decoder_pre_ffn_norm_mod_w / _b, decoder_final_norm_mod_w / _b
  decoder_time_mlp_in_w / _b, decoder_time_mlp_out_w / _b, decoder_action_in_proj_w (32, D) / _b,
  decoder_action_out_proj_w (D, 32) / _b
"""
from __future__ import annotations

import math

import numpy as np
import torch

DEC_D, DEC_H, DEC_NH, DEC_NKV, DEC_HD, DEC_L = 1024, 4096, 8, 1, 256, 18
ACTION_DIM = 32


# ------------------------------------------------------------------ synthetic configuration
def synthetic_checkpoint(seed: int = 0, layers: int = DEC_L, dtype=torch.float32) -> dict:
    """Random-init weights of the action expert: every matrix ~ N(0, 0.02), biases zero."""
    g = torch.Generator().manual_seed(seed)

    def w(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(dtype)

    D, H, L = DEC_D, DEC_H, layers
    qkv = (DEC_NH + 2 * DEC_NKV) * DEC_HD
    return {
        "decoder_attn_qkv_w": w(L, D, qkv),
        "decoder_attn_o_w": w(L, DEC_NH * DEC_HD, D),
        "decoder_ffn_gate_w": w(L, D, H),
        "decoder_ffn_up_w": w(L, D, H),
        "decoder_ffn_down_w": w(L, H, D),
        "decoder_pre_attn_norm_mod_w": w(L, D, 3 * D),
        "decoder_pre_attn_norm_mod_b": torch.zeros(L, 3 * D, dtype=dtype),
        "decoder_pre_ffn_norm_mod_w": w(L, D, 3 * D),
        "decoder_pre_ffn_norm_mod_b": torch.zeros(L, 3 * D, dtype=dtype),
        "decoder_final_norm_mod_w": w(D, 3 * D),
        "decoder_final_norm_mod_b": torch.zeros(3 * D, dtype=dtype),
        "decoder_time_mlp_in_w": w(D, D),
        "decoder_time_mlp_in_b": torch.zeros(D, dtype=dtype),
        "decoder_time_mlp_out_w": w(D, D),
        "decoder_time_mlp_out_b": torch.zeros(D, dtype=dtype),
        "decoder_action_in_proj_w": w(ACTION_DIM, D),
        "decoder_action_in_proj_b": torch.zeros(D, dtype=dtype),
        "decoder_action_out_proj_w": w(D, ACTION_DIM),
        "decoder_action_out_proj_b": torch.zeros(ACTION_DIM, dtype=dtype),
    }


def synthetic_prefix_kv(seed: int = 1, layers: int = DEC_L, prefix_len: int = 768):
    """Per-layer prefix keys / values ~ N(0, 1), (L, P, 256) each; K is stored post-RoPE, as the encoder leaves it."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(layers, prefix_len, DEC_NKV * DEC_HD, generator=g)
    v = torch.randn(layers, prefix_len, DEC_NKV * DEC_HD, generator=g)
    return k, v


def synthetic_noise(seed: int, chunk: int = 50):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(chunk, ACTION_DIM, generator=g)


# ------------------------------------------------------------------ conditioning
def time_embedding(t: float, dim: int = DEC_D) -> torch.Tensor:
    """[sin(2 pi t / p_j) | cos(2 pi t / p_j)], p_j = 4e-3 * (4 / 4e-3)^(j / (dim/2 - 1)), fp32."""
    min_period, max_period = 4e-3, 4.0
    fraction = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float32)
    period = min_period * (max_period / min_period) ** fraction
    sinusoid = torch.tensor(t, dtype=torch.float32) * (1.0 / period) * 2 * math.pi
    return torch.cat([torch.sin(sinusoid), torch.cos(sinusoid)], dim=-1)


def time_schedule(num_steps: int) -> list[float]:
    """t_0 = 1, t_{k+1} = t_k - 1/N, accumulated in fp32 like the reference's loop."""
    dt = torch.tensor(-1.0 / num_steps, dtype=torch.float32)
    t = torch.tensor(1.0, dtype=torch.float32)
    out = []
    for _ in range(num_steps):
        out.append(float(t))
        t = t + dt
    return out


def _silu(x):
    return x * torch.sigmoid(x)


def conditioning(ckpt: dict, t: float, round_bf16: bool = False) -> torch.Tensor:
    """cond = silu(W_out silu(W_in emb(t) + b_in) + b_out).  ``round_bf16`` reproduces the rounding points
    of the reference's bf16 precompute (embedding, each matmul result and each SiLU result rounded to bf16)."""
    r = (lambda z: z.to(torch.bfloat16).float()) if round_bf16 else (lambda z: z)
    te = r(time_embedding(t))
    W = {k: (r(v.float()) if round_bf16 else v.float()) for k, v in ckpt.items() if k.startswith("decoder_time_mlp")}
    h = r(r(te @ W["decoder_time_mlp_in_w"]) + W["decoder_time_mlp_in_b"])
    h = r(_silu(h))
    h = r(r(h @ W["decoder_time_mlp_out_w"]) + W["decoder_time_mlp_out_b"])
    return r(_silu(h))


def styles(ckpt: dict, num_steps: int, layers: int, round_bf16: bool = False):
    """style_attn / style_ffn (N, L, 3D) and style_final (N, 3D): cond . W_mod + b_mod, rows = [scale|shift|gate]."""
    r = (lambda z: z.to(torch.bfloat16).float()) if round_bf16 else (lambda z: z)
    sa = torch.empty(num_steps, layers, 3 * DEC_D)
    sf = torch.empty(num_steps, layers, 3 * DEC_D)
    fin = torch.empty(num_steps, 3 * DEC_D)
    for s, t in enumerate(time_schedule(num_steps)):
        c = conditioning(ckpt, t, round_bf16)
        for i in range(layers):
            sa[s, i] = r(r(c @ r(ckpt["decoder_pre_attn_norm_mod_w"][i].float())) +
                         r(ckpt["decoder_pre_attn_norm_mod_b"][i].float()))
            sf[s, i] = r(r(c @ r(ckpt["decoder_pre_ffn_norm_mod_w"][i].float())) +
                         r(ckpt["decoder_pre_ffn_norm_mod_b"][i].float()))
        fin[s] = r(r(c @ r(ckpt["decoder_final_norm_mod_w"].float())) + r(ckpt["decoder_final_norm_mod_b"].float()))
    return sa, sf, fin


# ------------------------------------------------------------------ RoPE
def rope_table(positions, head_dim: int = DEC_HD, theta: float = 10000.0) -> torch.Tensor:
    """Interleaved [cos0, sin0, cos1, sin1, ...] rows, phases in fp64 (pipeline_rtx.py:480-487)."""
    inv_freq = 1.0 / (theta ** (np.arange(0, head_dim, 2, dtype=np.float64) / head_dim))
    phase = np.asarray(positions, dtype=np.float64)[:, None] * inv_freq[None, :]
    tab = np.stack([np.cos(phase), np.sin(phase)], axis=-1).reshape(len(positions), head_dim)
    return torch.from_numpy(tab.astype(np.float32))


def rope_adjacent_pairs(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x (S, heads, hd); pair (2i, 2i+1) rotated by (cos_i, sin_i)  -- the kernel's form."""
    cos, sin = table[:, 0::2], table[:, 1::2]
    x0, x1 = x[..., 0::2], x[..., 1::2]
    o0 = x0 * cos[:, None, :] - x1 * sin[:, None, :]
    o1 = x1 * cos[:, None, :] + x0 * sin[:, None, :]
    return torch.stack([o0, o1], dim=-1).reshape(x.shape)


def rope_rotate_half(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x (S, heads, hd); HF form: x * cos + rotate_half(x) * sin with cos/sin repeated over both halves."""
    cos, sin = table[:, 0::2], table[:, 1::2]
    cos = torch.cat([cos, cos], dim=-1)[:, None, :]
    sin = torch.cat([sin, sin], dim=-1)[:, None, :]
    a, b = x.chunk(2, dim=-1)
    return x * cos + torch.cat([-b, a], dim=-1) * sin


def interleave_qk_rows(w: torch.Tensor, num_heads: int) -> torch.Tensor:
    """(out, in) weight: move output row j of the first half of each head to 2j and of the second half to
    2j+1, so rotate-half on the original equals adjacent-pair rotation on the result."""
    out_dim, in_dim = w.shape
    hd = out_dim // num_heads
    return w.reshape(num_heads, 2, hd // 2, in_dim).permute(0, 2, 1, 3).reshape(out_dim, in_dim)


# ------------------------------------------------------------------ block
def ada_rms(x: torch.Tensor, style_row: torch.Tensor, eps: float = 1e-6):
    """normed * (1 + scale) + shift and the gate; no learned norm weight (Pi0.5 passes ones)."""
    scale, shift, gate = style_row.chunk(3, dim=-1)
    n = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return n * (1.0 + scale) + shift, gate


def gelu_tanh(x):
    return torch.nn.functional.gelu(x, approximate="tanh")


def attention(q, k, v, scale):
    """q (S, NH, hd), k / v (Skv, NKV, hd) -> (S, NH, hd); non-causal, query heads share the KV head."""
    g = q.shape[1] // k.shape[1]
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    s = torch.einsum("shd,khd->hsk", q, kk) * scale
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hsk,khd->shd", p, vv)


class Nvfp4Linears:
    """W4A4 NVFP4 stand-in for the four projections of every layer, restating the arithmetic of the NVFP4
    decoder (flash_rt/models/pi05/pipeline_thor.py:255-490; quantisers csrc/quantize/quantize_fp4_sfa.cu:63-109):
    weights quantised once (e2m1, 16-element blocks, RN-even E4M3 block scale) after division by an FP32
    global scale amax / (448 * 6); activations quantised per call, block scales only; the product is taken on
    the dequantised values in fp32 and rounded to bf16 as the GEMM kernel stores it."""

    def __init__(self, W: dict, layers: int, weight_global_scale: bool = True):
        from . import oracle as O
        self.O = O
        self.w = {}
        for name in ("decoder_attn_qkv_w", "decoder_attn_o_w", "decoder_ffn_gate_w", "decoder_ffn_up_w",
                     "decoder_ffn_down_w"):
            for i in range(layers):
                wt = W[name][i].float().t().contiguous()                       # (N, K)
                wb = O.f32_to_bf16_bits(wt.numpy())
                g = float(np.float32(np.abs(O.bf16_bits_to_f32(wb)).max()) / np.float32(448.0 * 6.0)) \
                    if weight_global_scale else 1.0
                g = max(g, 1e-30)
                p, sf = O.quantize_nvfp4(wb, 1, g)
                self.w[(name, i)] = torch.from_numpy(O.dequantize_nvfp4(p, sf, g)).t().contiguous()   # (K, N)

    def act(self, h: torch.Tensor, round_bf16: bool = True) -> torch.Tensor:
        O = self.O
        a = h.detach().float().numpy()
        src = O.f32_to_bf16_bits(a) if round_bf16 else np.ascontiguousarray(a, np.float32)
        p, sf = O.quantize_nvfp4(src, 1)
        return torch.from_numpy(O.dequantize_nvfp4(p, sf))

    def __call__(self, h_q: torch.Tensor, name: str, i: int) -> torch.Tensor:
        return (h_q @ self.w[(name, i)]).to(torch.bfloat16).float()


class Fp8Linears:
    """Per-tensor FP8 E4M3 stand-in for the four projections of every layer, restating the arithmetic of the
    reference's FP8 decoder (weights: flash_rt/frontends/torch/pi05_rtx.py:344-350, scale = max(amax / 448, 1e-12);
    activations: static per-site per-step scales, x * (1 / s) clamped to +-448 and rounded to E4M3,
    csrc/kernels/quantize.cu:61-75; product on the dequantised values in fp32, result rounded to bf16,
    csrc/gemm/gemm_runner.cu:263-272).  ``act_scale``: the (steps, layers, 4) table of the device model, sites in
    the order qkv, o, gate|up, down.

    ``raw_scale`` ((steps, layers, 2), optional): restates the device loop's DEFERRED ROW SCALE instead of the
    reference's quantisation point in front of QKV (layers >= 1) and gate|up: the operand is e4m3(x * (1 + scale) /
    raw_scale) and the projection's result is bf16(acc * rms + W . shift) -- the same sum, since a row's rms commutes
    with the projection: W . (rms * x * (1 + scale) + shift) = rms * (W . (x * (1 + scale))) + W . shift."""
    SITES = ("qkv", "o", "gu", "d")

    def __init__(self, W: dict, layers: int, act_scale, raw_scale=None):
        self.scale = torch.as_tensor(act_scale, dtype=torch.float32).cpu()
        self.raw_scale = None if raw_scale is None else torch.as_tensor(raw_scale, dtype=torch.float32).cpu()
        self.w = {}
        gate_up = {}
        for name in ("decoder_attn_qkv_w", "decoder_attn_o_w", "decoder_ffn_gate_w", "decoder_ffn_up_w",
                     "decoder_ffn_down_w"):
            for i in range(layers):
                gate_up[(name, i)] = W[name][i].to(torch.bfloat16).float()           # (K, N)
        for (name, i), w in gate_up.items():
            # gate and up are one fused tensor on the device: one scale for both
            if name in ("decoder_ffn_gate_w", "decoder_ffn_up_w"):
                amax = max(float(gate_up[("decoder_ffn_gate_w", i)].abs().max()),
                           float(gate_up[("decoder_ffn_up_w", i)].abs().max()))
            else:
                amax = float(w.abs().max())
            s = max(np.float32(amax) / np.float32(448.0), np.float32(1e-12))
            q = (w / torch.tensor(s)).clamp(-448, 448).to(torch.float8_e4m3fn).float()
            self.w[(name, i)] = q * torch.tensor(s)

    def act(self, h: torch.Tensor, step: int, i: int, site: str) -> torch.Tensor:
        s = self.scale[step, i, self.SITES.index(site)]
        inv = torch.tensor(1.0, dtype=torch.float32) / s
        return (h.float() * inv).clamp(-448, 448).to(torch.float8_e4m3fn).float() * s

    def __call__(self, h_q: torch.Tensor, name: str, i: int) -> torch.Tensor:
        return (h_q @ self.w[(name, i)]).to(torch.bfloat16).float()

    def deferred(self, x: torch.Tensor, style_row: torch.Tensor, step: int, i: int, which: int, names, eps=1e-6):
        """Projections ``names`` of adaRMS(x; style) with the row scale applied behind the product (see the class
        docstring); x is the bf16-rounded residual.  Returns one bf16-rounded result per name."""
        scale, shift, _ = style_row.chunk(3, dim=-1)
        rs = self.raw_scale[step, i, which]
        inv = torch.tensor(1.0, dtype=torch.float32) / rs
        u = ((x * (1.0 + scale)) * inv).clamp(-448, 448).to(torch.float8_e4m3fn).float() * rs
        rms = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        return [((u @ self.w[(n, i)]) * rms + shift @ self.w[(n, i)]).to(torch.bfloat16).float() for n in names]


def decoder_block_fp8(x, lin: "Fp8Linears", step: int, i: int, style_attn_row, style_ffn_row, prefix_k, prefix_v,
                      rope_tab):
    """The layer of ``decoder_block`` with FP8 projections and the device path's 16-bit rounding points (bf16
    residual stream, bf16 GEMM outputs, bf16 attention output quantised to FP8, GeGLU product quantised straight from
    fp32)."""
    S = x.shape[0]
    bf = lambda t: t.to(torch.bfloat16).float()  # noqa: E731
    h, gate_a = ada_rms(x, style_attn_row)
    if lin.raw_scale is not None and i > 0:
        (qkv,) = lin.deferred(x, style_attn_row, step, i, 0, ("decoder_attn_qkv_w",))
    else:
        qkv = lin(lin.act(h, step, i, "qkv"), "decoder_attn_qkv_w", i)
    q = qkv[:, :DEC_NH * DEC_HD].reshape(S, DEC_NH, DEC_HD)
    k = qkv[:, DEC_NH * DEC_HD:(DEC_NH + DEC_NKV) * DEC_HD].reshape(S, DEC_NKV, DEC_HD)
    v = qkv[:, (DEC_NH + DEC_NKV) * DEC_HD:].reshape(S, DEC_NKV, DEC_HD)
    q = bf(rope_adjacent_pairs(q, rope_tab))
    k = bf(rope_adjacent_pairs(k, rope_tab))
    keys = torch.cat([prefix_k.reshape(-1, DEC_NKV, DEC_HD).float(), k], dim=0)
    vals = torch.cat([prefix_v.reshape(-1, DEC_NKV, DEC_HD).float(), v], dim=0)
    a = bf(attention(q, keys, vals, DEC_HD ** -0.5).reshape(S, DEC_NH * DEC_HD))
    o = lin(lin.act(a, step, i, "o"), "decoder_attn_o_w", i)
    x1 = bf(x + o * gate_a)
    h2, gate_f = ada_rms(x1, style_ffn_row)
    if lin.raw_scale is not None:
        g_, u_ = lin.deferred(x1, style_ffn_row, step, i, 1, ("decoder_ffn_gate_w", "decoder_ffn_up_w"))
        hidden = gelu_tanh(g_) * u_
    else:
        h2q = lin.act(h2, step, i, "gu")
        hidden = gelu_tanh(lin(h2q, "decoder_ffn_gate_w", i)) * lin(h2q, "decoder_ffn_up_w", i)
    f = lin(lin.act(hidden, step, i, "d"), "decoder_ffn_down_w", i)
    return bf(x1 + f * gate_f)


def decoder_block_nvfp4(x, lin: "Nvfp4Linears", i: int, style_attn_row, style_ffn_row, prefix_k, prefix_v,
                        rope_tab):
    """The layer of ``decoder_block`` with NVFP4 projections and the device path's 16-bit rounding points
    (bf16 GEMM outputs, bf16 attention output, GeGLU product quantised straight from fp32)."""
    S = x.shape[0]
    bf = lambda t: t.to(torch.bfloat16).float()  # noqa: E731
    h, gate_a = ada_rms(x, style_attn_row)
    qkv = lin(lin.act(h), "decoder_attn_qkv_w", i)
    q = qkv[:, :DEC_NH * DEC_HD].reshape(S, DEC_NH, DEC_HD)
    k = qkv[:, DEC_NH * DEC_HD:(DEC_NH + DEC_NKV) * DEC_HD].reshape(S, DEC_NKV, DEC_HD)
    v = qkv[:, (DEC_NH + DEC_NKV) * DEC_HD:].reshape(S, DEC_NKV, DEC_HD)
    q = bf(rope_adjacent_pairs(q, rope_tab))
    k = bf(rope_adjacent_pairs(k, rope_tab))
    keys = torch.cat([prefix_k.reshape(-1, DEC_NKV, DEC_HD).float(), k], dim=0)
    vals = torch.cat([prefix_v.reshape(-1, DEC_NKV, DEC_HD).float(), v], dim=0)
    a = bf(attention(q, keys, vals, DEC_HD ** -0.5).reshape(S, DEC_NH * DEC_HD))
    o = lin(lin.act(a), "decoder_attn_o_w", i)
    x1 = bf(x + o * gate_a)
    h2, gate_f = ada_rms(x1, style_ffn_row)
    h2q = lin.act(h2)
    hidden = gelu_tanh(lin(h2q, "decoder_ffn_gate_w", i)) * lin(h2q, "decoder_ffn_up_w", i)
    f = lin(lin.act(hidden, round_bf16=False), "decoder_ffn_down_w", i)
    return bf(x1 + f * gate_f)


def decoder_block(x, W: dict, i: int, style_attn_row, style_ffn_row, prefix_k, prefix_v, rope_tab,
                  return_parts: bool = False):
    """One action-expert layer in fp32.  x (S, D); prefix_k / prefix_v (P, 256); returns the new x."""
    S = x.shape[0]
    h, gate_a = ada_rms(x, style_attn_row)
    qkv = h @ W["decoder_attn_qkv_w"][i].float()
    q = qkv[:, :DEC_NH * DEC_HD].reshape(S, DEC_NH, DEC_HD)
    k = qkv[:, DEC_NH * DEC_HD:(DEC_NH + DEC_NKV) * DEC_HD].reshape(S, DEC_NKV, DEC_HD)
    v = qkv[:, (DEC_NH + DEC_NKV) * DEC_HD:].reshape(S, DEC_NKV, DEC_HD)
    q = rope_adjacent_pairs(q, rope_tab)
    k = rope_adjacent_pairs(k, rope_tab)
    keys = torch.cat([prefix_k.reshape(-1, DEC_NKV, DEC_HD).float(), k], dim=0)
    vals = torch.cat([prefix_v.reshape(-1, DEC_NKV, DEC_HD).float(), v], dim=0)
    a = attention(q, keys, vals, DEC_HD ** -0.5).reshape(S, DEC_NH * DEC_HD)
    o = a @ W["decoder_attn_o_w"][i].float()
    x1 = x + o * gate_a
    h2, gate_f = ada_rms(x1, style_ffn_row)
    hidden = gelu_tanh(h2 @ W["decoder_ffn_gate_w"][i].float()) * (h2 @ W["decoder_ffn_up_w"][i].float())
    f = hidden @ W["decoder_ffn_down_w"][i].float()
    x2 = x1 + f * gate_f
    if return_parts:
        return x2, {"h": h, "q": q, "k": k, "attn": a, "x1": x1, "h2": h2, "hidden": hidden}
    return x2


def denoise_loop(noise, ckpt: dict, prefix_k, prefix_v, num_steps: int = 10, layers: int = DEC_L,
                 prefix_len: int | None = None, styles_bf16: bool = True, return_trajectory: bool = False,
                 nvfp4: "Nvfp4Linears | None" = None, fp8: "Fp8Linears | None" = None):
    """10-step Euler flow matching in fp32: x <- x + dt * v(x, t), dt = -1/N, t from 1 down.

    ``styles_bf16``: the conditioning tables are data the device path reads from a bf16 precompute
    (pi05_rtx.py:369-448), so by default they are rounded the same way here and the comparison isolates the
    loop itself.  ``nvfp4`` / ``fp8``: run the four projections of every layer through :class:`Nvfp4Linears` /
    :class:`Fp8Linears` (the like-for-like restatement of the quantised device path).
    Returns the final actions (S, 32) and, optionally, the list of states after each step.
    """
    W = ckpt
    S = noise.shape[0]
    P = prefix_k.shape[1] if prefix_len is None else prefix_len
    sa, sf, fin = styles(ckpt, num_steps, layers, round_bf16=styles_bf16)
    tab = rope_table(np.arange(P, P + S))
    if styles_bf16:
        tab = tab.to(torch.bfloat16).float()
    x_act = noise.float().clone()
    traj = []
    dt = -1.0 / num_steps
    for s in range(num_steps):
        x = x_act @ W["decoder_action_in_proj_w"].float() + W["decoder_action_in_proj_b"].float()
        for i in range(layers):
            if nvfp4 is not None:
                x = decoder_block_nvfp4(x, nvfp4, i, sa[s, i], sf[s, i], prefix_k[i, :P], prefix_v[i, :P], tab)
            elif fp8 is not None:
                x = decoder_block_fp8(x, fp8, s, i, sa[s, i], sf[s, i], prefix_k[i, :P], prefix_v[i, :P], tab)
            else:
                x = decoder_block(x, W, i, sa[s, i], sf[s, i], prefix_k[i, :P], prefix_v[i, :P], tab)
        h, _ = ada_rms(x, fin[s])
        v = h @ W["decoder_action_out_proj_w"].float() + W["decoder_action_out_proj_b"].float()
        x_act = x_act + dt * v
        traj.append(x_act.clone())
    return (x_act, traj) if return_trajectory else x_act


def denoise_loop_cfg(noise, ckpt: dict, cond_kv, uncond_kv, beta: float, num_steps: int = 10, layers: int = DEC_L,
                     styles_bf16: bool = True, return_trajectory: bool = False):
    """Classifier-free guidance (flash_rt/refs/pi05_cfg_reference.py:8-15, Eq. 13 of the paper it cites): every
    Euler step runs the velocity network twice -- with the conditioned and with the unconditioned prefix -- and
    advances with v = (1 - beta) * v_uncond + beta * v_cond.  cond_kv / uncond_kv = (prefix_k, prefix_v)."""
    W = ckpt
    S = noise.shape[0]
    P = cond_kv[0].shape[1]
    sa, sf, fin = styles(ckpt, num_steps, layers, round_bf16=styles_bf16)
    tab = rope_table(np.arange(P, P + S))
    if styles_bf16:
        tab = tab.to(torch.bfloat16).float()
    x_act = noise.float().clone()
    traj = []
    dt = -1.0 / num_steps

    def velocity(x_in, s, kv):
        x = x_in @ W["decoder_action_in_proj_w"].float() + W["decoder_action_in_proj_b"].float()
        for i in range(layers):
            x = decoder_block(x, W, i, sa[s, i], sf[s, i], kv[0][i, :P], kv[1][i, :P], tab)
        h, _ = ada_rms(x, fin[s])
        return h @ W["decoder_action_out_proj_w"].float() + W["decoder_action_out_proj_b"].float()

    for s in range(num_steps):
        v_c, v_u = velocity(x_act, s, cond_kv), velocity(x_act, s, uncond_kv)
        x_act = x_act + dt * (v_u + beta * (v_c - v_u))
        traj.append(x_act.clone())
    return (x_act, traj) if return_trajectory else x_act


# ------------------------------------------------------------------ HF state dict -> kernel-layout dictionary
def from_hf_state_dict(sd: dict, layers: int = DEC_L) -> dict:
    """Restates the decoder part of the reference's checkpoint conversion (pi05_rtx.py:216-283): projections
    transposed to [K, N], q / k output rows interleaved for adjacent-pair RoPE, q|k|v concatenated."""
    dp = "paligemma_with_expert.gemma_expert.model.layers"
    f = lambda k: sd[k].float()  # noqa: E731
    qkv, o, gate, up, down, amw, amb, fmw, fmb = ([] for _ in range(9))
    for i in range(layers):
        q = interleave_qk_rows(f(f"{dp}.{i}.self_attn.q_proj.weight"), DEC_NH)
        k = interleave_qk_rows(f(f"{dp}.{i}.self_attn.k_proj.weight"), DEC_NKV)
        v = f(f"{dp}.{i}.self_attn.v_proj.weight")
        qkv.append(torch.cat([q, k, v], dim=0).t())
        o.append(f(f"{dp}.{i}.self_attn.o_proj.weight").t())
        gate.append(f(f"{dp}.{i}.mlp.gate_proj.weight").t())
        up.append(f(f"{dp}.{i}.mlp.up_proj.weight").t())
        down.append(f(f"{dp}.{i}.mlp.down_proj.weight").t())
        amw.append(f(f"{dp}.{i}.input_layernorm.dense.weight").t())
        amb.append(f(f"{dp}.{i}.input_layernorm.dense.bias"))
        fmw.append(f(f"{dp}.{i}.post_attention_layernorm.dense.weight").t())
        fmb.append(f(f"{dp}.{i}.post_attention_layernorm.dense.bias"))
    st = torch.stack
    fin = "paligemma_with_expert.gemma_expert.model.norm.dense"
    return {
        "decoder_attn_qkv_w": st(qkv), "decoder_attn_o_w": st(o), "decoder_ffn_gate_w": st(gate),
        "decoder_ffn_up_w": st(up), "decoder_ffn_down_w": st(down),
        "decoder_pre_attn_norm_mod_w": st(amw), "decoder_pre_attn_norm_mod_b": st(amb),
        "decoder_pre_ffn_norm_mod_w": st(fmw), "decoder_pre_ffn_norm_mod_b": st(fmb),
        "decoder_final_norm_mod_w": f(f"{fin}.weight").t(), "decoder_final_norm_mod_b": f(f"{fin}.bias"),
        "decoder_time_mlp_in_w": f("time_mlp_in.weight").t(), "decoder_time_mlp_in_b": f("time_mlp_in.bias"),
        "decoder_time_mlp_out_w": f("time_mlp_out.weight").t(), "decoder_time_mlp_out_b": f("time_mlp_out.bias"),
        "decoder_action_in_proj_w": f("action_in_proj.weight").t(), "decoder_action_in_proj_b": f("action_in_proj.bias"),
        "decoder_action_out_proj_w": f("action_out_proj.weight").t(),
        "decoder_action_out_proj_b": f("action_out_proj.bias"),
    }
