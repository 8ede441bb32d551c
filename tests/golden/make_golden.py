"""Generates ``tests/golden/cfg0_block.npz``: outputs of the REFERENCE's own plain-torch ground-truth
functions (``flash_rt/structures/catalog/*/reference.py``) for the CPU-runnable configuration 0 — one
action-expert block, batch 1, 50 tokens, width 1024, 8 query heads x 256 with one shared KV head over a
768-token prefix plus the 50 fresh tokens, rotate-half RoPE (theta 10000), GeGLU 1024-4096-1024, adaRMS
conditioning from the time embedding at t = 0.5; weights ~ N(0, 0.02), activations and prefix KV ~ N(0, 1).

Run where the reference tree is available:

    PYTHONPATH=<reference root> python tests/golden/make_golden.py

The reference works in the Hugging Face layout (rotate-half RoPE on un-permuted q/k projections); the device
path works on row-interleaved projections with adjacent-pair RoPE.  The seeded inputs are defined in the
device layout (``oracle.block_ref.synthetic_*``) and converted to the HF layout here by the inverse
permutation, so that both compute the same function.  Only outputs are stored (fp32); inputs are regenerated
from their seeds by the tests, and a checksum of each input guards the regeneration.
"""
import os
import sys
import zlib

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from flash_rt.structures.catalog.adaln_producer.reference import adaln_producer_ref  # noqa: E402
from flash_rt.structures.catalog.attention_core.reference import attention_core_ref  # noqa: E402
from flash_rt.structures.catalog.decoder_block.reference import decoder_block_ref  # noqa: E402
from flash_rt.structures.catalog.decoder_ffn.reference import decoder_ffn_ref  # noqa: E402
from flash_rt.structures.catalog.linear_proj.reference import linear_proj_ref  # noqa: E402
from flash_rt.structures.catalog.qkv_rope.reference import qkv_rope_ref  # noqa: E402

from oracle import block_ref as R  # noqa: E402  (seeded input definitions only)


def deinterleave_rows(w_il: torch.Tensor, heads: int) -> torch.Tensor:
    """Inverse of the q/k row interleave: device-layout (out, in) weight -> HF layout."""
    out_dim, in_dim = w_il.shape
    hd = out_dim // heads
    return w_il.reshape(heads, hd // 2, 2, in_dim).permute(0, 2, 1, 3).reshape(out_dim, in_dim)


def deinterleave_last(x_il: torch.Tensor) -> torch.Tensor:
    """(..., hd) device layout (pairs adjacent) -> HF layout (first halves | second halves)."""
    hd = x_il.shape[-1]
    return x_il.reshape(*x_il.shape[:-1], hd // 2, 2).transpose(-1, -2).reshape(*x_il.shape[:-1], hd)


def crc(t: torch.Tensor) -> int:
    return zlib.crc32(t.contiguous().numpy().tobytes())


def main():
    torch.manual_seed(0)
    S, P = 50, 768
    ck = R.synthetic_checkpoint(seed=0, layers=1)
    pk, pv = R.synthetic_prefix_kv(seed=1, layers=1, prefix_len=P)
    x = torch.randn(S, R.DEC_D, generator=torch.Generator().manual_seed(2))
    cond = R.conditioning(ck, 0.5)[None, :]                      # (1, 1024), fp32

    Wqkv = ck["decoder_attn_qkv_w"][0]                            # (D, 2560), device layout [K, N]
    q_il, k_il, v_w = Wqkv[:, :2048].t(), Wqkv[:, 2048:2304].t(), Wqkv[:, 2304:].t()
    W_hf = torch.cat([deinterleave_rows(q_il, 8), deinterleave_rows(k_il, 1), v_w], dim=0).t().contiguous()
    pk_hf = deinterleave_last(pk[0].reshape(P, 1, 256))
    tab = R.rope_table(np.arange(P, P + S))
    cos, sin = tab[:, 0::2][None], tab[:, 1::2][None]            # (1, S, 128)
    parts = {}

    def norm_in(xx, c):
        return adaln_producer_ref(xx, c, ck["decoder_pre_attn_norm_mod_w"][0], ck["decoder_pre_attn_norm_mod_b"][0])

    def norm_out(xx, c):
        return adaln_producer_ref(xx, c, ck["decoder_pre_ffn_norm_mod_w"][0], ck["decoder_pre_ffn_norm_mod_b"][0])

    def attn(h):
        parts["h"] = h
        qkv = linear_proj_ref(h, W_hf)
        q, k, v = qkv_rope_ref(qkv[None], torch.zeros(qkv.shape[-1]), cos, sin, q_heads=8, kv_heads=1, head_dim=256)
        parts["q_hf"], parts["k_hf"] = q[0], k[0]
        keys = torch.cat([pk_hf[None], k], dim=1)                 # (1, P+S, 1, 256)
        vals = torch.cat([pv[0].reshape(1, P, 1, 256), v], dim=1)
        o = attention_core_ref(q.transpose(1, 2), keys.transpose(1, 2), vals.transpose(1, 2), None, scale=256 ** -0.5)
        parts["attn"] = o[0].reshape(S, 2048)
        return linear_proj_ref(parts["attn"], ck["decoder_attn_o_w"][0])

    def ffn(h):
        parts["h2"] = h
        g = linear_proj_ref(h, ck["decoder_ffn_gate_w"][0])
        u = linear_proj_ref(h, ck["decoder_ffn_up_w"][0])
        return linear_proj_ref(torch.nn.functional.gelu(g, approximate="tanh") * u, ck["decoder_ffn_down_w"][0])

    out = decoder_block_ref(x, cond, norm_in=norm_in, attn=attn, norm_out=norm_out, ffn=ffn)

    # second half once more through the reference's fused FFN ground truth (norm + GeGLU + gated residual)
    h1, gate_a = norm_in(x, cond)
    x1 = x + attn(h1) * gate_a
    style_f = cond @ ck["decoder_pre_ffn_norm_mod_w"][0] + ck["decoder_pre_ffn_norm_mod_b"][0]
    sc, sh, gt = style_f.chunk(3, dim=-1)
    out_ffn = decoder_ffn_ref(x1, torch.zeros(R.DEC_D), ck["decoder_ffn_gate_w"][0], ck["decoder_ffn_up_w"][0],
                              ck["decoder_ffn_down_w"][0], activation="gelu", norm_weight_mode="offset",
                              cond_scale=sc, cond_shift=sh, cond_gate=gt)

    np.savez_compressed(
        os.path.join(HERE, "cfg0_block.npz"),
        out=out.numpy(), out_via_decoder_ffn_ref=out_ffn.numpy(), x1=x1.numpy(),
        h=parts["h"].numpy(), h2=parts["h2"].numpy(), attn=parts["attn"].numpy(),
        q_hf=parts["q_hf"].numpy(), k_hf=parts["k_hf"].numpy(),
        crc=np.array([crc(x), crc(cond), crc(Wqkv), crc(pk), crc(pv)], dtype=np.int64),
    )
    print("wrote cfg0_block.npz; |out| rms", float(out.pow(2).mean().sqrt()),
          "max diff between the two reference routes", float((out - out_ffn).abs().max()))


if __name__ == "__main__":
    main()
