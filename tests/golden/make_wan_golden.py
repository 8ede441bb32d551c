"""Generates ``wan_parts.npz``: outputs of the REFERENCE's own plain-torch ground-truth functions
(``flash_rt/structures/catalog/*/reference.py``) for the building blocks of the video-DiT block restated in
``oracle/wan_ref.py``: q/k RMSNorm over the whole projection + interleaved (complex-pair) RoPE, affine LayerNorm,
modulated affine-free LayerNorm -> q/k/v projections, LayerNorm -> fc1 -> GELU(tanh) -> fc2 -> residual.

Run where the reference tree is available:

    PYTHONPATH=<reference root> python tests/golden/make_wan_golden.py

Inputs are regenerated from the seed by the test (``inputs()`` below is imported there); only outputs are stored.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))

B, L, D, H, FFN = 2, 40, 256, 4, 512
HD = D // H


def inputs():
    g = torch.Generator().manual_seed(77)
    r = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc  # noqa: E731
    ang = torch.rand(L, HD // 2, generator=g) * 6.283
    return dict(
        x=r(B, L, D), q=r(B, L, H, HD), k=r(B, L, H, HD), v=r(B, L, H, HD),
        wq_norm=1.0 + r(D, sc=0.1), wk_norm=1.0 + r(D, sc=0.1), cos=torch.cos(ang), sin=torch.sin(ang),
        ln_w=1.0 + r(D, sc=0.1), ln_b=r(D, sc=0.1),
        cond=r(B, D), w_cond=r(2 * D, D, sc=0.05), b_cond=r(2 * D, sc=0.05),
        w_q=r(D, D, sc=0.05), b_q=r(D, sc=0.05), w_k=r(D, D, sc=0.05), b_k=r(D, sc=0.05),
        w_v=r(D, D, sc=0.05), b_v=r(D, sc=0.05),
        w_fc1=r(FFN, D, sc=0.05), b_fc1=r(FFN, sc=0.05), w_fc2=r(D, FFN, sc=0.05), b_fc2=r(D, sc=0.05))


def main():
    if "FLASHRT_REFERENCE" not in os.environ:
        raise SystemExit("set FLASHRT_REFERENCE=<path to a FlashRT checkout>")
    sys.path.insert(0, os.environ["FLASHRT_REFERENCE"])
    from flash_rt.structures.catalog.modnorm_qkv_chain.reference import modnorm_qkv_chain_ref
    from flash_rt.structures.catalog.norm_fused.reference import norm_fused_ref
    from flash_rt.structures.catalog.qk_norm_rope.reference import qk_norm_rope_ref
    from flash_rt.structures.catalog.vision_ffn.reference import vision_ffn_ref
    i = inputs()
    out = {}
    qo, ko, vo = qk_norm_rope_ref(i["q"], i["k"], i["v"], i["wq_norm"], i["wk_norm"], i["cos"], i["sin"], eps=1e-6,
                                  variant={"rope_layout": "interleaved", "normalization_scope": "projection",
                                           "norm_weight_mode": "direct"})
    out["qk_norm_rope_q"], out["qk_norm_rope_k"] = qo.numpy(), ko.numpy()
    out["norm_fused"] = norm_fused_ref(i["x"], i["ln_w"], i["ln_b"], eps=1e-6).numpy()
    q, k, v = modnorm_qkv_chain_ref(i["x"], i["cond"], i["w_cond"], i["b_cond"], i["w_q"], i["b_q"], i["w_k"],
                                    i["b_k"], i["w_v"], i["b_v"], eps=1e-6)
    out["modnorm_q"], out["modnorm_k"], out["modnorm_v"] = q.numpy(), k.numpy(), v.numpy()
    out["vision_ffn"] = vision_ffn_ref(i["x"], None, None, i["w_fc1"], i["b_fc1"], i["w_fc2"], i["b_fc2"],
                                       eps=1e-6).numpy()
    out["silu_cond_affine"] = F.linear(F.silu(i["cond"]), i["w_cond"], i["b_cond"]).numpy()
    np.savez_compressed(os.path.join(HERE, "wan_parts.npz"), **out)
    print("wrote wan_parts.npz:", ", ".join(f"{k} {v.shape}" for k, v in out.items()))


if __name__ == "__main__":
    main()
