"""Prefix producer on B200: the Gemma-2B encoder layers that turn the prompt / image embeddings into the
per-layer prefix keys and values the action expert attends to.

Host-side mirror of the reference's ``Pi05Pipeline._encoder_layer`` / ``transformer_encoder``
(flash_rt/models/pi05/pipeline_rtx.py:1209-1435, fused-FP8 branch) and of the encoder part of the checkpoint
conversion (flash_rt/frontends/torch/pi05_rtx.py:178-214: q / k rows interleaved for adjacent-pair RoPE, the
``1 + w`` of both RMSNorms folded into the following projections in fp32).  It is the step in front of the denoise
path and reuses its kernels unchanged, at M = prefix length where the GEMMs turn compute-bound:

  B1  rms_norm_fp8 (first layer) / residual_add_rms_norm_fp8 -> QKV GEMM -> qkv_split_rope (K, V straight into the
      layer's cache rows; K carries its RoPE)
  B2  bidirectional attention over the prefix (8 query heads, one KV head, head_dim 256), FP8 copy fused
  B3  attention out-projection
  B4  residual_add_rms_norm_fp8 -> gate|up GEMM -> GeGLU -> FP8
  B5  down projection (its residual add is fused into the next layer's B1)
The last layer stops after B1: the encoder's product is the KV cache, not its hidden state.
The vision tower and the token embedding are outside this module: ``embeds`` (seq, 2048) is the input.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import flash_rt_fa2 as fa2
from . import flash_rt_kernels as fvk
from .weight_loader import (DictSource, FlatCat, FoldNorm, FusedGateUp, FusedQKV, Item, LayerBlock, ModelWeightSpec,
                            Quant, SafetensorsSource, WeightLoader)

ENC_D, ENC_H, ENC_NH, ENC_NKV, ENC_HD, ENC_L = 2048, 16384, 8, 1, 256, 18
QKV_N = (ENC_NH + 2 * ENC_NKV) * ENC_HD
BF16 = torch.bfloat16
SITES = ("qkv", "o", "gu", "d")
EP = "paligemma_with_expert.paligemma.model.language_model.layers.{i}"


def build_encoder_spec(layers: int = ENC_L) -> ModelWeightSpec:
    blk = LayerBlock(prefix_fmt="", num_layers=layers, name="encoder", items=[
        Item("qkv_w", FoldNorm(FusedQKV(q=f"{EP}.self_attn.q_proj.weight", k=f"{EP}.self_attn.k_proj.weight",
                                        v=f"{EP}.self_attn.v_proj.weight", interleave_q_heads=ENC_NH,
                                        interleave_k_heads=ENC_NKV), norm=f"{EP}.input_layernorm.weight"),
             [Quant()], FlatCat("w_qkv"), scale_into="ws_qkv"),
        Item("o_w", f"{EP}.self_attn.o_proj.weight", [Quant()], FlatCat("w_o"), scale_into="ws_o"),
        Item("gu_w", FoldNorm(FusedGateUp(gate=f"{EP}.mlp.gate_proj.weight", up=f"{EP}.mlp.up_proj.weight"),
                              norm=f"{EP}.post_attention_layernorm.weight"),
             [Quant()], FlatCat("w_gu"), scale_into="ws_gu"),
        Item("d_w", f"{EP}.mlp.down_proj.weight", [Quant()], FlatCat("w_d"), scale_into="ws_d"),
    ])
    return ModelWeightSpec(framework="torch", blocks=[blk], dims={"D": ENC_D, "H": ENC_H, "L": layers})


def synthetic_encoder_state_dict(seed: int = 0, layers: int = ENC_L) -> dict:
    """Random-init Gemma-2B encoder layers under the HF key names (matrices ~ N(0, 0.02), norm weights ~ N(0, 0.1))."""
    g = torch.Generator().manual_seed(seed)
    w = lambda *shape, s=0.02: torch.randn(*shape, generator=g) * s  # noqa: E731
    sd = {}
    for i in range(layers):
        p = EP.format(i=i)
        sd[f"{p}.self_attn.q_proj.weight"] = w(ENC_NH * ENC_HD, ENC_D)
        sd[f"{p}.self_attn.k_proj.weight"] = w(ENC_NKV * ENC_HD, ENC_D)
        sd[f"{p}.self_attn.v_proj.weight"] = w(ENC_NKV * ENC_HD, ENC_D)
        sd[f"{p}.self_attn.o_proj.weight"] = w(ENC_D, ENC_NH * ENC_HD)
        sd[f"{p}.mlp.gate_proj.weight"] = w(ENC_H, ENC_D)
        sd[f"{p}.mlp.up_proj.weight"] = w(ENC_H, ENC_D)
        sd[f"{p}.mlp.down_proj.weight"] = w(ENC_D, ENC_H)
        sd[f"{p}.input_layernorm.weight"] = w(ENC_D, s=0.1)
        sd[f"{p}.post_attention_layernorm.weight"] = w(ENC_D, s=0.1)
    return sd


def rope_rows(count: int) -> torch.Tensor:
    """bf16 (count, 256) rows [cos0, sin0, ...] for positions 0 .. count-1, theta 10000 (pipeline_rtx.py:473-505)."""
    inv_freq = 1.0 / (10000 ** (np.arange(0, ENC_HD, 2, dtype=np.float64) / ENC_HD))
    phase = np.arange(count, dtype=np.float64)[:, None] * inv_freq[None, :]
    tab = np.stack([np.cos(phase), np.sin(phase)], axis=-1).reshape(count, ENC_HD)
    return torch.from_numpy(tab.astype(np.float32)).to(BF16)


class Pi05PrefixEncoderB200:
    def __init__(self, checkpoint, *, layers: int = ENC_L, max_seq: int = 768, device: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("flashrt_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.layers, self.max_seq = layers, max_seq
        if isinstance(checkpoint, dict):
            source = DictSource(checkpoint)
        elif isinstance(checkpoint, str) and checkpoint.startswith("synthetic"):
            seed = int(checkpoint.split(":")[1]) if ":" in checkpoint else 0
            source = DictSource(synthetic_encoder_state_dict(seed, layers))
        else:
            source = SafetensorsSource(str(checkpoint))
        self.WEIGHT_SPEC = build_encoder_spec(layers)
        WeightLoader(source, target=self, spec=self.WEIGHT_SPEC).run()
        dev = self.device
        for n in ("w_qkv", "w_o", "w_gu", "w_d"):
            setattr(self, n, getattr(self, n).view(torch.uint8).to(dev))
        for n in ("ws_qkv", "ws_o", "ws_gu", "ws_d"):
            setattr(self, n + "_t", torch.tensor(getattr(self, n), dtype=torch.float32, device=dev))
        S = max_seq
        z = lambda *shape, dtype=BF16: torch.zeros(*shape, dtype=dtype, device=dev)  # noqa: E731
        self.x, self.xn = z(S, ENC_D), z(S, ENC_D)
        self.h_bf16 = z(S, ENC_D)
        self.qkv, self.q, self.attn = z(S, QKV_N), z(S, ENC_NH * ENC_HD), z(S, ENC_NH * ENC_HD)
        self.merged, self.hidden = z(S, 2 * ENC_H), z(S, ENC_H)
        self.act8, self.attn8 = z(S, ENC_D, dtype=torch.uint8), z(S, ENC_NH * ENC_HD, dtype=torch.uint8)
        self.hid8 = z(S, ENC_H, dtype=torch.uint8)
        self.ones = torch.ones(ENC_D, dtype=BF16, device=dev)
        self.rope = rope_rows(S).to(dev)
        self.act_scale = torch.ones(layers, len(SITES), dtype=torch.float32, device=dev)
        self.scratch_scale = torch.zeros(1, dtype=torch.float32, device=dev)
        self.gemm = fvk.GemmRunner()
        self.stream = torch.cuda.Stream(device=dev)
        self.calibrated = False

    # ------------------------------------------------------------------
    def _sp(self, layer, site):
        return self.act_scale[layer, SITES.index(site)].data_ptr()

    def _dyn_quant(self, src, dst8, layer, site, st):
        fvk.quantize_fp8_device(src.data_ptr(), dst8.data_ptr(), self.scratch_scale.data_ptr(), src.numel(), st)
        fvk.fp8_accumulate_scale_max(self.scratch_scale.data_ptr(), self._sp(layer, site), st)
        fvk.quantize_fp8_static(src.data_ptr(), dst8.data_ptr(), self._sp(layer, site), src.numel(), st)

    def _norm(self, seq, delta, layer, site, st, calibrate):
        """(x += delta) ; RMSNorm with unit weight -> FP8 input of ``site``."""
        if not calibrate:
            fvk.call("frt_b200_norm_fp8", self.x.data_ptr(), delta.data_ptr() if delta is not None else None, None, 0,
                     self.ones.data_ptr(), None, 0, self.act8.data_ptr(), None, seq, ENC_D, 1e-6,
                     self._sp(layer, site), 0, st)
            return
        fvk.call("frt_b200_norm_bf16", self.x.data_ptr(), delta.data_ptr() if delta is not None else None, None, 0,
                 self.ones.data_ptr(), None, 0, self.h_bf16.data_ptr(), None, seq, ENC_D, 1e-6, 0, st)
        self._dyn_quant(self.h_bf16[:seq], self.act8[:seq], layer, site, st)

    def _gemm(self, a8, w8, ws, out, M, N, K, sp, st):
        self.gemm.fp8_nt_dev(a8.data_ptr(), w8.data_ptr(), out.data_ptr(), M, N, K, sp, ws.data_ptr(), st)

    def transformer_encoder(self, seq: int, k_out: torch.Tensor, v_out: torch.Tensor, st: int, calibrate: bool):
        """Runs the layers on ``self.x[:seq]``; layer i writes rows [0, seq) of k_out[i] / v_out[i] ((rows, 256))."""
        L = self.layers
        qs = (seq * ENC_NH * ENC_HD, ENC_NH * ENC_HD, ENC_HD)
        for i in range(L):
            self._norm(seq, self.xn if i > 0 else None, i, "qkv", st, calibrate)
            self._gemm(self.act8, self.w_qkv[i], self.ws_qkv_t[i], self.qkv, seq, QKV_N, ENC_D, self._sp(i, "qkv"), st)
            fvk.qkv_split_rope(self.qkv.data_ptr(), self.rope.data_ptr(), self.q.data_ptr(), k_out[i].data_ptr(),
                               v_out[i].data_ptr(), seq, ENC_NH * ENC_HD, ENC_NKV * ENC_HD, ENC_NKV * ENC_HD, ENC_HD, st)
            if i == L - 1:
                return
            ks = (k_out[i].shape[0] * ENC_HD, ENC_HD, ENC_HD)
            if calibrate:
                fa2.fwd_bf16(self.q.data_ptr(), k_out[i].data_ptr(), v_out[i].data_ptr(), self.attn.data_ptr(), 0, 0, 0,
                             1, seq, seq, ENC_NH, ENC_NKV, ENC_HD, qs, ks, ks, qs, 1.0 / math.sqrt(ENC_HD), 0, st)
                self._dyn_quant(self.attn[:seq], self.attn8[:seq], i, "o", st)
            else:
                fa2.fwd_bf16(self.q.data_ptr(), k_out[i].data_ptr(), v_out[i].data_ptr(), self.attn.data_ptr(), 0, 0, 0,
                             1, seq, seq, ENC_NH, ENC_NKV, ENC_HD, qs, ks, ks, qs, 1.0 / math.sqrt(ENC_HD), 0, st,
                             out_fp8=self.attn8.data_ptr(), out_scale=self._sp(i, "o"))
            self._gemm(self.attn8, self.w_o[i], self.ws_o_t[i], self.xn, seq, ENC_D, ENC_NH * ENC_HD, self._sp(i, "o"), st)
            self._norm(seq, self.xn, i, "gu", st, calibrate)
            self._gemm(self.act8, self.w_gu[i], self.ws_gu_t[i], self.merged, seq, 2 * ENC_H, ENC_D, self._sp(i, "gu"), st)
            if calibrate:
                fvk.gate_geglu_merged(self.merged.data_ptr(), self.hidden.data_ptr(), seq, ENC_H, st)
                self._dyn_quant(self.hidden[:seq], self.hid8[:seq], i, "d", st)
            else:
                fvk.gate_geglu_merged_fp8(self.merged.data_ptr(), self.hid8.data_ptr(), seq, ENC_H, self._sp(i, "d"), st)
            self._gemm(self.hid8, self.w_d[i], self.ws_d_t[i], self.xn, seq, ENC_D, ENC_H, self._sp(i, "d"), st)

    # ------------------------------------------------------------------
    def _check(self, embeds, k_out, v_out):
        seq = embeds.shape[0]
        if embeds.shape != (seq, ENC_D) or not 0 < seq <= self.max_seq:
            raise ValueError(f"embeds must be (seq <= {self.max_seq}, {ENC_D}), got {tuple(embeds.shape)}")
        for t in (k_out, v_out):
            if t.dim() != 3 or t.shape[0] != self.layers or t.shape[1] < seq or t.shape[2] != ENC_HD or t.dtype != BF16 \
                    or not t.is_cuda or not t[0].is_contiguous():
                raise ValueError("k_out / v_out must be bf16 CUDA tensors (layers, rows >= seq, 256) with contiguous rows")
        return seq

    def calibrate(self, embeds_list) -> None:
        """Static per-site activation scales: the max over the dynamic scales of the given sample prefixes."""
        k = torch.zeros(self.layers, self.max_seq, ENC_HD, dtype=BF16, device=self.device)
        v = torch.zeros_like(k)
        per = []
        with torch.cuda.stream(self.stream):
            for e in embeds_list:
                seq = self._check(e, k, v)
                self.act_scale.zero_()
                self.x[:seq].copy_(e.to(self.device, BF16))
                self.transformer_encoder(seq, k, v, self.stream.cuda_stream, True)
                self.stream.synchronize()
                per.append(self.act_scale.clone())
            self.act_scale.copy_(torch.stack(per).max(0).values.clamp_(min=1e-12))
        self.stream.synchronize()
        if fvk.tensor_core_status() != 0:
            raise RuntimeError("a tensor-core kernel reported a timed-out wait during calibration")
        self.calibrated = True

    def encode(self, embeds: torch.Tensor, k_out: torch.Tensor, v_out: torch.Tensor) -> int:
        """embeds (seq, 2048) -> rows [0, seq) of k_out[i], v_out[i] for every layer (K with its RoPE, in the
        interleaved feature order the decoder's Q uses).  Returns seq."""
        if not self.calibrated:
            raise RuntimeError("calibrate() first: the encoder runs with static activation scales")
        seq = self._check(embeds, k_out, v_out)
        with torch.cuda.stream(self.stream):
            self.x[:seq].copy_(embeds.to(self.device, BF16), non_blocking=True)
            self.transformer_encoder(seq, k_out, v_out, self.stream.cuda_stream, False)
        self.stream.synchronize()
        return seq
