"""NVFP4 (W4A4) variant of the Pi0.5 action-expert denoise loop on B200.

Host-side mirror of the reference's ``decoder_forward_fp4`` (flash_rt/models/pi05/pipeline_thor.py:255-490) and of
the weight preparation in ``flash_rt/executors/fp4_utils.py:62-99``: all four projections of every layer run as
block-scaled NVFP4 GEMMs (e2m1 elements, 16-element blocks, unsigned-E4M3 block scales), activations are
quantised on the fly by the kernels that produce them (no calibration pass), attention stays bf16.

What differs from the reference's composition:
  * any chunk length and a batch of independent chunks (the reference's kernels accept seq_len 10, batch 1 only);
  * the residual stream is bf16 (fp16 there) and the Euler state fp32;
  * weights carry an FP32 global scale amax / (448 * 6) per tensor, folded into the GEMM's alpha, so that their
    block scales stay in E4M3's normal range (the reference quantises weights with block scales only);
  * conditioning rows are read with stride 0 instead of one expanded copy per token;
  * for batch 1 the RoPE + split + KV append runs in the QKV GEMM's epilogue.
"""
from __future__ import annotations

import math

import torch

from . import flash_rt_fa2 as fa2
from . import flash_rt_fp4 as fp4
from . import flash_rt_kernels as fvk
from .pi05_decoder import ACTION_DIM, BF16, DEC_D, DEC_H, DEC_HD, DEC_NH, DEC_NKV, StepIO

QKV_N = (DEC_NH + 2 * DEC_NKV) * DEC_HD


class Nvfp4Weight:
    """One projection of one layer: packed e2m1 (N, K / 2), block scales, FP32 global scale (device scalar)."""

    def __init__(self, w_bf16: torch.Tensor, use_global_scale: bool = True):
        w = w_bf16.contiguous()
        self.N, self.K = w.shape
        dev = w.device
        self.packed = torch.empty(self.N, self.K // 2, dtype=torch.uint8, device=dev)
        self.sf = torch.zeros(fp4.sfa_size_bytes(self.N, self.K, True), dtype=torch.uint8, device=dev)
        g = float(w.float().abs().max()) / (448.0 * 6.0) if use_global_scale else 1.0
        self.g = float(torch.tensor(max(g, 1e-30), dtype=torch.float32))          # the fp32 value, as a host float
        self.global_scale = torch.tensor([self.g], dtype=torch.float32, device=dev)
        rc = fp4.quantize_fp4_dynamic_sfa_bf16_vec(w.data_ptr(), self.packed.data_ptr(), self.sf.data_ptr(), self.N,
                                                   self.K, True, 0, d_global_scale=self.global_scale.data_ptr())
        if rc != 0:
            raise RuntimeError(f"NVFP4 weight quantisation failed: status {rc}")
        torch.cuda.synchronize(dev)


class Pi05DecoderNvfp4Pipeline(StepIO):
    """Pointer-only composition of the NVFP4 denoise loop (what gets captured in the graph)."""

    def __init__(self, fe):
        self.fe = fe
        self.gemm = fvk.GemmRunner()
        dev = fe.device
        B, S = fe.batch, fe.chunk_size
        M = B * S
        self.M = M
        z = lambda *shape, dtype=BF16: torch.zeros(*shape, dtype=dtype, device=dev)  # noqa: E731
        sfb = lambda K: z(fp4.sfa_size_bytes(M, K), dtype=torch.uint8)               # noqa: E731  zero-filled once
        self._alloc_step_io()
        self.x = z(M, DEC_D)
        self.xn = z(M, DEC_D)
        self.qkv = z(M, QKV_N)
        self.q = z(M, DEC_NH * DEC_HD)
        self.attn = z(M, DEC_NH * DEC_HD)
        self.merged = z(M, 2 * DEC_H)
        self.act4, self.act4_sf = z(M, DEC_D // 2, dtype=torch.uint8), sfb(DEC_D)
        self.ctx4, self.ctx4_sf = z(M, DEC_NH * DEC_HD // 2, dtype=torch.uint8), sfb(DEC_NH * DEC_HD)
        self.hid4, self.hid4_sf = z(M, DEC_H // 2, dtype=torch.uint8), sfb(DEC_H)
        self.ones = torch.ones(DEC_D, dtype=BF16, device=dev)
        self.attn_splits = fe.attn_splits
        self.o_accum = z(self.attn_splits, B, S, DEC_NH, DEC_HD, dtype=torch.float32)
        self.lse_accum = z(self.attn_splits, B, DEC_NH, S, dtype=torch.float32)
        self.attn_counters = z(2 * B * ((S * DEC_NH + 127) // 128), dtype=torch.int32)
        self.calibrated = True            # dynamic block scales: nothing to calibrate

    def _style(self, which, step, layer=None):
        fe = self.fe
        t = {"attn": fe.style_attn, "ffn": fe.style_ffn, "final": fe.style_final}[which]
        row = t[step] if layer is None else t[step, layer]
        return row.data_ptr()

    def _gemm(self, a4, a_sf, w: Nvfp4Weight, out, stream, pdl):
        rc = fp4.cutlass_fp4_gemm_variant(0, a4.data_ptr(), a_sf.data_ptr(), w.packed.data_ptr(), w.sf.data_ptr(),
                                          out.data_ptr(), self.M, w.N, w.K, w.g, 0.0, stream, pdl=pdl)
        if rc != 0:
            raise fvk.KernelError(f"NVFP4 GEMM ({self.M}, {w.N}, {w.K}) failed: status {rc}")

    def _norm(self, delta, gate_from, style_kind, step, layer, stream, pdl):
        """(x += delta * gate) ; adaRMS(style) -> NVFP4 activations of the next projection."""
        style = self._style(style_kind, step, layer)
        gate = (self._style(*gate_from) + 2 * DEC_D * 2) if gate_from else None
        fvk.call("frt_b200_norm_nvfp4", self.x.data_ptr(), delta.data_ptr() if delta is not None else None, gate, 0,
                 None, style, 0, self.act4.data_ptr(), self.act4_sf.data_ptr(), None, self.M, DEC_D, 1e-6, fp4.FAMILY,
                 1 if pdl else 0, stream)

    def _attention(self, layer, stream, pdl):
        self._attend(layer, stream, pdl)

    def transformer_decoder(self, stream: int = 0, calibrate: bool = False, step_hook=None) -> None:
        """Run the N-step denoise on ``self.noise`` in place (pipeline_thor.py:355-490)."""
        fe, g = self.fe, self.gemm
        B, S, L, M = fe.batch, fe.chunk_size, fe.layers, self.M
        pdl = fe.use_pdl
        for step in range(fe.num_steps):
            self._step_in(stream, pdl)
            for i in range(L):
                if i == 0:
                    self._norm(None, None, "attn", step, i, stream, pdl)
                w = fe.w4[i]
                if B == 1 and fe.fuse_epilogues:
                    kp, vp, dp = self._kv_dst(i, 0)
                    rc = fp4.cutlass_fp4_gemm_rope_split(
                        self.act4.data_ptr(), self.act4_sf.data_ptr(), w["qkv"].packed.data_ptr(),
                        w["qkv"].sf.data_ptr(), fe.rope.data_ptr(), self.q.data_ptr(), kp, vp, M,
                        DEC_D, DEC_NH * DEC_HD, DEC_NKV * DEC_HD, DEC_NKV * DEC_HD, DEC_HD, devpos=dp,
                        alpha=w["qkv"].g, stream=stream, pdl=pdl)
                    if rc != 0:
                        raise fvk.KernelError(f"NVFP4 QKV GEMM failed: status {rc}")
                else:
                    self._gemm(self.act4, self.act4_sf, w["qkv"], self.qkv, stream, pdl)
                    for b in range(B):
                        self._split_rope(i, b, self.qkv[b * S:], self.q[b * S:], S, stream, pdl and b == 0)
                self._attention(i, stream, pdl)
                rc = fp4.quantize_fp4_dynamic_sfa_bf16_vec(self.attn.data_ptr(), self.ctx4.data_ptr(),
                                                           self.ctx4_sf.data_ptr(), M, DEC_NH * DEC_HD, False, stream,
                                                           pdl=pdl)
                if rc != 0:
                    raise fvk.KernelError(f"NVFP4 activation quantisation failed: status {rc}")
                self._gemm(self.ctx4, self.ctx4_sf, w["o"], self.xn, stream, pdl)
                self._norm(self.xn, ("attn", step, i), "ffn", step, i, stream, pdl)
                self._gemm(self.act4, self.act4_sf, w["gu"], self.merged, stream, pdl)
                rc = fp4.gate_geglu_fp4_sfa_vec_bf16(self.merged.data_ptr(), self.hid4.data_ptr(),
                                                     self.hid4_sf.data_ptr(), M, DEC_H, stream, pdl=pdl)
                if rc != 0:
                    raise fvk.KernelError(f"NVFP4 GeGLU failed: status {rc}")
                self._gemm(self.hid4, self.hid4_sf, w["d"], self.xn, stream, pdl)
                if i < L - 1:
                    self._norm(self.xn, ("ffn", step, i), "attn", step, i + 1, stream, pdl)
                else:
                    fvk.call("frt_b200_gate_mul_residual", self.x.data_ptr(), self.xn.data_ptr(),
                             self._style("ffn", step, i) + 2 * DEC_D * 2, 0, M, DEC_D, 1 if pdl else 0, stream)
            fvk.ada_rms_norm_style(self.x.data_ptr(), self.ones.data_ptr(), self._style("final", step),
                                   self.xn.data_ptr(), 0, M, DEC_D, 1e-6, stream, pdl=pdl, style_stride=0)
            self._step_out(stream, pdl)
            if step_hook is not None:
                step_hook(step)

    def launches_per_layer(self) -> int:
        fe = self.fe
        fused = fe.batch == 1 and fe.fuse_epilogues
        # qkv gemm (+ split/rope per batch element), attention, quantise, o gemm, norm, gate|up gemm, geglu, down gemm, norm
        return (1 if fused else 1 + fe.batch) + 8
