"""Pi0.5 action-expert denoise loop on B200: the frontend (weights -> FP8, conditioning tables, calibration,
graph capture, ``infer``) and the pointer-only kernel composition it captures.

Host-side mirror of the reference's
  * ``Pi05TorchFrontendRtx``  (flash_rt/frontends/torch/pi05_rtx.py:456-1614): weight conversion, FP8 weight
    quantisation (:344-350, :718-762), style precompute (:369-448), calibration (:1312-1463), ``infer`` (:1547-1614)
  * ``Pi05Pipeline.transformer_decoder`` / ``_decoder_layer`` / ``record_infer_graph`` / ``forward_decode_only``
    (flash_rt/models/pi05/pipeline_rtx.py:1451-1749, 1980-2049, 2175-2196)
restricted to the decoder: the prefix keys / values that the vision tower and the Gemma-2B encoder would leave
in the per-layer KV cache are an input (``set_prefix``).

What differs from the reference's composition (same arithmetic, fewer launches and bytes):
  * conditioning rows are stored once per (step, layer) and read with row stride 0 instead of being expanded to
    one copy per action token; the gate of the next residual is read straight from the style row;
  * the attention kernel also emits the FP8 copy the output projection reads (no separate quantise launch);
  * RoPE + split + KV append run in the epilogue of the QKV GEMM and GeGLU -> FP8 in the epilogue of the gate|up
    GEMM (byte-identical to the separate kernels, which the calibration pass still uses);
  * FP8 weights are (N, K) K-contiguous (``fp8_nt_dev``);
  * the action out-projection adds its bias and accumulates into the noise buffer in the same launch, and that
    Euler state is held in fp32 (the reference keeps it in bf16, whose half-ulp at |x| ~ 4 is already 0.016);
  * kernels are chained with programmatic dependent launch inside the captured graph.
PyTorch only provides device memory, streams and graph capture here.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from . import flash_rt_fa2 as fa2
from . import flash_rt_kernels as fvk
from .weight_loader import (Attr, DictSource, FlatCat, FusedGateUp, FusedQKV, Item, LayerBlock, ModelWeightSpec,
                            Quant, SafetensorsSource, Scale, TensorList, ToBf16, WeightLoader, tT)

DEC_D, DEC_H, DEC_NH, DEC_NKV, DEC_HD, DEC_L = 1024, 4096, 8, 1, 256, 18
ACTION_DIM = 32
NUM_STEPS_DEFAULT = 10
CHUNK_DEFAULT = 50
BF16 = torch.bfloat16


# ------------------------------------------------------------------ weight spec (plugin contract)
def build_spec(layers: int = DEC_L, num_steps: int = NUM_STEPS_DEFAULT, precision: str = "fp8") -> ModelWeightSpec:
    """HF key names of the Gemma expert and the action heads (pi05_rtx.py:216-283).  ``precision="nvfp4"`` keeps
    the four projections in bf16 (N, K) for the device-side NVFP4 quantiser (fp4_utils.py:62-99)."""
    dp = "paligemma_with_expert.gemma_expert.model.layers.{i}"
    if precision == "nvfp4":
        dec = LayerBlock(prefix_fmt="", num_layers=layers, name="decoder", items=[
            Item("qkv_w", FusedQKV(q=f"{dp}.self_attn.q_proj.weight", k=f"{dp}.self_attn.k_proj.weight",
                                   v=f"{dp}.self_attn.v_proj.weight", interleave_q_heads=DEC_NH,
                                   interleave_k_heads=DEC_NKV), [ToBf16()], TensorList("wb_qkv")),
            Item("o_w", f"{dp}.self_attn.o_proj.weight", [ToBf16()], TensorList("wb_o")),
            Item("gu_w", FusedGateUp(gate=f"{dp}.mlp.gate_proj.weight", up=f"{dp}.mlp.up_proj.weight"),
                 [ToBf16()], TensorList("wb_gu")),
            Item("d_w", f"{dp}.mlp.down_proj.weight", [ToBf16()], TensorList("wb_d")),
        ])
    else:
        dec = _fp8_decoder_block(dp, layers)
    return _finish_spec(dec, dp, layers, num_steps)


def _fp8_decoder_block(dp: str, layers: int) -> LayerBlock:
    return LayerBlock(prefix_fmt="", num_layers=layers, name="decoder", items=[
        Item("qkv_w", FusedQKV(q=f"{dp}.self_attn.q_proj.weight", k=f"{dp}.self_attn.k_proj.weight",
                               v=f"{dp}.self_attn.v_proj.weight", interleave_q_heads=DEC_NH,
                               interleave_k_heads=DEC_NKV),
             [Quant()], FlatCat("w_qkv"), scale_into="ws_qkv"),
        Item("o_w", f"{dp}.self_attn.o_proj.weight", [Quant()], FlatCat("w_o"), scale_into="ws_o"),
        Item("gu_w", FusedGateUp(gate=f"{dp}.mlp.gate_proj.weight", up=f"{dp}.mlp.up_proj.weight"),
             [Quant()], FlatCat("w_gu"), scale_into="ws_gu"),
        Item("d_w", f"{dp}.mlp.down_proj.weight", [Quant()], FlatCat("w_d"), scale_into="ws_d"),
    ])


def _finish_spec(dec: LayerBlock, dp: str, layers: int, num_steps: int) -> ModelWeightSpec:
    mods = LayerBlock(prefix_fmt="", num_layers=layers, name="decoder_mods", items=[
        Item("attn_mod_w", f"{dp}.input_layernorm.dense.weight", [tT(), ToBf16()], TensorList("attn_mod_w")),
        Item("attn_mod_b", f"{dp}.input_layernorm.dense.bias", [ToBf16()], TensorList("attn_mod_b")),
        Item("ffn_mod_w", f"{dp}.post_attention_layernorm.dense.weight", [tT(), ToBf16()], TensorList("ffn_mod_w")),
        Item("ffn_mod_b", f"{dp}.post_attention_layernorm.dense.bias", [ToBf16()], TensorList("ffn_mod_b")),
    ])
    fin = "paligemma_with_expert.gemma_expert.model.norm.dense"
    singles = [
        Item("final_mod_w", f"{fin}.weight", [tT(), ToBf16()], Attr("final_mod_w")),
        Item("final_mod_b", f"{fin}.bias", [ToBf16()], Attr("final_mod_b")),
        Item("time_in_w", "time_mlp_in.weight", [tT(), ToBf16()], Attr("time_in_w")),
        Item("time_in_b", "time_mlp_in.bias", [ToBf16()], Attr("time_in_b")),
        Item("time_out_w", "time_mlp_out.weight", [tT(), ToBf16()], Attr("time_out_w")),
        Item("time_out_b", "time_mlp_out.bias", [ToBf16()], Attr("time_out_b")),
        Item("action_in_w", "action_in_proj.weight", [tT(), ToBf16()], Attr("action_in_w")),       # (32, D)
        Item("action_in_b", "action_in_proj.bias", [ToBf16()], Attr("action_in_b")),
        # x <- x + dt * v with dt = -1/N is folded into the out-projection (pi05_rtx.py:587-593)
        Item("action_out_w", "action_out_proj.weight", [tT(), ToBf16(), Scale(-1.0 / num_steps), ToBf16()],
             Attr("action_out_w")),                                                                # (D, 32)
        Item("action_out_b", "action_out_proj.bias", [ToBf16(), Scale(-1.0 / num_steps), ToBf16()],
             Attr("action_out_b")),
    ]
    return ModelWeightSpec(framework="torch", blocks=[dec, mods], singletons=singles,
                           dims={"D": DEC_D, "H": DEC_H, "L": layers})


def synthetic_state_dict(seed: int = 0, layers: int = DEC_L) -> dict:
    """Random-init checkpoint with the HF key names and shapes of the Pi0.5 action expert
    (matrices ~ N(0, 0.02), biases zero) — the stand-in for a trained checkpoint in tests and benchmarks."""
    g = torch.Generator().manual_seed(seed)

    def w(*shape):
        return torch.randn(*shape, generator=g) * 0.02

    sd = {}
    for i in range(layers):
        p = f"paligemma_with_expert.gemma_expert.model.layers.{i}"
        sd[f"{p}.self_attn.q_proj.weight"] = w(DEC_NH * DEC_HD, DEC_D)
        sd[f"{p}.self_attn.k_proj.weight"] = w(DEC_NKV * DEC_HD, DEC_D)
        sd[f"{p}.self_attn.v_proj.weight"] = w(DEC_NKV * DEC_HD, DEC_D)
        sd[f"{p}.self_attn.o_proj.weight"] = w(DEC_D, DEC_NH * DEC_HD)
        sd[f"{p}.mlp.gate_proj.weight"] = w(DEC_H, DEC_D)
        sd[f"{p}.mlp.up_proj.weight"] = w(DEC_H, DEC_D)
        sd[f"{p}.mlp.down_proj.weight"] = w(DEC_D, DEC_H)
        sd[f"{p}.input_layernorm.dense.weight"] = w(3 * DEC_D, DEC_D)
        sd[f"{p}.input_layernorm.dense.bias"] = torch.zeros(3 * DEC_D)
        sd[f"{p}.post_attention_layernorm.dense.weight"] = w(3 * DEC_D, DEC_D)
        sd[f"{p}.post_attention_layernorm.dense.bias"] = torch.zeros(3 * DEC_D)
    sd["paligemma_with_expert.gemma_expert.model.norm.dense.weight"] = w(3 * DEC_D, DEC_D)
    sd["paligemma_with_expert.gemma_expert.model.norm.dense.bias"] = torch.zeros(3 * DEC_D)
    sd["time_mlp_in.weight"], sd["time_mlp_in.bias"] = w(DEC_D, DEC_D), torch.zeros(DEC_D)
    sd["time_mlp_out.weight"], sd["time_mlp_out.bias"] = w(DEC_D, DEC_D), torch.zeros(DEC_D)
    sd["action_in_proj.weight"], sd["action_in_proj.bias"] = w(DEC_D, ACTION_DIM), torch.zeros(DEC_D)
    sd["action_out_proj.weight"], sd["action_out_proj.bias"] = w(ACTION_DIM, DEC_D), torch.zeros(ACTION_DIM)
    return sd


# ------------------------------------------------------------------ conditioning tables (load time, host)
def _bf(t: torch.Tensor) -> torch.Tensor:
    return t.to(BF16).float()


def precompute_styles(fe, num_steps: int, layers: int):
    """Time embedding -> time MLP (SiLU in fp32) -> per-norm modulation rows [scale | shift | gate], with the
    reference's bf16 rounding points (pi05_rtx.py:394-437).  Returns bf16 tensors (N, L, 3D), (N, L, 3D), (N, 3D)."""
    dt = torch.tensor(-1.0 / num_steps, dtype=torch.float32)
    t = torch.tensor(1.0, dtype=torch.float32)
    fraction = torch.linspace(0.0, 1.0, DEC_D // 2, dtype=torch.float32)
    period = 4e-3 * (4.0 / 4e-3) ** fraction
    sa = torch.empty(num_steps, layers, 3 * DEC_D)
    sf = torch.empty(num_steps, layers, 3 * DEC_D)
    fin = torch.empty(num_steps, 3 * DEC_D)
    silu = lambda z: z * torch.sigmoid(z)  # noqa: E731
    for s in range(num_steps):
        sinus = t * (1.0 / period) * 2 * math.pi
        te = _bf(torch.cat([torch.sin(sinus), torch.cos(sinus)], dim=-1))
        h = _bf(_bf(te @ fe.time_in_w.float()) + fe.time_in_b.float())
        h = _bf(silu(h))
        h = _bf(_bf(h @ fe.time_out_w.float()) + fe.time_out_b.float())
        c = _bf(silu(h))
        for i in range(layers):
            sa[s, i] = _bf(_bf(c @ fe.attn_mod_w[i].float()) + fe.attn_mod_b[i].float())
            sf[s, i] = _bf(_bf(c @ fe.ffn_mod_w[i].float()) + fe.ffn_mod_b[i].float())
        fin[s] = _bf(_bf(c @ fe.final_mod_w.float()) + fe.final_mod_b.float())
        t = t + dt
    return sa.to(BF16), sf.to(BF16), fin.to(BF16)


def rope_table(start: int, count: int) -> torch.Tensor:
    """bf16 (count, 256) rows [cos0, sin0, cos1, sin1, ...] for positions start .. start+count-1, theta 10000,
    phases in fp64 (pipeline_rtx.py:473-505)."""
    inv_freq = 1.0 / (10000 ** (np.arange(0, DEC_HD, 2, dtype=np.float64) / DEC_HD))
    phase = np.arange(start, start + count, dtype=np.float64)[:, None] * inv_freq[None, :]
    tab = np.stack([np.cos(phase), np.sin(phase)], axis=-1).reshape(count, DEC_HD)
    return torch.from_numpy(tab.astype(np.float32)).to(BF16)


# ------------------------------------------------------------------ kernel composition
SITES = ("qkv", "o", "gu", "d")


class StepIO:
    """Entry and exit of one Euler step, shared by the FP8 and NVFP4 compositions.

    Plain / batched: ``noise`` is (batch * chunk, 32); the in-projection covers all rows, the out-projection
    (pre-scaled by dt) accumulates into it.  Classifier-free guidance (``fe.cfg_beta`` set, batch 2: slot 0 =
    conditioned prefix, slot 1 = unconditioned): ``noise`` is (chunk, 32) and feeds both slots; the out-projection
    writes the two velocities and ``cfg_combine_into_residual`` folds them into the noise
    (flash_rt/models/pi05/pipeline_rtx_cfg_batched.py:313-417)."""

    def _alloc_step_io(self):
        fe = self.fe
        rows = fe.chunk_size if fe.cfg_beta is not None else fe.batch * fe.chunk_size
        self.noise = torch.zeros(rows, ACTION_DIM, dtype=torch.float32, device=fe.device)   # Euler state, fp32
        self.v = (torch.zeros(fe.batch * fe.chunk_size, ACTION_DIM, dtype=torch.float32, device=fe.device)
                  if fe.cfg_beta is not None else None)

    def _step_in(self, stream, pdl):
        fe, g = self.fe, self.gemm
        S, M = fe.chunk_size, fe.batch * fe.chunk_size
        if fe.cfg_beta is None:
            g.bf16_nn(self.noise.data_ptr(), fe.action_in_w.data_ptr(), self.x.data_ptr(), M, DEC_D, ACTION_DIM,
                      stream, pdl=pdl, bias=fe.action_in_b.data_ptr(), a_f32=True)
        else:
            for b in range(fe.batch):
                g.bf16_nn(self.noise.data_ptr(), fe.action_in_w.data_ptr(), self.x[b * S:].data_ptr(), S, DEC_D,
                          ACTION_DIM, stream, pdl=pdl and b == 0, bias=fe.action_in_b.data_ptr(), a_f32=True)

    def _step_out(self, stream, pdl):
        fe, g = self.fe, self.gemm
        S, M = fe.chunk_size, fe.batch * fe.chunk_size
        if fe.cfg_beta is None:
            g.bf16_nn(self.xn.data_ptr(), fe.action_out_w.data_ptr(), self.noise.data_ptr(), M, ACTION_DIM, DEC_D,
                      stream, pdl=pdl, bias=fe.action_out_b.data_ptr(), accumulate=True, d_f32=True)
        else:
            g.bf16_nn(self.xn.data_ptr(), fe.action_out_w.data_ptr(), self.v.data_ptr(), M, ACTION_DIM, DEC_D,
                      stream, pdl=pdl, bias=fe.action_out_b.data_ptr(), accumulate=False, d_f32=True)
            fvk.cfg_combine_into_residual(self.noise.data_ptr(), self.v.data_ptr(), self.v[S:].data_ptr(),
                                          fe.cfg_beta, S * ACTION_DIM, stream, pdl=pdl, f32=True)

    def step_io_launches(self) -> int:
        fe = self.fe
        return (fe.batch + 2) if fe.cfg_beta is not None else 2

    # -- where the fresh K / V rows go, and how the attention sees the cache ---------------------------------
    def _kv_dst(self, layer, b):
        """(K pointer, V pointer, devpos pointer) for the KV append of batch element ``b``.  Fixed-shape mode
        (flash_rt/hardware/rtx/attn_backend.py:272-282, 481-537): cache base + a device-side row offset, so that
        one captured graph serves every valid prefix length."""
        fe = self.fe
        if fe.fixed_shape:
            return fe.k_cache[layer, b].data_ptr(), fe.v_cache[layer, b].data_ptr(), fe.dec_devpos.data_ptr()
        return (fe.k_cache[layer, b, fe.prefix_len:].data_ptr(), fe.v_cache[layer, b, fe.prefix_len:].data_ptr(), 0)

    def _split_rope(self, layer, b, qkv, q, rows, stream, pdl):
        fe = self.fe
        kp, vp, dp = self._kv_dst(layer, b)
        args = (qkv.data_ptr(), fe.rope.data_ptr(), q.data_ptr(), kp, vp)
        dims = (rows, DEC_NH * DEC_HD, DEC_NKV * DEC_HD, DEC_NKV * DEC_HD, DEC_HD, stream)
        if dp:
            fvk.qkv_split_rope_devpos(*args, dp, *dims, pdl=pdl)
        else:
            fvk.qkv_split_rope(*args, *dims, pdl=pdl)

    def _attend(self, layer, stream, pdl, out_fp8=0, out_scale=0):
        fe = self.fe
        S, T = fe.chunk_size, fe.prefix_len + fe.chunk_size
        qs = (S * DEC_NH * DEC_HD, DEC_NH * DEC_HD, DEC_HD)
        ks = (fe.kv_rows * DEC_NKV * DEC_HD, DEC_NKV * DEC_HD, DEC_HD)
        kw = dict(pdl=pdl, out_fp8=out_fp8, out_scale=out_scale, kv_splits=self.attn_splits,
                  counters=self.attn_counters.data_ptr())
        common = (fe.batch, S, T, DEC_NH, DEC_NKV, DEC_HD, qs, ks, ks, qs, 1.0 / math.sqrt(DEC_HD), fe.sm_count, stream)
        q, k, v, o = (self.q.data_ptr(), fe.k_cache[layer].data_ptr(), fe.v_cache[layer].data_ptr(),
                      self.attn.data_ptr())
        if fe.fixed_shape:      # keys beyond *dec_seqused are masked; nothing may be fetched before the producer ends
            fa2.fwd_bf16_seqused_splitkv(q, k, v, o, 0, fe.dec_seqused.data_ptr(), self.lse_accum.data_ptr(),
                                         self.o_accum.data_ptr(), *common, kv_static_rows=0, **kw)
        else:
            fa2.fwd_bf16(q, k, v, o, 0, self.lse_accum.data_ptr(), self.o_accum.data_ptr(), *common,
                         kv_static_rows=fe.prefix_len, **kw)


class ExpertLoopArgs(ctypes.Structure):
    """``frt_b200_expert_loop_args`` of the C header (same member order)."""
    _fields_ = ([(n, ctypes.c_void_p) for n in (
        "w_qkv", "w_o", "w_gu", "w_d", "ws_qkv", "ws_o", "ws_gu", "ws_d", "act_scale", "style_attn", "style_ffn",
        "style_final", "rope", "in_w", "in_b", "out_w", "out_b", "k_cache", "v_cache", "noise", "workspace")]
        + [("workspace_bytes", ctypes.c_longlong)]
        + [(n, ctypes.c_int) for n in ("steps", "layers", "S", "prefix_len", "kv_rows")])


class Pi05DecoderPipeline(StepIO):
    """Pointer-only composition of the denoise loop (what gets captured in the graph)."""

    def __init__(self, fe: "Pi05DecoderB200"):
        self.fe = fe
        self.gemm = fvk.GemmRunner()
        dev = fe.device
        S, L, N = fe.batch * fe.chunk_size, fe.layers, fe.num_steps     # S = rows of every activation buffer
        self.M = S
        z = lambda *shape, dtype=BF16: torch.zeros(*shape, dtype=dtype, device=dev)  # noqa: E731
        self._alloc_step_io()
        self.x = z(S, DEC_D)
        self.xn = z(S, DEC_D)
        self.h_bf16 = z(S, DEC_D)                      # calibration only: un-quantised norm output
        self.qkv = z(S, (DEC_NH + 2 * DEC_NKV) * DEC_HD)
        self.q = z(S, DEC_NH * DEC_HD)
        self.attn = z(S, DEC_NH * DEC_HD)
        self.merged = z(S, 2 * DEC_H)
        self.hidden = z(S, DEC_H)                      # calibration only
        self.act8 = z(S, DEC_D, dtype=torch.uint8)
        self.attn8 = z(S, DEC_NH * DEC_HD, dtype=torch.uint8)
        self.hid8 = z(S, DEC_H, dtype=torch.uint8)
        self.ones = torch.ones(DEC_D, dtype=BF16, device=dev)
        # split-KV scratch of the attention kernel (the reference's FA2 o_accum / softmax_lse_accum buffers)
        self.attn_splits = fe.attn_splits
        self.o_accum = z(self.attn_splits, S, DEC_NH, DEC_HD, dtype=torch.float32)
        self.lse_accum = z(self.attn_splits, DEC_NH, S, dtype=torch.float32)
        self.attn_counters = z(2 * fe.batch * ((fe.chunk_size * DEC_NH + 127) // 128), dtype=torch.int32)
        # activation scales: one per GEMM input site, per layer, per denoise step (pipeline_rtx.py:649-660)
        self.act_scale = torch.ones(N, L, len(SITES), dtype=torch.float32, device=dev)
        # per-tile row sums of squares handed from a row-parallel projection to the next column-parallel one
        self.row_stats = torch.zeros(16, 128, dtype=torch.float32, device=dev)
        # deferred row scale: scales of the un-normalised operands x * (1 + scale) ([..., 0]: QKV input of the layer,
        # [..., 1]: gate|up input) and the column terms W . shift of both projections, per step and layer
        self.raw_scale = torch.ones(N, L, 2, dtype=torch.float32, device=dev)
        self.col_qkv = self.col_gu = None
        if fe.defer_norm:
            f8 = torch.float8_e4m3fn
            self.col_qkv = torch.empty(N, L, (DEC_NH + 2 * DEC_NKV) * DEC_HD, dtype=torch.float32, device=dev)
            self.col_gu = torch.empty(N, L, 2 * DEC_H, dtype=torch.float32, device=dev)
            for i in range(L):
                wq = fe.w_qkv[i].view(f8).float() * fe.ws_qkv_t[i]
                wg = fe.w_gu[i].view(f8).float() * fe.ws_gu_t[i]
                self.col_qkv[:, i] = fe.style_attn[:, i, DEC_D:2 * DEC_D].float() @ wq.T
                self.col_gu[:, i] = fe.style_ffn[:, i, DEC_D:2 * DEC_D].float() @ wg.T
        self.scratch_scale = torch.zeros(1, dtype=torch.float32, device=dev)
        self.calibrated = False
        self.loop_args = None
        if fe.persistent_loop:
            self._init_persistent_loop()

    # ---- the loop as one persistent kernel ---------------------------------
    def _init_persistent_loop(self):
        """Scratch and argument block of ``frt_b200_expert_loop_fp8``: the whole N-step loop in one cooperative
        launch (same weights, scales, styles and caches as the operator-by-operator composition below, which stays
        the calibration pass)."""
        fe = self.fe
        if fe.batch != 1 or fe.cfg_beta is not None or fe.fixed_shape or fe.chunk_size > 64:
            raise ValueError("persistent_loop serves batch 1, no guidance pair, no fixed-shape mode, chunk <= 64")
        nbytes = ctypes.c_longlong(0)
        fvk.call("frt_b200_expert_loop_workspace_bytes", fe.chunk_size, fe.prefix_len, ctypes.addressof(nbytes))
        self.loop_ws = torch.zeros(nbytes.value, dtype=torch.uint8, device=fe.device)
        a = ExpertLoopArgs()
        for name, t in (("w_qkv", fe.w_qkv), ("w_o", fe.w_o), ("w_gu", fe.w_gu), ("w_d", fe.w_d),
                        ("ws_qkv", fe.ws_qkv_t), ("ws_o", fe.ws_o_t), ("ws_gu", fe.ws_gu_t), ("ws_d", fe.ws_d_t),
                        ("act_scale", self.act_scale), ("style_attn", fe.style_attn), ("style_ffn", fe.style_ffn),
                        ("style_final", fe.style_final), ("rope", fe.rope), ("in_w", fe.action_in_w),
                        ("in_b", fe.action_in_b), ("out_w", fe.action_out_w), ("out_b", fe.action_out_b),
                        ("k_cache", fe.k_cache), ("v_cache", fe.v_cache), ("noise", self.noise),
                        ("workspace", self.loop_ws)):
            assert t.is_contiguous(), name
            setattr(a, name, t.data_ptr())
        a.workspace_bytes = nbytes.value
        a.steps, a.layers, a.S, a.prefix_len, a.kv_rows = fe.num_steps, fe.layers, fe.chunk_size, fe.prefix_len, fe.kv_rows
        self.loop_args = a

    def _run_persistent(self, stream: int) -> None:
        fvk.call("frt_b200_expert_loop_fp8", ctypes.addressof(self.loop_args), ctypes.sizeof(self.loop_args), stream)

    # ---- small helpers -------------------------------------------------
    def _scale_ptr(self, step, layer, site):
        return self.act_scale[step, layer, SITES.index(site)].data_ptr()

    def _raw_ptr(self, step, layer, which):
        return self.raw_scale[step, layer, which].data_ptr()

    def scale_tables(self):
        """Every calibrated table, in the order the on-disk cache stores them."""
        return [self.act_scale, self.raw_scale]

    def _style(self, which, step, layer=None):
        fe = self.fe
        t = {"attn": fe.style_attn, "ffn": fe.style_ffn, "final": fe.style_final}[which]
        row = t[step] if layer is None else t[step, layer]
        return row.data_ptr()

    def _gemm(self, a8, w8, wscale, out, M, N, K, ascale_ptr, stream, pdl):
        self.gemm.fp8_nt_dev(a8.data_ptr(), w8.data_ptr(), out.data_ptr(), M, N, K, ascale_ptr, wscale.data_ptr(),
                             stream, pdl=pdl)

    def _attention(self, layer, stream, pdl, out8_scale_ptr):
        self._attend(layer, stream, pdl, out_fp8=self.attn8.data_ptr() if out8_scale_ptr else 0,
                     out_scale=out8_scale_ptr or 0)

    # ---- the loop --------------------------------------------------------
    def transformer_decoder(self, stream: int = 0, calibrate: bool = False, step_hook=None) -> None:
        """Run the N-step denoise on ``self.noise`` in place (pipeline_rtx.py:1451-1504).

        ``calibrate=True`` is the eager dynamic-scale pass: every FP8 input is produced in bf16, its
        amax / 448 is measured on the device and folded (max) into the per-site per-step scale table.
        ``step_hook(step)`` (eager runs only) is called after each Euler step, e.g. to snapshot the state."""
        fe, g = self.fe, self.gemm
        if self.loop_args is not None and not calibrate and step_hook is None:
            self._run_persistent(stream)
            return
        S, L, B, CS = self.M, fe.layers, fe.batch, fe.chunk_size    # S = batch * chunk rows
        pdl = fe.use_pdl and not calibrate
        fold = self._folds_norms() and not calibrate
        fused_io = fold and self._fuses_step_io() and step_hook is None
        for step in range(fe.num_steps):
            if fused_io:
                if step == 0:
                    self._step_boundary(None, 0, stream, pdl)
                self._folded_layers(step, stream, pdl, first_norm=False)
                self._step_boundary(step, step + 1 if step + 1 < fe.num_steps else None, stream, pdl)
                continue
            # C0: action tokens -> width D, + bias
            self._step_in(stream, pdl)
            if fold:
                self._folded_layers(step, stream, pdl)
                fvk.ada_rms_norm_style(self.x.data_ptr(), self.ones.data_ptr(), self._style("final", step),
                                       self.xn.data_ptr(), 0, S, DEC_D, 1e-6, stream, pdl=pdl, style_stride=0)
                self._step_out(stream, pdl)
                if step_hook is not None:
                    step_hook(step)
                continue
            for i in range(L):
                # C1: adaRMS(style_attn) -> FP8 (layer 0 only; later layers get it from C7 of the previous one)
                if i == 0:
                    self._norm(None, None, "attn", step, i, "qkv", stream, pdl, calibrate)
                # C2: QKV projection, split + RoPE, K/V appended behind the prefix (one launch when not calibrating)
                if calibrate or not fe.fuse_epilogues or B > 1:
                    self._gemm(self.act8, fe.w_qkv[i], fe.ws_qkv_t[i], self.qkv, S, 2560, DEC_D,
                               self._scale_ptr(step, i, "qkv"), stream, pdl)
                    for b in range(B):      # every batch element appends to its own cache
                        self._split_rope(i, b, self.qkv[b * CS:], self.q[b * CS:], CS, stream, pdl and b == 0)
                else:
                    kp, vp, dp = self._kv_dst(i, 0)
                    g.fp8_nt_dev_rope_split(self.act8.data_ptr(), fe.w_qkv[i].data_ptr(), S, DEC_D,
                                            self._scale_ptr(step, i, "qkv"), fe.ws_qkv_t[i].data_ptr(),
                                            fe.rope.data_ptr(), self.q.data_ptr(), kp, vp, DEC_NH * DEC_HD,
                                            DEC_NKV * DEC_HD, DEC_NKV * DEC_HD, DEC_HD, stream, devpos=dp, pdl=pdl)
                # C3 + C4: attention (FP8 copy fused), output projection
                if calibrate:
                    self._attention(i, stream, False, 0)
                    self._dyn_quant(self.attn, self.attn8, step, i, "o", stream)
                else:
                    self._attention(i, stream, pdl, self._scale_ptr(step, i, "o"))
                fuse_norm = fe.fuse_norm and not calibrate and S <= 64
                if fuse_norm:
                    # C4 + C5 in one launch: out-projection, x += o * gate_attn, adaRMS(style_ffn) -> FP8
                    g.fp8_nt_dev_gate_res_norm_fp8(self.attn8.data_ptr(), fe.w_o[i].data_ptr(), S, DEC_D,
                                                   DEC_NH * DEC_HD, self._scale_ptr(step, i, "o"),
                                                   fe.ws_o_t[i].data_ptr(), self.x.data_ptr(),
                                                   self._style("attn", step, i) + 2 * DEC_D * 2,
                                                   self._style("ffn", step, i), self.act8.data_ptr(),
                                                   self._scale_ptr(step, i, "gu"), stream, pdl=pdl)
                else:
                    self._gemm(self.attn8, fe.w_o[i], fe.ws_o_t[i], self.xn, S, DEC_D, DEC_NH * DEC_HD,
                               self._scale_ptr(step, i, "o"), stream, pdl)
                    # C5: x += o * gate_attn ; adaRMS(style_ffn) -> FP8 ; gate|up projection
                    self._norm(self.xn, ("attn", step, i), "ffn", step, i, "gu", stream, pdl, calibrate)
                # C6: GeGLU -> FP8 (fused into the gate|up GEMM when not calibrating) ; down projection
                if calibrate:
                    self._gemm(self.act8, fe.w_gu[i], fe.ws_gu_t[i], self.merged, S, 2 * DEC_H, DEC_D,
                               self._scale_ptr(step, i, "gu"), stream, pdl)
                    fvk.gate_geglu_merged(self.merged.data_ptr(), self.hidden.data_ptr(), S, DEC_H, stream)
                    self._dyn_quant(self.hidden, self.hid8, step, i, "d", stream)
                elif not fe.fuse_epilogues:
                    self._gemm(self.act8, fe.w_gu[i], fe.ws_gu_t[i], self.merged, S, 2 * DEC_H, DEC_D,
                               self._scale_ptr(step, i, "gu"), stream, pdl)
                    fvk.gate_geglu_merged_fp8(self.merged.data_ptr(), self.hid8.data_ptr(), S, DEC_H,
                                              self._scale_ptr(step, i, "d"), stream, pdl=pdl)
                else:
                    g.fp8_nt_dev_geglu_fp8(self.act8.data_ptr(), fe.w_gu[i].data_ptr(), self.hid8.data_ptr(), S,
                                           DEC_H, DEC_D, self._scale_ptr(step, i, "gu"), fe.ws_gu_t[i].data_ptr(),
                                           self._scale_ptr(step, i, "d"), stream, pdl=pdl)
                if fuse_norm and i < L - 1:
                    # down projection + C7 in one launch
                    g.fp8_nt_dev_gate_res_norm_fp8(self.hid8.data_ptr(), fe.w_d[i].data_ptr(), S, DEC_D, DEC_H,
                                                   self._scale_ptr(step, i, "d"), fe.ws_d_t[i].data_ptr(),
                                                   self.x.data_ptr(), self._style("ffn", step, i) + 2 * DEC_D * 2,
                                                   self._style("attn", step, i + 1), self.act8.data_ptr(),
                                                   self._scale_ptr(step, i + 1, "qkv"), stream, pdl=pdl)
                    continue
                self._gemm(self.hid8, fe.w_d[i], fe.ws_d_t[i], self.xn, S, DEC_D, DEC_H,
                           self._scale_ptr(step, i, "d"), stream, pdl)
                # C7: x += f * gate_ffn ; next layer's adaRMS(style_attn) -> FP8
                if i < L - 1:
                    self._norm(self.xn, ("ffn", step, i), "attn", step, i + 1, "qkv", stream, pdl, calibrate)
                else:
                    fvk.call("frt_b200_gate_mul_residual", self.x.data_ptr(), self.xn.data_ptr(),
                             self._style("ffn", step, i) + 2 * DEC_D * 2, 0, S, DEC_D, 1 if pdl else 0, stream)
            # C8: final adaRMS (bf16), out-projection (+bias, pre-scaled by -1/N) accumulated into the noise
            fvk.ada_rms_norm_style(self.x.data_ptr(), self.ones.data_ptr(), self._style("final", step),
                                   self.xn.data_ptr(), 0, S, DEC_D, 1e-6, stream, pdl=pdl, style_stride=0)
            self._step_out(stream, pdl)
            if step_hook is not None:
                step_hook(step)

    def _fuses_step_io(self) -> bool:
        fe = self.fe
        return fe.fuse_step_io and self._folds_norms() and fe.cfg_beta is None and DEC_D % 256 == 0

    def _step_boundary(self, ending, beginning, stream, pdl) -> None:
        """One launch between two Euler steps: final norm + out-projection (+ Euler update) of step ``ending`` (None at
        the start of the loop), in-projection + first norm -> FP8 of step ``beginning`` (None behind the last step)."""
        fe = self.fe
        fvk.call("frt_b200_step_boundary", self.x.data_ptr(), self.noise.data_ptr(),
                 self._style("final", ending) if ending is not None else None, fe.action_out_w.data_ptr(),
                 fe.action_out_b.data_ptr(), fe.action_in_w.data_ptr(), fe.action_in_b.data_ptr(),
                 self._style("attn", beginning, 0) if beginning is not None else None, self.act8.data_ptr(),
                 self._scale_ptr(beginning if beginning is not None else 0, 0, "qkv"), self.M, DEC_D, ACTION_DIM, 1e-6,
                 1 if pdl else 0, stream)

    def _folds_norms(self) -> bool:
        fe = self.fe
        return fe.fold_norms and fe.batch == 1 and self.M <= 128

    def _folded_layers(self, step, stream, pdl, attention: bool = True, first_norm: bool = True) -> None:
        """The 18 blocks of one Euler step with five launches each: QKV (RoPE + split + KV append behind), attention
        (+ FP8 copy), attention-out (+ gated residual + row statistics), gate|up (GeGLU -> FP8), FFN-down (+ gated
        residual + row statistics).  The norm in front of QKV / gate|up is folded in one of two ways: the row-parallel
        projection before it also writes x * (1 + scale) as FP8 and the projection applies 1 / rms and W . shift in its
        finish (``defer_norm``, the default), or the projection produces its own FP8 operand from the residual rows
        (the reference's quantisation point).  Layer 0 takes its FP8 input from the norm kernel that follows the
        in-projection.  ``attention=False`` leaves the attention launches out (the four weight-streaming launches of
        every block exactly as the loop issues them: what ``bench.py`` times for the roofline)."""
        fe, g = self.fe, self.gemm
        S, L = self.M, fe.layers
        x, stats = self.x.data_ptr(), self.row_stats.data_ptr()
        qd, kd = DEC_NH * DEC_HD, DEC_NKV * DEC_HD
        gate_off = 2 * DEC_D * 2
        n_stat = 0
        # tile width / split-K of the four projections at <= 64 tokens, from per-launch timings of the captured chain
        # (QKV 64 x 4, attention-out 64 x 8, gate|up 64 + 64 x 2, FFN-down 64 x 8); larger row counts use the
        # library's own choice
        tuned = S <= 64
        defer = fe.defer_norm
        t_qkv = dict(splits=4, tile_n=64) if tuned else {}
        t_o = dict(splits=8, tile_n=64) if tuned else {}
        t_gu = dict(splits=2, tile_n=128) if tuned else {}
        t_d = dict(splits=8, tile_n=64) if tuned else {}
        t_gu["fast_gelu"] = fe.fast_gelu
        for i in range(L):
            kp, vp, dp = self._kv_dst(i, 0)
            if i == 0:
                if attention and first_norm:
                    self._norm(None, None, "attn", step, 0, "qkv", stream, pdl, False)
                g.fp8_nt_dev_rope_split(self.act8.data_ptr(), fe.w_qkv[i].data_ptr(), S, DEC_D,
                                        self._scale_ptr(step, i, "qkv"), fe.ws_qkv_t[i].data_ptr(),
                                        fe.rope.data_ptr(), self.q.data_ptr(), kp, vp, qd, kd, kd, DEC_HD, stream,
                                        devpos=dp, pdl=pdl, **t_qkv)
            elif defer:
                g.fp8_nt_dev_rope_split_rowscale(self.act8.data_ptr(), fe.w_qkv[i].data_ptr(), S, DEC_D,
                                                 self._raw_ptr(step, i, 0), fe.ws_qkv_t[i].data_ptr(), stats, n_stat,
                                                 self.col_qkv[step, i].data_ptr(), fe.rope.data_ptr(),
                                                 self.q.data_ptr(), kp, vp, qd, kd, kd, DEC_HD, stream, devpos=dp,
                                                 pdl=pdl, **t_qkv)
            else:
                g.norm_fp8_nt_dev_rope_split(x, stats, n_stat, self._style("attn", step, i), fe.w_qkv[i].data_ptr(),
                                             S, DEC_D, self._scale_ptr(step, i, "qkv"), fe.ws_qkv_t[i].data_ptr(),
                                             fe.rope.data_ptr(), self.q.data_ptr(), kp, vp, qd, kd, kd, DEC_HD,
                                             stream, devpos=dp, pdl=pdl, **t_qkv)
            if attention:
                self._attention(i, stream, pdl, self._scale_ptr(step, i, "o"))
            q8 = (dict(next_scale=self._style("ffn", step, i), q8_out=self.act8.data_ptr(),
                       d_scale_q8=self._raw_ptr(step, i, 1)) if defer else {})
            n_stat = g.fp8_nt_dev_gate_residual(self.attn8.data_ptr(), fe.w_o[i].data_ptr(), S, DEC_D, qd,
                                                self._scale_ptr(step, i, "o"), fe.ws_o_t[i].data_ptr(), x,
                                                self._style("attn", step, i) + gate_off, stats, stream, pdl=pdl,
                                                **t_o, **q8)
            if defer:
                g.fp8_nt_dev_geglu_fp8_rowscale(self.act8.data_ptr(), fe.w_gu[i].data_ptr(), self.hid8.data_ptr(), S,
                                                DEC_H, DEC_D, self._raw_ptr(step, i, 1), fe.ws_gu_t[i].data_ptr(),
                                                stats, n_stat, self.col_gu[step, i].data_ptr(),
                                                self._scale_ptr(step, i, "d"), stream, pdl=pdl, **t_gu)
            else:
                g.norm_fp8_nt_dev_geglu_fp8(x, stats, n_stat, self._style("ffn", step, i), fe.w_gu[i].data_ptr(),
                                            self.hid8.data_ptr(), S, DEC_H, DEC_D, self._scale_ptr(step, i, "gu"),
                                            fe.ws_gu_t[i].data_ptr(), self._scale_ptr(step, i, "d"), stream, pdl=pdl,
                                            **t_gu)
            q8 = (dict(next_scale=self._style("attn", step, i + 1), q8_out=self.act8.data_ptr(),
                       d_scale_q8=self._raw_ptr(step, i + 1, 0)) if defer and i < L - 1 else {})
            n_stat = g.fp8_nt_dev_gate_residual(self.hid8.data_ptr(), fe.w_d[i].data_ptr(), S, DEC_D, DEC_H,
                                                self._scale_ptr(step, i, "d"), fe.ws_d_t[i].data_ptr(), x,
                                                self._style("ffn", step, i) + gate_off, stats, stream, pdl=pdl,
                                                **t_d, **q8)

    def launches_per_layer(self) -> float:
        """Average over the layers (the last layer keeps its separate residual kernel when the norms are fused)."""
        fe = self.fe
        if self._folds_norms():
            return 5.0
        qkv = 1 if fe.batch == 1 and fe.fuse_epilogues else 1 + fe.batch
        gu = 1 if fe.fuse_epilogues else 2
        if fe.fuse_norm and self.M <= 64:
            # qkv, attention, o + norm, gate|up, down + norm   (last layer: down, gated residual)
            return qkv + 1 + 1 + gu + 1 + 1.0 / fe.layers
        return qkv + 1 + 1 + 1 + gu + 1 + 1

    def _norm(self, delta, gate_from, style_kind, step, layer, site, stream, pdl, calibrate):
        """(x += delta * gate) ; adaRMS(style) -> FP8 for GEMM site ``site`` of ``layer``."""
        S = self.M
        style = self._style(style_kind, step, layer)
        gate = (self._style(*gate_from) + 2 * DEC_D * 2) if gate_from else None
        if not calibrate:
            fvk.call("frt_b200_norm_fp8", self.x.data_ptr(), delta.data_ptr() if delta is not None else None,
                     gate, 0, None, style, 0, self.act8.data_ptr(), None, S, DEC_D, 1e-6,
                     self._scale_ptr(step, layer, site), 1 if pdl else 0, stream)
            return
        fvk.call("frt_b200_norm_bf16", self.x.data_ptr(), delta.data_ptr() if delta is not None else None,
                 gate, 0, None, style, 0, self.h_bf16.data_ptr(), None, S, DEC_D, 1e-6, 0, stream)
        self._dyn_quant(self.h_bf16, self.act8, step, layer, site, stream)
        if self.fe.defer_norm:
            # amax / 448 of the updated residual times (1 + scale): the operand the deferred-row-scale launches read
            rows = {"attn": self.fe.style_attn, "ffn": self.fe.style_ffn}[style_kind]
            raw = (self.x.float() * (1.0 + rows[step, layer, :DEC_D].float())).abs().max() / 448.0
            slot = self.raw_scale[step, layer, 0 if site == "qkv" else 1]
            slot.copy_(torch.maximum(slot, raw))

    def _dyn_quant(self, src, dst8, step, layer, site, stream):
        """Dynamic quantisation used while calibrating (pipeline_rtx.py:804-821): scale of this call into the
        scratch word, running max into the table; the GEMM of this pass then reads the table entry."""
        fvk.quantize_fp8_device(src.data_ptr(), dst8.data_ptr(), self.scratch_scale.data_ptr(), src.numel(), stream)
        fvk.fp8_accumulate_scale_max(self.scratch_scale.data_ptr(), self._scale_ptr(step, layer, site), stream)
        # quantise again with the accumulated scale so that codes and GEMM scale agree
        fvk.quantize_fp8_static(src.data_ptr(), dst8.data_ptr(), self._scale_ptr(step, layer, site), src.numel(),
                                stream)


class Pi05DecoderB200:
    """Decoder-only Pi0.5 frontend for B200 (duck type of the reference frontends: ``infer``, ``calibrate``,
    ``calibrated``; ``set_prefix`` takes the place of ``set_prompt`` because the prefix producer is not part of
    this path)."""

    WEIGHT_SPEC = None  # built per instance (layer count / step count are constructor arguments)

    def __init__(self, checkpoint, *, num_steps: int = NUM_STEPS_DEFAULT, chunk_size: int = CHUNK_DEFAULT,
                 prefix_len: int = 768, layers: int = DEC_L, device: int | str = 0, use_pdl: bool = True,
                 use_cuda_graph: bool = True, fuse_epilogues: bool = True, precision: str = "fp8", batch: int = 1,
                 cfg_beta: float | None = None, fixed_shape: bool = False, attn_splits: int = 8,
                 fuse_norm: bool = False, fold_norms: bool = True, defer_norm: bool = True, fast_gelu: bool = True, fuse_step_io: bool = True,
                 persistent_loop: bool = False, **_ignored):
        if not torch.cuda.is_available():
            raise RuntimeError("flashrt_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        torch.cuda.set_device(self.device)
        if fvk.get_sm_version() != 100:
            raise RuntimeError(f"flashrt_b200 is built for sm_100a only; device reports sm_{fvk.get_sm_version()}")
        self.num_steps, self.chunk_size, self.prefix_len, self.layers = num_steps, chunk_size, prefix_len, layers
        self.use_pdl, self.use_cuda_graph, self.fuse_epilogues = use_pdl, use_cuda_graph, fuse_epilogues
        # projection + gated residual + adaRMS as one 16-CTA-cluster launch: measured slower than the two kernels
        # (10.17 ms vs 9.75 ms per loop, 950 vs 1300 launches), so off unless asked for
        self.fuse_norm = bool(fuse_norm) and fuse_epilogues
        # the two norm launches of a block folded into the projections around them: the row-parallel projections
        # (attention-out, FFN-down) update the residual and leave per-tile sums of squares, the column-parallel ones
        # (QKV, gate|up) produce their own FP8 input from them: 5 launches per block instead of 7
        self.fold_norms = bool(fold_norms) and fuse_epilogues and not self.fuse_norm
        # with the norms folded: the row-parallel projection also writes the next projection's FP8 operand, without the
        # row's 1 / rms (which commutes with the projection and is applied, with the precomputed W . shift, in the
        # next projection's finish) -- no CTA of QKV / gate|up then builds its operand behind the dependency wait.
        # False keeps the reference's quantisation point (after the row scale) through the in-kernel norm producer.
        self.defer_norm = bool(defer_norm) and self.fold_norms and precision == "fp8"
        # GELU of the fused gate|up finish through the hardware tanh (2^-11 relative, 1 / 128 of the FP8 step the result
        # is rounded to; the reference's kernel is built on the fast __expf): 0.10 ms per loop (5.66 -> 5.57 ms).
        # False selects the explicitly rounded exp + division that the C oracle restates bit for bit (the FP8 codes of
        # the gate|up output are then reproducible on a CPU).  Only the folded (token-major) composition has the option.
        self.fast_gelu = bool(fast_gelu) and self.fold_norms
        # the four launches between two Euler steps (final norm, action out-projection, action in-projection, first norm)
        # as one launch per step boundary, bit-identical to the four (batch 1 without guidance, folded norms)
        self.fuse_step_io = bool(fuse_step_io) and self.fold_norms
        # the whole loop as one cooperative kernel (phases separated by grid barriers) instead of 1300 launches
        self.persistent_loop = bool(persistent_loop)
        if self.persistent_loop and precision != "fp8":
            raise ValueError("persistent_loop is built for the FP8 loop")
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.kv_rows = prefix_len + chunk_size
        if precision not in ("fp8", "nvfp4"):
            raise ValueError(f"precision must be 'fp8' or 'nvfp4', got {precision!r}")
        if cfg_beta is not None and batch != 2:
            raise ValueError("classifier-free guidance runs the conditioned and the unconditioned slot: batch must be 2")
        self.cfg_beta = None if cfg_beta is None else float(cfg_beta)
        # fixed-shape mode: prefix_len is the LARGEST prefix; the valid length is a device-side value
        self.fixed_shape = bool(fixed_shape)
        self.attn_splits = int(attn_splits)      # kv splits of the decoder attention (combined through scratch)
        self.valid_prefix_len = prefix_len
        if batch < 1 or batch * ((chunk_size * DEC_NH + 127) // 128) * 8 > self.sm_count:
            raise ValueError(f"batch {batch} x chunk {chunk_size} does not fit the one-wave split-KV attention")
        self.precision, self.batch = precision, batch
        self.WEIGHT_SPEC = build_spec(layers, num_steps, precision)
        self.checkpoint_path = None
        if isinstance(checkpoint, dict):
            source = DictSource(checkpoint)
        elif isinstance(checkpoint, str) and checkpoint.startswith("synthetic"):
            seed = int(checkpoint.split(":")[1]) if ":" in checkpoint else 0
            source = DictSource(synthetic_state_dict(seed, layers))
        else:
            import os
            ck = str(checkpoint)
            if os.path.isdir(ck):
                ck = os.path.join(ck, "model.safetensors")
            self.checkpoint_path = ck
            source = SafetensorsSource(ck)
        WeightLoader(source, target=self, spec=self.WEIGHT_SPEC).run()
        dev = self.device
        if precision == "nvfp4":
            from .pi05_decoder_nvfp4 import Nvfp4Weight
            self.w4 = []
            for i in range(layers):
                self.w4.append({k: Nvfp4Weight(getattr(self, "wb_" + k)[i].to(dev)) for k in ("qkv", "o", "gu", "d")})
            for k in ("qkv", "o", "gu", "d"):
                delattr(self, "wb_" + k)
        else:
            # FP8 weights as raw bytes on the device, (L, N, K)
            for n in ("w_qkv", "w_o", "w_gu", "w_d"):
                setattr(self, n, getattr(self, n).view(torch.uint8).to(dev))
            for n in ("ws_qkv", "ws_o", "ws_gu", "ws_d"):
                setattr(self, n + "_t", torch.tensor(getattr(self, n), dtype=torch.float32, device=dev))
        sa, sf, fin = precompute_styles(self, num_steps, layers)
        self.style_attn, self.style_ffn, self.style_final = sa.to(dev), sf.to(dev), fin.to(dev)
        for n in ("action_in_w", "action_in_b", "action_out_w", "action_out_b"):
            setattr(self, n, getattr(self, n).contiguous().to(dev))
        self.rope = rope_table(prefix_len, chunk_size).to(dev)
        self.dec_devpos = torch.full((1,), prefix_len, dtype=torch.int32, device=dev)
        self.dec_seqused = torch.full((1,), prefix_len + chunk_size, dtype=torch.int32, device=dev)
        # one cache per batch element: (layers, batch, prefix + chunk, 256)
        self.k_cache = torch.zeros(layers, batch, self.kv_rows, DEC_NKV * DEC_HD, dtype=BF16, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        if precision == "nvfp4":
            from .pi05_decoder_nvfp4 import Pi05DecoderNvfp4Pipeline
            self.pipeline = Pi05DecoderNvfp4Pipeline(self)
        else:
            self.pipeline = Pi05DecoderPipeline(self)
        self.stream = torch.cuda.Stream(device=dev)
        self.graph = None
        rows = chunk_size if self.cfg_beta is not None else batch * chunk_size
        self._pinned_in = torch.zeros(rows, ACTION_DIM, dtype=torch.float32).pin_memory()
        self._pinned_out = torch.zeros(rows, ACTION_DIM, dtype=torch.float32).pin_memory()
        self._dev_in = torch.zeros(rows, ACTION_DIM, dtype=torch.float32, device=dev)
        self._dev_out = torch.zeros(rows, ACTION_DIM, dtype=torch.float32, device=dev)
        # status words of the tensor-core kernels, gathered by the last kernel of the captured loop and read back with
        # the actions (no blocking status call per inference)
        self._dev_status = torch.zeros(4, dtype=torch.int32, device=dev)
        self._pinned_status = torch.zeros(4, dtype=torch.int32).pin_memory()
        self.latency_records: list[float] = []

    # ---- prefix (what the encoder would have written) ---------------------
    def set_prefix(self, prefix_k: torch.Tensor, prefix_v: torch.Tensor) -> None:
        """prefix_k / prefix_v: (layers, prefix_len, 256), shared by every batch element, or
        (layers, batch, prefix_len, 256) with one prefix per element (classifier-free guidance: slot 0 = conditioned
        prompt, slot 1 = unconditioned).  K already carries its RoPE, as in the encoder's cache."""
        if prefix_k.dim() == 3:
            prefix_k, prefix_v = (t.unsqueeze(1).expand(-1, self.batch, -1, -1) for t in (prefix_k, prefix_v))
        assert prefix_k.shape == (self.layers, self.batch, self.prefix_len, DEC_NKV * DEC_HD), prefix_k.shape
        self.k_cache[:, :, :self.prefix_len].copy_(prefix_k.to(BF16))
        self.v_cache[:, :, :self.prefix_len].copy_(prefix_v.to(BF16))
        torch.cuda.synchronize(self.device)

    def set_valid_prefix_len(self, valid: int) -> None:
        """Fixed-shape mode: the first ``valid`` rows of the prefix are real, the rest padding.  Updates the three
        device-side values the captured graph reads -- KV append row, number of keys the attention sees, RoPE rows
        of the action tokens -- without re-capturing (``set_valid_prefix_len``,
        flash_rt/hardware/rtx/attn_backend.py:519-537)."""
        if not self.fixed_shape:
            raise RuntimeError("set_valid_prefix_len needs fixed_shape=True")
        if not 0 <= valid <= self.prefix_len:
            raise ValueError(f"valid prefix length {valid} outside [0, {self.prefix_len}]")
        self.valid_prefix_len = int(valid)
        self.dec_devpos.fill_(valid)
        self.dec_seqused.fill_(valid + self.chunk_size)
        self.rope.copy_(rope_table(valid, self.chunk_size).to(self.device))
        torch.cuda.synchronize(self.device)

    def set_prefix_pair(self, cond_k, cond_v, uncond_k, uncond_v) -> None:
        """Conditioned / unconditioned prefixes of the classifier-free-guidance pair
        (``set_language_embeds_pair``, flash_rt/models/pi05/pipeline_rtx_cfg_batched.py:197-229, one level later:
        the per-layer K/V the two prompts leave in the cache)."""
        self.set_prefix(torch.stack([cond_k, uncond_k], dim=1), torch.stack([cond_v, uncond_v], dim=1))

    # ---- calibration --------------------------------------------------------
    @property
    def calibrated(self) -> bool:
        return self.pipeline.calibrated

    def _cache_meta(self, n_samples: int, percentile) -> dict:
        return {"layers": self.layers, "num_steps": self.num_steps, "chunk": self.chunk_size, "batch": self.batch,
                "samples": n_samples, "percentile": percentile, "sites": list(SITES)}

    def calibrate(self, noises, percentile: float | None = None, use_cache: bool = False, cache_dir=None) -> None:
        """Static per-tensor activation scales from ``noises`` (list of (chunk, 32) tensors).  Each sample runs
        the eager dynamic-scale pass; the table keeps the max over samples (``percentile`` None) or the given
        percentile of the per-sample scales (flash_rt/core/calibration.py:38-64).  ``use_cache``: when the model
        was loaded from a file, reuse / store the table in the on-disk calibration cache
        (flash_rt/core/quant/calibrator.py:28-145) keyed by checkpoint hash and prefix length."""
        p = self.pipeline
        if self.precision == "nvfp4":
            return                      # block scales are computed by the producing kernels at run time
        from . import calibration_cache as cc
        cacheable = use_cache and self.checkpoint_path is not None
        if cacheable:
            tables = p.scale_tables()
            hit = cc.load_calibration(self.checkpoint_path, self.prefix_len,
                                      expected_count=sum(t.numel() for t in tables), cache_dir=cache_dir,
                                      metadata=self._cache_meta(len(noises), percentile))
            if hit is not None:
                flat, at = torch.tensor(hit["ae_scales"], dtype=torch.float32), 0
                for t in tables:
                    t.copy_(flat[at:at + t.numel()].reshape(t.shape))
                    at += t.numel()
                torch.cuda.synchronize(self.device)
                p.calibrated = True
                self.graph = None
                self.calibration_source = "cache"
                return
        self.calibration_source = "measured"
        tables = p.scale_tables()
        per_sample = [[] for _ in tables]
        with torch.cuda.stream(self.stream):
            for nz in noises:
                for t in tables:
                    t.zero_()
                p.noise.copy_(nz.to(self.device, torch.float32).reshape(p.noise.shape))
                p.transformer_decoder(self.stream.cuda_stream, calibrate=True)
                self.stream.synchronize()
                for t, acc in zip(tables, per_sample):
                    acc.append(t.clone())
            for t, acc in zip(tables, per_sample):
                stack = torch.stack(acc, 0)
                if percentile is None:
                    t.copy_(stack.max(0).values)
                else:
                    t.copy_(torch.quantile(stack, percentile / 100.0, dim=0))
                t.clamp_(min=1e-12)
        self.stream.synchronize()
        if fvk.tensor_core_status() != 0:
            raise RuntimeError("a tensor-core kernel reported a timed-out wait during calibration")
        p.calibrated = True
        self.graph = None
        self._calibration_record = dict(method="max" if percentile is None else "percentile", samples=len(noises),
                                        percentile=percentile)
        if cacheable:
            cc.save_calibration(self.checkpoint_path, self.prefix_len,
                                torch.cat([t.flatten() for t in tables]).cpu().tolist(),
                                metadata=self._cache_meta(len(noises), percentile), cache_dir=cache_dir)

    @property
    def precision_spec(self):
        """:class:`flashrt_b200.precision_spec.ModelPrecisionSpec` of the calibrated model (``None`` before), the record the
        reference's frontend keeps at calibration time (flash_rt/frontends/torch/pi05_rtx.py:1480-1545)."""
        if not self.calibrated:
            return None
        from .precision_spec import snapshot_decoder
        p, rec = self.pipeline, getattr(self, "_calibration_record", dict(method="cache", samples=0, percentile=None))
        if self.precision == "nvfp4":
            names = {f"decoder_{k}_w_{i}": None for i in range(self.layers) for k in ("attn_qkv", "attn_o", "ffn_gate_up",
                                                                                      "ffn_down")}
            return snapshot_decoder(None, SITES, names, precision="nvfp4", method=rec["method"], samples=rec["samples"],
                                    percentile=rec["percentile"])
        weights = {"decoder_attn_qkv_w": self.ws_qkv_t.cpu().numpy(), "decoder_attn_o_w": self.ws_o_t.cpu().numpy(),
                   "decoder_ffn_gate_up_w": self.ws_gu_t.cpu().numpy(), "decoder_ffn_down_w": self.ws_d_t.cpu().numpy()}
        return snapshot_decoder(p.act_scale.cpu().numpy(), SITES, weights, precision="fp8", method=rec["method"],
                                samples=rec["samples"], percentile=rec["percentile"],
                                raw_scale=p.raw_scale.cpu().numpy() if self.defer_norm else None)

    # ---- graph --------------------------------------------------------------
    def record_infer_graph(self) -> None:
        """Warm up, then capture the input copy, the whole N-step loop and the output copy as one graph
        (pipeline_rtx.py:1980-2049)."""
        if not self.calibrated:
            raise RuntimeError("calibrate() first: the captured loop uses static activation scales")
        p = self.pipeline
        s = self.stream
        with torch.cuda.stream(s):
            for _ in range(2):
                self._enqueue(s)
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s, capture_error_mode="relaxed"):
                self._enqueue(s)
        s.synchronize()
        self.graph = g

    def _enqueue(self, s) -> None:
        p = self.pipeline
        p.noise.copy_(self._dev_in)
        p.transformer_decoder(s.cuda_stream, calibrate=False)
        fvk.call("frt_b200_status_words_async", self._dev_status.data_ptr(), 0, 0, s.cuda_stream)
        self._dev_out.copy_(p.noise)

    def forward_decode_only(self) -> None:
        """Replay the captured loop on the frontend's stream (pipeline_rtx.py:2175-2196)."""
        if self.graph is None:
            if self.use_cuda_graph:
                self.record_infer_graph()
            else:
                with torch.cuda.stream(self.stream):
                    self._enqueue(self.stream)
                return
        with torch.cuda.stream(self.stream):
            self.graph.replay()

    # ---- public call ------------------------------------------------------------
    def infer(self, obs: dict) -> dict:
        """obs["noise"]: (chunk, 32) array or tensor on the HOST (a fresh N(0,1) draw if absent).  Uploads it,
        replays the loop, downloads the actions (pi05_rtx.py:1547-1614)."""
        nz = obs.get("noise") if obs else None
        single = self.batch == 1 or self.cfg_beta is not None
        shape = (self.chunk_size, ACTION_DIM) if single else (self.batch, self.chunk_size, ACTION_DIM)
        if nz is None:
            nz = torch.randn(*shape)
        nz = torch.as_tensor(nz, dtype=torch.float32)
        self._pinned_in.copy_(nz.reshape(self._pinned_in.shape))
        with torch.cuda.stream(self.stream):
            self._dev_in.copy_(self._pinned_in, non_blocking=True)
        self.forward_decode_only()
        with torch.cuda.stream(self.stream):
            self._pinned_out.copy_(self._dev_out, non_blocking=True)
            self._pinned_status.copy_(self._dev_status, non_blocking=True)
        self.stream.synchronize()
        # a bounded device-side wait that gave up leaves a status word and garbage actions: never return those
        status = int(self._pinned_status[0]) or int(self._pinned_status[1]) or int(self._pinned_status[2])
        if status != 0:
            fvk.tensor_core_status()          # clear the sticky words for the next call
            raise fvk.KernelError(f"a tensor-core kernel of the denoise loop gave up a bounded wait (status {status:#x}); "
                                  "the actions of this call are invalid")
        return {"actions": self._pinned_out.numpy().reshape(shape).copy()}

    def kernels_per_loop(self) -> int:
        """Launches of this library's kernels inside one replay (for reporting)."""
        L, N = self.layers, self.num_steps
        p = self.pipeline
        if getattr(p, "loop_args", None) is not None:
            return 2
        # in-projection(s), first norm, the blocks, final residual + final norm, out-projection (+ guidance combine) --
        # or one launch per step boundary; one status-gather launch behind the last step
        if hasattr(p, "_fuses_step_io") and p._fuses_step_io():
            return int(round(N * p.launches_per_layer() * L)) + (N + 1) + 1
        return int(round(N * (p.step_io_launches() + 1 + p.launches_per_layer() * L + 1))) + 1
