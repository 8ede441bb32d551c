"""CPU tests of the on-disk formats: calibration cache (keying, validation, atomic write), the synthetic
safetensors checkpoint read back through the weight loader, and the quantisation record (``precision_spec``) against a
JSON document written by the reference's own classes."""
import json
import os

import numpy as np
import pytest
import torch

from flashrt_b200 import calibration_cache as cc


def test_calibration_cache_roundtrip_and_validation(tmp_path):
    ck = tmp_path / "model.safetensors"
    ck.write_bytes(b"A" * 100000)
    scales = [0.5 + i * 1e-3 for i in range(10 * 18 * 4)]
    meta = {"layers": 18, "samples": 8}
    f = cc.save_calibration(str(ck), 768, scales, metadata=meta, cache_dir=tmp_path / "cache")
    assert f.name == f"{cc.checkpoint_hash(str(ck))}_Se768.b200dec.json"
    rec = cc.load_calibration(str(ck), 768, expected_count=720, cache_dir=tmp_path / "cache", metadata=meta)
    assert rec is not None and rec["ae_scales"] == scales and rec["version"] == 1 and rec["num_ae_scales"] == 720
    # every mismatch is a miss, never an exception
    assert cc.load_calibration(str(ck), 512, cache_dir=tmp_path / "cache") is None                    # other Se
    assert cc.load_calibration(str(ck), 768, expected_count=10, cache_dir=tmp_path / "cache") is None  # other count
    assert cc.load_calibration(str(ck), 768, cache_dir=tmp_path / "cache", metadata={"layers": 4}) is None
    assert cc.load_calibration(str(tmp_path / "missing.safetensors"), 768, cache_dir=tmp_path / "cache") is None
    other = tmp_path / "other.safetensors"
    other.write_bytes(b"B" * 100000)
    assert cc.load_calibration(str(other), 768, cache_dir=tmp_path / "cache") is None                  # other checkpoint
    # the hash covers the first 64 KB and the size
    same_head = tmp_path / "longer.safetensors"
    same_head.write_bytes(b"A" * 100001)
    assert cc.checkpoint_hash(str(same_head)) != cc.checkpoint_hash(str(ck))
    # a damaged or foreign-version file is a miss
    data = json.loads(f.read_text())
    data["version"] = 2
    f.write_text(json.dumps(data))
    assert cc.load_calibration(str(ck), 768, cache_dir=tmp_path / "cache") is None
    f.write_text("{not json")
    assert cc.load_calibration(str(ck), 768, cache_dir=tmp_path / "cache") is None
    # a file in the reference's own format under the reference's own name is neither read nor overwritten
    # (flash_rt/core/quant/calibrator.py:28-145: {hash}_Se{Se}.json with enc_* fields and layers * 4 decoder scales)
    theirs = tmp_path / "cache" / f"{cc.checkpoint_hash(str(ck))}_Se768.json"
    theirs.write_text(json.dumps({"version": 1, "ckpt_hash": cc.checkpoint_hash(str(ck)), "Se": 768,
                                  "enc_scales": [1.0], "ae_scales": [1.0] * 72, "num_ae_scales": 72}))
    before = theirs.read_text()
    assert cc.load_calibration(str(ck), 768, cache_dir=tmp_path / "cache") is None
    cc.save_calibration(str(ck), 768, scales, cache_dir=tmp_path / "cache")
    assert theirs.read_text() == before
    assert cc.load_calibration(str(ck), 768, cache_dir=tmp_path / "cache")["format"] == cc.CACHE_FORMAT
    # directory form of the checkpoint path
    d = tmp_path / "ckpt_dir"
    d.mkdir()
    (d / "model.safetensors").write_bytes(b"C" * 1000)
    cc.save_calibration(str(d), 768, [1.0, 2.0], cache_dir=tmp_path / "cache")
    assert cc.load_calibration(str(d), 768, cache_dir=tmp_path / "cache")["ae_scales"] == [1.0, 2.0]


def test_synthetic_checkpoint_reads_back_through_the_weight_loader(tmp_path):
    from flashrt_b200.pi05_decoder import build_spec, synthetic_state_dict
    from flashrt_b200.weight_loader import SafetensorsSource, WeightLoader
    L = 2
    path = cc.write_synthetic_checkpoint(str(tmp_path / "ckpt"), seed=3, layers=L)
    assert path.endswith("model.safetensors")
    sd = synthetic_state_dict(3, L)
    src = SafetensorsSource(path)
    for k in ("time_mlp_in.weight", "paligemma_with_expert.gemma_expert.model.layers.1.mlp.down_proj.weight"):
        assert src.has(k)
        assert torch.equal(src.get(k).to(torch.bfloat16), sd[k].to(torch.bfloat16))
    assert not src.has("no.such.key")

    class Target:
        pass
    a, b = Target(), Target()
    WeightLoader(src, target=a, spec=build_spec(L, 10)).run()
    from flashrt_b200.weight_loader import DictSource
    WeightLoader(DictSource({k: v.to(torch.bfloat16) for k, v in sd.items()}), target=b, spec=build_spec(L, 10)).run()
    assert a.w_qkv.shape == (L, 2560, 1024) and a.w_d.shape == (L, 1024, 4096)
    assert torch.equal(a.w_qkv.view(torch.uint8), b.w_qkv.view(torch.uint8))
    assert np.allclose(a.ws_gu, b.ws_gu)
    # the NVFP4 spec keeps bf16 (N, K) weights for the device-side quantiser
    c = Target()
    WeightLoader(src, target=c, spec=build_spec(L, 10, "nvfp4")).run()
    assert len(c.wb_qkv) == L and c.wb_qkv[0].shape == (2560, 1024) and c.wb_qkv[0].dtype == torch.bfloat16


def test_precision_spec_reads_and_rewrites_the_references_json(tmp_path):
    """``precision_spec_reference.json`` was written by the reference's own ``ModelPrecisionSpec.to_json``
    (tests/golden/make_precision_spec_golden.py): the mirror loads it, keeps every field, and writes the same document."""
    import json
    from flashrt_b200.precision_spec import ModelPrecisionSpec, PrecisionSpec
    gold = os.path.join(os.path.dirname(__file__), "golden", "precision_spec_reference.json")
    m = ModelPrecisionSpec.from_json(gold)
    m.validate()
    e = m.decoder_layer_specs["decoder_attn_qkv_w_3__step_7"]
    assert (e.dtype, e.granularity, e.scheme, e.scale_source) == ("fp8_e4m3", "per_tensor", "symmetric", "calibration")
    assert e.scale.dtype == np.float32 and abs(float(e.scale[0]) - 0.0123) < 1e-7
    assert (e.calibration_method, e.calibration_samples, e.calibration_percentile) == ("percentile", 8, 99.9)
    assert set(m.encoder_layer_specs) == {"encoder_ffn_down_w_0"} and set(m.activation_specs) == {"vision_patch"}
    assert m.weight_specs["decoder_ffn_down_w_1"].scale_source == "manual"
    out = str(tmp_path / "again.json")
    m.to_json(out)
    assert json.load(open(out)) == json.load(open(gold))
    # what no kernel computes is refused, as the reference's table refuses what its kernels lack
    for bad in (dict(dtype="int8"), dict(granularity="per_channel"), dict(dtype="nvfp4"),
                dict(dtype="nvfp4", granularity="per_group", group_size=32)):
        with pytest.raises(NotImplementedError):
            PrecisionSpec(**bad).validate()
    with pytest.raises(ValueError):
        PrecisionSpec(group_size=16).validate()
    with pytest.raises(ValueError):
        PrecisionSpec(scheme="asymmetric").validate()
    PrecisionSpec(dtype="nvfp4", granularity="per_group", group_size=16).validate()


def test_precision_spec_snapshot_of_a_decoder():
    from flashrt_b200.precision_spec import snapshot_decoder
    act = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 4) + 1
    raw = np.ones((2, 3, 2), np.float32) * 0.5
    spec = snapshot_decoder(act, ("qkv", "o", "gu", "d"), {"decoder_attn_qkv_w": np.array([0.1, 0.2, 0.3], np.float32)},
                            precision="fp8", method="max", samples=8, percentile=None, raw_scale=raw)
    spec.validate()
    assert len(spec.decoder_layer_specs) == 2 * 3 * (4 + 2)
    assert float(spec.decoder_layer_specs["decoder_ffn_gate_up_w_2__step_1"].scale[0]) == act[1, 2, 2]
    assert float(spec.decoder_layer_specs["decoder_attn_qkv_w_1__step_0__unnormalised"].scale[0]) == 0.5
    assert abs(float(spec.weight_specs["decoder_attn_qkv_w_2"].scale[0]) - 0.3) < 1e-7
