"""GPU parity of the classifier-free-guidance (batched) decoder: the combine kernel byte for byte against the C
oracle, the two-slot loop against the fp32 restatement of the reference's CFG flow (cosine >= 0.999,
max-abs <= 2e-2 x RMS per step), and a plain batch of two chunks against two single runs."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import block_ref as R  # noqa: E402
from oracle import oracle as O  # noqa: E402


def _cos(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float(a @ b / (a.norm() * b.norm()))


@pytest.mark.parametrize("n", [1600, 2, 100000])
def test_cfg_combine_bit_exact(n):
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, rand_bf16
    rng = np.random.default_rng(n)
    for beta in (1.5, 0.0, 1.0):
        r, vc, vu = rand_bf16(rng, (n,), 2.0), rand_bf16(rng, (n,)), rand_bf16(rng, (n,))
        d_r, d_c, d_u = Dev(r), Dev(vc), Dev(vu)
        fvk.cfg_combine_into_residual(d_r.ptr, d_c.ptr, d_u.ptr, beta, n, 0)
        assert np.array_equal(d_r.get(), O.cfg_combine(r, vc, vu, beta))
        rf, cf, uf = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
        d_r, d_c, d_u = Dev(rf), Dev(cf), Dev(uf)
        fvk.cfg_combine_into_residual(d_r.ptr, d_c.ptr, d_u.ptr, beta, n, 0, f32=True)
        assert np.array_equal(d_r.get(), O.cfg_combine(rf, cf, uf, beta))


@pytest.fixture(scope="module")
def setup():
    from flashrt_b200.pi05_decoder import synthetic_state_dict
    L = 3
    sd = synthetic_state_dict(seed=0, layers=L)
    ck = R.from_hf_state_dict({k: v.to(torch.bfloat16).float() for k, v in sd.items()}, layers=L)
    ck_, cv_ = R.synthetic_prefix_kv(seed=1, layers=L, prefix_len=768)
    uk_, uv_ = R.synthetic_prefix_kv(seed=2, layers=L, prefix_len=768)
    bf = lambda t: t.to(torch.bfloat16)  # noqa: E731
    return dict(sd=sd, ck=ck, L=L, cond=(bf(ck_), bf(cv_)), uncond=(bf(uk_), bf(uv_)))


@pytest.mark.parametrize("precision", ["fp8", "nvfp4"])
def test_cfg_loop_matches_fp32_restatement(setup, precision):
    from flashrt_b200 import load_model
    s = setup
    beta = 1.5
    model = load_model(s["sd"], config="pi05", layers=s["L"], num_steps=10, chunk_size=50, prefix_len=768,
                       precision=precision, batch=2, cfg_beta=beta)
    fe = model.frontend
    fe.set_prefix_pair(s["cond"][0], s["cond"][1], s["uncond"][0], s["uncond"][1])
    model.calibrate([R.synthetic_noise(100 + j) for j in range(4)])
    noise_b = R.synthetic_noise(1).to(torch.bfloat16).float()
    cond = tuple(t.float() for t in s["cond"])
    uncond = tuple(t.float() for t in s["uncond"])
    ref_final, ref_traj = R.denoise_loop_cfg(noise_b, s["ck"], cond, uncond, beta, num_steps=10, layers=s["L"],
                                             return_trajectory=True)
    p = fe.pipeline
    snaps = []
    with torch.cuda.stream(fe.stream):
        p.noise.copy_(noise_b.to(fe.device))
        p.transformer_decoder(fe.stream.cuda_stream, step_hook=lambda k: snaps.append(p.noise.float().clone()))
    fe.stream.synchronize()
    # the 4-bit path is compared with the un-quantised loop here, so its own quantisation error shows
    cos_bar, max_bar = (0.999, 2e-2) if precision == "fp8" else (0.995, 1.5e-1)
    for k, (got, ref) in enumerate(zip(snaps, ref_traj)):
        got = got.cpu()
        rms = float(ref.pow(2).mean().sqrt())
        assert _cos(got, ref) >= cos_bar, f"step {k}"
        assert float((got - ref).abs().max()) <= max_bar * rms, f"step {k}: {float((got - ref).abs().max()) / rms}"
    out = model.predict(noise=noise_b.numpy())             # one CUDA graph: both slots + the combine
    assert out.shape == (50, 32)
    assert np.array_equal(out, snaps[-1].cpu().numpy())
    assert np.array_equal(out, model.predict(noise=noise_b.numpy()))
    # guidance must matter on this input (the two prefixes differ) ...
    plain = R.denoise_loop(noise_b, s["ck"], cond[0], cond[1], num_steps=10, layers=s["L"])
    assert float((ref_final - plain).abs().max()) > 1e-2
    assert fe.kernels_per_loop() == 10 * ((2 + 2) + 1 + p.launches_per_layer() * s["L"] + 1) + 1


def test_fp8_batch2_equals_two_single_runs(setup):
    from flashrt_b200 import load_model
    s = setup
    cal = [R.synthetic_noise(100 + j) for j in range(4)]
    one = load_model(s["sd"], config="pi05", layers=s["L"], num_steps=10, chunk_size=50, prefix_len=768)
    one.set_prefix(*s["cond"])
    one.calibrate(cal)
    two = load_model(s["sd"], config="pi05", layers=s["L"], num_steps=10, chunk_size=50, prefix_len=768, batch=2)
    two.set_prefix(*s["cond"])
    two.calibrate([torch.stack([c, c]) for c in cal])
    noises = np.stack([R.synthetic_noise(10 + j).to(torch.bfloat16).float().numpy() for j in range(2)])
    got = two.predict(noise=noises)
    assert got.shape == (2, 50, 32)
    for j in range(2):
        single = one.predict(noise=noises[j])
        assert _cos(torch.from_numpy(got[j]), torch.from_numpy(single)) >= 0.9999
        assert np.abs(got[j] - single).max() <= 2e-2 * float(np.sqrt((single ** 2).mean()))
