"""The split-KV attention entry point that carries its own scratch (for hosts that cannot allocate device memory
where they call it) must give exactly what the entry point with caller-provided scratch gives, on repeated calls,
agree with the fp64 oracle, and refuse shapes beyond its fixed capacity or beyond one wave of CTAs.  Collected last
on purpose."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(seed, Sq, Skv, splits, Hq=8, Hkv=1, D=256):
    from flashrt_b200 import flash_rt_fa2 as fa2
    from gpu_util import Dev, cosine, rand_bf16, zeros
    from oracle import oracle as O
    rng = np.random.default_rng(seed)
    B = 1
    q, k, v = rand_bf16(rng, (B, Sq, Hq, D)), rand_bf16(rng, (B, Skv, Hkv, D)), rand_bf16(rng, (B, Skv, Hkv, D))
    d_q, d_k, d_v = Dev(q), Dev(k), Dev(v)
    qs, ks = (Sq * Hq * D, Hq * D, D), (Skv * Hkv * D, Hkv * D, D)
    scale = 1.0 / np.sqrt(D)
    # existing entry point: scratch owned by the caller
    d_o1, d_l1 = zeros((B, Sq, Hq, D), np.uint16), zeros((B, Hq, Sq), np.float32)
    d_oacc, d_lacc = zeros((splits, B, Hq, Sq, D), np.float32), zeros((splits, B, Hq, Sq), np.float32)
    d_cnt = zeros((2 * ((Sq * (Hq // Hkv) + 127) // 128) * Hkv,), np.int32)
    fa2.fwd_bf16(d_q.ptr, d_k.ptr, d_v.ptr, d_o1.ptr, d_l1.ptr, d_lacc.ptr, d_oacc.ptr, B, Sq, Skv, Hq, Hkv, D, qs, ks,
                 ks, qs, scale, 148, 0, kv_splits=splits, counters=d_cnt.ptr)
    # new entry point: scratch inside the library
    d_o2, d_l2 = zeros((B, Sq, Hq, D), np.uint16), zeros((B, Hq, Sq), np.float32)
    fa2.fwd_bf16_static_scratch(d_q.ptr, d_k.ptr, d_v.ptr, d_o2.ptr, d_l2.ptr, B, Sq, Skv, Hq, Hkv, D, qs, ks, ks, qs,
                                scale, 0, kv_splits=splits)
    a, b = d_o1.get(), d_o2.get()
    assert fa2.attention_status() == 0
    # same kernel, same summation order: the results are identical, not merely close
    assert np.array_equal(a, b)
    assert np.array_equal(d_l1.get(), d_l2.get())
    assert np.abs(a.view(np.int16)).max() > 0
    # and right: the fp64 oracle of the same attention, at the bar of the attention tests
    ref, lse_ref = O.attention(q, k, v, scale, Skv)
    got = O.bf16_bits_to_f32(b)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    assert cosine(got, ref) >= 0.9995
    assert (np.abs(got - ref) <= 2e-2 * rms + np.abs(ref) * 2.0 ** -8).all()
    assert np.abs(d_l2.get() - lse_ref).max() <= 2e-3


def test_static_scratch_matches_caller_scratch_two_calls_in_a_row():
    _case(1, 50, 818, 8)
    _case(2, 50, 818, 8)          # second call reuses the array and the counters the first one left
    _case(3, 33, 500, 4)


def test_static_scratch_head_dim_128():
    _case(4, 40, 1000, 4, Hq=8, Hkv=2, D=128)
    _case(5, 40, 1000, 4, Hq=8, Hkv=2, D=128)


def test_static_scratch_rejects_oversize_requests():
    from flashrt_b200 import flash_rt_fa2 as fa2
    from flashrt_b200._lib import KernelError
    from gpu_util import zeros
    d = zeros((16,), np.uint16)
    with pytest.raises(KernelError, match="-4"):      # 8 heads x 100 tokens = 800 rows > 512
        fa2.fwd_bf16_static_scratch(d.ptr, d.ptr, d.ptr, d.ptr, 0, 1, 100, 818, 8, 1, 256, (1, 1, 1), (1, 1, 1),
                                    (1, 1, 1), (1, 1, 1), 1.0, 0, kv_splits=8)


def test_static_scratch_refuses_a_grid_beyond_one_wave():
    """The kv splits of a tile wait for one another through the scratch, so all of them must be resident at once:
    32 kv heads x 8 splits = 256 CTAs do not fit the device and the call is refused (-2) before anything launches."""
    from flashrt_b200 import flash_rt_fa2 as fa2
    from flashrt_b200._lib import KernelError
    from gpu_util import Dev, rand_bf16, zeros
    rng = np.random.default_rng(9)
    B, Sq, Skv, H, D = 1, 16, 1024, 32, 128
    q, k = rand_bf16(rng, (B, Sq, H, D)), rand_bf16(rng, (B, Skv, H, D))
    d_q, d_k, d_o = Dev(q), Dev(k), zeros((B, Sq, H, D), np.uint16)
    qs, ks = (Sq * H * D, H * D, D), (Skv * H * D, H * D, D)
    with pytest.raises(KernelError, match="-2"):
        fa2.fwd_bf16_static_scratch(d_q.ptr, d_k.ptr, d_k.ptr, d_o.ptr, 0, B, Sq, Skv, H, H, D, qs, ks, ks, qs, 0.1, 0,
                                    kv_splits=8)
    assert fa2.attention_status() == 0
