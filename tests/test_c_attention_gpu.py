"""GPU parity: tcgen05 flash attention vs the fp64 oracle restated from the reference's torch ground truth.
Floating-point bar: cosine >= 0.999 and max-abs <= 2e-2 x RMS(ref) (+ one bf16 ulp of the element, see _run)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


def _run(B, Sq, Skv, Hq, Hkv, D, splits, seed, seqused=None, fused_fp8=False, kv_extra=0, scratch=False, flags=0,
         counters=None):
    from flashrt_b200 import flash_rt_fa2 as fa2
    from gpu_util import Dev, cosine, f32, rand_bf16, zeros
    rng = np.random.default_rng(seed)
    q = rand_bf16(rng, (B, Sq, Hq, D))
    k = rand_bf16(rng, (B, Skv + kv_extra, Hkv, D))
    v = rand_bf16(rng, (B, Skv + kv_extra, Hkv, D))
    d_q, d_k, d_v = Dev(q), Dev(k), Dev(v)
    d_o, d_lse = zeros((B, Sq, Hq, D), np.uint16), zeros((B, Hq, Sq), np.float32)
    qs = (Sq * Hq * D, Hq * D, D)
    ks = ((Skv + kv_extra) * Hkv * D, Hkv * D, D)
    scale = 1.0 / np.sqrt(D)
    kw = dict(kv_splits=splits, flags=flags)
    if scratch:      # split-KV through global scratch (FA2's o_accum / lse_accum layout) instead of the cluster
        ns = max(splits, 1)
        d_oacc, d_lacc = zeros((ns, B, Hq, Sq, D), np.float32), zeros((ns, B, Hq, Sq), np.float32)
        d_cnt = counters or zeros((2 * ((Sq * (Hq // Hkv) + 127) // 128) * Hkv * B,), np.int32)
        kw.update(counters=d_cnt.ptr)
    acc = (d_lacc.ptr, d_oacc.ptr) if scratch else (0, 0)
    d_o8 = d_s = None
    if fused_fp8:
        d_o8, d_s = zeros((B, Sq, Hq, D), np.uint8), f32(0.01)
        kw.update(out_fp8=d_o8.ptr, out_scale=d_s.ptr)
    if seqused is None:
        fa2.fwd_bf16(d_q.ptr, d_k.ptr, d_v.ptr, d_o.ptr, d_lse.ptr, acc[0], acc[1], B, Sq, Skv, Hq, Hkv, D, qs, ks, ks,
                     qs, scale, 148, 0, **kw)
        kv_len = Skv
    else:
        d_u = Dev(np.array([seqused], np.int32))
        (fa2.fwd_bf16_seqused_splitkv if scratch else fa2.fwd_bf16_seqused)(
            d_q.ptr, d_k.ptr, d_v.ptr, d_o.ptr, d_lse.ptr, d_u.ptr, *(acc if scratch else ()), B, Sq, Skv, Hq, Hkv, D,
            qs, ks, ks, qs, scale, 148, 0, **kw)
        kv_len = seqused
    got_bits = d_o.get()
    assert fa2.attention_status() == 0
    ref, lse_ref = O.attention(q, k, v, scale, kv_len)
    got = O.bf16_bits_to_f32(got_bits)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    assert cosine(got, ref) >= 0.9995
    # 2e-2 x RMS, plus one bf16 ulp of the value itself: the result (and P, as in FA2) is stored in bf16, and
    # with short key ranges single elements are several times the RMS
    assert (np.abs(got - ref) <= 2e-2 * rms + np.abs(ref) * 2.0 ** -8).all()
    assert np.abs(d_lse.get() - lse_ref).max() <= 2e-3
    if fused_fp8:
        # the fused FP8 copy is the bit-exact static quantisation of the bf16 result
        assert np.array_equal(d_o8.get(), O.quantize_fp8_static(got_bits, 0.01))
    cnt = None
    if scratch:
        cnt = d_cnt.get()[0::2]
        assert (cnt % 256 == 0).all()                   # every CTA of a tile has arrived: 256 per tile and launch
    return got_bits, d_lse.get(), cnt


@pytest.mark.parametrize("splits", [1, 2, 8, 0])
def test_action_expert_mqa_cross_attention(splits):
    """50 action tokens x 8 heads of 256 against one KV head of 768 prefix + 50 fresh keys."""
    _run(1, 50, 818, 8, 1, 256, splits, seed=splits)


@pytest.mark.parametrize("Sq,Skv", [(10, 778), (1, 1), (50, 112), (50, 113), (16, 224), (17, 1000)])
def test_mqa_ragged_shapes(Sq, Skv):
    _run(1, Sq, Skv, 8, 1, 256, 0, seed=Sq * 1000 + Skv)


def test_fused_fp8_output_and_seqused():
    _run(1, 50, 818, 8, 1, 256, 8, seed=3, fused_fp8=True)
    _run(1, 50, 818, 8, 1, 256, 8, seed=4, seqused=600)
    _run(1, 50, 818, 8, 1, 256, 1, seed=5, seqused=1)


@pytest.mark.parametrize("B,Sq,Hq,Hkv", [(1, 300, 4, 4), (2, 257, 24, 24), (1, 130, 8, 2)])
def test_head_dim_128_self_attention(B, Sq, Hq, Hkv):
    """Bidirectional self-attention, head_dim 128 (video-DiT shape, reduced length)."""
    _run(B, Sq, Sq, Hq, Hkv, 128, 0, seed=B + Sq + Hq)


def test_long_sequence_rows_sum_property():
    """Size-independent property on a long sequence: with V = all ones every output element is exactly 1
    (softmax rows sum to one), whatever the scores."""
    from flashrt_b200 import flash_rt_fa2 as fa2
    from gpu_util import Dev, rand_bf16, zeros
    rng = np.random.default_rng(9)
    B, S, H, D = 1, 4096, 2, 128
    q, k = rand_bf16(rng, (B, S, H, D)), rand_bf16(rng, (B, S, H, D))
    v = np.full((B, S, H, D), 0x3F80, np.uint16)
    d_q, d_k, d_v, d_o = Dev(q), Dev(k), Dev(v), zeros((B, S, H, D), np.uint16)
    st = (S * H * D, H * D, D)
    fa2.fwd_bf16(d_q.ptr, d_k.ptr, d_v.ptr, d_o.ptr, 0, 0, 0, B, S, S, H, H, D, st, st, st, st, 1.0 / np.sqrt(D),
                 148, 0)
    got = O.bf16_bits_to_f32(d_o.get())
    assert fa2.attention_status() == 0
    assert np.abs(got - 1.0).max() <= 2.0 ** -7


@pytest.mark.parametrize("splits", [2, 4, 8])
def test_split_kv_through_global_scratch(splits):
    """Same attention with the kv splits combined through the FA2-layout scratch buffers; run twice on the same
    counters (the wrapper's per-device default buffer serves every call that passes none)."""
    _run(1, 50, 818, 8, 1, 256, splits, seed=20 + splits, scratch=True)
    _run(1, 50, 818, 8, 1, 256, splits, seed=30 + splits, scratch=True, fused_fp8=True)
    _run(1, 17, 500, 8, 1, 256, splits, seed=40 + splits, scratch=True, seqused=333)
    _run(2, 130, 260, 8, 2, 128, 2, seed=50 + splits, scratch=True)


@pytest.mark.parametrize("Sq,Skv,splits,extra", [(50, 818, 8, {}), (50, 818, 4, {}), (50, 818, 2, {}), (3, 130, 8, {}),
                                                  (17, 500, 4, dict(seqused=333)), (50, 818, 8, dict(fused_fp8=True)),
                                                  (50, 600, 8, dict(seqused=70))])
def test_cluster_exchange_equals_scratch_combine(Sq, Skv, splits, extra):
    """With four head-dim parts per (tile, split) the kv splits of a part are one thread-block cluster and exchange
    their partials through distributed shared memory (the scratch and the counters stay untouched); flags bit 3 keeps
    the combine through the global scratch.  Same partials, same weights, same order of the sum: the same bits."""
    a, lse_a, cnt_a = _run(1, Sq, Skv, 8, 1, 256, splits, seed=7, scratch=True, **extra)
    b, lse_b, cnt_b = _run(1, Sq, Skv, 8, 1, 256, splits, seed=7, scratch=True, flags=8, **extra)
    assert np.array_equal(a, b) and np.array_equal(lse_a, lse_b)
    # the default call leaves the counters alone when the device can hold the clusters (else it is the scratch path too)
    assert ((cnt_a == 0).all() or (cnt_a == 256).all()) and (cnt_b == 256).all()


def test_launches_of_different_shapes_share_arrival_counters():
    """A tile's counter grows by 256 per launch whatever the number of CTAs of the tile (32, 8, 2 ...), so one zeroed
    buffer serves calls of any shape in any order."""
    from gpu_util import zeros
    cnt = zeros((64,), np.int32)
    for i, (args, kw) in enumerate([((1, 50, 818, 8, 1, 256, 8), dict(flags=8)), ((1, 50, 818, 8, 1, 256, 2), dict(flags=8)),
                                    ((2, 130, 260, 8, 2, 128, 2), {}), ((1, 50, 818, 8, 1, 256, 8), dict(flags=4)),
                                    ((1, 17, 500, 8, 1, 256, 4), dict(flags=8)), ((1, 50, 818, 8, 1, 256, 8), {})]):
        _run(*args, seed=90 + i, scratch=True, counters=cnt, **kw)


def test_split_kv_scratch_one_cta_per_split():
    """The scratch path picks four head-dim parts per (tile, split) at the action-expert shape; flags bit 2 keeps one
    CTA per (tile, split): the same bar."""
    _run(1, 50, 818, 8, 1, 256, 8, seed=64, scratch=True, flags=4)
    _run(1, 50, 818, 8, 1, 256, 8, seed=74, scratch=True, fused_fp8=True, seqused=700, flags=4)
    _run(1, 3, 130, 8, 1, 256, 8, seed=84, scratch=True, flags=4)


# ------------------------------------------------------------------ two-tile ping-pong kernel (head_dim 128, one kv split)
@pytest.mark.parametrize("B,Sq,Skv,Hq,Hkv", [(1, 300, 300, 4, 4), (2, 257, 257, 24, 24), (1, 130, 777, 8, 2),
                                             (1, 129, 128, 2, 2), (1, 1000, 1000, 3, 3), (2, 520, 512, 4, 1)])
def test_pair_kernel_head_dim_128(B, Sq, Skv, Hq, Hkv):
    """kv_splits = 1 with at least two row tiles routes to the kernel that overlaps softmax and MMAs over two
    query tiles; ragged query tails, a half-empty last tile pair, partial last key chunks, GQA packing."""
    _run(B, Sq, Skv, Hq, Hkv, 128, 1, seed=B * 7 + Sq + Skv + Hq)


def test_pair_kernel_fp8_seqused_and_wide_scores():
    _run(1, 300, 640, 4, 4, 128, 1, seed=61, fused_fp8=True)
    _run(1, 300, 640, 4, 4, 128, 1, seed=62, seqused=333)
    _run(1, 300, 640, 4, 4, 128, 1, seed=63, seqused=1)
    # scores spread over +-60 (log2 domain): the row maximum keeps growing by more than the lazy-rescale
    # threshold across chunks, so the O rescale path runs
    from flashrt_b200 import flash_rt_fa2 as fa2
    from gpu_util import Dev, cosine, rand_bf16, zeros
    rng = np.random.default_rng(64)
    B, S, H, D = 1, 640, 2, 128
    q, k, v = rand_bf16(rng, (B, S, H, D), 1.0), rand_bf16(rng, (B, S, H, D), 1.0), rand_bf16(rng, (B, S, H, D), 1.0)
    d_q, d_k, d_v, d_o = Dev(q), Dev(k), Dev(v), zeros((B, S, H, D), np.uint16)
    st = (S * H * D, H * D, D)
    scale = 4.0 / np.sqrt(D)
    fa2.fwd_bf16(d_q.ptr, d_k.ptr, d_v.ptr, d_o.ptr, 0, 0, 0, B, S, S, H, H, D, st, st, st, st, scale, 148, 0,
                 kv_splits=1)
    assert fa2.attention_status() == 0
    ref, _ = O.attention(q, k, v, scale, S)
    got = O.bf16_bits_to_f32(d_o.get())
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    assert cosine(got, ref) >= 0.9995
    assert (np.abs(got - ref) <= 2e-2 * rms + np.abs(ref) * 2.0 ** -8).all()


def test_pair_kernel_long_sequence_rows_sum_property():
    """20 280 keys (the video-DiT length, 158 full chunks + 56 keys): with V = all ones every output is 1."""
    from flashrt_b200 import flash_rt_fa2 as fa2
    from gpu_util import Dev, rand_bf16, zeros
    rng = np.random.default_rng(10)
    B, Sq, Skv, H, D = 1, 2048, 20280, 2, 128
    q, k = rand_bf16(rng, (B, Sq, H, D)), rand_bf16(rng, (B, Skv, H, D))
    v = np.full((B, Skv, H, D), 0x3F80, np.uint16)
    d_q, d_k, d_v, d_o = Dev(q), Dev(k), Dev(v), zeros((B, Sq, H, D), np.uint16)
    qs, ks = (Sq * H * D, H * D, D), (Skv * H * D, H * D, D)
    fa2.fwd_bf16(d_q.ptr, d_k.ptr, d_v.ptr, d_o.ptr, 0, 0, 0, B, Sq, Skv, H, H, D, qs, ks, ks, qs, 1.0 / np.sqrt(D),
                 148, 0, kv_splits=1)
    got = O.bf16_bits_to_f32(d_o.get())
    assert fa2.attention_status() == 0
    assert np.abs(got - 1.0).max() <= 2.0 ** -7
