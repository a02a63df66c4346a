"""GPU parity on the shapes and layouts the reference turns away: [B,S,H,D] tensors, sequence lengths
that are not multiples of the 128-row tile, and seqlen_q != seqlen_k (causal diagonal aligned
bottom-right).  Same gates and the same oracle as the square cases; every call goes through
shaobo_fa3_bwd_v2 with NaN-poisoned outputs and workspace."""
import numpy as np
import pytest

from oracle import golden

from tests.helpers import Problem, assert_parity, run_v2

pytestmark = pytest.mark.gpu

# (b, hq, hkv, sq, sk, d, dtype, causal, layout)
CASES = [
    # [B,S,H,D] on otherwise plain shapes, unsplit (>= 148 key tiles) and split tiles
    (2, 4, 4, 256, 256, 128, "fp16", True, "bshd"),
    (2, 8, 2, 2560, 2560, 64, "bf16", True, "bshd"),
    (1, 40, 40, 512, 512, 128, "bf16", False, "bshd"),
    # ragged lengths
    (1, 2, 2, 200, 200, 128, "fp16", True, "bhsd"),
    (2, 4, 2, 333, 333, 64, "bf16", False, "bhsd"),
    (1, 3, 3, 1000, 1000, 128, "bf16", True, "bshd"),
    (1, 2, 1, 77, 77, 64, "fp16", True, "bhsd"),
    # seqlen_q != seqlen_k, both directions, tile-aligned and not
    (1, 2, 2, 256, 512, 128, "fp16", True, "bhsd"),
    (1, 2, 2, 512, 256, 128, "fp16", True, "bhsd"),
    (1, 4, 2, 300, 700, 64, "bf16", True, "bshd"),
    (1, 4, 2, 700, 300, 128, "bf16", True, "bhsd"),
    (2, 2, 2, 130, 1000, 128, "fp16", False, "bshd"),
    (1, 2, 2, 1, 384, 128, "fp16", True, "bhsd"),
    # one call with >= 148 key tiles (no splitting) and everything at once
    (2, 16, 8, 1111, 1300, 64, "bf16", True, "bshd"),
]


@pytest.mark.parametrize("b,hq,hkv,sq,sk,d,dtype,causal,layout", CASES)
@pytest.mark.parametrize("deterministic", [False, True])
def test_widened_shapes(b, hq, hkv, sq, sk, d, dtype, causal, layout, deterministic):
    prob = Problem(b, hq, hkv, sq, d, dtype, causal, seed=1234 + sq + sk, sk=sk, layout=layout)
    res = run_v2(prob, deterministic=deterministic)
    assert_parity(res, prob, label=f"{(b, hq, hkv, sq, sk, d, dtype, causal, layout, deterministic)}")
    for name in ("dq", "dk", "dv", "delta"):
        assert np.isfinite(res[name]).all(), name


def test_rows_without_a_visible_key_get_zero_gradient():
    """causal, seqlen_q > seqlen_k: the first seqlen_q - seqlen_k queries see nothing (lse = -inf)."""
    prob = Problem(1, 2, 2, 512, 128, "fp16", True, seed=5, sk=200)
    assert np.isneginf(prob.ref["lse"][0, 0, :312]).all()
    res = run_v2(prob)
    assert_parity(res, prob)
    assert (res["dq"][:, :, :312] == 0).all()


def test_layouts_agree_bitwise_on_the_deterministic_path():
    a = Problem(1, 4, 2, 384, 64, "bf16", True, seed=9, layout="bhsd")
    b = Problem(1, 4, 2, 384, 64, "bf16", True, seed=9, layout="bshd")
    ra, rb = run_v2(a, deterministic=True), run_v2(b, deterministic=True)
    for name in ("dq", "dk", "dv", "delta"):
        assert np.array_equal(ra[name], rb[name]), name


# (b, hq, hkv, sq, sk, d, dtype, causal, window)
WINDOW_CASES = [
    (1, 4, 4, 1024, 1024, 128, "fp16", True, (256, -1)),     # causal sliding window
    (1, 4, 2, 1024, 1024, 64, "bf16", True, (100, -1)),      # window narrower than a tile
    (2, 2, 2, 640, 640, 128, "bf16", False, (128, 128)),     # two-sided, tile-aligned
    (1, 2, 2, 777, 1000, 64, "fp16", False, (50, 300)),      # two-sided, ragged, Sq != Sk
    (1, 2, 1, 900, 400, 128, "fp16", True, (64, -1)),        # Sq > Sk: leading queries see nothing
    (1, 2, 2, 512, 2048, 128, "bf16", False, (5, 5)),        # a thin band; key tiles without queries
    (1, 48, 48, 512, 512, 64, "bf16", True, (200, -1)),      # >= 148 key tiles: unsplit path
    (1, 40, 40, 256, 1024, 128, "fp16", False, (8, 64)),     # unsplit, key tiles that no query sees
]


@pytest.mark.parametrize("b,hq,hkv,sq,sk,d,dtype,causal,window", WINDOW_CASES)
@pytest.mark.parametrize("deterministic", [False, True])
def test_sliding_window(b, hq, hkv, sq, sk, d, dtype, causal, window, deterministic):
    prob = Problem(b, hq, hkv, sq, d, dtype, causal, seed=77 + sq + sk, sk=sk, window=window)
    res = run_v2(prob, deterministic=deterministic)
    assert_parity(res, prob, label=f"{(b, hq, hkv, sq, sk, d, dtype, causal, window, deterministic)}")
    for name in ("dq", "dk", "dv", "delta"):
        assert np.isfinite(res[name]).all(), name


def test_a_window_that_covers_everything_is_the_plain_mask():
    """A window at least as wide as the sequence gives bit-identical results to no window
    (the normalisation of reference src/shaobo_fa3_bwd_api.cpp:53-68)."""
    plain = Problem(1, 2, 2, 384, 128, "fp16", True, seed=3)
    wide = Problem(1, 2, 2, 384, 128, "fp16", True, seed=3, window=(383, 500))
    ra, rb = run_v2(plain, deterministic=True), run_v2(wide, deterministic=True)
    for name in ("dq", "dk", "dv"):
        assert np.array_equal(ra[name], rb[name]), name


# (b, hq, hkv, sq, sk, d, dtype, causal, window, softcap)
SOFTCAP_CASES = [
    (1, 4, 4, 512, 512, 128, "bf16", True, (-1, -1), 30.0),
    (2, 4, 2, 384, 384, 64, "fp16", False, (-1, -1), 5.0),
    (1, 2, 2, 300, 700, 128, "fp16", True, (100, -1), 2.0),
    (1, 40, 40, 512, 512, 64, "fp16", True, (-1, -1), 50.0),    # >= 148 key tiles: unsplit path
]


@pytest.mark.parametrize("b,hq,hkv,sq,sk,d,dtype,causal,window,softcap", SOFTCAP_CASES)
@pytest.mark.parametrize("deterministic", [False, True])
def test_softcap(b, hq, hkv, sq, sk, d, dtype, causal, window, softcap, deterministic):
    """Scores capped with softcap * tanh(x / softcap): backward against the oracle, and the forward kernel
    must reproduce the O and LSE the backward was fed."""
    from flash_attention3_b200 import ops
    from tests.helpers import host
    prob = Problem(b, hq, hkv, sq, d, dtype, causal, seed=900 + sq + sk, sk=sk, window=window, softcap=softcap)
    res = run_v2(prob, deterministic=deterministic)
    assert_parity(res, prob, label=f"{(b, hq, hkv, sq, sk, d, dtype, causal, window, softcap, deterministic)}")
    if not deterministic:
        x = prob.device_inputs()
        out, lse = ops.fa3_fwd(x["q"], x["k"], x["v"], causal, prob.scale, window=window, softcap=softcap, sync=True)
        assert golden.check_gradient(host(out), prob.ref["out"], dtype)["pass"]
        ref_lse = prob.ref["lse"]
        finite = np.isfinite(ref_lse)
        assert np.abs(host(lse)[finite] - ref_lse[finite]).max() <= 3e-3
