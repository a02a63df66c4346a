"""Pins the CPU oracle: restated NumPy golden == outputs of the unmodified
reference script (committed fixtures) == scalar C restatement."""
import ctypes
import hashlib
import json
import subprocess

import numpy as np
import pytest

from oracle import golden
from tests.conftest import ROOT

CASES = ["b1_h1_s128_c1", "b1_h1_s128_c0", "b1_hq4_hkv2_s256_c1", "b1_h1_s1024_c1",
         "b2_hq4_hkv1_s128_c0"]


def _sha(arr, dtype):
    return hashlib.sha256(np.ascontiguousarray(arr, dtype=dtype).tobytes()).hexdigest()


@pytest.mark.parametrize("case", CASES)
def test_restatement_matches_reference_script(case, golden_dir):
    fx = np.load(golden_dir / f"ref_{case}.npz")
    digests = json.loads((golden_dir / "ref_digests.json").read_text())[case]["files"]
    b, hq, hkv, s, d, causal = (int(x) for x in fx["shape"])
    stride = int(fx["row_stride"])
    scale = float(fx["softmax_scale"])
    q, k, v, do = golden.pattern_inputs(b, hq, hkv, s, d)
    # the closed-form inputs are bit-identical to the reference's payload files
    assert _sha(q, "<f2") == digests["q.f16"]
    assert _sha(k, "<f2") == digests["k.f16"]
    assert _sha(v, "<f2") == digests["v.f16"]
    assert _sha(do, "<f2") == digests["dout.f16"]
    res = golden.backward(q, k, v, do, bool(causal), scale, "fp16")
    o_ref = golden.from_storage_bits("fp16", fx["o_bits"])
    np.testing.assert_allclose(res["out"][:, :, ::stride], o_ref, rtol=0, atol=2e-6)
    np.testing.assert_allclose(res["scores_max"], fx["scores_max"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(res["scores_sum"], fx["scores_sum"], rtol=1e-6)
    np.testing.assert_allclose(res["delta"], fx["delta"], rtol=1e-5, atol=1e-8)
    for name in ("dq", "dk", "dv"):
        m = golden.compare(res[name][:, :, ::stride], fx[name])
        assert m["nonfinite"] == 0 and m["rel_l2"] < 1e-5, (name, m)
    # packed sidecar definition (reference scripts/generate_full_bwd_golden.py:190-195)
    side = res["packed_sidecar"]
    np.testing.assert_allclose(side[..., 0], fx["scores_max"] * np.float32(scale) * golden.LOG2_E,
                               rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(side[..., 1] * fx["scores_sum"], 1.0, rtol=1e-6)


def _scalar_lib():
    subprocess.run(["make", "-s", "-C", str(ROOT / "oracle")], check=True)
    lib = ctypes.CDLL(str(ROOT / "oracle" / "libgolden_scalar.so"))
    lib.fa3_golden_scalar.restype = ctypes.c_int
    return lib


def scalar_golden(q, k, v, do, causal, scale, dtype):
    lib = _scalar_lib()
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    fp = ctypes.POINTER(ctypes.c_float)
    arrs = [np.ascontiguousarray(t, np.float32) for t in (q, k, v, do)]
    out = np.empty((b, hq, s, d), np.float32)
    lse = np.empty((b, hq, s), np.float32)
    side = np.empty((b, hq, s, 3), np.float32)
    dq = np.empty((b, hq, s, d), np.float32)
    dk = np.empty((b, hkv, s, d), np.float32)
    dv = np.empty((b, hkv, s, d), np.float32)
    code = {"fp16": 0, "bf16": 1, None: -1}[dtype]
    rc = lib.fa3_golden_scalar(
        *[a.ctypes.data_as(fp) for a in arrs], b, hq, hkv, s, d, int(causal),
        ctypes.c_float(scale), code,
        *[a.ctypes.data_as(fp) for a in (out, lse, side, dq, dk, dv)])
    assert rc == 0
    return dict(out=out, lse=lse, packed_sidecar=side, delta=side[..., 2].copy(), dq=dq, dk=dk, dv=dv)


@pytest.mark.parametrize("dtype,d,hq,hkv,causal", [
    ("fp16", 128, 1, 1, True), ("bf16", 64, 4, 2, True), ("bf16", 128, 2, 1, False),
    ("fp16", 64, 2, 2, False),
])
def test_scalar_c_matches_numpy_on_seeded_inputs(dtype, d, hq, hkv, causal):
    s = 128
    scale = 1.0 / np.sqrt(d)
    q, k, v, do = golden.seeded_inputs(7, 1, hq, hkv, s, d, dtype)
    a = golden.backward(q, k, v, do, causal, scale, dtype)
    c = scalar_golden(q, k, v, do, causal, scale, dtype)
    np.testing.assert_allclose(c["lse"], a["lse"], rtol=1e-5, atol=1e-5)
    # O is rounded to storage: allow one-ulp flips on a tiny fraction of elements
    ulp = 2.0 ** (-10 if dtype == "fp16" else -7)
    assert np.mean(np.abs(c["out"] - a["out"]) > 0) < 0.02
    assert np.max(np.abs(c["out"] - a["out"]) / np.maximum(np.abs(a["out"]), 1e-3)) <= 2 * ulp
    for name in ("dq", "dk", "dv"):
        m = golden.compare(c[name], a[name])
        assert m["nonfinite"] == 0 and m["rel_l2"] < 2e-4, (name, m)
    m = golden.compare(c["delta"], a["delta"])
    assert m["rel_l2"] < golden.DELTA_REL, m


def test_scalar_c_matches_numpy_on_reference_pattern():
    q, k, v, do = golden.pattern_inputs(1, 2, 1, 128, 128)
    scale = 0.08838834764831845
    a = golden.backward(q, k, v, do, True, scale, "fp16")
    c = scalar_golden(q, k, v, do, True, scale, "fp16")
    for name in ("dq", "dk", "dv", "delta"):
        m = golden.compare(c[name], a[name])
        assert m["rel_l2"] < 1e-4, (name, m)


def test_bf16_rounding_is_nearest_even():
    import torch
    x = np.random.default_rng(0).standard_normal(1 << 16).astype(np.float32) * 37.0
    ours = golden.round_bf16(x)
    ref = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(ours, ref)
    bits = golden.to_storage_bits("bf16", ours)
    assert np.array_equal(golden.from_storage_bits("bf16", bits), ours)
    h = golden.round_fp16(x)
    assert np.array_equal(golden.from_storage_bits("fp16", golden.to_storage_bits("fp16", h)), h)


def test_lse_identity():
    """exp(s*scale - lse) reproduces prob: the identity the kernels rely on."""
    q, k, v, do = golden.seeded_inputs(3, 1, 1, 1, 128, 64, "bf16")
    scale = 0.125
    r = golden.head_backward(q[0, 0], k[0, 0], v[0, 0], do[0, 0], True, scale, "bf16")
    prob, _, _, _ = golden.head_forward(q[0, 0], k[0, 0], v[0, 0], True, scale, "bf16")
    s = (q[0, 0] @ k[0, 0].T) * np.float32(scale)
    p2 = np.exp(s - r.lse[:, None])
    p2[np.triu(np.ones_like(p2, dtype=bool), 1)] = 0
    np.testing.assert_allclose(p2, prob, rtol=2e-5, atol=1e-7)


# The reference's golden only covers seqlen_q == seqlen_k with a causal or full mask.  For the shapes
# and masks accepted beyond that, the oracle is checked against an independent float64 evaluation of
# the textbook formulas (softmax attention and its gradient), written without the oracle's helpers.
def _textbook_backward(q, k, v, do, scale, visible):
    s = (q @ k.T) * scale
    s = np.where(visible, s, -np.inf)
    m = np.max(s, axis=1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    e = np.where(visible, np.exp(s - m), 0.0)
    z = e.sum(axis=1, keepdims=True)
    p = np.where(z > 0, e / np.where(z > 0, z, 1.0), 0.0)
    o = p @ v
    dp = do @ v.T
    delta = (do * o).sum(axis=1, keepdims=True)
    ds = p * (dp - delta) * scale
    with np.errstate(divide="ignore"):
        lse = np.where(z[:, 0] > 0, m[:, 0] + np.log(np.where(z[:, 0] > 0, z[:, 0], 1.0)), -np.inf)
    return o, lse, ds @ k, ds.T @ q, p.T @ do


@pytest.mark.parametrize("sq,sk,causal,window", [
    (9, 9, True, (-1, -1)), (5, 9, True, (-1, -1)), (9, 5, True, (-1, -1)), (7, 11, False, (-1, -1)),
    (12, 12, True, (3, -1)), (12, 12, False, (2, 4)), (6, 14, False, (0, 5)), (14, 6, True, (4, -1)),
])
def test_oracle_matches_textbook_float64_on_widened_masks(sq, sk, causal, window):
    d, scale = 8, 0.37
    q, k, v, do = golden.seeded_inputs(99, 1, 1, 1, sq, d, "fp16", sk=sk)
    got = golden.backward(q, k, v, do, causal, scale, "fp16", window)
    i = np.arange(sq)[:, None]
    j = np.arange(sk)[None, :]
    off = sk - sq
    left, right = window
    if causal:
        right = 0
    visible = np.ones((sq, sk), bool)
    if right >= 0:
        visible &= j <= i + off + right
    if left >= 0:
        visible &= j >= i + off - left
    o, lse, dq, dk, dv = _textbook_backward(*(x[0, 0].astype(np.float64) for x in (q, k, v, do)), scale, visible)
    # the oracle rounds O to the storage dtype before delta (as the reference does): fp16 spacing
    assert np.abs(got["out"][0, 0] - o).max() < 2e-3
    finite = np.isfinite(lse)
    assert (np.isneginf(got["lse"][0, 0]) == ~finite).all()
    assert np.abs(got["lse"][0, 0][finite] - lse[finite]).max() < 1e-5
    for name, ref in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert np.abs(got[name][0, 0] - ref).max() < 2e-3, name


def test_oracle_softcap_gradients_match_finite_differences():
    """softcap * tanh(x / softcap) is not in the reference: the oracle's gradients for it are checked
    against central differences of a float64 forward."""
    sq, sk, d, cap, scale = 6, 7, 8, 2.0, 0.6
    q, k, v, do = golden.seeded_inputs(3, 1, 1, 1, sq, d, "fp16", sk=sk)
    got = golden.backward(q, k, v, do, True, scale, "fp16", (-1, -1), cap)
    Q, K, V, DO = (x[0, 0].astype(np.float64) for x in (q, k, v, do))
    i = np.arange(sq)[:, None]
    j = np.arange(sk)[None, :]

    def forward(Q, K, V):
        z = cap * np.tanh(Q @ K.T * scale / cap)
        z = np.where(j <= i + sk - sq, z, -np.inf)
        p = np.exp(z - z.max(axis=1, keepdims=True))
        return (p / p.sum(axis=1, keepdims=True)) @ V

    def numeric(f, X, eps=1e-6):
        g = np.zeros_like(X)
        for idx in np.ndindex(X.shape):
            hi, lo = X.copy(), X.copy()
            hi[idx] += eps
            lo[idx] -= eps
            g[idx] = ((f(hi) - f(lo)) * DO).sum() / (2 * eps)
        return g

    assert np.abs(got["dq"][0, 0] - numeric(lambda X: forward(X, K, V), Q)).max() < 2e-3
    assert np.abs(got["dk"][0, 0] - numeric(lambda X: forward(Q, X, V), K)).max() < 2e-3
    assert np.abs(got["dv"][0, 0] - numeric(lambda X: forward(Q, K, X), V)).max() < 1e-5


# The checks above share one thing with the oracle: the hand-derived formula dS = P o (dP - delta).
# This one does not.  torch differentiates a float64 forward, softmax(cap(q k^T * scale) + mask) v,
# by itself, and the oracle's gradients for the inputs the reference rejects (windows, seqlen_q !=
# seqlen_k, softcap, GQA on top) must agree with that.  (The reference cannot pin these: it turns them
# away, reference src/shaobo_fa3_bwd_api.cpp:53-68,109-118.)
@pytest.mark.parametrize("sq,sk,causal,window,softcap,hq,hkv", [
    (40, 40, True, (-1, -1), 0.0, 2, 1),      # the reference's own domain, as a baseline for the method
    (24, 56, True, (-1, -1), 0.0, 2, 2),      # more keys than queries, bottom-right diagonal
    (56, 24, True, (-1, -1), 0.0, 1, 1),      # more queries than keys: the first 32 queries see nothing
    (48, 48, True, (7, -1), 0.0, 4, 2),       # causal sliding window
    (33, 47, False, (5, 9), 0.0, 2, 1),       # two-sided window, ragged lengths
    (40, 40, True, (-1, -1), 3.0, 2, 1),      # softcap
    (31, 45, False, (6, 2), 1.5, 4, 2),       # everything at once
])
def test_oracle_gradients_match_autograd_of_a_float64_forward(sq, sk, causal, window, softcap, hq, hkv):
    import torch
    d, scale, b = 16, 0.29, 2
    q, k, v, do = golden.seeded_inputs(123, b, hq, hkv, sq, d, "fp16", sk=sk)
    got = golden.backward(q, k, v, do, causal, scale, "fp16", window, softcap)
    tq, tk, tv = (torch.tensor(x, dtype=torch.float64, requires_grad=True) for x in (q, k, v))
    tdo = torch.tensor(do, dtype=torch.float64)
    group = hq // hkv
    kk, vv = tk.repeat_interleave(group, dim=1), tv.repeat_interleave(group, dim=1)
    z = torch.einsum("bhid,bhjd->bhij", tq, kk) * scale
    if softcap > 0:
        z = softcap * torch.tanh(z / softcap)
    i = torch.arange(sq)[:, None]
    j = torch.arange(sk)[None, :]
    left, right = window
    if causal:
        right = 0
    visible = torch.ones(sq, sk, dtype=torch.bool)
    if right >= 0:
        visible &= j <= i + (sk - sq) + right
    if left >= 0:
        visible &= j >= i + (sk - sq) - left
    # rows that see no key: softmax over an all -inf row is NaN in torch; give them a finite row and
    # zero it afterwards, so that they contribute nothing, which is what the oracle defines
    any_visible = visible.any(dim=1, keepdim=True)
    z = z.masked_fill(~(visible | ~any_visible), float("-inf"))
    p = torch.softmax(z, dim=-1) * any_visible
    out = torch.einsum("bhij,bhjd->bhid", p, vv)
    (out * tdo).sum().backward()
    # the oracle rounds O to fp16 before delta, as the reference does: that moves dS by up to
    # 2^-11 * |dO . O| per row, which bounds the difference to the exact gradients
    for name, grad in (("dq", tq.grad), ("dk", tk.grad), ("dv", tv.grad)):
        ref = grad.numpy()
        err = np.abs(got[name] - ref).max()
        assert err < 3e-3 * max(1.0, np.abs(ref).max()), (name, err)
        assert golden.compare(got[name], ref)["rel_l2"] < 1e-3, name
    np.testing.assert_allclose(got["out"], out.detach().numpy(), atol=2e-3)
