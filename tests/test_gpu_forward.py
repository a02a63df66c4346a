"""GPU parity of the forward (shaobo_fa3_b200_fwd) against the oracle's forward: O in the storage
dtype and the natural-log LSE.  Gates: O rel-L2 <= 5e-3 and max-abs <= 2e-2 (the gates of the
gradients), LSE within 2e-3 absolute.  Then the round trip: the backward fed with this forward's
O and LSE meets the backward gates."""
import numpy as np
import pytest
import torch

from flash_attention3_b200 import ops
from oracle import golden
from tests.helpers import Problem, dev, host
from tests.test_gpu_varlen import packed_problem

pytestmark = pytest.mark.gpu

# (b, hq, hkv, sq, sk, d, dtype, causal, layout, window)
CASES = [
    (1, 1, 1, 1024, 1024, 128, "fp16", True, "bhsd", (-1, -1)),
    (1, 4, 4, 2048, 2048, 128, "fp16", True, "bhsd", (-1, -1)),
    (2, 4, 4, 512, 512, 64, "bf16", False, "bhsd", (-1, -1)),
    (2, 8, 2, 640, 640, 128, "bf16", True, "bshd", (-1, -1)),
    (1, 2, 2, 200, 333, 64, "fp16", True, "bhsd", (-1, -1)),
    (1, 2, 2, 700, 300, 128, "bf16", True, "bshd", (-1, -1)),
    (1, 4, 2, 1000, 1000, 128, "bf16", False, "bhsd", (-1, -1)),
    (1, 2, 2, 1024, 1024, 64, "fp16", True, "bhsd", (100, -1)),
    (1, 2, 2, 777, 1000, 128, "fp16", False, "bshd", (50, 300)),
    (1, 2, 1, 1, 384, 128, "fp16", True, "bhsd", (-1, -1)),
]


def check_forward(out, lse, ref_out, ref_lse, dtype, label):
    assert np.isfinite(out).all(), label
    m = golden.check_gradient(out, ref_out, dtype)
    assert m["pass"], (label, "out", m)
    both_inf = np.isneginf(lse) & np.isneginf(ref_lse)
    assert (np.isneginf(lse) == np.isneginf(ref_lse)).all(), (label, "lse -inf pattern")
    err = np.abs(np.where(both_inf, 0.0, lse - np.where(both_inf, 0.0, ref_lse)))
    assert err.max() <= 2e-3, (label, "lse", float(err.max()))


@pytest.mark.parametrize("b,hq,hkv,sq,sk,d,dtype,causal,layout,window", CASES)
def test_forward_parity(b, hq, hkv, sq, sk, d, dtype, causal, layout, window):
    prob = Problem(b, hq, hkv, sq, d, dtype, causal, seed=600 + sq + sk, sk=sk, layout=layout, window=window)
    x = prob.device_inputs()
    out, lse = ops.fa3_fwd(x["q"], x["k"], x["v"], causal, prob.scale, layout=layout, window=window, sync=True)
    check_forward(prob.from_layout(host(out)), host(lse), prob.ref["out"], prob.ref["lse"], dtype,
                  (b, hq, hkv, sq, sk, d, dtype, causal, layout, window))
    # round trip: backward on this forward's outputs
    dq, dk, dv = ops.fa3_bwd(x["dout"], x["q"], x["k"], x["v"], out, lse, causal, prob.scale, layout=layout,
                             window=window, sync=True)
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        m = golden.check_gradient(prob.from_layout(host(t)), prob.ref[name], dtype)
        assert m["pass"], (name, m)


def test_forward_rows_without_keys():
    prob = Problem(1, 2, 2, 512, 128, "fp16", True, seed=5, sk=200)
    x = prob.device_inputs()
    out, lse = ops.fa3_fwd(x["q"], x["k"], x["v"], True, prob.scale, sync=True)
    assert torch.isneginf(lse[:, :, :312]).all() and (out[:, :, :312] == 0).all()
    check_forward(host(out), host(lse), prob.ref["out"], prob.ref["lse"], "fp16", "no keys")


def test_forward_large_scores_move_the_reference_maximum():
    """Scores that grow along the key axis force the lazy maximum to move many times."""
    b, h, s, d = 1, 2, 1024, 64
    rng = np.random.default_rng(0)
    q = golden.round_to("fp16", rng.standard_normal((b, h, s, d), dtype=np.float32))
    k = golden.round_to("fp16", rng.standard_normal((b, h, s, d), dtype=np.float32) *
                        np.linspace(0.2, 6.0, s, dtype=np.float32)[None, None, :, None])
    v = golden.round_to("fp16", rng.standard_normal((b, h, s, d), dtype=np.float32))
    scale = 1.0 / np.sqrt(d)
    ref = golden.backward(q, k, v, v * 0, False, scale, "fp16")
    out, lse = ops.fa3_fwd(dev(q, "fp16"), dev(k, "fp16"), dev(v, "fp16"), False, scale, sync=True)
    check_forward(host(out), host(lse), ref["out"], ref["lse"], "fp16", "moving maximum")


def test_forward_packed_sequences():
    seqs = [(100, 100), (300, 450), (77, 77), (513, 513)]
    packed, refs, cu_q, cu_k = packed_problem(seqs, 4, 2, 64, "bf16", True, (-1, -1), seed=4000)
    t = {n: dev(packed[n], "bf16") for n in ("q", "k", "v")}
    out, lse = ops.fa3_fwd_varlen(t["q"], t["k"], t["v"], torch.from_numpy(cu_q).cuda(),
                                  torch.from_numpy(cu_k).cuda(), 513, 513, True, sync=True)
    out, lse = host(out), host(lse)
    for i, ref in enumerate(refs):
        q0, q1 = cu_q[i], cu_q[i + 1]
        check_forward(out[q0:q1].transpose(1, 0, 2)[None], lse[:, q0:q1][None], ref["out"], ref["lse"], "bf16",
                      ("packed", i))
