"""Parity of shaobo_fa3_bwd_v2 (CUDA, through the C ABI) against the CPU oracle.

Gates (benchmark specification): dQ/dK/dV rel-L2 <= 5e-3 and max-abs <= 2e-2,
delta rel-L2 <= 1e-3, no non-finite value.  The one relaxation, for bf16 outputs
whose golden magnitude is >= 4 (storage spacing above the gate), is stated in
oracle.golden.check_gradient.  Outputs and workspace are
NaN-poisoned before every call, so an unwritten element fails the test."""
import ctypes

import numpy as np
import pytest
import torch

from flash_attention3_b200 import capi, ops
from oracle import golden
from tests import helpers

pytestmark = pytest.mark.gpu

SMALL = [
    # b, hq, hkv, s, d, dtype, causal
    (1, 1, 1, 128, 128, "fp16", True),
    (1, 1, 1, 128, 128, "bf16", False),
    (1, 1, 1, 128, 64, "fp16", False),
    (1, 1, 1, 128, 64, "bf16", True),
    (1, 2, 2, 256, 128, "bf16", True),
    (1, 2, 1, 256, 64, "fp16", True),
    (2, 4, 2, 384, 128, "fp16", True),
    (2, 4, 1, 384, 64, "bf16", False),
    (1, 8, 1, 256, 128, "fp16", False),
    (3, 2, 2, 384, 64, "fp16", True),
    (1, 8, 2, 512, 128, "bf16", True),
]


@pytest.mark.parametrize("b,hq,hkv,s,d,dtype,causal", SMALL)
def test_small_shapes_seeded(b, hq, hkv, s, d, dtype, causal):
    prob = helpers.Problem(b, hq, hkv, s, d, dtype, causal, seed=1000 + s + d + hq)
    helpers.assert_parity(helpers.run_v2(prob), prob, label=str((b, hq, hkv, s, d, dtype, causal)))


@pytest.mark.parametrize("hq,hkv,s,causal", [(1, 1, 128, True), (1, 1, 128, False), (4, 2, 256, True), (1, 1, 1024, True)])
def test_reference_pattern_inputs(hq, hkv, s, causal):
    """The closed-form inputs of the reference golden (tiny magnitudes, |x| <= 0.13)."""
    prob = helpers.Problem(1, hq, hkv, s, 128, "fp16", causal, seed=None, scale=0.08838834764831845)
    r = helpers.run_v2(prob)
    assert r["code"] == 0 and r["device_error"] == 0
    m = helpers.metrics(r, prob)
    assert golden.delta_pass(m["delta"]), m["delta"]
    for name in ("dq", "dk", "dv"):
        # gradients are ~1e-4 here, so the absolute gate is vacuous; keep rel-L2 and the
        # reference harness's rmse alternative (src/full_bwd_correctness.cpp:483-487)
        assert m[name]["nonfinite"] == 0
        assert m[name]["rel_l2"] <= golden.GRAD_REL_L2 or m[name]["rmse"] <= 5e-5, (name, m[name])
        assert m[name]["max_abs"] <= golden.GRAD_MAX_ABS


def test_config1_b1_h1_s1024_d128_causal_fp16():
    prob = helpers.Problem(1, 1, 1, 1024, 128, "fp16", True, seed=1234)
    helpers.assert_parity(helpers.run_v2(prob), prob, "C1")


def test_config2_b1_h4_s2048_d128_causal_fp16():
    prob = helpers.Problem(1, 4, 4, 2048, 128, "fp16", True, seed=1235)
    helpers.assert_parity(helpers.run_v2(prob), prob, "C2")


def test_default_scale_matches_explicit_scale():
    prob = helpers.Problem(1, 2, 2, 256, 64, "bf16", True, seed=77)
    a = helpers.run_v2(prob, pass_scale=True)
    b = helpers.run_v2(prob, pass_scale=False)  # softmax_scale_is_set = 0 -> 1/sqrt(D)
    helpers.assert_parity(b, prob)
    assert np.array_equal(a["delta"], b["delta"])
    for name in ("dq", "dk", "dv"):  # small shape: tiles are split, sums go through fp32 reduce-adds
        assert golden.compare(a[name], b[name])["rel_l2"] < 2e-3


def test_softmax_d_is_optional():
    lib = capi.load()
    prob = helpers.Problem(1, 1, 1, 256, 128, "fp16", True, seed=5)
    x = prob.device_inputs()
    p = ops.make_params(x["q"], x["k"], True, prob.scale, sync_after_launch=1)
    need = lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p))
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    dq, dk, dv = (torch.empty_like(x[n]) for n in ("q", "k", "v"))
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    code = lib.shaobo_fa3_bwd_v2(vp(x["dout"]), vp(x["q"]), vp(x["k"]), vp(x["v"]), vp(x["out"]), vp(x["lse"]),
                                 vp(dq), vp(dk), vp(dv), None, ctypes.byref(p))
    assert code == 0
    # delta then lives in the workspace right after the dQ accumulator and the partial-sum slabs of
    # the split key tiles (2 key tiles < 148 SMs, so tiles are split): the fused stage's own workspace
    off = lib.shaobo_fa3_bwd_fused5_workspace_bytes(ctypes.byref(p))
    assert off > 256 * 128 * 4 and off % 256 == 0
    delta = ws[off:off + 256 * 4].view(torch.float32).cpu().numpy()
    assert golden.delta_pass(golden.compare(delta, prob.ref["delta"][0, 0]))
    assert golden.check_gradient(helpers.host(dq), prob.ref["dq"], "fp16")["pass"]


def test_errors_do_not_launch():
    """Invalid calls return a status and leave outputs untouched."""
    lib = capi.load()
    prob = helpers.Problem(1, 1, 1, 128, 64, "fp16", False, seed=9)
    x = prob.device_inputs()
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    dq = helpers.poison(x["q"].shape, torch.float16)
    p = ops.make_params(x["q"], x["k"], False, prob.scale, sync_after_launch=1)
    need = lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p))
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")

    def call(pp, lse=x["lse"]):
        return lib.shaobo_fa3_bwd_v2(vp(x["dout"]), vp(x["q"]), vp(x["k"]), vp(x["v"]), vp(x["out"]),
                                     vp(lse) if lse is not None else None, vp(dq), vp(dq), vp(dq), None,
                                     ctypes.byref(pp))

    assert call(p) == capi.STATUS_INVALID_VALUE  # no workspace
    p.workspace, p.workspace_bytes = ws.data_ptr(), need - 1
    assert call(p) == capi.STATUS_INVALID_VALUE  # short workspace
    p.workspace_bytes = need
    assert call(p, lse=None) == capi.STATUS_INVALID_VALUE
    p.dropout_p = 0.5
    assert call(p) == capi.STATUS_UNSUPPORTED
    p.dropout_p = 0.0
    p.struct_size = 100
    assert call(p) == capi.STATUS_INVALID_VALUE
    torch.cuda.synchronize()
    assert torch.isnan(dq).all()
    assert lib.shaobo_fa3_b200_device_error(1) == 0


def test_ops_wrapper_on_non_default_stream():
    prob = helpers.Problem(1, 2, 1, 256, 128, "bf16", True, seed=31)
    x = prob.device_inputs()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        dq, dk, dv, delta = ops.fa3_bwd(x["dout"], x["q"], x["k"], x["v"], x["out"], x["lse"], True,
                                        prob.scale, return_delta=True)
    stream.synchronize()
    r = dict(code=0, device_error=capi.load().shaobo_fa3_b200_device_error(1), dq=helpers.host(dq),
             dk=helpers.host(dk), dv=helpers.host(dv), delta=helpers.host(delta))
    helpers.assert_parity(r, prob)


def test_cpu_tensors_are_refused():
    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.fa3_bwd(q, q, q, q, q, torch.zeros(1, 1, 128), True)


def test_calls_queued_back_to_back_on_one_workspace():
    """Three different problems enqueued without a synchronisation in between, all on one stream and
    one workspace: the first kernel of a call is launched programmatically behind the last kernel of
    the call in front and must not clear or overwrite the workspace while that one still reads it."""
    lib = capi.load()
    probs = [helpers.Problem(1, 4, 4, 1024, 128, "fp16", True, seed=611),      # split key tiles: slabs in the workspace
             helpers.Problem(1, 4, 2, 512, 128, "bf16", False, seed=612),
             helpers.Problem(2, 2, 2, 384, 64, "bf16", True, seed=613)]
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    calls, need_max = [], 0
    for prob in probs:
        x = prob.device_inputs()
        p = ops.make_params(x["q"], x["k"], prob.causal, prob.scale)
        need_max = max(need_max, lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p)))
        td = helpers.TORCH_DTYPE[prob.dtype]
        out = dict(dq=helpers.poison(x["q"].shape, td), dk=helpers.poison(x["k"].shape, td),
                   dv=helpers.poison(x["k"].shape, td), delta=helpers.poison(x["lse"].shape, torch.float32))
        calls.append((prob, x, p, out))
    ws = torch.full((need_max,), 0xFF, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    codes = []
    for rep in range(2):                       # the second round finds the first one's leftovers
        for prob, x, p, out in calls:
            p.workspace, p.workspace_bytes = ws.data_ptr(), need_max
            codes.append(lib.shaobo_fa3_bwd_v2(vp(x["dout"]), vp(x["q"]), vp(x["k"]), vp(x["v"]), vp(x["out"]),
                                               vp(x["lse"]), vp(out["dq"]), vp(out["dk"]), vp(out["dv"]),
                                               vp(out["delta"]), ctypes.byref(p)))
    torch.cuda.synchronize()
    assert all(c == capi.STATUS_SUCCESS for c in codes), codes
    assert lib.shaobo_fa3_b200_device_error(1) == 0
    for prob, x, p, out in calls:
        got = dict(code=capi.STATUS_SUCCESS, device_error=0, dq=helpers.host(out["dq"]), dk=helpers.host(out["dk"]),
                   dv=helpers.host(out["dv"]), delta=helpers.host(out["delta"]))
        helpers.assert_parity(got, prob, "queued back to back")
