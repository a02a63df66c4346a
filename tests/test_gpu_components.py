"""Stage-level entry points and the atomic-free split path, against the oracle."""
import ctypes

import numpy as np
import pytest
import torch

from flash_attention3_b200 import capi, ops
from oracle import golden
from tests import helpers

pytestmark = pytest.mark.gpu
vp = lambda t: ctypes.c_void_p(t.data_ptr())


def _sidecar_inputs(prob, mode):
    """aux0, aux1 for shaobo_fa3_bwd_dot_do_o in the given aux mode."""
    if mode == capi.AUX_LSE:
        return helpers.dev(prob.ref["lse"]), None
    return helpers.dev(prob.ref["scores_max"]), helpers.dev(prob.ref["scores_sum"])


@pytest.mark.parametrize("dtype,d", [("fp16", 128), ("bf16", 128), ("fp16", 64), ("bf16", 64)])
@pytest.mark.parametrize("mode", [capi.AUX_LSE, capi.AUX_SMAX_SSUM])
def test_dot_do_o(dtype, d, mode):
    lib = capi.load()
    prob = helpers.Problem(2, 3, 3, 256, d, dtype, True, seed=11 + d)
    x = prob.device_inputs()
    aux0, aux1 = _sidecar_inputs(prob, mode)
    delta = helpers.poison((2, 3, 256), torch.float32)
    side = helpers.poison((2, 3, 256, 3), torch.float32)
    p = ops.make_params(x["q"], x["k"], True, prob.scale, softmax_aux_mode=mode, sync_after_launch=1)
    code = lib.shaobo_fa3_bwd_dot_do_o(vp(x["dout"]), vp(x["out"]), vp(aux0), vp(aux1) if aux1 is not None else None,
                                       vp(delta), vp(side), ctypes.byref(p))
    assert code == 0
    assert golden.delta_pass(golden.compare(helpers.host(delta), prob.ref["delta"]))
    side = helpers.host(side)
    np.testing.assert_array_equal(side[..., 2], helpers.host(delta))
    if mode == capi.AUX_LSE:
        np.testing.assert_allclose(side[..., 0], prob.ref["lse"] * golden.LOG2_E, rtol=1e-6, atol=1e-6)
        assert np.all(side[..., 1] == 1.0)
    else:
        np.testing.assert_allclose(side, prob.ref["packed_sidecar"], rtol=2e-6, atol=2e-6)


def _run_fused5(prob, sidecar):
    lib = capi.load()
    x = prob.device_inputs()
    p = ops.make_params(x["q"], x["k"], prob.causal, prob.scale, sync_after_launch=1)
    need = lib.shaobo_fa3_bwd_fused5_workspace_bytes(ctypes.byref(p))
    ws = torch.full((need,), 0xFF, dtype=torch.uint8, device="cuda")  # the stage must clear it itself
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    td = helpers.TORCH_DTYPE[prob.dtype]
    dq, dk, dv = helpers.poison(x["q"].shape, td), helpers.poison(x["k"].shape, td), helpers.poison(x["k"].shape, td)
    code = lib.shaobo_fa3_bwd_fused5(vp(x["dout"]), vp(x["q"]), vp(x["k"]), vp(x["v"]), vp(sidecar), vp(dq), vp(dk),
                                     vp(dv), ctypes.byref(p))
    return dict(code=code, device_error=lib.shaobo_fa3_b200_device_error(1), dq=helpers.host(dq),
                dk=helpers.host(dk), dv=helpers.host(dv), delta=prob.ref["delta"])


@pytest.mark.parametrize("dtype,d,hq,hkv,causal", [("fp16", 128, 2, 1, True), ("bf16", 64, 4, 4, False)])
def test_fused5_from_oracle_sidecar_smax_ssum_form(dtype, d, hq, hkv, causal):
    """The fused stage accepts the {max*scale*log2e, 1/sum, delta} sidecar of the reference
    golden (scripts/generate_full_bwd_golden.py:190-195), not only the LSE form."""
    prob = helpers.Problem(1, hq, hkv, 384, d, dtype, causal, seed=21)
    r = _run_fused5(prob, helpers.dev(prob.ref["packed_sidecar"]))
    helpers.assert_parity(r, prob)


def _run_split(prob):
    """delta -> shaobo_fa3_bwd_dkv (canonical) -> shaobo_fa3_bwd_dq (canonical): fp32 outputs."""
    lib = capi.load()
    x = prob.device_inputs()
    rows = x["lse"].shape
    delta = helpers.poison(rows, torch.float32)
    side = helpers.poison((*rows, 3), torch.float32)
    p = ops.make_params(x["q"], x["k"], prob.causal, prob.scale, sync_after_launch=1,
                        softmax_aux_mode=capi.AUX_SMAX_SSUM, dkv_path=capi.DKV_PATH_CANONICAL,
                        dq_path=capi.DQ_PATH_CANONICAL)
    smax, ssum = helpers.dev(prob.ref["scores_max"]), helpers.dev(prob.ref["scores_sum"])
    assert lib.shaobo_fa3_bwd_dot_do_o(vp(x["dout"]), vp(x["out"]), vp(smax), vp(ssum), vp(delta), vp(side),
                                       ctypes.byref(p)) == 0
    p.reserved_ptr[capi.RESERVED_PTR_SIDECAR] = side.data_ptr()
    p.reserved_ptr[capi.RESERVED_PTR_DELTA] = delta.data_ptr()
    dq = helpers.poison(x["q"].shape, torch.float32)
    dk = helpers.poison(x["k"].shape, torch.float32)
    dv = helpers.poison(x["k"].shape, torch.float32)
    c1 = lib.shaobo_fa3_bwd_dkv(vp(x["dout"]), vp(x["q"]), vp(x["k"]), vp(x["v"]), None, None, None, None, vp(dk), vp(dv),
                                ctypes.byref(p))
    c2 = lib.shaobo_fa3_bwd_dq(vp(x["dout"]), vp(x["q"]), vp(x["k"]), vp(x["v"]), None, vp(smax), vp(ssum), vp(dq), None,
                               None, ctypes.byref(p))
    return dict(code=c1 or c2, device_error=lib.shaobo_fa3_b200_device_error(1), dq=helpers.host(dq),
                dk=helpers.host(dk), dv=helpers.host(dv), delta=helpers.host(delta))


@pytest.mark.parametrize("dtype,d,hq,hkv,s,causal", [
    ("fp16", 128, 1, 1, 1024, True), ("bf16", 128, 4, 2, 384, True), ("fp16", 64, 2, 2, 256, False),
    ("bf16", 64, 4, 1, 256, True),
])
def test_split_path_components_fp32_outputs(dtype, d, hq, hkv, s, causal):
    prob = helpers.Problem(1, hq, hkv, s, d, dtype, causal, seed=41 + s)
    r = _run_split(prob)
    m = helpers.assert_parity(r, prob, out_dtype=None)
    # fp32 outputs: no output rounding, so the split path is tighter than the gates
    for name in ("dq", "dk", "dv"):
        assert m[name]["rel_l2"] <= 4e-3


@pytest.mark.parametrize("dtype,d,hq,hkv,s,causal", [
    ("fp16", 128, 2, 2, 512, True), ("bf16", 64, 4, 2, 384, False), ("bf16", 128, 8, 2, 256, True),
])
def test_v2_deterministic_is_bitwise_reproducible(dtype, d, hq, hkv, s, causal):
    prob = helpers.Problem(2, hq, hkv, s, d, dtype, causal, seed=51)
    runs = [helpers.run_v2(prob, deterministic=True) for _ in range(3)]
    helpers.assert_parity(runs[0], prob)
    for r in runs[1:]:
        for name in ("dq", "dk", "dv", "delta"):
            assert np.array_equal(runs[0][name], r[name]), name


def test_dk_dv_of_fused_path_are_bitwise_reproducible_when_tiles_are_not_split():
    """With at least 148 (batch x KV head x key tile) units a key tile belongs to one CTA: only dQ
    goes through fp32 reduce-adds, dK and dV have a fixed summation order."""
    prob = helpers.Problem(2, 16, 16, 640, 64, "bf16", True, seed=61)   # 2*16*5 = 160 units
    a, b = helpers.run_v2(prob), helpers.run_v2(prob)
    helpers.assert_parity(a, prob)
    for name in ("dk", "dv", "delta"):
        assert np.array_equal(a[name], b[name])


@pytest.mark.parametrize("b,hq,hkv,s,d,dtype,causal", [
    (1, 4, 4, 2048, 128, "fp16", True),    # 64 units -> 4-way split
    (1, 1, 1, 1024, 128, "fp16", True),    # 8 units -> 8-way split, some parts empty
    (1, 8, 2, 384, 64, "bf16", False),     # GQA: the steps of 4 query heads are cut across CTAs
    (1, 2, 2, 128, 128, "bf16", True),     # a single step per tile: 1 working part, the rest idle
])
def test_split_tiles_match_the_oracle(b, hq, hkv, s, d, dtype, causal):
    prob = helpers.Problem(b, hq, hkv, s, d, dtype, causal, seed=71 + s)
    helpers.assert_parity(helpers.run_v2(prob), prob)


def test_component_status_codes():
    lib = capi.load()
    prob = helpers.Problem(1, 1, 1, 128, 64, "fp16", True, seed=3)
    x = prob.device_inputs()
    side = helpers.dev(prob.ref["packed_sidecar"])
    out32 = helpers.poison(x["q"].shape, torch.float32)
    p = ops.make_params(x["q"], x["k"], True, prob.scale, sync_after_launch=1)
    args = (vp(x["dout"]), vp(x["q"]), vp(x["k"]), vp(x["v"]), None, None, None, vp(out32), vp(out32), vp(out32))
    assert lib.shaobo_fa3_bwd_dkv(*args, ctypes.byref(p)) == capi.STATUS_UNSUPPORTED  # dkv_path 0
    p.dkv_path = capi.DKV_PATH_CANONICAL
    assert lib.shaobo_fa3_bwd_dkv(*args, ctypes.byref(p)) == capi.STATUS_INVALID_VALUE  # no sidecar
    p.dkv_path = capi.DKV_PATH_REFERENCE
    assert lib.shaobo_fa3_bwd_dkv(*args, ctypes.byref(p)) == capi.STATUS_NOT_IMPLEMENTED
    p.dq_path = capi.DQ_PATH_CANONICAL
    assert lib.shaobo_fa3_bwd_dq(*args, ctypes.byref(p)) == capi.STATUS_INVALID_VALUE
    p.reserved_ptr[capi.RESERVED_PTR_SIDECAR] = side.data_ptr()
    p.head_dim_qk = p.head_dim_v = 96
    assert lib.shaobo_fa3_bwd_dq(*args, ctypes.byref(p)) == capi.STATUS_UNSUPPORTED
    assert lib.shaobo_fa3_bwd_dkv(None, None, None, None, None, None, None, None, None, None, None) == capi.STATUS_INVALID_VALUE
    torch.cuda.synchronize()
    assert torch.isnan(out32).all()
