"""shaobo_fa3_b200_bwd_v2_noalloc: the backward for callers that cannot allocate.

A plugin inside another framework's memory arena, or a loop that must not
allocate after start-up, has no workspace to hand to shaobo_fa3_bwd_v2.  The
extra entry point keeps the scratch in a fixed array inside the library
instead.  It must give what the ordinary entry point gives, call after call,
although all calls share that one array and find the previous call's leftovers
in it.  This file is collected last so that a failure here cannot hide one
elsewhere in a stop-at-first-failure run.
"""
import ctypes

import numpy as np
import pytest
import torch

from flash_attention3_b200 import capi, ops, synthetic
from oracle import golden
from tests import helpers

pytestmark = pytest.mark.gpu
vp = lambda t: ctypes.c_void_p(t.data_ptr())


def _call_noalloc(prob, x, deterministic=False):
    """One call through the C ABI with NaN-poisoned outputs and no workspace at all."""
    lib = capi.load()
    p = ops.make_params(x["q"], x["k"], prob.causal, prob.scale, sync_after_launch=1,
                        deterministic=int(deterministic))
    p.workspace, p.workspace_bytes = None, 0
    td = helpers.TORCH_DTYPE[prob.dtype]
    dq, dk, dv = helpers.poison(x["q"].shape, td), helpers.poison(x["k"].shape, td), helpers.poison(x["k"].shape, td)
    delta = helpers.poison(x["lse"].shape, torch.float32)
    code = lib.shaobo_fa3_b200_bwd_v2_noalloc(vp(x["dout"]), vp(x["q"]), vp(x["k"]), vp(x["v"]), vp(x["out"]),
                                               vp(x["lse"]), vp(dq), vp(dk), vp(dv), vp(delta), ctypes.byref(p))
    torch.cuda.synchronize()
    return dict(code=code, device_error=lib.shaobo_fa3_b200_device_error(1), dq=helpers.host(dq),
                dk=helpers.host(dk), dv=helpers.host(dv), delta=helpers.host(delta))


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    # two different problems back to back: the second finds the first one's data in the shared array
    probs = [helpers.Problem(1, 4, 2, 512, 128, "bf16", True, seed=901),
             helpers.Problem(2, 2, 2, 256, 64, "fp16", False, seed=902)]
    for prob in probs:
        expected = helpers.run_v2(prob)              # existing entry point, caller-owned workspace
        x = prob.device_inputs()
        for attempt in range(2):
            got = _call_noalloc(prob, x)
            assert got["code"] == capi.STATUS_SUCCESS and got["device_error"] == 0, (attempt, got["code"])
            # delta has a fixed summation order: identical bits
            assert np.array_equal(got["delta"], expected["delta"]), attempt
            # dQ goes through fp32 reduce-adds whose order may differ from run to run
            for name in ("dq", "dk", "dv"):
                m = golden.compare(got[name], expected[name])
                assert m["nonfinite"] == 0 and m["rel_l2"] <= golden.GRAD_REL_L2 and m["max_abs"] <= golden.GRAD_MAX_ABS, (name, m)
            # and it meets the same gates against the CPU oracle as every other path
            helpers.assert_parity(got, prob, f"noalloc attempt {attempt}")


def test_split_tiles_deterministic_path_and_a_problem_just_under_the_limit():
    lib = capi.load()
    # (a) the benchmark's small shape: its key tiles are split over 136 thread blocks, whose partial
    #     dK/dV sums live in the built-in array too (13 MiB of the 32)
    prob = helpers.Problem(1, 4, 4, 2048, 128, "fp16", True, seed=903)
    x = prob.device_inputs()
    p = ops.make_params(x["q"], x["k"], True, prob.scale)
    need = lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p))
    assert 8 << 20 < need <= capi.STATIC_SCRATCH_BYTES
    for attempt in range(2):
        helpers.assert_parity(_call_noalloc(prob, x), prob, f"split tiles, attempt {attempt}")
    # (b) the atomic-free path through the same array: bitwise the ordinary entry point's result
    expected = helpers.run_v2(prob, deterministic=True)
    got = _call_noalloc(prob, x, deterministic=True)
    assert got["code"] == capi.STATUS_SUCCESS and got["device_error"] == 0
    for name in ("dq", "dk", "dv", "delta"):
        assert np.array_equal(got[name], expected[name]), name
    # (c) 97 % of the array: B=1,H=15,S=4096,D=128 (sampled check of one head against the oracle)
    q, k, v, do = synthetic.make_inputs(904, 1, 15, 15, 4096, 128, torch.bfloat16)
    out, lse = ops.fa3_fwd(q, k, v, False, sync=True)
    p = ops.make_params(q, k, False, None, sync_after_launch=1)
    need = lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p))
    assert 0.95 * capi.STATIC_SCRATCH_BYTES < need <= capi.STATIC_SCRATCH_BYTES
    dq, dk, dv = (helpers.poison(t.shape, t.dtype) for t in (q, k, v))
    code = lib.shaobo_fa3_b200_bwd_v2_noalloc(vp(do), vp(q), vp(k), vp(v), vp(out), vp(lse), vp(dq), vp(dk), vp(dv),
                                               None, ctypes.byref(p))
    torch.cuda.synchronize()
    assert code == capi.STATUS_SUCCESS and lib.shaobo_fa3_b200_device_error(1) == 0
    h = 14
    r = golden.head_backward(helpers.host(q[0, h]), helpers.host(k[0, h]), helpers.host(v[0, h]), helpers.host(do[0, h]),
                             False, 1.0 / np.sqrt(128), "bf16")
    for name, got_t, ref in (("dq", dq, r.dq), ("dk", dk, r.dk), ("dv", dv, r.dv)):
        m = golden.check_gradient(helpers.host(got_t[0, h]), ref, "bf16")
        assert m["pass"], (name, m)
    assert torch.isfinite(dq).all() and torch.isfinite(dk).all() and torch.isfinite(dv).all()


def test_problem_larger_than_the_built_in_scratch_is_refused():
    lib = capi.load()
    # B=4,H=16,S=4096,D=128 needs ~129 MiB of scratch; the array holds 32 MiB
    q = torch.empty(1, dtype=torch.bfloat16, device="cuda")
    p = capi.new_params(batch=4, seqlen_q=4096, seqlen_k=4096, num_heads_q=16, num_heads_kv=16,
                        head_dim_qk=128, head_dim_v=128, causal=0, dtype=capi.DTYPE_BF16)
    assert lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p)) > capi.STATIC_SCRATCH_BYTES
    code = lib.shaobo_fa3_b200_bwd_v2_noalloc(vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), None,
                                               ctypes.byref(p))
    assert code == capi.STATUS_UNSUPPORTED
    # a missing tensor is reported before the size limit, as by the ordinary entry point
    assert lib.shaobo_fa3_b200_bwd_v2_noalloc(None, vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), None,
                                               ctypes.byref(p)) == capi.STATUS_INVALID_VALUE
    # malformed parameters are reported exactly as by the ordinary entry point
    p.struct_size = 0
    assert lib.shaobo_fa3_b200_bwd_v2_noalloc(vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), vp(q), None,
                                               ctypes.byref(p)) == capi.STATUS_INVALID_VALUE
