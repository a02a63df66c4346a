"""Benchmark-size configurations: sampled (batch, head) slices against the CPU
oracle, plus size-independent properties on the full tensors.

Inputs are generated on the GPU (seeded) and the forward's O / LSE come from an
fp32 torch softmax; the oracle recomputes everything for the sampled slices
from the downloaded inputs, so its own O and LSE are also cross-checked.

The gate is oracle.golden.check_gradient: rel-L2 <= 5e-3, max-abs <= 2e-2, or half a
storage spacing + 5e-3 where a bf16 output cannot be closer; every check prints how many elements
were off by more than the plain 2e-2 and the largest such error.  delta is gated at 1e-3 relative
against the oracle's delta of the O the kernel was given."""
import ctypes

import numpy as np
import pytest
import torch

from flash_attention3_b200 import capi, ops, synthetic
from oracle import golden
from tests import helpers

pytestmark = pytest.mark.gpu


def _call(q, k, v, do, out, lse, causal, deterministic=False):
    return ops.fa3_bwd(do, q, k, v, out, lse, causal, deterministic=deterministic, return_delta=True, sync=True)


def _gate(actual, expected, dtype, label):
    m = golden.check_gradient(actual, expected, dtype)
    print(f"{label}: rel_l2 {m['rel_l2']:.2e} max_abs {m['max_abs']:.2e} over 2e-2: {m['over_plain']} of "
          f"{np.size(expected)} (worst {m['worst_over_plain']:.2e}), worst excess over tolerance {m['worst_excess']:.2e}")
    assert m["pass"], (label, m)
    return m


def _check_slices(q, k, v, do, out, lse, res, causal, dtype, kv_slices):
    dq, dk, dv, delta = res
    b, hq, s, d = q.shape
    group = hq // k.shape[1]
    scale = 1.0 / np.sqrt(d)
    for (bi, kvh) in kv_slices:
        kf, vf = helpers.host(k[bi, kvh]), helpers.host(v[bi, kvh])
        dk_ref = np.zeros((s, d), np.float32)
        dv_ref = np.zeros((s, d), np.float32)
        for g in range(group):
            h = kvh * group + g
            r = golden.head_backward(helpers.host(q[bi, h]), kf, vf, helpers.host(do[bi, h]), causal, scale, dtype)
            dk_ref += r.dk
            dv_ref += r.dv
            # the torch forward used on the GPU agrees with the oracle's forward
            assert np.abs(helpers.host(lse[bi, h]) - r.lse).max() < 2e-4
            # delta = rowsum(dO o O) of the O the kernel was given (the oracle's own O differs from it by
            # storage rounding of a slightly different fp32 value)
            delta_ref = np.sum(helpers.host(do[bi, h]) * helpers.host(out[bi, h]), axis=1, dtype=np.float32)
            md = golden.compare(helpers.host(delta[bi, h]), delta_ref)
            assert golden.delta_pass(md), (f"delta[{bi},{h}]", md)
            _gate(helpers.host(dq[bi, h]), r.dq, dtype, f"dq[{bi},{h}]")
        _gate(helpers.host(dk[bi, kvh]), dk_ref, dtype, f"dk[{bi},{kvh}]")
        _gate(helpers.host(dv[bi, kvh]), dv_ref, dtype, f"dv[{bi},{kvh}]")


def _properties(q, k, v, do, out, lse, res, causal):
    """Linearity in dO: scaling dO by 2 scales delta, dQ, dK, dV by exactly 2 (powers of two
    commute with every rounding); dK/dV have a fixed summation order, so that holds bitwise."""
    dq, dk, dv, delta = res
    for t in (dq, dk, dv, delta):
        assert torch.isfinite(t).all()
    dq2, dk2, dv2, delta2 = _call(q, k, v, do * 2, out, lse, causal)
    assert torch.equal(dk2.float(), dk.float() * 2)
    assert torch.equal(dv2.float(), dv.float() * 2)
    assert torch.equal(delta2, delta * 2)
    rel = (dq2.float() - 2 * dq.float()).norm() / (2 * dq.float()).norm()
    assert rel < 2e-3  # fp32 reduce-add order may differ between the two runs


@pytest.mark.parametrize("d", [128, 64])
def test_config3_b4_h16_s4096_noncausal_bf16(d):
    q, k, v, do = synthetic.make_inputs(1236, 4, 16, 16, 4096, d, torch.bfloat16)
    out, lse = synthetic.forward_reference(q, k, v, False)
    res = _call(q, k, v, do, out, lse, False)
    assert capi.load().shaobo_fa3_b200_device_error(1) == 0
    _check_slices(q, k, v, do, out, lse, res, False, "bf16", [(0, 0), (3, 15)])
    _properties(q, k, v, do, out, lse, res, False)


def test_config4_gqa_b2_hq32_hkv8_s8192_causal_bf16():
    q, k, v, do = synthetic.make_inputs(1237, 2, 32, 8, 8192, 128, torch.bfloat16)
    out, lse = synthetic.forward_reference(q, k, v, True)
    res = _call(q, k, v, do, out, lse, True)
    assert capi.load().shaobo_fa3_b200_device_error(1) == 0
    _check_slices(q, k, v, do, out, lse, res, True, "bf16", [(0, 0), (1, 7)])
    _properties(q, k, v, do, out, lse, res, True)


def test_config5_one_eighth_shard_b2_h32_s8192_causal_bf16():
    """The per-GPU shard of B=16,H=32 at 8-way sharding (batch 2)."""
    q, k, v, do = synthetic.make_inputs(1238, 2, 32, 32, 8192, 128, torch.bfloat16)
    out, lse = synthetic.forward_reference(q, k, v, True)
    res = _call(q, k, v, do, out, lse, True)
    assert capi.load().shaobo_fa3_b200_device_error(1) == 0
    _check_slices(q, k, v, do, out, lse, res, True, "bf16", [(0, 0), (1, 31)])
    _properties(q, k, v, do, out, lse, res, True)


def test_sharding_by_batch_and_kv_head_is_exact():
    """A shard is a contiguous (batch x KV-head) range with offset pointers and smaller
    batch / head counts; results of the deterministic path are bitwise those of the whole."""
    b, hq, hkv, s, d = 2, 8, 4, 512, 128
    q, k, v, do = synthetic.make_inputs(99, b, hq, hkv, s, d, torch.float16)
    out, lse = synthetic.forward_reference(q, k, v, True)
    whole = _call(q, k, v, do, out, lse, True, deterministic=True)
    # shard 1: batch 0 only; shard 2: batch 1, KV heads 2..3 (query heads 4..7)
    for (bi, kv0, kv1) in [(0, 0, 4), (1, 2, 4), (1, 0, 1)]:
        g = hq // hkv
        sl_q = (slice(bi, bi + 1), slice(kv0 * g, kv1 * g))
        sl_k = (slice(bi, bi + 1), slice(kv0, kv1))
        part = _call(q[sl_q].contiguous(), k[sl_k].contiguous(), v[sl_k].contiguous(), do[sl_q].contiguous(),
                     out[sl_q].contiguous(), lse[sl_q].contiguous(), True, deterministic=True)
        assert torch.equal(part[0], whole[0][sl_q])
        assert torch.equal(part[1], whole[1][sl_k])
        assert torch.equal(part[2], whole[2][sl_k])
        assert torch.equal(part[3], whole[3][sl_q])
