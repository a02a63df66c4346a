"""GPU parity on packed ("varlen") sequences: q/out/dout [total_q, Hq, D], k/v [total_k, Hkv, D],
softmax_lse [Hq, total_q], row offsets in cu_seqlens_*.  Every sequence is checked against the oracle
run on that sequence alone; rows of neighbouring sequences must not leak into each other."""
import numpy as np
import pytest
import torch

from flash_attention3_b200 import ops
from oracle import golden
from tests.helpers import TORCH_DTYPE, dev, host

pytestmark = pytest.mark.gpu


def packed_problem(seqs, hq, hkv, d, dtype, causal, window, seed):
    """seqs: list of (seqlen_q, seqlen_k).  Returns packed host arrays and per-sequence oracle results."""
    parts, refs = [], []
    for i, (sq, sk) in enumerate(seqs):
        q, k, v, do = golden.seeded_inputs(seed + i, 1, hq, hkv, sq, d, dtype, sk=sk)
        ref = golden.backward(q, k, v, do, causal, 1.0 / np.sqrt(d), dtype, window)
        parts.append((q[0], k[0], v[0], do[0]))
        refs.append(ref)
    pack = lambda xs: np.ascontiguousarray(np.concatenate([x.transpose(1, 0, 2) for x in xs], axis=0))  # [total,H,D]
    packed = dict(
        q=pack([p[0] for p in parts]), k=pack([p[1] for p in parts]), v=pack([p[2] for p in parts]),
        dout=pack([p[3] for p in parts]), out=pack([r["out"][0] for r in refs]),
        lse=np.ascontiguousarray(np.concatenate([r["lse"][0] for r in refs], axis=1)),  # [Hq,total_q]
    )
    cu_q = np.concatenate([[0], np.cumsum([s[0] for s in seqs])]).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum([s[1] for s in seqs])]).astype(np.int32)
    return packed, refs, cu_q, cu_k


CASES = [
    # (seqs, hq, hkv, d, dtype, causal, window)
    ([(128, 128), (256, 256)], 2, 2, 128, "fp16", True, (-1, -1)),
    ([(100, 100), (300, 300), (77, 77), (513, 513)], 4, 2, 64, "bf16", True, (-1, -1)),
    ([(200, 333), (64, 1000), (500, 129)], 2, 2, 128, "bf16", False, (-1, -1)),
    ([(300, 450), (450, 300), (1, 5), (5, 3)], 4, 4, 64, "fp16", True, (-1, -1)),
    ([(640, 640), (130, 130), (384, 384)], 2, 1, 128, "fp16", True, (100, -1)),
    ([(256, 256)] * 3 + [(1024, 1024)], 8, 8, 128, "bf16", True, (-1, -1)),
]


@pytest.mark.parametrize("seqs,hq,hkv,d,dtype,causal,window", CASES)
@pytest.mark.parametrize("deterministic", [False, True])
def test_packed_sequences(seqs, hq, hkv, d, dtype, causal, window, deterministic):
    packed, refs, cu_q, cu_k = packed_problem(seqs, hq, hkv, d, dtype, causal, window, seed=4000)
    t = {n: dev(packed[n], dtype) for n in ("q", "k", "v", "dout", "out")}
    lse = dev(packed["lse"])
    # NaN-poisoned outputs would survive an element the kernels forget: ops allocates with empty(), so
    # poison the caching allocator's next blocks first
    for n in ("q", "k", "v"):
        junk = torch.full_like(t[n], float("nan"))
        del junk
    dq, dk, dv, delta = ops.fa3_bwd_varlen(
        t["dout"], t["q"], t["k"], t["v"], t["out"], lse, torch.from_numpy(cu_q).cuda(),
        torch.from_numpy(cu_k).cuda(), max(s[0] for s in seqs), max(s[1] for s in seqs), causal,
        deterministic=deterministic, window=window, return_delta=True, sync=True)
    dq, dk, dv, delta = host(dq), host(dk), host(dv), host(delta)
    for name, arr in (("dq", dq), ("dk", dk), ("dv", dv), ("delta", delta)):
        assert np.isfinite(arr).all(), name
    for i, ref in enumerate(refs):
        q0, q1, k0, k1 = cu_q[i], cu_q[i + 1], cu_k[i], cu_k[i + 1]
        got = {"dq": dq[q0:q1].transpose(1, 0, 2)[None], "dk": dk[k0:k1].transpose(1, 0, 2)[None],
               "dv": dv[k0:k1].transpose(1, 0, 2)[None]}
        for name in ("dq", "dk", "dv"):
            m = golden.check_gradient(got[name], ref[name], dtype)
            assert m["pass"], (i, seqs[i], name, m)
        assert golden.delta_pass(golden.compare(delta[:, q0:q1][None], ref["delta"])), (i, "delta")


def test_packed_equals_batched_bitwise_on_the_deterministic_path():
    """Equal-length sequences: the packed call and the [B,S,H,D] call are the same computation."""
    b, s, h, d, dtype = 3, 256, 2, 64, "bf16"
    packed, refs, cu_q, cu_k = packed_problem([(s, s)] * b, h, h, d, dtype, True, (-1, -1), seed=9)
    t = {n: dev(packed[n], dtype) for n in ("q", "k", "v", "dout", "out")}
    lse_packed = dev(packed["lse"])
    a = ops.fa3_bwd_varlen(t["dout"], t["q"], t["k"], t["v"], t["out"], lse_packed,
                           torch.from_numpy(cu_q).cuda(), torch.from_numpy(cu_k).cuda(), s, s, True,
                           deterministic=True, sync=True)
    tb = {n: t[n].view(b, s, h, d) for n in t}
    lse_b = lse_packed.view(h, b, s).permute(1, 0, 2).contiguous()
    bb = ops.fa3_bwd(tb["dout"], tb["q"], tb["k"], tb["v"], tb["out"], lse_b, True, deterministic=True,
                     sync=True, layout="bshd")
    for x, y in zip(a, bb):
        assert torch.equal(x.view(-1), y.reshape(-1))


def test_varlen_validation():
    import ctypes
    from flash_attention3_b200 import capi
    lib = capi.load()
    cu = torch.tensor([0, 128], dtype=torch.int32, device="cuda")
    base = dict(batch=1, seqlen_q=128, seqlen_k=128, num_heads_q=1, num_heads_kv=1, head_dim_qk=128,
                head_dim_v=128, cu_seqlens_q=cu.data_ptr(), cu_seqlens_k=cu.data_ptr(), max_seqlen_q=128,
                max_seqlen_k=128, total_q=128, total_k=128)
    ok = capi.new_params(**base)
    assert lib.shaobo_fa3_bwd_v2_validate(ctypes.byref(ok)) == capi.STATUS_SUCCESS
    for broken in (dict(cu_seqlens_k=None), dict(max_seqlen_q=0), dict(total_k=0)):
        p = capi.new_params(**{**base, **broken})
        assert lib.shaobo_fa3_bwd_v2_validate(ctypes.byref(p)) == capi.STATUS_UNSUPPORTED, broken


@pytest.mark.parametrize("deterministic", [False, True])
@pytest.mark.parametrize("layout", ["bhsd", "bshd"])
def test_seqused_lengths(deterministic, layout):
    """Fixed-length slots of which only the first seqused[b] rows take part: every batch entry equals
    the oracle on the truncated sequences, rows behind the used length get zero gradients, and the
    forward writes out = 0 / lse = -inf there."""
    b, hq, hkv, s, d, dtype = 3, 4, 2, 384, 64, "bf16"
    used_q, used_k = [100, 384, 257], [384, 200, 129]
    q, k, v, do = golden.seeded_inputs(31, b, hq, hkv, s, d, dtype)
    refs = [golden.backward(q[i:i + 1, :, :used_q[i]], k[i:i + 1, :, :used_k[i]], v[i:i + 1, :, :used_k[i]],
                            do[i:i + 1, :, :used_q[i]], True, 1.0 / np.sqrt(d), dtype) for i in range(b)]
    to_dev = lambda x: dev(np.ascontiguousarray(x.transpose(0, 2, 1, 3)) if layout == "bshd" else x, dtype)
    back = lambda t: host(t).transpose(0, 2, 1, 3) if layout == "bshd" else host(t)
    sq = torch.tensor(used_q, dtype=torch.int32, device="cuda")
    sk = torch.tensor(used_k, dtype=torch.int32, device="cuda")
    tq, tk, tv, tdo = to_dev(q), to_dev(k), to_dev(v), to_dev(do)
    out, lse = ops.fa3_fwd(tq, tk, tv, True, layout=layout, seqused_q=sq, seqused_k=sk, sync=True)
    dq, dk, dv = ops.fa3_bwd(tdo, tq, tk, tv, out, lse, True, deterministic=deterministic, layout=layout,
                             seqused_q=sq, seqused_k=sk, sync=True)
    out_h, lse_h, dq, dk, dv = back(out), host(lse), back(dq), back(dk), back(dv)
    for i, ref in enumerate(refs):
        uq, uk = used_q[i], used_k[i]
        assert golden.check_gradient(out_h[i:i + 1, :, :uq], ref["out"], dtype)["pass"], (i, "out")
        got_lse, ref_lse = lse_h[i:i + 1, :, :uq], ref["lse"]
        assert (np.isneginf(got_lse) == np.isneginf(ref_lse)).all(), (i, "lse -inf pattern")
        finite = np.isfinite(ref_lse)
        assert np.abs(got_lse[finite] - ref_lse[finite]).max() <= 2e-3, (i, "lse")
        assert (out_h[i, :, uq:] == 0).all() and np.isneginf(lse_h[i, :, uq:]).all(), (i, "forward tail")
        assert golden.check_gradient(dq[i:i + 1, :, :uq], ref["dq"], dtype)["pass"], (i, "dq")
        assert golden.check_gradient(dk[i:i + 1, :, :uk], ref["dk"], dtype)["pass"], (i, "dk")
        assert golden.check_gradient(dv[i:i + 1, :, :uk], ref["dv"], dtype)["pass"], (i, "dv")
        assert (dq[i, :, uq:] == 0).all() and (dk[i, :, uk:] == 0).all() and (dv[i, :, uk:] == 0).all(), (i, "tails")


@pytest.mark.parametrize("deterministic", [False, True])
def test_every_batch_entry_unused(deterministic):
    """seqused_q = 0 everywhere is valid input: no CTA of the GEMM kernel has any work, yet the call must
    stay ordered behind the clearing of the accumulators, and all gradients are exact zeros."""
    b, hq, hkv, s, d = 2, 4, 2, 256, 128
    td = TORCH_DTYPE["bf16"]
    gen = torch.Generator(device="cuda").manual_seed(5)
    q, do = (torch.randn(b, hq, s, d, device="cuda", generator=gen).to(td) for _ in range(2))
    k, v = (torch.randn(b, hkv, s, d, device="cuda", generator=gen).to(td) for _ in range(2))
    zero = torch.zeros(b, dtype=torch.int32, device="cuda")
    out, lse = ops.fa3_fwd(q, k, v, True, seqused_q=zero, sync=True)
    outputs = tuple(torch.full_like(t, float("nan")) for t in (q, k, v))
    for _ in range(3):  # repeated: a convert kernel that ran ahead of the clearing would read stale sums
        dq, dk, dv = ops.fa3_bwd(do, q, k, v, out, lse, True, deterministic=deterministic, seqused_q=zero,
                                 outputs=outputs, sync=True)
        for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):  # (sync=True has checked the device error flag)
            assert (t == 0).all(), name
