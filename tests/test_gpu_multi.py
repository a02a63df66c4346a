"""Two GPUs, one process: the (batch x KV head) shards of a reduced large configuration run on two
devices and must equal the one-device result bitwise on the deterministic path (the backward has no
reduction across shards).  Skipped on a one-GPU machine."""
import pytest
import torch

from flash_attention3_b200 import ops, sharding, synthetic

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.is_available() and torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_device_shards_equal_the_single_device_result_bitwise():
    b, hq, hkv, s, d = 4, 8, 8, 1024, 128   # the large sharded configuration, reduced
    q, k, v, do = synthetic.make_inputs(77, b, hq, hkv, s, d, torch.bfloat16)
    out, lse = ops.fa3_fwd(q, k, v, True, sync=True)
    whole = ops.fa3_bwd(do, q, k, v, out, lse, True, deterministic=True, return_delta=True, sync=True)
    fused_whole = ops.fa3_bwd(do, q, k, v, out, lse, True, sync=True)
    group = hq // hkv
    for rank, shards in enumerate(sharding.plan(b, hkv, 2)):
        dev = torch.device("cuda", rank)
        for sh in shards:
            (qs, dos, outs), (ks, vs), (lses,) = sharding.slice_tensors(sh, group, [q, do, out], [k, v], [lse])
            to = lambda t: t.contiguous().to(dev)
            part = ops.fa3_bwd(to(dos), to(qs), to(ks), to(vs), to(outs), to(lses), True, deterministic=True,
                               return_delta=True, sync=True)
            fused_part = ops.fa3_bwd(to(dos), to(qs), to(ks), to(vs), to(outs), to(lses), True, sync=True)
            (dq_w,), (dk_w, dv_w), (delta_w,) = sharding.slice_tensors(sh, group, [whole[0]], [whole[1], whole[2]],
                                                                       [whole[3]])
            assert torch.equal(part[0].cpu(), dq_w.cpu())
            assert torch.equal(part[1].cpu(), dk_w.cpu())
            assert torch.equal(part[2].cpu(), dv_w.cpu())
            assert torch.equal(part[3].cpu(), delta_w.cpu())
            # the fused path agrees to rounding: dQ is summed with atomics, and a shard small enough to be
            # split over more thread blocks adds its dK / dV partial sums in another order than the whole
            (fdq_w,), (fdk_w, fdv_w), _ = sharding.slice_tensors(sh, group, [fused_whole[0]],
                                                                  [fused_whole[1], fused_whole[2]], [])
            for got, want in ((fused_part[0], fdq_w), (fused_part[1], fdk_w), (fused_part[2], fdv_w)):
                rel = (got.cpu().float() - want.cpu().float()).norm() / want.cpu().float().norm()
                assert rel < 2e-3
