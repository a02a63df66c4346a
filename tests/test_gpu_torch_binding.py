"""The torch.library custom op and the autograd.Function built on the C ABI."""
import numpy as np
import pytest
import torch

from oracle import golden
from tests import helpers

pytestmark = pytest.mark.gpu


def test_autograd_backward_matches_the_oracle():
    from flash_attention3_b200 import torch_binding
    prob = helpers.Problem(1, 4, 2, 256, 64, "bf16", True, seed=301)
    x = prob.device_inputs()
    q, k, v = (x[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
    out = torch_binding.attention(q, k, v, causal=True, softmax_scale=prob.scale)
    # the forward kernel agrees with the oracle forward
    assert golden.compare(helpers.host(out), prob.ref["out"])["rel_l2"] < 3e-3
    out.backward(x["dout"])
    torch.cuda.synchronize()
    for name, grad in (("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
        m = golden.check_gradient(helpers.host(grad), prob.ref[name], "bf16")
        assert m["pass"], (name, m)


def test_custom_op_is_registered_with_a_fake_implementation():
    from flash_attention3_b200 import torch_binding  # noqa: F401
    prob = helpers.Problem(1, 2, 2, 128, 128, "fp16", False, seed=302)
    x = prob.device_inputs()
    dq, dk, dv = torch.ops.fa3b200.attention_bwd(x["dout"], x["q"], x["k"], x["v"], x["out"], x["lse"], False,
                                                 prob.scale, True)
    assert golden.check_gradient(helpers.host(dq), prob.ref["dq"], "fp16")["pass"]
    # shape propagation without running the kernel (meta tensors)
    metas = [t.to("meta") for t in (x["dout"], x["q"], x["k"], x["v"], x["out"], x["lse"])]
    mq, mk, mv = torch.ops.fa3b200.attention_bwd(*metas, False, prob.scale, False)
    assert mq.shape == x["q"].shape and mk.shape == x["k"].shape and mv.device.type == "meta"
    torch.library.opcheck(torch.ops.fa3b200.attention_bwd,
                          (x["dout"], x["q"], x["k"], x["v"], x["out"], x["lse"], False, prob.scale, True),
                          test_utils=("test_schema", "test_faketensor"))


def test_host_tensor_call_matches_the_oracle():
    """ops.HostBackward: pinned host tensors in and out, shards pipelined over streams."""
    from flash_attention3_b200 import ops
    prob = helpers.Problem(2, 4, 2, 384, 64, "bf16", True, seed=303)
    td = helpers.TORCH_DTYPE["bf16"]
    pin = lambda x, dt=td: torch.from_numpy(np.ascontiguousarray(x)).to(dt).pin_memory()
    q, k, v, do, out = (pin(x) for x in (prob.q, prob.k, prob.v, prob.do, prob.ref["out"]))
    lse = pin(prob.ref["lse"], torch.float32)
    dq, dk, dv = torch.empty_like(q).pin_memory(), torch.empty_like(k).pin_memory(), torch.empty_like(v).pin_memory()
    for shards in (1, 3, None):
        call = ops.HostBackward(2, 4, 2, 384, 64, td, True, softmax_scale=prob.scale, shards=shards)
        for t in (dq, dk, dv):
            t.fill_(float("nan"))
        call(do, q, k, v, out, lse, dq, dk, dv)
        torch.cuda.synchronize()
        for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
            m = golden.check_gradient(t.float().numpy(), prob.ref[name], "bf16")
            assert m["pass"], (shards, name, m)


def test_calls_from_a_fresh_host_thread():
    """The first CUDA-related thing a new host thread does may be a call into the library (an autograd
    worker, for one): forward and backward must work there as on the main thread."""
    import threading
    from flash_attention3_b200 import ops
    prob = helpers.Problem(1, 4, 2, 256, 64, "bf16", True, seed=304)
    x = prob.device_inputs()
    results = {}

    def work(tag):
        try:
            out, lse = ops.fa3_fwd(x["q"], x["k"], x["v"], True, prob.scale, sync=True)
            dq, _, _ = ops.fa3_bwd(x["dout"], x["q"], x["k"], x["v"], out, lse, True, prob.scale,
                                   deterministic=True, sync=True)
            results[tag] = helpers.host(dq)
        except Exception as exc:  # reported by the assertion below
            results[tag] = exc

    for tag in ("first", "second"):
        t = threading.Thread(target=work, args=(tag,))
        t.start()
        t.join()
    work("main")
    for tag in ("first", "second", "main"):
        assert isinstance(results[tag], np.ndarray), (tag, results[tag])
    assert np.array_equal(results["first"], results["main"]) and np.array_equal(results["second"], results["main"])
    assert golden.check_gradient(results["main"], prob.ref["dq"], "bf16")["pass"]


def test_host_tensor_entry_point_of_the_library():
    """shaobo_fa3_b200_bwd_v2_host: the shard pipeline inside the library, host tensors in and out."""
    from flash_attention3_b200 import ops
    for shape in ((2, 4, 2, 384, 64), (1, 8, 8, 1024, 128)):   # the second one is cut into several shards
        b, hq, hkv, s, d = shape
        prob = helpers.Problem(b, hq, hkv, s, d, "bf16", True, seed=305)
        td = helpers.TORCH_DTYPE["bf16"]
        pin = lambda x, dt=td: torch.from_numpy(np.ascontiguousarray(x)).to(dt).pin_memory()
        q, k, v, do, out = (pin(x) for x in (prob.q, prob.k, prob.v, prob.do, prob.ref["out"]))
        lse = pin(prob.ref["lse"], torch.float32)
        dq, dk, dv = (torch.full_like(t, float("nan")).pin_memory() for t in (q, k, v))
        call = ops.HostBackwardC(b, hq, hkv, s, d, td, True, softmax_scale=prob.scale)
        for _ in range(2):
            call(do, q, k, v, out, lse, dq, dk, dv)
        torch.cuda.synchronize()
        for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
            m = golden.check_gradient(t.float().numpy(), prob.ref[name], "bf16")
            assert m["pass"], (shape, name, m)


def test_autograd_with_window_softcap_and_bshd():
    from flash_attention3_b200 import torch_binding
    prob = helpers.Problem(2, 4, 2, 320, 64, "fp16", True, seed=306, window=(96, -1), softcap=8.0, layout="bshd")
    x = prob.device_inputs()
    q, k, v = (x[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
    out = torch_binding.attention(q, k, v, causal=True, softmax_scale=prob.scale, window=(96, -1), softcap=8.0,
                                  layout="bshd")
    assert golden.check_gradient(prob.from_layout(helpers.host(out)), prob.ref["out"], "fp16")["pass"]
    out.backward(x["dout"])
    torch.cuda.synchronize()
    for name, grad in (("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
        m = golden.check_gradient(prob.from_layout(helpers.host(grad)), prob.ref[name], "fp16")
        assert m["pass"], (name, m)


def test_autograd_with_transposed_views():
    """q, k, v given as strided views ([B,S,H,D] storage seen as [B,H,S,D]): forward and loss.backward()
    work, and the gradients land on the leaf tensors."""
    from flash_attention3_b200 import torch_binding
    prob = helpers.Problem(1, 4, 2, 256, 64, "fp16", True, seed=307)
    x = prob.device_inputs()
    leaves = {n: x[n].transpose(1, 2).contiguous().requires_grad_(True) for n in ("q", "k", "v")}   # [B,S,H,D]
    views = {n: t.transpose(1, 2) for n, t in leaves.items()}                                      # [B,H,S,D], strided
    assert not views["q"].is_contiguous()
    out = torch_binding.attention(views["q"], views["k"], views["v"], causal=True, softmax_scale=prob.scale)
    loss = (out.float() * x["dout"].float()).sum()
    loss.backward()
    torch.cuda.synchronize()
    for name, key in (("dq", "q"), ("dk", "k"), ("dv", "v")):
        grad = leaves[key].grad.transpose(1, 2)
        m = golden.check_gradient(helpers.host(grad), prob.ref[name], "fp16")
        assert m["pass"], (name, m)


def test_wrong_shapes_are_refused_before_the_call():
    from flash_attention3_b200 import ops
    prob = helpers.Problem(1, 2, 2, 128, 64, "fp16", True, seed=308)
    x = prob.device_inputs()
    with pytest.raises(ValueError):
        ops.fa3_bwd(x["dout"], x["q"], x["k"], x["v"], x["out"], x["lse"][:, :, :64].contiguous(), True)
    with pytest.raises(ValueError):
        ops.fa3_bwd(x["dout"], x["q"], x["k"], x["v"][:, :, :64].contiguous(), x["out"], x["lse"], True)
    with pytest.raises(TypeError):
        ops.fa3_bwd(x["dout"], x["q"], x["k"], x["v"], x["out"].float(), x["lse"], True)


def test_two_host_threads_with_separate_staging():
    """Two host threads drive the host-tensor entry point on one GPU at the same time, each with its own
    staging buffer and stream: both get the right answer."""
    import threading
    from flash_attention3_b200 import ops
    td = helpers.TORCH_DTYPE["bf16"]
    probs = [helpers.Problem(1, 8, 8, 1024, 128, "bf16", True, seed=311 + i) for i in range(2)]
    pin = lambda a, dt=td: torch.from_numpy(np.ascontiguousarray(a)).to(dt).pin_memory()
    jobs = []
    for prob in probs:
        q, k, v, do, out = (pin(a) for a in (prob.q, prob.k, prob.v, prob.do, prob.ref["out"]))
        lse = pin(prob.ref["lse"], torch.float32)
        outs = tuple(torch.full_like(t, float("nan")).pin_memory() for t in (q, k, v))
        call = ops.HostBackwardC(1, 8, 8, 1024, 128, td, True, softmax_scale=prob.scale)
        jobs.append((call, (do, q, k, v, out, lse) + outs, outs))
    errors = []

    def work(job):
        call, args, _ = job
        try:
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for _ in range(8):
                    call(*args)
            stream.synchronize()
        except Exception as exc:
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(job,)) for job in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    assert not errors, errors
    for prob, (_, _, outs) in zip(probs, jobs):
        for name, t in zip(("dq", "dk", "dv"), outs):
            m = golden.check_gradient(t.float().numpy(), prob.ref[name], "bf16")
            assert m["pass"], (name, m)
