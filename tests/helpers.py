"""Shared plumbing of the GPU parity tests: oracle inputs -> device tensors ->
C ABI -> numpy.  torch is used for device memory only."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from flash_attention3_b200 import capi, ops
from oracle import golden

TORCH_DTYPE = {"fp16": torch.float16, "bf16": torch.bfloat16}


def dev(x: np.ndarray, dtype: str | None = None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(x))
    if dtype is not None:
        t = t.to(TORCH_DTYPE[dtype])
    return t.cuda().contiguous()


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def poison(shape, dtype, device="cuda"):
    """NaN-filled tensor: an element the kernel forgets to write stays NaN."""
    return torch.full(shape, float("nan"), dtype=dtype, device=device)


class Problem:
    """Seeded (or closed-form) inputs plus the oracle's answers."""

    def __init__(self, b, hq, hkv, s, d, dtype, causal, seed=None, scale=None, sk=None, layout="bhsd",
                 window=(-1, -1), softcap=0.0):
        """s: query length; sk: key length when it differs; layout: how the device tensors are laid
        out ("bhsd" or "bshd") -- the oracle always works on [B,H,S,D]."""
        self.b, self.hq, self.hkv, self.s, self.d = b, hq, hkv, s, d
        self.sk = s if sk is None else sk
        self.layout = layout
        self.window = window
        self.softcap = float(softcap)
        self.dtype, self.causal = dtype, causal
        self.scale = float(scale) if scale is not None else 1.0 / float(np.sqrt(d))
        if seed is None:
            assert dtype == "fp16" and self.sk == s
            self.q, self.k, self.v, self.do = golden.pattern_inputs(b, hq, hkv, s, d)
        else:
            self.q, self.k, self.v, self.do = golden.seeded_inputs(seed, b, hq, hkv, s, d, dtype, sk=self.sk)
        self.ref = golden.backward(self.q, self.k, self.v, self.do, causal, self.scale, dtype, window, self.softcap)

    def to_layout(self, x: np.ndarray) -> np.ndarray:
        """[B,H,S,D] -> the device layout of this problem."""
        return np.ascontiguousarray(x.transpose(0, 2, 1, 3)) if self.layout == "bshd" else x

    def from_layout(self, x: np.ndarray) -> np.ndarray:
        return np.ascontiguousarray(x.transpose(0, 2, 1, 3)) if self.layout == "bshd" else x

    def device_inputs(self):
        t, f = self.dtype, self.to_layout
        return dict(q=dev(f(self.q), t), k=dev(f(self.k), t), v=dev(f(self.v), t), dout=dev(f(self.do), t),
                    out=dev(f(self.ref["out"]), t), lse=dev(self.ref["lse"]))


def run_v2(prob: Problem, deterministic=False, pass_scale=True, poison_ws=True):
    """Call shaobo_fa3_bwd_v2 through ctypes with NaN-poisoned outputs and workspace."""
    lib = capi.load()
    x = prob.device_inputs()
    p = ops.make_params(x["q"], x["k"], prob.causal, prob.scale if pass_scale else None, layout=prob.layout,
                        deterministic=int(deterministic), sync_after_launch=1,
                        window_left=prob.window[0], window_right=prob.window[1], softcap=prob.softcap)
    need = lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p))
    assert need > 0
    ws = torch.full((need,), 0xFF if poison_ws else 0, dtype=torch.uint8, device="cuda")
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    td = TORCH_DTYPE[prob.dtype]
    dq, dk, dv = poison(x["q"].shape, td), poison(x["k"].shape, td), poison(x["k"].shape, td)
    delta = poison(x["lse"].shape, torch.float32)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    torch.cuda.synchronize()
    code = lib.shaobo_fa3_bwd_v2(vp(x["dout"]), vp(x["q"]), vp(x["k"]), vp(x["v"]), vp(x["out"]), vp(x["lse"]),
                                 vp(dq), vp(dk), vp(dv), vp(delta), ctypes.byref(p))
    torch.cuda.synchronize()
    dev_err = lib.shaobo_fa3_b200_device_error(1)
    back = prob.from_layout
    return dict(code=code, device_error=dev_err, dq=back(host(dq)), dk=back(host(dk)), dv=back(host(dv)),
                delta=host(delta))


def metrics(result: dict, prob: Problem, out_dtype="storage") -> dict:
    """out_dtype: "storage" when dq/dk/dv were written in the input dtype, None for fp32 outputs."""
    dt = prob.dtype if out_dtype == "storage" else None
    m = {"delta": golden.compare(result["delta"], prob.ref["delta"])}
    for name in ("dq", "dk", "dv"):
        m[name] = golden.check_gradient(result[name], prob.ref[name], dt)
    return m


def assert_parity(result: dict, prob: Problem, label="", out_dtype="storage"):
    assert result["code"] == capi.STATUS_SUCCESS, (label, capi.status_string(result["code"]))
    assert result["device_error"] == 0, (label, "device error flag", result["device_error"])
    m = metrics(result, prob, out_dtype)
    assert golden.delta_pass(m["delta"]), (label, "delta", m["delta"])
    for name in ("dq", "dk", "dv"):
        assert m[name]["pass"], (label, name, m[name])
    return m
