"""Tensor-level wrapper over the C ABI (torch provides device memory only)."""
from __future__ import annotations

import ctypes
import math

import torch

from . import capi

_DTYPES = {torch.float16: capi.DTYPE_FP16, torch.bfloat16: capi.DTYPE_BF16}


class Fa3Error(RuntimeError):
    def __init__(self, entry: str, code: int):
        super().__init__(f"{entry} returned {code} ({capi.status_string(code)})")
        self.code = code


class Fa3DeviceError(RuntimeError):
    """A kernel gave up a bounded wait (1) or found its shared memory misaligned (2): its outputs are
    not valid."""


def _raise_on_device_error(lib, entry: str):
    """After a synchronous call: read and clear the device-side error flag (the C entry points return
    SUCCESS once the work is enqueued; a kernel that ran into trouble can only say so through the flag)."""
    flag = lib.shaobo_fa3_b200_device_error(1)
    if flag != 0:
        raise Fa3DeviceError(f"{entry}: device error flag {flag}")


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _seqused_ptr(t):
    if t is None:
        return None
    if t.dtype != torch.int32 or not t.is_cuda:
        raise TypeError("seqused must be an int32 CUDA tensor")
    return t.data_ptr()


def make_params(q: torch.Tensor, k: torch.Tensor, causal: bool, softmax_scale=None, layout: str = "bhsd",
                seqused_q=None, seqused_k=None, **extra) -> capi.Params:
    """layout "bhsd": q [B,Hq,Sq,D], k [B,Hkv,Sk,D]; "bshd": q [B,Sq,Hq,D], k [B,Sk,Hkv,D].
    seqused_q / seqused_k: optional int32 [B] device tensors, the used length of every batch entry."""
    if layout == "bhsd":
        (b, hq, s, d), hkv, sk = q.shape, k.shape[1], k.shape[2]
    elif layout == "bshd":
        (b, s, hq, d), hkv, sk = q.shape, k.shape[2], k.shape[1]
    else:
        raise ValueError(f"unknown layout {layout!r}")
    p = capi.new_params(batch=b, seqlen_q=s, seqlen_k=sk, num_heads_q=hq, num_heads_kv=hkv,
                        head_dim_qk=d, head_dim_v=d, causal=int(causal), dtype=_DTYPES[q.dtype],
                        layout=capi.LAYOUT_BSHD if layout == "bshd" else capi.LAYOUT_BHSD)
    if softmax_scale is not None:
        p.softmax_scale = float(softmax_scale)
        p.softmax_scale_is_set = 1
    p.seqused_q, p.seqused_k = _seqused_ptr(seqused_q), _seqused_ptr(seqused_k)
    for key, val in extra.items():
        setattr(p, key, val)
    return p


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flash_attention3_b200 has no CPU path: tensors must live on a CUDA device")
        if t is not None and not t.is_contiguous():
            raise RuntimeError("contiguous tensors are required ([B,H,S,D] or [B,S,H,D])")


def _check_problem(q, k, v, layout, out=None, dout=None, softmax_lse=None):
    """Shapes, dtypes and devices of one fixed-length problem: the C ABI takes raw pointers, so a
    tensor of the wrong size would be read or written out of bounds."""
    if q.dim() != 4 or k.dim() != 4:
        raise ValueError("q and k must be 4-D ([B,H,S,D] or [B,S,H,D])")
    if q.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {q.dtype}: fp16 or bf16")
    if v.shape != k.shape:
        raise ValueError(f"v {tuple(v.shape)} must have the shape of k {tuple(k.shape)}")
    hq, hkv = (q.shape[2], k.shape[2]) if layout == "bshd" else (q.shape[1], k.shape[1])
    sq = q.shape[1] if layout == "bshd" else q.shape[2]
    if q.shape[0] != k.shape[0] or q.shape[3] != k.shape[3] or hkv == 0 or hq % hkv != 0:
        raise ValueError(f"q {tuple(q.shape)} and k {tuple(k.shape)} do not describe one problem")
    for name, t in (("k", k), ("v", v), ("out", out), ("dout", dout)):
        if t is None:
            continue
        if t.dtype != q.dtype or t.device != q.device:
            raise TypeError(f"{name} must have the dtype and device of q")
        if name in ("out", "dout") and t.shape != q.shape:
            raise ValueError(f"{name} {tuple(t.shape)} must have the shape of q {tuple(q.shape)}")
    if softmax_lse is not None:
        if softmax_lse.dtype != torch.float32 or softmax_lse.device != q.device:
            raise TypeError("softmax_lse must be fp32 on the device of q")
        if tuple(softmax_lse.shape) != (q.shape[0], hq, sq):
            raise ValueError(f"softmax_lse {tuple(softmax_lse.shape)} must be [B,Hq,Sq] = {(q.shape[0], hq, sq)}")


def fa3_bwd(dout, q, k, v, out, softmax_lse, causal: bool, softmax_scale=None, deterministic=False,
            workspace=None, return_delta=False, sync=False, layout: str = "bhsd", window=(-1, -1),
            seqused_q=None, seqused_k=None, outputs=None, softcap: float = 0.0):
    """dq, dk, dv (and delta) = backward of softmax(q k^T * scale) v.

    layout "bhsd": q, out, dout [B,Hq,Sq,D]; k, v [B,Hkv,Sk,D].  layout "bshd": [B,Sq,Hq,D] and
    [B,Sk,Hkv,D].  fp16 or bf16; softmax_lse: fp32 [B,Hq,Sq] natural log in both layouts.  With
    causal=True and Sq != Sk the diagonal is aligned bottom-right.  window = (left, right): query i
    sees keys i+off-left .. i+off+right (off = Sk - Sq), -1 = unbounded; causal forces right = 0.
    seqused_q / seqused_k (int32 [B]): only the first seqused[b] rows of batch entry b take part; the
    gradient rows behind them are zero.  outputs = (dq, dk, dv): write into these tensors instead of
    allocating.  Calls shaobo_fa3_bwd_v2.
    """
    _require_cuda(dout, q, k, v, out, softmax_lse)
    _check_problem(q, k, v, layout, out, dout, softmax_lse)
    lib = capi.load()
    p = make_params(q, k, causal, softmax_scale, layout=layout, seqused_q=seqused_q, seqused_k=seqused_k,
                    softcap=float(softcap), deterministic=int(deterministic),
                    sync_after_launch=int(sync), window_left=int(window[0]), window_right=int(window[1]))
    need = lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p))
    if need == 0:
        raise Fa3Error("shaobo_fa3_bwd_v2_validate", lib.shaobo_fa3_bwd_v2_validate(ctypes.byref(p)))
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    p.workspace = workspace.data_ptr()
    p.workspace_bytes = workspace.numel() * workspace.element_size()
    if outputs is None:
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    else:
        dq, dk, dv = outputs
        _require_cuda(dq, dk, dv)
        for t, like in ((dq, q), (dk, k), (dv, v)):
            if t.shape != like.shape or t.dtype != like.dtype or t.device != like.device:
                raise ValueError("outputs must match q, k, v in shape, dtype and device")
    delta = (torch.empty((p.batch, p.num_heads_q, p.seqlen_q), dtype=torch.float32, device=q.device)
             if return_delta else None)
    with torch.cuda.device(q.device):
        p.reserved_ptr[capi.RESERVED_PTR_STREAM] = torch.cuda.current_stream().cuda_stream or None
        code = lib.shaobo_fa3_bwd_v2(_ptr(dout), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(softmax_lse),
                                     _ptr(dq), _ptr(dk), _ptr(dv), _ptr(delta), ctypes.byref(p))
    if code != capi.STATUS_SUCCESS:
        raise Fa3Error("shaobo_fa3_bwd_v2", code)
    if sync:
        _raise_on_device_error(lib, "shaobo_fa3_bwd_v2")
    return (dq, dk, dv, delta) if return_delta else (dq, dk, dv)


def fa3_fwd(q, k, v, causal: bool, softmax_scale=None, layout: str = "bhsd", window=(-1, -1), sync=False,
            seqused_q=None, seqused_k=None, softcap: float = 0.0):
    """out, softmax_lse = forward of softmax(q k^T * scale) v (shaobo_fa3_b200_fwd).  Shapes, layouts,
    masks as in fa3_bwd; softmax_lse is fp32 [B,Hq,Sq] natural log."""
    _require_cuda(q, k, v)
    _check_problem(q, k, v, layout)
    lib = capi.load()
    p = make_params(q, k, causal, softmax_scale, layout=layout, seqused_q=seqused_q, seqused_k=seqused_k,
                    softcap=float(softcap), sync_after_launch=int(sync),
                    window_left=int(window[0]), window_right=int(window[1]))
    out = torch.empty_like(q)
    lse = torch.empty((p.batch, p.num_heads_q, p.seqlen_q), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        p.reserved_ptr[capi.RESERVED_PTR_STREAM] = torch.cuda.current_stream().cuda_stream or None
        code = lib.shaobo_fa3_b200_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), ctypes.byref(p))
    if code != capi.STATUS_SUCCESS:
        raise Fa3Error("shaobo_fa3_b200_fwd", code)
    return out, lse


def _varlen_params(q, k, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal, softmax_scale, window,
                   **extra) -> capi.Params:
    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32:
        raise TypeError("cu_seqlens must be int32")
    total_q, hq, d = q.shape
    total_k, hkv, _ = k.shape
    p = capi.new_params(batch=cu_seqlens_q.numel() - 1, seqlen_q=int(max_seqlen_q), seqlen_k=int(max_seqlen_k),
                        num_heads_q=hq, num_heads_kv=hkv, head_dim_qk=d, head_dim_v=d, causal=int(causal),
                        dtype=_DTYPES[q.dtype], layout=capi.LAYOUT_BSHD,
                        window_left=int(window[0]), window_right=int(window[1]),
                        cu_seqlens_q=cu_seqlens_q.data_ptr(), cu_seqlens_k=cu_seqlens_k.data_ptr(),
                        max_seqlen_q=int(max_seqlen_q), max_seqlen_k=int(max_seqlen_k),
                        total_q=int(total_q), total_k=int(total_k), **extra)
    if softmax_scale is not None:
        p.softmax_scale = float(softmax_scale)
        p.softmax_scale_is_set = 1
    return p


def fa3_fwd_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, causal: bool,
                   softmax_scale=None, window=(-1, -1), sync=False):
    """Forward over packed sequences: q [total_q,Hq,D], k/v [total_k,Hkv,D] -> out [total_q,Hq,D],
    softmax_lse fp32 [Hq,total_q]."""
    _require_cuda(q, k, v, cu_seqlens_q, cu_seqlens_k)
    lib = capi.load()
    p = _varlen_params(q, k, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal, softmax_scale,
                       window, sync_after_launch=int(sync))
    out = torch.empty_like(q)
    lse = torch.empty((q.shape[1], q.shape[0]), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        p.reserved_ptr[capi.RESERVED_PTR_STREAM] = torch.cuda.current_stream().cuda_stream or None
        code = lib.shaobo_fa3_b200_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), ctypes.byref(p))
    if code != capi.STATUS_SUCCESS:
        raise Fa3Error("shaobo_fa3_b200_fwd", code)
    return out, lse


def fa3_bwd_varlen(dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int,
                   max_seqlen_k: int, causal: bool, softmax_scale=None, deterministic=False, window=(-1, -1),
                   return_delta=False, sync=False):
    """Backward over packed sequences.  q, out, dout: [total_q, Hq, D]; k, v: [total_k, Hkv, D];
    softmax_lse: fp32 [Hq, total_q]; cu_seqlens_*: int32 device tensors of batch+1 row offsets.
    Returns dq, dk, dv in the shapes of q, k, v (and delta [Hq, total_q]).  Calls shaobo_fa3_bwd_v2."""
    _require_cuda(dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k)
    lib = capi.load()
    total_q, hq = q.shape[0], q.shape[1]
    p = _varlen_params(q, k, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal, softmax_scale,
                       window, deterministic=int(deterministic), sync_after_launch=int(sync))
    need = lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p))
    if need == 0:
        raise Fa3Error("shaobo_fa3_bwd_v2_validate", lib.shaobo_fa3_bwd_v2_validate(ctypes.byref(p)))
    workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    p.workspace, p.workspace_bytes = workspace.data_ptr(), need
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty((hq, total_q), dtype=torch.float32, device=q.device) if return_delta else None
    with torch.cuda.device(q.device):
        p.reserved_ptr[capi.RESERVED_PTR_STREAM] = torch.cuda.current_stream().cuda_stream or None
        code = lib.shaobo_fa3_bwd_v2(_ptr(dout), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(softmax_lse),
                                     _ptr(dq), _ptr(dk), _ptr(dv), _ptr(delta), ctypes.byref(p))
    if code != capi.STATUS_SUCCESS:
        raise Fa3Error("shaobo_fa3_bwd_v2", code)
    if sync:
        _raise_on_device_error(lib, "shaobo_fa3_bwd_v2")
    return (dq, dk, dv, delta) if return_delta else (dq, dk, dv)


class HostBackward:
    """The backward for callers whose tensors live in host memory ([B,H,S,D], pinned for full speed).

    A call copies the inputs to the GPU, runs shaobo_fa3_bwd_v2 and copies dq, dk, dv back.  Large
    problems are cut into contiguous (batch, KV head) shards (the backward has no reduction across
    them) that go round-robin over a few CUDA streams, so that the host-to-device copy of one shard,
    the kernels of another and the device-to-host copy of a third overlap: over PCIe the copies, not
    the kernels, bound such a call.  Device staging tensors, workspaces and the parameter blocks of
    every shard are built once, here; a call itself only issues copies and launches.
    """

    def __init__(self, batch, heads_q, heads_kv, seqlen, head_dim, dtype, causal, softmax_scale=None,
                 shards=None, streams=3, device="cuda"):
        from . import sharding
        self.group = heads_q // heads_kv
        units = batch * heads_kv
        if shards is None:
            # a shard per ~8 MB of traffic: below that the per-shard host work (copies, launches)
            # costs more than the overlap gains (measured on B=1,H=4,S=2048,D=128, 16.8 MB: one shard
            # 389 us, two 370 us, four 419 us)
            elem = torch.empty((), dtype=dtype).element_size()
            total = (5 * batch * heads_q + 4 * batch * heads_kv) * seqlen * head_dim * elem
            shards = max(1, min(8, total // (8 << 20)))
        n = max(1, min(int(shards), units))
        self.shards = [sh for part in sharding.plan(batch, heads_kv, n) for sh in part]
        self._slice = sharding.slice_tensors
        mk = lambda *shape, dt=dtype: torch.empty(shape, dtype=dt, device=device)
        q_shape, kv_shape = (batch, heads_q, seqlen, head_dim), (batch, heads_kv, seqlen, head_dim)
        self.q, self.dout, self.out, self.dq = mk(*q_shape), mk(*q_shape), mk(*q_shape), mk(*q_shape)
        self.k, self.v, self.dk, self.dv = mk(*kv_shape), mk(*kv_shape), mk(*kv_shape), mk(*kv_shape)
        self.lse = mk(batch, heads_q, seqlen, dt=torch.float32)
        self.streams = [torch.cuda.Stream(device=device) for _ in range(max(1, min(streams, len(self.shards))))]
        self.lib = capi.load()
        # per shard: device views, parameter block (workspace and stream filled in), C arguments
        self.plans = []
        need = 0
        for i, sh in enumerate(self.shards):
            d_q, d_kv, d_row = self._slice(sh, self.group, [self.q, self.dout, self.out, self.dq],
                                           [self.k, self.v, self.dk, self.dv], [self.lse])
            p = make_params(d_q[0], d_kv[0], causal, softmax_scale)
            need = max(need, self.lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p)))
            self.plans.append((sh, d_q, d_kv, d_row, p))
        if need == 0:
            raise Fa3Error("shaobo_fa3_bwd_v2_validate", capi.STATUS_UNSUPPORTED)
        self.workspaces = [torch.empty(need, dtype=torch.uint8, device=device) for _ in self.streams]
        self.calls = []
        for i, (sh, d_q, d_kv, d_row, p) in enumerate(self.plans):
            lane = i % len(self.streams)
            p.workspace, p.workspace_bytes = self.workspaces[lane].data_ptr(), need
            p.reserved_ptr[capi.RESERVED_PTR_STREAM] = self.streams[lane].cuda_stream
            args = tuple(_ptr(t) for t in (d_q[1], d_q[0], d_kv[0], d_kv[1], d_q[2], d_row[0], d_q[3], d_kv[2], d_kv[3]))
            self.calls.append(args + (None, ctypes.byref(p)))
        self._host_key, self._host_views = None, None
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in (self.q, self.k, self.v, self.dout, self.out, self.lse))
        self.d2h_bytes = sum(t.numel() * t.element_size() for t in (self.dq, self.dk, self.dv))

    def __call__(self, dout, q, k, v, out, softmax_lse, dq, dk, dv):
        """All nine arguments are host tensors; dq, dk, dv are written.  Returns when the work has been
        queued: the caller's current stream waits for it (synchronise that stream before reading)."""
        main = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(main)
        # the per-shard views of the host tensors are kept for the next call with the same tensors
        key = tuple(t.data_ptr() for t in (dout, q, k, v, out, softmax_lse, dq, dk, dv))
        if key != self._host_key:
            if len(self.plans) == 1:
                self._host_views = [([q, dout, out, dq], [k, v, dk, dv], [softmax_lse])]
            else:
                self._host_views = [self._slice(sh, self.group, [q, dout, out, dq], [k, v, dk, dv], [softmax_lse])
                                    for sh, *_ in self.plans]
            self._host_key = key
        for i, (sh, d_q, d_kv, d_row, _) in enumerate(self.plans):
            st = self.streams[i % len(self.streams)]
            st.wait_event(start)
            h_q, h_kv, h_row = self._host_views[i]
            with torch.cuda.stream(st):
                d_q[0].copy_(h_q[0], non_blocking=True)
                d_kv[0].copy_(h_kv[0], non_blocking=True)
                d_kv[1].copy_(h_kv[1], non_blocking=True)
                d_q[1].copy_(h_q[1], non_blocking=True)
                d_q[2].copy_(h_q[2], non_blocking=True)
                d_row[0].copy_(h_row[0], non_blocking=True)
                code = self.lib.shaobo_fa3_bwd_v2(*self.calls[i])
                if code != capi.STATUS_SUCCESS:
                    raise Fa3Error("shaobo_fa3_bwd_v2", code)
                h_q[3].copy_(d_q[3], non_blocking=True)
                h_kv[2].copy_(d_kv[2], non_blocking=True)
                h_kv[3].copy_(d_kv[3], non_blocking=True)
        for st in self.streams:
            main.wait_stream(st)


class HostBackwardC:
    """The same call as HostBackward, with the shard pipeline inside the library
    (shaobo_fa3_b200_bwd_v2_host): one C call per backward, no per-copy Python overhead.  [B,H,S,D],
    fixed lengths.  The device staging buffer is allocated once, here."""

    def __init__(self, batch, heads_q, heads_kv, seqlen, head_dim, dtype, causal, softmax_scale=None,
                 device="cuda", seqlen_k=None):
        self.lib = capi.load()
        self.p = capi.new_params(batch=batch, seqlen_q=seqlen, seqlen_k=seqlen if seqlen_k is None else seqlen_k,
                                 num_heads_q=heads_q, num_heads_kv=heads_kv, head_dim_qk=head_dim,
                                 head_dim_v=head_dim, causal=int(causal), dtype=_DTYPES[dtype])
        if softmax_scale is not None:
            self.p.softmax_scale = float(softmax_scale)
            self.p.softmax_scale_is_set = 1
        need = self.lib.shaobo_fa3_b200_bwd_v2_host_staging_bytes(ctypes.byref(self.p))
        if need == 0:
            raise Fa3Error("shaobo_fa3_b200_bwd_v2_host_staging_bytes", capi.STATUS_UNSUPPORTED)
        self.staging = torch.empty(need, dtype=torch.uint8, device=device)
        elem = torch.empty((), dtype=dtype).element_size()
        nq, nkv = batch * heads_q * seqlen * head_dim * elem, batch * heads_kv * self.p.seqlen_k * head_dim * elem
        self.h2d_bytes = 3 * nq + 2 * nkv + batch * heads_q * seqlen * 4
        self.d2h_bytes = nq + 2 * nkv

    def __call__(self, dout, q, k, v, out, softmax_lse, dq, dk, dv):
        """Nine host tensors; dq, dk, dv are written once the current stream has been synchronised."""
        for t in (dout, q, k, v, out, softmax_lse, dq, dk, dv):
            if t.is_cuda or not t.is_contiguous():
                raise RuntimeError("contiguous host tensors are required")
        with torch.cuda.device(self.staging.device):
            self.p.reserved_ptr[capi.RESERVED_PTR_STREAM] = torch.cuda.current_stream().cuda_stream or None
            code = self.lib.shaobo_fa3_b200_bwd_v2_host(
                _ptr(dout), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(softmax_lse), _ptr(dq), _ptr(dk), _ptr(dv),
                _ptr(self.staging), self.staging.numel(), ctypes.byref(self.p))
        if code != capi.STATUS_SUCCESS:
            raise Fa3Error("shaobo_fa3_b200_bwd_v2_host", code)


def default_scale(d: int) -> float:
    return 1.0 / math.sqrt(d)
