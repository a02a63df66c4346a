"""PyTorch registration of the backward (the consumer the reference names for its C ABI,
reference docs/tridao_fa3_bwd_api.md:48-55, and never shipped).

* ``torch.ops.fa3b200.attention_bwd`` - a ``torch.library`` custom op over the C entry point
  ``shaobo_fa3_bwd_v2`` with a fake (meta) implementation, so it can sit inside traced graphs.
* ``torch.ops.fa3b200.attention_fwd`` - the same for the forward kernel (``shaobo_fa3_b200_fwd``),
  which returns O and the log-sum-exp the backward needs.
* ``attention`` - an ``autograd.Function`` over the two ops, so that the library can be driven from
  ``loss.backward()``.

Tensors are contiguous [B,H,S,D] (or [B,S,H,D] with layout="bshd"), fp16 or bf16, on a CUDA device;
there is no CPU path.  Sliding windows and softcap are passed through to the kernels.
"""
from __future__ import annotations

import torch

from . import ops


@torch.library.custom_op("fa3b200::attention_bwd", mutates_args=(), device_types="cuda")
def attention_bwd(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                  softmax_lse: torch.Tensor, causal: bool, softmax_scale: float,
                  deterministic: bool, window_left: int = -1, window_right: int = -1, softcap: float = 0.0,
                  layout: str = "bhsd") -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    # (the kernels read dense tensors: strided views are copied, as in the forward op)
    dq, dk, dv = ops.fa3_bwd(dout.contiguous(), q.contiguous(), k.contiguous(), v.contiguous(), out.contiguous(),
                             softmax_lse.contiguous(), causal, softmax_scale, deterministic=deterministic,
                             window=(window_left, window_right), softcap=softcap, layout=layout)
    return dq, dk, dv


@attention_bwd.register_fake
def _(dout, q, k, v, out, softmax_lse, causal, softmax_scale, deterministic, window_left=-1, window_right=-1,
      softcap=0.0, layout="bhsd"):
    # dense outputs whatever the strides of the inputs, like the real op
    return q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape)


@torch.library.custom_op("fa3b200::attention_fwd", mutates_args=(), device_types="cuda")
def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, softmax_scale: float,
                  window_left: int = -1, window_right: int = -1, softcap: float = 0.0,
                  layout: str = "bhsd") -> tuple[torch.Tensor, torch.Tensor]:
    out, lse = ops.fa3_fwd(q.contiguous(), k.contiguous(), v.contiguous(), causal, softmax_scale,
                           window=(window_left, window_right), softcap=softcap, layout=layout)
    return out, lse


@attention_fwd.register_fake
def _(q, k, v, causal, softmax_scale, window_left=-1, window_right=-1, softcap=0.0, layout="bhsd"):
    b, h, s = (q.shape[0], q.shape[2], q.shape[1]) if layout == "bshd" else q.shape[:3]
    return q.new_empty(q.shape), q.new_empty((b, h, s), dtype=torch.float32)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, softmax_scale, deterministic, window, softcap, layout):
        scale = softmax_scale if softmax_scale is not None else ops.default_scale(q.shape[-1])
        # strided inputs (a transposed view, say) are made dense once, here, and the dense copies are what
        # the backward gets; autograd maps the dense gradients back onto the views
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out, lse = torch.ops.fa3b200.attention_fwd(q, k, v, causal, scale, window[0], window[1], softcap, layout)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale, ctx.deterministic = causal, scale, deterministic
        ctx.window, ctx.softcap, ctx.layout = window, softcap, layout
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = torch.ops.fa3b200.attention_bwd(dout, q, k, v, out, lse, ctx.causal, ctx.scale,
                                                     ctx.deterministic, ctx.window[0], ctx.window[1],
                                                     ctx.softcap, ctx.layout)
        return dq, dk, dv, None, None, None, None, None, None


def attention(q, k, v, causal: bool = False, softmax_scale: float | None = None, deterministic: bool = False,
              window=(-1, -1), softcap: float = 0.0, layout: str = "bhsd"):
    """softmax(q k^T * scale) v with this library's forward and backward behind autograd."""
    return _Attention.apply(q, k, v, causal, softmax_scale, deterministic, tuple(window), float(softcap), layout)
