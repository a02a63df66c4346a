"""PyTorch registration of the backward (the consumer the reference names for its C ABI,
reference docs/tridao_fa3_bwd_api.md:48-55, and never shipped).

* ``torch.ops.fa3b200.attention_bwd`` - a ``torch.library`` custom op over the C entry point
  ``shaobo_fa3_bwd_v2`` with a fake (meta) implementation, so it can sit inside traced graphs.
* ``torch.ops.fa3b200.attention_fwd`` - the same for the forward kernel (``shaobo_fa3_b200_fwd``),
  which returns O and the log-sum-exp the backward needs.
* ``attention`` - an ``autograd.Function`` over the two ops, so that the library can be driven from
  ``loss.backward()``.

Tensors are BHSD, contiguous, fp16 or bf16, on a CUDA device; there is no CPU path.
"""
from __future__ import annotations

import torch

from . import ops


@torch.library.custom_op("fa3b200::attention_bwd", mutates_args=(), device_types="cuda")
def attention_bwd(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                  softmax_lse: torch.Tensor, causal: bool, softmax_scale: float,
                  deterministic: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    dq, dk, dv = ops.fa3_bwd(dout.contiguous(), q, k, v, out, softmax_lse, causal, softmax_scale,
                             deterministic=deterministic)
    return dq, dk, dv


@attention_bwd.register_fake
def _(dout, q, k, v, out, softmax_lse, causal, softmax_scale, deterministic):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


@torch.library.custom_op("fa3b200::attention_fwd", mutates_args=(), device_types="cuda")
def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool,
                  softmax_scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    out, lse = ops.fa3_fwd(q.contiguous(), k.contiguous(), v.contiguous(), causal, softmax_scale)
    return out, lse


@attention_fwd.register_fake
def _(q, k, v, causal, softmax_scale):
    return torch.empty_like(q), q.new_empty(q.shape[:3], dtype=torch.float32)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, softmax_scale, deterministic):
        scale = softmax_scale if softmax_scale is not None else ops.default_scale(q.shape[-1])
        out, lse = torch.ops.fa3b200.attention_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale, ctx.deterministic = causal, scale, deterministic
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = torch.ops.fa3b200.attention_bwd(dout, q, k, v, out, lse, ctx.causal, ctx.scale,
                                                     ctx.deterministic)
        return dq, dk, dv, None, None, None


def attention(q, k, v, causal: bool = False, softmax_scale: float | None = None, deterministic: bool = False):
    """softmax(q k^T * scale) v with this library's backward behind autograd (BHSD tensors)."""
    return _Attention.apply(q, k, v, causal, softmax_scale, deterministic)
