"""PyTorch registration of the backward (the consumer the reference names for its C ABI,
reference docs/tridao_fa3_bwd_api.md:48-55, and never shipped).

* ``torch.ops.fa3b200.attention_bwd`` - a ``torch.library`` custom op over the C entry point
  ``shaobo_fa3_bwd_v2`` with a fake (meta) implementation, so it can sit inside traced graphs.
* ``attention`` - an ``autograd.Function`` whose backward is that op.  Its forward is NOT part of
  this library: it is a plain fp32 torch softmax (``synthetic.forward_reference``) that exists so
  that the backward can be driven from ``loss.backward()``; a matching forward kernel is future work.

Tensors are BHSD, contiguous, fp16 or bf16, on a CUDA device; there is no CPU path.
"""
from __future__ import annotations

import torch

from . import ops, synthetic


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


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, softmax_scale, deterministic):
        scale = softmax_scale if softmax_scale is not None else ops.default_scale(q.shape[-1])
        out, lse = synthetic.forward_reference(q, k, v, causal, scale)
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
