"""Synthetic workloads for the benchmark and the large-shape tests.

Generates seeded N(0,1) Q, K, V, dO in the storage dtype directly on the GPU
and produces the forward's O (rounded to the storage dtype) and natural-log LSE
with a plain fp32 torch softmax, one (batch, head) slice at a time.  This is
set-up plumbing: it runs outside every timed region and is not the product.
"""
from __future__ import annotations

import math

import torch


def make_inputs(seed: int, b: int, hq: int, hkv: int, s: int, d: int, dtype: torch.dtype, device="cuda"):
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def normal(*shape):
        return torch.randn(*shape, generator=g, device=device, dtype=torch.float32).to(dtype)

    return normal(b, hq, s, d), normal(b, hkv, s, d), normal(b, hkv, s, d), normal(b, hq, s, d)


@torch.no_grad()
def forward_reference(q, k, v, causal: bool, scale: float | None = None, row_chunk: int = 2048):
    """O (storage dtype) and LSE (fp32, natural log) by an fp32 softmax."""
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    out = torch.empty_like(q)
    lse = torch.empty(b, hq, s, dtype=torch.float32, device=q.device)
    for bi in range(b):
        for h in range(hq):
            kf = k[bi, h // group].float()
            vf = v[bi, h // group].float()
            for r0 in range(0, s, row_chunk):
                r1 = min(s, r0 + row_chunk)
                keys = r1 if causal else s
                sc = (q[bi, h, r0:r1].float() @ kf[:keys].T) * scale
                if causal:
                    rows = torch.arange(r0, r1, device=q.device)[:, None]
                    cols = torch.arange(keys, device=q.device)[None, :]
                    sc = sc.masked_fill(cols > rows, float("-inf"))
                l = torch.logsumexp(sc, dim=1)
                out[bi, h, r0:r1] = (torch.exp(sc - l[:, None]) @ vf[:keys]).to(q.dtype)
                lse[bi, h, r0:r1] = l
    return out, lse


def bwd_flops(b: int, hq: int, s: int, d: int, causal: bool) -> float:
    """Algorithmic FLOPs of the backward: 2.5 x forward = 10*B*Hq*S^2*D, halved when causal."""
    f = 10.0 * b * hq * float(s) * float(s) * d
    return f / 2 if causal else f
