"""Norm parts and the residual sum around them."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ParamSpec, Part, register_part


class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * (offset + w).

    Gemma 2 uses offset 1 (wlejon/brolm src/gemma2.cpp:154-175 folds it into
    the gain at load; here the gain stays as stored and the kernel adds it).
    Statistics and the product are float32.
    """

    kind = "norm"
    graph_safe = True

    def __init__(self, size: int, eps: float, offset: float = 0.0):
        self.size, self.eps, self.offset = size, float(eps), float(offset)

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), "vector")}

    @property
    def weight(self) -> torch.Tensor:
        return self.params["weight"]

    def apply(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = rows.numel() if rows is not None else x.shape[0]
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        kernels.rmsnorm(x, self.weight, self.eps, self.offset, out, rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)


def add_then_norm(h: torch.Tensor, y: torch.Tensor, post: Optional[Part], nxt: Optional[Part],
                  out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """h += post(y) (or y);  return nxt(h) when ``nxt`` is given.

    h is the float32 residual stream and is updated in place.  Two RMSNorms
    run in one kernel with the sum; any other norm part is applied through its
    own ``apply`` and only the sum stays fused.
    """
    fused_post = post is None or isinstance(post, RMSNorm)
    fused_next = nxt is None or isinstance(nxt, RMSNorm)
    if fused_post and fused_next and post is not None and nxt is not None and post.weight.dtype != nxt.weight.dtype:
        fused_next = False
    if y.dim() == 3 and not fused_post:
        y = y.sum(dim=0)                       # partial sums, and a norm that wants the whole
    if not fused_post:
        y = post.apply(y, torch.float32)
        post = None
    out = None
    if fused_next and nxt is not None:
        out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
    kernels.residual_rmsnorm(
        h, y,
        post.weight if post is not None else None, post.eps if post is not None else 0.0,
        post.offset if post is not None else 0.0,
        nxt.weight if (fused_next and nxt is not None) else None, nxt.eps if (fused_next and nxt is not None) else 0.0,
        nxt.offset if (fused_next and nxt is not None) else 0.0, out)
    if nxt is not None and not fused_next:
        out = nxt.apply(h, out_dtype)
    return out
