"""Matrix products  Y = X W^T  with W stored (out, in), no bias
(wlejon/brolm include/brolm/detail/compute.h:49-86 dispatches on the weight's
element type in the same way).

* float32 weight: the framework's own CUDA-core kernel, true 32-bit.
* bfloat16 weight, up to 16 rows (decode steps): the framework's own
  weight-streaming tensor-core kernel, float32 accumulation.
* bfloat16 weight, 17 to 128 rows (wider decode batches, short prompts): the
  framework's tcgen05 weight stream (TMA ring, tokens on the N side of the
  instruction), float32 accumulation.
* bfloat16 weight, more rows: the framework's tcgen05 kernel (TMA loads,
  accumulator in tensor memory), float32 accumulation; the library product
  (cuBLAS through torch) only for operands that kernel does not take (a width
  that is no multiple of 8) or that leave most SMs without a tile.  The result
  is bfloat16 or, on request, float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None, parts_ok: bool = False) -> torch.Tensor:
    """``parts_ok``: the caller adds partial sums itself (the residual kernel
    does); the result may then be [parts, M, N] float32, the slices of a
    product that was cut along K so that more blocks stream the weights."""
    M = x.shape[0]
    N = weight.shape[0]
    if weight.dtype == torch.float32:
        x32 = x if x.dtype == torch.float32 else x.float()
        want = out_dtype or x.dtype
        y = out if (out is not None and out.dtype == torch.float32) else \
            torch.empty((M, N), dtype=torch.float32, device=x.device)
        kernels.linear_f32(x32, weight, y)
        if want != torch.float32:
            y = y.to(want)
            if out is not None:
                out.copy_(y)
                return out
        return y
    if weight.dtype == torch.bfloat16:
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        want = out_dtype or torch.bfloat16
        if kernels.skinny_ok(x, weight) and want in (torch.bfloat16, torch.float32):
            parts = kernels.skinny_parts(x, weight) if (parts_ok and want == torch.float32 and out is None) else 1
            if parts > 1:
                y = torch.empty((parts, M, N), dtype=torch.float32, device=x.device)
                kernels.skinny_gemm(x, weight, y)
                return y
            y = out if out is not None else torch.empty((M, N), dtype=want, device=x.device)
            kernels.skinny_gemm(x, weight, y)
            return y
        if kernels.stream_rows(x, weight) and want in (torch.bfloat16, torch.float32):
            # 17 to 128 tokens: still a stream of the weights, on tcgen05 with the tokens on the N side
            parts = kernels.gemm_stream_parts(x, weight) if (parts_ok and want == torch.float32 and out is None) else 1
            if parts > 1:
                y = torch.empty((parts, M, N), dtype=torch.float32, device=x.device)
                kernels.gemm_stream(x, weight, y)
                return y
            y = out if out is not None else torch.empty((M, N), dtype=want, device=x.device)
            if y.stride(1) == 1:
                kernels.gemm_stream(x, weight, y)
                return y
        if kernels.gemm_tc_ok(x, weight) and want in (torch.bfloat16, torch.float32):
            y = out if out is not None else torch.empty((M, N), dtype=want, device=x.device)
            if y.stride(1) == 1 and y.data_ptr() % 16 == 0:
                kernels.gemm_tc(x, weight, y)
                return y
        if want == torch.bfloat16:
            return torch.mm(x, weight.t(), out=out) if out is not None else torch.mm(x, weight.t())
        if out is not None:
            return torch.mm(x, weight.t(), out_dtype=want, out=out)
        return torch.mm(x, weight.t(), out_dtype=want)
    raise TypeError(f"linear: weights of type {weight.dtype} are not supported")
