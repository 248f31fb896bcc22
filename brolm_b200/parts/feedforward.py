"""Feed-forward parts."""
from __future__ import annotations

import torch

from .. import kernels
from .base import ParamSpec, Part, register_part
from .linear import linear


class GatedFeedForward(Part):
    """down(act(gate(x)) * up(x)), dense, no bias
    (wlejon/brolm src/gemma2.cpp:378-382 with act = gelu, tanh form).
    Gate and up run as one product over the rows [Wg; Wu]."""

    kind = "feedforward"
    graph_safe = True

    def __init__(self, hidden: int, inter: int, activation: str = "gelu_tanh"):
        if activation not in kernels.ACTIVATIONS:
            raise ValueError(f"feed-forward: unknown activation '{activation}'")
        self.hidden, self.inter, self.activation = hidden, inter, activation

    def param_specs(self):
        return {"gate": ParamSpec((self.inter, self.hidden)), "up": ParamSpec((self.inter, self.hidden)),
                "down": ParamSpec((self.hidden, self.inter))}

    def bind(self, params):
        kinds = {params[n].dtype for n in ("gate", "up")}
        dt = torch.float32 if (len(kinds) > 1 or torch.float32 in kinds) else next(iter(kinds))
        self.w_gate_up = torch.cat([params["gate"].to(dt), params["up"].to(dt)], dim=0).contiguous()
        self.w_down = params["down"]
        self.params = {}

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """x (tokens, hidden) -> (tokens, hidden) float32."""
        act = torch.empty((x.shape[0], self.inter), dtype=ctx.dtype, device=x.device)
        if kernels.skinny_ok(x, self.w_gate_up):
            # few tokens: both products and the activation in one pass over the weights
            kernels.skinny_gemm(x, self.w_gate_up, act, "gated", self.activation)
        elif self.inter % 64 == 0 and kernels.stream_rows(x, self.w_gate_up):
            # 17 to 128 tokens: the same on the tcgen05 weight stream
            kernels.gemm_stream(x, self.w_gate_up, act, "gated", self.activation)
        elif self.inter % 128 == 0 and kernels.gemm_tc_ok(x, self.w_gate_up, gated=True):
            # many tokens: the activation is the epilogue of the product; [gate | up] never reaches memory
            kernels.gemm_tc(x, self.w_gate_up, act, "gated", self.activation)
        else:
            gate_up = linear(x, self.w_gate_up, out_dtype=ctx.dtype)
            kernels.gated_act(gate_up, act, self.activation)
        return linear(act, self.w_down, out_dtype=torch.float32, parts_ok=True)


register_part("feedforward", "gated", GatedFeedForward)
