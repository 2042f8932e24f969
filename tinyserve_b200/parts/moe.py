"""Mixture of experts: ``num_experts`` small feed-forward layers, of which every token uses ``top``.

Router: z = W_r h in 32-bit, s = softmax(z) over all experts; the ``top`` largest s are the token's
experts and their weights, as they are (not divided by their sum).  Expert e:
W_down,e act(W_up,e h), no biases; the token's output is the weighted sum over its experts.

The experts' up-projections are stacked into one matrix [E ff, hidden] and their down-projections
side by side into one [hidden, E ff]: act(.) of an expert that a token did not choose is multiplied
by zero, the others by their weight, and one product over K = E ff adds the chosen experts'
outputs in 32-bit inside the product.  That is how a few tokens run (decoding: they touch most
experts' weights anyway) and how the 32-bit engine runs; a bfloat16 step of many tokens sorts its
rows by expert instead, so that an expert multiplies its own rows only (``ops.moe_grouped``)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, ParamSpec, Source, register_feed_forward

DEFAULT_NAMES = {"router": "router", "expert": "e{e}", "up": "up", "down": "down"}


class MixtureOfExperts(FeedForward):
    tree_name = "mlp"
    capturable = True
    accepts_scaled_rows = False

    def __init__(self, hidden_size, intermediate_size, num_experts, top, activation="relu_squared", names=None):
        super().__init__()
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        if activation != "relu_squared":
            raise ValueError(f"mixture of experts: unknown activation {activation!r}; known: relu_squared")
        if not 0 < top <= num_experts:
            raise ValueError(f"mixture of experts: {top} of {num_experts} experts")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top = int(num_experts), int(top)

    def param_specs(self):
        nm, E, ff, n = self.names, self.num_experts, self.intermediate_size, self.hidden_size
        expert = lambda e: nm["expert"].format(e=e)
        return {
            "router.weight": ParamSpec((E, n), sources=(Source(f"{nm['router']}.weight", 0, E),)),
            "up.weight": ParamSpec((E * ff, n), sources=tuple(
                Source(f"{expert(e)}.{nm['up']}.weight", e * ff, (e + 1) * ff) for e in range(E))),
            # stored expert by expert [E hidden, ff]; ``bind`` lays them side by side
            "down.weight": ParamSpec((E * n, ff), sources=tuple(
                Source(f"{expert(e)}.{nm['down']}.weight", e * n, (e + 1) * n) for e in range(E))),
        }

    def bind(self, tensors):
        E, ff, n = self.num_experts, self.intermediate_size, self.hidden_size
        if "down.weight" in tensors:
            down = tensors["down.weight"]
            tensors = dict(tensors)
            tensors["down.weight"] = down.view(E, n, ff).permute(1, 0, 2).reshape(n, E * ff).contiguous()
        super().bind(tensors)

    def forward(self, h, ctx):
        logits = ops.linear(h, self.w["router.weight"], out_float32=True)
        if (h.dtype == torch.bfloat16 and self.top < self.num_experts and h.shape[0] >= ops.MOE_GROUPED_MIN_TOKENS
                and self.hidden_size % 8 == 0 and self.intermediate_size % 8 == 0):
            gates = ops.moe_route(logits, self.top)
            return ops.moe_grouped(h, gates, self.w["up.weight"], self.w["down.weight"], self.top)
        a = ops.materialize(ops.linear(h, self.w["up.weight"]))
        ops.moe_activate_(a, None, self.num_experts, logits=logits, top=self.top)      # (routes in the same kernel)
        return ops.linear(a, self.w["down.weight"], allow_pending=True)


register_feed_forward("moe", MixtureOfExperts)
