"""Dense gated feed-forward: down( act(gate h) * (up h) ), act = SiLU, no bias
(crates/bitnet-core/src/llama/model.rs:116-120, 296-306).  The activation and
the product are float32 before any rounding to the compute dtype.

``activation`` "swish_limited": with g' = min(gate h, limit) and u' = clamp(up h, -limit, limit),
the inner rows are g' * sigmoid(alpha g') * (u' + shift); alpha = 1.702 and shift = 1 unless given."""
from __future__ import annotations

import torch

from .base import FeedForward
from .registry import register_part


class GatedDense(FeedForward):
    def __init__(self, width: int, inner: int, activation: str = "silu", limit: float = 0.0,
                 alpha: float = 1.702, shift: float = 1.0):
        if activation not in ("silu", "swish_limited"):
            raise ValueError(f"gated feed-forward: activation {activation!r} is not built "
                             "(only 'silu' and 'swish_limited')")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        #: (alpha, limit, shift) of the limited activation; None: SiLU(gate) * up
        self.act = None if activation == "silu" else (float(alpha), float(limit), float(shift))
        if self.act is not None and not self.act[1] > 0:
            raise ValueError("gated feed-forward: 'swish_limited' needs a positive limit")
        self.w_gate_up = self.w_down = None

    def weight_shapes(self):
        return {"gate": ((self.inner, self.width), "matrix"), "up": ((self.inner, self.width), "matrix"),
                "down": ((self.width, self.inner), "matrix")}

    def bind(self, weights, ops):
        self.w_gate_up = ops.prepare_gate_up(weights["gate"], weights["up"])
        self.w_down = ops.prepare_linear([weights["down"]])

    #: ``h`` may be rows with their norm pending, and ``then_norm`` is handed to the last product
    folds_norms = True

    def forward(self, ctx, h, accumulate_into=None, then_norm=None):
        if self.act is None:
            t = ctx.ops.gated_linear(h, self.w_gate_up)        # silu(gate h) * (up h)
        else:
            t = ctx.ops.gated_linear(h, self.w_gate_up, act=self.act)
        if accumulate_into is None:
            return ctx.ops.linear(t, self.w_down, out_dtype=torch.float32)
        if then_norm is None:
            ctx.ops.linear(t, self.w_down, accumulate_into=accumulate_into)
        else:
            ctx.ops.linear(t, self.w_down, accumulate_into=accumulate_into, then_norm=then_norm)


register_part("feed_forward", "gated_dense", GatedDense)
