"""Mixers that carry a fixed-size state from token to token instead of a cache of keys.

``GatedLinearRecurrence`` (the recurrent block of Griffin with its real-gated linear recurrent
unit): two branches of ``inner`` channels from the same input rows h,

    y = gelu_tanh(Wy h + by)                        u = conv(Wx h + bx)     (causal, per channel, K taps)
    r = sigmoid(Ra u + bra), i = sigmoid(Ri u + bri)                       (block-diagonal Ra, Ri)
    a = exp(-c r softplus(lam)),  S_t = a S_(t-1) + sqrt(1 - a^2) i u,  S_(-1) = 0
    result = Wo (S_t * y)

with c = 8.  State per sequence: S [inner] and the convolution's last inputs, kept as a ring of K rows by
position [K, inner] (the input of position q at row q mod K).

``MatrixMemory`` (the matrix memory cell of xLSTM): per head, keys and queries of ``head_dim``
and values of ``value_dim``,

    i = cap tanh((Wi h + bi) / cap),  f = logsigmoid(cap tanh((Wf h + bf) / cap))
    m_t = max(f + m_(t-1), i)                                      (m_(-1) = 0)
    C_t = e^(f + m_(t-1) - m_t) C_(t-1) + e^(i - m_t) k v^T,  n_t likewise with k alone
    o = C_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6),  q = Wq h / sqrt(head_dim)
    result = Wo (o / rms(o per head) * w * sigmoid(Wg h))

State per sequence: C [heads, head_dim, value_dim], n [heads, head_dim], m [heads].

States, gates, decays, exponentials and the sums over time are float32 in every mode; in
bfloat16 mode only the products' operands are rounded.  The projections of a mixer are one
stacked product whose float32 rows feed the recurrence's kernels.
"""
from __future__ import annotations

import torch

from .base import Mixer, StateNeed
from .registry import register_part


class GatedLinearRecurrence(Mixer):
    def __init__(self, width: int, inner: int, blocks: int, taps: int, decay_scale: float = 8.0):
        self.width, self.inner, self.blocks, self.taps = int(width), int(inner), int(blocks), int(taps)
        if self.inner % self.blocks:
            raise ValueError(f"gated recurrence: {inner} channels are not {blocks} equal blocks")
        if self.taps < 1:
            raise ValueError("gated recurrence: the convolution needs at least one tap")
        self.decay_scale = float(decay_scale)
        self.w_xy = self.w_o = self.w_gates = None
        self.f32 = {}

    def weight_shapes(self):
        W, E, B, K = self.inner, self.width, self.blocks, self.taps
        Wb = W // B
        return {"x": ((W, E), "matrix"), "x.b": ((W,), "matrix"), "y": ((W, E), "matrix"), "y.b": ((W,), "matrix"),
                "conv": ((W, K), "taps"), "conv.b": ((W,), "matrix"),
                "ra": ((B, Wb, Wb), "matrix"), "ra.b": ((B, Wb), "matrix"),
                "ri": ((B, Wb, Wb), "matrix"), "ri.b": ((B, Wb), "matrix"),
                "lam": ((W,), "matrix"), "o": ((E, W), "matrix")}

    def state_need(self):
        need = {"S": StateNeed((self.inner,))}
        if self.taps > 1:
            need["tail"] = StateNeed((self.taps, self.inner))
        return need

    def bind(self, weights, ops):
        # rows [x channels | y channels]: one product
        self.w_xy = ops.prepare_linear([weights["x"], weights["y"]])
        self.w_o = ops.prepare_linear([weights["o"]])
        # per block, the recurrence gate's rows followed by the input gate's: [B, 2 Wb, Wb], float32
        self.w_gates = torch.cat([weights["ra"], weights["ri"]], dim=1).to(torch.float32).contiguous()
        self.f32 = {k: weights[k].to(torch.float32).contiguous()
                    for k in ("x.b", "y.b", "conv", "conv.b", "ra.b", "ri.b", "lam")}

    def forward(self, ctx, h, entry, accumulate_into=None):
        ops = ctx.ops
        state = ctx.state_view(entry)
        proj = ops.linear(h, self.w_xy, out_dtype=torch.float32)          # [T, 2 inner]
        gated = ops.gated_recurrence(proj, self, state, ctx.meta)         # [T, inner], compute dtype
        if accumulate_into is None:
            return ops.linear(gated, self.w_o, out_dtype=torch.float32)
        return ops.linear(gated, self.w_o, accumulate_into=accumulate_into)


class MatrixMemory(Mixer):
    def __init__(self, width: int, n_heads: int, head_dim: int, value_dim: int, gate_cap: float, norm_eps: float,
                 floor: float = 1e-6):
        self.width, self.n_heads, self.head_dim, self.value_dim = int(width), int(n_heads), int(head_dim), int(value_dim)
        self.gate_cap, self.norm_eps, self.floor = float(gate_cap), float(norm_eps), float(floor)
        if not self.gate_cap > 0:
            raise ValueError("matrix memory: the gates' cap must be positive")
        self.w_all = self.w_o = self.norm_w = self.i_bias = self.f_bias = None

    def weight_shapes(self):
        H, D, Dv, E = self.n_heads, self.head_dim, self.value_dim, self.width
        return {"q": ((H * D, E), "matrix"), "k": ((H * D, E), "matrix"), "v": ((H * Dv, E), "matrix"),
                "g": ((H * Dv, E), "matrix"), "i": ((H, E), "matrix"), "i.b": ((H,), "matrix"),
                "f": ((H, E), "matrix"), "f.b": ((H,), "matrix"), "norm": ((H * Dv,), "norm"),
                "o": ((E, H * Dv), "matrix")}

    def state_need(self):
        H, D, Dv = self.n_heads, self.head_dim, self.value_dim
        return {"C": StateNeed((H, D, Dv)), "n": StateNeed((H, D)), "m": StateNeed((H,))}

    #: columns of the stacked product's rows
    def offsets(self):
        H, D, Dv = self.n_heads, self.head_dim, self.value_dim
        q, k, v = 0, H * D, 2 * H * D
        g = v + H * Dv
        i = g + H * Dv
        return {"q": q, "k": k, "v": v, "g": g, "i": i, "f": i + H}

    def bind(self, weights, ops):
        self.w_all = ops.prepare_linear([weights[k] for k in ("q", "k", "v", "g", "i", "f")])
        self.w_o = ops.prepare_linear([weights["o"]])
        self.norm_w = weights["norm"].to(torch.float32).contiguous()
        self.i_bias = weights["i.b"].to(torch.float32).contiguous()
        self.f_bias = weights["f.b"].to(torch.float32).contiguous()

    def forward(self, ctx, h, entry, accumulate_into=None):
        ops = ctx.ops
        state = ctx.state_view(entry)
        proj = ops.linear(h, self.w_all, out_dtype=torch.float32)
        out = ops.matrix_memory(proj, self, state, ctx.meta)               # [T, H Dv], compute dtype
        if accumulate_into is None:
            return ops.linear(out, self.w_o, out_dtype=torch.float32)
        return ops.linear(out, self.w_o, accumulate_into=accumulate_into)


register_part("mixer", "gated_linear_recurrence", GatedLinearRecurrence)
register_part("mixer", "matrix_memory", MatrixMemory)
