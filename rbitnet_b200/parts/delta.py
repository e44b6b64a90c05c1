"""``GatedDeltaRule``: a mixer that keeps one matrix memory S [head_dim, value_dim] per head and corrects, token by
token, what the memory holds for the token's key (the gated delta rule).

From the input rows h, without biases: q = Wq h and k = Wk h (``n_kv_heads`` heads of ``head_dim``), v = Wv h
(``n_heads`` heads of ``value_dim``); value head i reads key head i // (n_heads / n_kv_heads).  Each of q, k, v goes
through a short causal convolution per channel ("q.conv", "k.conv", "v.conv": [channels, taps], the last tap is the
current token's, zeros before the start of the sequence) and SiLU.  Then, per head,

    q <- q / sqrt(sum q^2 + unit_eps) / sqrt(head_dim),   k <- k / sqrt(sum k^2 + unit_eps)
    beta = sigmoid(Wb h),   g = exp(-exp(A_log) * softplus(Wa h + dt_bias))            (one number per head each)
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                   (the read-out sees the write)
    result = Wo (o / rms(o over value_dim, norm_eps) * w * silu(Wg h))                 (w: value_dim values, every head's)

State per sequence: S (float32, kept by value column: [heads, value_dim, head_dim]) and the convolution's last inputs
as a ring of ``taps`` rows by position.  Unit vectors, gates, decays, the memory and its sums are float32 in every
mode; the projections are one stacked product whose float32 rows feed the recurrence's kernels.
"""
from __future__ import annotations

import torch

from .base import Mixer, StateNeed
from .registry import register_part


class GatedDeltaRule(Mixer):
    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, value_dim: int, taps: int,
                 norm_eps: float, unit_eps: float = 1e-6):
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.head_dim, self.value_dim, self.taps = int(head_dim), int(value_dim), int(taps)
        self.norm_eps, self.unit_eps = float(norm_eps), float(unit_eps)
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"delta rule: {n_heads} heads are not a multiple of {n_kv_heads} key heads")
        if self.taps < 1:
            raise ValueError("delta rule: the convolution needs at least one tap")
        self.w_all = self.w_o = self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def weight_shapes(self):
        H, G, D, Dv, E, K = self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim, self.width, self.taps
        return {"q": ((G * D, E), "matrix"), "q.conv": ((G * D, K), "taps"),
                "k": ((G * D, E), "matrix"), "k.conv": ((G * D, K), "taps"),
                "v": ((H * Dv, E), "matrix"), "v.conv": ((H * Dv, K), "taps"),
                "b": ((H, E), "matrix"), "a": ((H, E), "matrix"), "A_log": ((H,), "matrix"), "dt_bias": ((H,), "matrix"),
                "norm": ((Dv,), "norm"), "g": ((H * Dv, E), "matrix"), "o": ((E, H * Dv), "matrix")}

    def state_need(self):
        need = {"S": StateNeed((self.n_heads, self.value_dim, self.head_dim))}
        if self.taps > 1:
            need["tail"] = StateNeed((self.taps, 2 * self.n_kv_heads * self.head_dim + self.n_heads * self.value_dim))
        return need

    def offsets(self):
        """Columns of the stacked product's rows."""
        H, G, D, Dv = self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim
        g = 2 * G * D + H * Dv
        return {"q": 0, "k": G * D, "v": 2 * G * D, "g": g, "b": g + H * Dv, "a": g + H * Dv + H}

    def bind(self, weights, ops):
        self.w_all = ops.prepare_linear([weights[k] for k in ("q", "k", "v", "g", "b", "a")])
        self.w_o = ops.prepare_linear([weights["o"]])
        f32 = dict(device=ops.device, dtype=torch.float32)
        # the three convolutions as one over the stacked channels [q | k | v]
        self.conv_w = torch.cat([weights[k].to(**f32) for k in ("q.conv", "k.conv", "v.conv")], dim=0).contiguous()
        self.a_log = weights["A_log"].to(**f32).contiguous()
        self.dt_bias = weights["dt_bias"].to(**f32).contiguous()
        self.norm_w = weights["norm"].to(**f32).contiguous()

    def forward(self, ctx, h, entry, accumulate_into=None):
        ops = ctx.ops
        state = ctx.state_view(entry)
        proj = ops.linear(h, self.w_all, out_dtype=torch.float32)         # [T, q | k | v | g | b | a]
        out = ops.gated_delta(proj, self, state, ctx.meta)                # [T, H Dv], compute dtype
        if accumulate_into is None:
            return ops.linear(out, self.w_o, out_dtype=torch.float32)
        return ops.linear(out, self.w_o, accumulate_into=accumulate_into)


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
