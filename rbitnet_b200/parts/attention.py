"""Grouped-query attention over the cache, as a mixer.

q = Wq h, k = Wk h, v = Wv h without bias; q and k take the position encoding;
k and v are appended to the sequence's cache; query head h reads kv head
h // (H/K); score = (q.k) * scale over the keys the mask allows (causal, and a
window if given); softmax in float32; o = P v; result Wo o is added to the
residual stream.  crates/bitnet-core/src/llama/model.rs:238-294

Options beyond the reference's, each off by default:
  value_dim        values (and the output per head) of another size than queries and keys
  qk_norm          "projection": q (and k) are divided by the root mean square of the WHOLE
                   projection, all heads at once, and multiplied by a weight of that size
                   ("q.norm", "k.norm"), before the rotation
                   "head": after the rotation, every q and k head is divided by its own root
                   mean square over the head (no weight)
  head_gate        head h's output is multiplied by sigmoid(Wg h)_h, one number per head ("g"),
                   read from the same input rows as q, k and v
  value_gate       the joined heads are multiplied value by value with sigmoid(Wg h) ("g" with a
                   row per value), read from the same input rows
With any of them, or a position encoding that turns only a part of a head or stretches its
frequencies, the q/k/v(/g) product is followed by one kernel that norms, turns and appends; keys
and values of unequal sizes share cache rows of the larger size, padded with zeros.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import Mixer, CacheNeed
from .registry import register_part, build_part
from .spec import PartSpec


class Attention(Mixer):
    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: Optional[dict] = None, window: Optional[int] = None,
                 scale: Optional[float] = None, value_dim: Optional[int] = None,
                 qk_norm: Optional[str] = None, norm_eps: float = 1e-6, head_gate: bool = False,
                 value_gate: bool = False):
        if n_heads % n_kv_heads:
            raise ValueError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = width, n_heads, n_kv_heads, head_dim
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        position = position or {"kind": "none", "params": {}}
        self.position = build_part("position", PartSpec(position["kind"], dict(position.get("params", {}))))
        self.value_dim = int(value_dim) if value_dim else head_dim
        if qk_norm not in (None, "projection", "head"):
            raise ValueError(f"attention: qk_norm {qk_norm!r} is not built (only 'projection' and 'head')")
        if head_gate and value_gate:
            raise ValueError("attention: a gate per head or a gate per value, not both")
        self.qk_norm, self.norm_eps, self.head_gate = qk_norm, float(norm_eps), bool(head_gate)
        self.value_gate = bool(value_gate)
        self.w_qkv = self.w_q = self.w_o = None
        self.q_norm_w = self.k_norm_w = None
        self.cache_width = head_dim

    @property
    def extended(self) -> bool:
        """Whether the options of this module's second paragraph are in use."""
        plain_position = getattr(self.position, "plain", True)
        return bool(self.value_dim != self.head_dim or self.qk_norm or self.head_gate or self.value_gate
                    or not plain_position)

    def weight_shapes(self):
        H, K, D, E, Dv = self.n_heads, self.n_kv_heads, self.head_dim, self.width, self.value_dim
        shapes = {"q": ((H * D, E), "matrix"), "k": ((K * D, E), "matrix"),
                  "v": ((K * Dv, E), "matrix"), "o": ((E, H * Dv), "matrix")}
        if self.qk_norm == "projection":
            shapes["q.norm"] = ((H * D,), "norm")
            shapes["k.norm"] = ((K * D,), "norm")
        if self.head_gate:
            shapes["g"] = ((H, E), "matrix")
        if self.value_gate:
            shapes["g"] = ((H * Dv, E), "matrix")
        return shapes

    def cache_need(self):
        return CacheNeed(self.n_kv_heads, self.cache_width, self.window)

    def bind(self, weights, ops):
        self.position.bind({}, ops)
        if self.extended:
            # one product for q, k, v and the gates: rows [q heads | k heads | v heads | gates]
            stack = [weights["q"], weights["k"], weights["v"]] + ([weights["g"]] if self.head_gate or self.value_gate else [])
            self.w_qkv = ops.prepare_linear(stack)
            self.w_o = ops.prepare_linear([weights["o"]])
            if self.qk_norm == "projection":
                self.q_norm_w = weights["q.norm"].to(torch.float32).contiguous()
                self.k_norm_w = weights["k.norm"].to(torch.float32).contiguous()
            self.cache_width = ops.cache_head_width(self.head_dim, self.value_dim)
            return
        # one product for q, k and v: rows [q heads | k heads | v heads]
        self.w_qkv = ops.prepare_linear([weights["q"], weights["k"], weights["v"]])
        self.w_q = None  # for a run that reads another layer's cache: the q rows of w_qkv, as a view
        self.w_o = ops.prepare_linear([weights["o"]])

    #: ``h`` may be rows with their norm pending, and ``then_norm`` is handed to the last product
    folds_norms = True

    def _forward_extended(self, ctx, h, entry, accumulate_into):
        ops = ctx.ops
        view = ctx.cache_view(entry)
        if not view.writes:
            raise ValueError("attention with a projection norm, a head gate or unequal key and value sizes "
                             "reads only its own cache")
        H, Kh, D, Dv = self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim
        table = self.position.table() if hasattr(self.position, "table") else None
        proj = ops.linear(ops.normed(h) if hasattr(h, "scaled") else h, self.w_qkv)
        if self.qk_norm == "head":
            q = ops.norm_rotate_append(proj, table, ctx.meta, view, H, D, Dv, None, None, self.norm_eps, head_norm=True)
        else:
            q = ops.norm_rotate_append(proj, table, ctx.meta, view, H, D, Dv, self.q_norm_w, self.k_norm_w, self.norm_eps)
        a = ops.attention(q, ctx.meta, view, H, self.scale, self.window)
        gate_column = (H + Kh) * D + Kh * Dv if self.head_gate or self.value_gate else None
        if self.value_gate:
            a = ops.head_gate(a, proj, gate_column, H, Dv, view.head_dim, per_value=True)
        else:
            a = ops.head_gate(a, proj, gate_column, H, Dv, view.head_dim)
        if accumulate_into is None:
            return ops.linear(a, self.w_o, out_dtype=torch.float32)
        return ops.linear(a, self.w_o, accumulate_into=accumulate_into)

    def forward(self, ctx, h, entry, accumulate_into=None, then_norm=None):
        if self.extended:
            return self._forward_extended(ctx, h, entry, accumulate_into)
        ops = ctx.ops
        view = ctx.cache_view(entry)
        if view.writes:
            w = self.w_qkv
        else:
            if self.w_q is None:
                self.w_q = ops.rows_of(self.w_qkv, 0, self.n_heads * self.head_dim)
            w = self.w_q
        q = ops.project_rotate_append(h, w, self.position.rotary(), ctx.meta, view, self.n_heads)
        a = ops.attention(q, ctx.meta, view, self.n_heads, self.scale, self.window)
        if accumulate_into is None:
            return ops.linear(a, self.w_o, out_dtype=torch.float32)
        if then_norm is None:
            ops.linear(a, self.w_o, accumulate_into=accumulate_into)
        else:
            ops.linear(a, self.w_o, accumulate_into=accumulate_into, then_norm=then_norm)


register_part("mixer", "attention", Attention)
