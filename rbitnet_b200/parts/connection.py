"""How a sublayer's result enters the residual state.

"residual": one row per token; the sublayer reads it and its result is added to it.

"hyper": s rows X_1..X_s per token (hyper-connections).  A sublayer reads u = sum_k in[k] X_k, and
its result y is written to all rows at once from the old ones: X'_j = sum_k mix[k, j] X_k + out[j] y.
Weights "in" [s], "out" [s], "mix" [s, s] (indexed [from, to]).  All float32.
"""
from __future__ import annotations

import torch

from .base import Connection
from .registry import register_part


class ResidualConnection(Connection):
    streams = 1

    def __init__(self, **_):
        self._w = None

    def bind(self, weights, ops):
        one = torch.ones(1, dtype=torch.float32, device=ops.device)
        self._w = (one, one, one.view(1, 1))

    def weights(self):
        return self._w


class HyperConnection(Connection):
    def __init__(self, streams: int):
        self.streams = int(streams)
        if self.streams < 1:
            raise ValueError("hyper-connection: at least one stream")
        self._w = None

    def weight_shapes(self):
        s = self.streams
        return {"in": ((s,), "share"), "out": ((s,), "norm"), "mix": ((s, s), "identity")}

    def bind(self, weights, ops):
        self._w = tuple(weights[k].to(device=ops.device, dtype=torch.float32).contiguous() for k in ("in", "out", "mix"))

    def weights(self):
        return self._w


register_part("connection", "residual", ResidualConnection)
register_part("connection", "hyper", HyperConnection)
