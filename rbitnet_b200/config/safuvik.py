"""SafuvikConfig: the hyper-parameters of the Safuvik decoder, by config.json key.

config.json names the design under "architecture" and gives

  vocab, width        sizes of the embedding table and of a row of the residual state
  norm.eps            eps of every RMS norm
  streams             rows of residual state per token (hyper-connections); absent: one, with the ordinary residual sum
  logit_scale         multiplies the logits (absent: 1)
  layers              a list, one entry per layer, in order:
      type            "parallel" (window attention beside a gated linear recurrence) or "mlstm" (matrix memory)
      mixer           the mixer's sizes; for "parallel" under "left" (heads, kv_heads, dim, vdim, scale,
                      mask.size, rot.{base, dims, scaling.{factor, original, fast, slow}}) and "right"
                      (width, blocks, conv); for "mlstm": heads, dim, vdim, gate_cap
      mlp             null, or {"kind": "dense", "ff": inner size, "limit": clamp of the activation}
  max_positions       optional: the longest sequence an engine may be asked to hold (default 131072;
                      nothing in the design depends on it)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar, List, Optional

from .base import ModelConfig, ConfigError


def _positive_int(v, what):
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, found {v!r}")
    return v


def _need(d, keys, what):
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {what} must be an object")
    missing = [k for k in keys if d.get(k) is None]
    if missing:
        raise ConfigError(f"config.json: {what} is missing {', '.join(missing)}")


@dataclass
class SafuvikConfig(ModelConfig):
    architecture: ClassVar[str] = "Safuvik"
    required: ClassVar[tuple] = ("vocab", "width", "layers", "norm")

    vocab: int = 0
    width: int = 0
    layers: List[dict] = field(default_factory=list)
    norm: dict = field(default_factory=dict)
    streams: Optional[int] = None
    logit_scale: float = 1.0
    max_positions: int = 131072

    def validate(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_positions, "max_positions")
        if self.streams is not None:
            _positive_int(self.streams, "streams")
        _need(self.norm, ("eps",), "norm")
        if not float(self.norm["eps"]) > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind, m = layer["type"], layer["mixer"]
            if kind == "parallel":
                _need(m, ("left", "right"), f"{where}.mixer")
                left, right = m["left"], m["right"]
                _need(left, ("heads", "kv_heads", "dim", "vdim", "scale"), f"{where}.mixer.left")
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    _positive_int(left[k], f"{where}.mixer.left.{k}")
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"config.json: {where}: {left['heads']} heads are not a multiple of "
                                      f"{left['kv_heads']} kv_heads")
                if left.get("mask"):
                    _need(left["mask"], ("size",), f"{where}.mixer.left.mask")
                    _positive_int(left["mask"]["size"], f"{where}.mixer.left.mask.size")
                rot = left.get("rot")
                if rot:
                    _need(rot, ("base", "dims"), f"{where}.mixer.left.rot")
                    _positive_int(rot["dims"], f"{where}.mixer.left.rot.dims")
                    if rot["dims"] % 2 or rot["dims"] > left["dim"]:
                        raise ConfigError(f"config.json: {where}: rot.dims {rot['dims']} must be even and at most dim "
                                          f"{left['dim']}")
                    if rot.get("scaling"):
                        _need(rot["scaling"], ("factor", "original", "fast", "slow"), f"{where}.mixer.left.rot.scaling")
                _need(right, ("width", "blocks", "conv"), f"{where}.mixer.right")
                for k in ("width", "blocks", "conv"):
                    _positive_int(right[k], f"{where}.mixer.right.{k}")
                if right["width"] % right["blocks"]:
                    raise ConfigError(f"config.json: {where}: right.width {right['width']} is not {right['blocks']} "
                                      "equal blocks")
            elif kind == "mlstm":
                _need(m, ("heads", "dim", "vdim", "gate_cap"), f"{where}.mixer")
                for k in ("heads", "dim", "vdim"):
                    _positive_int(m[k], f"{where}.mixer.{k}")
                if not float(m["gate_cap"]) > 0:
                    raise ConfigError(f"config.json: {where}.mixer.gate_cap must be positive")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a layer of this design "
                                  "('parallel', 'mlstm')")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind", "ff", "limit"), f"{where}.mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not built (only 'dense')")
                _positive_int(mlp["ff"], f"{where}.mlp.ff")
                if not float(mlp["limit"]) > 0:
                    raise ConfigError(f"config.json: {where}.mlp.limit must be positive")

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": self.norm,
             "layers": self.layers, "logit_scale": self.logit_scale, "max_positions": self.max_positions}
        if self.streams is not None:
            d["streams"] = self.streams
        return d
