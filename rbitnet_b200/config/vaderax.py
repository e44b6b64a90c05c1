"""VaderaxConfig: the hyper-parameters of the Vaderax decoder, by config.json key.

config.json names the design under "architecture" and gives

  vocab, width          sizes of the embedding table and of the residual stream
  embedding.scale       multiplies the embedded rows
  norm.eps              eps of every layer norm, of the attention's norm per head and of the delta rule's output norm
  layers                a list, one entry per layer, in order:
      type              "attention" or "delta"
      mixer             "attention": heads, kv_heads, dim, vdim, scale, and optionally rot.{base, dims}
                        "delta": heads, kv_heads, dim, vdim, conv (taps of the short convolution)
      mlp               null, {"kind": "dense", "ff": inner size}, or {"kind": "moe", "expert": {"ff": inner size},
                        "router": {"experts", "top", and optionally "identity", "groups": {"count", "keep"}}}
  loop                  optional {"start", "stop", "times"}: layers start .. stop-1 run `times` times in a row
  max_positions         optional: the longest sequence an engine may be asked to hold (default 131072;
                        nothing in the design depends on it)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar, List, Optional

from .base import ModelConfig, ConfigError
from .safuvik import _positive_int, _need


@dataclass
class VaderaxConfig(ModelConfig):
    architecture: ClassVar[str] = "Vaderax"
    required: ClassVar[tuple] = ("vocab", "width", "layers", "norm", "embedding")

    vocab: int = 0
    width: int = 0
    layers: List[dict] = field(default_factory=list)
    norm: dict = field(default_factory=dict)
    embedding: dict = field(default_factory=dict)
    loop: Optional[dict] = None
    max_positions: int = 131072

    def validate(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_positions, "max_positions")
        _need(self.norm, ("eps",), "norm")
        if not float(self.norm["eps"]) > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        _need(self.embedding, ("scale",), "embedding")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind, m = layer["type"], layer["mixer"]
            if kind not in ("attention", "delta"):
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a layer of this design ('attention', 'delta')")
            _need(m, ("heads", "kv_heads", "dim", "vdim") + (("scale",) if kind == "attention" else ("conv",)),
                  f"{where}.mixer")
            for k in ("heads", "kv_heads", "dim", "vdim"):
                _positive_int(m[k], f"{where}.mixer.{k}")
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"config.json: {where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
            if kind == "delta":
                _positive_int(m["conv"], f"{where}.mixer.conv")
            rot = m.get("rot") if kind == "attention" else None
            if rot:
                _need(rot, ("base", "dims"), f"{where}.mixer.rot")
                _positive_int(rot["dims"], f"{where}.mixer.rot.dims")
                if rot["dims"] % 2 or rot["dims"] > m["dim"]:
                    raise ConfigError(f"config.json: {where}: rot.dims {rot['dims']} must be even and at most dim {m['dim']}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            _need(mlp, ("kind",), f"{where}.mlp")
            if mlp["kind"] == "dense":
                _need(mlp, ("ff",), f"{where}.mlp")
                _positive_int(mlp["ff"], f"{where}.mlp.ff")
            elif mlp["kind"] == "moe":
                _need(mlp, ("expert", "router"), f"{where}.mlp")
                _need(mlp["expert"], ("ff",), f"{where}.mlp.expert")
                _positive_int(mlp["expert"]["ff"], f"{where}.mlp.expert.ff")
                r = mlp["router"]
                _need(r, ("experts", "top"), f"{where}.mlp.router")
                _positive_int(r["top"], f"{where}.mlp.router.top")
                if not isinstance(r["experts"], int) or r["experts"] < 0:
                    raise ConfigError(f"config.json: {where}.mlp.router.experts must be an integer, 0 or more")
                ident = r.get("identity") or 0
                if not isinstance(ident, int) or ident < 0:
                    raise ConfigError(f"config.json: {where}.mlp.router.identity must be an integer, 0 or more")
                n = r["experts"] + ident
                if r["top"] > n:
                    raise ConfigError(f"config.json: {where}.mlp.router: top {r['top']} of {n} experts")
                g = r.get("groups")
                if g:
                    _need(g, ("count", "keep"), f"{where}.mlp.router.groups")
                    _positive_int(g["count"], f"{where}.mlp.router.groups.count")
                    _positive_int(g["keep"], f"{where}.mlp.router.groups.keep")
                    if n % g["count"] or g["keep"] > g["count"]:
                        raise ConfigError(f"config.json: {where}.mlp.router.groups: {n} experts in {g['count']} groups, "
                                          f"{g['keep']} kept")
            else:
                raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not built ('dense', 'moe')")
        if self.loop:
            _need(self.loop, ("start", "stop", "times"), "loop")
            a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            _positive_int(times, "loop.times")
            if not (isinstance(a, int) and isinstance(b, int) and 0 <= a < b <= len(self.layers)):
                raise ConfigError(f"config.json: loop {a}..{b} does not name layers of the {len(self.layers)}")

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": self.norm,
             "embedding": self.embedding, "layers": self.layers, "max_positions": self.max_positions}
        if self.loop:
            d["loop"] = self.loop
        return d
