"""The Vaderax decoder as data: which parts its layers are made of, in which order they run, and its tensor names.

Embedding times `embedding.scale`; pre-norm layers (layer norms with weight and bias), each a mixer and, unless
"mlp" is null, a feed-forward; a final layer norm; a linear head.  A span of layers ("loop") runs several times in
a row with the same weights: every run has its own cache or state, and before every pass but the first the embedded
rows are added to the residual stream.

Layer types:
  "attention"  grouped causal attention: rotation of a prefix of every head in pairs (i, i + dims/2), then a
               weightless RMS norm of every q and k head, softmax with the scale config.json gives, a sigmoid gate
               per value on the joined heads
  "delta"      the gated delta rule behind short convolutions
Feed-forwards: "dense" (down(relu2(up h))) and "moe" (routed experts of that form, identity experts, a choice among
the best groups by score plus correction).

Tensor names: "embed", "head", "final.norm", "final.norm.b"; layer i: "l<i>.norm1", "l<i>.norm1.b", "l<i>.norm2",
"l<i>.norm2.b", "l<i>.mix.<key>", "l<i>.mlp.<key>", where <key> is the part's weight key ("q", "q.conv", "A_log",
"router", "e3.up", ...).
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vaderax import VaderaxConfig
from ..parts import PartSpec, BlockSpec, ScheduleEntry, ModelSpec, build_part

#: added to the sum of squares under the root when q and k of the delta rule are made unit vectors, fixed by the design
_UNIT_EPS = 1e-6


def _attention(cfg: VaderaxConfig, m: dict) -> PartSpec:
    rot = m.get("rot")
    position = None
    if rot:
        position = {"kind": "rotary", "params": {"head_dim": m["dim"], "theta": float(rot["base"]), "pairing": "half",
                                                 "rot_dim": rot["dims"], "max_positions": cfg.max_positions}}
    return PartSpec("attention", {
        "width": cfg.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "position": position, "scale": float(m["scale"]), "qk_norm": "head",
        "norm_eps": float(cfg.norm["eps"]), "value_gate": True})


def _delta(cfg: VaderaxConfig, m: dict) -> PartSpec:
    return PartSpec("gated_delta_rule", {
        "width": cfg.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "taps": m["conv"], "norm_eps": float(cfg.norm["eps"]), "unit_eps": _UNIT_EPS})


def _feed_forward(cfg: VaderaxConfig, mlp: dict) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("dense", {"width": cfg.width, "inner": mlp["ff"], "activation": "relu2"})
    r = mlp["router"]
    g = r.get("groups") or {}
    return PartSpec("routed_experts", {
        "width": cfg.width, "inner": mlp["expert"]["ff"], "n_experts": r["experts"], "top": r["top"],
        "n_identity": r.get("identity") or 0, "groups": g.get("count", 0), "keep": g.get("keep", 0),
        "correction": True, "activation": "relu2"})


_MIXERS = {"attention": _attention, "delta": _delta}


def layer_schedule(n_layers: int, loop) -> list:
    """The runs of the layers in order: [(layer, adds the embedded rows first)]."""
    if not loop:
        return [(i, False) for i in range(n_layers)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for p in range(times):
        runs += [(i, p > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n_layers)]


def build_vaderax_spec(cfg: VaderaxConfig) -> ModelSpec:
    norm = PartSpec("layernorm", {"width": cfg.width, "eps": float(cfg.norm["eps"]), "bias": True})
    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = {"mixer": _MIXERS[layer["type"]](cfg, layer["mixer"]), "mixer_norm": norm}
        names = {"mixer_norm.weight": f"l{i}.norm1", "mixer_norm.bias": f"l{i}.norm1.b"}
        mlp = layer.get("mlp")
        if mlp is not None:
            parts["feed_forward"], parts["ffn_norm"] = _feed_forward(cfg, mlp), norm
            names["ffn_norm.weight"], names["ffn_norm.bias"] = f"l{i}.norm2", f"l{i}.norm2.b"
        for part_name, prefix in (("mixer", "mix"), ("feed_forward", "mlp")):
            if part_name in parts:
                for key in build_part(part_name, parts[part_name]).weight_shapes():
                    names[f"{part_name}.{key}"] = f"l{i}.{prefix}.{key}"
        layers.append(BlockSpec(parts=parts, names=names, arrangement="pre_norm"))
    return ModelSpec(
        width=cfg.width, vocab_size=cfg.vocab, embedding_name="embed", layers=layers,
        schedule=[ScheduleEntry(i, adds_embedding=again) for i, again in layer_schedule(len(layers), cfg.loop)],
        final_norm=norm, final_norm_names={"weight": "final.norm", "bias": "final.norm.b"}, head_name="head",
        max_positions=cfg.max_positions, stop_ids=[], embedding_scale=float(cfg.embedding["scale"]))


register_architecture("Vaderax", VaderaxConfig, build_vaderax_spec)
