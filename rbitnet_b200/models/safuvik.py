"""The Safuvik decoder as data: which parts its layers are made of, and its tensor names.

Embedding; layers in the order config.json lists them, each a mixer and (unless "mlp" is null) a
limited gated feed-forward, each behind an RMS norm, over `streams` residual rows per token
(hyper-connections); the sum of the rows; a final RMS norm; a linear head whose logits are
multiplied by `logit_scale`.

Layer types:
  "parallel"  grouped window attention (norm over the whole q and k projections, rotation of a prefix of
              every head with stretched frequencies, a sigmoid gate per head, values of their own size)
              beside a gated linear recurrence behind a short convolution; the mean of the two results,
              each under its own RMS norm
  "mlstm"     a matrix memory per head with capped exponential gates

Tensor names: "embed", "head", "final.norm"; layer i: "l<i>.norm1", "l<i>.norm2", "l<i>.hc1.{in,out,mix}",
"l<i>.hc2.{...}", "l<i>.mix.<key>", "l<i>.mlp.{gate,up,down}", where <key> is the mixer's weight key
("left.q", "right.conv.b", "q", "i.b", ...).
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.safuvik import SafuvikConfig
from ..parts import PartSpec, BlockSpec, ScheduleEntry, ModelSpec, build_part

#: the decay exponent's multiplier in the gated linear recurrence, fixed by the design
_DECAY_SCALE = 8.0
#: the limited feed-forward's sigmoid slope and the up branch's shift, fixed by the design
_FF_ALPHA, _FF_SHIFT = 1.702, 1.0


def _parallel(cfg: SafuvikConfig, m: dict) -> PartSpec:
    left, right = m["left"], m["right"]
    eps = float(cfg.norm["eps"])
    rot = left.get("rot")
    position = None
    if rot:
        position = {"kind": "rotary", "params": {"head_dim": left["dim"], "theta": float(rot["base"]),
                                                 "pairing": "interleaved", "rot_dim": rot["dims"],
                                                 "scaling": rot.get("scaling"), "max_positions": cfg.max_positions}}
    attention = {"kind": "attention", "params": {
        "width": cfg.width, "n_heads": left["heads"], "n_kv_heads": left["kv_heads"], "head_dim": left["dim"],
        "value_dim": left["vdim"], "position": position, "window": (left.get("mask") or {}).get("size"),
        "scale": float(left["scale"]), "qk_norm": "projection", "norm_eps": eps, "head_gate": True}}
    recurrence = {"kind": "gated_linear_recurrence", "params": {
        "width": cfg.width, "inner": right["width"], "blocks": right["blocks"], "taps": right["conv"],
        "decay_scale": _DECAY_SCALE}}
    return PartSpec("parallel", {"width": cfg.width, "norm_eps": eps,
                                 "branches": {"left": attention, "right": recurrence}})


def _matrix_memory(cfg: SafuvikConfig, m: dict) -> PartSpec:
    return PartSpec("matrix_memory", {"width": cfg.width, "n_heads": m["heads"], "head_dim": m["dim"],
                                      "value_dim": m["vdim"], "gate_cap": float(m["gate_cap"]),
                                      "norm_eps": float(cfg.norm["eps"])})


_MIXERS = {"parallel": _parallel, "mlstm": _matrix_memory}


def build_safuvik_spec(cfg: SafuvikConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"width": cfg.width, "eps": float(cfg.norm["eps"])})
    s = cfg.streams
    connection = PartSpec("hyper", {"streams": s}) if s is not None else PartSpec("residual", {})
    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = {"mixer": _MIXERS[layer["type"]](cfg, layer["mixer"]), "mixer_norm": norm, "mixer_connection": connection}
        mlp = layer.get("mlp")
        if mlp is not None:
            parts["feed_forward"] = PartSpec("gated_dense", {"width": cfg.width, "inner": mlp["ff"],
                                                            "activation": "swish_limited", "limit": float(mlp["limit"]),
                                                            "alpha": _FF_ALPHA, "shift": _FF_SHIFT})
            parts["ffn_norm"], parts["ffn_connection"] = norm, connection
        names = {"mixer_norm.weight": f"l{i}.norm1"}
        if mlp is not None:
            names["ffn_norm.weight"] = f"l{i}.norm2"
        for part_name, prefix in (("mixer", "mix"), ("feed_forward", "mlp"), ("mixer_connection", "hc1"),
                                  ("ffn_connection", "hc2")):
            if part_name in parts:
                spec = parts[part_name]
                role = {"mixer": "mixer", "feed_forward": "feed_forward"}.get(part_name, "connection")
                for key in build_part(role, spec).weight_shapes():
                    names[f"{part_name}.{key}"] = f"l{i}.{prefix}.{key}"
        layers.append(BlockSpec(parts=parts, names=names, arrangement="multi_stream"))
    return ModelSpec(
        width=cfg.width, vocab_size=cfg.vocab, embedding_name="embed", layers=layers,
        schedule=[ScheduleEntry(i) for i in range(len(layers))],
        final_norm=norm, final_norm_names={"weight": "final.norm"}, head_name="head",
        max_positions=cfg.max_positions, stop_ids=[], logit_scale=float(cfg.logit_scale),
        residual_streams=int(s) if s is not None else 1)


register_architecture("Safuvik", SafuvikConfig, build_safuvik_spec)
