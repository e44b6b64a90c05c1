"""Small Safuvik configurations for the tests, random weights for them, and ways to run an engine.

The configurations differ from one another in every size and option: streams (several, one, absent),
layer order, a layer without feed-forward, grouped / ungrouped / single key heads, value size below and
above the key size, a rotated prefix and whole heads, stretched and plain frequencies, windows that end
inside a page, on a page border and beyond the sequence, one and several blocks, two to four taps, one
and several memory heads, key sizes that one or two lanes hold.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from rbitnet_b200.config import config_from_dict
from rbitnet_b200.config.registry import get_architecture
from rbitnet_b200.weights import random_tensors, write_safetensors


def _left(heads, kv, dim, vdim, window, rot_dims, scaling=None, base=1000.0, scale=None):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window:
        left["mask"] = {"size": window}
    if rot_dims:
        left["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            left["rot"]["scaling"] = scaling
    return left


def parallel_layer(left, width, blocks, conv, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv}}, "mlp": mlp}


def memory_layer(heads, dim, vdim, cap, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


#: three streams; memory first; a layer without feed-forward; a short window; a rotated prefix with stretched frequencies
CFG_A = {"architecture": "Safuvik", "vocab": 96, "width": 64, "norm": {"eps": 1e-5}, "streams": 3, "logit_scale": 0.5,
         "layers": [memory_layer(2, 16, 24, 8.0, dense(80, 2.0)),
                    parallel_layer(_left(4, 2, 32, 16, 9, 8, {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 2.0}, scale=0.6),
                                   48, 3, 3, dense(72, 0.75)),
                    parallel_layer(_left(4, 2, 32, 16, 9, 8, {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 2.0}, scale=0.6),
                                   48, 3, 3, None)]}

#: one stream with its weights; ungrouped heads; values wider than keys; whole heads turn, plain frequencies; a window
#: that spans a page border; one block; two taps; one memory head whose keys take two lanes; no logit scale
CFG_B = {"architecture": "Safuvik", "vocab": 64, "width": 80, "norm": {"eps": 1e-6}, "streams": 1,
         "layers": [parallel_layer(_left(2, 2, 16, 40, 70, 16, None, base=50.0, scale=0.7), 32, 1, 2, dense(96, 3.0)),
                    memory_layer(1, 40, 8, 15.0, None),
                    memory_layer(3, 8, 8, 4.0, dense(40, 1.0))]}

#: no streams key (the ordinary residual sum); no window, no rotation; four taps; a window of exactly one page elsewhere
CFG_C = {"architecture": "Safuvik", "vocab": 48, "width": 48, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
         "layers": [parallel_layer(_left(3, 1, 24, 24, None, None, scale=0.5), 24, 2, 4, dense(64, 1.5)),
                    parallel_layer(_left(2, 1, 16, 8, 64, 4, None, base=100.0, scale=0.9), 40, 5, 1, dense(64, 1.5))]}

#: only matrix memories (no cache of keys at all); a width that the tensor-core products refuse; five streams
CFG_D = {"architecture": "Safuvik", "vocab": 70, "width": 100, "norm": {"eps": 1e-6}, "streams": 5, "logit_scale": 1.5,
         "layers": [memory_layer(2, 12, 20, 6.0, dense(50, 2.5)), memory_layer(5, 4, 36, 20.0, None)]}

#: only parallel layers; windows of one and two tokens; one head whose keys and values have the same size; one rotated pair
CFG_E = {"architecture": "Safuvik", "vocab": 50, "width": 64, "norm": {"eps": 1e-5}, "streams": 2,
         "layers": [parallel_layer(_left(1, 1, 64, 64, 1, 2, None, base=10.0, scale=0.3), 64, 8, 2, dense(64, 1.0)),
                    parallel_layer(_left(6, 3, 16, 16, 2, 16, {"factor": 8.0, "original": 8, "fast": 4.0, "slow": 1.0}, scale=0.5),
                                   16, 1, 5, dense(48, 4.0))]}

#: larger heads: key sizes of 64 and 128 (the tensor-core attention and the memory kernel's sixteen lanes per column),
#: blocks of 128 channels, four streams
CFG_F = {"architecture": "Safuvik", "vocab": 300, "width": 256, "norm": {"eps": 1e-6}, "streams": 4, "logit_scale": 0.25,
         "layers": [parallel_layer(_left(4, 2, 64, 64, 100, 32, {"factor": 2.0, "original": 64, "fast": 16.0, "slow": 2.0}, scale=0.4),
                                   256, 2, 4, dense(512, 6.0)),
                    memory_layer(2, 128, 128, 10.0, dense(384, 2.0)),
                    parallel_layer(_left(2, 1, 128, 96, 40, 64, None, base=5000.0, scale=0.3), 128, 4, 3, None)]}

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D, "E": CFG_E, "F": CFG_F}


def spec_of(cfg_dict):
    cfg = config_from_dict(cfg_dict)
    return get_architecture(cfg.architecture).build_spec(cfg)


def make_tensors(cfg_dict, seed, spread=8.0, long_memory=True):
    """Random weights, then made so that faults show: matrices are scaled up (random weights of deviation
    0.02 give nearly uniform attention and gates stuck at one half); with ``long_memory`` the recurrent
    layers forget slowly, so that a token far back still moves the logits."""
    t = random_tensors(spec_of(cfg_dict), seed)
    out = {}
    for name, v in t.items():
        v = v.clone()
        if v.dim() >= 2 and ".hc" not in name and not name.endswith(".conv"):
            v = v * spread
        if name.endswith(".b") and not name.endswith("conv.b"):
            v = v * 20.0
        if long_memory and name.endswith(".lam"):
            v = v * 30.0 - 4.0            # softplus small: decays near one
        if long_memory and name.endswith(".f.b"):
            v = v + 4.0                   # forget gates near one
        out[name] = v.to(torch.bfloat16).to(torch.float32)     # values both dtypes of the engine can hold
    return out


def write_model(folder, cfg_dict, tensors, store=torch.float32):
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg_dict))
    write_safetensors(folder / "model.safetensors", {k: v.to(store).contiguous() for k, v in tensors.items()})
    return folder


def tokens_for(cfg_dict, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg_dict["vocab"], (n,), generator=g).tolist()


def run_cut(engine, tokens, cuts, want_all=True):
    """One sequence alone, its tokens cut into steps at ``cuts`` (ascending positions inside it);
    returns the logits at every position [T, vocab]."""
    from rbitnet_b200.engine.step import StepEntry
    slot = engine.new_sequence()
    edges = [0] + sorted({c for c in cuts if 0 < c < len(tokens)}) + [len(tokens)]
    outs = []
    for a, b in zip(edges[:-1], edges[1:]):
        outs.append(engine.step([StepEntry(slot, tokens[a:b], list(range(b - a)))]))
    engine.end_sequence(slot)
    return torch.cat(outs).float().cpu()


def rel_err(got, ref):
    """Largest difference as a fraction of the largest reference value."""
    got, ref = got.double().cpu(), ref.double()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all()
    return float((got - ref).abs().max() / ref.abs().max())
