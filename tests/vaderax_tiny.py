"""Small Vaderax configurations for the tests and random weights for them.

The configurations differ from one another in every size and option: layer order, a layer without feed-forward,
grouped / ungrouped / single key heads, value size below and above the key size, a rotated prefix, whole heads and
no rotation, one to five taps, experts with and without identity experts, one and several choices, groups absent,
all kept and some kept, a loop at the start, in the middle, over one layer, and none, widths that the tensor-core
products take and refuse.
"""
from __future__ import annotations

import torch

from rbitnet_b200.config import config_from_dict
from rbitnet_b200.config.registry import get_architecture
from rbitnet_b200.weights import random_tensors


def attention_layer(heads, kv, dim, vdim, rot_dims=None, base=100.0, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def delta_layer(heads, kv, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=None, groups=None):
    r = {"experts": experts, "top": top}
    if identity is not None:
        r["identity"] = identity
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


#: a loop over the first two layers; a delta layer first; identity experts; two of four groups kept; a layer without feed-forward
CFG_A = {"architecture": "Vaderax", "vocab": 96, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
         "layers": [delta_layer(4, 2, 16, 24, 3, moe(6, 2, 40, identity=2, groups=(4, 2))),
                    attention_layer(4, 2, 32, 16, 8, base=100.0, scale=0.6, mlp=dense(80)),
                    delta_layer(2, 2, 8, 8, 5, None)],
         "loop": {"start": 0, "stop": 2, "times": 2}}

#: no loop; ungrouped heads; values wider than keys; whole heads turn; one choice, no identity experts, no groups; one tap
CFG_B = {"architecture": "Vaderax", "vocab": 64, "width": 80, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
         "layers": [attention_layer(2, 2, 16, 40, 16, base=50.0, scale=0.7, mlp=moe(5, 1, 24)),
                    delta_layer(1, 1, 40, 8, 1, dense(96))]}

#: a width the tensor-core products refuse; no rotation; a single key head; as many identity experts as experts, every
#: group kept; a loop of one layer, three times
CFG_C = {"architecture": "Vaderax", "vocab": 70, "width": 100, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
         "layers": [attention_layer(3, 1, 24, 24, None, scale=0.5, mlp=moe(3, 3, 36, identity=3, groups=(3, 3))),
                    delta_layer(6, 3, 8, 12, 2, moe(4, 2, 20, identity=0, groups=(2, 1)))],
         "loop": {"start": 1, "stop": 2, "times": 3}}

#: larger heads: keys of 64 and 128 (the tensor-core attention), a delta rule whose keys take eight lanes, many experts,
#: a loop in the middle that runs once only
CFG_D = {"architecture": "Vaderax", "vocab": 300, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
         "layers": [attention_layer(4, 2, 64, 64, 32, base=10000.0, scale=0.2, mlp=moe(8, 2, 128, groups=(2, 1))),
                    delta_layer(4, 2, 128, 64, 4, dense(512)),
                    attention_layer(2, 1, 128, 96, 64, base=5000.0, scale=0.15, mlp=moe(16, 4, 64, identity=4, groups=(5, 2)))],
         "loop": {"start": 1, "stop": 3, "times": 1}}

#: only delta layers (no cache of keys at all), two of them looped to the end
CFG_E = {"architecture": "Vaderax", "vocab": 50, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
         "layers": [delta_layer(3, 1, 16, 16, 4, dense(64)), delta_layer(2, 2, 24, 8, 2, moe(2, 2, 16, identity=1))],
         "loop": {"start": 0, "stop": 2, "times": 2}}

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D, "E": CFG_E}


def spec_of(cfg_dict):
    cfg = config_from_dict(cfg_dict)
    return get_architecture(cfg.architecture).build_spec(cfg)


def make_tensors(cfg_dict, seed, spread=8.0, long_memory=True):
    """Random weights, then made so that faults show: matrices are scaled up (random weights of deviation 0.02 give
    nearly uniform attention, gates stuck at one half and a router without preferences); with ``long_memory`` the
    delta rule forgets slowly, so that a token far back still moves the logits."""
    t = random_tensors(spec_of(cfg_dict), seed)
    out = {}
    for name, v in t.items():
        v = v.clone()
        if name.endswith(".router"):
            v = v * 3.0 * spread
        elif name.endswith(".correction"):
            v = v * 2.0                       # of the size of the scores' differences: both decide the choice
        elif name.endswith(".A_log"):
            v = v * 20.0 - (4.0 if long_memory else 0.0)
        elif name.endswith(".dt_bias"):
            v = v * 20.0
        elif name.endswith("norm1.b") or name.endswith("norm2.b") or name == "final.norm.b":
            v = v * 10.0
        elif v.dim() >= 2 and not name.endswith(".conv"):
            v = v * spread
        out[name] = v.to(torch.bfloat16).to(torch.float32)     # values both dtypes of the engine can hold
    return out
