"""A plain, slow implementation of the Vaderax decoder, for tests only: one function per
mechanism, whole sequences, no cache, no batching, any float type.  It shares no code with
the package: it reads config.json's dictionary and the stored tensors by name.

Notation: h [T, E] are a sequence's rows, positions 0..T-1; weights are stored [out, in].

  layer_norm(x)   (x - mean) / sqrt(var + eps) * w + b
  rotate_half     the first `dims` values of a head turn in pairs (i, i + dims/2)
  attention       grouped heads, rotation, a weightless RMS norm per head on q and k after the
                  rotation, causal softmax, an elementwise sigmoid gate on the joined heads
  delta rule      per head S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
  relu2 feed-forward, and a routed one: softmax scores, choice among the best groups by the
                  score plus a correction, identity experts, weights not renormalised
  loop            a span of layers runs several times, the embedded rows added before every pass but the first
"""
from __future__ import annotations

import math

import torch


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def relu2(z):
    return torch.clamp(z, min=0.0) ** 2


def rotate_half(x, base, dims, first_position=0):
    """x [T, heads, D]: value i of the first ``dims`` turns with value i + dims/2 by position * base^(-2i/dims)."""
    T = x.shape[0]
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    ang = (torch.arange(T, dtype=torch.float64) + first_position)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    out = x.clone()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def attention(h, m, w, eps):
    """m: the layer's "mixer" dictionary; w: name -> tensor of the mixer ("q", "k", "v", "g", "o")."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, D)
    k = (h @ w["k"].T).view(T, G, D)
    v = (h @ w["v"].T).view(T, G, Dv)
    rot = m.get("rot")
    if rot:
        q, k = rotate_half(q, rot["base"], rot["dims"]), rotate_half(k, rot["base"], rot["dims"])
    q, k = rms(q, eps), rms(k, eps)
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for head in range(H):
        kv = head // (H // G)
        s = (q[:, head] @ k[:, kv].T) * float(m["scale"])
        s = s.masked_fill(~visible, -math.inf)
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, kv]
    gate = torch.sigmoid(h @ w["g"].T)
    return (out.reshape(T, H * Dv) * gate) @ w["o"].T


def short_conv(x, taps):
    """x [T, C], taps [C, K]: y_t = sum_j taps[:, K-1-j] x_(t-j), zeros before the start."""
    T, K = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j]
    return y


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g):
    """q, k [T, H, D], v [T, H, Dv], beta, g [T, H] -> o [T, H, Dv]; the state starts at zero."""
    T, H, D = q.shape
    Dv = v.shape[-1]
    S = torch.zeros(H, D, Dv, dtype=q.dtype)
    o = torch.zeros(T, H, Dv, dtype=q.dtype)
    for t in range(T):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o


def delta_mixer(h, m, w, eps):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).view(T, G, D)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).view(T, G, D)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).view(T, H, Dv)
    q, k = unit(q) * D ** -0.5, unit(k)
    share = torch.arange(H) // (H // G)
    q, k = q[:, share], k[:, share]
    beta = torch.sigmoid(h @ w["b"].T)
    g = torch.exp(-torch.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))
    o = delta_rule(q, k, v, beta, g)
    o = rms(o, eps) * w["norm"] * silu(h @ w["g"].T).view(T, H, Dv)
    return o.reshape(T, H * Dv) @ w["o"].T


def dense_ff(h, w):
    return relu2(h @ w["up"].T) @ w["down"].T


def route(h, r, w):
    """-> (chosen [T, top] indices, weights [T, top]); indices >= r["experts"] are identity experts."""
    n, ident, top = r["experts"], r.get("identity", 0), r["top"]
    s = torch.softmax(h @ w["router"].T, dim=-1)                     # [T, n + ident]
    choice = s + w["correction"]
    groups = r.get("groups")
    if groups:
        per = (n + ident) // groups["count"]
        best = choice.view(-1, groups["count"], per).max(-1).values
        keep = best.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, keep, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    chosen = choice.topk(top, dim=-1).indices
    return chosen, s.gather(1, chosen)


def routed_ff(h, mlp, w):
    r = mlp["router"]
    chosen, weights = route(h, r, w)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(chosen[t].tolist(), weights[t]):
            if e >= r["experts"]:
                out[t] += p * h[t]
            else:
                out[t] += p * (relu2(h[t] @ w[f"e{e}.up"].T) @ w[f"e{e}.down"].T)
    return out


def layer_order(cfg):
    """[(layer, adds the embedded rows first)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for p in range(times):
        order += [(i, p > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def _sub(tensors, prefix, dt):
    return {k[len(prefix):]: v.to(dt) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, dt=torch.float64, layer_outputs=None):
    """Logits [T, vocab] of one sequence."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x0 = tensors["embed"].to(dt)[ids] * float(cfg["embedding"]["scale"])
    x = x0.clone()
    for i, again in layer_order(cfg):
        layer = cfg["layers"][i]
        w = _sub(tensors, f"l{i}.", dt)
        if again:
            x = x + x0
        h = layer_norm(x, w["norm1"], w["norm1.b"], eps)
        mix = _sub(w, "mix.", dt)
        x = x + (attention if layer["type"] == "attention" else delta_mixer)(h, layer["mixer"], mix, eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w["norm2"], w["norm2.b"], eps)
            ff = _sub(w, "mlp.", dt)
            x = x + (dense_ff(h, ff) if mlp["kind"] == "dense" else routed_ff(h, mlp, ff))
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = layer_norm(x, tensors["final.norm"].to(dt), tensors["final.norm.b"].to(dt), eps)
    return x @ tensors["head"].to(dt).T
