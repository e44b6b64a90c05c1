"""A plain, slow implementation of the Safuvik decoder, for tests only: one function per
mechanism, whole sequences, no cache, no batching, any float type.  It shares no code with
the package: it reads config.json's dictionary and the stored tensors by name.

Notation: h [T, E] are a sequence's rows, positions 0..T-1; weights are stored [out, in].

  rms(x)        x / sqrt(mean(x^2) + eps)
  hyper-connections: s residual streams X [s, T, E]; a sublayer reads u = sum_s in[s] X_s, and writes
                X'_t = sum_s mix[s, t] X_s + out[t] * sublayer(norm(u))
  window attention with grouped heads, a norm over the whole q (k) projection, rotation of a prefix of
                every head with stretched frequencies, a sigmoid gate per head
  gated linear recurrence: S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t behind a short causal convolution
  matrix memory: C_t = e^(f + m' - m) C_(t-1) + e^(i - m) k v^T with a running maximum m
  clamped gated feed-forward
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_tables(rot, T, dt):
    """cos, sin [T, dims/2] of the rotated prefix, with the stretched frequencies and the magnitude."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def dim_of(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(T, dtype=torch.float64)[:, None] * f[None, :]
    return (torch.cos(ang) * mag).to(dt), (torch.sin(ang) * mag).to(dt)


def rotate_prefix(x, cos, sin, dims):
    """x [T, heads, D]: pairs (2i, 2i+1) of the first ``dims`` values of every head turn by the position's angle."""
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    c, s = cos[:, None, :], sin[:, None, :]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def window_attention(w, p, h, eps):
    """The left half of the parallel mixer.  ``w``: its tensors by short name; ``p``: its sizes."""
    T = h.shape[0]
    H, G, D, Dv = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    q = rms(q, eps) * w["q.norm"]
    k = rms(k, eps) * w["k.norm"]
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, Dv)
    rot = p.get("rot")
    if rot:
        cos, sin = rotary_tables(rot, T, h.dtype)
        q, k = rotate_prefix(q, cos, sin, int(rot["dims"])), rotate_prefix(k, cos, sin, int(rot["dims"]))
    size = (p.get("mask") or {}).get("size")
    pos = torch.arange(T)
    dist = pos[:, None] - pos[None, :]
    seen = dist >= 0
    if size:
        seen = seen & (dist < int(size))
    gate = torch.sigmoid(h @ w["g"].T)                        # [T, H]
    out = torch.empty(T, H, Dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd, :] @ k[:, g, :].T) * float(p["scale"])
        s = s.masked_fill(~seen, -math.inf)
        out[:, hd, :] = torch.softmax(s, dim=-1) @ v[:, g, :]
    out = out * gate[:, :, None]
    return out.reshape(T, H * Dv) @ w["o"].T


def causal_conv(x, taps, bias):
    """x [T, C], taps [C, K] (the last column is the current token's), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], dim=0)
    out = bias.expand(T, C).clone()
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j]
    return out


def gated_recurrence(w, p, h):
    """The right half of the parallel mixer."""
    T = h.shape[0]
    W, B = int(p["width"]), int(p["blocks"])
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    u = causal_conv(h @ w["x"].T + w["x.b"], w["conv"], w["conv.b"])
    ub = u.view(T, B, W // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w["ra"], ub) + w["ra.b"]).reshape(T, W)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w["ri"], ub) + w["ri.b"]).reshape(T, W)
    log_a = -8.0 * r * torch.nn.functional.softplus(w["lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(W, dtype=h.dtype)
    states = torch.empty(T, W, dtype=h.dtype)
    for t in range(T):
        S = a[t] * S + drive[t]
        states[t] = S
    return (states * y) @ w["o"].T


def parallel_mixer(w, p, h, eps):
    left = {k[len("left."):]: v for k, v in w.items() if k.startswith("left.")}
    right = {k[len("right."):]: v for k, v in w.items() if k.startswith("right.")}
    a = rms(window_attention(left, p["left"], h, eps), eps) * w["left.out"]
    b = rms(gated_recurrence(right, p["right"], h), eps) * w["right.out"]
    return 0.5 * (a + b)


def matrix_memory(w, p, h, eps):
    T = h.shape[0]
    H, D, Dv, cap = int(p["heads"]), int(p["dim"]), int(p["vdim"]), float(p["gate_cap"])
    q = (h @ w["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).view(T, H, D)
    v = (h @ w["v"].T).view(T, H, Dv)
    ig = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)                               # [T, H]
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    C = torch.zeros(H, D, Dv, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    m = torch.zeros(H, dtype=h.dtype)
    out = torch.empty(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        keep, take = torch.exp(fg[t] + m - m_new), torch.exp(ig[t] - m_new)
        C = keep[:, None, None] * C + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", C, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    out = rms(out, eps).reshape(T, H * Dv) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def clamped_feed_forward(w, p, h):
    limit = float(p["limit"])
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def hyper_read(X, w_in):
    return torch.einsum("s,ste->te", w_in, X)


def hyper_write(X, mix, w_out, y):
    return torch.einsum("st,sne->tne", mix, X) + w_out[:, None, None] * y[None]


def forward(cfg: dict, tensors: dict, tokens, dt=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the sum of the
    streams after every layer."""
    W = {k: v.to(dt) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    s = cfg.get("streams")
    X = x[None].repeat(int(s), 1, 1) if s else None
    for li, layer in enumerate(cfg["layers"]):
        pre = f"l{li}."
        mw = {k[len(pre + "mix."):]: v for k, v in W.items() if k.startswith(pre + "mix.")}
        fw = {k[len(pre + "mlp."):]: v for k, v in W.items() if k.startswith(pre + "mlp.")}

        def mixer(hh):
            if layer["type"] == "parallel":
                return parallel_mixer(mw, layer["mixer"], hh, eps)
            if layer["type"] == "mlstm":
                return matrix_memory(mw, layer["mixer"], hh, eps)
            raise ValueError(layer["type"])
        subs = [(1, mixer)]
        if layer.get("mlp"):
            subs.append((2, lambda hh: clamped_feed_forward(fw, layer["mlp"], hh)))
        for qn, fn in subs:
            nw = W[f"{pre}norm{qn}"]
            if X is None:
                x = x + fn(rms(x, eps) * nw)
            else:
                u = hyper_read(X, W[f"{pre}hc{qn}.in"])
                X = hyper_write(X, W[f"{pre}hc{qn}.mix"], W[f"{pre}hc{qn}.out"], fn(rms(u, eps) * nw))
        if layers_out is not None:
            layers_out.append((X.sum(0) if X is not None else x).clone())
    if X is not None:
        x = X.sum(0)
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T * float(cfg.get("logit_scale", 1.0))
