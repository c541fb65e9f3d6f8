"""Zepalorn, stated plainly: one slow function per mechanism, whole sequences, no cache, no batching.

Nothing here is shared with the package: the functions take the raw ``config.json`` dictionary and a dictionary of
checkpoint tensors by name, and work on one sequence ``[T, width]`` at a time in the dtype they are given (float64 for
an oracle that rounding does not touch). The recurrent mixers are loops over the tokens, the attention builds its mask
as a matrix.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------------------------ small pieces
def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w, the variance being the mean squared deviation; no bias."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def causal_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([u.new_zeros(taps - 1, C), u])
    y = u.new_zeros(T, C)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    if bias is not None:
        y = y + bias
    return y


# ------------------------------------------------------------------------------------------------------------ rotation
def rotary_frequencies(rot: dict, dtype):
    """(frequency of every pair [dims / 2], factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor = float(sc["factor"])

        def dim_of(turns):
            return dims * math.log(float(sc["original"]) / (2 * math.pi * turns)) / (2 * math.log(base))

        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
        ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=torch.float64)
        f = f / factor * ramp + f * (1 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    return f.to(dtype), mult


def rotate(x, positions, rot: Optional[dict], interleaved: bool):
    """x [T, heads, dim]; the first rot.dims entries of every head turn, the rest pass."""
    if not rot:
        return x
    dims = int(rot["dims"])
    f, mult = rotary_frequencies(rot, x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]                    # [T, dims / 2]
    cos, sin = (torch.cos(a) * mult)[:, None, :], (torch.sin(a) * mult)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * cos - v * sin
        out[..., dims // 2:dims] = v * cos + u * sin
    return out


# ------------------------------------------------------------------------------------------------------------ attention
def visible(T: int, kind: str, mask: Optional[dict]):
    """Boolean [T, T]: row i sees column j."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if mask:
        size = int(mask["size"])
        if kind == "chunk":
            ok = ok & (i // size == j // size)
        else:
            ok = ok & ((i - j < size) | (j < int(mask.get("keep_first", 0))))
    return ok


def softmax_attention(m: dict, W: Dict[str, torch.Tensor], p: str, h, eps: float, flavour: str):
    """The two attention mixers. ``flavour`` 'window': plain projections, rotate-half layout, sliding window with kept first
    tokens. 'chunk': short convolutions, query/key norm, interleaved layout, soft cap on the scores, chunked mask."""
    T = h.shape[0]
    H, G, D, DV = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m.get("vdim", m["dim"]))
    q, k, v = h @ W[p + ".q"].T, h @ W[p + ".k"].T, h @ W[p + ".v"].T
    if flavour == "chunk":
        q, k, v = causal_conv(q, W[p + ".q.conv"]), causal_conv(k, W[p + ".k.conv"]), causal_conv(v, W[p + ".v.conv"])
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, DV)
    if flavour == "chunk":
        q = rms_unit(q, eps) * W[p + ".q.norm"]
        k = rms_unit(k, eps) * W[p + ".k.norm"]
    pos = torch.arange(T)
    q = rotate(q, pos, m.get("rot"), interleaved=(flavour == "chunk"))
    k = rotate(k, pos, m.get("rot"), interleaved=(flavour == "chunk"))
    ok = visible(T, flavour, m.get("mask"))
    out = h.new_zeros(T, H, DV)
    for head in range(H):
        kv = head // (H // G)
        s = (q[:, head] @ k[:, kv].T) * float(m["scale"])
        if m.get("softcap"):
            cap = float(m["softcap"])
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~ok, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, kv]
    return out.reshape(T, H * DV) @ W[p + ".o"].T


# ------------------------------------------------------------------------------------------------------------ gated delta rule
def channel_delta(m: dict, W: Dict[str, torch.Tensor], p: str, h, eps: float):
    T = h.shape[0]
    H, G, D, DV = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_conv(h @ W[p + ".q"].T, W[p + ".q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ W[p + ".k"].T, W[p + ".k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ W[p + ".v"].T, W[p + ".v.conv"])).view(T, H, DV)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + ".b"].T)                                                  # [T, H]
    dt = softplus((h @ W[p + ".a1"].T) @ W[p + ".a2"].T + W[p + ".dt_bias"]).view(T, H, D)
    decay = torch.exp(-torch.exp(W[p + ".A_log"])[None, :, None] * dt)                       # [T, H, D]
    gate = torch.sigmoid((h @ W[p + ".g1"].T) @ W[p + ".g2"].T).view(T, H, DV)
    out = h.new_zeros(T, H, DV)
    for head in range(H):
        kv = head // (H // G)
        S = h.new_zeros(D, DV)
        for t in range(T):
            S = decay[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, head] = S.T @ q[t, kv]
    out = rms_unit(out, eps) * W[p + ".norm"] * gate
    return out.reshape(T, H * DV) @ W[p + ".o"].T


# ------------------------------------------------------------------------------------------------------------ state-space mixer
def state_space(m: dict, W: Dict[str, torch.Tensor], p: str, h, eps: float):
    T = h.shape[0]
    H, DV, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * DV
    zxbcdt = h @ W[p + ".in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + ".conv"], W[p + ".conv.b"]))
    x = xbc[:, :inner].view(T, H, DV)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[p + ".dt_bias"])                                                     # [T, H]
    a = torch.exp(-torch.exp(W[p + ".A_log"])[None, :] * dt)
    y = h.new_zeros(T, H, DV)
    for head in range(H):
        g = head // (H // G)
        S = h.new_zeros(N, DV)
        for t in range(T):
            S = a[t, head] * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + W[p + ".D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * W[p + ".norm"]
    return y @ W[p + ".o"].T


def parallel(m: dict, W: Dict[str, torch.Tensor], p: str, h, eps: float):
    left = softmax_attention(m["left"], W, p + ".left", h, eps, "chunk")
    right = state_space(m["right"], W, p + ".right", h, eps)
    return 0.5 * (rms_unit(left, eps) * W[p + ".left.out"] + rms_unit(right, eps) * W[p + ".right.out"])


# ------------------------------------------------------------------------------------------------------------ feed-forward, model
def feed_forward(f: dict, W: Dict[str, torch.Tensor], p: str, h):
    limit = float(f["limit"])
    g = torch.clamp(h @ W[p + ".gate"].T, max=limit)
    u = torch.clamp(h @ W[p + ".up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ W[p + ".down"].T


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, dtype=torch.float64, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, if asked, the residual stream after every layer run)."""
    W = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()}
    eps = float(config["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(config.get("embedding", {}).get("scale", 1.0))
    after: List[torch.Tensor] = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', i)}"
        h = layer_norm(x, W[p + ".norm1"], eps)
        kind = layer["type"]
        if kind == "channel_delta":
            y = channel_delta(layer["mixer"], W, p + ".mix", h, eps)
        elif kind == "attention":
            y = softmax_attention(layer["mixer"], W, p + ".mix", h, eps, "window")
        elif kind == "parallel":
            y = parallel(layer["mixer"], W, p + ".mix", h, eps)
        else:
            raise ValueError(kind)
        x = x + layer_norm(y, W[p + ".norm1b"], eps)
        if layer.get("mlp"):
            y = feed_forward(layer["mlp"], W, p + ".mlp", layer_norm(x, W[p + ".norm2"], eps))
            x = x + layer_norm(y, W[p + ".norm2b"], eps)
        after.append(x)
    logits = layer_norm(x, W["final.norm"], eps) @ W["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits
