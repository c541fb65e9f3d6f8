"""A plain, slow statement of the Luvutar decoder: whole sequences, dense masks, no cache, no kernels.

One function per mechanism, written from the design's equations and sharing nothing with the
package's product path: the tests compare the engine (pages, portions, batches, kernels) with it.
Everything is computed in ``dtype`` (float64 by default) on the CPU from a dict of named tensors
and the model's ``config.json`` dict.

Notation: ``T`` tokens of one sequence at positions 0..T-1, ``W`` the model's width, ``S`` streams.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose stored weight is the distance from one."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dense_ff(h, up, down):
    return gelu_tanh(h @ up.T) @ down.T


def rotate_pairs(x, positions, base: float, dims: int):
    """Neighbouring pairs (2i, 2i+1) of the first ``dims`` entries of the last axis turn by ``position * base^(-2i/dims)``;
    the rest passes. ``x`` is [T, ..., D]."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = ang.cos().view(shape), ang.sin().view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance table for distance ``n``: one row per distance below ``rows / 2``, then rows that widen
    logarithmically up to distance ``far``; everything beyond shares the last row."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def query_temperature(positions, coef: float, every: int, dtype):
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(dtype) + 1.0)


def biased_attention(h, w: Dict[str, torch.Tensor], m: dict, k=None, v=None):
    """The mixer 'attention': grouped heads, no rotation, a query temperature that grows with the position, a learned
    bias by bucketed distance, causal softmax, one output gate per head. ``k``/``v`` given: another layer's keys and
    values are used instead of projections of its own. Returns (output, k, v)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w["q"].T).view(T, H, d)
    if k is None:
        k = (h @ w["k"].T).view(T, G, d)
        v = (h @ w["v"].T).view(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(pos, float(qt["coef"]), int(qt["every"]), h.dtype)[:, None, None]
    rel = w.get("rel")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    causal = pos[:, None] >= pos[None, :]
    if rel is not None:
        rows = rel.shape[0]
        far = float(m["bias_max"])
        bucket = torch.tensor([[distance_bucket(i - j, rows, far) if i >= j else 0 for j in range(T)] for i in range(T)])
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * float(m["scale"])
        if rel is not None:
            s = s + rel[:, head][bucket]
        s = s.masked_fill(~causal, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    gate = torch.sigmoid(h @ w["g"].T)          # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w["o"].T, k, v


def latent_attention(h, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """The mixer 'latent_attention': queries and keys/values through low-rank latents, one rotated key part shared by
    all heads, a sliding window, a sink in the softmax's denominator, an output gate per element."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = norm_plain(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, d + r)
    q_flat, q_rot = q[..., :d], q[..., d:]
    dkv = h @ w["dkv"].T
    c = norm_plain(dkv[:, :rank], w["dkv.norm"], eps)
    k_rot = dkv[:, rank:]
    rot = m.get("rot")
    if rot:
        q_rot = rotate_pairs(q_rot, pos, float(rot["base"]), int(rot["dims"]))
        k_rot = rotate_pairs(k_rot, pos, float(rot["base"]), int(rot["dims"]))
    k_flat = (c @ w["uk"].T).view(T, H, d)
    val = (c @ w["uv"].T).view(T, H, dv)
    dist = pos[:, None] - pos[None, :]
    seen = dist >= 0
    mask = m.get("mask")
    if mask:
        seen = seen & (dist < int(mask["size"]))
    sink = w.get("sink")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        s = (q_flat[:, head] @ k_flat[:, head].T + q_rot[:, head] @ k_rot.T) * float(m["scale"])
        s = s.masked_fill(~seen, float("-inf"))
        if sink is not None:
            top = torch.maximum(s.max(-1, keepdim=True).values, sink[head])
            e = torch.exp(s - top)
            p = e / (e.sum(-1, keepdim=True) + torch.exp(sink[head] - top))
        else:
            p = torch.softmax(s, dim=-1)
        out[:, head] = p @ val[:, head]
    out = out.reshape(T, H * dv) * torch.sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def hyper_step(xs, coef_in, mix, coef_out, sublayer):
    """One sublayer under hyper-connections. ``xs`` [S, T, W]: the sublayer reads a weighted sum of the streams; every new
    stream is a mix of the old ones plus its share of the sublayer's result."""
    u = torch.einsum("s,stw->tw", coef_in, xs)
    y = sublayer(u)
    return torch.einsum("sr,stw->rtw", mix, xs) + coef_out[:, None, None] * y[None]


def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layer_outputs: Optional[list] = None):
    """Logits [T, vocab] of one whole sequence. ``layer_outputs``: a list that receives the residual stream (the sum of the
    streams, if there are several) after every layer."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    S = config.get("streams")
    x = t["embed"][torch.tensor(tokens)]
    xs = x[None].repeat(S, 1, 1) if S else None
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        w = sub(t, p + "mix.")

        def mixer(h, i=i, m=m, w=w, kind=layer["type"]):
            if kind == "latent_attention":
                return latent_attention(h, w, m, eps)
            if kind == "attention":
                src = m.get("kv_from")
                if src is not None:
                    y, _, _ = biased_attention(h, w, m, *kept[src])
                    return y
                y, k, v = biased_attention(h, w, m)
                kept[i] = (k, v)
                return y
            raise ValueError(f"unknown mixer {kind}")

        steps = [(1, mixer)]
        if layer.get("mlp"):
            steps.append((2, lambda h, p=p: dense_ff(h, t[p + "mlp.up"], t[p + "mlp.down"])))
        for n, fn in steps:
            normed = lambda u, n=n, fn=fn, p=p: fn(norm_around_zero(u, t[f"{p}norm{n}"], eps))
            if S:
                xs = hyper_step(xs, t[f"{p}hc{n}.in"], t[f"{p}hc{n}.mix"], t[f"{p}hc{n}.out"], normed)
            else:
                x = x + normed(x)
        if layer_outputs is not None:
            layer_outputs.append(xs.sum(0) if S else x)
    if S:
        x = xs.sum(0)
    return norm_around_zero(x, t["final.norm"], eps) @ t["head"].T
