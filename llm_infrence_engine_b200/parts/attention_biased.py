"""Grouped-query attention whose only knowledge of position is a bias by distance and a query temperature."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..cache.spec import PagedKVSpec
from .base import ANY, INIT_SMALL, MATRIX, VECTOR, Mixer, ParamSpec, Source


def distance_rows(rows: int, far: float) -> list:
    """Row of a distance-bias table with ``rows`` rows for every distance ``0 .. ceil(far) - 1``; any distance from ``far``
    on uses the last row. Distances below ``rows / 2`` have a row each; from there the rows widen logarithmically:
    ``rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2)) * (rows - rows/2))``."""
    half = rows // 2
    if not far > half >= 1:
        raise ValueError(f"a distance table of {rows} rows needs a largest distance beyond {half}, got {far}")
    out = []
    for n in range(int(math.ceil(far))):
        out.append(n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


class BiasedAttention(Mixer):
    """``o(gate * softmax(temp(p) * scale * q k^T + rel[row(i - j), head]) v)`` over a paged cache, causal.

    * no rotation; the query at position ``p`` is scaled by ``1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)``;
    * ``rel [rows, heads]`` is added to the scaled scores, its row chosen by the distance (``distance_rows``); the number
      of rows is the checkpoint's;
    * keys and values may differ in size (``head_dim``, ``v_head_dim``);
    * one output gate per head: ``sigmoid(g h)``, read from the same input as the projections;
    * ``own_kv = False``: the layer has no key/value projections and reads the cache entry of another layer
      (the running order binds it with ``write=False``).

    All projections of the input are one matrix (rows padded to a multiple of 8 so that every row of the product starts on
    a 16-byte boundary); the new keys and values go to the pages by one kernel; the attention kernel applies temperature,
    bias and gate itself, scores and softmax in 32-bit.
    """

    graph_safe = True

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, scale: float, prefix: str,
                 bias_far: Optional[float] = None, temp_coef: float = 0.0, temp_every: int = 0, own_kv: bool = True,
                 window: Optional[int] = None, random_rel_rows: int = 16):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
        self.hidden, self.num_heads, self.num_kv_heads = hidden, num_heads, num_kv_heads
        self.head_dim, self.v_head_dim, self.scale, self.prefix = head_dim, v_head_dim, float(scale), prefix
        self.bias_far, self.temp_coef, self.temp_every = bias_far, float(temp_coef), int(temp_every)
        self.own_kv, self.window, self.random_rel_rows = own_kv, window, random_rel_rows
        self.w_in: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.rel: Optional[torch.Tensor] = None
        self.rel_rows: Optional[torch.Tensor] = None   # int32 [ceil(bias_far)]: distance -> row of ``rel``
        q, k, v = num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * v_head_dim
        self.k_col = q
        self.v_col = q + k
        self.g_col = q + (k + v if own_kv else 0)

    def params(self) -> Dict[str, ParamSpec]:
        p, h = self.prefix, self.hidden
        rows = [("q", self.num_heads * self.head_dim)]
        if self.own_kv:
            rows += [("k", self.num_kv_heads * self.head_dim), ("v", self.num_kv_heads * self.v_head_dim)]
        rows.append(("g", self.num_heads))
        out = {"w_in": ParamSpec(tuple(Source(f"{p}.{n}", (r, h)) for n, r in rows), MATRIX),
               "w_o": ParamSpec((Source(f"{p}.o", (h, self.num_heads * self.v_head_dim)),), MATRIX)}
        if self.bias_far is not None:
            out["rel"] = ParamSpec((Source(f"{p}.rel", (ANY, self.num_heads), INIT_SMALL, free=self.random_rel_rows),), VECTOR)
        return out

    def bind(self, tensors) -> None:
        w = tensors["w_in"]
        pad = -w.shape[0] % 8
        self.w_in = torch.cat([w, w.new_zeros((pad, w.shape[1]))]).contiguous() if pad else w
        self.w_o = tensors["w_o"]
        if "rel" in tensors:
            self.rel = tensors["rel"].contiguous()
            self.rel_rows = torch.tensor(distance_rows(self.rel.shape[0], self.bias_far), dtype=torch.int32, device=self.rel.device)

    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window, self.v_head_dim)

    def forward(self, ctx, h, cache, residual):
        K = ctx.K
        z = K.linear(h, self.w_in, out_dtype=ctx.dtype)
        slots = ctx.slot_mapping[cache.group]
        if cache.write:
            K.kv_store(z, self.k_col, self.v_col, slots, cache.k, cache.v, self.num_kv_heads, self.head_dim, self.v_head_dim, ctx.page_size)
        attn = K.attention_ext(z, 0, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim, cache.k, cache.v,
                               ctx.block_tables[cache.group], ctx.token_seq, ctx.positions, ctx.page_size, self.scale,
                               self.window or 0, ctx.max_context, temp=(self.temp_coef, self.temp_every),
                               rel=self.rel, rel_rows=self.rel_rows, gate=z, gate_col=self.g_col, gate_per_head=True, batch=ctx)
        K.linear(attn, self.w_o, add_to=residual)
