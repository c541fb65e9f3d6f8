"""Hyper-connections: several residual streams instead of one, mixed by learned coefficients around every sublayer.

With ``S`` streams ``x_1 .. x_S`` (all equal to the embedding at the start), a sublayer ``f`` with coefficients
``a [S]`` (in), ``M [S, S]`` (mix, indexed [from, to]) and ``b [S]`` (out) does

    u = sum_s a_s x_s;   y = f(norm(u));   x_t <- sum_s M[s, t] x_s + b_t y   (all t at once, from the old streams)

and the model's output reads the sum of the streams. The streams are one 32-bit tensor ``[N, S, hidden]`` (a token's
streams side by side); the weighted sum and the norm are one kernel, and a sublayer's update is put off until that kernel
of the NEXT sublayer, which then updates, sums and normalises in one pass over the streams.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .base import INIT_EYE, INIT_ONES, INIT_SHARE, VECTOR, FeedForward, Mixer, Norm, ParamSpec, Part, Source


class HyperConnection(Part):
    """The three coefficient tensors of one sublayer: ``<prefix>.in [S]``, ``<prefix>.mix [S, S]``, ``<prefix>.out [S]``."""

    graph_safe = True

    def __init__(self, streams: int, prefix: str):
        self.streams, self.prefix = streams, prefix
        self.coef_in: Optional[torch.Tensor] = None
        self.mix: Optional[torch.Tensor] = None
        self.coef_out: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        s, p = self.streams, self.prefix
        return {"coef_in": ParamSpec((Source(f"{p}.in", (s,), INIT_SHARE),), VECTOR),
                "mix": ParamSpec((Source(f"{p}.mix", (s, s), INIT_EYE),), VECTOR),
                "coef_out": ParamSpec((Source(f"{p}.out", (s,), INIT_ONES),), VECTOR)}


class HyperConnectionBlock(Part):
    """A pre-norm layer over several residual streams: mixer, then (if the layer has one) feed-forward, each under its
    own hyper-connection. The sublayers are ordinary parts: they add their result into a zeroed ``[N, hidden]`` tensor."""

    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, hc1: HyperConnection, norm2: Optional[Norm] = None,
                 ff: Optional[FeedForward] = None, hc2: Optional[HyperConnection] = None):
        if (ff is None) != (norm2 is None) or (ff is None) != (hc2 is None):
            raise ValueError("a feed-forward comes with its norm and its hyper-connection, or none of the three")
        self.norm1, self.mixer, self.hc1, self.norm2, self.ff, self.hc2 = norm1, mixer, hc1, norm2, ff, hc2

    def children(self) -> Sequence[Part]:
        return tuple(p for p in (self.norm1, self.mixer, self.hc1, self.norm2, self.ff, self.hc2) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, streams: torch.Tensor, cache) -> None:
        K = ctx.K
        h = self.norm1.norm_streams(ctx, streams, self.hc1.coef_in)
        y = K.zeros_like_rows(streams)
        self.mixer.forward(ctx, h, cache, y)
        K.streams_update(streams, y, self.hc1.mix, self.hc1.coef_out)
        if self.ff is not None:
            h = self.norm2.norm_streams(ctx, streams, self.hc2.coef_in)
            y = K.zeros_like_rows(streams)
            self.ff.forward(ctx, h, y)
            K.streams_update(streams, y, self.hc2.mix, self.hc2.coef_out)


class ResidualStreams(Part):
    """The model's two ends of the streams: ``S`` copies of the embedding going in, the norm of their sum coming out."""

    graph_safe = True

    def __init__(self, streams: int):
        self.streams = streams
        self._ones = {}

    def expand(self, ctx, x: torch.Tensor) -> torch.Tensor:
        return ctx.K.streams_expand(x, self.streams)

    def norm_rows(self, ctx, norm: Norm, streams: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        dev = str(streams.device)
        if dev not in self._ones:
            self._ones[dev] = torch.ones(self.streams, dtype=torch.float32, device=streams.device)
        return norm.norm_streams(ctx, streams, self._ones[dev], rows)
