"""Luvutar: a decoder whose layers are listed one by one in config.json.

Every layer is a pre-norm block (RMS norms with weights stored around zero) of one of two mixers, grouped attention
with a distance bias and a query temperature or latent attention with a window and a sink, and, where the layer has
one, a dense GELU feed-forward. With ``streams`` the residual is several streams under hyper-connections. A layer may
read the keys and values of an earlier layer instead of making its own. Tensor names: ``embed``, ``l<i>.norm1/2``,
``l<i>.mix.*``, ``l<i>.mlp.up/down``, ``l<i>.hc1/2.in/mix/out``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.model_config import LuvutarConfig
from ..parts import OutputHead, PreNormBlock, RMSNorm, RotaryEncoding, TokenEmbedding
from ..parts.attention_biased import BiasedAttention
from ..parts.attention_latent import LatentAttention
from ..parts.hyper import HyperConnection, HyperConnectionBlock, ResidualStreams
from ..parts.mlp import DenseMLP
from .registry import register_architecture
from .spec import LayerCall, ModelSpec


def build_luvutar(cfg: LuvutarConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.eps
    rotary = {}
    layers, schedule, entry_of = [], [], {}
    for i, lc in enumerate(cfg.layers):
        p, m = f"l{i}", lc.mixer
        if lc.kind == "attention":
            mixer = BiasedAttention(W, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, f"{p}.mix", bias_far=m.bias_max,
                                    temp_coef=m.temp_coef, temp_every=m.temp_every, own_kv=m.kv_from is None)
        else:
            position = None
            if m.rot_dims:
                position = rotary.setdefault((m.rot_dims, m.rot_base), RotaryEncoding(m.rot_dims, m.rot_base))
            mixer = LatentAttention(W, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, eps, position, f"{p}.mix",
                                    window=m.window, sink=m.sink)
        src = getattr(m, "kv_from", None)
        if src is None:
            entry_of[i] = len(entry_of)
            schedule.append(LayerCall(i, entry_of[i]))
        else:
            schedule.append(LayerCall(i, entry_of[src], write=False))
        norm1 = RMSNorm(W, eps, f"{p}.norm1", offset=1.0)
        norm2 = RMSNorm(W, eps, f"{p}.norm2", offset=1.0) if lc.ff else None
        ff = DenseMLP(W, lc.ff, f"{p}.mlp.up", f"{p}.mlp.down") if lc.ff else None
        if cfg.streams is None:
            layers.append(PreNormBlock(norm1, mixer, norm2, ff))
        else:
            layers.append(HyperConnectionBlock(norm1, mixer, HyperConnection(cfg.streams, f"{p}.hc1"), norm2, ff,
                                               HyperConnection(cfg.streams, f"{p}.hc2") if lc.ff else None))
    return ModelSpec(
        config=cfg,
        embedding=TokenEmbedding(cfg.vocab, W, "embed"),
        layers=layers,
        schedule=schedule,
        final_norm=RMSNorm(W, eps, "final.norm", offset=1.0),
        head=OutputHead(cfg.vocab, W, "head"),
        streams=ResidualStreams(cfg.streams) if cfg.streams is not None else None,
    )


register_architecture("Luvutar", LuvutarConfig, build_luvutar)
