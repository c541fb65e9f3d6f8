"""Zepalorn: a decoder whose layers are listed one by one in config.json.

Every layer norms its sublayers on both sides (layer norms with a weight and no bias): ``x += norm1b(mixer(norm1(x)))``, then
``x += norm2b(ff(norm2(x)))`` where the layer has a feed-forward (a clamped gated unit). The mixer is one of

* ``channel_delta``: the gated delta rule with a decay per head and key channel (a recurrent state of fixed size);
* ``attention``: grouped softmax attention, partly rotated heads (pairs half a rotation apart), a sliding window that keeps the
  request's first tokens;
* ``parallel``: chunked softmax attention (short convolutions, query/key norm, neighbouring pairs rotated, soft-capped scores)
  beside a state-space mixer, each result normed by its root mean square, then their mean.

A layer with ``weights_of: j`` has no tensors: it is layer j's part run once more, with a cache entry of its own, which the
running order expresses directly. The embedding is scaled; the output head is the embedding table itself, unscaled.
Tensor names: ``embed``, ``l<i>.norm1/norm1b/norm2/norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.gate/up/down``, ``final.norm``.
"""
from __future__ import annotations

from ..config.model_config import MaskedAttentionConfig, ZepalornConfig
from ..parts import OutputHead, TokenEmbedding
from ..parts.attention_masked import MaskedAttention
from ..parts.block import SandwichBlock
from ..parts.mlp import ClampedGLU
from ..parts.norm import LayerNorm
from ..parts.recurrent import GatedDeltaMixer, ParallelMixer, StateSpaceMixer
from ..parts.rotary import RampedRotary
from .registry import register_architecture
from .spec import LayerCall, ModelSpec


def build_zepalorn(cfg: ZepalornConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.eps
    rotary = {}

    def attention(m: MaskedAttentionConfig, prefix: str) -> MaskedAttention:
        position = None
        if m.rot is not None:
            r = m.rot
            position = rotary.setdefault(r, RampedRotary(r.dims, r.base, r.factor, r.original, r.fast, r.slow))
        return MaskedAttention(W, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, prefix, position=position, interleaved=m.interleaved,
                               window=None if m.chunked else m.mask_size, keep_first=m.keep_first, chunk=m.mask_size if m.chunked else None,
                               softcap=m.softcap, conv_taps=m.conv, qk_norm=m.qk_norm, eps=eps)

    layers, part_of = [], {}
    for i, lc in enumerate(cfg.layers):
        if lc.weights_of is not None:      # no part of its own: the running order below names the other layer's part once more
            continue
        p, m = f"l{i}", lc.mixer
        if lc.kind == "channel_delta":
            mixer = GatedDeltaMixer(W, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, eps, f"{p}.mix")
        elif lc.kind == "attention":
            mixer = attention(m, f"{p}.mix")
        else:
            right = StateSpaceMixer(W, m.right.heads, m.right.vdim, m.right.state, m.right.groups, m.right.norm_groups, m.right.conv, eps,
                                    f"{p}.mix.right")
            mixer = ParallelMixer(W, attention(m.left, f"{p}.mix.left"), right, eps, f"{p}.mix.left.out", f"{p}.mix.right.out")
        ff = ClampedGLU(W, lc.ff, f"{p}.mlp.gate", f"{p}.mlp.up", f"{p}.mlp.down", lc.ff_limit) if lc.ff else None
        part_of[i] = len(layers)
        layers.append(SandwichBlock(LayerNorm(W, eps, f"{p}.norm1"), mixer, LayerNorm(W, eps, f"{p}.norm1b"),
                                    LayerNorm(W, eps, f"{p}.norm2") if ff else None, ff, LayerNorm(W, eps, f"{p}.norm2b") if ff else None))
    # layer i runs its own part, or the part of the layer whose weights it runs on, always with cache entry i
    schedule = [LayerCall(part_of[i if lc.weights_of is None else lc.weights_of], i) for i, lc in enumerate(cfg.layers)]
    embedding = TokenEmbedding(cfg.vocab, W, "embed", scale=cfg.embedding_scale)
    return ModelSpec(
        config=cfg,
        embedding=embedding,
        layers=layers,
        schedule=schedule,
        final_norm=LayerNorm(W, eps, "final.norm"),
        head=OutputHead(cfg.vocab, W, "head", tied_to=embedding),
    )


register_architecture("Zepalorn", ZepalornConfig, build_zepalorn)
