from .attention import PagedAttention
from .attention_biased import BiasedAttention
from .attention_latent import LatentAttention
from .base import (ANY, INIT_EYE, INIT_NORM, INIT_NORMAL, INIT_ONES, INIT_SHARE, INIT_SMALL, MATRIX, TABLE, VECTOR, FeedForward, Mixer, Norm, ParamSpec, Part,
                   PositionEncoding, Source, walk)
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .hyper import HyperConnection, HyperConnectionBlock, ResidualStreams
from .mlp import DenseMLP, GatedMLP
from .norm import RMSNorm
from .rotary import RotaryEncoding

__all__ = ["PagedAttention", "BiasedAttention", "LatentAttention", "HyperConnection", "HyperConnectionBlock", "ResidualStreams", "DenseMLP", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part", "PositionEncoding", "Source", "walk",
           "PreNormBlock", "OutputHead", "TokenEmbedding", "GatedMLP", "RMSNorm", "RotaryEncoding",
           "ANY", "INIT_EYE", "INIT_NORM", "INIT_NORMAL", "INIT_ONES", "INIT_SHARE", "INIT_SMALL", "MATRIX", "TABLE", "VECTOR"]
