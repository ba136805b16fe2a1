from .attention import CausalSelfAttention
from .base import Block, FeedForward, Mixer, Norm, Part, PositionEncoding
from .block import PreNormBlock
from .embedding import LinearReadout, TiedReadout, TokenEmbedding
from .feed_forward import DenseFeedForward, GatedFeedForward
from .latent_attention import LatentAttention
from .lightning import LightningAttention
from .norm import LayerNorm, RmsNorm
from .position import InterleavedRotary, LearnedPositions, NoPositions

__all__ = ["CausalSelfAttention", "Block", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "PreNormBlock",
           "LinearReadout", "TiedReadout", "TokenEmbedding", "DenseFeedForward", "GatedFeedForward", "LatentAttention",
           "LightningAttention", "LayerNorm", "RmsNorm", "InterleavedRotary", "LearnedPositions", "NoPositions"]
