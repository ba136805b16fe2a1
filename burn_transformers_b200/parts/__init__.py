from .attention import CausalSelfAttention
from .base import Block, FeedForward, Mixer, Norm, Part, PositionEncoding
from .block import ParallelBlock, PreNormBlock
from .embedding import LinearReadout, StreamVectors, TiedReadout, TokenEmbedding
from .feed_forward import DenseFeedForward, GatedFeedForward
from .latent_attention import LatentAttention
from .lightning import LightningAttention
from .matrix_memory import MatrixMemory
from .norm import LayerNorm, RmsNorm
from .routed import RoutedFeedForward
from .side_by_side import SideBySideMixers
from .position import InterleavedRotary, LearnedPositions, NoPositions

__all__ = ["CausalSelfAttention", "Block", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "PreNormBlock",
           "LinearReadout", "StreamVectors", "TiedReadout", "TokenEmbedding", "DenseFeedForward", "GatedFeedForward", "LatentAttention",
           "LightningAttention", "MatrixMemory", "ParallelBlock", "RoutedFeedForward", "SideBySideMixers",
           "LayerNorm", "RmsNorm", "InterleavedRotary", "LearnedPositions", "NoPositions"]
