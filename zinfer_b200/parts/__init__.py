"""Parts of a decoder layer: mixers, feed-forwards, norms, position encodings, blocks."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward, KVRequest, Mixer,
                   Norm, Part, PositionEncoding, Registry, RotaryParams, StateRequest, WeightSpec, walk_parts)
from .attention import GqaAttention
from .block import PreNormBlock, SublayerNormBlock
from .depth import DepthAverage
from .embedding import LMHead, TokenEmbedding
from .feedforward import ActMlp, SwiGLU
from .linear import linear
from .moe import TableMoE
from .norm import RMSNorm
from .rope import RotaryEncoding
from .seqconv import InputConv
from .shortconv import ShortConv
