"""Parts of a decoder layer: mixers, feed-forwards, norms, position encodings, blocks."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward, KVRequest, Mixer,
                   Norm, Part, PositionEncoding, Registry, RotaryParams, StateRequest, WeightSpec, walk_parts)
from .attention import GqaAttention
from .block import ParallelBlock, PreNormBlock, SublayerNormBlock
from .depth import DepthAverage
from .embedding import LMHead, TokenEmbedding
from .feedforward import ActMlp, ClampedGLU, SwiGLU
from .hgrn2 import Hgrn2
from .latent import LatentAttention
from .linear import linear
from .loop import PassInput
from .moe import RoutedMoE, TableMoE
from .norm import LayerNorm, RMSNorm
from .pair import MixerPair
from .retention import Retention
from .rope import RotaryEncoding
from .seqconv import InputConv
from .shift import TokenShift
from .shortconv import ShortConv
