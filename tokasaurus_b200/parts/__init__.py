from tokasaurus_b200.parts.base import (  # noqa: F401
    FeedForward,
    Mixer,
    Norm,
    PagedCacheNeed,
    Part,
    PositionEncoding,
    QkvStage,
    ResidualStream,
    StateNeed,
    WeightSpec,
)
from tokasaurus_b200.parts.norm import RMSNorm  # noqa: F401
from tokasaurus_b200.parts.rope import NoPositionEncoding, RotaryEncoding  # noqa: F401
from tokasaurus_b200.parts.attention import PagedAttention  # noqa: F401
from tokasaurus_b200.parts.mlp import GatedMLP  # noqa: F401
from tokasaurus_b200.parts.block import PreNormBlock  # noqa: F401
from tokasaurus_b200.parts.embedding import OutputHead, TokenEmbedding  # noqa: F401
from tokasaurus_b200.parts.model import DecoderModel, LayerCall  # noqa: F401
