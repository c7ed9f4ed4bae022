from .base import (Embedding, FeedForward, Head, Mixer, Norm, PagedCacheSpec, Part, PositionEncoding, StateSpec, TokenInput,
                   build_embedding, build_feed_forward, build_head, build_mixer, build_norm, build_position, build_reentry, build_token_input,
                   part_factory, register_part, register_step_layout, unregister_part)
from .linear import linear, prepare_weight
from .norm import DynamicTanh, LayerNormStream, RMSNorm, StreamRMSNorm
from .rope import RotaryEncoding
from .attention import Attention
from .feed_forward import ExpertMixture, SwiGLU
from .sink_attention import SinkAttention
from .gated_delta import GatedDeltaRule
from .general_delta import GeneralDeltaRule
from .latent_attention import LatentAttention
from .selective_scan import SelectiveScan
from .token_input import GatedTokenInput
from .branches import BranchMixer
from .reentry import ConcatReentry
from .block import ParallelBlock, PostNormStreamBlock, PreNormBlock, SandwichStreamBlock, StreamPreNormBlock, build_block
from .embedding import PairHashEmbedding, TableEmbedding
from .head import LinearHead

__all__ = [
    "Embedding", "Head", "build_embedding", "build_head", "TableEmbedding", "LinearHead", "FeedForward", "Mixer", "Norm", "PagedCacheSpec", "Part", "PositionEncoding", "StateSpec",
    "build_feed_forward", "build_mixer", "build_norm", "build_position", "part_factory",
    "register_part", "register_step_layout", "unregister_part", "linear", "RMSNorm", "RotaryEncoding", "Attention",
    "SwiGLU", "PreNormBlock", "build_block", "build_reentry", "DynamicTanh", "ExpertMixture", "SinkAttention",
    "GatedDeltaRule", "BranchMixer", "ConcatReentry", "ParallelBlock", "StreamRMSNorm", "GeneralDeltaRule",
    "GatedTokenInput", "StreamPreNormBlock", "LayerNormStream", "LatentAttention", "SelectiveScan", "SandwichStreamBlock", "PostNormStreamBlock", "PairHashEmbedding", "TokenInput", "build_token_input",
]
