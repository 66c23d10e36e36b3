from .spec import PartSpec, BlockSpec, ScheduleEntry, ModelSpec
from .base import (Part, Norm, PositionEncoding, Mixer, FeedForward, Connection, CacheNeed, StateNeed, InputFilter,
                   ResultGate, TokenInput)
from .registry import register_part, unregister_part, known_parts, build_part, build_block
from .norm import RMSNorm, LayerNorm
from .position import RotaryEncoding, NoPositionEncoding
from .attention import Attention
from .feed_forward import GatedDense, Dense, RoutedExperts
from .block import PreNormBlock, StreamBlock, GatedPreNormBlock, PostNormBlock
from .recurrent import GatedLinearRecurrence, MatrixMemory
from .delta import GatedDeltaRule
from .gla import GatedLinearAttention
from .latent import LatentAttention
from .retention import Retention
from .sublayer import CausalTapsFilter, SigmoidGate, GatedTokenEmbedding
from .parallel import ParallelMixers
from .connection import ResidualConnection, HyperConnection

__all__ = ["PartSpec", "BlockSpec", "ScheduleEntry", "ModelSpec", "Part", "Norm", "PositionEncoding",
           "Mixer", "FeedForward", "CacheNeed", "StateNeed", "register_part", "unregister_part",
           "known_parts", "build_part", "build_block", "RMSNorm", "RotaryEncoding", "NoPositionEncoding", "Attention",
           "GatedDense", "PreNormBlock", "StreamBlock", "Connection", "GatedLinearRecurrence", "MatrixMemory",
           "ParallelMixers", "ResidualConnection", "HyperConnection", "LayerNorm", "Dense", "RoutedExperts",
           "GatedDeltaRule", "GatedLinearAttention", "LatentAttention", "CausalTapsFilter", "SigmoidGate",
           "InputFilter", "ResultGate", "GatedPreNormBlock", "PostNormBlock", "Retention",
           "GatedTokenEmbedding", "TokenInput"]
