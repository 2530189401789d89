from .base import (BuildContext, ParamSpec, Part, PartSpec, ProductChoice, build_part,
                   known_parts, register_part, unregister_part)
from .block import Block, ParallelBlock, PostNormBlock, PreNormBlock, SandwichBlock
from .feedforward import FeedForward, GatedMLP, ReluSquaredMLP, RoutedExperts, SwiGLU
from .io import Embedding, Head, LinearHead, TokenEmbedding, TokenPositionalEmbedding
from .linear import Linear
from .mixer import GQAAttention, LatentAttention, Mixer, SideBySide
from .recurrent import ForgetGateAttention, GatedDelta, GatedLinearRecurrence, Retention
from .norm import Averaged, Contribution, LayerNorm, Norm, RMSNorm, residual_add, stream_add
from .plan import LayerPlan, ModelPlan, ScheduleEntry
from .position import NoPosition, PositionEncoding, RotaryHalfSplit, RotaryTable

__all__ = ["BuildContext", "ParamSpec", "Part", "PartSpec", "ProductChoice", "build_part", "known_parts",
           "register_part", "unregister_part", "Block", "PostNormBlock", "PreNormBlock", "SandwichBlock", "FeedForward", "ReluSquaredMLP", "SwiGLU", "GatedMLP", "RoutedExperts", "GatedDelta", "TokenPositionalEmbedding", "stream_add",
           "Contribution", "LayerNorm",
           "Embedding", "Head", "LinearHead", "TokenEmbedding", "Linear", "GQAAttention", "Mixer",
           "Norm", "RMSNorm", "residual_add", "LayerPlan", "ModelPlan", "ScheduleEntry",
           "NoPosition", "PositionEncoding", "RotaryHalfSplit", "RotaryTable"]
