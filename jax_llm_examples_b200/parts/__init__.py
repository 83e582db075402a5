from .attention import PagedAttention, plan_attention_tiles
from .base import (Block, FeedForward, KVNeed, LayerCache, Mixer, Norm, Part, PositionEncoding, Rows, RowSum, Runtime, StateNeed,
                   StepContext, StepShape, Workspace, as_rows, known_parts, make_part, register_part)
from .block import PreNormBlock
from .decoder import CachePlan, DecoderModel, LayerRun
from .feedforward import DenseSwiGLU, RoutedExperts
from .linear import grouped_linear, grouped_swiglu_linear, interleave_gate_up, linear, swiglu_linear
from .norms import RMSNorm
from .positions import InterleavedRope, NoPositionWithTemperature, UnfusedEncoding, llama3_scaled_frequencies

__all__ = [
    "Block", "CachePlan", "DecoderModel", "DenseSwiGLU", "FeedForward", "InterleavedRope", "KVNeed", "LayerCache",
    "LayerRun", "Mixer", "NoPositionWithTemperature", "Norm", "PagedAttention", "Part", "PositionEncoding",
    "PreNormBlock", "RMSNorm", "RoutedExperts", "Rows", "RowSum", "Runtime", "Workspace", "as_rows", "grouped_swiglu_linear", "interleave_gate_up", "swiglu_linear", "StateNeed", "StepContext", "StepShape", "plan_attention_tiles", "UnfusedEncoding",
    "grouped_linear", "known_parts", "linear", "llama3_scaled_frequencies", "make_part", "register_part",
]
