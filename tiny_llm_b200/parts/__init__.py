from .registry import (build_block, build_part, register_block, register_part, registered_blocks,
                       registered_parts)
from .norm import DynamicTanh, RMSNorm
from .position import NoPosition, Rotary
from .attention import GQAttention
from .diff_attention import DiffAttention, scaled_pair_frequencies
from .recurrent import GatedDeltaRule, GatedLinearAttention, LinearAttention, Mamba2, MinGRU, Retention
from .window_attention import PooledWindowAttention, half_frequencies
from .side_by_side import SideBySide
from .sink_attention import LatentAttention, SinkAttention, pair_frequencies, stretched_frequencies
from .experts import RoutedExperts
from .hooks import BigramEmbedding, LearnedPositions
from .feed_forward import DenseMLP, SwiGLU, interleave_gate_up
from .model import Block, BranchNormBlock, DecoderModel, SandwichBlock

__all__ = ["build_part", "register_part", "registered_parts", "build_block", "register_block", "registered_blocks", "RMSNorm", "Rotary", "NoPosition",
           "GQAttention", "DiffAttention", "scaled_pair_frequencies", "MinGRU", "LinearAttention", "Retention", "GatedLinearAttention", "GatedDeltaRule", "SinkAttention", "LatentAttention", "pair_frequencies", "SandwichBlock", "PooledWindowAttention", "half_frequencies", "SideBySide", "RoutedExperts", "LearnedPositions", "DynamicTanh", "SwiGLU", "interleave_gate_up", "Block", "DecoderModel", "Mamba2", "stretched_frequencies", "BigramEmbedding", "DenseMLP", "BranchNormBlock"]
