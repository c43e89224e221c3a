"""Layer classes of the decode path (mirror of pygpukit/llm/layers/__init__.py)."""
from .attention import Attention
from .block import ParallelBlock, PostNormBlock, PreNormBlock, SandwichBlock, TransformerBlock
from .dense_rows import GatedDenseRows, PolyNormRows, SquaredReluRows
from .gated_recurrent import DeltaRuleMixer, GatedLinearMixer
from .linear_attention import LinearAttentionMixer, ParallelMixer
from .latent_attention import LatentAttentionMixer
from .token_side import TokenSideInput
from .linear import Linear, LinearBF16, LinearFP8, LinearNVF4, LinearRows, interleave_gate_up
from .mlp import MLP
from .moe import MoELayer
from .moe_rows import BiasedRouterMoE, GroupedRouterMoE
from .norm import CausalConvRows, Norm, RowNorm
from .paged_attention import PagedAttentionMixer
from .rope import apply_rotary_pos_emb_numpy, precompute_freqs_cis

__all__ = ["Attention", "TransformerBlock", "Linear", "LinearBF16", "LinearFP8", "LinearNVF4", "MLP", "MoELayer",
           "Norm", "RowNorm", "CausalConvRows", "PostNormBlock", "ParallelBlock", "PreNormBlock", "SandwichBlock", "GatedDenseRows", "SquaredReluRows", "PolyNormRows",
           "GatedLinearMixer", "DeltaRuleMixer", "BiasedRouterMoE",
           "LinearAttentionMixer", "ParallelMixer", "LatentAttentionMixer", "TokenSideInput", "LinearRows", "interleave_gate_up", "GroupedRouterMoE", "PagedAttentionMixer", "apply_rotary_pos_emb_numpy", "precompute_freqs_cis"]
