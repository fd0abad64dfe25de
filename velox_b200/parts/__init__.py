from .attention import PagedAttention
from .base import (Block, CacheParts, Embedding, FeedForward, FixedState, Mixer, Norm, PagedKV, PagedLatent, Part, Position, Runtime,
                   TensorSpec)
from .block import (HyperConnectionBlock, ParallelSublayersBlock, PendingStreams, PendingSum, PostNormBlock, PreNormBlock,
                    SandwichNormBlock)
from .differential_attention import DifferentialAttention
from .embedding import OutputHead, PairHashEmbedding, TokenEmbedding
from .linear import Linear, matmul
from .latent_attention import LatentAttention
from .linear_attention import DecayedLinearAttention, GatedLinearAttention
from .mlp import CappedGatedMLP, DenseMLP, GatedMLP
from .moe import RoutedExperts
from .norm import LayerNorm, RMSNorm
from .parallel import ParallelMixer
from .plan import LayerSpec, ModelPlan, PartSpec
from .position import NoPosition, RotaryPosition
from .registry import (build_part, part_class, register_block, register_feed_forward, register_mixer,
                       register_norm, register_part, register_position, unregister_part)

register_part("mixer", "paged_attention", PagedAttention)
register_part("mixer", "decayed_linear_attention", DecayedLinearAttention)
register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "latent_attention", LatentAttention)
register_part("mixer", "parallel", ParallelMixer)
register_part("mixer", "differential_attention", DifferentialAttention)
register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "dense_mlp", DenseMLP)
register_part("feed_forward", "capped_gated_mlp", CappedGatedMLP)
register_part("feed_forward", "routed_experts", RoutedExperts)
register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "layer_norm", LayerNorm)
register_part("position", "rotary", RotaryPosition)
register_part("position", "none", NoPosition)
register_part("block", "pre_norm", PreNormBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
register_part("block", "post_norm", PostNormBlock)
register_part("block", "parallel_sublayers", ParallelSublayersBlock)
register_part("block", "hyper_connections", HyperConnectionBlock)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "pair_hash_embedding", PairHashEmbedding)
register_part("head", "linear_head", OutputHead)
