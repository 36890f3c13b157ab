from .base import (INDEX, MATRIX, TABLE, VECTOR, Block, DeferredNorm, FeedForward, KVRequest, Mixer, Norm,
                   ParamSpec, Part, PartSpec, Position, Side, StateRequest, bind_params, build_part,
                   collect_param_specs, register_part, registered_parts)
from .linear import Linear
from .norm import LayerNorm, RMSNorm
from .position import LearnedAbsolute, NoPosition
from .embedding import HashedPairEmbedding, LMHead, TokenEmbedding
from .attention import CausalSelfAttention
from .latent_attention import LatentAttention
from .feed_forward import DenseMLP, GatedMLP
from .routed_experts import RoutedExperts
from .block import ParallelBlock, PreNormBlock, SandwichBlock
from .pooled_attention import PooledWindowAttention
from .delta_rule import DeltaRule
from .token_side import GatedTokenInput
from .capped_attention import CappedAttention
from .masked_attention import MaskedAttention
from .selective_scan import SelectiveScan
from .linear_attention import DecayedLinearAttention
from .mixer_pair import NormedPair
from .stream_input import EmbeddingRemix
