from . import attention, block, delta_rule, feedforward, gated_delta, latent, matrix_memory, model, norms, positions, recurrence, routed, talking  # noqa: F401  (register the built-in parts)
from .attention import CacheView, PagedAttention
from .block import GatedPreNormBlock, OutputNormBlock, PreNormBlock, SandwichBlock
from .delta_rule import GeneralDeltaMixer
from .feedforward import GatedMLP, PolyNormMLP
from .gated_delta import GatedDeltaMixer
from .latent import DifferentialAttention, LatentAttention
from .linear import Linear
from .matrix_memory import MatrixMemory
from .model import BigramDecoderModel, DecoderModel, PassOffsetDecoderModel, ReinjectDecoderModel
from .norms import LayerNorm, RMSNorm
from .positions import BucketedBias, NoPosition, PartialRotation, Rotary, RotaryPairs, distance_bucket, rotary_inv_freq, rotary_tables
from .recurrence import GatedLinearRecurrence, MinGRU, ParallelMixer
from .registry import (
    BLOCKS,
    FEEDFORWARDS,
    MIXERS,
    MODELS,
    NORMS,
    POSITIONS,
    expected_tensors,
    register_block,
    register_feedforward,
    register_mixer,
    register_model,
    register_norm,
    register_position,
)
from .routed import RoutedExperts
from .talking import TalkingAttention
from .runtime import Runtime, Staging, Workspace
