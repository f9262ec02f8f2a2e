"""The parts a layer is put together from. Importing this package registers them."""
from .base import FeedForward, KVNeed, Mixer, Norm, Part, StateNeed, TensorSpec
from .norm import RMSNorm
from .layernorm import LayerNorm
from .rope import RotaryTable, ScaledRotaryTable
from .attention import AttentionMixer
from .short_conv import ShortConvMixer
from .swiglu import SwiGLU
from .latent_attention import LatentAttentionMixer
from .mamba2 import Mamba2Mixer
from .gated_units import ClampedGLU, RoutedExperts, SquaredRelu
from .mlstm import MLstmMixer
from .lightning import LightningMixer
from .gated_delta import GatedDeltaMixer
from .parallel import ParallelMixer
from .embedding import LearnedPositionEmbedding, PairHashEmbedding
from .block import Block, BranchNormBlock, GatedPreNormBlock, ResidualStream

__all__ = ["FeedForward", "KVNeed", "Mixer", "Norm", "RMSNorm", "Part", "StateNeed", "TensorSpec", "RotaryTable",
           "AttentionMixer", "ShortConvMixer", "SwiGLU", "Block", "ResidualStream", "LayerNorm", "ScaledRotaryTable",
           "LatentAttentionMixer", "Mamba2Mixer", "ClampedGLU", "RoutedExperts", "SquaredRelu", "MLstmMixer",
           "PairHashEmbedding", "BranchNormBlock", "GatedDeltaMixer", "ParallelMixer", "LearnedPositionEmbedding",
           "GatedPreNormBlock", "LightningMixer"]
