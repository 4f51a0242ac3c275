from .base import (AddedToResidual, NormedUpdate, PendingNorm, Upcoming, DiskSource, FeedForward, KVCacheNeed, Mixer, Norm, ParamDecl, Part,
                   PositionEncoding, StateNeed, StreamCopy, StreamUpdate, PendingSum)
from .registry import (PartSpec, build_block, build_part, register_block, register_feed_forward, register_mixer,
                       register_norm, register_position_encoding, registered)
from .norm import GroupRMSNorm, LayerNorm, RMSNorm
from .rope import FrequencyRotary, InterleavedRotary, RotaryEmbedding
from .linear import Linear
from .attention import GQAAttention
from .mlp import ActivationMLP, SwiGLU
from .conv import CausalShortConv
from .polynorm_mlp import PolyNormMLP
from .latent_attention import LatentAttention
from .mlstm import MLSTM
from .gla import GatedLinearAttention
from .masked_attention import MaskedSinkAttention
from .sink_attention import SinkAttention
from .pooled_attention import PooledWindowAttention
from .glu_mlp import ClampedGLU, RoutedExperts
from .token_side import TokenSideInput
from .embed import LMHead, TokenEmbedding
from .block import Block, BlockSpec, HyperConnectionBlock, ParallelBlock, PostNormBlock, PreNormBlock, SandwichNormBlock, SharedRef
from .model import DecoderModel, LayerCall, ModelPlan, PassVectors
