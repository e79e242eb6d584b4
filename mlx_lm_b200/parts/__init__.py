from .base import (INT_TABLE, MATRIX, VECTOR, Block, FeedForward, Init, Mixer, Norm, PagedKVSpec, ParamSpec, Part,
                   PositionEncoding, StateSpec, make_part, register_part, registered_parts)
from .block import ParallelBlock, PreNormBlock, SandwichBlock, StreamBlock
from .feed_forward import MLP, ExpertsMLP, GatedMLP, LearnedActMLP
from .linear import FusedLinear, Linear
from .mixers import (Attention, DifferentialAttention, LatentAttention, ParallelMixer, SinkAttention,
                     TalkingHeadsAttention)
from .model import LoopInput, Model, ModelDescription, OutputHead, Reentry, RunEntry, TokenEmbedding
from .norms import DynamicTanh, LayerNorm, RMSNorm
from .recurrent import GatedDeltaMixer, Mamba2Mixer, WKVMixer
from .side import TokenSideInput
from .positions import LearnedAbsolute, NoPosition, Sinusoidal, rotation_frequencies

__all__ = ["INT_TABLE", "MATRIX", "VECTOR", "Block", "FeedForward", "Init", "Mixer", "Norm", "PagedKVSpec",
           "ParamSpec", "Part", "PositionEncoding", "StateSpec", "make_part", "register_part", "registered_parts",
           "PreNormBlock", "MLP", "Linear", "Attention", "Model", "ModelDescription", "OutputHead", "RunEntry",
           "TokenEmbedding", "LayerNorm", "LearnedAbsolute", "NoPosition", "StreamBlock", "GatedMLP", "FusedLinear",
           "ParallelMixer", "SinkAttention", "LoopInput", "Reentry", "RMSNorm", "GatedDeltaMixer", "Mamba2Mixer",
           "TokenSideInput", "LearnedActMLP", "LatentAttention", "TalkingHeadsAttention", "WKVMixer", "DynamicTanh",
           "ExpertsMLP", "SandwichBlock", "Sinusoidal", "ParallelBlock", "DifferentialAttention", "rotation_frequencies"]
