from .base import (INT_TABLE, MATRIX, VECTOR, Block, FeedForward, Init, Mixer, Norm, PagedKVSpec, ParamSpec, Part,
                   PositionEncoding, StateSpec, make_part, register_part, registered_parts)
from .block import PreNormBlock
from .feed_forward import MLP
from .linear import Linear
from .mixers import Attention
from .model import Model, ModelDescription, OutputHead, RunEntry, TokenEmbedding
from .norms import LayerNorm
from .positions import LearnedAbsolute, NoPosition

__all__ = ["INT_TABLE", "MATRIX", "VECTOR", "Block", "FeedForward", "Init", "Mixer", "Norm", "PagedKVSpec",
           "ParamSpec", "Part", "PositionEncoding", "StateSpec", "make_part", "register_part", "registered_parts",
           "PreNormBlock", "MLP", "Linear", "Attention", "Model", "ModelDescription", "OutputHead", "RunEntry",
           "TokenEmbedding", "LayerNorm", "LearnedAbsolute", "NoPosition"]
