"""Parts that models are put together from.  Importing this package registers
the built-in kinds."""

from . import (attention, block, conv, embedding, grouped_attention, head, hgrn2, latent_attention, mlp, mlstm, moe, norm,  # noqa: F401
               position, recurrent, shift, sigmoid_attention)
from .base import (Block, Embedding, FeedForward, Head, Init, KVNeed, LayerSpec, Mixer, ModelSpec,
                   Norm, Part, PartSpec, PositionEncoding, RunStep, Source, StateNeed, TensorDecl,
                   make_block, make_part, pre_norm_layer, register_block, register_part)

__all__ = ["Part", "Norm", "Mixer", "FeedForward", "PositionEncoding", "Embedding", "Head", "Block",
           "Init", "TensorDecl", "Source", "PartSpec", "LayerSpec", "RunStep", "ModelSpec", "KVNeed",
           "StateNeed", "pre_norm_layer", "register_part", "register_block", "make_part", "make_block"]
