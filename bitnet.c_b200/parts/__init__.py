"""Parts of a layer: norms, position encodings, mixers, feed-forwards, block arrangements."""
from .base import (Block, BuildContext, FeedForward, Head, KvRequest, Mixer, Norm, ParamSpec, Part, Position,
                   StateRequest)
from .registry import (build_part, known, register_block, register_ffn, register_head, register_mixer, register_norm,
                       register_position, register_side, unregister)
from . import (norm, position, attention, bias_attention, sigmoid_attention, latent_attention, normed_attention, mlstm, delta_rule, mlp, moe, token_side,  # noqa: F401
               block, head)  # (registers the built-in kinds)

__all__ = ["Block", "BuildContext", "FeedForward", "Head", "KvRequest", "Mixer", "Norm", "ParamSpec", "Part",
           "Position", "StateRequest", "build_part", "known", "register_block", "register_ffn", "register_head",
           "register_mixer", "register_norm", "register_position", "register_side", "unregister"]
