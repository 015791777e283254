"""Parts of a model: mixers, feed-forwards, norms, position encodings, blocks."""
from . import attention, block, embed_head, latent, mlp, moe, norm, position, recurrent, side, state_space  # noqa: F401  (register the built-in parts)
from .base import (Biased, Block, BlockExtra, Embedding, FeedForward, Head, Mixer, Norm, ParamSpec, Part, PartSpec, PositionEncoding,
                   build_part, register_part)
from .spec import ModelSpec, ScheduleEntry

__all__ = ["Biased", "Block", "BlockExtra", "Embedding", "FeedForward", "Head", "Mixer", "ModelSpec", "Norm", "ParamSpec", "Part", "PartSpec",
           "PositionEncoding", "ScheduleEntry", "build_part", "register_part"]
