from .base import (BLOCKS, BRANCH_SCALES, FEED_FORWARDS, INPUT_PARTS, LOGITS_PARTS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheSpec,
                   FeedForward, InputPart, LogitsPart, Mixer, Norm, ParamSpec, Part, PartSpec, PositionEncoding, Runtime,
                   StateSpec, build_part, register_part)
from . import (attention, block, delta_rule, embedding, latent_attention, lightning, logits, mlp, moe, norm, parallel, rope,
               selective_scan, sink_attention)  # noqa: F401  (registers the built-in parts)

__all__ = ["BLOCKS", "BRANCH_SCALES", "FEED_FORWARDS", "INPUT_PARTS", "LOGITS_PARTS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block",
           "CacheSpec", "FeedForward", "InputPart", "LogitsPart", "Mixer", "Norm", "ParamSpec", "Part", "PartSpec", "PositionEncoding", "Runtime", "StateSpec",
           "build_part", "register_part"]
