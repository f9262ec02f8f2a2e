"""Typed configurations and the architecture-neutral model description."""
from .json_util import ConfigError, read_json
from .lfm3 import Lfm3Config, Lfm3Rope
from .saralix import SaralixConfig
from .nimelorn import NimelornConfig
from .tozarax import TozaraxConfig
from .vekuzen import VekuzenConfig
from .spec import (AttentionSpec, LayerCall, LayerSpec, ModelSpec, NormSpec, RopeSpec,
                   ShortConvSpec, SwiGLUSpec)

__all__ = ["ConfigError", "read_json", "Lfm3Config", "Lfm3Rope", "SaralixConfig", "NimelornConfig", "TozaraxConfig", "VekuzenConfig", "AttentionSpec", "LayerCall",
           "LayerSpec", "ModelSpec", "NormSpec", "RopeSpec", "ShortConvSpec", "SwiGLUSpec"]
