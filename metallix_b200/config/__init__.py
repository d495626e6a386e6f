"""Typed configurations, the architecture-independent model description and
the architecture registry."""
from .dimorax import DimoraxConfig
from .mekazen import MekazenConfig
from .qwen3 import ConfigError, Qwen3Config
from .registry import (ModelFamily, family_by_kind, parse_config, read_config, register,
                       resolve, unregister)
from .sadosun import SadosunConfig
from .zitezen import ZitezenConfig
from .spec import CacheNeed, LayerRun, LayerSpec, ModelSpec, PartSpec

__all__ = ["ConfigError", "MekazenConfig", "Qwen3Config", "ZitezenConfig", "SadosunConfig", "DimoraxConfig", "ModelFamily", "family_by_kind", "parse_config",
           "read_config", "register", "resolve", "unregister", "CacheNeed", "LayerRun",
           "LayerSpec", "ModelSpec", "PartSpec"]
