"""Typed configurations and the architecture registry."""
from .registry import (ConfigError, load_model_config, load_model_spec, read_config_json, register_architecture,
                       registered_architectures, resolve_architecture, unregister_architecture)
from . import qwen3 as _qwen3  # noqa: F401  (registers Qwen3)
from . import pabelix as _pabelix  # noqa: F401  (registers Pabelix)
from . import kolisun as _kolisun  # noqa: F401  (registers Kolisun)
from . import nedesun as _nedesun  # noqa: F401  (registers Nedesun)
from . import pepolorn as _pepolorn  # noqa: F401  (registers Pepolorn)
from .kolisun import KolisunConfig
from .nedesun import NedesunConfig
from .pabelix import PabelixConfig
from .pepolorn import PepolornConfig
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "Qwen3Config", "PabelixConfig", "KolisunConfig", "NedesunConfig", "PepolornConfig", "load_model_config", "load_model_spec", "read_config_json",
           "register_architecture", "registered_architectures", "resolve_architecture", "unregister_architecture"]
