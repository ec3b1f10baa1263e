"""Typed configurations and the architecture registry."""
from .guravik import GuravikConfig  # noqa: F401
from .minimax_m3 import ConfigError, MiniMaxM3Config  # noqa: F401
from .puvolix import PuvolixConfig  # noqa: F401
from .tarulix import TarulixConfig  # noqa: F401
from .tirizen import TirizenConfig  # noqa: F401
from .registry import known_architectures, load_config, register_architecture, resolve  # noqa: F401
