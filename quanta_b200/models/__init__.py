"""Architectures: each module maps a configuration to a model specification and registers itself."""
from . import guravik, minimax_m3, puvolix, tarulix, tirizen  # noqa: F401
