"""The Venizen decoder: layers of two kinds (an attention mixer beside a
retention mixer; the generalized delta rule), PolyNorm feed-forwards, and a span
of layers that runs several times with the embedding output fed in again.  Its
configuration checks and its plan are the host core's (csrc/host/venizen.hpp);
this module registers the configuration class on the Python side.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.venizen import VenizenConfig
from .spec import ModelSpec


def build_venizen(config: VenizenConfig) -> ModelSpec:
    return ModelSpec.from_library(config)


register_architecture("Venizen", VenizenConfig, build_venizen)
