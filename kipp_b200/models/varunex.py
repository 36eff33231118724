"""The Varunex decoder: layers whose mixer is a gated matrix memory, attention over
a cached latent, or differential attention with a sliding window, each beside a
dense feed-forward on the output of one shared layer norm.  Its configuration
checks and its plan are the host core's (csrc/host/varunex.hpp); this module
registers the configuration class on the Python side.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.varunex import VarunexConfig
from .spec import ModelSpec


def build_varunex(config: VarunexConfig) -> ModelSpec:
    return ModelSpec.from_library(config)


register_architecture("Varunex", VarunexConfig, build_varunex)
