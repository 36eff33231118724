"""Dense SwiGLU feed-forward: x += W_down (silu(W_gate n) * (W_up n))
(src/kipp.c:2994-3010, silu src/kipp.c:2402-2404), and the dense feed-forward with
one up projection, x += W_down act(W_up n).  The parts themselves:
csrc/host/parts.hpp."""
from __future__ import annotations

from .base import FeedForward


class SwiGLUFeedForward(FeedForward):
    kind = "swiglu"

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size}


class DenseFeedForward(FeedForward):
    """``activation``: relu, relu_squared, gelu_tanh or silu."""
    kind = "dense_mlp"

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu_squared",
                 names: dict | None = None):
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.names = dict(names or {})

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
                "activation": self.activation, "names": self.names}
