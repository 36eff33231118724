"""Attention whose keys and values are made from one small latent per token:
queries through a latent of their own, a rotated key part shared by all heads,
optionally a sink per head in the softmax's denominator, a sigmoid gate per head
and a window.  Only the latent and the rotated key part are cached.  The part
itself: csrc/host/latent_parts.hpp."""
from __future__ import annotations

from typing import Optional

from .base import Mixer, PositionEncoding


class LatentAttentionMixer(Mixer):
    kind = "latent_attention"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, kv_rank: int, q_rank: int,
                 position: PositionEncoding, eps: float, *, value_dim: Optional[int] = None,
                 scale: Optional[float] = None, sink: bool = False, gate: str = "none", window: int = 0,
                 output_scale: float = 1.0, names: Optional[dict] = None):
        self.hidden_size, self.num_heads, self.head_dim, self.rot_dim = hidden_size, num_heads, head_dim, rot_dim
        self.kv_rank, self.q_rank, self.position, self.eps = kv_rank, q_rank, position, eps
        self.value_dim, self.scale, self.sink, self.gate = value_dim or head_dim, scale, sink, gate
        self.window, self.output_scale, self.names = window, output_scale, dict(names or {})

    def params(self, prefix, ctx) -> dict:
        out = {"hidden_size": self.hidden_size, "num_heads": self.num_heads, "head_dim": self.head_dim,
               "rot_dim": self.rot_dim, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "value_dim": self.value_dim,
               "position": self.position.describe(prefix, ctx), "eps": self.eps, "sink": bool(self.sink),
               "gate": self.gate, "window": int(self.window), "output_scale": float(self.output_scale),
               "names": self.names}
        if self.scale is not None:
            out["scale"] = float(self.scale)
        return out
