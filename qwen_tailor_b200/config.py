"""Model constants of the hot path (mirror of the reference's ``Cfg`` dataclass, qwen35/model.py:35-60)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Cfg:
    hidden: int = 1024
    layers: int = 24
    full_attn_interval: int = 4
    n_heads: int = 8
    n_kv: int = 2
    head_dim: int = 256
    rope_dim: int = 64
    rope_theta: float = 1e7
    hk: int = 16
    hv: int = 16
    dk: int = 128
    dv: int = 128
    conv_k: int = 4
    eps: float = 1e-6

    @property
    def conv_dim(self) -> int:
        return 2 * self.hk * self.dk + self.hv * self.dv

    def is_linear(self, i: int) -> bool:
        """Layer i is a GatedDeltaNet layer unless (i + 1) is a multiple of the full-attention interval."""
        return (i + 1) % self.full_attn_interval != 0

    @property
    def n_linear(self) -> int:
        return sum(self.is_linear(i) for i in range(self.layers))

    @property
    def n_full(self) -> int:
        return self.layers - self.n_linear
