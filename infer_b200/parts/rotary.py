"""Rotary position encodings: half-split over the whole head, and adjacent pairs over part of it.

inv_freq[j] = 1 / theta^(2j / head_dim) in float32, angle = float32(pos) * inv_freq[j] (a float32
product), and element j of a head is rotated together with element j + head_dim/2:
x1' = x1*cos - x2*sin, x2' = x2*cos + x1*sin (src/forward.cpp:52-95).  As in the reference
(kernels/batch_gpu.cu:122-127) the tables are built on the host in float32 and uploaded, so the host's
plain implementation and the device rotate by identical angles.
"""
from __future__ import annotations

import torch

from ..config.specs import PartSpec
from .base import PositionEncoding, register_position


def rotary_tables(head_dim: int, theta: float, n_positions: int):
    """(cos, sin), float32 [n_positions, head_dim/2], on the CPU."""
    half = head_dim // 2
    exponent = torch.arange(0, half, dtype=torch.float32) * 2.0 / float(head_dim)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    angle = torch.arange(n_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(angle), torch.sin(angle)


@register_position("rotary_half")
class RotaryHalf(PositionEncoding):
    layout = "half"

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.head_dim, self.theta = int(spec["head_dim"]), float(spec["theta"])
        self.max_positions = int(spec["max_positions"])
        if self.head_dim % 2 or self.head_dim <= 0:
            raise ValueError(f"rotary_half needs an even head_dim, got {self.head_dim}")
        if self.theta <= 0:
            raise ValueError("rotary_half needs a positive theta")
        self._tables = {}

    def rotary_tables(self, n_positions: int = None):
        """Tables for positions [0, n_positions) on the device; cached per length."""
        n = min(self.max_positions, n_positions or self.max_positions)
        cache_key = (self.head_dim, self.theta, n, str(self.rt.device))
        t = _SHARED_TABLES.get(cache_key)
        if t is None:
            cos, sin = rotary_tables(self.head_dim, self.theta, n)
            t = (cos.to(self.rt.device).contiguous(), sin.to(self.rt.device).contiguous())
            _SHARED_TABLES[cache_key] = t
        return t

    def apply(self, q, k, positions):
        raise NotImplementedError("rotary_half is applied by the attention part's rotate-and-store kernel")


# Layers of one model share their tables (same head size, theta and length).
_SHARED_TABLES = {}


def pair_rotation_tables(rotary_dims: int, theta: float, n_positions: int):
    """(cos, sin), float32 [n_positions, rotary_dims/2], on the CPU: pair i turns by float32(pos) * float32(theta^(-2i /
    rotary_dims)), a float32 product; cosine and sine of that float32 angle are taken in float64 and rounded once."""
    i = torch.arange(rotary_dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / float(rotary_dims)).to(torch.float32)
    angle = (torch.arange(n_positions, dtype=torch.float32)[:, None] * freq[None, :]).to(torch.float64)
    return torch.cos(angle).to(torch.float32), torch.sin(angle).to(torch.float32)


@register_position("rotary_pairs")
class RotaryPairs(PositionEncoding):
    """Channels (2i, 2i + 1) of a head, for 2i < rotary_dims, turn together: (u, v) -> (u cos a - v sin a, v cos a +
    u sin a), a = pos * theta^(-2i / rotary_dims); channels from rotary_dims on pass unchanged. The attention part's
    prepare kernel applies it from the tables."""
    layout = "pairs"

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.head_dim, self.theta = int(spec["head_dim"]), float(spec["theta"])
        self.rotary_dims = int(spec.get("rotary_dims") or self.head_dim)
        self.max_positions = int(spec["max_positions"])
        if self.rotary_dims <= 0 or self.rotary_dims % 2 or self.rotary_dims > self.head_dim:
            raise ValueError(f"rotary_pairs needs an even number of rotated channels within the head, got "
                             f"{self.rotary_dims} of {self.head_dim}")
        if self.theta <= 0:
            raise ValueError("rotary_pairs needs a positive theta")

    def rotary_tables(self, n_positions: int = None):
        n = min(self.max_positions, n_positions or self.max_positions)
        cache_key = ("pairs", self.rotary_dims, self.theta, n, str(self.rt.device))
        t = _SHARED_TABLES.get(cache_key)
        if t is None:
            cos, sin = pair_rotation_tables(self.rotary_dims, self.theta, n)
            t = (cos.to(self.rt.device).contiguous(), sin.to(self.rt.device).contiguous())
            _SHARED_TABLES[cache_key] = t
        return t

    def apply(self, q, k, positions):
        raise NotImplementedError("rotary_pairs is applied by the attention part's prepare kernel")
