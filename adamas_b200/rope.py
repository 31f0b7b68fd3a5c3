"""Rotation-frequency tables for the RoPE-fused append and the table form of apply_rope_in_place.

The reference's CUDA path knows one rotary scheme: Llama's, with linear position scaling
(adamas/models/Adamas.py:52-61, kernels/include/decode/decode_page.cuh:650-659).  Models that were
stretched with YaRN use a different inverse frequency for every dimension pair and scale the rotated
values; both fit a table of 64 frequencies plus one factor, which the kernels here take by pointer
(`rope={"inv_freq": tensor, "mscale": float}` in the Python operators).  Everything in this module is
host arithmetic in float32 / float64 on small arrays.
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

HEAD_DIM = 128


def linear_inv_freq(rope_scale: float = 1.0, rope_theta: float = 1e4, head_dim: int = HEAD_DIM) -> torch.Tensor:
    """inv_freq[j] = 1 / (rope_scale * theta^(2j/d)): the table that reproduces linear position scaling."""
    j = torch.arange(0, head_dim, 2, dtype=torch.float32)
    return (1.0 / (torch.tensor(rope_theta, dtype=torch.float32) ** (j / head_dim))) / rope_scale


def yarn_inv_freq(factor: float, original_max_position: int, rope_theta: float = 1e4, head_dim: int = HEAD_DIM,
                  beta_fast: float = 32.0, beta_slow: float = 1.0) -> Tuple[torch.Tensor, float]:
    """YaRN ("NTK-by-parts") frequencies and attention factor: dimension pairs that turn more than
    beta_fast times over the original context keep their frequency, pairs that turn less than
    beta_slow times are interpolated by `factor`, a linear ramp blends the pairs in between; the
    rotated values are scaled by 0.1 * ln(factor) + 1.  Returns (inv_freq float32 [head_dim / 2], mscale)."""
    j = torch.arange(0, head_dim, 2, dtype=torch.float32)
    pos_freqs = torch.tensor(rope_theta, dtype=torch.float32) ** (j / head_dim)
    extrapolation = 1.0 / pos_freqs
    interpolation = 1.0 / (factor * pos_freqs)

    def correction_dim(num_rotations: float) -> float:
        return (head_dim * math.log(original_max_position / (num_rotations * 2 * math.pi))) / (2 * math.log(rope_theta))

    low = max(math.floor(correction_dim(beta_fast)), 0)
    high = min(math.ceil(correction_dim(beta_slow)), head_dim - 1)
    if low == high:
        high += 0.001
    ramp = torch.clamp((torch.arange(head_dim // 2, dtype=torch.float32) - low) / (high - low), 0, 1)
    keep = 1.0 - ramp                       # 1: keep the original frequency, 0: interpolate
    inv_freq = interpolation * (1 - keep) + extrapolation * keep
    return inv_freq, 0.1 * math.log(factor) + 1.0
