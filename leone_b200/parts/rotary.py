"""Rotary position encoding, with half-split or adjacent pairing.

Pair ``i`` of a head is elements ``(i, i + rotary_dim/2)`` (half-split) or
``(2i, 2i + 1)`` (adjacent; crates/leone/src/backend.rs:1216-1222,
crates/leone/src/cpu.rs:1767-1770); its angle at
position ``p`` is ``p * theta^(-2i/rotary_dim)``, inverse frequency and angle
in float64 (crates/leone/src/cpu.rs:1735-1745 and 1747-1779); the rotation is
``x'_i = x_i cos - x_j sin``, ``x'_j = x_i sin + x_j cos``.  The reference's
CUDA path also rotates with an fp32 (cos, sin) table made from float64 trig
(crates/leone-cuda/cuda/ie_cuda.cu:2382-2402).  The table is a constant of the
part, built once for ``max_positions``.
"""
from __future__ import annotations

import torch

from ..registry import POSITION_ENCODINGS
from .base import PositionEncoding


def build_rotary_table(max_positions: int, rotary_dim: int, theta: float) -> torch.Tensor:
    half = rotary_dim // 2
    pair = torch.arange(half, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * pair / rotary_dim)
    pos = torch.arange(max_positions, dtype=torch.float64)
    angle = pos[:, None] * inv_freq[None, :]
    return torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32).contiguous()


@POSITION_ENCODINGS.register("rotary_half_split")
class RotaryHalfSplit(PositionEncoding):
    pairing = "half_split"

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim")
        self._table = None

    def rotary_table(self):
        if self._table is None:
            self._table = build_rotary_table(
                self.max_positions, self.rotary_dim, self.theta).to(self.rt.device)
        return self._table


@POSITION_ENCODINGS.register("rotary_adjacent")
class RotaryAdjacent(RotaryHalfSplit):
    """The same angles with pair ``i`` made of elements ``(2i, 2i + 1)``: the table is the same,
    the kernels are told which elements belong together."""
    pairing = "adjacent"


def scaled_frequencies(dims: int, base: float, scaling=None):
    """Per pair ``i`` the frequency ``f_i = base^(-2i/dims)``, blended by YaRN if ``scaling``
    (a mapping with ``factor``, ``original``, ``fast``, ``slow``) is given, and the factor that
    multiplies cos and sin.

    YaRN (Peng et al., "YaRN: Efficient Context Window Extension of Large Language Models"): a
    pair that turns more than ``fast`` times within ``original`` positions keeps its frequency,
    one that turns fewer than ``slow`` times has it divided by ``factor``, and those between are
    blended linearly in the pair index: with ``idx(t) = dims * ln(original / (2 pi t)) / (2 ln
    base)``, ``lo = max(floor(idx(fast)), 0)``, ``hi = min(ceil(idx(slow)), dims - 1)`` and
    ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency is ``f_i / factor *
    ramp_i + f_i * (1 - ramp_i)``; cos and sin are multiplied by ``0.1 ln(factor) + 1``."""
    import math
    half = dims // 2
    freqs = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return freqs, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def idx(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(idx(float(scaling["fast"]))), 0)
    hi = min(math.ceil(idx(float(scaling["slow"]))), dims - 1)
    span = max(hi - lo, 0.001)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / span, 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


@POSITION_ENCODINGS.register("rotary_computed")
class RotaryComputed(PositionEncoding):
    """A rotary encoding without a table and so without a limit on positions: it offers its
    per-pair frequencies (fp32) and a magnitude, and the kernel that applies it forms the angle
    ``position * frequency`` and its cos and sin in fp32 itself.  ``scaling``: YaRN constants or
    ``None``.  ``pairing``: ``"adjacent"`` (pair i = elements 2i, 2i+1) or ``"half_split"``."""

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.rotary_dim = int(params["rotary_dim"])
        self.base = float(params["base"])
        self.scaling = params.get("scaling")
        self.pairing = params.get("pairing", "adjacent")
        if self.rotary_dim % 2 or self.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and positive")
        if self.pairing not in ("adjacent", "half_split"):
            raise ValueError(f"rotary pairing '{self.pairing}'")
        freqs, self.magnitude = scaled_frequencies(self.rotary_dim, self.base, self.scaling)
        self._freqs_host = torch.tensor(freqs, dtype=torch.float64).to(torch.float32)
        self._freqs = None

    def frequencies(self):
        """fp32 ``[rotary_dim / 2]`` on the device."""
        if self._freqs is None:
            self._freqs = self._freqs_host.to(self.rt.device)
        return self._freqs
