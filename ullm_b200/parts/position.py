"""Position encodings.  The rotary table is built as the reference builds it
(ullm/layers/rotary_embedding.py:58-75): inv_freq_i = 1 / theta^(2i/dim) and
angle[p, i] = p * inv_freq_i in float32 on the host, cos and sin of it in
float32.  The mixer's kernel reads row `position` of the tables and rotates in
32-bit registers.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from .registry import register_position_encoding


@register_position_encoding("rope")
class RotaryPositions(PositionEncoding):
    def __init__(self, rotary_dim: int, theta: float, max_positions: int):
        super().__init__()
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim={rotary_dim} must be a positive even number")
        if max_positions <= 0:
            raise ValueError("max_positions must be positive")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.max_positions = max_positions
        self._tables: dict[str, torch.Tensor] = {}

    def build_tables(self, device) -> None:
        inv_freq = 1.0 / (
            self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim)
        )
        t = torch.arange(self.max_positions, dtype=torch.float32)
        freqs = torch.einsum("i,j->ij", t, inv_freq)
        self._tables = {
            "cos": freqs.cos().contiguous().to(device),
            "sin": freqs.sin().contiguous().to(device),
        }

    def tables(self):
        return self._tables


def scaled_frequencies(rotary_dim: int, theta: float, scaling: dict | None = None) -> torch.Tensor:
    """f_i = theta^(-2i / rotary_dim) in 64-bit, i < rotary_dim / 2.  `scaling` (factor, low, high, original)
    rescales by wavelength l = 2 pi / f: waves shorter than original / high stay; waves longer than
    original / low are slowed by `factor`; between the two the slowed and the original frequency are blended
    linearly in original / l."""
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / rotary_dim)
    if scaling:
        try:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        except KeyError as e:
            raise ValueError(f"frequency scaling lacks {e.args[0]!r} (factor, low, high, original)") from None
        if factor <= 0 or high <= low or orig <= 0 or low <= 0:
            raise ValueError("frequency scaling needs factor > 0, 0 < low < high and original > 0")
        wave = 2.0 * math.pi / f
        s = ((orig / wave - low) / (high - low)).clamp(0.0, 1.0)
        blended = (1.0 - s) * f / factor + s * f
        f = torch.where(wave < orig / high, f, torch.where(wave > orig / low, f / factor, blended))
    return f


@register_position_encoding("rope_computed")
class ComputedRotaryPositions(PositionEncoding):
    """A rotation whose angles the mixer's kernel computes itself: `tables()` holds only `inv_freq`
    (rotary_dim / 2 floats, built in 64-bit, kept in 32-bit); the kernel forms the 32-bit product position x
    frequency and its sine and cosine, so there is no table per position and no largest position.  Dimension i of
    a head is rotated with dimension i + rotary_dim / 2, or with `interleaved` dimension 2i with 2i + 1 (the
    mixer's kernel must know the pairing asked for: a mixer checks this flag).  `scaling`: see `scaled_frequencies`."""

    computed = True

    def __init__(self, rotary_dim: int, theta: float, max_positions: int = 0, scaling: dict | None = None,
                 interleaved: bool = False):
        super().__init__()
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim={rotary_dim} must be a positive even number")
        if not theta > 0:
            raise ValueError("the rotation's base must be positive")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.max_positions = max_positions
        self.scaling = dict(scaling) if scaling else None
        self.interleaved = bool(interleaved)
        scaled_frequencies(rotary_dim, self.theta, self.scaling)  # (refuses bad constants now, not at load time)
        self._tables: dict[str, torch.Tensor] = {}

    def build_tables(self, device) -> None:
        f = scaled_frequencies(self.rotary_dim, self.theta, self.scaling)
        self._tables = {"inv_freq": f.to(torch.float32).contiguous().to(device)}

    def tables(self):
        return self._tables


@register_position_encoding("none")
class NoPositions(PositionEncoding):
    def __init__(self, rotary_dim: int = 0, theta: float = 0.0, max_positions: int = 0):
        super().__init__()
        self.rotary_dim = 0
        self.max_positions = max_positions

    def build_tables(self, device) -> None:
        pass


@register_position_encoding("sinusoid_added")
class AddedSinusoid(PositionEncoding):
    """An absolute encoding that is ADDED to the token embedding, not applied to queries and keys: column 2i of
    position p is sin(p f_i), column 2i + 1 is cos(p f_i), f_i = theta^(-2i / width).  `rotary_dim` is the width of
    the embedding.  The table of the f_i is built in 64-bit and kept in 32-bit; the embedding kernel forms the
    32-bit angle and the sinusoids itself, so there is no table per position and no largest position."""

    def __init__(self, rotary_dim: int, theta: float = 10000.0, max_positions: int = 0):
        super().__init__()
        if rotary_dim <= 0:
            raise ValueError("the width of an added encoding must be positive")
        self.width = rotary_dim
        self.rotary_dim = 0  # nothing is rotated
        self.theta = float(theta)
        self.max_positions = max_positions
        self._tables: dict[str, torch.Tensor] = {}

    def adds_to_embedding(self) -> bool:
        return True

    def build_tables(self, device) -> None:
        i = torch.arange((self.width + 1) // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.width)
        self._tables = {"inv_freq": inv.to(torch.float32).contiguous().to(device)}

    def tables(self):
        return self._tables
