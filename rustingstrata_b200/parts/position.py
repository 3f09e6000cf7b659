"""Rotary position encoding, NEOX pairing (i, i + n_rot/2).

Reference: theta = pos * base^(-2i/n_rot) in float64, sin/cos rounded to float32
(src/ops.rs:36-45; device src/cuda/kernels.cu:2192-2194,2212-2220).  Here the table
[position, cos(n_rot/2) | sin(n_rot/2)] is computed once on the host in float64 for all
positions the engine can reach and shared by every layer with the same parameters.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding
from .registry import register_part


@register_part("position", "rope_neox")
class RotaryNeox(PositionEncoding):
    """params: n_rot (rotated dims of a head), base, base_bits (32, the default: the base is held as float32 and widened,
    as the reference holds it; 64: the base as config.json gives it).  Coordinate i < n_rot / 2 turns together with
    i + n_rot / 2 (``pairing`` "half")."""
    chain_safe = True
    pairing = "half"

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.n_rot = int(spec.params["n_rot"])
        self.base = float(spec.params["base"])
        if self.n_rot % 2:
            raise ValueError(f"rope_neox: n_rot {self.n_rot} must be even")
        self.base_bits = int(spec.params.get("base_bits", 32))
        if self.base_bits not in (32, 64):
            raise ValueError(f"rope_neox: base_bits {self.base_bits} (32 or 64)")
        # as many positions as a request can reach: the model's limit, or what the cache pool holds if that is less
        self.rows = max(1, min(runtime.max_positions, runtime.pool_tokens))
        self._key = ("rope_neox", self.n_rot, self.base, self.base_bits, self.rows)

    @property
    def cos_sin(self) -> torch.Tensor:
        """[positions, cos(n_rot/2) | sin(n_rot/2)] float32, built at first use, one per parameter set."""
        return self.runtime.shared(self._key, self._table)

    def _table(self) -> torch.Tensor:
        half = self.n_rot // 2
        i = np.arange(half, dtype=np.float64)
        # the reference holds the base as float32 and widens it (src/ops.rs:39)
        base = np.float64(np.float32(self.base)) if self.base_bits == 32 else np.float64(self.base)
        inv = np.power(base, -2.0 * i / self.n_rot)
        theta = np.arange(self.rows, dtype=np.float64)[:, None] * inv[None, :]
        tab = np.concatenate([np.cos(theta), np.sin(theta)], axis=1).astype(np.float32)
        return torch.from_numpy(tab).to(self.runtime.device)


@register_part("position", "none")
class NoPosition(PositionEncoding):
    chain_safe = True
    n_rot = 0
    cos_sin = None


def scaled_frequencies(freq: np.ndarray, scaling) -> np.ndarray:
    """Rotation frequencies rescaled by wavelength; ``scaling`` = (factor, low, high, original) or None."""
    if scaling is None:
        return freq
    factor, low, high, original = scaling
    wave = 2.0 * np.pi / freq
    s = (original / wave - low) / (high - low)
    blend = (1.0 - s) * freq / factor + s * freq
    return np.where(wave < original / high, freq, np.where(wave > original / low, freq / factor, blend))


@register_part("position", "rope_interleaved")
class RotaryInterleaved(PositionEncoding):
    """Rotation of neighbouring pairs (2i, 2i + 1), i < n_rot / 2, by position * base^(-2i / n_rot).

    params: n_rot, base, scaling (None, or {factor, low, high, original}: frequencies rescaled by wavelength).  The table
    has the layout of the NEOX kind ([position, cos(n_rot/2) | sin(n_rot/2)], float64 angles rounded to float32); what
    differs is which coordinates a kernel pairs, which ``pairing`` tells.  It holds as many positions as a request can
    reach: the model's limit, or what the cache pool holds if that is less.

    ``scaling`` stretches the slow rotations of a model trained on ``original`` positions: with wavelength
    l = 2 pi / f, a frequency with l < original / high is kept, one with l > original / low becomes f / factor, and in
    between, with s = (original / l - low) / (high - low), it becomes (1 - s) f / factor + s f."""
    chain_safe = True
    pairing = "interleaved"

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.n_rot = int(spec.params["n_rot"])
        self.base = float(spec.params["base"])
        if self.n_rot % 2:
            raise ValueError(f"rope_interleaved: n_rot {self.n_rot} must be even")
        sc = spec.params.get("scaling")
        self.scaling = None if not sc else (float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"]))
        if self.scaling is not None and (self.scaling[0] <= 0 or self.scaling[2] <= self.scaling[1] or self.scaling[3] <= 0):
            raise ValueError(f"rope_interleaved: scaling needs factor > 0, high > low and original > 0, got {sc}")
        self.rows = max(1, min(runtime.max_positions, runtime.pool_tokens))
        self._key = ("rope_interleaved", self.n_rot, self.base, self.scaling, self.rows)

    @property
    def cos_sin(self) -> torch.Tensor:
        return self.runtime.shared(self._key, self._table)

    def _table(self) -> torch.Tensor:
        half = self.n_rot // 2
        inv = scaled_frequencies(np.power(np.float64(self.base), -2.0 * np.arange(half, dtype=np.float64) / self.n_rot),
                                 self.scaling)
        theta = np.arange(self.rows, dtype=np.float64)[:, None] * inv[None, :]
        tab = np.concatenate([np.cos(theta), np.sin(theta)], axis=1).astype(np.float32)
        return torch.from_numpy(tab).to(self.runtime.device)
