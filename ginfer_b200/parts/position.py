"""Position encodings.

Rotary, as the reference computes it (``ginfer/core/op/kernels/cuda/rope_kernel.cu:13-16,61-71``
for the table, ``:84-102`` for the rotation): ``inv_j = 1 / theta^(j / (hd/2))``,
``angle = pos * inv_j`` in fp32, pairs ``(j, j + hd/2)`` rotated by
``o_j = x_j cos - x_{j+hd/2} sin``, ``o_{j+hd/2} = x_j sin + x_{j+hd/2} cos``; applied to queries
and keys, not to values.  Here ``inv_j`` is computed in double and rounded once to fp32, the
product ``float(pos) * inv_j`` is an fp32 product, and cos/sin of that fp32 angle are evaluated
in double and rounded to fp32, so host and device cannot disagree on a table entry.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, register_position


class RotaryPosition(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_positions: int,
                 rotary_dim: int | None = None):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(head_dim if rotary_dim is None else rotary_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and <= head_dim "
                             f"{self.head_dim}")
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self._table: torch.Tensor | None = None

    def load(self, tensors, dtype, device):
        half = self.rotary_dim // 2
        inv = (1.0 / np.power(np.float64(self.theta),
                              np.arange(half, dtype=np.float64) / half)).astype(np.float32)
        pos = np.arange(self.max_positions, dtype=np.float32)
        ang = (pos[:, None] * inv[None, :]).astype(np.float32)      # fp32 product
        ang64 = ang.astype(np.float64)
        table = np.concatenate([np.cos(ang64), np.sin(ang64)], axis=1).astype(np.float32)
        self._table = torch.from_numpy(table).to(device)

    def rotary_table(self):
        return self._table, self.rotary_dim


class NoPosition(PositionEncoding):
    """No position information is added to queries and keys."""

    def __init__(self, **_):
        pass

    def rotary_table(self):
        return None, 0


class PairRotary(PositionEncoding):
    """Rotation of channel pairs by ``position * f_i`` with ``f_i = base^(-2i/dims)`` over the
    first ``dims`` channels of a head; the pairs are neighbours ``(2i, 2i+1)`` (``interleaved``) or
    halves ``(i, i + dims/2)``.  ``scaling = {factor, low, high, original}`` stretches the long
    wavelengths: with ``l = 2 pi / f``, ``f`` stays where ``l < original/high``, becomes
    ``f / factor`` where ``l > original/low`` and ``(1 - s) f / factor + s f`` with
    ``s = (original/l - low) / (high - low)`` in between.  ``linear_factor`` divides every
    frequency (positions stretched evenly).  Nothing is tabulated by position: the
    mixer's kernel forms ``float(p) * f_i`` in 32-bit and takes sine and cosine of it."""

    def __init__(self, dims: int, base: float, scaling=None, interleaved: bool = True,
                 linear_factor: float = 1.0):
        self.dims, self.base = int(dims), float(base)
        self.linear_factor = float(linear_factor)
        if not (self.linear_factor > 0):
            raise ValueError(f"linear_factor must be > 0, got {linear_factor}")
        if self.dims % 2 or self.dims < 0:
            raise ValueError(f"{self.dims} rotated channels: must be an even number")
        self.scaling = None if scaling is None else {k: float(scaling[k]) for k in
                                                     ("factor", "low", "high", "original")}
        if self.scaling is not None and self.scaling["high"] == self.scaling["low"]:
            raise ValueError("frequency scaling needs high != low")
        self.interleaved = bool(interleaved)
        self._freqs: torch.Tensor | None = None

    def host_frequencies(self) -> np.ndarray:
        i = np.arange(self.dims // 2, dtype=np.float64)
        f = np.power(np.float64(self.base), -2.0 * i / max(self.dims, 1))
        sc = self.scaling
        if sc is not None:
            wave = 2.0 * np.pi / f
            ramp = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            mid = (1.0 - ramp) * f / sc["factor"] + ramp * f
            f = np.where(wave < sc["original"] / sc["high"], f,
                         np.where(wave > sc["original"] / sc["low"], f / sc["factor"], mid))
        return (f / self.linear_factor).astype(np.float32)

    def load(self, tensors, dtype, device):
        self._freqs = torch.from_numpy(self.host_frequencies()).to(device)

    def frequencies(self) -> torch.Tensor:
        """fp32 ``[dims / 2]`` on the device."""
        return self._freqs


register_position("rotary", RotaryPosition)
register_position("pair_rotary", PairRotary)
register_position("none", NoPosition)
