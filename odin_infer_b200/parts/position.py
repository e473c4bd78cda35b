"""Position encodings."""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, register_part


@register_part("position_encoding", "rope")
class RotaryEncoding(PositionEncoding):
    """Half-split rotary encoding: pairs (i, i + rotary_dim/2), frequency
    1 / theta^(i / (rotary_dim/2)), angle = position * frequency, both formed in
    32-bit as the reference does (infer/forward.odin:67-70); cos and sin of that
    angle are tabulated on the host, so every kernel reads the same values.

    stretch = {"factor", "low", "high", "original"}: frequencies are stretched by their wavelength
    l = 2 pi / f: kept where l < original / high, divided by `factor` where l > original / low, and
    between the two blended, (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
    precise (always so with a stretch): the frequencies are formed in double and rounded to 32-bit once, instead of
    by the reference's 32-bit power."""

    graph_safe = True

    def __init__(self, rotary_dim: int, theta: float, stretch: dict | None = None, precise: bool = False):
        if rotary_dim % 2:
            raise ValueError(f"rotary_dim must be even, got {rotary_dim}")
        self.rotary_dim, self.theta, self.precise = rotary_dim, float(theta), bool(precise)
        self.stretch = None
        if stretch is not None:
            self.stretch = {k: float(stretch[k]) for k in ("factor", "low", "high", "original")}
            if not (self.stretch["high"] > self.stretch["low"] and self.stretch["factor"] > 0):
                raise ValueError(f"frequency stretch needs high > low and a positive factor, got {self.stretch}")
        self.cos = self.sin = None

    def frequencies(self) -> np.ndarray:
        """The rotary_dim / 2 frequencies as 32-bit floats."""
        half = self.rotary_dim // 2
        i = np.arange(half, dtype=np.float32)
        if self.stretch is None and not self.precise:
            return (np.float32(1.0) / np.power(np.float32(self.theta), i / np.float32(max(half, 1)))).astype(np.float32)
        f = np.power(np.float64(self.theta), -np.arange(half, dtype=np.float64) / max(half, 1))
        if self.stretch is None:
            return f.astype(np.float32)
        st = self.stretch
        wavelength = 2.0 * np.pi / f
        s = (st["original"] / wavelength - st["low"]) / (st["high"] - st["low"])
        blended = (1.0 - s) * f / st["factor"] + s * f
        f = np.where(wavelength < st["original"] / st["high"], f,
                     np.where(wavelength > st["original"] / st["low"], f / st["factor"], blended))
        return f.astype(np.float32)

    def prepare(self, rt, n_positions: int) -> None:
        freq = self.frequencies()
        pos = np.arange(max(n_positions, 1), dtype=np.float32)[:, None]
        ang = (pos * freq[None, :]).astype(np.float32).astype(np.float64)
        self.cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(rt.device).contiguous()
        self.sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(rt.device).contiguous()

    def rotation(self):
        return self.cos, self.sin, self.rotary_dim


@register_part("position_encoding", "none")
class NoEncoding(PositionEncoding):
    """No position information beyond the causal mask."""

    graph_safe = True
