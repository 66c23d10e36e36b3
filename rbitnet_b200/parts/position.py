"""Position encodings.

Rotary: each head's pairs are rotated by angle = pos * theta^(-2i/D), the
inverse frequencies and the angle in float32
(crates/bitnet-core/src/llama/model.rs:122-136).  ``pairing`` "interleaved"
rotates (2i, 2i+1) as the reference does; "half" rotates (i, i+D/2), the row
order of checkpoints with Hugging Face tensor names.  Keys are cached after the
rotation, values are not rotated (:242-257).

Options beyond the reference's: only the first ``rot_dim`` values of a head turn (the
rest pass), and ``scaling`` stretches the slow frequencies for contexts longer than the
``original`` one:  with d(t) = rot_dim * ln(original / (2 pi t)) / (2 ln theta),
lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rot_dim - 1) and
ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns with
f_i * (ramp_i / factor + 1 - ramp_i), and sines and cosines are multiplied by
0.1 ln(factor) + 1.
``scaling`` with "kind": "wavelength" (keys factor, low, high, original) decides pair by pair from the pair's
wavelength l = 2 pi / f:  f stays where l < original / high; it becomes f / factor where l > original / low; between
the two, with s = (original / l - low) / (high - low), it becomes (1 - s) f / factor + s f.  Sines and cosines keep
magnitude 1.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from .registry import register_part


class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, pairing: str = "half", max_positions: int = 0,
                 rot_dim: int = 0, scaling: dict = None):
        self.rot_dim = int(rot_dim) if rot_dim else int(head_dim)
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ValueError(f"rotary encoding turns an even number of values of a head of {head_dim}, found {self.rot_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.head_dim, self.theta, self.pairing = int(head_dim), float(theta), pairing
        self.max_positions = int(max_positions)
        self.scaling = dict(scaling) if scaling else None
        if self.scaling:
            by_wavelength = self.scaling.get("kind") == "wavelength"
            missing = [k for k in (("factor", "original", "low", "high") if by_wavelength else
                                   ("factor", "original", "fast", "slow")) if k not in self.scaling]
            if missing:
                raise ValueError(f"rotary scaling needs {', '.join(missing)}")
        self.inv_freq = self.freq64 = None
        self.magnitude = 1.0

    def frequencies(self):
        """(float64 frequencies of the rot_dim/2 pairs, magnitude of sines and cosines)."""
        n = self.rot_dim
        i = torch.arange(n // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / n)
        if not self.scaling:
            return f, 1.0
        sc = self.scaling
        factor, original = float(sc["factor"]), float(sc["original"])
        if sc.get("kind") == "wavelength":
            low, high = float(sc["low"]), float(sc["high"])
            length = 2.0 * math.pi / f
            s = ((original / length - low) / (high - low)).clamp(0.0, 1.0) if high != low else torch.ones_like(f)
            blended = (1.0 - s) * f / factor + s * f
            out = torch.where(length < original / high, f, torch.where(length > original / low, f / factor, blended))
            return out, 1.0

        def pair_of(turns):
            return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
        lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(pair_of(float(sc["slow"]))), n - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0

    def bind(self, weights, ops):
        f, self.magnitude = self.frequencies()
        self.freq64 = f.to(ops.device)
        if not self.scaling:
            # the float32 table of the kernels that turn whole heads
            i = torch.arange(self.rot_dim // 2, dtype=torch.float32)
            inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), 2.0 * i / self.rot_dim)
            self.inv_freq = inv.to(ops.device)
        else:
            self.inv_freq = f.to(torch.float32).to(ops.device)

    @property
    def plain(self) -> bool:
        """Whole heads turn with unscaled frequencies and magnitude 1."""
        return self.rot_dim == self.head_dim and not self.scaling

    def rotary(self):
        return self.inv_freq, self.pairing == "interleaved", self.rot_dim

    def table(self):
        """(float64 frequencies on the device, magnitude, interleaved, rot_dim)."""
        return self.freq64, float(self.magnitude), self.pairing == "interleaved", self.rot_dim


class NoPositionEncoding(PositionEncoding):
    """Positions enter only through the causal mask."""
    def __init__(self, **_):
        pass


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
