"""Position encodings.  Rotary: inv_freq[i] = theta^(-2i/rot_dim) in float32
(crates/fellm-model/src/rope.rs:13-21); pairs (2i, 2i+1) or (i, i+rot_dim/2)
(crates/backend-cpu/src/kernels/rope.rs:28-62).  The rotation itself happens inside the kernel
that also norms q/k and writes the cache (fellm_b200/csrc/qk_rope_write.cu).

Frequencies scaled for contexts beyond the trained one (`scaling` = (factor, original, fast, slow)): with
pair(t) = rot_dim ln(original / (2 pi t)) / (2 ln theta), the pair index at which a rotation makes t turns over
`original` positions, lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)), rot_dim - 1) and
ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at f_i / factor * ramp_i + f_i (1 - ramp_i):
fast pairs keep their frequency, slow ones are divided by the factor.  `magnitude` = 0.1 ln(factor) + 1 then
multiplies cos and sin (1 without scaling); a kernel that rotates takes it beside inv_freq.

Frequencies rescaled by wavelength (`bands` = (factor, low, high, original)): with l = 2 pi / f, a pair keeps f where
l < original / high, turns at f / factor where l > original / low, and between the two, with
s = (original / l - low) / (high - low), at (1 - s) f / factor + s f.  No magnitude goes with it."""
from __future__ import annotations

import math

import torch

from ..config.errors import ConfigError
from .base import PositionEncoding, register_part


@register_part("position", "none")
class NoPosition(PositionEncoding):
    def __init__(self, *, dtype: str):
        super().__init__()
        self.inv_freq = None
        self.pairing = "adjacent"

    def to(self, device):
        return self


@register_part("position", "rope")
class Rotary(PositionEncoding):
    def __init__(self, *, dtype: str, rot_dim: int, theta: float, pairing: str, table64: bool = False, scaling=None,
                 bands=None):
        """table64: the frequencies are computed in float64 and rounded once (default: float32 powers, as FeLLM's).
        scaling: (factor, original, fast, slow), see the module's head; computed in float64 and rounded once."""
        super().__init__()
        self.magnitude = 1.0
        if rot_dim % 2:
            raise ConfigError(f"rotary dimension {rot_dim} must be even")
        if pairing not in ("adjacent", "split_half"):
            raise ConfigError(f"unknown rotary pairing {pairing!r}")
        self.rot_dim, self.theta, self.pairing = int(rot_dim), float(theta), pairing
        if bands and scaling:
            raise ConfigError("rotary: `scaling` and `bands` are two ways to rescale the frequencies; name one")
        if bands:
            factor, low, high, original = (float(v) for v in bands)
            if min(factor, low, high, original) <= 0 or self.theta <= 0:
                raise ConfigError(f"rotary bands {bands!r} need positive numbers")
            freqs = []
            for i in range(self.rot_dim // 2):          # float64 on the host, rounded once
                f = self.theta ** (-2.0 * i / self.rot_dim)
                wavelength = 2.0 * math.pi / f
                if wavelength < original / high:
                    freqs.append(f)
                elif wavelength > original / low:
                    freqs.append(f / factor)
                else:
                    s = (original / wavelength - low) / ((high - low) or 1.0)
                    freqs.append((1.0 - s) * f / factor + s * f)
            self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32)
            return
        if scaling:
            factor, original, fast, slow = (float(v) for v in scaling)
            if min(factor, original, fast, slow) <= 0 or self.theta <= 1.0:
                raise ConfigError(f"rotary scaling {scaling!r} needs positive numbers and a base above 1")
            n = self.rot_dim

            def pair(turns):
                return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

            lo, hi = max(math.floor(pair(fast)), 0), min(math.ceil(pair(slow)), n - 1)
            freqs = []
            for i in range(n // 2):
                f = self.theta ** (-2.0 * i / n)
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                freqs.append(f / factor * ramp + f * (1.0 - ramp))
            self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32)
            self.magnitude = 0.1 * math.log(factor) + 1.0
            return
        if table64:
            i = torch.arange(self.rot_dim // 2, dtype=torch.float64)
            self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                      -(2.0 * i) / float(self.rot_dim)).to(torch.float32)
            return
        i = torch.arange(self.rot_dim // 2, dtype=torch.float32)
        self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float32),
                                  -(2.0 * i) / float(self.rot_dim))

    def to(self, device):
        self.inv_freq = self.inv_freq.to(device)
        return self
