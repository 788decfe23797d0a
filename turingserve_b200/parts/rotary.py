"""Rotate-half rotary position encoding: the fp32 cos/sin tables.

inv_freq[i] = 1 / theta**(2i/rotary_dim); angle = position * inv_freq, all in 32-bit
(turingserve/model/layers.py:13-18).  The rotation itself runs inside the kernel that also
writes keys and values to the cache; it uses the table rows cast to the model dtype and does
its arithmetic in 32-bit with one rounding (turingserve/ops/triton_rope.py:10-24).
"""

from __future__ import annotations

import math

import torch

from turingserve_b200.parts.base import BuildContext, register


class RotaryEncoding:
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.rotary_dim = int(spec.rotary_dim)
        self.theta = float(spec.theta)
        if self.rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        n = min(int(spec.max_positions), ctx.max_positions) if ctx.max_positions else int(spec.max_positions)
        self.max_positions = n
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).float()
                                         / self.rotary_dim))
        freqs = torch.outer(torch.arange(n).float(), inv_freq)
        self.cos = freqs.cos().to(ctx.device).contiguous()
        self.sin = freqs.sin().to(ctx.device).contiguous()


class PairRotaryEncoding:
    """Rotation of neighbouring pairs (2i, 2i+1) with YaRN-blended frequencies.  No table over positions:
    the kernels take the angle as position * ``freq[i]`` in 32-bit and multiply cosine and sine by
    ``magnitude``, so no longest sequence has to be known.  ``freq`` is float32 [dims / 2] on the device."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.dims = int(spec.dims)
        if self.dims % 2 or self.dims <= 0:
            raise ValueError("the rotated dimensions come in pairs")
        base = float(spec.base)
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        f = base ** (-2.0 * i / self.dims)
        self.magnitude = 1.0
        if spec.factor:
            def index_of(turns: float) -> float:
                """The (fractional) pair index whose frequency turns ``turns`` times within ``original`` positions."""
                return self.dims * math.log(spec.original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
            first = max(math.floor(index_of(spec.fast)), 0)
            last = min(math.ceil(index_of(spec.slow)), self.dims - 1)
            share = ((i - first) / max(last - first, 0.001)).clamp(0.0, 1.0)      # of the slowed frequency
            f = f * (1.0 - share) + (f / float(spec.factor)) * share
            self.magnitude = 1.0 + 0.1 * math.log(float(spec.factor))
        self.freq = f.to(torch.float32).to(ctx.device).contiguous()


class HalfRotaryEncoding:
    """Rotation of the pairs (i, i + dims / 2) without a table over positions: the kernels take the angle as
    position * ``freq[i]`` in 32-bit.  ``freq`` is float32 [dims / 2] on the device, base^(-2i/dims) worked out in
    double and rounded once."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.dims = int(spec.dims)
        if self.dims % 2 or self.dims < 0:
            raise ValueError("the rotated dimensions come in pairs")
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        f = float(spec.base) ** (-2.0 * i / max(self.dims, 1))
        self.freq = f.to(torch.float32).to(ctx.device).contiguous()


class BandScaledPairEncoding:
    """Rotation of neighbouring pairs (2i, 2i+1) with frequencies rescaled by wavelength bands.  No table over
    positions: the kernels take the angle as position * ``freq[i]`` in 32-bit.  ``freq`` is float32 [dims / 2] on the
    device, worked out in double and rounded once."""

    pairing = "neighbours"
    magnitude = 1.0

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.dims = int(spec.dims)
        if self.dims % 2 or self.dims < 0:
            raise ValueError("the rotated dimensions come in pairs")
        base = float(spec.base)
        freqs = []
        for i in range(self.dims // 2):
            f = base ** (-2.0 * i / self.dims)
            if spec.factor:
                factor, low, high, original = float(spec.factor), float(spec.low), float(spec.high), float(spec.original)
                wavelength = 2.0 * math.pi / f
                if wavelength > original / low:
                    f = f / factor
                elif wavelength >= original / high:
                    s = (original / wavelength - low) / (high - low)
                    f = (1.0 - s) * f / factor + s * f
            freqs.append(f)
        self.freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(ctx.device).contiguous()


HalfRotaryEncoding.pairing = "halves"
PairRotaryEncoding.pairing = "neighbours"

register("position", "rope", RotaryEncoding)
register("position", "rope_pairs_banded", BandScaledPairEncoding)
register("position", "rope_half", HalfRotaryEncoding)
register("position", "yarn_pairs", PairRotaryEncoding)
