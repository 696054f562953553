"""Rotary position encoding as a part: a table of (cos, sin) per position.

Angles as the reference's oracle computes them
(plugins/model-qwen3/qwen3_cpu_oracle.cpp:146-155): ``inv_i =
theta^(-2i/rotary_dim)``, ``angle = pos * inv_i`` in double, cast to
float32.  (Its GPU kernel uses float32 ``powf`` and has theta fixed in code,
kernels/cuda/qwen_bf16_primitives.cu:367-383; the two sides of the reference
differ there, and the double form is the one that does not drift at long
positions.)  The table is a pure function of the position, so cutting a
prompt into portions cannot change it.  The rotation itself (rotate-half
pairs ``(x_i, x_{i+rotary_dim/2})``, qwen_bf16_primitives.cu:326-347) is
done by the mixer's kernel, which reads this table.
"""
from __future__ import annotations

import torch

from .registry import Runtime, register_position

_TABLES = {}


@register_position("rope")
class RotaryEncoding:
    @classmethod
    def expected_tensors(cls, spec):
        return {}

    def __init__(self, spec, weights, rt: Runtime):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim must be even and within head_dim, got {spec.rotary_dim}")
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        key = (spec.rotary_dim, float(spec.theta), spec.max_positions, str(rt.device))
        if key not in _TABLES:
            pair = torch.arange(spec.rotary_dim // 2, dtype=torch.float64)
            inv = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * pair / spec.rotary_dim)
            angle = torch.arange(spec.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
            table = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32)
            _TABLES[key] = table.to(rt.device).contiguous()
        self._table = _TABLES[key]

    def rotation_table(self):
        """fp32 [max_positions, rotary_dim/2, 2] holding (cos, sin)."""
        return self._table


@register_position("rope_computed")
class ComputedRotary:
    """The same rotate-half rotation without a table: the mixer's kernel forms ``angle = position * f_i`` in 32-bit
    from the frequencies ``f_i = theta^(-2i/rotary_dim)`` (computed in double here, rounded once) and takes its
    cosine and sine there.  No longest context has to be known.  ``interleaved``: the pairs are neighbours instead of
    halves.  With ``stretch`` = (factor, low, high, original) the slow pairs are slowed down: with ``turns_i = original
    f_i / (2 pi)`` and ``t_i = clamp((turns_i - low) / (high - low), 0, 1)`` the frequency is ``f_i (t_i + (1 - t_i) /
    factor)``."""

    @classmethod
    def expected_tensors(cls, spec):
        return {}

    def __init__(self, spec, weights, rt: Runtime):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim must be even and within head_dim, got {spec.rotary_dim}")
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        self.interleaved = bool(getattr(spec, "interleaved", False))
        self._frequencies = self.frequencies_of(spec).to(torch.float32).to(rt.device).contiguous()

    @staticmethod
    def frequencies_of(spec) -> torch.Tensor:
        """float64 [rotary_dim / 2]."""
        import math
        pair = torch.arange(spec.rotary_dim // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * pair / spec.rotary_dim)
        stretch = getattr(spec, "stretch", None)
        if stretch is None:
            return f
        factor, low, high, original = (float(v) for v in stretch)
        if factor <= 0 or original <= 0 or low <= 0 or high <= 0 or low == high:
            raise ValueError("stretched rotation: factor, low, high and original must be positive, low and high differ")
        turns = original * f / (2.0 * math.pi)
        t = torch.clamp((turns - low) / (high - low), 0.0, 1.0)
        return f * (t + (1.0 - t) / factor)

    def rotation_table(self):
        return None

    def frequencies(self):
        """fp32 [rotary_dim / 2]."""
        return self._frequencies


@register_position("rope_scaled")
class ScaledRotary:
    """A table of (cos, sin) per position whose low frequencies may be stretched (``ScaledRopeSpec``).  With
    ``f_i = theta^(-2i / rotary_dim)`` and, where the spec has a ``factor``,

        turn(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta)
        lo = max(floor(turn(fast)), 0);   hi = min(ceil(turn(slow)), rotary_dim - 1)
        ramp_i = clamp((i - lo) / max(hi - lo, ramp_floor), 0, 1)
        f_i <- f_i / factor * ramp_i + f_i (1 - ramp_i);   gain = gain_slope ln(factor) + 1

    the table holds ``gain cos(p f_i), gain sin(p f_i)``, computed in double and rounded once.  ``pairing`` says which
    columns of a head make a pair: neighbours ``(2i, 2i + 1)`` or halves ``(i, i + rotary_dim / 2)``; the mixer's
    kernel does the rotation."""

    @classmethod
    def expected_tensors(cls, spec):
        return {}

    def __init__(self, spec, weights, rt: Runtime):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim must be even and within head_dim, got {spec.rotary_dim}")
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        self.interleaved = bool(spec.interleaved)
        key = ("scaled", spec.rotary_dim, float(spec.theta), spec.max_positions, spec.factor, float(spec.original),
               float(spec.fast), float(spec.slow), float(spec.gain_slope), float(spec.ramp_floor), str(rt.device))
        if key not in _TABLES:
            _TABLES[key] = self.table(spec).to(torch.float32).to(rt.device).contiguous()
        self._table = _TABLES[key]

    @staticmethod
    def frequencies_and_gain(spec):
        """(float64 [rotary_dim / 2], gain)."""
        import math
        dims = spec.rotary_dim
        pair = torch.arange(dims // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * pair / dims)
        if spec.factor is None:
            return f, 1.0
        if spec.factor <= 0 or spec.original <= 0 or spec.fast <= 0 or spec.slow <= 0 or spec.theta <= 1:
            raise ValueError("stretched rotation: factor, original, fast and slow must be positive, theta above 1")

        def turn(t):
            return dims * math.log(spec.original / (2.0 * math.pi * t)) / (2.0 * math.log(spec.theta))

        lo = max(math.floor(turn(spec.fast)), 0)
        hi = min(math.ceil(turn(spec.slow)), dims - 1)
        ramp = torch.clamp((pair - lo) / max(hi - lo, spec.ramp_floor), 0.0, 1.0)
        return f / spec.factor * ramp + f * (1.0 - ramp), spec.gain_slope * math.log(spec.factor) + 1.0

    @classmethod
    def table(cls, spec):
        f, gain = cls.frequencies_and_gain(spec)
        angle = torch.arange(spec.max_positions, dtype=torch.float64)[:, None] * f[None, :]
        return torch.stack([torch.cos(angle) * gain, torch.sin(angle) * gain], dim=-1)

    def rotation_table(self):
        """fp32 [max_positions, rotary_dim/2, 2] holding (gain cos, gain sin)."""
        return self._table
