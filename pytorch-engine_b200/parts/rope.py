"""Rotary position encoding with precomputed float32 cos/sin tables, in either layout of pairs (split-half "neox":
feature j with j + rotary_dim/2; "interleaved": 2j with 2j + 1), optionally with YaRN-scaled frequencies.

Formulas: ``inv_freq_j = 1 / theta^(2j / rotary_dim)`` (pygguf_engine/model.py:147-156),
``angle = position * inv_freq`` with float32 positions, then cos and sin (183-185); rotation of the
first ``rotary_dim`` features ``[x1*cos - x2*sin, x2*cos + x1*sin]``, the rest passing through
(232-251).  ``inv_freq`` is computed on the host so that it is bit-identical everywhere; the
product and cos/sin are taken on the device in float32.

YaRN (``scaling`` = factor, original, fast, slow): with ``turn(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta)``
the pair index at which a pair makes ``t`` turns over ``original`` positions, ``lo = max(floor(turn(fast)), 0)``,
``hi = min(ceil(turn(slow)), rotary_dim - 1)`` and ``ramp_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1)``, pair j
turns with ``f_j / factor * ramp_j + f_j * (1 - ramp_j)``, and cos and sin carry the factor ``0.1 ln(factor) + 1``.
The scaled frequencies are computed in float64 on the host and rounded once to float32.
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from .registry import register
from .spec import WeightDecl


@register("position", "rope")
class RotaryPosition:
    """params: ``rotary_dim`` (even, <= head size), ``theta``, ``max_positions``, ``style`` ("neox" or
    "interleaved"), ``scaling`` (None, or a mapping with factor, original, fast, slow), ``exact`` (true: the tables are
    computed in float64 and rounded once; otherwise the angle is a float32 product, as the reference has it).  The tables hold
    ``max_positions`` rows, or as many as the engine can hold in one sequence if that is fewer
    (``runtime.position_limit``)."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    fusable_rotary = True

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        return {}

    def __init__(self, params, weights, runtime) -> None:
        self.rotary_dim = int(params["rotary_dim"])
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        limit = getattr(runtime, "position_limit", None)
        if limit:
            self.max_positions = min(self.max_positions, int(limit))
        self.style = params.get("style", "neox")
        if self.style not in ("neox", "interleaved"):
            raise ValueError(f"rotary layout {self.style!r} is not built ('neox' and 'interleaved' are)")
        self.interleaved = self.style == "interleaved"
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {self.rotary_dim}")
        scaling = params.get("scaling")
        mult = 1.0
        if params.get("exact") and not scaling:
            # frequencies, angles, cos and sin in float64 on the host, each table entry rounded once to float32
            idx = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
            ang = torch.outer(torch.arange(0, self.max_positions, dtype=torch.float64), self.theta ** (-idx / self.rotary_dim))
            self.cos = torch.cos(ang).to(torch.float32).to(runtime.device).contiguous()
            self.sin = torch.sin(ang).to(torch.float32).to(runtime.device).contiguous()
            return
        if not scaling:
            idx = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
            inv_freq = (1.0 / (self.theta ** (idx / self.rotary_dim))).to(runtime.device)
        else:
            inv_freq, mult = yarn_frequencies(self.rotary_dim, self.theta, scaling)
            inv_freq = inv_freq.to(runtime.device)
        pos = torch.arange(0, self.max_positions, dtype=torch.float32, device=runtime.device)
        freqs = torch.outer(pos, inv_freq)
        self.cos = torch.cos(freqs)
        self.sin = torch.sin(freqs)
        if mult != 1.0:
            self.cos *= mult
            self.sin *= mult
        self.cos = self.cos.contiguous()
        self.sin = self.sin.contiguous()

    def tables(self):
        return self.cos, self.sin, self.rotary_dim


def yarn_frequencies(rotary_dim: int, theta: float, scaling):
    """(float32 frequencies ``[rotary_dim / 2]``, factor on cos and sin) of a YaRN-scaled encoding."""
    factor, original = float(scaling["factor"]), float(scaling["original"])
    j = torch.arange(rotary_dim // 2, dtype=torch.float64)
    f = float(theta) ** (-2.0 * j / rotary_dim)

    def turn(t: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(theta))

    lo = max(math.floor(turn(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn(float(scaling["slow"]))), rotary_dim - 1)
    ramp = ((j - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f.to(torch.float32), 0.1 * math.log(factor) + 1.0
