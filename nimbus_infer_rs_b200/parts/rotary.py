"""Rotary position angles as data: per pair of rotated dimensions its angular frequency.

A head's first ``dims`` numbers are turned; dimension ``i`` is paired with ``i + dims/2``
(``i < dims/2``), and the pair ``(u, v)`` of a token at position ``p`` becomes
``(u cos a - v sin a, v cos a + u sin a)`` with ``a = p * f_i``, ``f_i = base^(-2i/dims)``.

With frequency scaling for contexts longer than the ``original`` one (``factor, original,
fast, slow``): a pair that makes ``t`` turns over the original context sits at dimension
``dim(t) = dims * ln(original / (2 pi t)) / (2 ln base)``; pairs below ``lo = floor(dim(fast))``
keep their frequency, pairs above ``hi = ceil(dim(slow))`` get ``f_i / factor``, the ones
between a linear blend (``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``), and cos and
sin are both multiplied by ``0.1 ln(factor) + 1``.

The frequencies are computed once on the host in float64 and handed to the kernels as an fp32
table; the angle ``p * f_i`` and its cos and sin are fp32 on the device.
"""
from __future__ import annotations

import math

import torch


def rotary_frequencies(dims: int, base: float, scaling: dict | None = None):
    """``(fp32 tensor [dims/2], factor on cos and sin)``.  ``scaling``: ``None`` or a mapping
    with ``factor``, ``original``, ``fast``, ``slow``."""
    dims = int(dims)
    if dims < 2 or dims % 2:
        raise ValueError(f"rotated dimensions come in pairs, got dims={dims}")
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    amplitude = 1.0
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def dim_of(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        amplitude = 0.1 * math.log(factor) + 1.0
    return f.to(torch.float32), float(amplitude)


def rotary_frequencies_by_wavelength(dims: int, base: float, scaling: dict | None = None):
    """fp32 tensor ``[dims/2]`` of ``f_i = base^(-2i/dims)``, with scaling by wavelength for
    contexts longer than the ``original`` one (``factor, low, high, original``): a pair whose
    wavelength ``2 pi / f`` is shorter than ``original / high`` keeps its frequency, one longer
    than ``original / low`` gets ``f / factor``, and between the two, with ``s = (original /
    wavelength - low) / (high - low)``, the blend ``(1 - s) f / factor + s f``.  cos and sin
    keep their size."""
    dims = int(dims)
    if dims < 2 or dims % 2:
        raise ValueError(f"rotated dimensions come in pairs, got dims={dims}")
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, original = float(scaling["factor"]), float(scaling["original"])
            low, high = float(scaling["low"]), float(scaling["high"])
            wavelength = 2.0 * math.pi / f
            if wavelength > original / low:
                f = f / factor
            elif wavelength >= original / high:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)
