"""Position encodings.

``LearnedAbsolute``: a table ``[n_positions, width]`` added to the token
embedding at each token's position in its request; the position of a token
is the number of tokens the request's cache held before it
(mlx_lm/models/gpt2.py:137-144).  The add is fused into the embedding kernel.
``NoPosition``: nothing is added and nothing is rotated.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import MATRIX, Init, ParamSpec, PositionEncoding, register_part


class LearnedAbsolute(PositionEncoding):
    replayable = True
    def __init__(self, name: str, n_positions: int, width: int, init: Init = Init()):
        self.name, self.n_positions, self.width, self.init = name, n_positions, width, init
        self.max_positions = n_positions
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.name + ".weight", (self.n_positions, self.width), MATRIX, self.init)]

    def bind(self, tensors, dtype, device) -> None:
        self.table = tensors[self.name + ".weight"]

    def embedding_table(self):
        return self.table


class NoPosition(PositionEncoding):
    replayable = True
    max_positions = None


class Sinusoidal(PositionEncoding):
    """A fixed sinusoid of the position added to the token embedding: column ``2i`` gets
    ``sin(p * base**(-2i / width))`` and column ``2i + 1`` the cosine of the same angle.  No tensors.  The
    frequencies are rounded to float32 once, here; the angle is a float32 product and the sum is float32, formed
    in the embedding kernel."""
    replayable = True
    max_positions = None

    def __init__(self, width: int, base: float = 10000.0):
        self.width, self.base = width, float(base)
        self.freq: Optional[torch.Tensor] = None

    def bind(self, tensors, dtype, device) -> None:
        i = torch.arange((self.width + 1) // 2, dtype=torch.float64)
        self.freq = (self.base ** (-2.0 * i / self.width)).to(torch.float32).to(device)

    def embedding_frequencies(self):
        return self.freq


def rotation_frequencies(dims: int, base: float, scaling: Optional[dict] = None):
    """``(frequencies, factor)`` of a rotation of ``dims`` dimensions: pair ``i`` turns by ``p * f_i`` with
    ``f_i = base**(-2i / dims)`` (float64 list), cosine and sine both times ``factor``.  ``scaling`` (``factor``,
    ``original``, ``fast``, ``slow``) stretches the slow pairs for sequences longer than ``original`` positions: with
    ``d(t) = dims * ln(original / (2 pi t)) / (2 ln base)`` (the pair that makes ``t`` turns over ``original``
    positions), ``lo = max(floor(d(fast)), 0)``, ``hi = min(ceil(d(slow)), dims - 1)`` and
    ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, the frequency becomes
    ``f_i / factor * ramp_i + f_i * (1 - ramp_i)`` and cosine and sine are multiplied by ``0.1 ln(factor) + 1``."""
    import math

    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


register_part("position", "learned_absolute", LearnedAbsolute)
register_part("position", "sinusoidal", Sinusoidal)
register_part("position", "none", NoPosition)
