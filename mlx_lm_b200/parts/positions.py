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


register_part("position", "learned_absolute", LearnedAbsolute)
register_part("position", "sinusoidal", Sinusoidal)
register_part("position", "none", NoPosition)
