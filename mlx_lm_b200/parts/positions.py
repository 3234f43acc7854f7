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


register_part("position", "learned_absolute", LearnedAbsolute)
register_part("position", "none", NoPosition)
