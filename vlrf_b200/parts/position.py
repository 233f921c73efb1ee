"""Position encodings.

A position encoding acts at one of two places and says which through `where`:
  "embedding"  it is added to the token embedding (learned absolute positions do this)
  "qk"         it transforms queries and keys inside a mixer (rotary encodings would do this)
The step gives every token its position, so an encoding never counts tokens itself.
"""
from __future__ import annotations

import torch

from .registry import register_part


@register_part("position", "learned_absolute")
class LearnedAbsolutePositions:
    """x[t] += table[position[t]] (reference: include/model/transformer.hpp:350-361).  The table's
    row count bounds the length of a sequence."""

    where = "embedding"

    def __init__(self, table: torch.Tensor):
        if table.dim() != 2:
            raise ValueError("LearnedAbsolutePositions: the table is [positions, width]")
        self.table = table
        self.max_positions = table.shape[0]
