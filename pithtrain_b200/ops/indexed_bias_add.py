"""``x + bias[group_ids]`` with the call signature of the reference (pithtrain/operators/indexed_bias_add.py:115-127).

The reference passes the group id of every row and the cumulative *end* offsets of the groups; the operator of this
package (:func:`pithtrain_b200.ops.activations.indexed_bias_add`) takes ``offs[E+1]`` starting at zero, from which
the group ids follow, so ``group_ids`` is only checked for its length here.
"""
from __future__ import annotations

import torch

from .activations import indexed_bias_add as _indexed_bias_add

__all__ = ["indexed_bias_add"]


def indexed_bias_add(x: torch.Tensor, bias: torch.Tensor, group_ids: torch.Tensor, grouped_mm_offs: torch.Tensor) -> torch.Tensor:
    assert group_ids.numel() == x.shape[0], "one group id per row"
    ends = grouped_mm_offs.to(torch.int32)
    offs = torch.cat([ends.new_zeros(1), ends])
    return _indexed_bias_add(x, bias, offs)
