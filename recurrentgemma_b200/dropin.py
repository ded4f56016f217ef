"""Swaps the B200 recurrent path into a reference `recurrentgemma.torch` model.

Two ways, both leaving state_dict keys unchanged (recurrentgemma/torch/modules.py:803-813,
549-560 resolve the classes through module globals at construction time):

  * ``install()`` before building `Griffin`: rebinds `RecurrentBlock` in
    `recurrentgemma.torch.modules` (and `RGLRU` / `Conv1D` in `recurrentgemma.torch.layers`), so
    every recurrent block constructed afterwards is ours.
  * ``convert(model)`` after building (or loading) it: replaces each
    `model.blocks[i].recurrent_block` by a `RecurrentBlock` that shares the same parameters.

The reference package is not a dependency of this library; it is imported only here, on request.
"""
from __future__ import annotations

import torch
from torch import nn

from recurrentgemma_b200 import layers as b200_layers
from recurrentgemma_b200 import modules as b200_modules


def install() -> None:
  """Rebinds the reference's class names to the B200 implementations."""
  from recurrentgemma.torch import layers as ref_layers  # pylint: disable=import-outside-toplevel
  from recurrentgemma.torch import modules as ref_modules  # pylint: disable=import-outside-toplevel
  ref_layers.RGLRU = b200_layers.RGLRU
  ref_layers.Conv1D = b200_layers.Conv1D
  ref_layers.BlockDiagonalLinear = b200_layers.BlockDiagonalLinear
  ref_layers.rnn_scan = b200_layers.rnn_scan
  ref_modules.RecurrentBlock = b200_modules.RecurrentBlock
  ref_modules.RecurrentBlockCache = b200_modules.RecurrentBlockCache


def from_reference(block: nn.Module) -> b200_modules.RecurrentBlock:
  """Builds a B200 `RecurrentBlock` that shares the parameters of a reference one."""
  p = block.linear_x.weight
  new = b200_modules.RecurrentBlock(
      width=block.width, num_heads=block.num_heads, lru_width=block.lru_width,
      conv1d_temporal_width=block.conv1d_temporal_width,
      final_w_init_variance_scale=block.final_w_init_variance_scale, device="meta", dtype=p.dtype)
  new.load_state_dict(block.state_dict(), assign=True)
  return new


def convert(model: nn.Module) -> nn.Module:
  """Replaces every `recurrent_block` of a reference `Griffin` in place; returns the model."""
  for block in model.blocks:
    if hasattr(block, "recurrent_block"):
      block.recurrent_block = from_reference(block.recurrent_block)
  return model
