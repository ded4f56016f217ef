"""Swaps the B200 recurrent path into a reference `recurrentgemma.torch` model.

Two ways, both leaving state_dict keys unchanged (recurrentgemma/torch/modules.py:803-813,
549-560 resolve the classes through module globals at construction time):

  * ``install()`` before building `Griffin`: rebinds `RecurrentBlock` in
    `recurrentgemma.torch.modules` (and `RGLRU` / `Conv1D` in `recurrentgemma.torch.layers`), so
    every recurrent block constructed afterwards is ours.
  * ``convert(model)`` after building (or loading) it: replaces each
    `model.blocks[i].recurrent_block` by a `RecurrentBlock` that shares the same parameters.
  * ``fuse_temporal_residual(model)`` after ``convert``: each residual block with a recurrent block
    computes `recurrent_block(temporal_pre_norm(x)) + x` (recurrentgemma/torch/modules.py:897-902)
    through `modules.recurrent_residual`; its channel norm and MLP stay the reference's.
  * ``fuse_residual_block(model)`` after ``convert``: the whole forward of every residual block
    (recurrentgemma/torch/modules.py:897-911) runs on this library: both norms, the temporal block
    (recurrent, or local attention), the MLP and both residual adds.

The reference package is not a dependency of this library; it is imported only here, on request.
"""
from __future__ import annotations

import types

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


def _residual_forward(self, x, segment_pos, cache=None, return_cache=True):
  """ResidualBlock.forward (recurrentgemma/torch/modules.py:897-911) with the temporal half as one
  library call."""
  residual, cache = b200_modules.recurrent_residual(
      x, segment_pos, self.temporal_pre_norm, self.recurrent_block, cache, return_cache)
  x = self.channel_pre_norm(residual)
  x = self.mlp_block(x)
  return x + residual, cache


def fuse_temporal_residual(model: nn.Module) -> nn.Module:
  """For every converted recurrent residual block: `temporal_pre_norm` becomes a B200 `RMSNorm`
  sharing the same parameter, and `forward` routes the temporal half through
  `modules.recurrent_residual`.  state_dict keys are unchanged.  Returns the model."""
  for block in model.blocks:
    if isinstance(getattr(block, "recurrent_block", None), b200_modules.RecurrentBlock):
      old = block.temporal_pre_norm
      norm = b200_layers.RMSNorm(old.width, old.eps, device="meta", dtype=old.scale.dtype)
      norm.load_state_dict(old.state_dict(), assign=True)
      block.temporal_pre_norm = norm
      block.forward = types.MethodType(_residual_forward, block)
  return model


def _share(new: nn.Module, old: nn.Module) -> nn.Module:
  new.load_state_dict(old.state_dict(), assign=True)
  return new


def _full_residual_forward(self, x, segment_pos, cache=None, return_cache=True):
  """ResidualBlock.forward (recurrentgemma/torch/modules.py:897-911), every step on this library."""
  return b200_modules.residual_block(x, segment_pos, self.temporal_pre_norm, self.temporal_block,
                                     self.channel_pre_norm, self.mlp_block, cache, return_cache)


def fuse_residual_block(model: nn.Module) -> nn.Module:
  """For every residual block: both norms become B200 `RMSNorm`s, the MLP a B200 `MLPBlock` and a
  local attention block a B200 `LocalAttentionBlock` (recurrent blocks were replaced by
  ``convert``), all sharing the existing parameters, and `forward` becomes
  `modules.residual_block`.  state_dict keys are unchanged.  Returns the model."""
  for block in model.blocks:
    if hasattr(block, "attention_block"):
      old = block.attention_block
      if not isinstance(old, b200_modules.LocalAttentionBlock):
        block.attention_block = _share(b200_modules.LocalAttentionBlock(
            old.width, old.num_heads, old.window_size, old.final_w_init_variance_scale,
            device="meta", dtype=old.proj_q.weight.dtype), old)
    elif not isinstance(getattr(block, "recurrent_block", None), b200_modules.RecurrentBlock):
      continue
    for name in ("temporal_pre_norm", "channel_pre_norm"):
      old = getattr(block, name)
      if not isinstance(old, b200_layers.RMSNorm):
        setattr(block, name, _share(
            b200_layers.RMSNorm(old.width, old.eps, device="meta", dtype=old.scale.dtype), old))
    old = block.mlp_block
    if not isinstance(old, b200_modules.MLPBlock):
      block.mlp_block = _share(b200_modules.MLPBlock(
          old.width, old.expanded_width, old.final_w_init_variance_scale, device="meta",
          dtype=old.ffw_down.weight.dtype), old)
    block.forward = types.MethodType(_full_residual_forward, block)
  return model
