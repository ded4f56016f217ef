"""Counterpart of recurrentgemma.torch.griffin.Griffin (griffin.py:31-210) on this library.

Same constructor, module tree (`embedder`, `blocks.{i}`, `final_norm`: identical state_dict keys),
forward signature and cache dictionary (`"blocks.{i}"` -> the block's cache), so a reference
checkpoint loads with `load_state_dict` and the reference `Sampler` can drive it.  Inference only.
"""
from __future__ import annotations

import enum
import itertools
from typing import Dict, NamedTuple, Optional, Tuple

import torch
from torch import nn

from recurrentgemma_b200 import layers
from recurrentgemma_b200 import modules


@enum.unique
class TemporalBlockType(enum.Enum):
  """Kind of temporal mixing of a residual block (recurrentgemma/common.py:24-29)."""
  ATTENTION = enum.auto()
  RECURRENT = enum.auto()


class GriffinConfig(NamedTuple):
  """The fields of recurrentgemma/common.py:117-160 that the torch model reads."""
  vocab_size: int
  width: int
  mlp_expanded_width: int
  num_heads: int
  block_types: Tuple[TemporalBlockType, ...]
  embeddings_scale_by_sqrt_dim: bool
  attention_window_size: int
  logits_soft_cap: float
  lru_width: Optional[int] = None

  @property
  def max_cache_length(self) -> int:
    return self.attention_window_size

  @property
  def num_layers(self) -> int:
    return len(self.block_types)

  @classmethod
  def recurrent_gemma_2b(cls, vocab_size: int = 256_000,
                         max_sequence_length: Optional[int] = None) -> "GriffinConfig":
    """The RECURRENT_GEMMA_2B_V1 preset (recurrentgemma/common.py:92-103): 26 blocks in the
    pattern (recurrent, recurrent, attention)."""
    pattern = itertools.cycle([TemporalBlockType.RECURRENT, TemporalBlockType.RECURRENT,
                               TemporalBlockType.ATTENTION])
    window = 2048 if max_sequence_length is None else min(2048, max_sequence_length)
    return cls(vocab_size=vocab_size, width=2560, mlp_expanded_width=3 * 2560, num_heads=10,
               block_types=tuple(itertools.islice(pattern, 26)),
               embeddings_scale_by_sqrt_dim=True, attention_window_size=window,
               logits_soft_cap=30.0, lru_width=2560)


Cache = Dict[str, NamedTuple]


class Griffin(nn.Module):
  """Griffin model (https://arxiv.org/abs/2402.19427) as recurrentgemma/torch/griffin.py builds it.

  `config` may be this module's `GriffinConfig` or the reference's (same field names).
  `gradient_checkpointing` is accepted and ignored: forwards run without autograd."""

  def __init__(self, config, gradient_checkpointing: bool = False, device=None, dtype=None):
    super().__init__()
    self.config = config
    self.gradient_checkpointing = gradient_checkpointing
    self.embedder = modules.Embedder(
        vocab_size=config.vocab_size, embed_dim=config.width,
        scale_by_sqrt_dim=config.embeddings_scale_by_sqrt_dim, device=device, dtype=dtype)
    self.blocks = nn.ModuleList([
        modules.ResidualBlock(
            width=config.width, mlp_expanded_width=config.mlp_expanded_width,
            num_heads=config.num_heads, attention_window_size=config.attention_window_size,
            temporal_block_type=block_type, lru_width=config.lru_width,
            final_w_init_variance_scale=2.0 / len(config.block_types), device=device, dtype=dtype)
        for block_type in config.block_types])
    self.final_norm = layers.RMSNorm(width=config.width, device=device, dtype=dtype)

  def reset_parameters(self) -> None:
    self.embedder.reset_parameters()
    for block in self.blocks:
      block.reset_parameters()
    self.final_norm.reset_parameters()

  @torch.no_grad()
  def forward(self, tokens: torch.Tensor, segment_pos: torch.Tensor,
              cache: Optional[Cache] = None, return_logits: bool = True,
              return_cache: bool = True, inplace_cache: bool = False,
              ) -> Tuple[Optional[torch.Tensor], Optional[Cache]]:
    """tokens [B,T], segment_pos [B,T] -> (logits [B,T,vocab] or None, updated cache or None),
    as recurrentgemma/torch/griffin.py:136-194.  `inplace_cache` (an extension): a decode step
    overwrites the tensors of `cache` and returns the same dictionary, so that a captured CUDA
    graph of the step can be replayed."""
    if not return_logits and not return_cache:
      return None, None
    x = self.embedder.encode(tokens)
    new_cache = {}
    for i, block in enumerate(self.blocks):
      name = f"blocks.{i}"
      block_cache = None if cache is None else cache[name]
      x, new_cache[name] = block(x, segment_pos, block_cache, return_cache, inplace_cache)
    if not return_logits:
      return None, new_cache
    logits = self.embedder.decode(self.final_norm(x), self.config.logits_soft_cap or 0.0)
    if not return_cache:
      return logits, None
    return logits, new_cache

  def init_cache(self, batch_size: int, dtype: torch.dtype, device=None) -> Cache:
    """Empty cache for the model (recurrentgemma/torch/griffin.py:196-210); `device` is an
    extension (the reference creates the cache on the default device)."""
    cache = {}
    for i, block_type in enumerate(self.config.block_types):
      cache[f"blocks.{i}"] = modules.ResidualBlock.init_cache(
          batch_size=batch_size, width=self.config.width, num_heads=self.config.num_heads,
          attention_window_size=self.config.attention_window_size,
          temporal_block_type=block_type, dtype=dtype, lru_width=self.config.lru_width,
          device=device)
    return cache
