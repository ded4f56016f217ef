"""Seeded synthetic inputs of the benchmark workloads (shapes and distributions only; there is no
dataset behind this path).  Shared by bench.py and the tests so that both draw identical tensors."""
from __future__ import annotations

import math

import torch


def geometric_segment_pos(batch: int, seq: int, mean_len: float, seed: int) -> torch.Tensor:
  """int64 [batch, seq] positions of documents with Geometric(1/mean_len) lengths (support >= 1);
  t = 0 starts a document, and a zero marks every document start."""
  g = torch.Generator(device="cpu").manual_seed(seed)
  starts = torch.rand((batch, seq), generator=g) < (1.0 / mean_len)
  starts[:, 0] = True
  idx = torch.arange(seq, dtype=torch.int64).repeat(batch, 1)
  last_start = torch.where(starts, idx, torch.zeros_like(idx)).cummax(dim=1).values
  return (idx - last_start).contiguous()


def ring_a_param(width: int, generator: torch.Generator, dtype=torch.float32) -> torch.Tensor:
  """softplus^-1(-0.5 ln u), u ~ U(0.9^2, 0.999^2): the RG-LRU's initialisation of a_param
  (recurrentgemma torch/layers.py:194-213, 289-291)."""
  u = torch.rand((width,), generator=generator).double() * (0.999 ** 2 - 0.9 ** 2) + 0.9 ** 2
  return torch.log(torch.expm1(-0.5 * torch.log(u))).float().to(dtype)


def rglru_params(width: int, heads: int, generator: torch.Generator, dtype) -> dict:
  """RGLRU state_dict: gate weights ~ N(0, 1/block_width), zero biases, ring a_param."""
  bw = width // heads
  std = math.sqrt(1.0 / bw)
  return {
      "a_param": ring_a_param(width, generator, dtype),
      "input_gate.w": (torch.randn((heads, bw, bw), generator=generator) * std).to(dtype),
      "input_gate.b": torch.zeros((heads, bw), dtype=dtype),
      "a_gate.w": (torch.randn((heads, bw, bw), generator=generator) * std).to(dtype),
      "a_gate.b": torch.zeros((heads, bw), dtype=dtype),
  }
