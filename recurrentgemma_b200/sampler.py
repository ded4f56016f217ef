"""Greedy sampling loop of recurrentgemma.torch.sampler.Sampler (sampler.py:70-420) on token ids.

The reference's sampler tokenises strings with a SentencePiece vocabulary and then runs
`_prompt_processing_fn` (prefill of all prompt tokens but the last, one step for the last) and
`_sample_fn` (a Python `while` that syncs with the device every token to test for EOS).  This
module is the numeric part of that loop on token ids: the same positions, the same split of the
prompt, argmax on the device, and no host synchronisation inside the loop - the decode step
(embedding, 26 residual blocks, final norm, logits, argmax) is captured once as a CUDA graph and
replayed, with the caches updated in place.  Strings, chat formatting and the vocabulary stay with
the reference `Sampler`, which can drive a `recurrentgemma_b200.Griffin` unchanged.
"""
from __future__ import annotations

from typing import NamedTuple, Optional

import torch

from recurrentgemma_b200 import _lib
from recurrentgemma_b200 import modules


class SamplerOutput(NamedTuple):
  """tokens [B, total_generation_steps] int32; logits [B, steps, vocab] or None."""
  tokens: torch.Tensor
  logits: Optional[torch.Tensor]


class GreedySampler:
  """`Sampler(model, vocab, greedy_sampling=True)` of the reference, for prompts given as ids."""

  def __init__(self, model, eos_id: Optional[int] = None, pad_id: int = 0,
               use_cuda_graph: bool = True):
    self.model = model
    self.eos_id = eos_id
    self.pad_id = pad_id
    self.use_cuda_graph = use_cuda_graph
    self._state = None
    self._graph = None
    self._graph_key = None

  @property
  def dtype(self) -> torch.dtype:
    return next(self.model.parameters()).dtype

  @property
  def device(self) -> torch.device:
    return next(self.model.parameters()).device

  def positions(self, prompt_length: int, input_lengths: torch.Tensor) -> torch.Tensor:
    """Positions of left-padded prompts (recurrentgemma/torch/sampler.py:253-256): padding gets
    -1, the last prompt token input_length - 1."""
    pos = torch.arange(prompt_length, device=self.device, dtype=torch.int32)[None]
    pos = pos - prompt_length + input_lengths.to(self.device, torch.int32)[:, None]
    return torch.clip(pos, min=-1)

  def _captured_step(self, b: int, cache):
    """Static buffers for a batch of b sequences and the CUDA graph of one step on them, made on
    first use and kept; `cache` (a model cache holding the prompt) is copied into the buffers."""
    dev = self.device
    if self._graph_key != (b, dev):
      state = {"last_token": torch.zeros((b, 1), dtype=torch.int32, device=dev),
               "next_token": torch.zeros((b, 1), dtype=torch.int32, device=dev),
               "positions": torch.zeros((b, 1), dtype=torch.int32, device=dev),
               "cache": _own(cache), "logits": None}
      # one eager step creates every lazily made buffer of a decode step; capturing then records
      # the launches without running them
      self._step(state)
      graph = torch.cuda.CUDAGraph()
      torch.cuda.synchronize(dev)
      with torch.cuda.graph(graph):
        self._step(state)
      self._state, self._graph, self._graph_key = state, graph, (b, dev)
    for name, c in cache.items():
      for dst, src in zip(self._state["cache"][name], c):
        dst.copy_(src)
    return self._state, self._graph

  def _step(self, state) -> None:
    """One sampling step (recurrentgemma/torch/sampler.py:137-187) on static buffers: reads
    `last_token` and `positions`, updates the cache in place, writes `next_token`, `logits`."""
    logits, _ = self.model(state["last_token"], state["positions"], state["cache"],
                           return_logits=True, return_cache=True, inplace_cache=True)
    state["logits"] = logits
    state["next_token"].copy_(modules.argmax(logits[:, 0])[:, None])
    state["last_token"].copy_(state["next_token"])
    state["positions"].add_(1)

  @torch.no_grad()
  def __call__(self, tokens: torch.Tensor, total_generation_steps: int,
               input_lengths: Optional[torch.Tensor] = None,
               return_logits: bool = False, check_status: bool = False) -> SamplerOutput:
    """tokens [B, prompt_length] (left padded; `input_lengths` [B] gives the true lengths,
    default: no padding).  Generates `total_generation_steps` tokens per sequence greedily.
    Sequences that produce `eos_id` keep running (the reference stops the whole batch only when
    every sequence is done); positions after the first EOS are overwritten with `pad_id`.
    The call enqueues the whole generation and returns without synchronising; with
    `check_status` it waits for the device at the end and raises if a kernel gave up on a bounded
    wait (the tokens are then invalid) - otherwise call `recurrentgemma_b200.check_status()` where
    the host synchronises next."""
    dev = self.device
    tokens = tokens.to(dev)
    b, prompt_length = tokens.shape
    if input_lengths is None:
      input_lengths = torch.full((b,), prompt_length, dtype=torch.int32, device=dev)
    pos = self.positions(prompt_length, input_lengths)
    out_tokens = torch.full((b, total_generation_steps), self.pad_id, dtype=torch.int32, device=dev)
    out_logits = None
    if total_generation_steps == 0:
      return SamplerOutput(out_tokens, out_logits)
    # the prompt: all tokens but the last fill the cache, the last one yields the first logits
    if prompt_length == 1:
      logits, cache = self.model(tokens, pos, None, return_logits=True, return_cache=True)
    else:
      _, cache = self.model(tokens[:, :-1], pos[:, :-1], None, return_logits=False,
                            return_cache=True)
      cache = _own(cache)
      logits, cache = self.model(tokens[:, -1:], pos[:, -1:], cache, return_logits=True,
                                 return_cache=True, inplace_cache=True)
    if return_logits:
      out_logits = torch.zeros((b, total_generation_steps, logits.shape[-1]), dtype=logits.dtype,
                               device=dev)
      out_logits[:, 0] = logits[:, 0]
    first = modules.argmax(logits[:, 0])
    out_tokens[:, 0] = first
    graph = None
    if self.use_cuda_graph and total_generation_steps > 1:
      state, graph = self._captured_step(b, cache)
      state["last_token"].copy_(first[:, None])
      state["positions"].copy_(pos[:, -1:] + 1)
    else:
      state = {"last_token": first[:, None].clone(),
               "next_token": torch.empty((b, 1), dtype=torch.int32, device=dev),
               "positions": (pos[:, -1:] + 1).contiguous(), "cache": _own(cache), "logits": None}
    for step in range(1, total_generation_steps):
      if graph is None:
        self._step(state)
      else:
        graph.replay()
      out_tokens[:, step] = state["next_token"][:, 0]
      if return_logits:
        out_logits[:, step] = state["logits"][:, 0]
    if self.eos_id is not None:
      done = torch.cumsum((out_tokens == self.eos_id).int(), dim=1)
      after = (done - (out_tokens == self.eos_id).int()) > 0
      out_tokens = torch.where(after, torch.full_like(out_tokens, self.pad_id), out_tokens)
    if check_status:
      _lib.check_status(dev)
    return SamplerOutput(out_tokens, out_logits)


def _own(cache):
  """A cache whose tensors are contiguous and not shared with anything else, so that steps may
  overwrite them."""
  return {name: type(c)(*[t.contiguous().clone() for t in c]) for name, c in cache.items()}
