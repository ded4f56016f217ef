"""The recurrent sub-path for callers whose activations live in (pinned) host memory.

Batch rows never interact on this path, so a batch is streamed row-group by row-group through
three CUDA streams: while group i is computed, group i+1 is copied host->device and group i-1 is
copied device->host.  PCIe moves both directions at once, so the wall time of a step approaches the
larger of the two copy times instead of their sum plus the compute.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from recurrentgemma_b200 import _lib
from recurrentgemma_b200 import layers
from recurrentgemma_b200 import modules


class HostPipeline:
  """Reusable device staging buffers and streams for `recurrent_path` on host tensors."""

  def __init__(self, conv_1d: layers.Conv1D, rg_lru: layers.RGLRU, seq_len: int,
               rows_per_group: int = 1, device: Optional[torch.device] = None):
    self.conv_1d, self.rg_lru = conv_1d, rg_lru
    self.device = device or conv_1d.w.device
    self.rows = rows_per_group
    e, dt = rg_lru.width, conv_1d.w.dtype
    shape = (rows_per_group, seq_len, e)
    self.slots = []
    with torch.cuda.device(self.device):
      for _ in range(2):
        self.slots.append({
            "x": torch.empty(shape, dtype=dt, device=self.device),
            "y": torch.empty(shape, dtype=dt, device=self.device),
            "o": torch.empty(shape, dtype=dt, device=self.device),
            "in_done": torch.cuda.Event(), "cmp_done": torch.cuda.Event(),
            "out_done": torch.cuda.Event(),
        })
      self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))

  @torch.no_grad()
  def __call__(self, xb_host: torch.Tensor, yb_host: torch.Tensor, segment_pos: torch.Tensor,
               out_host: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """out_host <- RGLRU(Conv1D(xb)) * gelu(yb) for pinned host tensors [B,T,E]; segment_pos is a
    device tensor [B,T].  Returns (rg_lru_state [B,E] float32, conv1d_state [B,3,E]) on the device.
    The call returns once out_host is complete."""
    b = xb_host.shape[0]
    assert b % self.rows == 0, "batch must be a multiple of rows_per_group"
    assert xb_host.is_pinned() and yb_host.is_pinned() and out_host.is_pinned()
    e = self.rg_lru.width
    with torch.cuda.device(self.device):
      h_all = torch.empty((b, e), dtype=torch.float32, device=self.device)
      c_all = torch.empty((b, 3, e), dtype=xb_host.dtype, device=self.device)
      start = torch.cuda.Event()
      start.record(torch.cuda.current_stream(self.device))
      for st in (self.s_in, self.s_cmp, self.s_out):
        st.wait_event(start)
      for i, r0 in enumerate(range(0, b, self.rows)):
        slot = self.slots[i % 2]
        r1 = r0 + self.rows
        with torch.cuda.stream(self.s_in):
          if i >= 2:
            self.s_in.wait_event(slot["cmp_done"])      # inputs of group i-2 have been consumed
          slot["x"].copy_(xb_host[r0:r1], non_blocking=True)
          slot["y"].copy_(yb_host[r0:r1], non_blocking=True)
          slot["in_done"].record(self.s_in)
        with torch.cuda.stream(self.s_cmp):
          self.s_cmp.wait_event(slot["in_done"])
          if i >= 2:
            self.s_cmp.wait_event(slot["out_done"])     # output buffer of group i-2 has left
          _, cache = modules.recurrent_path(slot["x"], slot["y"], segment_pos[r0:r1], self.conv_1d,
                                            self.rg_lru, out=slot["o"])
          h_all[r0:r1].copy_(cache.rg_lru_state)
          c_all[r0:r1].copy_(cache.conv1d_state)
          slot["cmp_done"].record(self.s_cmp)
        with torch.cuda.stream(self.s_out):
          self.s_out.wait_event(slot["cmp_done"])
          out_host[r0:r1].copy_(slot["o"], non_blocking=True)
          slot["out_done"].record(self.s_out)
      cur = torch.cuda.current_stream(self.device)
      cur.wait_stream(self.s_cmp)
      cur.wait_stream(self.s_out)
      self.s_out.synchronize()
    # the host is synchronised here anyway: a bounded device wait that gave up must not go unseen
    _lib.check_status(self.device)
    return h_all, c_all
