"""Sharding of the recurrent path across the GPUs of one node (one process per GPU).

The recurrence and the Conv1D act per channel and the gate projections are block diagonal, so a
slice of WHOLE heads needs only its own slice of every parameter, of the activations and of both
caches: inside the path there is nothing to communicate.  Two partitions are provided:

  * by heads (`head_range`, `shard_state_dict`, `shard_channels`): rank r owns heads
    [r H / n, (r + 1) H / n); used when H is divisible by the world size (e.g. 16 heads over
    1/2/4/8 GPUs).  `gather_channels` reassembles a [B, T, E / n] output with one all_gather.
  * by batch (`batch_range`): rank r owns rows [r B / n, (r + 1) B / n) and a full copy of the
    parameters; no collective at all.  Used where the head count does not divide (10 heads, 8 GPUs).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

# Parameters of the path whose channel axis is sharded, and which axis that is, by state_dict
# suffix (names of recurrentgemma/torch/modules.py:531-560, layers.py:105-112, 262-278, 409-412).
_HEAD_AXIS = {"input_gate.w": 0, "input_gate.b": 0, "a_gate.w": 0, "a_gate.b": 0}
_CHANNEL_AXIS = {"a_param": 0, "conv_1d.w": 1, "conv_1d.b": 0}


def head_range(num_heads: int, world: int, rank: int) -> Tuple[int, int]:
  """Heads [h0, h1) owned by `rank`; the head count must divide evenly."""
  if world < 1 or not 0 <= rank < world:
    raise ValueError(f"bad rank {rank} of {world}")
  if num_heads % world != 0:
    raise ValueError(
        f"{num_heads} heads do not split over {world} ranks in whole heads; shard by batch instead")
  per = num_heads // world
  return rank * per, (rank + 1) * per


def channel_range(width: int, num_heads: int, world: int, rank: int) -> Tuple[int, int]:
  h0, h1 = head_range(num_heads, world, rank)
  bw = width // num_heads
  return h0 * bw, h1 * bw


def batch_range(batch: int, world: int, rank: int) -> Tuple[int, int]:
  """Rows [b0, b1) owned by `rank`; earlier ranks take the remainder."""
  if world < 1 or not 0 <= rank < world:
    raise ValueError(f"bad rank {rank} of {world}")
  base, rem = divmod(batch, world)
  b0 = rank * base + min(rank, rem)
  return b0, b0 + base + (1 if rank < rem else 0)


def shard_state_dict(sd: Dict[str, torch.Tensor], width: int, num_heads: int, world: int,
                     rank: int) -> Dict[str, torch.Tensor]:
  """Slices the RG-LRU / Conv1D entries of a state_dict to this rank's heads: the state_dict of an
  RGLRU, of a Conv1D (bare keys `w` [W, width] and `b` [width]) or of a RecurrentBlock.  Entries
  that are not on the path are returned whole - in particular the block's dense projections
  (`linear_x`, `linear_y`: a head-sharded block needs their output rows sliced, `linear_out` its
  input columns, with a reduction after it), which this function does not attempt.  Raises if
  nothing in the dictionary was recognised, rather than returning it unsliced."""
  h0, h1 = head_range(num_heads, world, rank)
  e0, e1 = channel_range(width, num_heads, world, rank)
  out = {}
  hits = 0
  for name, t in sd.items():
    sliced = t
    for suffix, axis in _HEAD_AXIS.items():
      if name.endswith(suffix):
        sliced = t.narrow(axis, h0, h1 - h0)
        hits += 1
    for suffix, axis in _CHANNEL_AXIS.items():
      if name.endswith(suffix):
        sliced = t.narrow(axis, e0, e1 - e0)
        hits += 1
    # a Conv1D's own state_dict: w [W, width], b [width]
    if name == "w" and t.ndim == 2 and t.shape[1] == width:
      sliced = t.narrow(1, e0, e1 - e0)
      hits += 1
    if name == "b" and t.ndim == 1 and t.shape[0] == width:
      sliced = t.narrow(0, e0, e1 - e0)
      hits += 1
    out[name] = sliced.contiguous()
  if sd and hits == 0:
    raise ValueError("no RG-LRU / Conv1D parameter found in the state_dict: nothing was sliced "
                     f"(keys: {sorted(sd)[:6]} ...)")
  return out


def shard_channels(x: torch.Tensor, width: int, num_heads: int, world: int, rank: int
                   ) -> torch.Tensor:
  """This rank's channel slice [..., e0:e1] of an activation or cache tensor, contiguous."""
  e0, e1 = channel_range(width, num_heads, world, rank)
  return x[..., e0:e1].contiguous()


def gather_channels(y_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None
                    ) -> torch.Tensor:
  """Reassembles [..., E / n] slices into [..., E] on every rank (one all_gather; NCCL on GPUs)."""
  world = dist.get_world_size(group)
  if world == 1:
    return y_local
  parts = [torch.empty_like(y_local) for _ in range(world)]
  dist.all_gather(parts, y_local.contiguous(), group=group)
  return torch.cat(parts, dim=-1)
