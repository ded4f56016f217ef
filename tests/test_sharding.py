"""Host-side sharding logic, on CPU: unit checks plus a world_size-2 gloo run in which every rank
computes its head slice of an RG-LRU (with the CPU oracle standing in for the kernels, which have
no CPU path) and the all_gather of the slices must equal the unsharded result exactly - the
property the multi-GPU path relies on: no information crosses a head boundary."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from recurrentgemma_b200 import sharding
from tests import cases as C


def test_ranges():
  assert sharding.head_range(16, 8, 3) == (6, 8)
  assert sharding.channel_range(4096, 16, 4, 1) == (1024, 2048)
  with pytest.raises(ValueError):
    sharding.head_range(10, 8, 0)            # 2B dims do not split over 8 GPUs by heads
  got = [sharding.batch_range(10, 4, r) for r in range(4)]
  assert got == [(0, 3), (3, 6), (6, 8), (8, 10)]
  assert sharding.batch_range(64, 8, 7) == (56, 64)
  with pytest.raises(ValueError):
    sharding.batch_range(8, 2, 2)


def test_shard_state_dict_shapes():
  case = C.Case("shard_sd", "block", "float32", 1, 4, 512, 4, width=128)
  sd = C.make_params(case)
  s1 = sharding.shard_state_dict(sd, 512, 4, 2, 1)
  assert s1["rg_lru.input_gate.w"].shape == (2, 128, 128)
  assert s1["rg_lru.a_gate.b"].shape == (2, 128)
  assert s1["rg_lru.a_param"].shape == (256,)
  assert s1["conv_1d.w"].shape == (4, 256) and s1["conv_1d.b"].shape == (256,)
  assert s1["linear_x.weight"].shape == sd["linear_x.weight"].shape   # not on the sharded path
  assert torch.equal(s1["rg_lru.a_param"], sd["rg_lru.a_param"][256:])
  assert torch.equal(s1["conv_1d.w"], sd["conv_1d.w"][:, 256:])
  # a Conv1D's own state_dict has bare keys
  bare = sharding.shard_state_dict({"w": sd["conv_1d.w"], "b": sd["conv_1d.b"]}, 512, 4, 2, 0)
  assert torch.equal(bare["w"], sd["conv_1d.w"][:, :256]) and bare["b"].shape == (256,)
  # a dictionary with nothing of the path in it is refused rather than passed through
  with pytest.raises(ValueError):
    sharding.shard_state_dict({"linear_x.weight": sd["linear_x.weight"]}, 512, 4, 2, 0)


def _worker(rank: int, world: int, port: int, out_dir: str):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    from oracle import oracle
    case = C.Case("shard_run", "rglru", "bfloat16", 2, 40, 512, 4, pos="multi", with_h0=True)
    sd = C.make_params(case)
    inp = C.make_inputs(case)
    x, pos, h0 = inp["x"], inp["segment_pos"], inp["h0"]

    def run(p, xs, hs):
      conv, cache = oracle.conv1d(xs, pos, p["conv_1d.w"], p["conv_1d.b"])
      y, h = oracle.rglru(conv, pos, p["rg_lru.a_param"], p["rg_lru.input_gate.w"],
                          p["rg_lru.input_gate.b"], p["rg_lru.a_gate.w"], p["rg_lru.a_gate.b"], hs)
      return y, h, cache

    local = sharding.shard_state_dict(sd, 512, 4, world, rank)
    y_l, h_l, c_l = run(local, sharding.shard_channels(x, 512, 4, world, rank),
                        sharding.shard_channels(h0, 512, 4, world, rank))
    y = sharding.gather_channels(y_l)
    h = sharding.gather_channels(h_l)
    c = sharding.gather_channels(c_l)
    y_ref, h_ref, c_ref = run(sd, x, h0)
    ok = torch.equal(y, y_ref) and torch.equal(h, h_ref) and torch.equal(c, c_ref)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
      f.write("ok" if ok else "mismatch")
  finally:
    dist.destroy_process_group()


def test_head_sharded_run_equals_unsharded_gloo_world2(tmp_path):
  world = 2
  port = 29500 + (os.getpid() % 2000)
  mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
  for r in range(world):
    assert (tmp_path / f"rank{r}.txt").read_text() == "ok"
