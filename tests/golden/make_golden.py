"""Generates tests/golden/*.npz by running the reference torch implementation on seeded inputs.

Run where the reference checkout is available (it is imported, never copied):

    python tests/golden/make_golden.py --reference /path/to/recurrentgemma-checkout

`recurrentgemma/__init__.py` imports the JAX half of the package, which needs flax; registering an
empty parent package first lets `recurrentgemma.torch` import on a torch-only machine.

Each file holds the reference outputs of one case of tests/cases.py (prefill, then the decode
steps fed with the returned cache) and a checksum of the generated inputs and parameters.
bfloat16 tensors are stored widened to float32, which is exact.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests import cases as C  # noqa: E402


def import_reference(path: str):
  pkg = types.ModuleType("recurrentgemma")
  pkg.__path__ = [os.path.join(path, "recurrentgemma")]
  sys.modules["recurrentgemma"] = pkg
  import recurrentgemma.torch as rg  # pylint: disable=import-outside-toplevel
  from recurrentgemma.torch import layers, modules  # pylint: disable=import-outside-toplevel
  return rg, layers, modules


PARAM_INIT_SEED, PARAM_INIT_WIDTH = 7, 2560


def _np(t):
  # a copy: the reference updates its attention cache in place during later decode steps
  return t.detach().to(torch.float32).numpy().copy()


def run_case(case: C.Case, layers, modules) -> dict:
  dt = case.torch_dtype
  p = C.make_params(case)
  inp = C.make_inputs(case)
  pos = inp["segment_pos"]
  out = {"input_checksum": np.float64(C.checksum({**p, **inp}))}

  with torch.no_grad():
    if case.kind == "blockdiag":
      m = layers.BlockDiagonalLinear(case.lru_width, case.heads, dtype=dt)
      m.load_state_dict({"w": p["rg_lru.input_gate.w"], "b": p["rg_lru.input_gate.b"]})
      out["out"] = _np(m(inp["x"]))

    elif case.kind == "conv1d":
      m = layers.Conv1D(case.lru_width, case.temporal_width, dtype=dt)
      m.load_state_dict({"w": p["conv_1d.w"], "b": p["conv_1d.b"]})
      y, cache = m(inp["x"].clone(), pos)   # the reference masks its input in place
      out["out"], out["cache"] = _np(y), _np(cache)
      for i in range(case.decode_steps):
        y, cache = m(inp[f"x_step{i}"].clone(), C.decode_positions(case, pos, i), cache)
        out[f"out_step{i}"], out[f"cache_step{i}"] = _np(y), _np(cache)

    elif case.kind == "rnn_scan":
      y, h = layers.rnn_scan(inp["x"], inp["a"], pos == 0, inp["h0"])
      out["out"], out["h"] = _np(y), _np(h)

    elif case.kind == "rglru":
      m = layers.RGLRU(case.lru_width, case.heads, dtype=dt)
      m.load_state_dict({k[len("rg_lru."):]: v for k, v in p.items() if k.startswith("rg_lru.")})
      y, h = m(inp["x"], pos, inp["h0"])
      out["out"], out["h"] = _np(y), _np(h)
      assert h.dtype == torch.float32
      for i in range(case.decode_steps):
        y, h = m(inp[f"x_step{i}"], C.decode_positions(case, pos, i), h)
        out[f"out_step{i}"], out[f"h_step{i}"] = _np(y), _np(h)

    elif case.kind == "block":
      m = modules.RecurrentBlock(case.model_width, case.heads, case.lru_width,
                                 case.temporal_width, dtype=dt)
      m.load_state_dict(p)
      y, cache = m(inp["x"], pos)
      out["out"], out["h"], out["cache"] = _np(y), _np(cache.rg_lru_state), _np(cache.conv1d_state)
      for i in range(case.decode_steps):
        y, cache = m(inp[f"x_step{i}"], C.decode_positions(case, pos, i), cache)
        out[f"out_step{i}"] = _np(y)
        out[f"h_step{i}"] = _np(cache.rg_lru_state)
        out[f"cache_step{i}"] = _np(cache.conv1d_state)
    elif case.kind == "rmsnorm":
      m = layers.RMSNorm(case.lru_width, dtype=dt)
      m.load_state_dict(p)
      out["out"] = _np(m(inp["x"]))

    elif case.kind == "residual":
      # the temporal half of ResidualBlock.forward (modules.py:897-902) from its own parts:
      # residual = recurrent_block(temporal_pre_norm(x)) + x
      norm = layers.RMSNorm(case.model_width, dtype=dt)
      norm.load_state_dict({"scale": p["temporal_pre_norm.scale"]})
      m = modules.RecurrentBlock(case.model_width, case.heads, case.lru_width,
                                 case.temporal_width, dtype=dt)
      m.load_state_dict({k: v for k, v in p.items() if not k.startswith("temporal_pre_norm.")})
      y, cache = m(norm(inp["x"]), pos)
      out["out"] = _np(y + inp["x"])
      out["h"], out["cache"] = _np(cache.rg_lru_state), _np(cache.conv1d_state)
      for i in range(case.decode_steps):
        xs = inp[f"x_step{i}"]
        y, cache = m(norm(xs), C.decode_positions(case, pos, i), cache)
        out[f"out_step{i}"] = _np(y + xs)
        out[f"h_step{i}"] = _np(cache.rg_lru_state)
        out[f"cache_step{i}"] = _np(cache.conv1d_state)
    elif case.kind == "attention":
      m = modules.LocalAttentionBlock(case.model_width, case.heads, case.window, dtype=dt)
      m.load_state_dict(p)
      y, cache = m(inp["x"], pos)
      out["out"] = _np(y)
      out["keys"], out["values"] = _np(cache.keys), _np(cache.values)
      out["num_tokens"] = cache.num_tokens.numpy().astype(np.int64)
      for i in range(case.decode_steps):
        y, cache = m(inp[f"x_step{i}"], C.decode_positions(case, pos, i), cache)
        out[f"out_step{i}"] = _np(y)
        out[f"keys_step{i}"], out[f"values_step{i}"] = _np(cache.keys), _np(cache.values)
        out[f"num_tokens_step{i}"] = cache.num_tokens.numpy().astype(np.int64)

    elif case.kind == "resblock_attn":
      from recurrentgemma import common  # pylint: disable=import-outside-toplevel
      m = modules.ResidualBlock(
          width=case.model_width, mlp_expanded_width=case.expanded, num_heads=case.heads,
          attention_window_size=case.window, temporal_block_type=common.TemporalBlockType.ATTENTION,
          dtype=dt)
      m.load_state_dict(p)
      y, cache = m(inp["x"], pos)
      out["out"] = _np(y)
      out["keys"], out["values"] = _np(cache.keys), _np(cache.values)
      for i in range(case.decode_steps):
        y, cache = m(inp[f"x_step{i}"], C.decode_positions(case, pos, i), cache)
        out[f"out_step{i}"] = _np(y)

    elif case.kind == "griffin":
      from recurrentgemma import common  # pylint: disable=import-outside-toplevel
      from recurrentgemma.torch import griffin  # pylint: disable=import-outside-toplevel
      kinds = {"recurrent": common.TemporalBlockType.RECURRENT,
               "attention": common.TemporalBlockType.ATTENTION}
      cfg = common.GriffinConfig(
          vocab_size=case.vocab, width=case.model_width, mlp_expanded_width=case.expanded,
          num_heads=case.heads, block_types=tuple(kinds[k] for k in C.GRIFFIN_BLOCKS),
          embeddings_scale_by_sqrt_dim=True, attention_window_size=case.window,
          logits_soft_cap=C.GRIFFIN_SOFT_CAP, lru_width=case.lru_width)
      m = griffin.Griffin(cfg, gradient_checkpointing=False, dtype=dt)
      m.load_state_dict(p)
      logits, cache = m(inp["tokens"], pos)
      out["logits"] = _np(logits)
      out["h_0"] = _np(cache["blocks.0"].rg_lru_state)
      out["conv_1"] = _np(cache["blocks.1"].conv1d_state)
      out["keys_2"] = _np(cache["blocks.2"].keys)
      tok = torch.argmax(logits[:, -1], dim=-1)
      for i in range(case.decode_steps):
        out[f"tokens_step{i}"] = tok.numpy().astype(np.int64)
        logits, cache = m(tok[:, None], C.decode_positions(case, pos, i), cache)
        out[f"logits_step{i}"] = _np(logits)
        tok = torch.argmax(logits[:, 0], dim=-1)
      out["tokens_final"] = tok.numpy().astype(np.int64)
      out["h_0_final"] = _np(cache["blocks.0"].rg_lru_state)
      out["keys_2_final"] = _np(cache["blocks.2"].keys)

    elif case.kind == "mlp":
      m = modules.MLPBlock(case.model_width, case.expanded, dtype=dt)
      m.load_state_dict({k[len("mlp_block."):]: v for k, v in p.items()})
      out["out"] = _np(m(inp["x"]))

    elif case.kind == "resblock":
      from recurrentgemma import common  # pylint: disable=import-outside-toplevel
      m = modules.ResidualBlock(
          width=case.model_width, mlp_expanded_width=case.expanded, num_heads=case.heads,
          attention_window_size=16, temporal_block_type=common.TemporalBlockType.RECURRENT,
          lru_width=case.lru_width, conv1d_temporal_width=case.temporal_width, dtype=dt)
      m.load_state_dict(p)
      y, cache = m(inp["x"], pos)
      out["out"] = _np(y)
      out["h"], out["cache"] = _np(cache.rg_lru_state), _np(cache.conv1d_state)
      for i in range(case.decode_steps):
        y, cache = m(inp[f"x_step{i}"], C.decode_positions(case, pos, i), cache)
        out[f"out_step{i}"] = _np(y)
        out[f"h_step{i}"] = _np(cache.rg_lru_state)
        out[f"cache_step{i}"] = _np(cache.conv1d_state)
    else:
      raise ValueError(case.kind)
  return out


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--reference", default=os.environ.get("RECURRENTGEMMA_REFERENCE", "reference"),
                  help="path of a recurrentgemma checkout")
  ap.add_argument("--only-missing", action="store_true",
                  help="leave fixtures that already exist untouched")
  args = ap.parse_args()
  _, layers, modules = import_reference(args.reference)
  total = 0
  for case in C.golden_cases():
    path = os.path.join(HERE, case.name + ".npz")
    if args.only_missing and os.path.exists(path):
      continue
    res = run_case(case, layers, modules)
    np.savez_compressed(path, **res)
    total += os.path.getsize(path)
    print(f"{case.name:44s} {os.path.getsize(path)/1024:8.1f} KiB")
  # rnn_param_init (torch/layers.py:194-213) draws from torch's global generator: the fixture pins
  # what a given seed produces, in both dtypes the path runs in.
  path = os.path.join(HERE, "rnn_param_init.npz")
  if not (args.only_missing and os.path.exists(path)):
    res = {}
    for name, dt in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
      torch.manual_seed(PARAM_INIT_SEED)
      res[name] = _np(layers.rnn_param_init(torch.empty(PARAM_INIT_WIDTH, dtype=dt), min_rad=0.9,
                                            max_rad=0.999))
    np.savez_compressed(path, **res)
    total += os.path.getsize(path)
  print(f"total {total/1024:.1f} KiB")


if __name__ == "__main__":
  main()
