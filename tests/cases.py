"""Seeded input generators shared by the golden-vector script and the parity tests.

Every tensor is drawn on the CPU in float32 from its own ``torch.Generator`` (seed derived from
the case name and the tensor name) and then cast, so the golden script (run where the reference
can be imported), the CPU oracle and the CUDA path all see bit-identical inputs.  The golden files
store checksums of these inputs, so a drift of the generator is detected rather than silently
compared against stale outputs.
"""
from __future__ import annotations

import dataclasses
import math
import zlib
from typing import Dict, Optional

import torch


@dataclasses.dataclass(frozen=True)
class Case:
  name: str
  kind: str            # "blockdiag" | "conv1d" | "rglru" | "rnn_scan" | "block" | "rmsnorm" | "residual" | "mlp" | "resblock"
                       # | "attention" | "resblock_attn" | "griffin"
  dtype: str           # "float32" | "bfloat16"
  batch: int
  seq: int
  lru_width: int
  heads: int = 1
  width: int = 0       # block (model) width; 0 -> lru_width
  temporal_width: int = 4
  pos: str = "half"    # segment_pos pattern, see make_segment_pos
  with_h0: bool = False
  decode_steps: int = 2
  expanded: int = 0    # mlp expanded width (kinds "mlp" and "resblock")
  window: int = 0      # attention window size (kind "attention")
  vocab: int = 0       # vocabulary size (kind "griffin")

  @property
  def torch_dtype(self) -> torch.dtype:
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[self.dtype]

  @property
  def model_width(self) -> int:
    return self.width or self.lru_width


def _seed(case_name: str, tensor_name: str) -> int:
  return zlib.crc32(f"{case_name}/{tensor_name}".encode()) & 0x7FFFFFFF


def normal(case: str, name: str, shape, std: float = 1.0, dtype=torch.float32) -> torch.Tensor:
  g = torch.Generator(device="cpu").manual_seed(_seed(case, name))
  return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(dtype)


def uniform(case: str, name: str, shape, lo: float, hi: float) -> torch.Tensor:
  g = torch.Generator(device="cpu").manual_seed(_seed(case, name))
  return torch.rand(shape, generator=g, dtype=torch.float32) * (hi - lo) + lo


def make_a_param(case: str, width: int, dtype=torch.float32) -> torch.Tensor:
  """softplus^-1(-0.5 ln u), u ~ U(0.9^2, 0.999^2): the RG-LRU's ring init (layers.py:194-213)."""
  u = uniform(case, "a_param", (width,), 0.9 ** 2 + 1e-8, 0.999 ** 2 + 1e-8).double()
  a_real = -0.5 * torch.log(u)
  return torch.log(torch.expm1(a_real)).float().to(dtype)


def make_segment_pos(pattern: str, batch: int, seq: int, case: str = "") -> torch.Tensor:
  """int64 [batch, seq] positions; a zero marks the first token of a document."""
  ar = torch.arange(seq, dtype=torch.int64)
  if pattern == "arange":
    pos = ar.repeat(batch, 1)
  elif pattern == "half":
    # The reference tests' pattern (torch/test_utils.py:74-75): two documents per row.
    first = seq // 2
    pos = torch.cat([torch.arange(first), torch.arange(seq - first)]).repeat(batch, 1)
  elif pattern == "padded":
    # Left padding as the sampler produces it (torch/sampler.py:235-238): padded slots hold -1,
    # the first real token holds 0.  Row b is padded by (3*b + 1) % seq slots.
    rows = []
    for b in range(batch):
      pad = (3 * b + 1) % max(seq, 1)
      rows.append(torch.clamp(ar - pad, min=-1))
    pos = torch.stack(rows)
  elif pattern == "multi":
    # Random document lengths, including one-token documents (consecutive zeros) and a
    # document start in each of the last three slots of some row.
    g = torch.Generator(device="cpu").manual_seed(_seed(case, "segment_pos"))
    rows = []
    for b in range(batch):
      starts = torch.rand(seq, generator=g) < 0.12
      starts[0] = True
      if seq >= 3:
        starts[seq - 1 - (b % 3)] = True
      if seq >= 8:
        starts[5] = True
        starts[6] = True
      p = torch.zeros(seq, dtype=torch.int64)
      c = 0
      for t in range(seq):
        c = 0 if bool(starts[t]) else c + 1
        p[t] = c
      rows.append(p)
    pos = torch.stack(rows)
  elif pattern == "noreset":
    # No document start at all (continuation of an earlier chunk): positions begin at 1.
    pos = (ar + 1).repeat(batch, 1)
  else:
    raise ValueError(pattern)
  return pos.contiguous()


from recurrentgemma_b200.synthetic import geometric_segment_pos  # noqa: E402,F401  (re-exported)


GRIFFIN_BLOCKS = ("recurrent", "recurrent", "attention")   # the model's repeating pattern
GRIFFIN_SOFT_CAP = 30.0


def make_griffin_params(case: Case) -> Dict[str, torch.Tensor]:
  """The state_dict of a three-block Griffin (griffin.py:52-80): embedder, blocks.{i}, final_norm."""
  dt = case.torch_dtype
  d, xw = case.model_width, case.expanded
  p = {"embedder.input_embedding": normal(case.name, "embedding", (case.vocab, d),
                                          math.sqrt(1.0 / d), dt),
       "final_norm.scale": normal(case.name, "final_norm_scale", (d,), 0.3, dt)}
  for i, kind in enumerate(GRIFFIN_BLOCKS):
    sub = dataclasses.replace(case, name=f"{case.name}/blocks.{i}",
                              kind="resblock" if kind == "recurrent" else "resblock_attn")
    p.update({f"blocks.{i}.{k}": v for k, v in make_params(sub).items()})
  return p


def make_params(case: Case) -> Dict[str, torch.Tensor]:
  """Parameters named as in the reference state_dict of RecurrentBlock (modules.py:531-560)."""
  if case.kind == "griffin":
    return make_griffin_params(case)
  dt = case.torch_dtype
  e, h, d, w = case.lru_width, case.heads, case.model_width, case.temporal_width
  bw = e // h
  n = case.name
  p = {
      "rg_lru.a_param": make_a_param(n, e, dt),
      "rg_lru.input_gate.w": normal(n, "gate_x_w", (h, bw, bw), math.sqrt(1.0 / bw), dt),
      "rg_lru.input_gate.b": normal(n, "gate_x_b", (h, bw), 0.3, dt),
      "rg_lru.a_gate.w": normal(n, "gate_a_w", (h, bw, bw), math.sqrt(1.0 / bw), dt),
      "rg_lru.a_gate.b": normal(n, "gate_a_b", (h, bw), 0.3, dt),
      "conv_1d.w": normal(n, "conv_w", (w, e), math.sqrt(1.0 / w), dt),
      "conv_1d.b": normal(n, "conv_b", (e,), 0.2, dt),
  }
  if case.kind == "rmsnorm":
    return {"scale": normal(n, "norm_scale", (e,), 0.3, dt)}
  if case.kind in ("attention", "resblock_attn"):
    hd = d // h
    pre = "attention_block." if case.kind == "resblock_attn" else ""
    att = {
        pre + "proj_q.weight": normal(n, "proj_q_w", (d, d), math.sqrt(1.0 / d), dt),
        pre + "proj_k.weight": normal(n, "proj_k_w", (hd, d), math.sqrt(1.0 / d), dt),
        pre + "proj_v.weight": normal(n, "proj_v_w", (hd, d), math.sqrt(1.0 / d), dt),
        pre + "proj_final.weight": normal(n, "proj_final_w", (d, d), math.sqrt(1.0 / d), dt),
        pre + "proj_final.bias": normal(n, "proj_final_b", (d,), 0.1, dt),
    }
    if case.kind == "resblock_attn":
      xw = case.expanded
      att.update({
          "temporal_pre_norm.scale": normal(n, "norm_scale", (d,), 0.3, dt),
          "channel_pre_norm.scale": normal(n, "channel_norm_scale", (d,), 0.3, dt),
          "mlp_block.ffw_up.w": normal(n, "ffw_up_w", (2, d, xw), math.sqrt(1.0 / d), dt),
          "mlp_block.ffw_up.b": normal(n, "ffw_up_b", (2, 1, 1, xw), 0.2, dt),
          "mlp_block.ffw_down.weight": normal(n, "ffw_down_w", (d, xw), math.sqrt(1.0 / xw), dt),
          "mlp_block.ffw_down.bias": normal(n, "ffw_down_b", (d,), 0.1, dt),
      })
    return att
  mlp = {}
  if case.kind in ("mlp", "resblock"):
    xw = case.expanded
    mlp = {
        "mlp_block.ffw_up.w": normal(n, "ffw_up_w", (2, d, xw), math.sqrt(1.0 / d), dt),
        "mlp_block.ffw_up.b": normal(n, "ffw_up_b", (2, 1, 1, xw), 0.2, dt),
        "mlp_block.ffw_down.weight": normal(n, "ffw_down_w", (d, xw), math.sqrt(1.0 / xw), dt),
        "mlp_block.ffw_down.bias": normal(n, "ffw_down_b", (d,), 0.1, dt),
    }
  if case.kind == "mlp":
    return mlp
  if case.kind in ("residual", "resblock"):
    p["temporal_pre_norm.scale"] = normal(n, "norm_scale", (d,), 0.3, dt)
  if case.kind == "resblock":
    p["channel_pre_norm.scale"] = normal(n, "channel_norm_scale", (d,), 0.3, dt)
    p.update(mlp)
    p = {("recurrent_block." + k if k.split(".")[0] in ("rg_lru", "conv_1d") else k): v
         for k, v in p.items()}
  if case.kind in ("block", "residual", "resblock"):
    pre = "recurrent_block." if case.kind == "resblock" else ""
    p.update({
        pre + "linear_y.weight": normal(n, "linear_y_w", (e, d), math.sqrt(1.0 / d), dt),
        pre + "linear_y.bias": normal(n, "linear_y_b", (e,), 0.1, dt),
        pre + "linear_x.weight": normal(n, "linear_x_w", (e, d), math.sqrt(1.0 / d), dt),
        pre + "linear_x.bias": normal(n, "linear_x_b", (e,), 0.1, dt),
        pre + "linear_out.weight": normal(n, "linear_out_w", (d, e), math.sqrt(1.0 / e), dt),
        pre + "linear_out.bias": normal(n, "linear_out_b", (d,), 0.1, dt),
    })
  return p


def make_inputs(case: Case) -> Dict[str, Optional[torch.Tensor]]:
  """Activations, positions, optional initial state and the decode-step tokens of a case."""
  dt = case.torch_dtype
  n = case.name
  if case.kind == "griffin":
    g = torch.Generator(device="cpu").manual_seed(_seed(n, "tokens"))
    return {"tokens": torch.randint(0, case.vocab, (case.batch, case.seq), generator=g),
            "segment_pos": make_segment_pos(case.pos, case.batch, case.seq, n), "h0": None}
  in_width = (case.model_width
              if case.kind in ("block", "residual", "mlp", "resblock", "attention", "resblock_attn")
              else case.lru_width)
  out: Dict[str, Optional[torch.Tensor]] = {
      "x": normal(n, "x", (case.batch, case.seq, in_width), 1.0, dt),
      "segment_pos": make_segment_pos(case.pos, case.batch, case.seq, n),
      "h0": normal(n, "h0", (case.batch, case.lru_width), 0.5) if case.with_h0 else None,
  }
  if case.kind == "rnn_scan":
    a = uniform(n, "a", (case.batch, case.seq, case.lru_width), 0.5, 0.999).to(dt)
    out["a"] = a
  for i in range(case.decode_steps):
    out[f"x_step{i}"] = normal(n, f"x_step{i}", (case.batch, 1, in_width), 1.0, dt)
  return out


def decode_positions(case: Case, segment_pos: torch.Tensor, step: int) -> torch.Tensor:
  """Positions fed to decode step `step`: they continue from the last prefill position."""
  return (segment_pos[:, -1:] + 1 + step).contiguous()


def checksum(tensors: Dict[str, Optional[torch.Tensor]]) -> float:
  s = 0.0
  for k in sorted(tensors):
    t = tensors[k]
    if t is None:
      continue
    s += float(t.double().abs().sum()) + 0.5 * float(t.double().sum())
  return s


def _c(name, kind, dtype, b, t, e, h=1, **kw) -> Case:
  return Case(name=name, kind=kind, dtype=dtype, batch=b, seq=t, lru_width=e, heads=h, **kw)


def golden_cases():
  """The cases whose reference outputs are committed under tests/golden/.

  Shapes follow the reference's own parameterised tests (torch/layers_test.py:96-172,
  torch/modules_test.py:119-159) shrunk where that keeps the fixture small, plus ragged lengths
  and position patterns those tests do not reach.
  """
  cases = []
  for dt in ("float32", "bfloat16"):
    s = "f32" if dt == "float32" else "bf16"
    cases += [
        _c(f"bdl_{s}_128x1", "blockdiag", dt, 2, 8, 128, 1, decode_steps=0),
        _c(f"bdl_{s}_1024x16", "blockdiag", dt, 2, 8, 1024, 16, decode_steps=0),
        _c(f"bdl_{s}_512x2", "blockdiag", dt, 2, 8, 512, 2, decode_steps=0),
        _c(f"conv_{s}_128_w4", "conv1d", dt, 2, 32, 128),
        _c(f"conv_{s}_256_w4_multi", "conv1d", dt, 3, 37, 256, pos="multi"),
        _c(f"conv_{s}_128_w8", "conv1d", dt, 2, 32, 128, temporal_width=8),
        _c(f"conv_{s}_128_w4_t1", "conv1d", dt, 2, 1, 128, pos="arange"),
        _c(f"conv_{s}_128_w4_t2", "conv1d", dt, 2, 2, 128, pos="multi"),
        _c(f"conv_{s}_128_w4_t3", "conv1d", dt, 3, 3, 128, pos="multi"),
        _c(f"conv_{s}_128_w4_pad", "conv1d", dt, 3, 9, 128, pos="padded"),
        _c(f"scan_{s}_128", "rnn_scan", dt, 2, 40, 128, pos="multi", with_h0=True, decode_steps=0),
        _c(f"scan_{s}_128_t1", "rnn_scan", dt, 2, 1, 128, pos="noreset", with_h0=True,
           decode_steps=0),
        _c(f"scan_{s}_128_t1_noh0", "rnn_scan", dt, 2, 1, 128, pos="noreset", decode_steps=0),
        _c(f"rglru_{s}_128x1_t32", "rglru", dt, 2, 32, 128, 1),
        _c(f"rglru_{s}_256x1_t128", "rglru", dt, 2, 128, 256, 1),
        _c(f"rglru_{s}_1024x16_t32", "rglru", dt, 2, 32, 1024, 16),
        _c(f"rglru_{s}_512x2_t131_multi_h0", "rglru", dt, 2, 131, 512, 2, pos="multi",
           with_h0=True),
        _c(f"rglru_{s}_256x1_t7_pad", "rglru", dt, 3, 7, 256, 1, pos="padded"),
        _c(f"block_{s}_128_h1_l128", "block", dt, 2, 64, 128, 1, width=128),
        _c(f"block_{s}_128_h1_l256_multi", "block", dt, 2, 67, 256, 1, width=128, pos="multi"),
        _c(f"block_{s}_256_h8_l256", "block", dt, 2, 64, 256, 8, width=256),
        _c(f"block_{s}_128_h2_l512_pad", "block", dt, 3, 21, 512, 2, width=128, pos="padded"),
        # Row counts are multiples of 64 in the prefill form: ATen's CPU kernels round the
        # bfloat16 rsqrt of RMSNorm once in their vectorised body (as CUDA does and as the oracle
        # does) but twice (sqrt, then reciprocal) in the scalar loop that handles the last
        # n mod 64 elements, so only full vector blocks pin the rounding model exactly.
        _c(f"rmsnorm_{s}_128", "rmsnorm", dt, 2, 32, 128, decode_steps=0),
        _c(f"rmsnorm_{s}_2560", "rmsnorm", dt, 4, 16, 2560, decode_steps=0),
        _c(f"residual_{s}_128_h1_l256_multi", "residual", dt, 2, 64, 256, 1, width=128,
           pos="multi"),
        _c(f"residual_{s}_256_h2_l512", "residual", dt, 4, 48, 512, 2, width=256),
        _c(f"mlp_{s}_128_x384", "mlp", dt, 2, 32, 128, width=128, expanded=384, decode_steps=0),
        _c(f"mlp_{s}_256_x768", "mlp", dt, 2, 33, 256, width=256, expanded=768, decode_steps=0),
        # local attention (modules.py:399-493): window shorter and longer than the sequence,
        # documents inside the window, the model's head dimension of 256
        _c(f"attn_{s}_128_h2_w16", "attention", dt, 2, 40, 128, 2, width=128, window=16, pos="multi"),
        _c(f"attn_{s}_128_h2_w64", "attention", dt, 2, 24, 128, 2, width=128, window=64),
        _c(f"attn_{s}_512_h2_w64", "attention", dt, 2, 80, 512, 2, width=512, window=64),
        # a whole residual block of the attention kind, head dimension 256
        _c(f"resblock_attn_{s}_512_h2_w48", "resblock_attn", dt, 2, 64, 512, 2, width=512,
           window=48, expanded=384, pos="multi"),
        # a three-block Griffin (recurrent, recurrent, attention) from token ids to capped logits,
        # two documents per row, then greedy decode steps that wrap the attention window
        _c(f"griffin_{s}_512_h2_v1024", "griffin", dt, 2, 64, 512, 2, width=512, window=48,
           expanded=768, vocab=1024, decode_steps=3),
        # a whole residual block of the recurrent kind (modules.py:897-911)
        _c(f"resblock_{s}_128_h1_l256_x384", "resblock", dt, 2, 64, 256, 1, width=128,
           expanded=384, pos="multi"),
    ]
  return cases


def case_by_name(name: str) -> Case:
  for c in golden_cases():
    if c.name == name:
      return c
  raise KeyError(name)
