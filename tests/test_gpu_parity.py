"""Parity of the CUDA path (through the drop-in modules, hence through the C ABI of librgk.so)
with the reference-generated golden vectors and with the CPU oracle.  Needs a B200."""
import pytest
import torch

from tests import cases as C
from tests.util import TOL, assert_close, load_golden

pytestmark = pytest.mark.gpu

CASES = C.golden_cases()
DEV = "cuda:0"


def _cuda(d):
  return {k: (None if v is None else v.to(DEV)) for k, v in d.items()}


@pytest.fixture(scope="module")
def rg():
  import recurrentgemma_b200 as m
  from recurrentgemma_b200 import _lib
  _lib.load()
  return m


@pytest.fixture(autouse=True)
def _library_gemm_at_every_size(request, monkeypatch):
  """The modules hand contractions of fewer than `modules.SMALL_M` rows to library GEMMs (decode
  steps); the fixtures are small, so the tests lower that bound to reach this library's GEMM
  kernels - except the sampler test, which keeps the default and so covers the other route."""
  if not request.node.name.startswith("test_greedy_sampler"):
    from recurrentgemma_b200 import modules
    monkeypatch.setattr(modules, "SMALL_M", 1)


def _block(rg, case, p):
  m = rg.RecurrentBlock(case.model_width, case.heads, case.lru_width, case.temporal_width,
                        device=DEV, dtype=case.torch_dtype)
  m.load_state_dict(p)
  return m


def _griffin(rg, case, p):
  kinds = {"recurrent": rg.TemporalBlockType.RECURRENT, "attention": rg.TemporalBlockType.ATTENTION}
  cfg = rg.GriffinConfig(
      vocab_size=case.vocab, width=case.model_width, mlp_expanded_width=case.expanded,
      num_heads=case.heads, block_types=tuple(kinds[k] for k in C.GRIFFIN_BLOCKS),
      embeddings_scale_by_sqrt_dim=True, attention_window_size=case.window,
      logits_soft_cap=C.GRIFFIN_SOFT_CAP, lru_width=case.lru_width)
  m = rg.Griffin(cfg, device=DEV, dtype=case.torch_dtype)
  m.load_state_dict(p)
  return m


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_golden(case, rg, oracle):
  g = load_golden(case.name)
  p = C.make_params(case)
  inp = C.make_inputs(case)
  assert abs(C.checksum({**p, **inp}) - float(g["input_checksum"])) <= 1e-6 * abs(
      float(g["input_checksum"]))
  tol = TOL[case.torch_dtype]
  pc, ic = _cuda(p), _cuda(inp)
  pos = ic["segment_pos"]

  def chk(out, key):
    assert_close(out, g[key], tol, f"{case.name}:{key}")

  if case.kind == "blockdiag":
    m = rg.BlockDiagonalLinear(case.lru_width, case.heads, device=DEV, dtype=case.torch_dtype)
    m.load_state_dict({"w": p["rg_lru.input_gate.w"], "b": p["rg_lru.input_gate.b"]})
    chk(m(ic["x"]), "out")

  elif case.kind == "conv1d":
    m = rg.Conv1D(case.lru_width, case.temporal_width, device=DEV, dtype=case.torch_dtype)
    m.load_state_dict({"w": p["conv_1d.w"], "b": p["conv_1d.b"]})
    if case.temporal_width != 4:
      with pytest.raises(NotImplementedError):
        m(ic["x"], pos)
      return
    x_before = ic["x"].clone()
    y, cache = m(ic["x"], pos)
    assert torch.equal(ic["x"], x_before), "the input must not be modified"
    chk(y, "out"); chk(cache, "cache")
    assert cache.dtype == case.torch_dtype and cache.shape == (case.batch, 3, case.lru_width)
    for i in range(case.decode_steps):
      y, cache = m(ic[f"x_step{i}"], C.decode_positions(case, inp["segment_pos"], i).to(DEV), cache)
      chk(y, f"out_step{i}"); chk(cache, f"cache_step{i}")

  elif case.kind == "rnn_scan":
    y, h = rg.rnn_scan(ic["x"], ic["a"], pos == 0, ic["h0"])
    chk(y, "out"); chk(h, "h")
    assert h.dtype == torch.float32

  elif case.kind == "rglru":
    m = rg.RGLRU(case.lru_width, case.heads, device=DEV, dtype=case.torch_dtype)
    m.load_state_dict({k[len("rg_lru."):]: v for k, v in p.items() if k.startswith("rg_lru.")})
    y, h = m(ic["x"], pos, ic["h0"])
    chk(y, "out"); chk(h, "h")
    assert h.dtype == torch.float32
    for i in range(case.decode_steps):
      y, h = m(ic[f"x_step{i}"], C.decode_positions(case, inp["segment_pos"], i).to(DEV), h)
      chk(y, f"out_step{i}"); chk(h, f"h_step{i}")
    y2, none = m(ic["x"], pos, ic["h0"], return_cache=False)
    assert none is None
    assert_close(y2, g["out"], tol, "return_cache=False")

  elif case.kind == "block":
    m = _block(rg, case, p)
    y, cache = m(ic["x"], pos)
    assert isinstance(cache, rg.RecurrentBlockCache)
    assert cache._fields == ("rg_lru_state", "conv1d_state")
    chk(y, "out"); chk(cache.rg_lru_state, "h"); chk(cache.conv1d_state, "cache")
    for i in range(case.decode_steps):
      y, cache = m(ic[f"x_step{i}"], C.decode_positions(case, inp["segment_pos"], i).to(DEV), cache)
      chk(y, f"out_step{i}"); chk(cache.rg_lru_state, f"h_step{i}")
      chk(cache.conv1d_state, f"cache_step{i}")
    y3, none = m(ic["x"], pos, return_cache=False)
    assert none is None
    assert_close(y3, g["out"], tol, "return_cache=False")

  elif case.kind == "rmsnorm":
    m = rg.RMSNorm(case.lru_width, device=DEV, dtype=case.torch_dtype)
    m.load_state_dict(p)
    chk(m(ic["x"]), "out")

  elif case.kind == "residual":
    norm = rg.RMSNorm(case.model_width, device=DEV, dtype=case.torch_dtype)
    norm.load_state_dict({"scale": p["temporal_pre_norm.scale"]})
    m = _block(rg, case, {k: v for k, v in p.items() if not k.startswith("temporal_pre_norm.")})
    y, cache = rg.recurrent_residual(ic["x"], pos, norm, m)
    chk(y, "out"); chk(cache.rg_lru_state, "h"); chk(cache.conv1d_state, "cache")
    for i in range(case.decode_steps):
      y, cache = rg.recurrent_residual(ic[f"x_step{i}"],
                                       C.decode_positions(case, inp["segment_pos"], i).to(DEV),
                                       norm, m, cache)
      chk(y, f"out_step{i}"); chk(cache.rg_lru_state, f"h_step{i}")
      chk(cache.conv1d_state, f"cache_step{i}")

  elif case.kind == "attention":
    m = rg.LocalAttentionBlock(case.model_width, case.heads, case.window, device=DEV,
                               dtype=case.torch_dtype)
    m.load_state_dict(p)
    y, cache = m(ic["x"], pos)
    assert cache._fields == ("keys", "values", "num_tokens")
    chk(y, "out"); chk(cache.keys, "keys"); chk(cache.values, "values")
    assert torch.equal(cache.num_tokens.cpu().long(), torch.from_numpy(g["num_tokens"]))
    assert cache.num_tokens.dtype == torch.int32
    for i in range(case.decode_steps):
      y, cache = m(ic[f"x_step{i}"], C.decode_positions(case, inp["segment_pos"], i).to(DEV), cache)
      chk(y, f"out_step{i}"); chk(cache.keys, f"keys_step{i}"); chk(cache.values, f"values_step{i}")
      assert torch.equal(cache.num_tokens.cpu().long(), torch.from_numpy(g[f"num_tokens_step{i}"]))

  elif case.kind == "resblock_attn":
    dt = case.torch_dtype
    tn = rg.RMSNorm(case.model_width, device=DEV, dtype=dt)
    tn.load_state_dict({"scale": p["temporal_pre_norm.scale"]})
    cn = rg.RMSNorm(case.model_width, device=DEV, dtype=dt)
    cn.load_state_dict({"scale": p["channel_pre_norm.scale"]})
    att = rg.LocalAttentionBlock(case.model_width, case.heads, case.window, device=DEV, dtype=dt)
    att.load_state_dict({k[len("attention_block."):]: v for k, v in p.items()
                         if k.startswith("attention_block.")})
    mlp = rg.MLPBlock(case.model_width, case.expanded, device=DEV, dtype=dt)
    mlp.load_state_dict({k[len("mlp_block."):]: v for k, v in p.items()
                         if k.startswith("mlp_block.")})
    y, cache = rg.residual_block(ic["x"], pos, tn, att, cn, mlp)
    chk(y, "out"); chk(cache.keys, "keys"); chk(cache.values, "values")
    for i in range(case.decode_steps):
      y, cache = rg.residual_block(ic[f"x_step{i}"],
                                   C.decode_positions(case, inp["segment_pos"], i).to(DEV),
                                   tn, att, cn, mlp, cache)
      chk(y, f"out_step{i}")

  elif case.kind == "griffin":
    m = _griffin(rg, case, p)
    logits, cache = m(ic["tokens"], pos)
    chk(logits, "logits"); chk(cache["blocks.0"].rg_lru_state, "h_0")
    chk(cache["blocks.1"].conv1d_state, "conv_1"); chk(cache["blocks.2"].keys, "keys_2")
    only_logits, none = m(ic["tokens"], pos, return_cache=False)
    assert none is None and torch.equal(only_logits, logits)
    assert m(ic["tokens"], pos, return_logits=False, return_cache=False) == (None, None)
    # decode steps on the reference's greedy tokens: new tensors per step (the reference's
    # contract), and the in-place form on a private copy of the cache
    from recurrentgemma_b200 import sampler as sampler_lib
    own = sampler_lib._own(cache)
    for i in range(case.decode_steps):
      tok = torch.from_numpy(g[f"tokens_step{i}"])[:, None].to(DEV)
      ps = C.decode_positions(case, inp["segment_pos"], i).to(DEV)
      logits, cache = m(tok, ps, cache)
      chk(logits, f"logits_step{i}")
      logits2, own2 = m(tok, ps, own, inplace_cache=True)
      assert own2["blocks.2"].keys is own["blocks.2"].keys
      assert_close(logits2, g[f"logits_step{i}"], tol, f"in-place logits_step{i}")
    chk(cache["blocks.0"].rg_lru_state, "h_0_final"); chk(cache["blocks.2"].keys, "keys_2_final")
    chk(own["blocks.0"].rg_lru_state, "h_0_final"); chk(own["blocks.2"].keys, "keys_2_final")
    assert torch.equal(own["blocks.2"].num_tokens, cache["blocks.2"].num_tokens)

  elif case.kind == "mlp":
    m = rg.MLPBlock(case.model_width, case.expanded, device=DEV, dtype=case.torch_dtype)
    m.load_state_dict({k[len("mlp_block."):]: v for k, v in p.items()})
    chk(m(ic["x"]), "out")

  elif case.kind == "resblock":
    dt = case.torch_dtype
    tn = rg.RMSNorm(case.model_width, device=DEV, dtype=dt)
    tn.load_state_dict({"scale": p["temporal_pre_norm.scale"]})
    cn = rg.RMSNorm(case.model_width, device=DEV, dtype=dt)
    cn.load_state_dict({"scale": p["channel_pre_norm.scale"]})
    blk = _block(rg, case, {k[len("recurrent_block."):]: v for k, v in p.items()
                            if k.startswith("recurrent_block.")})
    mlp = rg.MLPBlock(case.model_width, case.expanded, device=DEV, dtype=dt)
    mlp.load_state_dict({k[len("mlp_block."):]: v for k, v in p.items()
                         if k.startswith("mlp_block.")})
    y, cache = rg.residual_block(ic["x"], pos, tn, blk, cn, mlp)
    chk(y, "out"); chk(cache.rg_lru_state, "h"); chk(cache.conv1d_state, "cache")
    for i in range(case.decode_steps):
      y, cache = rg.residual_block(ic[f"x_step{i}"],
                                   C.decode_positions(case, inp["segment_pos"], i).to(DEV),
                                   tn, blk, cn, mlp, cache)
      chk(y, f"out_step{i}"); chk(cache.rg_lru_state, f"h_step{i}")
      chk(cache.conv1d_state, f"cache_step{i}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", [(2, 1031, 320), (1, 9000, 64), (3, 257, 72), (1, 5, 8),
                                   (2, 128, 64), (2, 129, 64)],
                         ids=lambda s: "x".join(map(str, s)))
def test_scan_vs_oracle(rg, oracle, dtype, shape):
  """rnn_scan over many tiles (look-back windows of several tiles), ragged T and E, resets, an
  initial state and the fused gelu join, against the oracle."""
  b, t, e = shape
  name = f"scan_{b}_{t}_{e}_{dtype}"
  x = C.normal(name, "x", shape, 1.0, dtype)
  a = C.uniform(name, "a", shape, 0.6, 1.0).to(dtype)
  ym = C.normal(name, "ym", shape, 1.0, dtype)
  h0 = C.normal(name, "h0", (b, e), 0.5)
  reset = C.uniform(name, "reset", (b, t), 0.0, 1.0) < 0.01
  tol = TOL[dtype]
  y_ref, h_ref = oracle.rnn_scan(x, a, reset, h0)
  y, h = rg.rnn_scan(x.to(DEV), a.to(DEV), reset.to(DEV), h0.to(DEV))
  assert_close(y, y_ref, tol, "y"); assert_close(h, h_ref, TOL[torch.float32] * 3, "h")
  y2, _ = rg.rnn_scan(x.to(DEV), a.to(DEV), reset.to(DEV), None, y_mul=ym.to(DEV))
  y_ref2, _ = oracle.rnn_scan(x, a, reset, None)
  assert_close(y2, oracle.gelu_mul(y_ref2, ym), tol, "y*gelu")


@pytest.mark.parametrize("name", ["block_f32_128_h1_l256_multi", "block_bf16_256_h8_l256"])
def test_prefill_state_equals_decode_state(rg, name):
  """State after prefill(T) == state after prefill(T-1) + one decode step (what the sampler relies
  on, recurrentgemma/torch/sampler_test.py:150-230)."""
  case = C.case_by_name(name)
  p = C.make_params(case)
  inp = _cuda(C.make_inputs(case))
  m = _block(rg, case, p)
  x, pos = inp["x"], inp["segment_pos"]
  tol = TOL[case.torch_dtype]
  y_full, c_full = m(x, pos)
  _, c_a = m(x[:, :-1].contiguous(), pos[:, :-1].contiguous())
  y_b, c_b = m(x[:, -1:].contiguous(), pos[:, -1:].contiguous(), c_a)
  keep = (pos[:, -1] != 0).cpu()   # a decode step never starts a document in the sampler
  assert keep.any()
  assert_close(c_b.rg_lru_state.cpu()[keep], c_full.rg_lru_state.cpu()[keep], tol, "state")
  assert_close(y_b.cpu()[keep], y_full[:, -1:].cpu()[keep], tol, "last output")
  assert_close(c_b.conv1d_state.cpu()[keep][:, -1], c_full.conv1d_state.cpu()[keep][:, -1], tol,
               "newest conv row")


def test_full_size_slice_vs_oracle(rg, oracle):
  """The 2B-dims prefill workload (batch 8, 4096 tokens, 2560 channels, 10 heads, bfloat16) at
  full size; channels of different heads and different batch rows never mix, so the oracle checks
  one (row, head) slice of the full-size result."""
  torch.manual_seed(0)
  b, t, e, h = 8, 4096, 2560, 10
  dt = torch.bfloat16
  case = C.Case("full_cfg1", "rglru", "bfloat16", b, t, e, h)
  p = C.make_params(case)
  g = torch.Generator(device="cpu").manual_seed(1234)
  xb = torch.randn((b, t, e), generator=g, dtype=torch.float32).to(dt)
  yb = torch.randn((b, t, e), generator=g, dtype=torch.float32).to(dt)
  pos = C.geometric_segment_pos(b, t, 1024.0, 7)
  conv = rg.Conv1D(e, 4, device=DEV, dtype=dt)
  conv.load_state_dict({"w": p["conv_1d.w"], "b": p["conv_1d.b"]})
  lru = rg.RGLRU(e, h, device=DEV, dtype=dt)
  lru.load_state_dict({k[len("rg_lru."):]: v for k, v in p.items() if k.startswith("rg_lru.")})
  out, cache = rg.recurrent_path(xb.to(DEV), yb.to(DEV), pos.to(DEV), conv, lru)
  from recurrentgemma_b200 import _lib
  _lib.workspace_status(_lib.workspace(torch.device(DEV), 1))
  row, head, bw = 5, 7, 256
  sl = slice(head * bw, (head + 1) * bw)
  op = {
      "conv_w": p["conv_1d.w"][:, sl], "conv_b": p["conv_1d.b"][sl],
      "a_param": p["rg_lru.a_param"][sl],
      "gate_x_w": p["rg_lru.input_gate.w"][head:head + 1],
      "gate_x_b": p["rg_lru.input_gate.b"][head:head + 1],
      "gate_a_w": p["rg_lru.a_gate.w"][head:head + 1],
      "gate_a_b": p["rg_lru.a_gate.b"][head:head + 1],
  }
  o_ref, h_ref, c_ref = oracle.recurrent_path(xb[row:row + 1, :, sl].contiguous(),
                                              yb[row:row + 1, :, sl].contiguous(),
                                              pos[row:row + 1], op)
  assert_close(out[row:row + 1, :, sl], o_ref, TOL[dt], "out slice")
  assert_close(cache.rg_lru_state[row:row + 1, sl], h_ref, TOL[dt], "state slice")
  assert_close(cache.conv1d_state[row:row + 1, :, sl], c_ref, TOL[dt], "conv state slice")


def test_errors(rg):
  """Error behaviour: no CPU path, shape / dtype mismatches raise instead of computing."""
  from recurrentgemma_b200 import _lib
  conv = rg.Conv1D(128, 4, device=DEV, dtype=torch.float32)
  with pytest.raises(RuntimeError):
    conv(torch.zeros(1, 4, 128), torch.zeros(1, 4, dtype=torch.int64))          # CPU tensors
  with pytest.raises(TypeError):
    conv(torch.zeros(1, 4, 128, device=DEV, dtype=torch.bfloat16),
         torch.zeros(1, 4, dtype=torch.int64, device=DEV))                       # dtype mismatch
  with pytest.raises(AssertionError):
    conv(torch.zeros(1, 2, 128, device=DEV), torch.zeros(1, 2, dtype=torch.int64, device=DEV),
         torch.zeros(1, 3, 128, device=DEV))                                     # decode needs T == 1
  lib = _lib.load()
  assert lib.rgk_conv1d_prefill(None, None, 0, None, None, 1, 1, 128, 4, 0, None, None, None) == -1
  assert b"NULL" in lib.rgk_last_error()
  assert lib.rgk_conv1d_prefill(1, 1, 0, 1, 1, 1, 1, 130, 4, 0, 1, None, None) == -2


@pytest.mark.parametrize("shape", [(1, 133, 256, 1), (3, 700, 512, 2), (2, 2048, 2560, 10),
                                   (256, 1, 2560, 10)],
                         ids=lambda s: "x".join(map(str, s)))
def test_gates_tcgen05_matches_simt_and_oracle(rg, oracle, shape):
  """The tensor-core gate kernel against the CUDA-core one (both re-create the reference's
  bfloat16 roundings, so they may differ only where an accumulation-order difference flips a
  rounding) and, on the smaller shapes, against the oracle."""
  from recurrentgemma_b200 import _lib
  b, t, e, h = shape
  case = C.Case(f"tc_{b}_{t}_{e}", "rglru", "bfloat16", b, t, e, h, pos="multi" if t > 8 else "noreset")
  p = C.make_params(case)
  inp = C.make_inputs(case)
  m = rg.RGLRU(e, h, device=DEV, dtype=torch.bfloat16)
  m.load_state_dict({k[len("rg_lru."):]: v for k, v in p.items() if k.startswith("rg_lru.")})
  x, pos = inp["x"].to(DEV), inp["segment_pos"].to(DEV)
  h0 = C.normal(case.name, "h0", (b, e), 0.5).to(DEV)
  m.gates_impl = _lib.GATES_TCGEN05
  y_tc, h_tc = m(x, pos, h0)
  _lib.workspace_status(_lib.workspace(torch.device(DEV), 1))
  m.gates_impl = _lib.GATES_SIMT
  y_si, h_si = m(x, pos, h0)
  assert_close(y_tc, y_si, 5e-3, "tcgen05 vs simt y")
  assert_close(h_tc, h_si, 5e-3, "tcgen05 vs simt h")
  assert float((y_tc != y_si).float().mean()) < 0.02
  if b * t * e <= 3 * 700 * 512:
    y_ref, h_ref = oracle.rglru(inp["x"], inp["segment_pos"], p["rg_lru.a_param"],
                                p["rg_lru.input_gate.w"], p["rg_lru.input_gate.b"],
                                p["rg_lru.a_gate.w"], p["rg_lru.a_gate.b"], h0.cpu())
    assert_close(y_tc, y_ref, TOL[torch.bfloat16], "tcgen05 vs oracle y")
    assert_close(h_tc, h_ref, TOL[torch.bfloat16], "tcgen05 vs oracle h")


@pytest.mark.parametrize("shape", [(256, 2560, 10), (5, 256, 1), (130, 512, 2)],
                         ids=lambda s: "x".join(map(str, s)))
def test_fused_decode_step_matches_unfused_and_oracle(rg, oracle, shape):
  """The single-kernel decode step (conv step + tcgen05 gates + state update + join) against the
  three-kernel CUDA-core path and against the oracle, including rows whose position is 0."""
  from recurrentgemma_b200 import _lib
  b, e, h = shape
  case = C.Case(f"dec_{b}_{e}", "rglru", "bfloat16", b, 1, e, h)
  p = C.make_params(case)
  dt = torch.bfloat16
  conv = rg.Conv1D(e, 4, device=DEV, dtype=dt)
  conv.load_state_dict({"w": p["conv_1d.w"], "b": p["conv_1d.b"]})
  lru = rg.RGLRU(e, h, device=DEV, dtype=dt)
  lru.load_state_dict({k[len("rg_lru."):]: v for k, v in p.items() if k.startswith("rg_lru.")})
  xb = C.normal(case.name, "xb", (b, 1, e), 1.0, dt)
  yb = C.normal(case.name, "yb", (b, 1, e), 1.0, dt)
  h0 = C.normal(case.name, "h0", (b, e), 0.5)
  cc = C.normal(case.name, "cc", (b, 3, e), 1.0, dt)
  pos = torch.randint(0, 3, (b, 1), generator=torch.Generator().manual_seed(3))
  cache = rg.RecurrentBlockCache(rg_lru_state=h0.to(DEV), conv1d_state=cc.to(DEV))
  lru.gates_impl = _lib.GATES_SIMT
  o_u, c_u = rg.recurrent_path(xb.to(DEV), yb.to(DEV), pos.to(DEV), conv, lru, cache)
  tol = TOL[dt]
  # the variant with every rounding of the reference agrees closely with the CUDA-core kernels;
  # the default one (packed-tanh input gate and gelu, table for exp(log_a)) within the parity bar
  lru.gates_impl = _lib.GATES_FUSED_EXACT
  o_e, c_e = rg.recurrent_path(xb.to(DEV), yb.to(DEV), pos.to(DEV), conv, lru, cache)
  assert_close(o_e, o_u, 5e-3, "fused (exact) vs unfused out")
  assert_close(c_e.rg_lru_state, c_u.rg_lru_state, 5e-3, "fused (exact) vs unfused state")
  assert torch.equal(c_e.conv1d_state, c_u.conv1d_state)
  lru.gates_impl = _lib.GATES_AUTO
  o_f, c_f = rg.recurrent_path(xb.to(DEV), yb.to(DEV), pos.to(DEV), conv, lru, cache)
  _lib.workspace_status(_lib.workspace(torch.device(DEV), 1))
  assert_close(o_f, o_u, tol, "fused vs unfused out")
  assert_close(c_f.rg_lru_state, c_u.rg_lru_state, tol, "fused vs unfused state")
  assert torch.equal(c_f.conv1d_state, c_u.conv1d_state)
  op = {"conv_w": p["conv_1d.w"], "conv_b": p["conv_1d.b"], "a_param": p["rg_lru.a_param"],
        "gate_x_w": p["rg_lru.input_gate.w"], "gate_x_b": p["rg_lru.input_gate.b"],
        "gate_a_w": p["rg_lru.a_gate.w"], "gate_a_b": p["rg_lru.a_gate.b"]}
  o_r, h_r, c_r = oracle.recurrent_path(xb, yb, pos, op, h0, cc)
  assert_close(o_f, o_r, tol, "fused vs oracle out")
  assert_close(c_f.rg_lru_state, h_r, tol, "fused vs oracle state")
  assert_close(c_f.conv1d_state, c_r, tol, "fused vs oracle conv cache")
  # no y branch
  lru.gates_impl = _lib.GATES_AUTO
  o_n, _ = rg.recurrent_path(xb.to(DEV), None, pos.to(DEV), conv, lru, cache)
  o_rn, _, _ = oracle.recurrent_path(xb, torch.zeros_like(yb), pos, op, h0, cc)
  y_plain, _ = oracle.rglru(oracle.conv1d(xb, pos, op["conv_w"], op["conv_b"], cc)[0], pos,
                            op["a_param"], op["gate_x_w"], op["gate_x_b"], op["gate_a_w"],
                            op["gate_a_b"], h0)
  assert_close(o_n, y_plain, tol, "fused, no join")


@pytest.mark.parametrize("shape", [(300, 128, 256), (1000, 2560, 2560), (129, 72, 520), (4096, 2560, 2560)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("gelu", [False, True], ids=["plain", "gelu"])
def test_dense_linear_tcgen05(rg, oracle, shape, gelu):
  """The tensor-core nn.Linear (optionally + gelu) against a float32 evaluation of the same
  bfloat16 inputs, and on the small shapes against the oracle (ragged M, K and N included)."""
  m, k, n = shape
  name = f"dense_{m}_{k}_{n}"
  dt = torch.bfloat16
  x = C.normal(name, "x", (m, k), 1.0, dt)
  w = C.normal(name, "w", (n, k), (1.0 / k) ** 0.5, dt)
  b = C.normal(name, "b", (n,), 0.2, dt)
  out = rg.dense_linear(x.to(DEV), w.to(DEV), b.to(DEV), gelu=gelu)
  ref = torch.nn.functional.linear(x.to(DEV).float(), w.to(DEV).float(), b.to(DEV).float())
  ref = ref.to(dt).float()
  if gelu:
    ref = torch.nn.functional.gelu(ref, approximate="tanh")
  assert_close(out, ref.to(dt), TOL[dt], "vs float32 torch")
  assert float((out.float() - ref.to(dt).float()).abs().max()) <= 0.05
  if m * k * n <= 300 * 128 * 256 * 4:
    o_ref = oracle.linear(x, w, b)
    if gelu:
      o_ref = oracle.gelu_mul(torch.ones_like(o_ref), o_ref)
    assert_close(out, o_ref, TOL[dt], "vs oracle")
  out_nb = rg.dense_linear(x.to(DEV), w.to(DEV), None, gelu=gelu)
  ref_nb = torch.nn.functional.linear(x.to(DEV).float(), w.to(DEV).float()).to(dt).float()
  if gelu:
    ref_nb = torch.nn.functional.gelu(ref_nb, approximate="tanh")
  assert_close(out_nb, ref_nb.to(dt), TOL[dt], "no bias")


def test_block_fused_matches_composed(rg):
  """RecurrentBlock prefill through the single fused-block call (tcgen05 projections) against the
  same module composed from torch linears + the sub-path call."""
  from recurrentgemma_b200 import _lib
  case = C.Case("blockfused", "block", "bfloat16", 2, 777, 2560, 10, width=2560, pos="multi")
  p = C.make_params(case)
  inp = _cuda(C.make_inputs(case))
  m = _block(rg, case, p)
  y_f, c_f = m(inp["x"], inp["segment_pos"])
  _lib.workspace_status(_lib.workspace(torch.device(DEV), 1))
  m.rg_lru.gates_impl = _lib.GATES_TCGEN05
  yb = m.linear_y(inp["x"]); xb = m.linear_x(inp["x"])
  z, c_c = rg.recurrent_path(xb, yb, inp["segment_pos"], m.conv_1d, m.rg_lru)
  y_c = m.linear_out(z)
  assert_close(y_f, y_c, TOL[torch.bfloat16], "fused vs composed out")
  assert_close(c_f.rg_lru_state, c_c.rg_lru_state, TOL[torch.bfloat16], "state")
  assert_close(c_f.conv1d_state, c_c.conv1d_state, TOL[torch.bfloat16], "conv state")


@pytest.mark.parametrize("shape", [(1, 128, 256, 1), (2, 384, 512, 2), (1, 8192, 256, 1),
                                   (3, 77, 256, 1), (2, 200, 512, 2), (1, 1001, 256, 1),
                                   (3, 1024, 2560, 10), (37, 384, 512, 2), (40, 256, 512, 2),
                                   (8, 4096, 2560, 10)],
                         ids=lambda s: "x".join(map(str, s)))
def test_fused_rglru_kernel(rg, oracle, shape):
  """Gates + gate arithmetic + scan (+ join) in one tensor-core kernel against the two-kernel
  tensor-core route (same roundings; only the association of the carries differs) and, on the
  smaller shapes, against the oracle.  Covers one unit per sequence, carries inside one round of
  CTAs (B = 1, long T), sequence lengths that end inside a time tile, carries across rounds, and
  workloads with as many (sequence, half head) pairs as SMs or a few more (B = 37 and 40 with two
  heads: the incoming state comes from the same CTA's previous round, or from another CTA's)."""
  from recurrentgemma_b200 import _lib
  b, t, e, h = shape
  case = C.Case(f"fused_{b}_{t}_{e}", "rglru", "bfloat16", b, t, e, h, pos="multi")
  p = C.make_params(case)
  inp = C.make_inputs(case)
  dt = torch.bfloat16
  m = rg.RGLRU(e, h, device=DEV, dtype=dt)
  m.load_state_dict({k[len("rg_lru."):]: v for k, v in p.items() if k.startswith("rg_lru.")})
  conv = rg.Conv1D(e, 4, device=DEV, dtype=dt)
  conv.load_state_dict({"w": p["conv_1d.w"], "b": p["conv_1d.b"]})
  x, pos = inp["x"].to(DEV), inp["segment_pos"].to(DEV)
  h0 = C.normal(case.name, "h0", (b, e), 0.5).to(DEV)
  yb = C.normal(case.name, "yb", (b, t, e), 1.0, dt).to(DEV)
  ws = _lib.workspace(torch.device(DEV), 1)
  m.gates_impl = _lib.GATES_TCGEN05
  y_u, h_u = m(x, pos, h0)
  o_u, c_u = rg.recurrent_path(x, yb, pos, conv, m)
  tol = TOL[dt]
  y_r = None
  if b * t * e <= 8 << 20:
    y_r, h_r = oracle.rglru(inp["x"], inp["segment_pos"], p["rg_lru.a_param"],
                            p["rg_lru.input_gate.w"], p["rg_lru.input_gate.b"],
                            p["rg_lru.a_gate.w"], p["rg_lru.a_gate.b"], h0.cpu())
  # GATES_FUSED_EXACT keeps every rounding of the reference: it must agree with the two-kernel route
  # almost bit for bit.  GATES_FUSED evaluates the input gate and the gelu with packed tanh
  # approximations: it is held to the path's tolerance (against the oracle where that is affordable).
  for impl, cmp_tol, max_mismatch in ((_lib.GATES_FUSED_EXACT, 1e-2, 0.02), (_lib.GATES_FUSED, tol, 0.7)):
    m.gates_impl = impl
    y_f, h_f = m(x, pos, h0)
    _lib.workspace_status(ws)
    o_f, c_f = rg.recurrent_path(x, yb, pos, conv, m)
    _lib.workspace_status(ws)
    assert_close(y_f, y_u, cmp_tol, f"fused ({impl}) vs two-kernel y")
    assert_close(h_f, h_u, cmp_tol, f"fused ({impl}) vs two-kernel h")
    assert_close(o_f, o_u, cmp_tol, f"fused ({impl}) vs two-kernel path out")
    assert_close(c_f.rg_lru_state, c_u.rg_lru_state, cmp_tol, f"fused ({impl}) vs two-kernel path state")
    assert float((y_f != y_u).float().mean()) < max_mismatch
    if y_r is not None:
      assert_close(y_f, y_r, tol, f"fused ({impl}) vs oracle y")
      assert_close(h_f, h_r, tol, f"fused ({impl}) vs oracle h")
  with pytest.raises(_lib.RgkError):      # head width other than 256
    m2 = rg.RGLRU(256, 2, device=DEV, dtype=dt)
    m2.gates_impl = _lib.GATES_FUSED
    m2(torch.zeros(1, 128, 256, device=DEV, dtype=dt), torch.arange(128, device=DEV)[None])


def test_host_pipeline_matches_device_call(rg):
  """The host-buffer pipeline (rows streamed through copy-in / compute / copy-out streams) returns
  what the device-resident call returns."""
  from recurrentgemma_b200 import host
  case = C.Case("hostpipe", "rglru", "bfloat16", 4, 512, 512, 2, pos="multi")
  p = C.make_params(case)
  dt = torch.bfloat16
  conv = rg.Conv1D(512, 4, device=DEV, dtype=dt)
  conv.load_state_dict({"w": p["conv_1d.w"], "b": p["conv_1d.b"]})
  lru = rg.RGLRU(512, 2, device=DEV, dtype=dt)
  lru.load_state_dict({k[len("rg_lru."):]: v for k, v in p.items() if k.startswith("rg_lru.")})
  xb = C.normal(case.name, "xb", (4, 512, 512), 1.0, dt).pin_memory()
  yb = C.normal(case.name, "yb", (4, 512, 512), 1.0, dt).pin_memory()
  pos = C.make_segment_pos("multi", 4, 512, case.name).to(DEV)
  out_h = torch.empty_like(xb).pin_memory()
  pipe = host.HostPipeline(conv, lru, 512, rows_per_group=1)
  for _ in range(2):       # second call reuses the staging buffers
    h_state, c_state = pipe(xb, yb, pos, out_h)
  o_ref, cache = rg.recurrent_path(xb.to(DEV), yb.to(DEV), pos, conv, lru)
  assert_close(out_h, o_ref, 1e-6, "out")
  assert_close(h_state, cache.rg_lru_state, 1e-6, "state")
  assert torch.equal(c_state, cache.conv1d_state)


def test_gate_kernel_repeatable_at_full_size(rg):
  """The tensor-core gate kernel hands each conv-output slice back to the copy engine as soon as
  its epilogue warps have read their values from it; the reads must be complete by then.  Repeated
  runs of the two-kernel route on the full-size workload agree with each other (a slice refilled
  too early shows up as a handful of 16-byte pieces with errors of tens of percent)."""
  from recurrentgemma_b200 import _lib
  b, t, e, h = 8, 4096, 2560, 10
  case = C.Case(f"fused_{b}_{t}_{e}", "rglru", "bfloat16", b, t, e, h, pos="multi")
  p = C.make_params(case)
  inp = C.make_inputs(case)
  dt = torch.bfloat16
  m = rg.RGLRU(e, h, device=DEV, dtype=dt)
  m.load_state_dict({k[len("rg_lru."):]: v for k, v in p.items() if k.startswith("rg_lru.")})
  x, pos = inp["x"].to(DEV), inp["segment_pos"].to(DEV)
  for impl in (_lib.GATES_TCGEN05, _lib.GATES_FUSED):
    m.gates_impl = impl
    ys = []
    for _ in range(6):
      y, _h = m(x, pos)
      ys.append(y.clone())
    for y in ys[1:]:
      assert_close(y, ys[0], 2e-3, f"run-to-run, gates_impl {impl}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", [(1, 8), (5, 136), (33, 2560), (7, 4096), (3, 8192)],
                         ids=lambda s: "x".join(map(str, s)))
def test_rmsnorm_vs_oracle(rg, oracle, dtype, shape):
  """RMSNorm rows of every register-tile size of the kernel, against the oracle."""
  m_rows, d = shape
  if dtype == torch.float32 and d > 4096:
    pytest.skip("float32 rows hold at most 1024 packs of 4")
  name = f"rmsnorm_{m_rows}_{d}_{dtype}"
  x = (C.normal(name, "x", (m_rows, d), 1.0) * C.uniform(name, "row", (m_rows, 1), 0.01, 30.0)).to(dtype)
  sc = C.normal(name, "scale", (d,), 0.3, dtype)
  norm = rg.RMSNorm(d, device=DEV, dtype=dtype)
  norm.load_state_dict({"scale": sc})
  assert_close(norm(x.to(DEV)), oracle.rmsnorm(x, sc), TOL[dtype], "rmsnorm")
  with pytest.raises(Exception):
    rg.RMSNorm(10, device=DEV, dtype=dtype)(torch.zeros(2, 10, device=DEV, dtype=dtype))


def test_residual_fused_vs_composed_and_oracle(rg, oracle):
  """recurrent_block(rmsnorm(x)) + x in one library call (RMSNorm kernel, residual in the epilogue
  of linear_out) against the composition of the modules and against the oracle."""
  case = C.Case("residual_fused", "residual", "bfloat16", 2, 300, 512, 2, width=384, pos="multi")
  p = C.make_params(case)
  inp = C.make_inputs(case)
  dt = torch.bfloat16
  norm = rg.RMSNorm(384, device=DEV, dtype=dt)
  norm.load_state_dict({"scale": p["temporal_pre_norm.scale"]})
  bp = {k: v for k, v in p.items() if not k.startswith("temporal_pre_norm.")}
  m = _block(rg, case, bp)
  x, pos = inp["x"].to(DEV), inp["segment_pos"].to(DEV)
  y_f, c_f = rg.recurrent_residual(x, pos, norm, m)
  y_b, c_b = m(norm(x), pos)
  y_c = y_b + x
  assert_close(y_f, y_c, 1e-6, "fused vs composed")
  assert torch.equal(c_f.conv1d_state, c_b.conv1d_state)
  y_r, h_r, c_r = oracle.residual_temporal(inp["x"], inp["segment_pos"],
                                           p["temporal_pre_norm.scale"], oracle.params_of(bp))
  assert_close(y_f, y_r, TOL[dt], "fused vs oracle")
  assert_close(c_f.rg_lru_state, h_r, TOL[dt], "state")
  assert_close(c_f.conv1d_state, c_r, TOL[dt], "conv state")


@pytest.mark.parametrize("shape", [(1, 64, 64), (200, 256, 768), (300, 384, 7680), (129, 2560, 320)],
                         ids=lambda s: "x".join(map(str, s)))
def test_mlp_vs_oracle(rg, oracle, shape):
  """The GeGLU GEMM (gate/value-interleaved packed weights, gelu(gate) * value in the epilogue) and
  the down projection with the residual in its epilogue, against the oracle: partial row tiles,
  expanded widths that end inside a 256-column tile, and many tiles."""
  m_rows, d, xw = shape
  dt = torch.bfloat16
  case = C.Case(f"mlp_{m_rows}_{d}_{xw}", "mlp", "bfloat16", 1, m_rows, d, width=d, expanded=xw,
                decode_steps=0)
  p = C.make_params(case)
  x = C.make_inputs(case)["x"][0]
  mlp = rg.MLPBlock(d, xw, device=DEV, dtype=dt)
  mlp.load_state_dict({k[len("mlp_block."):]: v for k, v in p.items()})
  args = (p["mlp_block.ffw_up.w"], p["mlp_block.ffw_up.b"], p["mlp_block.ffw_down.weight"],
          p["mlp_block.ffw_down.bias"])
  assert_close(mlp(x.to(DEV)), oracle.mlp(x, *args), TOL[dt], "mlp")
  sc = C.normal(case.name, "scale", (d,), 0.3, dt)
  norm = rg.RMSNorm(d, device=DEV, dtype=dt)
  norm.load_state_dict({"scale": sc})
  assert_close(mlp(x.to(DEV), pre_norm=norm), oracle.residual_channel(x, sc, *args), TOL[dt],
               "channel half")
  # in-place modification of a parameter invalidates the packed copy
  with torch.no_grad():
    mlp.ffw_up.b.add_(1.0)
  assert_close(mlp(x.to(DEV)), oracle.mlp(x, args[0], (args[1].float() + 1.0).to(dt), *args[2:]),
               TOL[dt], "after bias update")


@pytest.mark.parametrize("shape", [(2, 300, 2, 100, "multi"), (1, 129, 3, 512, "half"),
                                   (3, 77, 1, 16, "padded"), (2, 1000, 2, 257, "multi"),
                                   (1, 2500, 2, 2048, "arange")],
                         ids=lambda s: "x".join(map(str, s)))
def test_attention_kernel_vs_oracle(rg, oracle, shape):
  """The two-pass tcgen05 attention kernel (head dimension 256) against the oracle: windows shorter
  and longer than the sequence, documents inside the window, left padding, sequence lengths that end
  inside a tile, query tiles whose window spans many key tiles."""
  b, t, heads, window, pattern = shape
  d = heads * 256
  dt = torch.bfloat16
  case = C.Case(f"attn_{b}_{t}_{heads}_{window}", "attention", "bfloat16", b, t, d, heads, width=d,
                window=window, pos=pattern, decode_steps=1)
  p = C.make_params(case)
  inp = C.make_inputs(case)
  m = rg.LocalAttentionBlock(d, heads, window, device=DEV, dtype=dt)
  m.load_state_dict(p)
  x, pos = inp["x"], inp["segment_pos"]
  y, cache = m(x.to(DEV), pos.to(DEV))
  w = (p["proj_q.weight"], p["proj_k.weight"], p["proj_v.weight"], p["proj_final.weight"],
       p["proj_final.bias"])
  y_r, c_r = oracle.attention_block(x, pos, *w, heads, window)
  assert_close(y, y_r, TOL[dt], "prefill output")
  assert_close(cache.keys, c_r[0], TOL[dt], "cached keys")
  assert_close(cache.values, c_r[1], TOL[dt], "cached values")
  assert torch.equal(cache.num_tokens.cpu(), c_r[2])
  xs, ps = inp["x_step0"], C.decode_positions(case, pos, 0)
  y1, cache1 = m(xs.to(DEV), ps.to(DEV), cache)
  y1_r, c1_r = oracle.attention_block(xs, ps, *w, heads, window, c_r)
  assert_close(y1, y1_r, TOL[dt], "decode output")
  assert_close(cache1.keys, c1_r[0], TOL[dt], "decode keys")
  assert torch.equal(cache1.num_tokens.cpu(), c1_r[2])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed_logits_argmax_vs_oracle(rg, oracle, dtype):
  """Embedder.encode / decode + soft cap / argmax through the C ABI against the oracle."""
  dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
  v, d, m = 1000 if dtype == "float32" else 1024, 256, 70
  g = torch.Generator(device="cpu").manual_seed(5)
  emb = rg.Embedder(v, d, scale_by_sqrt_dim=True, device=DEV, dtype=dt)
  table = (torch.randn((v, d), generator=g) * d ** -0.5).to(dt)
  emb.load_state_dict({"input_embedding": table})
  tok = torch.randint(0, v, (2, 35), generator=g)
  for t in (tok, tok.to(torch.int32)):
    assert_close(emb.encode(t.to(DEV)), oracle.embed(tok, table, True), 0.0, "encode")
  x = (torch.randn((m, d), generator=g) * 6.0).to(dt)
  for cap in (0.0, 30.0):
    assert_close(emb.decode(x.to(DEV), cap), oracle.logits(x, table, cap), TOL[dt], f"decode cap {cap}")
  # argmax: the first maximum, also where a row holds the same value many times
  lg = oracle.logits(x, table, 30.0)
  lg[3, 17] = lg[3, 900] = lg[3].max() + 1
  lg[5] = 0.25
  assert torch.equal(rg.argmax(lg.to(DEV)).cpu().long(), torch.argmax(lg.float(), dim=-1))
  with pytest.raises(TypeError):
    emb.encode(tok.to(DEV).float())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_sampler(rg, dtype):
  """The captured decode loop reproduces step-by-step decoding, the reference's greedy tokens in
  float32, and prefill(T) followed by decoding == prefill(T-1) + the last token as a step."""
  s = "f32" if dtype == "float32" else "bf16"
  case = C.case_by_name(f"griffin_{s}_512_h2_v1024")
  g = load_golden(case.name)
  m = _griffin(rg, case, C.make_params(case))
  tokens = C.make_inputs(case)["tokens"].to(DEV)
  steps = 9
  eager = rg.GreedySampler(m, use_cuda_graph=False)(tokens, steps, return_logits=True)
  graph = rg.GreedySampler(m, use_cuda_graph=True)(tokens, steps, return_logits=True)
  assert eager.tokens.shape == (case.batch, steps) and eager.tokens.dtype == torch.int32
  assert torch.equal(eager.tokens, graph.tokens)
  assert torch.equal(eager.logits, graph.logits)
  # the prompt's positions here are 0..T-1 (one document), not the fixture's two documents, so
  # compare with a plain forward of the same positions
  pos = torch.arange(case.seq, device=DEV, dtype=torch.int32).repeat(case.batch, 1)
  logits, cache = m(tokens, pos)
  assert_close(eager.logits[:, 0], logits[:, -1], TOL[case.torch_dtype], "first logits")
  tok = rg.argmax(logits[:, -1])
  if dtype == "float32":
    assert torch.equal(tok, eager.tokens[:, 0])
  ref = [tok]
  for i in range(steps - 1):
    lg, cache = m(ref[-1][:, None], pos[:, -1:] + 1 + i, cache)
    ref.append(rg.argmax(lg[:, 0]))
    assert_close(eager.logits[:, i + 1], lg[:, 0], TOL[case.torch_dtype], f"logits {i + 1}")
  if dtype == "float32":
    assert torch.equal(torch.stack(ref, dim=1), eager.tokens)
  # left padding: lengths differ, positions of the padding are -1
  lengths = torch.tensor([case.seq, case.seq - 5])
  padded = rg.GreedySampler(m)(tokens, 4, input_lengths=lengths)
  assert padded.tokens.shape == (case.batch, 4)
  assert torch.equal(padded.tokens[0], eager.tokens[0, :4]) or dtype == "bfloat16"
  # EOS: everything after a sequence's first EOS is padding
  eos = int(eager.tokens[0, 2])
  out = rg.GreedySampler(m, eos_id=eos, pad_id=-7)(tokens, steps)
  first = int((eager.tokens[0] == eos).nonzero()[0])
  assert torch.equal(out.tokens[0, :first + 1], eager.tokens[0, :first + 1])
  assert bool((out.tokens[0, first + 1:] == -7).all())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,window,prompt", [(10, 40, 7), (10, 40, 40), (4, 24, 61), (1, 8, 1),
                                                 (8, 300, 310), (10, 2048, 150)])
def test_attention_decode_kernels_vs_oracle(rg, oracle, dtype, heads, window, prompt):
  """The decode-step kernels on the ring cache (head dimension 256) against the oracle: a ring that
  is not yet full, one that is exactly full, one that has wrapped; six steps each, in the
  reference's functional form and in place."""
  d = heads * 256
  dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
  case = C.Case(f"attn_dec_{heads}_{window}_{prompt}", "attention", dtype, 3, prompt, d, heads,
                width=d, window=window, pos="arange", decode_steps=6)
  p = C.make_params(case)
  inp = C.make_inputs(case)
  m = rg.LocalAttentionBlock(d, heads, window, device=DEV, dtype=dt)
  m.load_state_dict(p)
  w = (p["proj_q.weight"], p["proj_k.weight"], p["proj_v.weight"], p["proj_final.weight"],
       p["proj_final.bias"])
  pos = inp["segment_pos"]
  _, cache = m(inp["x"].to(DEV), pos.to(DEV))
  _, c_r = oracle.attention_block(inp["x"], pos, *w, heads, window)
  own = rg.AttentionBlockCache(*[t.clone() for t in cache])
  for i in range(case.decode_steps):
    xs, ps = inp[f"x_step{i}"], C.decode_positions(case, pos, i)
    before = [t.clone() for t in cache]
    y, cache_new = m(xs.to(DEV), ps.to(DEV), cache)
    assert all(torch.equal(a, b) for a, b in zip(before, cache)), "the functional form must not write"
    y2, own2 = m(xs.to(DEV), ps.to(DEV), own, inplace=True)
    assert own2 is own
    y_r, c_r = oracle.attention_block(xs, ps, *w, heads, window, c_r)
    for out, ring, what in ((y, cache_new, "functional"), (y2, own, "in place")):
      assert_close(out, y_r, TOL[dt], f"step {i} output ({what})")
      assert_close(ring.keys, c_r[0], TOL[dt], f"step {i} keys ({what})")
      assert_close(ring.values, c_r[1], TOL[dt], f"step {i} values ({what})")
      assert torch.equal(ring.num_tokens.cpu(), c_r[2])
    y3, none = m(xs.to(DEV), ps.to(DEV), cache, return_cache=False)
    assert none is None and torch.equal(y3, y)
    cache = cache_new


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_sampler_mlp_few_rows(rg, oracle, dtype):
  """(Named so that the bound on library GEMMs keeps its default.)  The MLP for a handful of rows,
  as in a decode step: library contractions around the element-wise kernel, against the oracle,
  alone and as the channel half of a residual block."""
  dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
  case = C.case_by_name("mlp_f32_256_x768" if dtype == "float32" else "mlp_bf16_256_x768")
  p = C.make_params(case)
  x = C.make_inputs(case)["x"][:, :5]
  m = rg.MLPBlock(case.model_width, case.expanded, device=DEV, dtype=dt)
  m.load_state_dict({k[len("mlp_block."):]: v for k, v in p.items()})
  args = (p["mlp_block.ffw_up.w"], p["mlp_block.ffw_up.b"], p["mlp_block.ffw_down.weight"],
          p["mlp_block.ffw_down.bias"])
  assert_close(m(x.to(DEV)), oracle.mlp(x, *args), TOL[dt], "mlp")
  norm = rg.RMSNorm(case.model_width, device=DEV, dtype=dt)
  scale = C.normal(case.name, "norm", (case.model_width,), 0.3, dt)
  norm.load_state_dict({"scale": scale})
  assert_close(m(x.to(DEV), pre_norm=norm), oracle.residual_channel(x, scale, *args), TOL[dt],
               "channel half")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,width", [(64, 2560), (5, 128), (130, 512)])
def test_add_rmsnorm_vs_oracle(rg, oracle, dtype, rows, width):
  """The residual add fused into the norm kernel: the sum is the rounded a + b, the normalised
  output equals the norm kernel (and the oracle) on that sum."""
  dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
  a = C.normal(f"addnorm_{rows}_{width}", "a", (rows, width), 1.0, dt)
  b = C.normal(f"addnorm_{rows}_{width}", "b", (rows, width), 2.0, dt)
  scale = C.normal(f"addnorm_{rows}_{width}", "scale", (width,), 0.3, dt)
  norm = rg.RMSNorm(width, device=DEV, dtype=dt)
  norm.load_state_dict({"scale": scale})
  total, normed = norm.add_norm(a.to(DEV), b.to(DEV))
  ref_total = (a.float() + b.float()).to(dt)
  assert torch.equal(total.cpu(), ref_total)
  assert torch.equal(normed, norm(total))
  assert_close(normed, oracle.rmsnorm(ref_total, scale), TOL[dt], "normalised sum")
