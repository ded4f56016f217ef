"""Pins the CPU oracle against outputs of the reference torch implementation (tests/golden/).

The fixtures were produced by tests/golden/make_golden.py importing the reference itself.  The
float32 oracle must reproduce them to 2e-6 (it differs from ATen only in summation order and in
libm vs vectorised transcendental rounding); the bfloat16 oracle, which re-creates every
intermediate rounding, to 1e-2 with at most a few elements off by one bfloat16 step.
"""
import pytest
import torch

from tests import cases as C
from tests.util import assert_close, as_f32, load_golden

CASES = C.golden_cases()
ORACLE_TOL = {"float32": 2e-6, "bfloat16": 1e-2}


def _frac_mismatch(out, ref) -> float:
  o, r = as_f32(out), as_f32(ref)
  return float((o != r).float().mean())


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_oracle_matches_reference(case, oracle):
  g = load_golden(case.name)
  p = C.make_params(case)
  inp = C.make_inputs(case)
  assert abs(C.checksum({**p, **inp}) - float(g["input_checksum"])) <= 1e-6 * abs(
      float(g["input_checksum"])), "seeded inputs differ from those the fixture was made with"
  tol = ORACLE_TOL[case.dtype]
  pos = inp["segment_pos"]
  mism = []

  def chk(out, key, loose=False):
    # loose: decode steps of the residual cases, where the reference's CPU kernel rounds the
    # bfloat16 rsqrt of RMSNorm twice (see tests/cases.py); the tolerance is the path's own.
    assert_close(out, g[key], 2e-2 if loose and case.dtype == "bfloat16" else tol,
                 f"{case.name}:{key}")
    if not loose:
      mism.append(_frac_mismatch(out, g[key]))

  if case.kind == "blockdiag":
    chk(oracle.blockdiag_linear(inp["x"], p["rg_lru.input_gate.w"], p["rg_lru.input_gate.b"]),
        "out")
  elif case.kind == "conv1d":
    y, cache = oracle.conv1d(inp["x"], pos, p["conv_1d.w"], p["conv_1d.b"])
    chk(y, "out"); chk(cache, "cache")
    for i in range(case.decode_steps):
      y, cache = oracle.conv1d(inp[f"x_step{i}"], C.decode_positions(case, pos, i), p["conv_1d.w"],
                               p["conv_1d.b"], cache)
      chk(y, f"out_step{i}"); chk(cache, f"cache_step{i}")
  elif case.kind == "rnn_scan":
    y, h = oracle.rnn_scan(inp["x"], inp["a"], pos == 0, inp["h0"])
    chk(y, "out"); chk(h, "h")
  elif case.kind == "rglru":
    args = (p["rg_lru.a_param"], p["rg_lru.input_gate.w"], p["rg_lru.input_gate.b"],
            p["rg_lru.a_gate.w"], p["rg_lru.a_gate.b"])
    y, h = oracle.rglru(inp["x"], pos, *args, inp["h0"])
    chk(y, "out"); chk(h, "h")
    for i in range(case.decode_steps):
      y, h = oracle.rglru(inp[f"x_step{i}"], C.decode_positions(case, pos, i), *args, h)
      chk(y, f"out_step{i}"); chk(h, f"h_step{i}")
  elif case.kind == "block":
    op = oracle.params_of(p)
    y, h, cache = oracle.recurrent_block(inp["x"], pos, op)
    chk(y, "out"); chk(h, "h"); chk(cache, "cache")
    for i in range(case.decode_steps):
      y, h, cache = oracle.recurrent_block(inp[f"x_step{i}"], C.decode_positions(case, pos, i), op,
                                           h, cache)
      chk(y, f"out_step{i}"); chk(h, f"h_step{i}"); chk(cache, f"cache_step{i}")
  elif case.kind == "rmsnorm":
    chk(oracle.rmsnorm(inp["x"], p["scale"]), "out")
  elif case.kind == "residual":
    op = oracle.params_of(p)
    ns = p["temporal_pre_norm.scale"]
    y, h, cache = oracle.residual_temporal(inp["x"], pos, ns, op)
    chk(y, "out"); chk(h, "h"); chk(cache, "cache")
    for i in range(case.decode_steps):
      y, h, cache = oracle.residual_temporal(inp[f"x_step{i}"], C.decode_positions(case, pos, i),
                                             ns, op, h, cache)
      chk(y, f"out_step{i}", True); chk(h, f"h_step{i}", True); chk(cache, f"cache_step{i}", True)
  elif case.kind == "attention":
    w = (p["proj_q.weight"], p["proj_k.weight"], p["proj_v.weight"], p["proj_final.weight"],
         p["proj_final.bias"])
    y, cache = oracle.attention_block(inp["x"], pos, *w, case.heads, case.window)
    chk(y, "out"); chk(cache[0], "keys"); chk(cache[1], "values")
    assert torch.equal(cache[2].long(), torch.from_numpy(g["num_tokens"]))
    for i in range(case.decode_steps):
      y, cache = oracle.attention_block(inp[f"x_step{i}"], C.decode_positions(case, pos, i), *w,
                                        case.heads, case.window, cache)
      chk(y, f"out_step{i}"); chk(cache[0], f"keys_step{i}"); chk(cache[1], f"values_step{i}")
      assert torch.equal(cache[2].long(), torch.from_numpy(g[f"num_tokens_step{i}"]))
  elif case.kind == "resblock_attn":
    w = tuple(p["attention_block." + k] for k in ("proj_q.weight", "proj_k.weight", "proj_v.weight",
                                                  "proj_final.weight", "proj_final.bias"))
    mlp = (p["channel_pre_norm.scale"], p["mlp_block.ffw_up.w"], p["mlp_block.ffw_up.b"],
           p["mlp_block.ffw_down.weight"], p["mlp_block.ffw_down.bias"])
    ns = p["temporal_pre_norm.scale"]
    x = inp["x"]
    y, cache = oracle.attention_block(oracle.rmsnorm(x, ns), pos, *w, case.heads, case.window)
    r = (y.float() + x.float()).to(x.dtype)
    chk(oracle.residual_channel(r, *mlp), "out"); chk(cache[0], "keys"); chk(cache[1], "values")
    for i in range(case.decode_steps):
      xs = inp[f"x_step{i}"]
      y, cache = oracle.attention_block(oracle.rmsnorm(xs, ns), C.decode_positions(case, pos, i), *w,
                                        case.heads, case.window, cache)
      r = (y.float() + xs.float()).to(xs.dtype)
      chk(oracle.residual_channel(r, *mlp), f"out_step{i}", True)
  elif case.kind == "griffin":
    run = lambda tok, ps, cache: oracle.griffin(p, C.GRIFFIN_BLOCKS, case.heads, case.window,
                                                C.GRIFFIN_SOFT_CAP, tok, ps, cache)
    lg, cache = run(inp["tokens"], pos, None)
    # the first block's state pins the rounding model bit for bit; three blocks deep, one-ulp
    # differences of a few elements have passed through dense contractions, so the later tensors
    # are held to the path's tolerance only
    chk(cache["blocks.0"][0], "h_0"); chk(cache["blocks.1"][1], "conv_1")
    chk(lg, "logits", True); chk(cache["blocks.2"][0], "keys_2", True)
    for i in range(case.decode_steps):
      tok = torch.from_numpy(g[f"tokens_step{i}"])[:, None]
      lg, cache = run(tok, C.decode_positions(case, pos, i), cache)
      chk(lg, f"logits_step{i}", True)
    chk(cache["blocks.0"][0], "h_0_final", True); chk(cache["blocks.2"][0], "keys_2_final", True)
  elif case.kind == "mlp":
    chk(oracle.mlp(inp["x"], p["mlp_block.ffw_up.w"], p["mlp_block.ffw_up.b"],
                   p["mlp_block.ffw_down.weight"], p["mlp_block.ffw_down.bias"]), "out")
  elif case.kind == "resblock":
    op = oracle.params_of(p, "recurrent_block.")
    mlp = (p["channel_pre_norm.scale"], p["mlp_block.ffw_up.w"], p["mlp_block.ffw_up.b"],
           p["mlp_block.ffw_down.weight"], p["mlp_block.ffw_down.bias"])
    r, h, cache = oracle.residual_temporal(inp["x"], pos, p["temporal_pre_norm.scale"], op)
    chk(oracle.residual_channel(r, *mlp), "out"); chk(h, "h"); chk(cache, "cache")
    for i in range(case.decode_steps):
      r, h, cache = oracle.residual_temporal(inp[f"x_step{i}"], C.decode_positions(case, pos, i),
                                             p["temporal_pre_norm.scale"], op, h, cache)
      chk(oracle.residual_channel(r, *mlp), f"out_step{i}", True)
      chk(h, f"h_step{i}", True); chk(cache, f"cache_step{i}", True)
  # bfloat16: the rounding model must hold almost everywhere, not merely within tolerance.
  if case.dtype == "bfloat16":
    assert max(mism) < 0.03, f"{case.name}: {max(mism):.3%} of elements differ from the reference"


def test_prefill_state_equals_decode_state(oracle):
  """prefill(T) == prefill(T-1) followed by one decode step (the sampler's contract,
  torch/sampler_test.py:150-230), checked on the oracle itself."""
  case = C.case_by_name("block_f32_128_h1_l256_multi")
  p = oracle.params_of(C.make_params(case))
  inp = C.make_inputs(case)
  x, pos = inp["x"], inp["segment_pos"]
  y_full, h_full, c_full = oracle.recurrent_block(x, pos, p)
  _, h_a, c_a = oracle.recurrent_block(x[:, :-1].contiguous(), pos[:, :-1].contiguous(), p)
  # the final position of this case starts no document, as in a decode continuation
  keep = (pos[:, -1] != 0)
  y_b, h_b, c_b = oracle.recurrent_block(x[:, -1:].contiguous(), pos[:, -1:].contiguous(), p, h_a,
                                         c_a)
  assert keep.any()
  assert_close(h_b[keep], h_full[keep], 1e-6, "state")
  assert_close(y_b[keep], y_full[keep][:, -1:], 1e-6, "last output")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_jax_linear_scan_restatement_equals_rnn_scan(oracle, dtype):
  """The restatement of the JAX reference's lru_linear_scan (jax/scan.py:74-120: a vmapped lax.scan
  of h = a h + x in the accumulation dtype, outputs cast to the input dtype) computes what the torch
  reference's rnn_scan computes once the reset mask is folded into a (torch/layers.py:166-168)."""
  b, t, e = 3, 97, 130
  x = C.normal("jaxscan", "x", (b, t, e), 1.0, dtype)
  a = C.uniform("jaxscan", "a", (b, t, e), 0.3, 0.999).to(dtype)
  h0 = C.normal("jaxscan", "h0", (b, e), 0.5)
  reset = C.make_segment_pos("multi", b, t, "jaxscan") == 0
  y_t, h_t = oracle.rnn_scan(x, a, reset, h0)
  a_masked = (a.float() * (~reset)[..., None].float()).to(dtype)
  y_j, h_j = oracle.jax_linear_scan(x, a_masked, h0)
  assert torch.equal(y_t, y_j)
  assert torch.equal(h_t, h_j)


def test_thread_count_is_settable(oracle):
  """Timed baselines set the OpenMP thread count themselves (a launcher may export
  OMP_NUM_THREADS=1): the oracle reports the count in force."""
  import os
  before = oracle.set_threads(0)
  assert before >= 1
  want = min(2, os.cpu_count() or 1)
  assert oracle.set_threads(want) in (want, 1)      # 1: built without OpenMP
  oracle.set_threads(before)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_rnn_param_init_matches_reference_on_a_seed(dtype):
  """rnn_param_init (torch/layers.py:194-213) draws from torch's global generator; the same seed
  must give the reference's a_param exactly (fixture generated by the reference)."""
  from recurrentgemma_b200 import layers
  from tests.golden import make_golden as G
  g = load_golden("rnn_param_init")
  torch.manual_seed(G.PARAM_INIT_SEED)
  t = layers.rnn_param_init(torch.empty(G.PARAM_INIT_WIDTH, dtype=dtype), min_rad=0.9, max_rad=0.999)
  name = "float32" if dtype == torch.float32 else "bfloat16"
  assert torch.equal(t.float(), torch.from_numpy(g[name]))
