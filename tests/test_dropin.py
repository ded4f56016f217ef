"""Drop-in checks against the reference checkout, when one is available.

On CPU: the reference `Griffin` is built, its recurrent blocks are swapped for ours, and the
state_dict keys, cache types and the "no CPU path" behaviour are checked.  Where a checkout AND a
GPU are present, the converted model also runs on the GPU against the untouched model on the CPU.
The checkout is found through RECURRENTGEMMA_REFERENCE, else as a directory `reference` beside
this repository; without one every test here is skipped (the reference sources are never copied
into this repository, so a machine that only receives the repository has none)."""
import os
import sys
import types

import pytest
import torch

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("RECURRENTGEMMA_REFERENCE") or os.path.join(os.path.dirname(_REPO), "reference")

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "recurrentgemma", "torch")),
                                reason="reference checkout not available")


@pytest.fixture(scope="module")
def rg():
  if "recurrentgemma" not in sys.modules:
    pkg = types.ModuleType("recurrentgemma")
    pkg.__path__ = [os.path.join(REF, "recurrentgemma")]
    sys.modules["recurrentgemma"] = pkg
  import recurrentgemma.torch as m
  return m


def _config():
  from recurrentgemma import common
  return common.GriffinConfig(
      vocab_size=64, width=128, mlp_expanded_width=256, num_heads=2, lru_width=256,
      block_types=(common.TemporalBlockType.RECURRENT, common.TemporalBlockType.RECURRENT,
                   common.TemporalBlockType.ATTENTION),
      embeddings_scale_by_sqrt_dim=True, attention_window_size=16, logits_soft_cap=30.0)


def test_convert_keeps_state_dict_and_cache_layout(rg):
  from recurrentgemma_b200 import dropin, modules
  model = rg.Griffin(_config(), dtype=torch.float32)
  before = {k: v.clone() for k, v in model.state_dict().items()}
  model = dropin.convert(model)
  after = model.state_dict()
  assert sorted(after) == sorted(before)
  for k in before:
    assert torch.equal(before[k], after[k]), k
  assert isinstance(model.blocks[0].recurrent_block, modules.RecurrentBlock)
  assert isinstance(model.blocks[1].recurrent_block, modules.RecurrentBlock)
  assert not hasattr(model.blocks[2], "recurrent_block")
  # Griffin.init_cache goes through the reference's own RecurrentBlock.init_cache; ours must
  # produce the same field names, shapes and dtypes.
  ref_cache = rg.RecurrentBlock.init_cache(batch_size=3, lru_width=256, dtype=torch.bfloat16)
  our_cache = modules.RecurrentBlock.init_cache(batch_size=3, lru_width=256, dtype=torch.bfloat16)
  assert ref_cache._fields == our_cache._fields
  for a, b in zip(ref_cache, our_cache):
    assert a.shape == b.shape and a.dtype == b.dtype
  with pytest.raises(RuntimeError, match="no CPU path"):
    model(torch.zeros(1, 4, dtype=torch.long), torch.arange(4)[None])
  # the temporal half of the residual blocks as one call: same keys, same parameter storage
  from recurrentgemma_b200 import layers
  model = dropin.fuse_temporal_residual(model)
  after = model.state_dict()
  assert sorted(after) == sorted(before)
  for k in before:
    assert torch.equal(before[k], after[k]), k
  assert isinstance(model.blocks[0].temporal_pre_norm, layers.RMSNorm)
  assert not isinstance(model.blocks[2].temporal_pre_norm, layers.RMSNorm)
  with pytest.raises(RuntimeError, match="no CPU path"):
    model(torch.zeros(1, 4, dtype=torch.long), torch.arange(4)[None])
  # ... and the whole residual block
  model = dropin.fuse_residual_block(model)
  after = model.state_dict()
  assert sorted(after) == sorted(before)
  for k in before:
    assert torch.equal(before[k], after[k]), k
  assert isinstance(model.blocks[1].mlp_block, modules.MLPBlock)
  assert isinstance(model.blocks[1].channel_pre_norm, layers.RMSNorm)
  assert isinstance(model.blocks[2].mlp_block, modules.MLPBlock)
  assert isinstance(model.blocks[2].attention_block, modules.LocalAttentionBlock)
  ref_ac = rg.LocalAttentionBlock.init_cache(batch_size=3, window_size=16, heads_dim=64,
                                             dtype=torch.bfloat16)
  our_ac = modules.LocalAttentionBlock.init_cache(batch_size=3, window_size=16, heads_dim=64,
                                                  dtype=torch.bfloat16)
  assert ref_ac._fields == our_ac._fields
  for a, b in zip(ref_ac, our_ac):
    assert a.shape == b.shape and a.dtype == b.dtype
  with pytest.raises(RuntimeError, match="no CPU path"):
    model(torch.zeros(1, 4, dtype=torch.long), torch.arange(4)[None])


def test_install_rebinds_reference_names(rg):
  from recurrentgemma.torch import layers as ref_layers, modules as ref_modules
  from recurrentgemma_b200 import dropin, layers, modules
  saved = (ref_layers.RGLRU, ref_layers.Conv1D, ref_layers.BlockDiagonalLinear, ref_layers.rnn_scan,
           ref_modules.RecurrentBlock, ref_modules.RecurrentBlockCache)
  try:
    dropin.install()
    model = rg.Griffin(_config(), dtype=torch.float32)
    assert isinstance(model.blocks[0].recurrent_block, modules.RecurrentBlock)
    assert isinstance(model.blocks[0].recurrent_block.rg_lru, layers.RGLRU)
  finally:
    (ref_layers.RGLRU, ref_layers.Conv1D, ref_layers.BlockDiagonalLinear, ref_layers.rnn_scan,
     ref_modules.RecurrentBlock, ref_modules.RecurrentBlockCache) = saved


def test_signatures_match_reference(rg):
  """Constructor and forward parameter names of the mirrored classes equal the reference's; what
  a mirror adds comes after them and has a default (`inplace`, `device`, a fused soft cap)."""
  import inspect
  from recurrentgemma.torch import griffin as ref_griffin
  from recurrentgemma.torch import layers as ref_layers, modules as ref_modules
  from recurrentgemma_b200 import griffin, layers, modules

  def same(ref_fn, our_fn, what):
    ref_p = list(inspect.signature(ref_fn).parameters)
    ours = inspect.signature(our_fn).parameters
    our_p = list(ours)
    assert our_p[:len(ref_p)] == ref_p, (what, ref_p, our_p)
    for extra in our_p[len(ref_p):]:
      assert ours[extra].default is not inspect.Parameter.empty, (what, extra)

  pairs = [(ref_layers.RGLRU, layers.RGLRU), (ref_layers.Conv1D, layers.Conv1D),
           (ref_layers.RMSNorm, layers.RMSNorm), (ref_layers.Einsum, layers.Einsum),
           (ref_modules.LocalAttentionBlock, modules.LocalAttentionBlock),
           (ref_layers.BlockDiagonalLinear, layers.BlockDiagonalLinear),
           (ref_modules.RecurrentBlock, modules.RecurrentBlock),
           (ref_modules.ResidualBlock, modules.ResidualBlock),
           (ref_griffin.Griffin, griffin.Griffin)]
  for ref_cls, our_cls in pairs:
    for fn in ("__init__", "forward", "reset_parameters"):
      same(getattr(ref_cls, fn), getattr(our_cls, fn), (ref_cls.__name__, fn))
    if hasattr(ref_cls, "init_cache"):
      same(ref_cls.init_cache, our_cls.init_cache, (ref_cls.__name__, "init_cache"))
  for fn in ("__init__", "encode", "decode", "reset_parameters"):
    same(getattr(ref_modules.Embedder, fn), getattr(modules.Embedder, fn), ("Embedder", fn))
  # the whole model: the same state_dict keys and shapes, the same cache structure
  ref_model = ref_griffin.Griffin(_config(), device="meta", dtype=torch.float32)
  our_model = griffin.Griffin(_config(), device="meta", dtype=torch.float32)
  ref_sd, our_sd = ref_model.state_dict(), our_model.state_dict()
  assert list(ref_sd) == list(our_sd)
  assert all(ref_sd[k].shape == our_sd[k].shape for k in ref_sd)
  ref_cache = ref_model.init_cache(2, torch.float32)
  our_cache = our_model.init_cache(2, torch.float32)
  assert list(ref_cache) == list(our_cache)
  for k in ref_cache:
    assert type(ref_cache[k])._fields == type(our_cache[k])._fields
    assert all(a.shape == b.shape and a.dtype == b.dtype for a, b in zip(ref_cache[k], our_cache[k]))
  # MLPBlock: same constructor; forward takes the reference's argument first (two optional
  # extensions follow)
  assert (list(inspect.signature(ref_modules.MLPBlock.__init__).parameters) ==
          list(inspect.signature(modules.MLPBlock.__init__).parameters))
  assert list(inspect.signature(modules.MLPBlock.forward).parameters)[:2] == ["self", "x"]
  ref_scan = list(inspect.signature(ref_layers.rnn_scan).parameters)
  our_scan = list(inspect.signature(layers.rnn_scan).parameters)
  assert our_scan[:len(ref_scan)] == ref_scan


def test_config_preset_and_sampler_positions(rg):
  """The 2B preset equals the reference's, and prompt positions follow the reference sampler's
  formula for left-padded prompts (torch/sampler.py:253-256)."""
  from recurrentgemma import common
  from recurrentgemma_b200 import griffin, sampler
  ref = common.GriffinConfig.from_preset(common.Preset.RECURRENT_GEMMA_2B_V1)
  ours = griffin.GriffinConfig.recurrent_gemma_2b()
  for f in ours._fields:
    a, b = getattr(ref, f), getattr(ours, f)
    if f == "block_types":
      assert [t.name for t in a] == [t.name for t in b]
    else:
      assert a == b, f
  assert ours.num_layers == ref.num_layers == 26
  assert griffin.GriffinConfig.recurrent_gemma_2b(max_sequence_length=512).attention_window_size == 512
  model = griffin.Griffin(_config(), device="cpu", dtype=torch.float32)
  s = sampler.GreedySampler(model)
  lengths = torch.tensor([7, 3, 1])
  pos = s.positions(7, lengths)
  expect = torch.clip(torch.arange(7)[None] - 7 + lengths[:, None], min=-1).to(torch.int32)
  assert torch.equal(pos, expect)
  assert pos[1].tolist() == [-1, -1, -1, -1, 0, 1, 2]
  # a private copy of a cache shares no storage with the original
  cache = model.init_cache(2, torch.float32)
  own = sampler._own(cache)
  assert list(own) == list(cache)
  assert all(a.data_ptr() != b.data_ptr() for k in cache for a, b in zip(cache[k], own[k]))


@pytest.mark.gpu
def test_converted_reference_model_on_gpu_matches_reference_on_cpu(rg):
  """The reference `Griffin` (recurrentgemma/torch/griffin.py:131-190) with `dropin.convert` and
  `dropin.fuse_residual_block` applied, on the GPU in bfloat16, against the untouched reference model
  on the CPU: logits and caches of a prefill and of two decode steps fed with the returned caches -
  the equivalence the reference checks for itself in torch/sampler_test.py:150-230."""
  import copy
  from recurrentgemma_b200 import dropin
  from tests.util import TOL, assert_close
  if not torch.cuda.is_available():
    pytest.skip("needs a GPU")
  torch.manual_seed(3)
  dt = torch.bfloat16
  ref = rg.Griffin(_config(), dtype=dt)
  with torch.no_grad():
    for prm in ref.parameters():          # norm scales and biases start at zero: make them count
      if prm.abs().sum() == 0:
        prm.normal_(0.0, 0.1)
  ours = dropin.fuse_residual_block(dropin.convert(copy.deepcopy(ref))).to("cuda")
  b, t = 2, 24
  tokens = torch.randint(0, 64, (b, t + 2))
  pos = torch.arange(t + 2)[None].repeat(b, 1)
  with torch.no_grad():
    lr, cr = ref(tokens[:, :t], pos[:, :t], None, return_logits=True, return_cache=True)
    lo, co = ours(tokens[:, :t].cuda(), pos[:, :t].cuda(), None, return_logits=True, return_cache=True)
    assert_close(lo, lr, TOL[dt], "prefill logits")
    for i in range(2):
      lr, cr = ref(tokens[:, t + i:t + i + 1], pos[:, t + i:t + i + 1], cr, return_logits=True,
                   return_cache=True)
      lo, co = ours(tokens[:, t + i:t + i + 1].cuda(), pos[:, t + i:t + i + 1].cuda(), co,
                    return_logits=True, return_cache=True)
      assert_close(lo, lr, TOL[dt], f"decode step {i} logits")
    for name in cr:
      for a, r in zip(co[name], cr[name]):
        if r.dtype.is_floating_point:
          assert_close(a, r, TOL[dt], f"cache {name}")
