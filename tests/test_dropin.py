"""Structural drop-in check against the reference checkout, when one is available.

Runs on CPU: the reference `Griffin` is built, its recurrent blocks are swapped for ours, and the
state_dict keys, cache types and the "no CPU path" behaviour are checked.  Skipped where the
checkout is absent (e.g. on a GPU box)."""
import os
import sys
import types

import pytest
import torch

REF = os.environ.get("RECURRENTGEMMA_REFERENCE", "/root/reference")

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
  """Constructor and forward parameter names of the mirrored classes equal the reference's."""
  import inspect
  from recurrentgemma.torch import layers as ref_layers, modules as ref_modules
  from recurrentgemma_b200 import layers, modules
  pairs = [(ref_layers.RGLRU, layers.RGLRU), (ref_layers.Conv1D, layers.Conv1D),
           (ref_layers.RMSNorm, layers.RMSNorm), (ref_layers.Einsum, layers.Einsum),
           (ref_modules.LocalAttentionBlock, modules.LocalAttentionBlock),
           (ref_layers.BlockDiagonalLinear, layers.BlockDiagonalLinear),
           (ref_modules.RecurrentBlock, modules.RecurrentBlock)]
  for ref_cls, our_cls in pairs:
    for fn in ("__init__", "forward", "reset_parameters"):
      ref_p = list(inspect.signature(getattr(ref_cls, fn)).parameters)
      our_p = list(inspect.signature(getattr(our_cls, fn)).parameters)
      assert ref_p == our_p, (ref_cls.__name__, fn, ref_p, our_p)
    if hasattr(ref_cls, "init_cache"):
      assert (list(inspect.signature(ref_cls.init_cache).parameters) ==
              list(inspect.signature(our_cls.init_cache).parameters)), ref_cls.__name__
  # MLPBlock: same constructor; forward takes the reference's argument first (two optional
  # extensions follow)
  assert (list(inspect.signature(ref_modules.MLPBlock.__init__).parameters) ==
          list(inspect.signature(modules.MLPBlock.__init__).parameters))
  assert list(inspect.signature(modules.MLPBlock.forward).parameters)[:2] == ["self", "x"]
  ref_scan = list(inspect.signature(ref_layers.rnn_scan).parameters)
  our_scan = list(inspect.signature(layers.rnn_scan).parameters)
  assert our_scan[:len(ref_scan)] == ref_scan
