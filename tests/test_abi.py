"""CPU-side checks of the C ABI: the shared library loads, exports every symbol that
include/rgk.h declares, the ctypes table covers each of them, and argument validation (which
runs before any CUDA call) reports the documented codes.  No kernel is launched here."""
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
  with open(os.path.join(ROOT, "include", "rgk.h")) as f:
    text = f.read()
  return sorted(set(re.findall(r"RGK_API\s+[\w\s\*]+?\b(rgk_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
  from recurrentgemma_b200 import build, _lib
  build.build_library()
  return _lib.load()


def test_header_symbols_exported(lib):
  from recurrentgemma_b200 import _lib
  names = _declared()
  assert len(names) >= 12
  for n in names:
    assert hasattr(lib, n), f"{n} declared in include/rgk.h but not exported"
    assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
  assert sorted(_lib.SIGNATURES) == names


def test_version_and_error_text(lib):
  assert lib.rgk_abi_version() == 8
  assert isinstance(lib.rgk_last_error(), bytes)


def test_validation_codes(lib):
  # NULL pointers -> RGK_EINVAL, before any device is touched
  assert lib.rgk_conv1d_prefill(None, None, 0, None, None, 1, 4, 128, 4, 0, None, None, None) == -1
  # width not a multiple of the 16-byte pack -> RGK_ESHAPE
  assert lib.rgk_conv1d_prefill(16, 16, 0, 16, 16, 1, 4, 130, 4, 0, 16, None, None) == -2
  assert b"130" in lib.rgk_last_error()
  # temporal width other than 4 -> RGK_ESHAPE
  assert lib.rgk_conv1d_prefill(16, 16, 0, 16, 16, 1, 4, 128, 8, 0, 16, None, None) == -2
  # misaligned pointer -> RGK_EALIGN
  assert lib.rgk_conv1d_prefill(17, 16, 0, 16, 16, 1, 4, 128, 4, 0, 16, None, None) == -3
  # unknown dtype -> RGK_EINVAL
  assert lib.rgk_conv1d_decode(16, 16, 16, 16, 1, 128, 4, 7, 16, None, None) == -1
  # scan without workspace -> RGK_EWORKSPACE
  assert lib.rgk_linear_scan(16, 16, None, None, None, 1, 8, 128, 0, 16, None, None, 0, None) == -6
  # head width not a multiple of 16
  assert lib.rgk_blockdiag_linear(16, 16, 16, 4, 1, 24, 0, 16, None) == -2


def test_workspace_bytes(lib):
  small = lib.rgk_workspace_bytes(1, 1, 128, 0)
  big = lib.rgk_workspace_bytes(8, 4096, 2560, 1)
  assert 0 < small < big
  # three activation-sized intermediates plus the look-back records
  assert big >= 3 * 8 * 4096 * 2560 * 2
  assert lib.rgk_workspace_bytes(-1, 1, 128, 0) == 0
  assert lib.rgk_workspace_bytes(1, 1, 128, 5) == 0


def test_no_cpu_path():
  """The product path must refuse CPU tensors instead of computing on the host."""
  import recurrentgemma_b200 as rg
  conv = rg.Conv1D(128, 4)
  with pytest.raises(RuntimeError, match="no CPU path"):
    conv(torch.zeros(1, 4, 128), torch.zeros(1, 4, dtype=torch.int64))
  lru = rg.RGLRU(128, 1)
  with pytest.raises(RuntimeError, match="no CPU path"):
    lru(torch.zeros(1, 4, 128), torch.zeros(1, 4, dtype=torch.int64))
  blk = rg.RecurrentBlock(128, 1)
  with pytest.raises(RuntimeError, match="no CPU path"):
    blk(torch.zeros(1, 4, 128), torch.zeros(1, 4, dtype=torch.int64))


def test_product_does_not_import_oracle():
  """Nothing under the package may reference the oracle."""
  pkg = os.path.join(ROOT, "recurrentgemma_b200")
  for dirpath, _, files in os.walk(pkg):
    for fn in files:
      if fn.endswith((".py", ".cu", ".cuh", ".h")):
        with open(os.path.join(dirpath, fn)) as f:
          assert "oracle" not in f.read().lower(), os.path.join(dirpath, fn)


def test_state_dict_keys_match_reference_names():
  """Parameter names of recurrentgemma/torch/modules.py:531-560 and layers.py:105-112, 262-278,
  409-412, so reference checkpoints load unchanged."""
  import recurrentgemma_b200 as rg
  blk = rg.RecurrentBlock(128, 2, 256)
  assert sorted(blk.state_dict()) == sorted([
      "linear_y.weight", "linear_y.bias", "linear_x.weight", "linear_x.bias", "linear_out.weight",
      "linear_out.bias", "conv_1d.w", "conv_1d.b", "rg_lru.a_param", "rg_lru.input_gate.w",
      "rg_lru.input_gate.b", "rg_lru.a_gate.w", "rg_lru.a_gate.b"])
  sd = blk.state_dict()
  assert sd["rg_lru.input_gate.w"].shape == (2, 128, 128)
  assert sd["conv_1d.w"].shape == (4, 256)
  cache = rg.RecurrentBlock.init_cache(3, 256, torch.bfloat16)
  assert cache.rg_lru_state.dtype == torch.float32 and cache.rg_lru_state.shape == (3, 256)
  assert cache.conv1d_state.dtype == torch.bfloat16 and cache.conv1d_state.shape == (3, 3, 256)
