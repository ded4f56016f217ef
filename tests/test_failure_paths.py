"""The failure path of the bounded device-side waits, and one process driving two GPUs.

No test here faults, traps or hangs a GPU: the expiry is produced by a wait that is given nothing to
wait for (records that are never published) with its poll limit lowered, after which the kernel
finishes on its own and leaves an error status for the host to read."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def lib():
  from recurrentgemma_b200 import _lib
  return _lib.load()


def test_bounded_wait_expires_and_is_reported(lib):
  """rgk_selftest_wait_expiry launches a scan whose first time tile is never run: the look-back of
  the next tile gives up after 200 polls, the kernel returns, and the status word holds
  RGK_ETIMEOUT.  Reading the word reports it once and clears it; the next (healthy) call on the
  same workspace leaves it clean."""
  from recurrentgemma_b200 import _lib
  import recurrentgemma_b200 as rg
  dev = torch.device(DEV)
  ws = _lib.workspace(dev, 1 << 20)
  _lib.workspace_status(ws)                       # clean before
  with torch.cuda.device(dev):
    _lib.check(lib.rgk_selftest_wait_expiry(ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
  torch.cuda.synchronize()                        # the kernel has returned by itself
  with pytest.raises(_lib.RgkError) as err:
    rg.check_status(dev)
  assert err.value.code == _lib.RGK_ETIMEOUT
  rg.check_status(dev)                            # reported once, then cleared
  # a healthy scan on the same workspace afterwards
  x = torch.randn(2, 300, 128, device=dev)
  a = torch.rand(2, 300, 128, device=dev)
  reset = torch.zeros(2, 300, dtype=torch.bool, device=dev)
  y, h = rg.rnn_scan(x, a, reset, None)
  ref = torch.zeros(2, 128, device=dev)
  for t in range(300):
    ref = a[:, t] * ref + x[:, t]
  torch.testing.assert_close(h, ref, rtol=1e-5, atol=1e-5)
  rg.check_status(dev)


def test_status_word_survives_workspace_growth(lib):
  """The package's per-stream workspace grows on demand; a raised status word moves with it."""
  from recurrentgemma_b200 import _lib
  import recurrentgemma_b200 as rg
  dev = torch.device(DEV)
  ws = _lib.workspace(dev, 1 << 20)
  with torch.cuda.device(dev):
    _lib.check(lib.rgk_selftest_wait_expiry(ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
  bigger = _lib.workspace(dev, ws.numel() * 2)
  assert bigger.numel() >= ws.numel() * 2
  with pytest.raises(_lib.RgkError):
    rg.check_status(dev)
  rg.check_status(dev)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_second_device_in_one_process():
  """Function attributes (dynamic shared memory above the default limit) are per device: after
  cuda:0 has run the kernels, the same process runs them on cuda:1 - the built-in-scratch scan and
  a tensor-core entry point (plain kernels on each device's own memory, no peer access)."""
  import ctypes
  import recurrentgemma_b200 as rg
  from recurrentgemma_b200 import _lib, synthetic
  lib = _lib.load()
  outs = []
  for index in (0, 1):
    dev = torch.device("cuda", index)
    with torch.cuda.device(dev):
      g = torch.Generator().manual_seed(5)
      p = synthetic.rglru_params(512, 2, g, torch.bfloat16)
      x = torch.randn((2, 384, 512), generator=g).to(torch.bfloat16).to(dev)
      pos = torch.arange(384).repeat(2, 1).to(dev)
      m = rg.RGLRU(512, 2, device=dev, dtype=torch.bfloat16)
      m.load_state_dict(p)
      y, h = m(x, pos)                                        # fused tcgen05 kernel
      w = torch.randn((512, 512), generator=g).to(torch.bfloat16).to(dev)
      z = rg.dense_linear(x, w, None)                         # tcgen05 GEMM
      xs = torch.randn((2, 300, 128), generator=g).to(dev)
      a = torch.rand((2, 300, 128), generator=g).to(dev)
      ys = torch.empty_like(xs)
      hs = torch.empty((2, 128), device=dev)
      _lib.check(lib.rgk_linear_scan_static(xs.data_ptr(), a.data_ptr(), None, None, None, 2, 300,
                                            128, _lib.RGK_F32, ys.data_ptr(), hs.data_ptr(), None,
                                            _lib.stream_ptr(dev)))
      torch.cuda.synchronize(dev)
      rg.check_status(dev)
      outs.append((y.float().cpu(), z.float().cpu(), ys.cpu()))
  for a0, a1 in zip(outs[0], outs[1]):
    torch.testing.assert_close(a0, a1, rtol=2e-2, atol=2e-2)


def test_packed_gate_weights_follow_uncounted_writes():
  """`param.data.copy_()` (the usual checkpoint-loader idiom) neither moves the tensor nor bumps its
  version counter, so the K-major copy of the gate weights cannot notice it: load_state_dict and
  `.to()` refresh the copy by themselves, a `.data` write needs `invalidate_packed()`."""
  import recurrentgemma_b200 as rg
  from recurrentgemma_b200 import synthetic
  dev = torch.device(DEV)
  g = torch.Generator().manual_seed(11)
  p1 = synthetic.rglru_params(256, 1, g, torch.bfloat16)
  p2 = synthetic.rglru_params(256, 1, g, torch.bfloat16)
  x = torch.randn((1, 256, 256), generator=g).to(torch.bfloat16).to(dev)
  pos = torch.arange(256).repeat(1, 1).to(dev)
  ref = rg.RGLRU(256, 1, device=dev, dtype=torch.bfloat16)
  ref.load_state_dict(p2)
  y2, _ = ref(x, pos)
  m = rg.RGLRU(256, 1, device=dev, dtype=torch.bfloat16)
  m.load_state_dict(p1)
  y1, _ = m(x, pos)
  assert not torch.equal(y1, y2)
  m.load_state_dict(p2)                       # refreshed by the load hook
  assert torch.equal(m(x, pos)[0], y2)
  m.load_state_dict(p1)
  m(x, pos)
  for name, t in p2.items():                  # an uncounted write ...
    mod, attr = name.rsplit(".", 1) if "." in name else ("", name)
    getattr(m.get_submodule(mod) if mod else m, attr).data.copy_(t.to(dev))
  m.invalidate_packed()                       # ... needs the explicit call
  assert torch.equal(m(x, pos)[0], y2)


def test_range_checked_build_runs_the_path_tests_clean():
  """librgk_checks.so (-DRGK_CHECKS) range-checks the computed indices of the look-back records, the
  states and the outputs of the scan and of the fused RG-LRU kernel: an index outside its array would
  raise the status word to RGK_EBOUNDS and skip the access.  The scan and fused-kernel parity tests
  (ragged lengths, many time tiles, carries across rounds, the long shard) run on that build in a
  child process; they check the status word after every call, so a bad index fails them."""
  import os
  import subprocess
  import sys
  from recurrentgemma_b200 import _lib
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  lib_path = os.path.join(root, "recurrentgemma_b200", "librgk_checks.so")
  if not os.path.exists(lib_path):
    pytest.skip("librgk_checks.so not built (python -m recurrentgemma_b200.build --checks)")
  env = dict(os.environ, RGK_LIBRARY=lib_path)
  cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu",
         os.path.join(root, "tests", "test_gpu_parity.py"), os.path.join(root, "tests", "test_config_sizes.py"),
         "-k", "fused_rglru_kernel or scan_vs_oracle or long_scan_shard or static", "-p", "no:cacheprovider"]
  r = subprocess.run(cmd, env=env, cwd=root, capture_output=True, text=True, timeout=900)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
  assert " passed" in r.stdout
