"""The allocation-free scan entry point, rgk_linear_scan_static, against rgk_linear_scan.

Some hosts of the library cannot allocate device memory when they call it - a serving loop whose
buffers are all planned ahead and that bans allocation on the request path, or a process whose
own arena already holds the whole GPU.  For them the scan has a variant whose look-back scratch is
an 8 MiB array inside the library.  This file checks, through the C ABI, that the variant returns
what the workspace-taking entry point returns, twice in a row on the same array (the second call
meets the first call's leftovers), that it does not take device memory, and that it refuses
problems that do not fit.  It is named to be collected last, so that a run stopping at the first
failure has already run everything else; it passes alone in a fresh process as well.
"""
import pytest
import torch

from tests import cases as C
from tests.util import TOL, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _problem(name, b, t, e, dtype):
  x = C.normal(name, "x", (b, t, e), 1.0, dtype).to(DEV)
  a = C.uniform(name, "a", (b, t, e), 0.6, 1.0).to(dtype).to(DEV)
  ym = C.normal(name, "ym", (b, t, e), 1.0, dtype).to(DEV)
  h0 = C.normal(name, "h0", (b, e), 0.5).to(DEV)
  reset = (C.uniform(name, "reset", (b, t), 0.0, 1.0) < 0.02).to(torch.uint8).to(DEV)
  return x, a, ym, h0, reset


def _run(lib, _lib, static, x, a, ym, h0, reset):
  b, t, e = x.shape
  dt = _lib.dtype_code(x.dtype)
  y = torch.empty_like(x)
  h = torch.empty((b, e), dtype=torch.float32, device=DEV)
  stream = torch.cuda.current_stream().cuda_stream
  if static:
    status = torch.full((1,), 123, dtype=torch.int32, device=DEV)
    _lib.check(lib.rgk_linear_scan_static(x.data_ptr(), a.data_ptr(), reset.data_ptr(),
                                          h0.data_ptr(), ym.data_ptr(), b, t, e, dt, y.data_ptr(),
                                          h.data_ptr(), status.data_ptr(), stream))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
  else:
    ws = _lib.workspace(torch.device(DEV), _lib.workspace_bytes(b, t, e, x.dtype))
    _lib.check(lib.rgk_linear_scan(x.data_ptr(), a.data_ptr(), reset.data_ptr(), h0.data_ptr(),
                                   ym.data_ptr(), b, t, e, dt, y.data_ptr(), h.data_ptr(),
                                   ws.data_ptr(), ws.numel(), stream))
    torch.cuda.synchronize()
  return y, h


def test_static_scan_matches_workspace_scan_twice_in_a_row():
  from recurrentgemma_b200 import _lib
  lib = _lib.load()
  # Two different problems back to back on the shared array: a long bfloat16 one (many tiles per
  # sequence, so the look-back records are really used), then a smaller float32 one that finds the
  # first call's flags and records still in place.
  problems = [("noalloc_a", 2, 3000, 320, torch.bfloat16), ("noalloc_b", 3, 700, 200, torch.float32)]
  first = True
  for name, b, t, e, dtype in problems:
    args = _problem(name, b, t, e, dtype)
    if first:
      _run(lib, _lib, True, *args)      # set-up call: looks up the array's address on this device
      first = False
    free_before = torch.cuda.mem_get_info()[0]
    y_s, h_s = _run(lib, _lib, True, *args)
    free_after = torch.cuda.mem_get_info()[0]
    y_w, h_w = _run(lib, _lib, False, *args)
    assert_close(y_s, y_w, TOL[dtype], f"{name}: y")
    assert_close(h_s, h_w, TOL[torch.float32] * 3, f"{name}: h")
    # the only device memory taken between the two readings is torch's own for y, h and status,
    # which comes out of its cache or is at most these few MB; a cudaMalloc of scratch would not be
    assert free_before - free_after <= y_s.numel() * y_s.element_size() + (4 << 20)


def test_static_scan_rejects_problems_beyond_its_scratch():
  from recurrentgemma_b200 import _lib
  lib = _lib.load()
  # 16 x 8192 x 2560 bfloat16 needs ~32 MiB of look-back records: over the 8 MiB limit.  The check
  # comes before any pointer is touched, so small dummy buffers are enough.
  d = torch.zeros(64, dtype=torch.bfloat16, device=DEV)
  rc = lib.rgk_linear_scan_static(d.data_ptr(), d.data_ptr(), None, None, None, 16, 8192, 2560, 1,
                                  d.data_ptr(), None, None, None)
  assert rc == -2
  msg = lib.rgk_last_error().decode()
  assert "built-in scratch" in msg and "rgk_linear_scan" in msg
