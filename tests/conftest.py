import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
  from oracle import oracle as o
  o.lib()
  return o


@pytest.fixture(autouse=True)
def _no_kernel_gave_up(request):
  """After every GPU test: no kernel launched through the package may have left a raised status word
  behind (a bounded wait that expired, or - on the range-checked build - an index outside its
  array).  Tests that raise the word on purpose read it themselves, which clears it."""
  yield
  if request.node.get_closest_marker("gpu") is None:
    return
  import sys
  lib = sys.modules.get("recurrentgemma_b200._lib")
  if lib is not None and lib._lib is not None:
    lib.check_status()
