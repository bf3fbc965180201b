import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cuda_device():
  import torch
  if not torch.cuda.is_available():
    pytest.skip("no CUDA device")
  return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_clean(request):
  """After every GPU test: no bounded device-side wait may have expired."""
  yield
  if request.node.get_closest_marker("gpu") is None:
    return
  import ctypes
  from deepgengraph_b200 import _lib
  word = ctypes.c_int(0)
  st = _lib.load().b200_device_status(ctypes.byref(word))
  assert st == 0 and word.value == 0, f"device status word = {word.value:#x} (a bounded wait expired)"
