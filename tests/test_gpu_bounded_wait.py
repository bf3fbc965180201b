"""Failure detection without a GPU fault: a device-side wait that nothing will ever satisfy runs out after its
limit, the kernel returns normally, the host reads the recorded status, and the device keeps working."""
import ctypes

import pytest
import torch

from deepgengraph_b200 import _lib
from deepgengraph_b200 import attention as att

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_the_device_stays_usable(cuda_device):
  lib = _lib.load()
  word = ctypes.c_int(0)
  assert lib.b200_device_status(ctypes.byref(word)) == 0 and word.value == 0
  gave_up = torch.zeros(1, dtype=torch.int32, device=cuda_device)
  assert lib.b200_selftest_bounded_wait(50, gave_up.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
  st = lib.b200_device_status(ctypes.byref(word))          # synchronises
  assert st == 7 and (word.value & 0xff) == 17             # B200_ERR_DEVICE_TIMEOUT, code WAIT_SELFTEST
  assert gave_up.item() == 1
  # the word was cleared by the read, and kernels run normally afterwards
  assert lib.b200_device_status(ctypes.byref(word)) == 0 and word.value == 0
  q = torch.randn(1, 256, 2, 128, device=cuda_device, dtype=torch.bfloat16)
  out = att.attn_fwd(q, q, q)
  assert torch.isfinite(out.float()).all()
  assert lib.b200_device_status(ctypes.byref(word)) == 0 and word.value == 0


def test_launches_drain_while_the_status_word_is_set(cuda_device):
  # a kernel that follows an expired wait returns at once (its output stays untouched) until the host has read
  # and cleared the status word
  lib = _lib.load()
  word = ctypes.c_int(0)
  lib.b200_selftest_bounded_wait(20, None, torch.cuda.current_stream().cuda_stream)
  torch.cuda.synchronize()
  q = torch.randn(1, 256, 2, 128, device=cuda_device, dtype=torch.bfloat16)
  out = torch.full_like(q, 7.0)
  st = lib.b200_attn_fwd(q.data_ptr(), q.data_ptr(), q.data_ptr(), out.data_ptr(), None, 1, 256, 256, 2, 2, 128,
                         _lib.BF16, 1, 0, 0.0, 0.088, torch.cuda.current_stream().cuda_stream)
  assert st == 0
  torch.cuda.synchronize()
  assert torch.all(out == 7.0)
  assert lib.b200_device_status(ctypes.byref(word)) == 7
  ok = att.attn_fwd(q, q, q)
  assert torch.isfinite(ok.float()).all() and not torch.all(ok == 7.0)
  assert lib.b200_device_status(ctypes.byref(word)) == 0
