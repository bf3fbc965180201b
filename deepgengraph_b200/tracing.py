"""Optional NVTX ranges around the library's operators.

The reference's tracing hooks are empty stubs (profile_start / profile_stop with the cudaProfilerStart calls
commented out, deepgengraph_exp/utils.py:34-47).  Here every public operator can be bracketed by an NVTX range named
after it, so that a timeline tool shows which launches belong to which call.  Off by default (a range costs a few
hundred nanoseconds of host time per call); switched on with B200_NVTX=1 in the environment or `enable(True)`.
"""
import functools
import os

import torch

_enabled = os.environ.get("B200_NVTX", "0") not in ("", "0")


def enable(on: bool = True) -> None:
  global _enabled
  _enabled = bool(on)


def enabled() -> bool:
  return _enabled


def traced(fn):
  """Decorator: run `fn` inside an NVTX range `b200::<name>` when tracing is on."""
  name = "b200::" + fn.__name__

  @functools.wraps(fn)
  def wrapper(*args, **kwargs):
    if not _enabled:
      return fn(*args, **kwargs)
    torch.cuda.nvtx.range_push(name)
    try:
      return fn(*args, **kwargs)
    finally:
      torch.cuda.nvtx.range_pop()

  return wrapper
