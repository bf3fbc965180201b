"""b200_attn_score_static: the score variant for callers that may not allocate device memory.

Some hosts of this library cannot call cudaMalloc at the point where they need attention scores -- they run
inside a region where allocation is forbidden, or the device memory is already fully handed out.  For them the
library keeps a fixed 32 MiB scratch array in its own device image.  This test drives that entry point directly
through the C ABI (no torch allocation for scratch) and checks, on two calls in a row with different inputs, that
it returns what the workspace-taking entry point returns -- the second call proves that whatever the first call
left in the shared scratch does not leak into later results.  It is collected last on purpose.
"""
import ctypes
import math

import pytest
import torch

from deepgengraph_b200 import _lib
from deepgengraph_b200 import attention as att

pytestmark = pytest.mark.gpu


def _call_static(q, k, v, want_sq):
  B, Sq, H, D = q.shape
  Skv = k.shape[1]
  out = torch.empty_like(q)
  score = torch.empty(B, H, Skv, dtype=torch.float32, device=q.device)
  score_sq = torch.empty_like(score) if want_sq else None
  st = _lib.load().b200_attn_score_static(
      q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), score.data_ptr(),
      score_sq.data_ptr() if want_sq else None, B, Sq, Skv, H, D, _lib.BF16, 1, 0, 0.0, 1.0 / math.sqrt(D),
      torch.cuda.current_stream(q.device).cuda_stream)
  return st, out, score, score_sq


def test_static_scratch_entry_point_matches_workspace_entry_point(cuda_device):
  for seed, (B, S, H) in ((1, (2, 512, 3)), (2, (1, 1000, 2))):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, S, H, 128, generator=g).to(torch.bfloat16).to(cuda_device) for _ in range(3))
    st, out, score, score_sq = _call_static(q, k, v, want_sq=True)
    assert st == 0, _lib.STATUS_NAMES.get(st, st)
    ref_out, ref_score, ref_sq = att.attn_score_fwd(q, k, v, want_sq=True)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), ref_out.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(score, ref_score, rtol=1e-3, atol=1e-6)
    torch.testing.assert_close(score_sq, ref_sq, rtol=1e-3, atol=1e-6)


def test_static_scratch_rejects_problems_beyond_its_limit(cuda_device):
  # batch 16 x 32 heads x 4096 needs 48 MiB of scratch: more than the built-in 32 MiB.  Nothing is launched.
  assert _lib.load().b200_attn_score_workspace_bytes(16, 4096, 4096, 32) > 32 * 2 ** 20
  dummy = torch.zeros(16, dtype=torch.bfloat16, device=cuda_device)
  st = _lib.load().b200_attn_score_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                          dummy.data_ptr(), None, 16, 4096, 4096, 32, 128, _lib.BF16, 1, 0, 0.0, 0.088,
                                          None)
  assert st == 5   # B200_ERR_WORKSPACE
