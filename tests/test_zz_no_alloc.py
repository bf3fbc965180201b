"""b200_attn_score_static: the score variant for callers that may not allocate device memory.

Some hosts of this library cannot call cudaMalloc at the point where they need attention scores -- they run
inside a region where allocation is forbidden, or the device memory is already fully handed out.  For them the
library keeps a fixed 32 MiB scratch array in its own device image.  This test drives that entry point directly
through the C ABI (no torch allocation for scratch) on several calls in a row -- a larger problem first, then
smaller ones with other options -- and checks each result bit for bit against the workspace-taking entry point
(both run the same deterministic kernels) and, within the path's tolerances, against the CPU oracle.  The later
calls prove that whatever an earlier, larger call left in the shared scratch does not leak into later results.
It is collected last on purpose.
"""
import math

import pytest
import torch

from deepgengraph_b200 import _lib
from deepgengraph_b200 import attention as att
from oracle import reference_math as rm

pytestmark = pytest.mark.gpu


def _call_static(q, k, v, want_sq, window=0, softcap=0.0):
  B, Sq, H, D = q.shape
  Skv = k.shape[1]
  out = torch.empty_like(q)
  score = torch.empty(B, H, Skv, dtype=torch.float32, device=q.device)
  score_sq = torch.empty_like(score) if want_sq else None
  st = _lib.load().b200_attn_score_static(
      q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), score.data_ptr(),
      score_sq.data_ptr() if want_sq else None, B, Sq, Skv, H, D, _lib.BF16, 1, window, softcap, 1.0 / math.sqrt(D),
      torch.cuda.current_stream(q.device).cuda_stream)
  return st, out, score, score_sq


def test_static_scratch_entry_point_matches_workspace_entry_point_and_oracle(cuda_device):
  # (seed, (B, Sq, Skv, H), window, softcap): the first call fills far more of the scratch than the later ones use
  calls = ((1, (2, 2304, 2304, 4), 0, 0.0), (2, (2, 512, 512, 3), 0, 0.0), (3, (1, 1000, 1000, 2), 300, 0.0),
           (4, (1, 200, 456, 2), 0, 30.0))
  for seed, (B, Sq, Skv, H), window, softcap in calls:
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, H, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(B, Skv, H, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Skv, H, 128, generator=g).to(torch.bfloat16)
    qd, kd, vd = q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)
    st, out, score, score_sq = _call_static(qd, kd, vd, want_sq=True, window=window, softcap=softcap)
    assert st == 0, _lib.STATUS_NAMES.get(st, st)
    ref_out, ref_score, ref_sq = att.attn_score_fwd(qd, kd, vd, want_sq=True, window=window, softcap=softcap)
    torch.cuda.synchronize()
    assert torch.equal(out, ref_out) and torch.equal(score, ref_score) and torch.equal(score_sq, ref_sq)
    oracle = rm.attention_ref(q, k, v, window=window, softcap=softcap, want=("out", "colsum", "colsum_sq"), head_chunk=2)
    torch.testing.assert_close(out.float().cpu(), oracle["out"], rtol=2e-2, atol=2e-2)
    stol = dict(rtol=1e-3, atol=1e-6) if softcap == 0.0 else dict(rtol=1e-2, atol=1e-5)   # tanh.approx on capped logits
    torch.testing.assert_close(score.cpu(), oracle["colsum"], **stol)
    torch.testing.assert_close(score_sq.cpu(), oracle["colsum_sq"], **stol)


def test_static_scratch_rejects_problems_beyond_its_limit_and_empty_inputs(cuda_device):
  # batch 16 x 32 heads x 4096 needs 48 MiB of scratch: more than the built-in 32 MiB.  Nothing is launched.
  lib = _lib.load()
  assert lib.b200_attn_score_workspace_bytes(16, 4096, 4096, 32) > 32 * 2 ** 20
  dummy = torch.zeros(16, dtype=torch.bfloat16, device=cuda_device)
  p = dummy.data_ptr()
  assert lib.b200_attn_score_static(p, p, p, p, p, None, 16, 4096, 4096, 32, 128, _lib.BF16, 1, 0, 0.0, 0.088, None) == 5
  # an empty batch or no queries is a bad argument at the C ABI (the Python operators return empty results themselves)
  assert lib.b200_attn_score_static(p, p, p, p, p, None, 0, 128, 128, 2, 128, _lib.BF16, 1, 0, 0.0, 0.088, None) == 1
  assert lib.b200_attn_score_static(p, p, p, p, p, None, 1, 0, 128, 2, 128, _lib.BF16, 1, 0, 0.0, 0.088, None) == 1
