"""Unwritten-region and out-of-bounds checks through the C ABI: outputs, the LSE vector and the scratch workspace are
filled with NaN (and the outputs are followed by a guard band) before the call.  Every element of the outputs must
have been written, nothing past their end may change, and results may not depend on what the scratch held."""
import ctypes
import math

import pytest
import torch

from deepgengraph_b200 import _lib
from deepgengraph_b200 import attention as att

pytestmark = pytest.mark.gpu
GUARD = 4096   # elements


def _guarded(shape, dtype, device):
  n = math.prod(shape)
  flat = torch.full((n + GUARD,), float("nan"), dtype=dtype, device=device)
  return flat, flat[:n].view(shape)


def _stream(dev):
  return torch.cuda.current_stream(dev).cuda_stream


@pytest.mark.parametrize("shape", [(1, 300, 300, 3, 3, 128), (2, 200, 456, 4, 2, 128), (1, 130, 257, 2, 1, 256),
                                   (3, 1000, 1000, 40, 40, 128)])
def test_attention_writes_every_output_element_and_nothing_else(cuda_device, shape):
  B, Sq, Skv, H, Hk, D = shape
  g = torch.Generator().manual_seed(sum(shape))
  q = torch.randn(B, Sq, H, D, generator=g).to(torch.bfloat16).to(cuda_device)
  k = torch.randn(B, Skv, Hk, D, generator=g).to(torch.bfloat16).to(cuda_device)
  v = torch.randn(B, Skv, Hk, D, generator=g).to(torch.bfloat16).to(cuda_device)
  out_flat, out = _guarded((B, Sq, H, D), torch.bfloat16, cuda_device)
  lse_flat, lse = _guarded((B, H, Sq), torch.float32, cuda_device)
  st = _lib.load().b200_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, Sq, Skv, H,
                                 Hk, D, _lib.BF16, 1, 0, 0.0, 1.0 / math.sqrt(D), _stream(cuda_device))
  assert st == 0, _lib.STATUS_NAMES.get(st, st)
  torch.cuda.synchronize()
  assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
  assert torch.isnan(out_flat[out.numel():].float()).all() and torch.isnan(lse_flat[lse.numel():]).all()
  assert torch.equal(out, att.attn_fwd(q, k, v))


def test_scores_do_not_depend_on_scratch_contents(cuda_device):
  B, S, H, D = 2, 700, 3, 128
  g = torch.Generator().manual_seed(5)
  q, k, v = (torch.randn(B, S, H, D, generator=g).to(torch.bfloat16).to(cuda_device) for _ in range(3))
  lib = _lib.load()
  nbytes = lib.b200_attn_score_workspace_bytes(B, S, S, H)
  results = []
  for fill in (float("nan"), 0.0, 1e30):
    ws = torch.full((nbytes // 4 + 64,), fill, dtype=torch.float32, device=cuda_device)
    out_flat, out = _guarded((B, S, H, D), torch.bfloat16, cuda_device)
    s_flat, score = _guarded((B, H, S), torch.float32, cuda_device)
    q_flat, score_sq = _guarded((B, H, S), torch.float32, cuda_device)
    st = lib.b200_attn_score(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), score.data_ptr(),
                             score_sq.data_ptr(), ws.data_ptr(), nbytes, B, S, S, H, D, _lib.BF16, 1, 0, 0.0,
                             1.0 / math.sqrt(D), _stream(cuda_device))
    assert st == 0, _lib.STATUS_NAMES.get(st, st)
    torch.cuda.synchronize()
    for flat, t in ((out_flat, out), (s_flat, score), (q_flat, score_sq)):
      assert torch.isfinite(t.float()).all()
      assert torch.isnan(flat[t.numel():].float()).all()
    tail = ws[nbytes // 4:]
    assert (torch.isnan(tail).all() if math.isnan(fill) else (tail == fill).all())   # nothing past the stated size
    results.append((out.clone(), score.clone(), score_sq.clone()))
  for r in results[1:]:
    assert all(torch.equal(a, b) for a, b in zip(results[0], r))


def test_eviction_writes_exactly_its_cache(cuda_device):
  B, S, H, D, budget = 2, 900, 3, 128, 100
  g = torch.Generator().manual_seed(6)
  score = torch.rand(B, H, S, generator=g).to(cuda_device)
  k = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16).to(cuda_device)
  v = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16).to(cuda_device)
  cache_flat, cache = _guarded((B, 2, budget, H, D), torch.bfloat16, cuda_device)
  st = _lib.load().b200_kv_evict_topk(score.data_ptr(), k.data_ptr(), v.data_ptr(), cache.data_ptr(), None, B, S, H, D,
                                      budget, _lib.BF16, _stream(cuda_device))
  assert st == 0, _lib.STATUS_NAMES.get(st, st)
  torch.cuda.synchronize()
  assert torch.isfinite(cache.float()).all() and torch.isnan(cache_flat[cache.numel():].float()).all()
  assert torch.equal(cache, att.kv_evict_topk(score, k, v, budget))
