"""KV-cache eviction (top-`budget` keys by score, position order, gathered K/V rows) against the oracle's verbatim
restatement of the reference's topk -> sort -> gather.  Index work: bit-exact."""
import pytest
import torch

from deepgengraph_b200 import attention as att
from oracle import reference_math as rm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,budget", [((1, 4096, 32, 128), 512), ((2, 1000, 3, 128), 1), ((2, 1000, 3, 128), 1000),
                                           ((1, 777, 2, 64), 300), ((1, 2048, 4, 256), 512)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_matches_topk_sort_gather(cuda_device, shape, budget, dtype):
  B, S, H, D = shape
  g = torch.Generator().manual_seed(S + budget)
  score = torch.rand(B, H, S, generator=g) * 10 - 2          # distinct values with overwhelming probability
  k = torch.randn(B, S, H, D, generator=g).to(dtype)
  v = torch.randn(B, S, H, D, generator=g).to(dtype)
  ref_cache, ref_idx = rm.kv_evict_topk_ref(score, k, v, budget)
  cache, idx = att.kv_evict_topk(score.to(cuda_device), k.to(cuda_device), v.to(cuda_device), budget,
                                 return_indices=True)
  assert torch.equal(idx.cpu().long(), ref_idx)
  assert torch.equal(cache.cpu(), ref_cache)


def test_scores_from_the_fused_kernel_and_ties(cuda_device):
  # end to end: H2O scores from the fused kernel feed the eviction, as in the reference's model glue
  g = torch.Generator().manual_seed(3)
  q, k, v = (torch.randn(1, 1024, 2, 128, generator=g).to(torch.bfloat16).to(cuda_device) for _ in range(3))
  _, score = att.attn_score_fwd(q, k, v)
  cache, idx = att.kv_evict_topk(score, k, v, 256, return_indices=True)
  ref_cache, ref_idx = rm.kv_evict_topk_ref(score.cpu(), k.cpu(), v.cpu(), 256)
  assert torch.equal(idx.cpu().long(), ref_idx) and torch.equal(cache.cpu(), ref_cache)
  # ties: all scores equal -> any `budget` keys are a valid top-k; this kernel keeps the lowest positions
  flat = torch.ones(1, 2, 500, device=cuda_device)
  kk = torch.randn(1, 500, 2, 128, device=cuda_device, dtype=torch.bfloat16)
  cache, idx = att.kv_evict_topk(flat, kk, kk, 100, return_indices=True)
  assert torch.equal(idx.cpu(), torch.arange(100, dtype=torch.int32).expand(1, 2, 100))
  assert torch.equal(cache[:, 0], kk[:, :100])
  # negative values and zeros order correctly
  sc = torch.tensor([[[-3.0, 0.0, -0.0, 5.0, -1.0, 2.0, -7.0, 1.0]]], device=cuda_device)
  kk = torch.randn(1, 8, 1, 128, device=cuda_device, dtype=torch.bfloat16)
  _, idx = att.kv_evict_topk(sc, kk, kk, 3, return_indices=True)
  assert idx.cpu().tolist() == [[[3, 5, 7]]]


def _roco_stats(B, H, Sq, S, seed):
  g = torch.Generator().manual_seed(seed)
  logits = torch.randn(B, H, Sq, S, generator=g) * 2
  mask = torch.triu(torch.full((Sq, S), float("-inf")), diagonal=S - Sq + 1)
  p = torch.softmax(logits + mask, dim=-1)
  return p.sum(dim=2).contiguous(), (p * p).sum(dim=2).contiguous()


@pytest.mark.parametrize("shape,budget,recent", [((1, 2048, 4, 128), 512, 32), ((2, 1000, 3, 128), 100, 1),
                                                  ((1, 777, 2, 64), 0, 50), ((1, 640, 2, 256), 600, 40),
                                                  ((1, 512, 2, 128), 64, 0)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_roco_selection_matches_the_reference_sequence(cuda_device, shape, budget, recent, dtype):
  B, S, H, D = shape
  score, score_sq = _roco_stats(B, H, S, S, seed=S + budget)
  g = torch.Generator().manual_seed(recent)
  k = torch.randn(B, S, H, D, generator=g).to(dtype)
  v = torch.randn(B, S, H, D, generator=g).to(dtype)
  ref_cache, ref_idx = rm.kv_evict_roco_ref(score, score_sq, k, v, S, budget, recent)
  cache, idx = att.kv_evict_roco(score.to(cuda_device), score_sq.to(cuda_device), k.to(cuda_device),
                                 v.to(cuda_device), S, budget, recent, return_indices=True)
  assert torch.equal(idx.cpu().long(), ref_idx)
  assert torch.equal(cache.cpu(), ref_cache)


def test_roco_end_to_end_with_the_fused_scores(cuda_device):
  # column sums of p and p^2 from the fused kernel feed the selection, as in models/roco.py:45-66
  g = torch.Generator().manual_seed(5)
  q, k, v = (torch.randn(1, 1024, 2, 128, generator=g).to(torch.bfloat16).to(cuda_device) for _ in range(3))
  _, score, score_sq = att.attn_score_fwd(q, k, v, want_sq=True)
  cache, idx = att.kv_evict_roco(score, score_sq, k, v, 1024, 256, 32, return_indices=True)
  ref_cache, ref_idx = rm.kv_evict_roco_ref(score.cpu(), score_sq.cpu(), k.cpu(), v.cpu(), 1024, 256, 32)
  assert torch.equal(idx.cpu().long(), ref_idx) and torch.equal(cache.cpu(), ref_cache)
  with pytest.raises(RuntimeError):
    att.kv_evict_roco(score, score_sq, k, v, 1024, 1000, 100)      # keeps more keys than there are


def test_vectors_too_long_for_shared_memory_staging(cuda_device):
  # above ~50k keys (top-k) / ~22k keys (RoCo) the order keys no longer fit in shared memory beside the index
  # list and every pass re-reads the scores instead
  g = torch.Generator().manual_seed(77)
  B, S, H, D = 1, 52000, 1, 64
  score = torch.rand(B, H, S, generator=g) * 10 - 2
  k = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
  ref_cache, ref_idx = rm.kv_evict_topk_ref(score, k, k, 100)
  cache, idx = att.kv_evict_topk(score.to(cuda_device), k.to(cuda_device), k.to(cuda_device), 100, return_indices=True)
  assert torch.equal(idx.cpu().long(), ref_idx) and torch.equal(cache.cpu(), ref_cache)
  S, Sq = 30000, 64
  score, score_sq = _roco_stats(B, H, Sq, S, seed=78)
  k = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
  ref_cache, ref_idx = rm.kv_evict_roco_ref(score, score_sq, k, k, Sq, 200, 20)
  cache, idx = att.kv_evict_roco(score.to(cuda_device), score_sq.to(cuda_device), k.to(cuda_device), k.to(cuda_device),
                                 Sq, 200, 20, return_indices=True)
  assert torch.equal(idx.cpu().long(), ref_idx) and torch.equal(cache.cpu(), ref_cache)


@pytest.mark.parametrize("seq,budget", [(11500, 100), (11600, 12), (11700, 300), (12000, 100), (39936, 12288), (50000, 12288)])
def test_shared_memory_sizes_around_the_opt_in_threshold(cuda_device, seq, budget):
  # dynamic shared memory = 4 * budget (+ the padded key array while it fits): sizes just below and just above the
  # 48 KB default limit (which static and dynamic shared memory share), the largest budget with the keys left in
  # global memory, and a sequence beyond what shared memory can stage
  g = torch.Generator().manual_seed(seq + budget)
  score = torch.rand(1, 1, seq, generator=g)
  k = torch.randn(1, seq, 1, 64, generator=g).to(torch.bfloat16)
  ref_cache, ref_idx = rm.kv_evict_topk_ref(score, k, k, budget)
  cache, idx = att.kv_evict_topk(score.to(cuda_device), k.to(cuda_device), k.to(cuda_device), budget,
                                 return_indices=True)
  assert torch.equal(idx.cpu().long(), ref_idx) and torch.equal(cache.cpu(), ref_cache)


def test_fp32_and_16bit_rows_alternate_at_a_long_sequence(cuda_device):
  # each element width is its own kernel with its own shared-memory opt-in: a 16-bit call must not satisfy the
  # fp32 kernel's set-up, nor the other way round
  seq, budget = 20000, 64
  g = torch.Generator().manual_seed(5)
  score = torch.rand(1, 2, seq, generator=g)
  sq = score * score / 7 + torch.rand(1, 2, seq, generator=g) * 1e-3
  for dtype in (torch.bfloat16, torch.float32, torch.float16, torch.float32):
    k = torch.randn(1, seq, 2, 64, generator=g).to(dtype)
    ref_cache, ref_idx = rm.kv_evict_topk_ref(score, k, k, budget)
    cache, idx = att.kv_evict_topk(score.to(cuda_device), k.to(cuda_device), k.to(cuda_device), budget,
                                   return_indices=True)
    assert torch.equal(idx.cpu().long(), ref_idx) and torch.equal(cache.cpu(), ref_cache)
    ref_cache, ref_idx = rm.kv_evict_roco_ref(score, sq, k, k, 7, budget, 16)
    cache, idx = att.kv_evict_roco(score.to(cuda_device), sq.to(cuda_device), k.to(cuda_device), k.to(cuda_device), 7,
                                   budget, 16, return_indices=True)
    assert torch.equal(idx.cpu().long(), ref_idx) and torch.equal(cache.cpu(), ref_cache)
