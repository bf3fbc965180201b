"""Parity of the score-producing variants (H2O, RoCo, KeyFormer) with the oracle and the golden outputs
of the reference modules.  fp32 score vectors: rtol 1e-3 (the bar stated for this path)."""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import cases  # noqa: E402

from deepgengraph_b200 import attention as att
from oracle import reference_math as rm

pytestmark = pytest.mark.gpu
TOL = dict(rtol=2e-2, atol=2e-2)
STOL = dict(rtol=1e-3, atol=1e-6)


def _randn(shape, dtype, seed):
  return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(dtype)


def _qkv(B, Sq, Skv, H, D, dtype, seed=0, Hk=None):
  Hk = Hk or H
  return (_randn((B, Sq, H, D), dtype, seed + 1), _randn((B, Skv, Hk, D), dtype, seed + 2),
          _randn((B, Skv, Hk, D), dtype, seed + 3))


@pytest.mark.parametrize("name", [n for n, c in cases.CASES.items() if c["model"] in ("h2o", "roco", "kf")])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_golden_cases_of_the_reference_modules(cuda_device, name, dtype):
  c = cases.CASES[name]
  inp = {k: t.to(cuda_device) for k, t in cases.make_inputs(name, dtype).items()}
  g = np.load(os.path.join(HERE, "golden", name + ".npz"))
  # (the grouped-query cases come from the reference's GQA-capable modules, figure/membound/attn.py)
  if c["model"] == "kf":
    outs = att.attn_kf_fwd(inp["q"], inp["k"], inp["v"], inp["exp_rand"], tau=c["tau"])
  else:
    outs = att.attn_score_fwd(inp["q"], inp["k"], inp["v"], want_sq=c["model"] == "roco")
  torch.testing.assert_close(outs[0].float().cpu()[:, ::cases.ROW_STRIDE], torch.from_numpy(g["out_rows"]), **TOL)
  for i, s in enumerate(outs[1:]):
    assert s.dtype == torch.float32
    torch.testing.assert_close(s.cpu(), torch.from_numpy(g[f"score{i}"]), **STOL)


@pytest.mark.parametrize("shape", [(1, 128, 128, 1), (2, 512, 512, 3), (1, 1000, 1000, 2), (1, 200, 456, 2),
                                   (1, 2304, 2304, 2), (1, 1, 300, 2)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_h2o_roco_scores_match_oracle(cuda_device, shape, dtype):
  B, Sq, Skv, H = shape
  q, k, v = _qkv(B, Sq, Skv, H, 128, dtype, seed=sum(shape))
  ref = rm.attention_ref(q, k, v, want=("out", "colsum", "colsum_sq"))
  out, s1, s2 = att.attn_score_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), want_sq=True)
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(s1.cpu(), ref["colsum"], **STOL)
  torch.testing.assert_close(s2.cpu(), ref["colsum_sq"], **STOL)
  # each row of probabilities sums to one: the column sums total the number of queries
  torch.testing.assert_close(s1.sum(-1).cpu(), torch.full((B, H), float(Sq)), rtol=1e-4, atol=1e-3)
  out_b, s1_b = att.attn_score_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
  assert torch.equal(s1, s1_b) and torch.equal(out, out_b)      # same bits with or without the squares, run to run


def test_scores_with_window_and_softcap(cuda_device):
  q, k, v = _qkv(1, 640, 640, 2, 128, torch.bfloat16, seed=3)
  q = (q.float() * 20).to(torch.bfloat16)
  ref = rm.attention_ref(q, k, v, window=200, softcap=30.0, want=("out", "colsum"))
  out, s = att.attn_score_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), window=200, softcap=30.0)
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(s.cpu(), ref["colsum"], rtol=5e-3, atol=1e-5)   # tanh.approx on capped logits


@pytest.mark.parametrize("shape,tau", [((1, 128, 128, 1), 1.0), ((2, 448, 448, 2), 1.5), ((1, 200, 456, 2), 1.0),
                                       ((1, 1100, 1100, 2), 0.7)])
def test_keyformer_scores_match_oracle(cuda_device, shape, tau):
  B, Sq, Skv, H = shape
  q, k, v = _qkv(B, Sq, Skv, H, 128, torch.bfloat16, seed=sum(shape))
  u = torch.rand(B, H, Sq, Skv, generator=torch.Generator().manual_seed(11)).clamp_min(1e-7)
  exp_rand = -torch.log(u)             # -log(exp_rand) is then exactly Gumbel(0, 1) noise
  ref = rm.attention_ref(q, k, v, exp_rand=exp_rand, tau=tau, want=("out", "kf"))
  out, s = att.attn_kf_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), exp_rand.to(cuda_device), tau=tau)
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(s.cpu(), ref["kf"], **STOL)
  torch.testing.assert_close(s.sum(-1).cpu(), torch.full((B, H), float(Sq)), rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_snapkv_and_corm_golden_cases_of_the_reference_modules(cuda_device, dtype):
  inp = {k: t.to(cuda_device) for k, t in cases.make_inputs("snapkv_s192", dtype).items()}
  g = np.load(os.path.join(HERE, "golden", "snapkv_s192.npz"))
  out, pooled = att.attn_snapkv_fwd(inp["q"], inp["k"], inp["v"], kernel_size=5)
  torch.testing.assert_close(out.float().cpu()[:, ::cases.ROW_STRIDE], torch.from_numpy(g["out_rows"]), **TOL)
  torch.testing.assert_close(pooled.cpu(), torch.from_numpy(g["score0"]), **STOL)
  inp = {k: t.to(cuda_device) for k, t in cases.make_inputs("corm_s192", dtype).items()}
  g = np.load(os.path.join(HERE, "golden", "corm_s192.npz"))
  out, flags = att.attn_corm_fwd(inp["q"], inp["k"], inp["v"])
  assert flags.dtype == torch.bool and tuple(flags.shape) == (1, 2, 192)
  torch.testing.assert_close(out.float().cpu()[:, ::cases.ROW_STRIDE], torch.from_numpy(g["out_rows"]), **TOL)
  # exact thresholds: allow a flip only where a probability sits within rounding of 1 / (i + 1)
  assert (flags.cpu().numpy() != g["score0"]).mean() <= 0.01


def test_snapkv_grouped_query_golden_case_of_the_reference_module(cuda_device):
  inp = {k: t.to(cuda_device) for k, t in cases.make_inputs("snapkv_gqa_s192", torch.bfloat16).items()}
  g = np.load(os.path.join(HERE, "golden", "snapkv_gqa_s192.npz"))
  out, pooled = att.attn_snapkv_fwd(inp["q"], inp["k"], inp["v"], kernel_size=5)
  torch.testing.assert_close(out.float().cpu()[:, ::cases.ROW_STRIDE], torch.from_numpy(g["out_rows"]), **TOL)
  torch.testing.assert_close(pooled.cpu(), torch.from_numpy(g["score0"]), **STOL)


@pytest.mark.parametrize("shape", [(1, 640, 640, 2), (2, 300, 300, 3), (1, 1500, 1500, 2)])
def test_snapkv_and_corm_match_oracle(cuda_device, shape):
  B, Sq, Skv, H = shape
  q, k, v = _qkv(B, Sq, Skv, H, 128, torch.bfloat16, seed=sum(shape) + 5)
  ref = rm.attention_ref(q, k, v, want=("out", "snapkv", "corm", "colsum"))
  out, pooled = att.attn_snapkv_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
  torch.testing.assert_close(pooled.cpu(), ref["snapkv"], **STOL)
  out2, flags = att.attn_corm_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
  torch.testing.assert_close(out2.float().cpu(), ref["out"], **TOL)
  assert (flags.cpu() != ref["corm"]).float().mean().item() <= 0.01
  assert flags.any() and not flags.all()


def test_config3_slice_full_length(cuda_device):
  q, k, v = _qkv(1, 4096, 4096, 2, 128, torch.bfloat16, seed=12)
  ref = rm.attention_ref(q, k, v, want=("out", "colsum"), head_chunk=1)
  out, s = att.attn_score_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(s.cpu(), ref["colsum"], **STOL)


def test_config4_slice_full_length(cuda_device):
  q, k, v = _qkv(1, 2048, 2048, 2, 128, torch.bfloat16, seed=13)
  u = torch.rand(1, 2, 2048, 2048, generator=torch.Generator().manual_seed(14)).clamp_min(1e-7)
  exp_rand = -torch.log(u)
  ref = rm.attention_ref(q, k, v, exp_rand=exp_rand, tau=1.0, want=("out", "kf"), head_chunk=1)
  out, s = att.attn_kf_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), exp_rand.to(cuda_device), tau=1.0)
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(s.cpu(), ref["kf"], **STOL)


@pytest.mark.parametrize("shape", [(1, 512, 512, 4, 2), (2, 384, 640, 6, 2), (1, 1024, 1024, 8, 1)])
def test_grouped_query_scores_are_the_group_mean(cuda_device, shape):
  # heads > kv heads: probabilities averaged over the query heads of a K/V head, then summed over the queries
  # (the group_size > 1 branch of kernels/roco.py:39-40, never run by the reference's own modules)
  B, Sq, Skv, H, Hk = shape
  q = _randn((B, Sq, H, 128), torch.bfloat16, 41)
  k = _randn((B, Skv, Hk, 128), torch.bfloat16, 42)
  v = _randn((B, Skv, Hk, 128), torch.bfloat16, 43)
  ref = rm.attention_ref(q, k, v, causal=True, want=("out", "colsum"))
  out, score = att.attn_score_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
  assert score.shape == (B, Hk, Skv)
  torch.testing.assert_close(out.float().cpu(), ref["out"], rtol=2e-2, atol=2e-2)
  torch.testing.assert_close(score.cpu(), ref["colsum"], **STOL)
  torch.testing.assert_close(score.sum(dim=-1).cpu(), torch.full((B, Hk), float(Sq)), rtol=1e-3, atol=1e-3)


GQA_SHAPES = [
    # B, Sq, Skv, H, Hk
    (1, 512, 512, 4, 2),
    (2, 384, 640, 6, 2),        # kv longer than q, three query heads per K/V head
    (1, 1000, 1000, 8, 1),      # ragged tiles, eight query heads on one K/V head
    (1, 4352, 4352, 2, 1),      # more than one chunk of query blocks per key tile
]


@pytest.mark.parametrize("shape", GQA_SHAPES)
def test_grouped_query_squares_and_corm_use_the_group_mean(cuda_device, shape):
  # mean over the query heads of a K/V head BEFORE the square / the threshold test (kernels/roco.py:39-46,
  # figure/membound/attn.py:123-131,240-242)
  B, Sq, Skv, H, Hk = shape
  q, k, v = _qkv(B, Sq, Skv, H, 128, torch.bfloat16, seed=sum(shape), Hk=Hk)
  ref = rm.attention_ref(q, k, v, causal=True, want=("out", "colsum", "colsum_sq", "corm"), head_chunk=4)
  qd, kd, vd = q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)
  out, s1, s2 = att.attn_score_fwd(qd, kd, vd, want_sq=True)
  assert s1.shape == (B, Hk, Skv) and s2.shape == (B, Hk, Skv)
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(s1.cpu(), ref["colsum"], **STOL)
  torch.testing.assert_close(s2.cpu(), ref["colsum_sq"], **STOL)
  out_b, s1_b, s2_b = att.attn_score_fwd(qd, kd, vd, want_sq=True)
  assert torch.equal(s1, s1_b) and torch.equal(s2, s2_b)        # run to run the same bits
  out_c, flags = att.attn_corm_fwd(qd, kd, vd)
  assert flags.shape == (B, Hk, Skv) and flags.dtype == torch.bool and torch.equal(out_c, out)
  assert (flags.cpu() != ref["corm"]).float().mean().item() <= 0.01
  assert flags.any() and not flags.all()


def test_grouped_query_squares_with_window_and_softcap(cuda_device):
  q, k, v = _qkv(1, 640, 640, 4, 128, torch.bfloat16, seed=77, Hk=2)
  q = (q.float() * 20).to(torch.bfloat16)
  ref = rm.attention_ref(q, k, v, window=200, softcap=30.0, want=("out", "colsum", "colsum_sq"))
  out, s1, s2 = att.attn_score_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), want_sq=True, window=200,
                                   softcap=30.0)
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(s1.cpu(), ref["colsum"], rtol=5e-3, atol=1e-5)   # tanh.approx on capped logits
  torch.testing.assert_close(s2.cpu(), ref["colsum_sq"], rtol=1e-2, atol=1e-5)


@pytest.mark.parametrize("shape,tau", [((1, 448, 448, 4, 2), 1.0), ((2, 200, 456, 6, 2), 1.5)])
def test_grouped_query_keyformer_score_is_the_group_mean(cuda_device, shape, tau):
  B, Sq, Skv, H, Hk = shape
  q, k, v = _qkv(B, Sq, Skv, H, 128, torch.bfloat16, seed=sum(shape), Hk=Hk)
  exp_rand = -torch.log(torch.rand(B, H, Sq, Skv, generator=torch.Generator().manual_seed(12)).clamp_min(1e-7))
  ref = rm.attention_ref(q, k, v, exp_rand=exp_rand, tau=tau, want=("out", "kf"))
  out, s = att.attn_kf_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), exp_rand.to(cuda_device), tau=tau)
  assert s.shape == (B, Hk, Skv)
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(s.cpu(), ref["kf"], **STOL)
