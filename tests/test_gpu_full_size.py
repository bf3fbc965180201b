"""The five benchmark configurations at FULL size, every (batch, head) unit, against the fp32 oracle.

The oracle (oracle/reference_math.py, the restatement pinned to the reference modules' golden outputs) is plain
fp32 torch; here it is evaluated on the GPU, per batch element and per chunk of heads, so that its [heads, Sq, Skv]
temporaries stay bounded -- the math is independent per head.  torch's fp32 matmul on CUDA does not use TF32
unless asked to, and this file makes sure it is off.

Tolerances are the ones stated for this path: 16-bit outputs rtol = atol = 2e-2 against the fp32 reference,
fp32 score vectors rtol 1e-3.
"""
import math

import pytest
import torch

from deepgengraph_b200 import attention as att
from deepgengraph_b200 import layer as L
from oracle import reference_math as rm

pytestmark = pytest.mark.gpu
TOL = dict(rtol=2e-2, atol=2e-2)
STOL = dict(rtol=1e-3, atol=1e-6)


@pytest.fixture(autouse=True)
def _true_fp32_matmul():
  old = torch.backends.cuda.matmul.allow_tf32
  torch.backends.cuda.matmul.allow_tf32 = False
  yield
  torch.backends.cuda.matmul.allow_tf32 = old


def _randn(shape, dev, seed, dtype=torch.bfloat16, scale=1.0):
  g = torch.Generator(device=dev).manual_seed(seed)
  x = torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
  return (x * scale).to(dtype)


def test_config1_reference_case_b1_h32_s1024(cuda_device):
  # config 1 is the reference's own CPU-runnable case: fp32, q, k, v ~ N(0, 1) / sqrt(128).  The kernels take
  # 16-bit inputs, so both sides see the bf16-rounded values; the oracle runs on the CPU as the reference would.
  B, H, S, D = 1, 32, 1024, 128
  q, k, v = (_randn((B, S, H, D), cuda_device, 100 + i, scale=1.0 / math.sqrt(D)) for i in range(3))
  ref = rm.attention_ref(q.cpu(), k.cpu(), v.cpu(), causal=True, want=("out", "lse2"), head_chunk=8)
  out, lse = att.attn_fwd_with_lse(q, k, v, causal=True)
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(lse.cpu(), ref["lse2"], rtol=1e-3, atol=1e-3)


def test_config2_every_unit(cuda_device):
  B, H, S, D = 4, 32, 4096, 128
  q, k, v = (_randn((B, S, H, D), cuda_device, 200 + i) for i in range(3))
  out, lse = att.attn_fwd_with_lse(q, k, v, causal=True)
  for b in range(B):
    ref = rm.attention_ref(q[b:b + 1], k[b:b + 1], v[b:b + 1], causal=True, want=("out", "lse2"), head_chunk=4)
    torch.testing.assert_close(out[b:b + 1].float(), ref["out"], **TOL)
    torch.testing.assert_close(lse[b:b + 1], ref["lse2"], rtol=1e-3, atol=1e-3)


def test_config3_every_unit_h2o_and_roco(cuda_device):
  B, H, S, D = 2, 32, 4096, 128
  q, k, v = (_randn((B, S, H, D), cuda_device, 300 + i) for i in range(3))
  out, s1, s2 = att.attn_score_fwd(q, k, v, want_sq=True)
  out_h2o, s1_h2o = att.attn_score_fwd(q, k, v)
  assert torch.equal(out, out_h2o) and torch.equal(s1, s1_h2o)
  for b in range(B):
    ref = rm.attention_ref(q[b:b + 1], k[b:b + 1], v[b:b + 1], want=("out", "colsum", "colsum_sq"), head_chunk=4)
    torch.testing.assert_close(out[b:b + 1].float(), ref["out"], **TOL)
    torch.testing.assert_close(s1[b:b + 1], ref["colsum"], **STOL)
    torch.testing.assert_close(s2[b:b + 1], ref["colsum_sq"], **STOL)
  torch.testing.assert_close(s1.sum(-1), torch.full((B, H), float(S), device=cuda_device), rtol=1e-4, atol=1e-2)


def test_config4_every_unit_keyformer_gumbel_noise(cuda_device):
  B, H, S, D = 2, 32, 2048, 128
  q, k, v = (_randn((B, S, H, D), cuda_device, 400 + i) for i in range(3))
  g = torch.Generator(device=cuda_device).manual_seed(404)
  u = torch.rand(B, H, S, S, generator=g, device=cuda_device).clamp_min_(1e-7)
  exp_rand = -torch.log(u)               # -log(exp_rand) is then exactly Gumbel(0, 1) noise
  del u
  out, s = att.attn_kf_fwd(q, k, v, exp_rand, tau=1.0)
  for b in range(B):
    ref = rm.attention_ref(q[b:b + 1], k[b:b + 1], v[b:b + 1], exp_rand=exp_rand[b:b + 1], tau=1.0,
                           want=("out", "kf"), head_chunk=4)
    torch.testing.assert_close(out[b:b + 1].float(), ref["out"], **TOL)
    torch.testing.assert_close(s[b:b + 1], ref["kf"], **STOL)


def test_config5_attention_every_unit(cuda_device):
  # B1 S8192, 16 query / 8 kv heads, head_dim 256, window 4096, soft-cap 50: all eight K/V groups
  S, H, Hk, D = 8192, 16, 8, 256
  q = _randn((1, S, H, D), cuda_device, 500, scale=2.0)
  k = _randn((1, S, Hk, D), cuda_device, 501)
  v = _randn((1, S, Hk, D), cuda_device, 502)
  out = att.attn_fwd(q, k, v, window=4096, softcap=50.0)
  ref = rm.attention_ref(q, k, v, causal=True, window=4096, softcap=50.0, head_chunk=2)["out"]
  torch.testing.assert_close(out.float(), ref, **TOL)


def test_config5_layer_all_tokens_against_fp32(cuda_device):
  # The whole decoder layer at config size, every one of the 8192 tokens, against the layer evaluated in fp32 end
  # to end (nothing rounded after the inputs and weights).  The layer is a chain of fourteen bf16 roundings, each of
  # which alone moves the output by 0.004-0.006 rms at these weights (see tests/test_gpu_layer.py): the kernels must
  # be at least as close to fp32, element for element at rtol = atol = 2e-2, as the exact-arithmetic bf16 pipeline is.
  from test_gpu_layer import assert_layer_close
  cfg = L.Gemma2LayerConfig()
  w = L.init_weights(cfg, torch.bfloat16, cuda_device, seed=4)
  x = _randn((1, 8192, cfg.hidden), cuda_device, 503)
  y = L.gemma2_layer(x, w, cfg).float()
  assert torch.isfinite(y).all()
  ref32 = rm.gemma2_layer_ref_fp32(x, w, cfg.as_dict(), head_chunk=2)
  model16 = rm.gemma2_layer_ref(x, w, cfg.as_dict())
  assert_layer_close(y, ref32, model16)
