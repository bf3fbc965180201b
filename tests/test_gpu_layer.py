"""Gemma-2-style decoder layer (config 5 shapes scaled down, and the attention part at full size) against the
fp32 oracle restatement."""
import pytest
import torch

from deepgengraph_b200 import attention as att
from deepgengraph_b200 import layer as L
from oracle import reference_math as rm

pytestmark = pytest.mark.gpu


def assert_layer_close(got, ref):
  """A chain of a dozen 16-bit ops: single-ulp flips of intermediate bf16 values (GEMM summation order) move a
  small fraction of the outputs by a few ulps.  Bar: relative Frobenius error < 1e-2 (bf16 rounds at 2^-9 = 2e-3 per op), at most 2 % of the
  elements outside rtol = atol = 2e-2, and no element off by more than 0.1 * (1 + |ref|)."""
  diff = (got - ref).abs()
  assert (diff.norm() / ref.norm()).item() < 1e-2
  outside = (diff > 2e-2 + 2e-2 * ref.abs()).float().mean().item()
  assert outside < 2e-2, outside
  assert (diff / (1 + ref.abs())).max().item() < 0.1


@pytest.mark.parametrize("S,window", [(384, 128), (600, 4096)])
def test_layer_matches_oracle_small(cuda_device, S, window):
  cfg = L.Gemma2LayerConfig(hidden=512, heads=4, kv_heads=2, head_dim=256, window=window, intermediate=1024)
  w = L.init_weights(cfg, torch.bfloat16, cuda_device, seed=1, std=0.05)
  x = torch.randn(1, S, cfg.hidden, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
  y = L.gemma2_layer(x.to(cuda_device), w, cfg)
  ref = rm.gemma2_layer_ref(x, {k: t.cpu() for k, t in w.items()}, cfg.as_dict())
  assert_layer_close(y.float().cpu(), ref)


def test_config5_attention_full_size_slice(cuda_device):
  # S 8192, head_dim 256, window 4096, softcap 50, GQA 2:1 -- one kv group (2 query heads) against the oracle
  S, D = 8192, 256
  g = torch.Generator().manual_seed(3)
  q = (torch.randn(1, S, 2, D, generator=g) * 2).to(torch.bfloat16)
  k = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
  v = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
  ref = rm.attention_ref(q, k, v, causal=True, window=4096, softcap=50.0, head_chunk=1)["out"]
  out = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), window=4096, softcap=50.0)
  torch.testing.assert_close(out.float().cpu(), ref, rtol=2e-2, atol=2e-2)


def test_config5_layer_full_size_runs_and_is_finite(cuda_device):
  cfg = L.Gemma2LayerConfig()
  w = L.init_weights(cfg, torch.bfloat16, cuda_device, seed=4)
  x = torch.randn(1, 8192, cfg.hidden, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(cuda_device)
  y = L.gemma2_layer(x, w, cfg)
  assert y.shape == x.shape and torch.isfinite(y.float()).all()
  # first 256 tokens only depend on themselves (causal): compare that prefix with the oracle on the prefix
  ref = rm.gemma2_layer_ref(x[:, :256].cpu(), {k: t.cpu() for k, t in w.items()}, cfg.as_dict())
  assert_layer_close(y[:, :256].float().cpu(), ref)
