"""KeyFormer with the noise generated inside the kernels (attn_kf_fwd(..., exp_rand=None, seed=...)) against the
tensor-input path and the CPU oracle fed the SAME noise, materialised by the host function kf_noise.
fp32 score vectors: rtol 1e-3, the bar stated for this path."""
import pytest
import torch

from deepgengraph_b200 import attention as att
from oracle import reference_math as rm

pytestmark = pytest.mark.gpu
TOL = dict(rtol=2e-2, atol=2e-2)
STOL = dict(rtol=1e-3, atol=1e-6)


def _randn(shape, seed):
  return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)


def test_fill_kernel_writes_the_host_functions_tensor(cuda_device):
  for seed, (B, H, Sq, Skv) in ((3, (2, 3, 70, 130)), (1 << 40, (1, 2, 33, 64))):
    host = att.kf_noise(seed, B, H, Sq, Skv)
    dev = att.kf_noise_fill(seed, B, H, Sq, Skv, cuda_device).cpu()
    # both take the logarithm in double precision and round once: equal up to a rare double-rounding flip
    assert (host != dev).float().mean().item() < 1e-4
    torch.testing.assert_close(dev, host, rtol=2e-7, atol=0)
    torch_dev = att.kf_noise(seed, B, H, Sq, Skv, device=cuda_device).cpu()
    torch.testing.assert_close(torch_dev, host, rtol=2e-7, atol=0)


SHAPES = [
    # B, Sq, Skv, H, Hk, tau
    (1, 128, 128, 1, 1, 1.0),
    (2, 448, 448, 2, 2, 1.5),
    (1, 200, 456, 2, 2, 1.0),        # ragged, kv longer than q
    (1, 2304, 2304, 2, 2, 0.7),      # more than one chunk of query blocks per key tile
    (1, 384, 640, 6, 2, 1.0),        # grouped K/V heads: score = mean over the group
]


@pytest.mark.parametrize("shape", SHAPES)
def test_seeded_keyformer_matches_oracle_and_tensor_path(cuda_device, shape):
  B, Sq, Skv, H, Hk, tau = shape
  seed = 1000 + sum(shape[:5])
  q, k, v = _randn((B, Sq, H, 128), seed + 1), _randn((B, Skv, Hk, 128), seed + 2), _randn((B, Skv, Hk, 128), seed + 3)
  qd, kd, vd = q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)
  out, s = att.attn_kf_fwd(qd, kd, vd, None, tau=tau, seed=seed)
  assert s.shape == (B, Hk, Skv) and s.dtype == torch.float32
  exp_rand = att.kf_noise(seed, B, H, Sq, Skv)
  ref = rm.attention_ref(q, k, v, exp_rand=exp_rand, tau=tau, want=("out", "kf"), head_chunk=2)
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(s.cpu(), ref["kf"], **STOL)
  torch.testing.assert_close(s.sum(-1).cpu(), torch.full((B, Hk), float(Sq)), rtol=1e-4, atol=1e-3)
  out_t, s_t = att.attn_kf_fwd(qd, kd, vd, exp_rand.to(cuda_device), tau=tau)       # the reference's signature
  assert torch.equal(out, out_t)
  torch.testing.assert_close(s, s_t, **STOL)
  out2, s2 = att.attn_kf_fwd(qd, kd, vd, None, tau=tau, seed=seed)
  assert torch.equal(s, s2) and torch.equal(out, out2)                              # same seed, same bits
  _, s3 = att.attn_kf_fwd(qd, kd, vd, None, tau=tau, seed=seed + 1)
  assert not torch.equal(s, s3)


def test_config4_every_unit_with_generated_noise(cuda_device):
  B, H, S, D = 2, 32, 2048, 128
  g = torch.Generator(device=cuda_device).manual_seed(41)
  q, k, v = (torch.randn(B, S, H, D, generator=g, device=cuda_device).to(torch.bfloat16) for _ in range(3))
  out, s = att.attn_kf_fwd(q, k, v, None, tau=1.0, seed=77)
  for b in range(B):
    exp_rand = att.kf_noise_fill(77, B, H, S, S, cuda_device)[b:b + 1]     # 0.5 GB per batch element
    ref = rm.attention_ref(q[b:b + 1], k[b:b + 1], v[b:b + 1], exp_rand=exp_rand, tau=1.0, want=("out", "kf"), head_chunk=4)
    torch.testing.assert_close(out[b:b + 1].float(), ref["out"], **TOL)
    torch.testing.assert_close(s[b:b + 1], ref["kf"], **STOL)
    del exp_rand, ref
