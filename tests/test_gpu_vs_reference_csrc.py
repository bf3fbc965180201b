"""This package's bandwidth ops against the REFERENCE's own CUDA kernels (csrc/norm.cu, activation.cu,
pos_encoding.cu) built for sm_100a by oracle/build_ref.py into oracle/_ref/.  Skipped when that build is
absent (it needs the reference tree at build time; the built library is loaded from oracle/_ref/)."""
import importlib.util
import os

import pytest
import torch

from deepgengraph_b200 import native_ops as ops

pytestmark = pytest.mark.gpu
REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")
REF_SO = os.path.join(REF_DIR, "_csrc_ref.so")
REF_EXTRA_SO = os.path.join(REF_DIR, "_csrc_ref_extra.so")


@pytest.fixture(scope="module")
def ref():
  if not os.path.exists(REF_SO):
    pytest.skip("oracle/_ref/_csrc_ref.so not built")
  spec = importlib.util.spec_from_file_location("_csrc_ref", REF_SO)
  m = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(m)
  return m


@pytest.fixture(scope="module")
def ref_extra():
  """The reference's fused_add_rms_norm (csrc/norm.cu:59-83,100-113), which its own ffi.cpp does not register:
  built by oracle/build_ref.py from the reference's norm.cu and oracle/ref_extra_binding.cpp."""
  if not os.path.exists(REF_EXTRA_SO):
    pytest.skip("oracle/_ref/_csrc_ref_extra.so not built")
  spec = importlib.util.spec_from_file_location("_csrc_ref_extra", REF_EXTRA_SO)
  m = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(m)
  return m


def _randn(shape, dtype, seed, dev, scale=1.0):
  return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).to(dtype).to(dev)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("tokens,hidden", [(64, 4096), (33, 3584), (8, 1000)])
def test_rms_norm_equals_reference_kernel(cuda_device, ref, dtype, tokens, hidden):
  x = _randn((tokens, hidden), dtype, 1, cuda_device)
  w = (1 + 0.1 * _randn((hidden,), torch.float32, 2, cuda_device)).to(dtype)
  a, b = torch.empty_like(x), torch.empty_like(x)
  ref.rms_norm(a, x, w, 1e-6)
  ops.rms_norm(b, x, w, 1e-6)
  # same rounding points as the reference (normalise -> round -> multiply -> round); the only freedom is the
  # summation order of the fp32 variance, i.e. at most an occasional last-bit flip
  if dtype != torch.float32:   # in fp32 nothing is rounded away, so last-bit differences are the norm
    mism = (a != b).float().mean().item()
    assert mism < 2e-3, mism
  torch.testing.assert_close(b.float(), a.float(), rtol=1e-2 if dtype != torch.float32 else 1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("tokens,hidden", [(64, 4096), (33, 3584), (8, 1000)])
def test_fused_add_rms_norm_equals_reference_kernel(cuda_device, ref_extra, dtype, tokens, hidden):
  x = _randn((tokens, hidden), dtype, 6, cuda_device)
  r = _randn((tokens, hidden), dtype, 7, cuda_device)
  w = (1 + 0.1 * _randn((hidden,), torch.float32, 8, cuda_device)).to(dtype)
  xa, ra, xb, rb = x.clone(), r.clone(), x.clone(), r.clone()
  ref_extra.fused_add_rms_norm(xa, ra, w, 1e-6)
  ops.fused_add_rms_norm(xb, rb, w, 1e-6)
  # the updated residual is a single rounding of the fp32 sum on both sides: identical bits
  assert torch.equal(ra, rb)
  if dtype != torch.float32:
    mism = (xa != xb).float().mean().item()
    assert mism < 2e-3, mism
  torch.testing.assert_close(xb.float(), xa.float(), rtol=1e-2 if dtype != torch.float32 else 1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_silu_and_mul_equals_reference_kernel(cuda_device, ref, dtype):
  x = _randn((37, 2 * 11008), dtype, 3, cuda_device, 2.0)
  a = torch.empty(37, 11008, dtype=dtype, device=cuda_device)
  b = torch.empty_like(a)
  ref.silu_and_mul(a, x)
  ops.silu_and_mul(b, x)
  if dtype != torch.float32:
    mism = (a != b).float().mean().item()
    assert mism < 2e-3, mism
  torch.testing.assert_close(b.float(), a.float(), rtol=1e-2 if dtype != torch.float32 else 1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rotary_close_to_reference_kernel_at_small_positions(cuda_device, ref, dtype):
  # The reference evaluates angles with fast-math __powf/__sincosf in fp32; this package evaluates them in fp64 and
  # reduces the range before the fp32 sine/cosine.  At small positions both agree to rounding; at positions of
  # thousands of radians the reference itself is off by ~1e-3 (hence the wider bar below).
  T, H, Hk, D = 64, 8, 4, 128
  q, k = _randn((T, H * D), dtype, 4, cuda_device), _randn((T, Hk * D), dtype, 5, cuda_device)
  pos = torch.arange(T, dtype=torch.int32, device=cuda_device)
  qa, ka, qb, kb = q.clone(), k.clone(), q.clone(), k.clone()
  ref.rotary_embedding_online(pos, qa, ka, D, 10000.0)
  ops.rotary_embedding_online(pos, qb, kb, D, 10000.0)
  tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-3, atol=2e-3)
  torch.testing.assert_close(qb.float(), qa.float(), **tol)
  torch.testing.assert_close(kb.float(), ka.float(), **tol)
  pos = pos + 8000
  qa, qb, ka, kb = q.clone(), q.clone(), k.clone(), k.clone()
  ref.rotary_embedding_online(pos, qa, ka, D, 10000.0)
  ops.rotary_embedding_online(pos, qb, kb, D, 10000.0)
  torch.testing.assert_close(qb.float(), qa.float(), rtol=3e-2, atol=3e-2)
