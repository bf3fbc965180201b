"""Parity of the bandwidth ops (called through the C ABI) with the CPU oracle on seeded inputs."""
import pytest
import torch

from deepgengraph_b200 import native_ops as ops
from oracle import reference_math as rm

pytestmark = pytest.mark.gpu

TOL = {torch.float32: dict(rtol=1e-5, atol=1e-5), torch.float16: dict(rtol=2e-3, atol=2e-3),
       torch.bfloat16: dict(rtol=2e-2, atol=2e-2)}
DTYPES = [torch.bfloat16, torch.float16, torch.float32]


def _gen(shape, dtype, seed, scale=1.0):
  g = torch.Generator().manual_seed(seed)
  return (torch.randn(shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,hidden", [(1, 128), (7, 3584), (33, 4096), (5, 8192), (3, 100), (2, 12288), (4, 1000)])
def test_rms_norm(cuda_device, dtype, tokens, hidden):
  x = _gen((tokens, hidden), dtype, 1)
  w = _gen((hidden,), dtype, 2) * 0.1 + 1
  w = w.to(dtype)
  ref = rm.rms_norm_ref(x, w, 1e-6)
  out = torch.full_like(x, float("nan"), device=cuda_device)
  ops.rms_norm(out, x.to(cuda_device), w.to(cuda_device), 1e-6)
  torch.testing.assert_close(out.float().cpu(), ref, **TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,hidden", [(9, 3584), (4, 4096), (3, 100)])
def test_fused_add_rms_norm_in_place(cuda_device, dtype, tokens, hidden):
  x, r = _gen((tokens, hidden), dtype, 3), _gen((tokens, hidden), dtype, 4)
  w = (_gen((hidden,), dtype, 5) * 0.1 + 1).to(dtype)
  ref_x, ref_r = rm.fused_add_rms_norm_ref(x, r, w, 1e-5)
  xd, rd = x.to(cuda_device), r.to(cuda_device)
  ops.fused_add_rms_norm(xd, rd, w.to(cuda_device), 1e-5)
  torch.testing.assert_close(rd.float().cpu(), ref_r, **TOL[dtype])
  torch.testing.assert_close(xd.float().cpu(), ref_x, **TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,d", [(1, 128), (13, 11008), (6, 14336), (5, 77)])
@pytest.mark.parametrize("op", ["silu_and_mul", "gelu_tanh_and_mul"])
def test_gated_activation(cuda_device, dtype, tokens, d, op):
  x = _gen((tokens, 2 * d), dtype, 6, scale=2.0)
  ref = getattr(rm, op + "_ref")(x)
  # poison the output AND a guard row behind it: the op must write exactly [tokens, d]
  out = torch.full((tokens + 1, d), 7.0, dtype=dtype, device=cuda_device)
  getattr(ops, op)(out[:tokens], x.to(cuda_device))
  torch.testing.assert_close(out[:tokens].float().cpu(), ref, **TOL[dtype])
  assert torch.all(out[tokens] == 7.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,heads,kv_heads,head_dim", [(17, 4, 4, 128), (9, 16, 8, 256), (5, 3, 1, 64)])
def test_rotary_embedding_online_in_place(cuda_device, dtype, tokens, heads, kv_heads, head_dim):
  q = _gen((tokens, heads * head_dim), dtype, 7)
  k = _gen((tokens, kv_heads * head_dim), dtype, 8)
  pos = torch.randint(0, 8192, (tokens,), generator=torch.Generator().manual_seed(9), dtype=torch.int32)
  pos[0] = 8191
  ref_q, ref_k = rm.rotary_online_ref(pos, q, k, head_dim, 10000.0)
  qd, kd = q.to(cuda_device), k.to(cuda_device)
  ops.rotary_embedding_online(pos.to(cuda_device), qd, kd, head_dim, 10000.0)
  # the result is the fp64-angle rotation rounded to T: angles and their range reduction are fp64 in the kernel,
  # so fp32 data at position 8191 (angles of thousands of radians) agree with the fp64 oracle to 2e-5
  tol = TOL[dtype] if dtype != torch.float32 else dict(rtol=1e-5, atol=2e-5)
  torch.testing.assert_close(qd.float().cpu(), ref_q, **tol)
  torch.testing.assert_close(kd.float().cpu(), ref_k, **tol)


def test_rotary_fp32_at_the_largest_positions_is_accurate(cuda_device):
  # every token sits at a position of thousands of radians for the lowest frequencies' neighbours; an fp32 angle
  # alone would be off by 5e-4 there (and the reference's fast-math build by ~1e-3)
  T, H, D = 64, 2, 256
  q = _gen((T, H * D), torch.float32, 21)
  k = _gen((T, H * D), torch.float32, 22)
  pos = torch.arange(8191 - T + 1, 8192, dtype=torch.int32)
  ref_q, ref_k = rm.rotary_online_ref(pos, q, k, D, 10000.0)
  qd, kd = q.to(cuda_device), k.to(cuda_device)
  ops.rotary_embedding_online(pos.to(cuda_device), qd, kd, D, 10000.0)
  torch.testing.assert_close(qd.cpu(), ref_q, rtol=0, atol=2e-5)
  torch.testing.assert_close(kd.cpu(), ref_k, rtol=0, atol=2e-5)


def test_rotary_on_strided_rows(cuda_device):
  # q and k as column slices of one fused qkv buffer, like the reference's caller (models/attn.py:36-41)
  tokens, H, Hk, D = 11, 4, 2, 128
  qkv = _gen((tokens, (H + 2 * Hk) * D), torch.bfloat16, 10)
  pos = torch.arange(tokens, dtype=torch.int32)
  ref_q, ref_k = rm.rotary_online_ref(pos, qkv[:, :H * D], qkv[:, H * D:(H + Hk) * D], D, 10000.0)
  d = qkv.to(cuda_device)
  ops.rotary_embedding_online(pos.to(cuda_device), d[:, :H * D], d[:, H * D:(H + Hk) * D], D, 10000.0)
  torch.testing.assert_close(d[:, :H * D].float().cpu(), ref_q, rtol=2e-2, atol=2e-2)
  torch.testing.assert_close(d[:, H * D:(H + Hk) * D].float().cpu(), ref_k, rtol=2e-2, atol=2e-2)
  assert torch.equal(d[:, (H + Hk) * D:].cpu(), qkv[:, (H + Hk) * D:])   # v untouched


def test_argument_validation_raises(cuda_device):
  x = torch.zeros(4, 128, dtype=torch.bfloat16, device=cuda_device)
  with pytest.raises(RuntimeError):
    ops.rms_norm(torch.empty_like(x), x.cpu(), torch.ones(128, dtype=torch.bfloat16), 1e-6)
  with pytest.raises(TypeError):
    ops.rms_norm(torch.empty_like(x), x, torch.ones(128, dtype=torch.float32, device=cuda_device), 1e-6)
  with pytest.raises(ValueError):
    ops.silu_and_mul(torch.empty(4, 63, dtype=torch.bfloat16, device=cuda_device), x)
  with pytest.raises(TypeError):
    ops.rotary_embedding_online(torch.zeros(4, dtype=torch.int64, device=cuda_device), x, x.clone(), 128, 1e4)
