"""Parity of the fused attention forward (through the C ABI) with the CPU oracle and with the golden
outputs of the reference's own modules.  Tolerances: rtol = atol = 2e-2 on 16-bit outputs against the
fp32 reference (the bar stated for this path), 1e-3 relative on the fp32 log-sum-exp."""
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


def _randn(shape, dtype, seed, scale=1.0):
  g = torch.Generator().manual_seed(seed)
  return (torch.randn(shape, generator=g) * scale).to(dtype)


def _qkv(B, Sq, Skv, H, Hk, D, dtype, seed=0, q_scale=1.0):
  return (_randn((B, Sq, H, D), dtype, seed + 1, q_scale), _randn((B, Skv, Hk, D), dtype, seed + 2),
          _randn((B, Skv, Hk, D), dtype, seed + 3))


@pytest.mark.parametrize("name", [n for n, c in cases.CASES.items() if c["model"] in ("attn", "gemma2")])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_golden_cases_of_the_reference_modules(cuda_device, name, dtype):
  c = cases.CASES[name]
  inp = cases.make_inputs(name, dtype)   # exactly representable: the kernel sees the golden run's values
  g = np.load(os.path.join(HERE, "golden", name + ".npz"))
  out = att.attn_fwd(inp["q"].to(cuda_device), inp["k"].to(cuda_device), inp["v"].to(cuda_device), causal=True,
                     softcap=50.0 if c["model"] == "gemma2" else 0.0)
  assert out.shape == inp["q"].shape and out.dtype == dtype
  got = out.float().cpu()
  torch.testing.assert_close(got[:, ::cases.ROW_STRIDE], torch.from_numpy(g["out_rows"]), **TOL)
  assert abs(got.double().sum().item() - float(g["out_sum"])) <= 5e-3 * float(g["out_abssum"])


SHAPES = [
    # B, Sq, Skv, H, Hk, D
    (1, 128, 128, 1, 1, 128),
    (1, 256, 256, 2, 2, 128),
    (2, 384, 384, 3, 3, 128),
    (1, 1024, 1024, 2, 2, 128),
    (1, 100, 100, 2, 2, 128),       # ragged: one partial tile
    (1, 300, 333, 2, 2, 128),       # ragged, kv longer than q
    (1, 128, 640, 2, 2, 128),       # decode-like suffix: delta = 512
    (1, 1, 257, 2, 2, 128),         # single query
    (1, 512, 512, 4, 2, 128),       # grouped-query attention
    (1, 256, 256, 2, 2, 256),
    (1, 200, 456, 4, 2, 256),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_causal_attention_matches_oracle(cuda_device, shape, dtype):
  B, Sq, Skv, H, Hk, D = shape
  q, k, v = _qkv(B, Sq, Skv, H, Hk, D, dtype, seed=sum(shape))
  ref = rm.attention_ref(q, k, v, causal=True, want=("out", "lse2"))
  out, lse = att.attn_fwd_with_lse(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=True)
  torch.testing.assert_close(out.float().cpu(), ref["out"], **TOL)
  torch.testing.assert_close(lse.cpu(), ref["lse2"], rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("D", [128, 256])
@pytest.mark.parametrize("window", [1, 64, 128, 200, 4096])
def test_sliding_window(cuda_device, D, window):
  q, k, v = _qkv(1, 640, 640, 2, 1, D, torch.bfloat16, seed=window)
  ref = rm.attention_ref(q, k, v, causal=True, window=window)["out"]
  out = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=True, window=window)
  torch.testing.assert_close(out.float().cpu(), ref, **TOL)


@pytest.mark.parametrize("D", [128, 256])
def test_softcap_with_large_logits(cuda_device, D):
  q, k, v = _qkv(1, 384, 384, 2, 2, D, torch.bfloat16, seed=5, q_scale=30.0)   # logits ~ N(0, 30^2): the cap bites
  ref = rm.attention_ref(q, k, v, causal=True, softcap=50.0)["out"]
  out = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=True, softcap=50.0)
  torch.testing.assert_close(out.float().cpu(), ref, **TOL)


def test_non_causal_and_custom_scale(cuda_device):
  q, k, v = _qkv(1, 256, 320, 2, 2, 128, torch.bfloat16, seed=6)
  ref = rm.attention_ref(q, k, v, causal=False, scale=0.05)["out"]
  out = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=False, scale=0.05)
  torch.testing.assert_close(out.float().cpu(), ref, **TOL)


def test_large_maximum_drift_exercises_the_rescale_path(cuda_device):
  # keys ordered so that the row maximum keeps growing along the sequence: O must be rescaled repeatedly
  B, S, H, D = 1, 1024, 1, 128
  q, k, v = _qkv(B, S, S, H, H, D, torch.bfloat16, seed=7)
  k = (k.float() * torch.linspace(0.2, 6.0, S)[None, :, None, None]).to(torch.bfloat16)
  ref = rm.attention_ref(q, k, v, causal=True)["out"]
  out = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=True)
  torch.testing.assert_close(out.float().cpu(), ref, **TOL)


def test_reruns_are_bitwise_identical_and_cover_every_element(cuda_device):
  q, k, v = (t.to(cuda_device) for t in _qkv(2, 512, 512, 4, 4, 128, torch.bfloat16, seed=8))
  a = att.attn_fwd(q, k, v)
  b = att.attn_fwd(q, k, v)
  assert torch.equal(a, b)
  assert torch.isfinite(a.float()).all()


def test_config2_slice_full_length(cuda_device):
  # seq 4096, head_dim 128 (the benchmark's shape) on a few heads; oracle evaluated per head chunk
  q, k, v = _qkv(1, 4096, 4096, 4, 4, 128, torch.bfloat16, seed=9)
  ref = rm.attention_ref(q, k, v, causal=True, head_chunk=2)["out"]
  out = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
  torch.testing.assert_close(out.float().cpu(), ref, **TOL)


def test_full_size_config2_properties(cuda_device):
  # B4 H32 S4096 D128: too large for the CPU oracle in a test; check size-independent properties instead.
  # With v = ones every output element is exactly 1; with v[b, j, h, :] = j/S the output of row i is the
  # probability-weighted mean key position, which must lie in [0, i/S] and be non-decreasing in expectation.
  B, S, H, D = 4, 4096, 32, 128
  g = torch.Generator(device=cuda_device).manual_seed(0)
  q = torch.randn(B, S, H, D, generator=g, device=cuda_device, dtype=torch.bfloat16)
  k = torch.randn(B, S, H, D, generator=g, device=cuda_device, dtype=torch.bfloat16)
  ones = torch.ones(B, S, H, D, device=cuda_device, dtype=torch.bfloat16)
  out = att.attn_fwd(q, k, ones)
  torch.testing.assert_close(out.float(), torch.ones_like(out, dtype=torch.float32), rtol=1e-2, atol=1e-2)
  ramp = (torch.arange(S, device=cuda_device, dtype=torch.float32) / S)[None, :, None, None].expand(B, S, H, D)
  out = att.attn_fwd(q, k, ramp.to(torch.bfloat16).contiguous()).float()
  bound = (torch.arange(S, device=cuda_device, dtype=torch.float32) / S)[None, :, None, None] + 1e-2
  assert (out >= -1e-2).all() and (out <= bound).all()
  # linearity in v: attn(q, k, a + b) = attn(q, k, a) + attn(q, k, b)
  v1 = torch.randn(B, S, H, D, generator=g, device=cuda_device, dtype=torch.bfloat16)
  o1 = att.attn_fwd(q, k, v1).float()
  o2 = att.attn_fwd(q, k, (v1.float() * 2).to(torch.bfloat16)).float()
  torch.testing.assert_close(o2, 2 * o1, rtol=2e-2, atol=2e-2)


def test_more_tiles_than_resident_ctas(cuda_device):
  # head_dim 128 runs a persistent grid (2 CTAs per SM) whose CTAs walk several query tiles each: 2 x 10 x 20 = 400
  # tiles is more than any B200 holds at once, so barrier phases, the K/V ring and the TMEM buffers carry over
  # from tile to tile inside a CTA.
  q, k, v = _qkv(2, 2560, 2560, 10, 10, 128, torch.bfloat16, seed=21)
  ref = rm.attention_ref(q, k, v, causal=True, head_chunk=5)["out"]
  out = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
  torch.testing.assert_close(out.float().cpu(), ref, **TOL)


def test_many_ragged_tiles_gqa_window_softcap(cuda_device):
  # 24 heads x 16 ragged query tiles (q_len not a multiple of 128, kv_len > q_len), grouped K/V heads, sliding
  # window and soft-cap together, again more tiles than resident CTAs
  q, k, v = _qkv(1, 2000, 2304, 24, 8, 128, torch.float16, seed=22, q_scale=2.0)
  ref = rm.attention_ref(q, k, v, causal=True, window=700, softcap=30.0, head_chunk=6)["out"]
  out = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=True, window=700, softcap=30.0)
  torch.testing.assert_close(out.float().cpu(), ref, **TOL)


def test_launches_on_two_streams_interleave(cuda_device):
  # every launch takes its own tile counter; launches in flight on different streams must not share one
  q, k, v = (t.to(cuda_device) for t in _qkv(2, 1536, 1536, 16, 16, 128, torch.bfloat16, seed=23))
  want = att.attn_fwd(q, k, v)
  torch.cuda.synchronize()
  streams = [torch.cuda.Stream(device=cuda_device) for _ in range(2)]
  outs = []
  for rep in range(4):
    for st in streams:
      with torch.cuda.stream(st):
        outs.append(att.attn_fwd(q, k, v))
  torch.cuda.synchronize()
  for o in outs:
    assert torch.equal(o, want)


@pytest.mark.parametrize("D,H,Hk", [(128, 6, 2), (256, 2, 1)])
def test_views_of_a_fused_qkv_projection_need_no_copy(cuda_device, D, H, Hk):
  # q, k, v as slices of one [B, S, (H + 2 Hk) D] buffer (what the model glue gets from its QKV GEMM,
  # models/attn.py:35-36): the strided entry point must give the bits of the contiguous one
  B, S = 2, 640
  g = torch.Generator().manual_seed(31)
  qkv = torch.randn(B, S, (H + 2 * Hk) * D, generator=g).to(torch.bfloat16).to(cuda_device)
  q = qkv[:, :, :H * D].unflatten(-1, (H, D))
  k = qkv[:, :, H * D:(H + Hk) * D].unflatten(-1, (Hk, D))
  v = qkv[:, :, (H + Hk) * D:].unflatten(-1, (Hk, D))
  assert not q.is_contiguous() and q.data_ptr() == qkv.data_ptr()
  got, lse = att.attn_fwd_with_lse(q, k, v, causal=True, window=300)
  want, lse_want = att.attn_fwd_with_lse(q.contiguous(), k.contiguous(), v.contiguous(), causal=True, window=300)
  assert got.is_contiguous() and torch.equal(got, want) and torch.equal(lse, lse_want)
  ref = rm.attention_ref(q.cpu(), k.cpu(), v.cpu(), causal=True, window=300)["out"]
  torch.testing.assert_close(got.float().cpu(), ref, **TOL)


def test_views_with_unaligned_strides_are_rejected(cuda_device):
  qkv = torch.zeros(1, 256, 3 * 128 + 4, dtype=torch.bfloat16, device=cuda_device)   # row stride not 16-byte aligned
  q, k, v = (qkv[:, :, i * 128:(i + 1) * 128].unflatten(-1, (1, 128)) for i in range(3))
  with pytest.raises(ValueError):
    att.attn_fwd(q, k, v)


@pytest.mark.parametrize("case", ["short_sequences", "narrow_window", "head_dim_256"])
def test_many_tiny_tiles_per_cta(cuda_device, case):
  # tiles of one or two key blocks, several per persistent CTA: the MMA issuer and the loader can run a whole
  # tile ahead of the softmax warpgroup, so the tile hand-over itself is what is exercised here
  if case == "short_sequences":
    B, S, H, D, window = 8, 128, 64, 128, 0            # 512 tiles of 2 key blocks
  elif case == "narrow_window":
    B, S, H, D, window = 2, 2048, 16, 128, 32          # 512 tiles of <= 2 key blocks
  else:
    B, S, H, D, window = 4, 256, 48, 256, 0            # 384 tiles on a one-CTA-per-SM grid
  q, k, v = _qkv(B, S, S, H, H, D, torch.bfloat16, seed=51)
  ref = rm.attention_ref(q, k, v, causal=True, window=window, head_chunk=16)["out"]
  qd, kd, vd = q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)
  out = att.attn_fwd(qd, kd, vd, causal=True, window=window)
  torch.testing.assert_close(out.float().cpu(), ref, **TOL)
  for _ in range(3):
    assert torch.equal(att.attn_fwd(qd, kd, vd, causal=True, window=window), out)


def test_empty_batch_returns_empty_tensors(cuda_device):
  # the reference's torch modules return empty tensors for an empty batch; nothing is launched here
  q = torch.empty(0, 256, 4, 128, dtype=torch.bfloat16, device=cuda_device)
  out, lse = att.attn_fwd_with_lse(q, q, q)
  assert out.shape == (0, 256, 4, 128) and lse.shape == (0, 4, 256)
  out, score, score_sq = att.attn_score_fwd(q, q, q, want_sq=True)
  assert out.shape == q.shape and score.shape == (0, 4, 256) and score_sq.shape == (0, 4, 256)


def test_long_sequence_32k(cuda_device):
  # 256 query tiles of up to 512 key blocks per head: long barrier-phase and ring-counter runs inside one CTA.
  # The oracle is evaluated for a few query rows only (each row is independent of the others).
  B, S, H, D = 1, 32768, 2, 128
  q, k, v = _qkv(B, S, S, H, H, D, torch.bfloat16, seed=61)
  out = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)).float().cpu()
  assert torch.isfinite(out).all()
  rows = torch.tensor([0, 1, 127, 128, 4095, 20000, 32767 - 128, 32767])
  scale = D ** -0.5
  for h in range(H):
    logits = (q[0, rows, h].float() @ k[0, :, h].float().T) * scale                  # [rows, S]
    logits = logits.masked_fill(torch.arange(S)[None, :] > rows[:, None], float("-inf"))
    p = torch.softmax(logits, dim=-1).to(torch.bfloat16).float()
    ref = p @ v[0, :, h].float()
    torch.testing.assert_close(out[0, rows, h], ref, **TOL)
  ones = torch.ones(B, S, H, D, dtype=torch.bfloat16, device=cuda_device)
  o1 = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), ones).float()
  torch.testing.assert_close(o1, torch.ones_like(o1), rtol=1e-2, atol=1e-2)


def test_rescale_path_in_ctas_that_walk_several_tiles(cuda_device):
  # growing key norms force repeated rescales of the O accumulator; with 400 tiles every persistent CTA meets them
  # in its second tile too, where the O barriers are addressed by the CTA-wide block counter
  B, S, H, D = 2, 2560, 10, 128
  q, k, v = _qkv(B, S, S, H, H, D, torch.bfloat16, seed=71)
  k = (k.float() * torch.linspace(0.2, 5.0, S)[None, :, None, None]).to(torch.bfloat16)
  ref = rm.attention_ref(q, k, v, causal=True, head_chunk=5)["out"]
  out = att.attn_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=True)
  torch.testing.assert_close(out.float().cpu(), ref, **TOL)


def test_cuda_graph_replay_of_the_persistent_kernel(cuda_device):
  # a captured launch keeps the tile-counter pair it drew at capture time; the last CTA of every replay must
  # return it to zero for the next replay
  q, k, v = (t.to(cuda_device) for t in _qkv(2, 1536, 1536, 12, 4, 128, torch.bfloat16, seed=81))
  want = att.attn_fwd(q, k, v, window=700)
  torch.cuda.synchronize()
  stream = torch.cuda.Stream(device=cuda_device)
  stream.wait_stream(torch.cuda.current_stream(cuda_device))
  with torch.cuda.stream(stream):
    att.attn_fwd(q, k, v, window=700)          # warm-up on the capture stream
  torch.cuda.current_stream(cuda_device).wait_stream(stream)
  graph = torch.cuda.CUDAGraph()
  with torch.cuda.graph(graph):
    outs = [att.attn_fwd(q, k, v, window=700) for _ in range(3)]
  for _ in range(4):
    for o in outs:
      o.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    for o in outs:
      assert torch.equal(o, want)
  assert torch.equal(att.attn_fwd(q, k, v, window=700), want)     # eager launches still fine afterwards


def test_host_validation(cuda_device):
  q, k, v = (t.to(cuda_device) for t in _qkv(1, 128, 128, 2, 2, 128, torch.bfloat16))
  with pytest.raises(TypeError):
    att.attn_fwd(q.float(), k.float(), v.float())
  with pytest.raises(ValueError):
    att.attn_fwd(q.transpose(1, 2), k, v)
  with pytest.raises(RuntimeError):
    att.attn_fwd(q.cpu(), k.cpu(), v.cpu())
  with pytest.raises(RuntimeError):   # unsupported head_dim comes back as a status code from the C ABI
    att.attn_fwd(q[..., :64].contiguous(), k[..., :64].contiguous(), v[..., :64].contiguous())


def test_head_sliced_views_give_the_bits_of_the_full_problem(cuda_device):
  # a rank's shard of the plain attention is a head range of the full tensors: attn_fwd reads it as a view (no copy)
  # and, a unit's result not depending on its neighbours, returns the bits of the one-GPU run
  from deepgengraph_b200 import sharding as sh
  q, k, v = (t.to(cuda_device) for t in _qkv(2, 640, 640, 12, 4, 128, torch.bfloat16, seed=91))
  full = att.attn_fwd(q, k, v)
  world = 3
  for rank in range(world):
    for piece, out in sh.run_sharded(lambda a, b, c: att.attn_fwd(a, b, c), q, k, v, world, rank, dense=False):
      assert torch.equal(out[0], full[piece.b, :, piece.hk_lo * 3:piece.hk_hi * 3])


@pytest.mark.parametrize("shape,opt", [((1, 2048, 2048, 4, 2, 256), {"window": 1024, "softcap": 50.0}),
                                       ((2, 1024, 1536, 6, 3, 128), {}),
                                       ((1, 1152, 1152, 2, 2, 128), {"window": 300})])
def test_query_row_shards_give_the_bits_of_the_full_problem(cuda_device, shape, opt):
  # problems with fewer (batch, kv-head) units than GPUs are also cut along their query rows, on tile boundaries,
  # every piece a view of the full tensors with the keys its rows can see: same tiles, same key blocks, same bits
  from deepgengraph_b200 import sharding as sh
  B, Sq, Skv, H, Hk, D = shape
  q, k, v = (t.to(cuda_device) for t in _qkv(B, Sq, Skv, H, Hk, D, torch.bfloat16, seed=131))
  window = opt.get("window", 0)
  full = att.attn_fwd(q, k, v, **opt)
  world = 4 * B * Hk
  got = torch.full_like(full, float("nan"))
  g = H // Hk
  n_pieces = 0
  for rank in range(world):
    for pc, out in sh.run_row_sharded(lambda a, b, c: att.attn_fwd(a, b, c, **opt), q, k, v, world, rank, True, window):
      got[pc.b, pc.r0:pc.r1, pc.hk * g:(pc.hk + 1) * g] = out[0]
      n_pieces += 1
  assert n_pieces > B * Hk
  assert torch.equal(got, full)
