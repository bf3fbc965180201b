"""Host logic of the batch x head sharding: partition arithmetic, piece slicing, and the score gather on
world_size-2 (and 3) gloo process groups on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepgengraph_b200 import sharding as sh


def test_unit_ranges_partition_exactly():
  for n in (1, 7, 8, 64, 128, 130):
    for world in (1, 2, 3, 4, 8):
      spans = [sh.unit_range(n, world, r) for r in range(world)]
      assert spans[0][0] == 0 and spans[-1][1] == n
      for (a, b), (c, d) in zip(spans, spans[1:]):
        assert b == c
      sizes = [b - a for a, b in spans]
      assert max(sizes) - min(sizes) <= 1
  with pytest.raises(ValueError):
    sh.unit_range(8, 2, 2)


def test_pieces_cover_every_unit_once():
  for batch, kvh, world in ((4, 32, 8), (2, 32, 3), (1, 8, 8), (2, 8, 5), (3, 5, 4)):
    seen = []
    for r in range(world):
      for p in sh.shard_pieces(batch, kvh, world, r):
        assert 0 <= p.hk_lo < p.hk_hi <= kvh
        seen += [p.b * kvh + h for h in range(p.hk_lo, p.hk_hi)]
    assert seen == list(range(batch * kvh))


def test_slice_piece_and_run_sharded_reassemble_the_full_problem():
  B, S, H, Hk, D = 2, 16, 6, 3, 8
  q = torch.arange(B * S * H * D, dtype=torch.float32).view(B, S, H, D)
  k = torch.arange(B * S * Hk * D, dtype=torch.float32).view(B, S, Hk, D) + 0.5
  v = -k
  extra = torch.arange(B * H * S * S, dtype=torch.float32).view(B, H, S, S)
  world = 4
  out = torch.full_like(q, float("nan"))
  ex = torch.full_like(extra, float("nan"))
  for r in range(world):
    for piece, (qs, ks, vs, es) in sh.run_sharded(lambda a, b, c, e: (a, b, c, e), q, k, v, world, r, extra=extra):
      g = H // Hk
      assert qs.is_contiguous() and ks.shape[2] * g == qs.shape[2]
      assert torch.equal(vs, -ks)
      out[piece.b, :, piece.hk_lo * g:piece.hk_hi * g] = qs[0]
      ex[piece.b, piece.hk_lo * g:piece.hk_hi * g] = es[0]
  assert torch.equal(out, q) and torch.equal(ex, extra)


def _free_port():
  s = socket.socket()
  s.bind(("127.0.0.1", 0))
  port = s.getsockname()[1]
  s.close()
  return port


def _gather_worker(rank, world, port, n_units, kv_len, fail_rank):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    lo, hi = sh.unit_range(n_units, world, rank)
    local = torch.stack([torch.full((kv_len,), float(u)) + torch.arange(kv_len) / 1000.0 for u in range(lo, hi)]) \
        if hi > lo else torch.empty(0, kv_len)
    full = sh.gather_scores(local, n_units, world, rank)
    expect = torch.stack([torch.full((kv_len,), float(u)) + torch.arange(kv_len) / 1000.0 for u in range(n_units)])
    assert torch.equal(full, expect), f"rank {rank}: gathered layout is wrong"
    if rank == fail_rank:
      # a rank that passes the wrong number of rows is caught on the host, before any collective
      try:
        sh.gather_scores(local[:-1], n_units, world, rank)
        raise AssertionError("row-count mismatch was not detected")
      except ValueError:
        pass
  finally:
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n_units", [(2, 64), (2, 7), (3, 8)])
def test_score_gather_on_gloo(world, n_units):
  mp.spawn(_gather_worker, args=(world, _free_port(), n_units, 33, 0), nprocs=world, join=True)


# ---- host-side failure detection: a rank that raises, or never arrives, is reported by its peers ----
def _failure_worker(rank, world, port, mode, result_dir):
  import pathlib
  import time
  store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
  B, S, H, D = 2, 16, 4, 8
  g = torch.Generator().manual_seed(0)
  q, k, v = (torch.randn(B, S, H, D, generator=g) for _ in range(3))

  def fn(qs, ks, vs):
    if mode == "raise" and rank == 1:
      raise ValueError("injected failure in the local step")
    return (qs + ks + vs,)

  outcome = "none"
  try:
    if mode == "absent" and rank == 1:
      time.sleep(3.0)          # never reports within the peers' time limit, then leaves
      outcome = "left"
    else:
      t0 = time.monotonic()
      res = sh.run_sharded_checked(fn, q, k, v, world, rank, store, step="s0", timeout_s=1.0)
      outcome = f"ok:{len(res)}"
  except sh.PeerFailure as e:
    outcome = f"peer_failure:failed={sorted(e.failed)}:missing={e.missing}:{time.monotonic() - t0:.1f}s"
  except ValueError as e:
    outcome = f"own_error:{e}"
  pathlib.Path(result_dir, f"rank{rank}.txt").write_text(outcome)
  if rank == 0:
    time.sleep(3.5 if mode == "absent" else 0.5)   # the store's host outlives its clients


@pytest.mark.parametrize("mode,world", [("ok", 2), ("raise", 3), ("absent", 2)])
def test_failed_or_absent_rank_is_reported_without_a_collective(tmp_path, mode, world):
  mp.spawn(_failure_worker, args=(world, _free_port(), mode, str(tmp_path)), nprocs=world, join=True)
  got = {r: (tmp_path / f"rank{r}.txt").read_text() for r in range(world)}
  if mode == "ok":
    assert all(v.startswith("ok:") for v in got.values()), got
  elif mode == "raise":
    assert got[1].startswith("own_error:injected failure"), got
    for r in (0, 2):
      assert got[r].startswith("peer_failure:failed=[1]:missing=[]"), got
  else:
    assert got[1] == "left" and got[0].startswith("peer_failure:failed=[]:missing=[1]"), got
    assert float(got[0].rsplit(":", 1)[1][:-1]) < 2.5, got   # reported at the time limit, not when the rank left


@pytest.mark.parametrize("args", [(8192, 8192, 4, True, 4096), (8192, 8192, 2, True, 0), (1000, 1500, 3, True, 0),
                                  (300, 300, 8, True, 0), (4096, 4096, 4, False, 0), (128, 128, 4, True, 0),
                                  (4096, 4096, 3, True, 700)])
def test_row_ranges_cover_the_rows_on_tile_boundaries_with_balanced_work(args):
  q_len, kv_len, parts, causal, window = args
  ranges = sh.row_ranges(q_len, kv_len, parts, causal, window)
  assert ranges[0][0] == 0 and ranges[-1][1] == q_len and len(ranges) <= parts
  for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
    assert a1 == b0
  assert all(r0 % 128 == 0 and r1 > r0 for r0, r1 in ranges)
  delta = kv_len - q_len

  def visible(i):
    hi = min(i + delta, kv_len - 1) if causal else kv_len - 1
    lo = max(0, i + delta - window + 1) if (causal and window > 0) else 0
    return hi - lo + 1
  work = [sum(visible(i) for i in range(r0, r1)) for r0, r1 in ranges]
  if len(ranges) == parts and q_len >= 16 * 128 * parts:   # enough tiles per part for the greedy cut to balance
    assert max(work) <= 1.15 * sum(work) / parts


def test_row_shard_pieces_partition_the_problem():
  batch, kv_heads, q_len, kv_len = 1, 8, 8192, 8192      # config 5: eight units
  for world in (1, 2, 8, 16, 24, 32):
    seen = []
    for rank in range(world):
      seen += sh.row_shard_pieces(batch, kv_heads, q_len, kv_len, world, rank, True, 4096)
    rows = {}
    for pc in seen:
      rows.setdefault((pc.b, pc.hk), []).append((pc.r0, pc.r1))
    assert len(rows) == batch * kv_heads
    for spans in rows.values():
      spans.sort()
      assert spans[0][0] == 0 and spans[-1][1] == q_len
      assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    if world >= 16:
      assert all(len(sh.row_shard_pieces(batch, kv_heads, q_len, kv_len, world, r, True, 4096)) >= 1 for r in range(world - world % 8))


def test_slice_rows_keeps_the_mask_alignment():
  import torch
  from oracle import reference_math as rm
  g = torch.Generator().manual_seed(5)
  q = torch.randn(1, 384, 2, 16, generator=g)
  k = torch.randn(1, 512, 1, 16, generator=g)
  v = torch.randn(1, 512, 1, 16, generator=g)
  for window in (0, 100):
    full = rm.attention_ref(q, k, v, causal=True, window=window)["out"]
    for r0, r1 in ((0, 128), (128, 384), (256, 384)):
      qs, ks, vs = sh.slice_rows(q, k, v, r0, r1, causal=True)
      part = rm.attention_ref(qs, ks, vs, causal=True, window=window)["out"]
      torch.testing.assert_close(part, full[:, r0:r1], rtol=1e-6, atol=1e-6)
