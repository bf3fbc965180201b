"""Batch x head sharding of the core modules over the GPUs of one node (one process per GPU).

Every (batch, kv-head) pair -- with the `group` query heads that share it -- is an independent unit of
work: attention rows never mix heads, and the per-key score vectors of a head only sum over that head's
own queries.  So the path shards with NO data-path collective: rank r owns the contiguous unit range
[r*U/N, (r+1)*U/N) of the flattened (batch, kv_head) index space and runs the single-GPU kernels on it.
The only communication is optional and off the critical path: gathering the small fp32 score vectors
([units, kv_len], ~1 MiB in total) so that every rank sees the scores of all heads (a KV-eviction policy
needs them where the layer's cache lives).  That gather is one NCCL all-gather over NVLink/NVSwitch;
attention outputs stay sharded.

The plain attention can also be cut along its query rows (row_ranges / run_row_sharded below) when a problem has
fewer units than GPUs.

The reference is single-GPU (our_env.sh:35,52); this module has no counterpart there.
"""
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def unit_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
  """Contiguous, balanced split: the first (n_units % world) ranks own one extra unit."""
  if world <= 0 or not (0 <= rank < world):
    raise ValueError(f"bad rank/world {rank}/{world}")
  base, extra = divmod(n_units, world)
  lo = rank * base + min(rank, extra)
  return lo, lo + base + (1 if rank < extra else 0)


@dataclass(frozen=True)
class Piece:
  """A rectangular piece of a rank's shard: kv heads [hk_lo, hk_hi) of batch element b."""
  b: int
  hk_lo: int
  hk_hi: int

  @property
  def n_units(self):
    return self.hk_hi - self.hk_lo


def shard_pieces(batch: int, kv_heads: int, world: int, rank: int) -> List[Piece]:
  """The rank's unit range cut at batch boundaries (units are numbered b * kv_heads + hk)."""
  lo, hi = unit_range(batch * kv_heads, world, rank)
  pieces = []
  u = lo
  while u < hi:
    b, hk = divmod(u, kv_heads)
    end = min(hi, (b + 1) * kv_heads)
    pieces.append(Piece(b, hk, hk + (end - u)))
    u = end
  return pieces


def slice_piece(q, k, v, piece: Piece, group: int, extra=None, dense: bool = True):
  """One piece of the problem: q heads [hk_lo*group, hk_hi*group), kv heads [hk_lo, hk_hi) of batch element b, BSHD.
  dense=True copies the slices into contiguous tensors (what the score variants take); dense=False returns the head
  slices as VIEWS -- attention.attn_fwd reads such row-strided views through its TMA descriptors, so a shard of the
  plain attention costs no copy.  `extra` (optional) is a [B, H, Sq, Skv] tensor sliced the same way (KeyFormer's
  exp_rand; always contiguous, a head range of it already is)."""
  b, lo, hi = piece.b, piece.hk_lo, piece.hk_hi
  qs, ks, vs = q[b:b + 1, :, lo * group:hi * group], k[b:b + 1, :, lo:hi], v[b:b + 1, :, lo:hi]
  if dense:
    qs, ks, vs = qs.contiguous(), ks.contiguous(), vs.contiguous()
  if extra is None:
    return qs, ks, vs
  return qs, ks, vs, extra[b:b + 1, lo * group:hi * group].contiguous()


def run_sharded(fn, q, k, v, world: int, rank: int, extra=None, dense: bool = True):
  """Runs `fn(q_piece, k_piece, v_piece[, extra_piece])` on this rank's pieces of the full problem.
  Returns a list of (piece, result) -- results stay on the device, sharded.  dense=False hands `fn` views
  (for attention.attn_fwd, which needs no copy)."""
  group = q.size(2) // k.size(2)
  out = []
  for piece in shard_pieces(q.size(0), k.size(2), world, rank):
    args = slice_piece(q, k, v, piece, group, extra, dense)
    out.append((piece, fn(*args)))
  return out


# --------------------------------------------------------------------------------------------
# Query-row sharding of the PLAIN attention, for problems with fewer (batch, kv-head) units than GPUs (config 5 has
# eight).  Attention rows are independent, so a rank may also own a range of query rows of a unit: it needs the keys
# up to its last row only, and no reduction follows.  (The score variants sum over queries; cutting their rows would
# need one -- they shard by units only.)
# --------------------------------------------------------------------------------------------
def row_ranges(q_len: int, kv_len: int, parts: int, causal: bool = True, window: int = 0,
               align: int = 128) -> List[Tuple[int, int]]:
  """Cuts the query rows [0, q_len) into `parts` contiguous ranges of about equal WORK -- visible (query, key) pairs
  under the causal / sliding-window mask -- with boundaries on multiples of `align` rows: query tiles stay whole, so
  a range computes exactly what the full problem computes for those rows.  Fewer than `parts` ranges come back when
  there are fewer tiles; no range is empty."""
  if parts <= 0 or q_len <= 0 or kv_len < q_len:
    raise ValueError(f"bad row split: q_len {q_len}, kv_len {kv_len}, parts {parts}")
  delta = kv_len - q_len
  n_tiles = -(-q_len // align)

  def visible(i):
    hi = min(i + delta, kv_len - 1) if causal else kv_len - 1
    lo = max(0, i + delta - window + 1) if (causal and window > 0) else 0
    return hi - lo + 1
  tile_work = [sum(visible(i) for i in (t * align, min(q_len, (t + 1) * align) - 1)) * 0.5 *
               (min(q_len, (t + 1) * align) - t * align) for t in range(n_tiles)]   # trapezoid: work is linear per tile
  total = sum(tile_work)
  parts = min(parts, n_tiles)
  cuts, acc, nxt = [0], 0.0, 1
  for t in range(n_tiles):
    acc += tile_work[t]
    tiles_left, parts_left = n_tiles - (t + 1), parts - nxt
    if nxt < parts and (acc >= total * nxt / parts or tiles_left == parts_left):
      cuts.append(t + 1)
      nxt += 1
  cuts.append(n_tiles)
  return [(cuts[i] * align, min(q_len, cuts[i + 1] * align)) for i in range(len(cuts) - 1) if cuts[i + 1] > cuts[i]]


def slice_rows(q, k, v, r0: int, r1: int, causal: bool = True):
  """Views of the inputs that make attention of query rows [r0, r1) a problem of its own: the rows of q, and the keys
  the last of them can see.  With the mask aligned bottom-right (key j visible to row i iff j <= i + kv_len - q_len,
  kernels/attn.py:22-23) the slice's offset r1 + (kv_len - q_len) - (r1 - r0) equals the full problem's for the same
  rows; a sliding window is relative to the row and carries over unchanged."""
  kv_hi = k.size(1) if not causal else r1 + (k.size(1) - q.size(1))
  return q[:, r0:r1], k[:, :kv_hi], v[:, :kv_hi]


@dataclass(frozen=True)
class RowPiece:
  """Query rows [r0, r1) of kv head hk (with its query heads) of batch element b."""
  b: int
  hk: int
  r0: int
  r1: int


def row_shard_pieces(batch: int, kv_heads: int, q_len: int, kv_len: int, world: int, rank: int, causal: bool = True,
                     window: int = 0) -> List[RowPiece]:
  """This rank's pieces when every unit is cut into world // units row ranges (at least one): the (unit, range) pairs
  are numbered unit-major and dealt out in contiguous, balanced runs like the units themselves."""
  units = batch * kv_heads
  ranges = row_ranges(q_len, kv_len, max(1, world // units), causal, window)
  lo, hi = unit_range(units * len(ranges), world, rank)
  pieces = []
  for idx in range(lo, hi):
    u, part = divmod(idx, len(ranges))
    b, hk = divmod(u, kv_heads)
    pieces.append(RowPiece(b, hk, ranges[part][0], ranges[part][1]))
  return pieces


def run_row_sharded(fn, q, k, v, world: int, rank: int, causal: bool = True, window: int = 0):
  """Runs `fn(q_piece, k_piece, v_piece)` -- the plain attention with the same causal / window arguments -- on this
  rank's (unit, row range) pieces; every piece is a view (no copy).  Returns a list of (piece, result); result rows
  are the piece's query rows, heads its unit's query heads."""
  group = q.size(2) // k.size(2)
  out = []
  for pc in row_shard_pieces(q.size(0), k.size(2), q.size(1), k.size(1), world, rank, causal, window):
    qs, ks, vs = slice_rows(q[pc.b:pc.b + 1, :, pc.hk * group:(pc.hk + 1) * group], k[pc.b:pc.b + 1, :, pc.hk:pc.hk + 1],
                            v[pc.b:pc.b + 1, :, pc.hk:pc.hk + 1], pc.r0, pc.r1, causal)
    out.append((pc, fn(qs, ks, vs)))
  return out


def gather_scores(local_scores: torch.Tensor, n_units_total: int, world: int, rank: int,
                  group: Optional["dist.ProcessGroup"] = None) -> torch.Tensor:
  """All-gathers per-unit score vectors.  local_scores: [units_local, kv_len] float32, rows in unit order.
  Returns [n_units_total, kv_len] on every rank (unit u = b * heads + h).  Uneven splits are padded to the
  largest shard for the collective and trimmed afterwards."""
  lo, hi = unit_range(n_units_total, world, rank)
  if local_scores.size(0) != hi - lo:
    raise ValueError(f"rank {rank} owns {hi - lo} units but passed {local_scores.size(0)} score rows")
  if world == 1:
    return local_scores
  kv_len = local_scores.size(1)
  max_units = -(-n_units_total // world)
  send = local_scores
  if send.size(0) < max_units:
    send = torch.cat([send, send.new_zeros(max_units - send.size(0), kv_len)], dim=0)
  recv = send.new_empty(world * max_units, kv_len)
  dist.all_gather_into_tensor(recv, send.contiguous(), group=group)
  rows = []
  for r in range(world):
    rlo, rhi = unit_range(n_units_total, world, r)
    rows.append(recv[r * max_units:r * max_units + (rhi - rlo)])
  return torch.cat(rows, dim=0)


def scores_from_pieces(results, index: int = 1) -> torch.Tensor:
  """Stacks the score output `index` of run_sharded results into [units_local, kv_len] in unit order."""
  rows = [res[index].reshape(-1, res[index].size(-1)) for _, res in results]
  return torch.cat(rows, dim=0) if rows else torch.empty(0)


# --------------------------------------------------------------------------------------------
# Host-side failure detection.  The data path has no collective, so a failed rank can only hang
# its peers at the optional score gather (or at a barrier of the caller).  Every rank therefore
# reports the outcome of its local step to a key-value store (a torch.distributed Store, e.g. the
# TCPStore of the process group) BEFORE entering the collective, and checks that all peers did:
# a rank that raised, exited or never arrived is named in a PeerFailure raised on every surviving
# rank within `timeout_s`, and no collective is launched.  Nothing here touches a GPU.
# --------------------------------------------------------------------------------------------
class PeerFailure(RuntimeError):
  """Raised on a surviving rank: `failed` ranks reported an error, `missing` ranks never reported."""

  def __init__(self, step, failed, missing):
    self.step, self.failed, self.missing = step, dict(failed), list(missing)
    parts = [f"rank {r} failed: {msg}" for r, msg in sorted(self.failed.items())]
    parts += [f"rank {r} did not report within the time limit" for r in self.missing]
    super().__init__(f"step {step}: " + "; ".join(parts))


def report_step(store, rank: int, step, ok: bool = True, message: str = "") -> None:
  """Publishes this rank's outcome of `step` (any hashable label) to the store."""
  store.set(f"b200/step/{step}/rank/{rank}", "ok" if ok else "failed:" + message[:200])


def check_peers(store, world: int, step, timeout_s: float = 30.0, poll_s: float = 0.02) -> None:
  """Returns once every rank has reported `step` as ok; raises PeerFailure otherwise (after at most
  `timeout_s` for ranks that never report)."""
  import time
  deadline = time.monotonic() + timeout_s
  pending = set(range(world))
  failed = {}
  while pending:
    for r in sorted(pending):
      key = f"b200/step/{step}/rank/{r}"
      if store.check([key]):
        val = store.get(key).decode()
        pending.discard(r)
        if val != "ok":
          failed[r] = val[len("failed:"):]
    if failed:   # no point in waiting for the others: the step is lost
      raise PeerFailure(step, failed, [])
    if pending:
      if time.monotonic() > deadline:
        raise PeerFailure(step, failed, sorted(pending))
      time.sleep(poll_s)


def run_sharded_checked(fn, q, k, v, world: int, rank: int, store, step, extra=None, timeout_s: float = 30.0):
  """run_sharded with failure detection: an exception in this rank's pieces is reported to the peers and
  re-raised; otherwise the call returns only when every rank has finished `step`, or raises PeerFailure."""
  try:
    out = run_sharded(fn, q, k, v, world, rank, extra)
  except Exception as e:   # noqa: BLE001 -- reported to the peers, then re-raised unchanged
    report_step(store, rank, step, ok=False, message=f"{type(e).__name__}: {e}")
    raise
  report_step(store, rank, step)
  check_peers(store, world, step, timeout_s)
  return out
