"""Two-GPU run of the sharded score path: each rank runs the single-GPU kernels on its (batch, head) shard, the
score vectors are all-gathered over NCCL, and rank 0 compares the assembled result with the one-GPU run.
Skipped on boxes with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
  s = socket.socket()
  s.bind(("127.0.0.1", 0))
  port = s.getsockname()[1]
  s.close()
  return port


def _worker(rank, world, port):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  torch.cuda.set_device(rank)
  dev = torch.device("cuda", rank)
  dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
  try:
    from deepgengraph_b200 import attention as att
    from deepgengraph_b200 import sharding as sh
    B, S, H, D = 2, 512, 6, 128
    g = torch.Generator().manual_seed(0)                       # same full problem on every rank
    q, k, v = (torch.randn(B, S, H, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(3))
    results = sh.run_sharded(lambda a, b, c: att.attn_score_fwd(a, b, c), q, k, v, world, rank)
    local = sh.scores_from_pieces(results, index=1)
    full = sh.gather_scores(local, B * H, world, rank)
    assert tuple(full.shape) == (B * H, S)
    ref_out, ref_score = att.attn_score_fwd(q, k, v)
    torch.cuda.synchronize()
    # per-unit results are bit-identical to the one-GPU run: a unit's computation does not depend on its neighbours
    assert torch.equal(full, ref_score.reshape(B * H, S))
    for piece, (out, _) in results:
      assert torch.equal(out[0], ref_out[piece.b, :, piece.hk_lo:piece.hk_hi])
  finally:
    dist.destroy_process_group()


def test_sharded_scores_match_single_gpu():
  if torch.cuda.device_count() < 2:
    pytest.skip("needs two GPUs")
  mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
