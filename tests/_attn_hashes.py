"""Helper of test_gpu_persistent_vs_one_tile.py: runs seeded random attention problems and prints one SHA-1 per
problem (output + log-sum-exp bytes) as JSON.  Run as a child process so that the kernel variant -- chosen once
per process from the environment -- can differ between two runs."""
import hashlib
import json
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

from deepgengraph_b200 import attention as att  # noqa: E402


def cases(n, seed=1234):
  rnd = random.Random(seed)
  out = []
  for _ in range(n):
    D = rnd.choice([128, 128, 128, 256])
    Hk = rnd.choice([1, 2, 3, 4, 8])
    H = Hk * rnd.choice([1, 1, 2, 4])
    B = rnd.choice([1, 2, 3, 5])
    Sq = rnd.choice([1, 64, 127, 128, 129, 300, 512, 777, 1024, 1500, 2048, 3000])
    Skv = Sq + rnd.choice([0, 0, 0, 1, 64, 200])
    window = rnd.choice([0, 0, 0, 1, 17, 64, 128, 500])
    softcap = rnd.choice([0.0, 0.0, 30.0])
    dtype = rnd.choice(["bfloat16", "float16"])
    out.append((B, Sq, Skv, H, Hk, D, window, softcap, dtype))
  return out


def main(n):
  hashes = []
  for ci, (B, Sq, Skv, H, Hk, D, window, softcap, dtype) in enumerate(cases(n)):
    gen = torch.Generator(device="cuda").manual_seed(ci)
    dt = getattr(torch, dtype)
    q = torch.randn(B, Sq, H, D, generator=gen, device="cuda", dtype=dt)
    k = torch.randn(B, Skv, Hk, D, generator=gen, device="cuda", dtype=dt)
    v = torch.randn(B, Skv, Hk, D, generator=gen, device="cuda", dtype=dt)
    first = None
    for _ in range(2):   # a rerun must give the same bits
      out, lse = att.attn_fwd_with_lse(q, k, v, causal=True, window=window, softcap=softcap)
      assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all(), (ci, B, Sq, Skv, H, Hk, D, window)
      h = hashlib.sha1(out.cpu().view(torch.int16).numpy().tobytes() + lse.cpu().numpy().tobytes()).hexdigest()
      assert first is None or first == h, f"rerun differs for problem {ci}"
      first = h
    hashes.append(first)
  print("HASHES " + json.dumps(hashes))


if __name__ == "__main__":
  main(int(sys.argv[1]))
