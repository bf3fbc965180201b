"""The persistent attention kernel (CTAs walk many query tiles, barrier phases and rings carried across tiles,
dynamic tile order) must produce the bits of the one-tile-per-CTA kernel (same per-tile arithmetic, static
order) on random shapes: ragged lengths, grouped heads, windows, soft-cap, both head dims, both dtypes."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
N_PROBLEMS = 40


def _run(env_extra):
  env = dict(os.environ)
  env.pop("B200_ATTN_ONE_TILE_PER_CTA", None)
  env.update(env_extra)
  res = subprocess.run([sys.executable, os.path.join(HERE, "_attn_hashes.py"), str(N_PROBLEMS)], env=env,
                       capture_output=True, text=True, timeout=600)
  assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
  line = [ln for ln in res.stdout.splitlines() if ln.startswith("HASHES ")][-1]
  return json.loads(line[len("HASHES "):])


def test_same_bits_from_both_launch_schemes(cuda_device):
  persistent = _run({})
  one_tile = _run({"B200_ATTN_ONE_TILE_PER_CTA": "1"})
  assert len(persistent) == N_PROBLEMS
  differing = [i for i, (a, b) in enumerate(zip(persistent, one_tile)) if a != b]
  assert not differing, f"problems {differing} differ between the persistent and the one-tile-per-CTA kernel"
