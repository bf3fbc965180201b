"""The counter-based noise generator of the seeded KeyFormer path (host side: deepgengraph_b200.attention.kf_noise).
No GPU needed."""
import math

import torch

from deepgengraph_b200 import attention as att


def _run(counter, key):
  words = att.philox4x32_10(*[torch.tensor([c], dtype=torch.int64) for c in counter], key[0], key[1])
  return [int(w) for w in words]


def test_philox4x32_10_known_answers():
  # known-answer vectors published with the generator (Random123, kat_vectors: philox4x32 10)
  assert _run([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
  assert _run([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
  assert _run([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
      [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_kf_noise_is_exponential_and_its_negative_log_is_gumbel():
  n = att.kf_noise(seed=1234, batch=2, heads=3, q_len=64, kv_len=250)      # kv_len not a multiple of 4
  assert n.shape == (2, 3, 64, 250) and n.dtype == torch.float32 and (n > 0).all() and torch.isfinite(n).all()
  assert abs(n.mean().item() - 1.0) < 0.02 and abs(n.var().item() - 1.0) < 0.05          # Exponential(1)
  g = -torch.log(n)
  assert abs(g.mean().item() - 0.5772156649) < 0.02 and abs(g.var().item() - math.pi ** 2 / 6) < 0.06   # Gumbel(0, 1)


def test_kf_noise_is_a_pure_function_of_seed_and_position():
  a = att.kf_noise(7, 1, 2, 16, 32)
  assert torch.equal(a, att.kf_noise(7, 1, 2, 16, 32))
  assert not torch.equal(a, att.kf_noise(8, 1, 2, 16, 32))
  big = att.kf_noise(7, 2, 2, 24, 40)             # element (b, h, i, j) depends on b * heads + h, i, j only
  assert torch.equal(big[0, :, :16, :32], a[0])
  hi = att.kf_noise(7 + (1 << 32), 1, 2, 16, 32)  # the upper seed word is the second key word
  assert not torch.equal(a, hi)
