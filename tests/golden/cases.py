"""Seeded inputs of the golden parity cases, generated without any library RNG so that the exact
same values can be rebuilt anywhere: an integer hash of the element index mapped onto a grid that is exactly representable
in fp16 / bf16.  Shared by make_golden.py (which feeds them to the reference modules) and by the
tests (which feed them to the oracle and to the CUDA kernels)."""
import numpy as np
import torch


def lcg_grid(shape, seed, lo=-2.0, step=1.0 / 64, levels=257):
  """Values lo + step * (h(index, seed) % levels), h = a splitmix64-style hash of the flat index;
  float32 array of `shape`.  Pure integer arithmetic, so the values are identical on every machine."""
  n = int(np.prod(shape))
  state = np.uint64((seed * 2654435761 + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF)
  a, c = np.uint64(6364136223846793005), np.uint64(1442695040888963407)
  idx = np.arange(n, dtype=np.uint64)
  with np.errstate(over="ignore"):
    z = idx * a + state + c
    z ^= z >> np.uint64(30)
    z *= np.uint64(0xBF58476D1CE4E5B9)
    z ^= z >> np.uint64(27)
    z *= np.uint64(0x94D049BB133111EB)
    z ^= z >> np.uint64(31)
  out = (lo + step * (z % np.uint64(levels)).astype(np.float32)).astype(np.float32)
  return out.reshape(shape)


# name -> dict(model, ctor kwargs, B, Sq, Skv, H[, Hk], D, q_gain[, source])
CASES = {
    "attn_s192": dict(model="attn", B=1, Sq=192, Skv=192, H=2, D=128),
    "attn_sq128_skv320": dict(model="attn", B=1, Sq=128, Skv=320, H=2, D=128),
    "attn_b2_s256": dict(model="attn", B=2, Sq=256, Skv=256, H=3, D=128),
    "gemma2_s192": dict(model="gemma2", B=1, Sq=192, Skv=192, H=2, D=128, q_gain=16.0),
    "h2o_s256": dict(model="h2o", B=1, Sq=256, Skv=256, H=2, D=128),
    "h2o_sq64_skv192": dict(model="h2o", B=1, Sq=64, Skv=192, H=2, D=128),
    "roco_s192": dict(model="roco", B=1, Sq=192, Skv=192, H=2, D=128),
    "kf_s192_tau1p5": dict(model="kf", B=1, Sq=192, Skv=192, H=2, D=128, tau=1.5),
    "kf_s256_tau1": dict(model="kf", B=1, Sq=256, Skv=256, H=2, D=128, tau=1.0),
    "snapkv_s192": dict(model="snapkv", B=1, Sq=192, Skv=192, H=2, D=128),
    "corm_s192": dict(model="corm", B=1, Sq=192, Skv=192, H=2, D=128),
    # grouped-query attention (Hk < H): produced by the reference's GQA-capable module variants
    # (deepgengraph_exp/figure/membound/attn.py), whose scores are the group mean of the probabilities
    "attn_gqa_s192": dict(model="attn", B=1, Sq=192, Skv=192, H=4, Hk=2, D=128, source="membound"),
    "h2o_gqa_s192": dict(model="h2o", B=1, Sq=192, Skv=192, H=4, Hk=2, D=128, source="membound"),
    "roco_gqa_sq128_skv256": dict(model="roco", B=2, Sq=128, Skv=256, H=6, Hk=2, D=128, source="membound"),
    "snapkv_gqa_s192": dict(model="snapkv", B=1, Sq=192, Skv=192, H=4, Hk=1, D=128, source="membound"),
}


def make_inputs(name, dtype=torch.float32):
  """Returns dict(q, k, v[, exp_rand]) as torch tensors (q/k/v in `dtype`, values exact in fp16/bf16)."""
  c = CASES[name]
  seed = sum(ord(ch) * (i + 1) for i, ch in enumerate(name))
  B, Sq, Skv, H, D = c["B"], c["Sq"], c["Skv"], c["H"], c["D"]
  Hk = c.get("Hk", H)
  q = lcg_grid((B, Sq, H, D), seed + 1) * c.get("q_gain", 1.0)
  k = lcg_grid((B, Skv, Hk, D), seed + 2)
  v = lcg_grid((B, Skv, Hk, D), seed + 3)
  out = {"q": torch.from_numpy(q).to(dtype), "k": torch.from_numpy(k).to(dtype), "v": torch.from_numpy(v).to(dtype)}
  if c["model"] == "kf":
    # strictly positive, exactly representable: 1/256 .. 4
    er = lcg_grid((B, H, Sq, Skv), seed + 4, lo=1.0 / 256, step=1.0 / 256, levels=1024)
    out["exp_rand"] = torch.from_numpy(er)
  return out


ROW_STRIDE = 8  # golden files keep every 8th query row of `out` plus whole-tensor checksums
