"""Decoder layers built from this package's ops.

gemma2_layer -- Gemma-2-style layer (config: hidden 3584, 16 query / 8 kv heads, head_dim 256, sliding window
4096, logit soft-cap 50, RMSNorm eps 1e-6, RoPE base 10000, GeGLU 14336).  Structure follows the reference's
LlamaLayer (deepgengraph_exp/cases/models/gemma2.py:55-80 with the op wrappers of llama_base.py:257-314):
RMSNorm -> QKV projection -> RoPE -> attention -> output projection -> residual -> RMSNorm -> gate/up projection
-> gated activation -> down projection -> residual.

llama_score_layer -- the reference's Llama-shaped layer with a score-producing attention variant and the KV-cache
eviction that follows it (deepgengraph_exp/cases/models/h2o.py:34-86, roco.py, kf.py): RMSNorm -> QKV projection
-> RoPE -> attn_f (out + per-key scores) -> top-k eviction into the compact cache -> output projection ->
residual -> RMSNorm -> SiLU-gated MLP -> residual.

The four projections of a layer are plain library GEMMs (torch.matmul -> cuBLAS); everything else is this
package's CUDA: rms_norm / fused_add_rms_norm, rotary_embedding_online in place on the q and k column ranges of
the fused QKV buffer, the fused attention kernels, the eviction kernels and the gated activations.  In
gemma2_layer q, k, v stay VIEWS of the projection output (the attention kernel reads them through strided TMA
descriptors: no split copies); the score variants take dense tensors, so llama_score_layer splits them once.
Unlike the reference's layers there is no torch.cuda.synchronize() between the ops (models/attn.py:42).
"""
import torch

from . import attention as _att
from . import native_ops as _ops


class Gemma2LayerConfig:
  def __init__(self, hidden=3584, heads=16, kv_heads=8, head_dim=256, window=4096, softcap=50.0, eps=1e-6,
               rope_theta=10000.0, intermediate=14336):
    self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
    self.window, self.softcap, self.eps, self.rope_theta, self.intermediate = window, softcap, eps, rope_theta, intermediate

  def as_dict(self):
    return dict(hidden=self.hidden, heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim,
                window=self.window, softcap=self.softcap, eps=self.eps, rope_theta=self.rope_theta,
                intermediate=self.intermediate)


def init_weights(cfg, dtype=torch.bfloat16, device="cuda", seed=0, std=0.02):
  """Random weights ~ N(0, std) in the layout gemma2_layer expects; norm scales are 1 + N(0, std)."""
  g = torch.Generator().manual_seed(seed)
  qkv_out = (cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim

  def w(*shape):
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

  return dict(ln1=(1 + torch.randn(cfg.hidden, generator=g) * std).to(dtype).to(device),
              qkv=w(qkv_out, cfg.hidden), o=w(cfg.hidden, cfg.heads * cfg.head_dim),
              ln2=(1 + torch.randn(cfg.hidden, generator=g) * std).to(dtype).to(device),
              gate_up=w(2 * cfg.intermediate, cfg.hidden), down=w(cfg.hidden, cfg.intermediate))


def gemma2_layer(x, w, cfg, positions=None):
  """x [B, S, hidden] (fp16/bf16, CUDA). Returns a new [B, S, hidden] tensor."""
  B, S, hidden = x.shape
  H, Hk, D = cfg.heads, cfg.kv_heads, cfg.head_dim
  T = B * S
  xf = x.reshape(T, hidden)
  h = torch.empty_like(xf)
  _ops.rms_norm(h, xf, w["ln1"], cfg.eps)
  qkv = torch.matmul(h, w["qkv"].t())                                  # [T, (H + 2 Hk) D]
  if positions is None:
    positions = torch.arange(S, dtype=torch.int32, device=x.device).repeat(B)
  _ops.rotary_embedding_online(positions, qkv[:, :H * D], qkv[:, H * D:(H + Hk) * D], D, cfg.rope_theta)
  # q / k / v stay views of the projection output (no split copies; the reference makes three,
  # models/attn.py:37-40, and synchronises the device, :43): the attention kernel reads them through strided
  # TMA descriptors
  qkv3 = qkv.view(B, S, (H + 2 * Hk) * D)
  q = qkv3[:, :, :H * D].unflatten(-1, (H, D))
  k = qkv3[:, :, H * D:(H + Hk) * D].unflatten(-1, (Hk, D))
  v = qkv3[:, :, (H + Hk) * D:].unflatten(-1, (Hk, D))
  a = _att.attn_fwd(q, k, v, causal=True, window=cfg.window, softcap=cfg.softcap)
  o = torch.matmul(a.reshape(T, H * D), w["o"].t())                    # attention block output
  # residual add fused with the second norm: res <- x + o (in place in `res`), o <- rms_norm(res)
  res = xf.clone()
  _ops.fused_add_rms_norm(o, res, w["ln2"], cfg.eps)
  gu = torch.matmul(o, w["gate_up"].t())
  act = torch.empty(T, cfg.intermediate, dtype=x.dtype, device=x.device)
  _ops.gelu_tanh_and_mul(act, gu)
  dn = torch.matmul(act, w["down"].t())
  return (res + dn).reshape(B, S, hidden)


class LlamaLayerConfig:
  """The reference's random-weight layer setup (run_e2e.py:24-46,48-66): Llama-7B shapes, cache budget 512."""

  def __init__(self, hidden=4096, heads=32, kv_heads=32, eps=1e-6, rope_theta=10000.0, intermediate=11008,
               cache_budget=512, roco_recent=256, tau=1.5):
    self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, hidden // heads
    self.eps, self.rope_theta, self.intermediate = eps, rope_theta, intermediate
    self.cache_budget, self.roco_recent, self.tau = cache_budget, roco_recent, tau


def init_llama_weights(cfg, dtype=torch.float16, device="cuda", seed=0, std=0.02):
  g = torch.Generator().manual_seed(seed)
  qkv_out = (cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim

  def w(*shape):
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

  return dict(ln1=torch.ones(cfg.hidden, dtype=dtype, device=device), qkv=w(qkv_out, cfg.hidden),
              o=w(cfg.hidden, cfg.heads * cfg.head_dim), ln2=torch.ones(cfg.hidden, dtype=dtype, device=device),
              gate_up=w(2 * cfg.intermediate, cfg.hidden), down=w(cfg.hidden, cfg.intermediate))


def llama_score_layer(x, w, cfg, variant="h2o", exp_rand=None):
  """x [B, S, hidden].  variant: 'h2o' (column sums -> top-k eviction, models/h2o.py:34-59), 'roco' (column sums of
  p and p^2 -> RoCo's two-stage eviction, models/roco.py:36-68) or 'kf' (KeyFormer score -> top-k, models/kf.py:36-62;
  exp_rand [B, heads, S, S] float32).  Returns (y [B, S, hidden], score(s), kv_cache)."""
  B, S, hidden = x.shape
  H, Hk, D = cfg.heads, cfg.kv_heads, cfg.head_dim
  T = B * S
  xf = x.reshape(T, hidden)
  h = torch.empty_like(xf)
  _ops.rms_norm(h, xf, w["ln1"], cfg.eps)
  qkv = torch.matmul(h, w["qkv"].t())
  positions = torch.arange(S, dtype=torch.int32, device=x.device).repeat(B)
  _ops.rotary_embedding_online(positions, qkv[:, :H * D], qkv[:, H * D:(H + Hk) * D], D, cfg.rope_theta)
  q, k, v = (t.contiguous().view(B, S, -1, D) for t in qkv.split([H * D, Hk * D, Hk * D], dim=-1))
  if variant == "h2o":
    a, score = _att.attn_score_fwd(q, k, v, causal=True)
    kv_cache = _att.kv_evict_topk(score, k, v, cfg.cache_budget)
    scores = (score,)
  elif variant == "roco":
    a, score, score_sq = _att.attn_score_fwd(q, k, v, want_sq=True, causal=True)
    kv_cache = _att.kv_evict_roco(score, score_sq, k, v, S, cfg.cache_budget, cfg.roco_recent)   # models/roco.py:55-59
    scores = (score, score_sq)
  elif variant == "kf":
    a, score = _att.attn_kf_fwd(q, k, v, exp_rand, tau=cfg.tau, causal=True)
    kv_cache = _att.kv_evict_topk(score, k, v, cfg.cache_budget)
    scores = (score,)
  else:
    raise ValueError(f"unknown variant {variant!r}")
  o = torch.matmul(a.reshape(T, H * D), w["o"].t())
  res = xf.clone()
  _ops.fused_add_rms_norm(o, res, w["ln2"], cfg.eps)        # res <- x + attention block; o <- rms_norm(res)
  gu = torch.matmul(o, w["gate_up"].t())
  act = torch.empty(T, cfg.intermediate, dtype=x.dtype, device=x.device)
  _ops.silu_and_mul(act, gu)
  dn = torch.matmul(act, w["down"].t())
  return (res + dn).reshape(B, S, hidden), scores, kv_cache
