"""Gemma-2-style decoder layer built from this package's ops (config: hidden 3584, 16 query / 8 kv heads,
head_dim 256, sliding window 4096, logit soft-cap 50, RMSNorm eps 1e-6, RoPE base 10000, GeGLU 14336).

Structure follows the reference's LlamaLayer (deepgengraph_exp/cases/models/gemma2.py:55-80 with the op
wrappers of llama_base.py:257-314): RMSNorm -> QKV projection -> RoPE -> attention -> output projection
-> residual -> RMSNorm -> gate/up projection -> gated activation -> down projection -> residual.
The four projections are plain library GEMMs (torch.matmul -> cuBLAS), everything else is this
package's CUDA: rms_norm / fused_add_rms_norm, rotary_embedding_online (in place on the fused QKV buffer,
no split copies), the fused attention kernel reading q, k, v as strided BSHD views is not possible (TMA
needs dense tensors), so q/k/v are split once, and gelu_tanh_and_mul.
Unlike the reference's layer there is no torch.cuda.synchronize() between the ops (models/attn.py:42).
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
