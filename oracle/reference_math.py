"""CPU restatement (PyTorch, fp32/fp64) of the reference's hot-path math.  Every function computes on the device
of its inputs, so a test may also evaluate it with plain fp32 torch on a GPU for the full-size configurations
(per batch element and head chunk, which bounds the [heads, Sq, Skv] temporaries).

THIS FILE IS TEST INFRASTRUCTURE.  Only tests/, __graft_entry__.smoke() and the cpu_baseline /
reference arms of bench.py may import it; the product (deepgengraph_b200/) never does.

Parity pin: every function below that has a counterpart among the reference's PyTorch modules
is checked in tests/test_oracle.py against golden outputs produced by importing and running
those modules themselves (tests/golden/make_golden.py, which needs the reference tree).  The csrc/ ops (RMSNorm, SiLU-gate, RoPE) are CUDA sources in
the reference; their restatements here are additionally compared on the GPU with the
reference kernels themselves when oracle/_ref holds a build of them (oracle/build_ref.py).
Features with no reference code at all (sliding window, grouped-query attention, head_dim 256,
GeGLU) are documented restatements: parity unpinned for exactly those options.

All line numbers are paths inside the reference project (DeepGenGroup/DeepGenGraph).
"""
import math

import torch
import torch.nn.functional as F


def _visible_mask(q_len, kv_len, causal=True, window=0, device="cpu"):
  """Boolean [q_len, kv_len]: key j visible to query i.

  causal: torch.triu(full(-inf), diagonal=kv_len - q_len + 1)  => visible iff j <= i + (kv_len - q_len)
          (deepgengraph_exp/cases/kernels/attn.py:22-23)
  window: additionally i + (kv_len - q_len) - j < window        (no reference lines; Gemma-2 semantics)
  """
  i = torch.arange(q_len, device=device)[:, None]
  j = torch.arange(kv_len, device=device)[None, :]
  delta = kv_len - q_len
  vis = torch.ones(q_len, kv_len, dtype=torch.bool, device=device)
  if causal:
    vis &= j <= i + delta
    if window and window > 0:
      vis &= (i + delta - j) < window
  return vis


def attention_ref(q, k, v, causal=True, window=0, softcap=0.0, scale=None, exp_rand=None, tau=1.0,
                  want=("out",), head_chunk=8):
  """fp32 restatement of the attention core modules.

  q [B, Sq, H, D], k/v [B, Skv, Hk, D] (any float dtype; upcast to fp32 first so that the oracle sees
  exactly the values the kernel sees).  Returns a dict with the requested entries:
    out       [B, Sq, H, D]  fp32   attn.py:29-34 (scores/sqrt(D), += mask, softmax in fp32, probs @ v);
                                    probs are rounded to the INPUT dtype before the product, as the
                                    reference does (attn.py:32 `probs.to(q.dtype)`)
    lse2      [B, H, Sq]     fp32   base-2 log-sum-exp of the masked logits (what b200_attn_fwd emits)
    colsum    [B, H, Skv]    fp32   h2o.py:35-38   sum over queries of fp32 probs
    colsum_sq [B, H, Skv]    fp32   roco.py:42-48  sum over queries of probs ** 2
    kf        [B, H, Skv]    fp32   kf.py:36-42    column sums of softmax((scores - log(exp_rand)) / tau)
    snapkv    [B, H, Skv]    fp32   snapkv.py:36-38 avg_pool1d(colsum, kernel 5, padding 2, stride 1)
    corm      [B, H, Skv]    bool   corm.py:35-37  any over queries of probs >= 1 / (i + 1)
  softcap > 0: scores = tanh(scores / softcap) * softcap after the scale, before the mask (gemma2.py:30-34).
  Grouped-query attention (H > Hk) expands k/v per group like roco.py:25-27, and every per-key statistic is
  taken from the probabilities AVERAGED over the H / Hk query heads of a K/V head (roco.py:39-40,
  figure/membound/attn.py:84-88,123-124,162-164,200-204): the score entries are then [B, Hk, Skv].
  (figure/membound/attn.py:240-244 computes Corm's group mean and then thresholds the un-averaged
  probabilities, after which its view to [B, Hk, Skv] cannot succeed; the restatement here thresholds the mean.)
  """
  in_dtype = q.dtype
  B, Sq, H, D = q.shape
  Skv, Hk = k.shape[1], k.shape[2]
  g = H // Hk
  scale = scale if scale else 1.0 / math.sqrt(D)
  dev = q.device
  vis = _visible_mask(Sq, Skv, causal, window, dev)
  res = {}
  if "out" in want:
    res["out"] = torch.empty(B, Sq, H, D, dtype=torch.float32, device=dev)
  if "lse2" in want:
    res["lse2"] = torch.empty(B, H, Sq, dtype=torch.float32, device=dev)
  for name in ("colsum", "colsum_sq", "kf", "snapkv"):
    if name in want:
      res[name] = torch.empty(B, Hk, Skv, dtype=torch.float32, device=dev)
  if "corm" in want:
    res["corm"] = torch.empty(B, Hk, Skv, dtype=torch.bool, device=dev)
  head_chunk = max(g, head_chunk // g * g)        # whole groups per chunk

  def group_mean(t):                              # [h, Sq, Skv] -> [h / g, Sq, Skv]
    return t if g == 1 else t.reshape(t.shape[0] // g, g, Sq, Skv).mean(dim=1)

  for b in range(B):
    for h0 in range(0, H, head_chunk):
      h1 = min(H, h0 + head_chunk)
      k0, k1 = h0 // g, h1 // g
      qh = q[b, :, h0:h1].float().transpose(0, 1)                       # [h, Sq, D]
      kv_idx = torch.arange(h0, h1, device=dev) // g
      kh = k[b][:, kv_idx].float().transpose(0, 1)                      # [h, Skv, D]
      vh = v[b][:, kv_idx].float().transpose(0, 1)
      scores = torch.matmul(qh, kh.transpose(-2, -1)) * scale           # attn.py:29
      if softcap and softcap > 0:
        scores = torch.tanh(scores / softcap) * softcap                 # gemma2.py:30-33
      scores = scores.masked_fill(~vis, float("-inf"))                  # attn.py:30
      probs = F.softmax(scores, dim=-1)                                 # attn.py:31
      if "out" in want:
        p_lo = probs.to(in_dtype).float() if in_dtype != torch.float32 else probs
        res["out"][b, :, h0:h1] = torch.matmul(p_lo, vh).transpose(0, 1)  # attn.py:32-34
      if "lse2" in want:
        res["lse2"][b, h0:h1] = torch.logsumexp(scores, dim=-1) / math.log(2.0)
      pm = group_mean(probs) if any(n in want for n in ("colsum", "colsum_sq", "snapkv", "corm")) else None
      if "colsum" in want:
        res["colsum"][b, k0:k1] = pm.sum(dim=1)                         # h2o.py:35-36 (sum over queries)
      if "colsum_sq" in want:
        res["colsum_sq"][b, k0:k1] = (pm ** 2).sum(dim=1)               # roco.py:39-46 (mean, then square)
      if "snapkv" in want:
        res["snapkv"][b, k0:k1] = F.avg_pool1d(pm.sum(dim=1)[None], kernel_size=5, padding=2, stride=1)[0]
      if "corm" in want:
        thr = 1.0 / torch.arange(1, Sq + 1, dtype=torch.float32, device=dev)[:, None]   # corm.py:47-49
        res["corm"][b, k0:k1] = (pm >= thr).any(dim=1)
      if "kf" in want:
        gumbels = -exp_rand[b, h0:h1].float().log()                     # kf.py:36-37
        z = (scores + gumbels) / tau                                    # kf.py:38 (masked entries stay -inf)
        res["kf"][b, k0:k1] = group_mean(F.softmax(z, dim=-1)).sum(dim=1)   # kf.py:39-40
  return res


def kv_evict_topk_ref(score, k, v, budget):
  """KV-cache eviction of the reference's model glue, verbatim semantics
  (deepgengraph_exp/cases/models/h2o.py:51-57): topk(score, budget) -> sort the indices -> gather k and v rows ->
  cat([k_cache, v_cache], dim=1).  score [B, H, S] fp32, k/v [B, S, H, D].  Returns (kv_cache [B, 2, budget, H, D],
  sorted indices [B, H, budget])."""
  B, S, H, D = k.shape
  _, sel = torch.topk(score, k=budget, dim=-1, sorted=True)
  sel = sel.sort(dim=-1)[0]                                            # [B, H, budget]
  index = sel.transpose(1, 2)[:, :, :, None].expand(B, budget, H, D)
  k_cache = torch.gather(k, dim=1, index=index).view(B, 1, budget, H, D)
  v_cache = torch.gather(v, dim=1, index=index).view(B, 1, budget, H, D)
  return torch.cat([k_cache, v_cache], dim=1), sel


def kv_evict_roco_ref(score, score_sq, k, v, q_len, budget, recent):
  """RoCo's KV-cache eviction, the reference's own sequence of torch calls
  (deepgengraph_exp/cases/models/roco.py:52-66): std from the two column sums, the `recent` keys of largest std are
  always kept, of the others the `budget` keys of largest mean score; sorted, gathered, concatenated.
  score, score_sq [B, H, S] fp32; k/v [B, S, H, D].  Returns (kv_cache [B, 2, budget + recent, H, D],
  sorted indices [B, H, budget + recent])."""
  B, S, H, D = k.shape
  std = torch.sqrt(score_sq / q_len - (score / q_len) ** 2)
  _, other = torch.topk(std, largest=False, k=S - recent, dim=-1)
  _, rec = torch.topk(std, largest=True, k=recent, dim=-1)
  _, sel_in_other = torch.topk(score.gather(dim=-1, index=other) / q_len, dim=-1, k=budget)
  sel = other.gather(dim=-1, index=sel_in_other)
  sel = torch.cat([sel, rec], dim=-1).sort(dim=-1)[0]                  # [B, H, budget + recent]
  keep = budget + recent
  index = sel.transpose(1, 2)[:, :, :, None].expand(B, keep, H, D)
  k_cache = torch.gather(k, dim=1, index=index).view(B, 1, keep, H, D)
  v_cache = torch.gather(v, dim=1, index=index).view(B, 1, keep, H, D)
  return torch.cat([k_cache, v_cache], dim=1), sel


# --------------------------------------------------------------------------------------------
# csrc/ ops.  Semantic truth = the CUDA sources (csrc/norm.cu, activation.cu, pos_encoding.cu);
# the Python stand-ins in deepgengraph_exp/cases/models/llama_base.py discard their results.
# --------------------------------------------------------------------------------------------
def rms_norm_ref(x, weight, eps):
  """out = T(x * rsqrt(mean(x^2) + eps)) * w with the last product taken in T (csrc/norm.cu:42-55).
  Returned in fp32 (exactly representable: it is the T-rounded product)."""
  xf = x.float()
  inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
  normed = (xf * inv).to(x.dtype)
  return (normed.float() * weight.float()).to(x.dtype).float()


def fused_add_rms_norm_ref(x, residual, weight, eps):
  """residual' = T(x + residual); x' = T(residual' * rsqrt(mean((x + residual)^2) + eps)) * w
  -- variance from the UNROUNDED fp32 sum (csrc/norm.cu:68-70), scaling from the rounded residual (:80).
  Returns (x', residual') in fp32."""
  s = x.float() + residual.float()
  inv = torch.rsqrt(s.pow(2).mean(dim=-1, keepdim=True) + eps)
  res_new = s.to(x.dtype)
  normed = (res_new.float() * inv).to(x.dtype)
  return (normed.float() * weight.float()).to(x.dtype).float(), res_new.float()


def silu_and_mul_ref(x):
  """out = T(silu(x[..., :d])) * x[..., d:] (csrc/activation.cu:6-22)."""
  d = x.shape[-1] // 2
  a, b = x[..., :d].float(), x[..., d:].float()
  act = (a / (1.0 + torch.exp(-a))).to(x.dtype)
  return (act.float() * b).to(x.dtype).float()


def gelu_tanh_and_mul_ref(x):
  """GeGLU sibling of silu_and_mul: out = T(gelu(x[..., :d], approximate='tanh')) * x[..., d:].
  No reference lines (config 5 needs it; the reference asserts hidden_act == 'silu',
  deepgengraph_exp/cases/models/llama_base.py:299)."""
  d = x.shape[-1] // 2
  a, b = x[..., :d].float(), x[..., d:].float()
  act = F.gelu(a, approximate="tanh").to(x.dtype)
  return (act.float() * b).to(x.dtype).float()


def rotary_online_ref(positions, query, key, head_dim, theta):
  """NeoX-style rotation with on-the-fly frequencies (csrc/pos_encoding.cu:83-111):
  freq_i = pos / theta^(2i/D); (x, y) = (a[i], a[i + D/2]); a[i] = x cos - y sin; a[i+D/2] = y cos + x sin.
  Angles in fp64 (the reference's fast-math __powf/__sincosf are an approximation of this).
  Returns rotated (query, key) in fp32, same shapes as the inputs ([T, heads*D])."""
  half = head_dim // 2
  i = torch.arange(half, dtype=torch.float64, device=positions.device)
  inv_freq = 1.0 / (float(theta) ** (2.0 * i / head_dim))
  ang = positions.double()[:, None] * inv_freq[None, :]          # [T, D/2]
  cos, sin = ang.cos(), ang.sin()

  def rot(t):
    T = t.shape[0]
    a = t.double().reshape(T, -1, head_dim)
    x, y = a[..., :half], a[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x * c - y * s, y * c + x * s], dim=-1).reshape(T, -1).float()

  return rot(query), rot(key)


# --------------------------------------------------------------------------------------------
# Gemma-2-style decoder layer (config 5).  Structure = the reference's LlamaLayer
# (deepgengraph_exp/cases/models/gemma2.py:55-80: pre-norm x2, plain `w` scale as in csrc/norm.cu:54),
# with the options the reference has no code for (GQA, head_dim 256, sliding window, GeGLU).
# --------------------------------------------------------------------------------------------
def gemma2_layer_ref(x, w, cfg):
  """x [B, S, hidden] (bf16/fp16/fp32). w: dict of weights (ln1, qkv, o, ln2, gate_up, down), each stored in
  the model dtype.  Linear layers are evaluated in fp32 on the stored values and rounded to the model dtype
  after every op, mirroring a 16-bit pipeline.  Returns fp32 [B, S, hidden]."""
  dt = x.dtype
  B, S, hidden = x.shape
  H, Hk, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]

  def lin(t, wt):  # y = t @ wt^T in fp32, rounded to the model dtype
    return (t.float() @ wt.float().t()).to(dt)

  h = rms_norm_ref(x, w["ln1"], cfg["eps"]).to(dt)
  qkv = lin(h, w["qkv"])
  q, k, v = qkv.split([H * D, Hk * D, Hk * D], dim=-1)
  pos = torch.arange(S, dtype=torch.int32, device=x.device).repeat(B)
  qr, kr = rotary_online_ref(pos, q.reshape(B * S, H * D), k.reshape(B * S, Hk * D), D, cfg["rope_theta"])
  qr, kr = qr.to(dt).view(B, S, H, D), kr.to(dt).view(B, S, Hk, D)
  a = attention_ref(qr, kr, v.reshape(B, S, Hk, D), causal=True, window=cfg["window"], softcap=cfg["softcap"],
                    want=("out",), head_chunk=2)["out"].to(dt)
  o = lin(a.reshape(B, S, H * D), w["o"])
  x1 = (x.float() + o.float()).to(dt)
  h2 = rms_norm_ref(x1, w["ln2"], cfg["eps"]).to(dt)
  gu = lin(h2, w["gate_up"])
  act = gelu_tanh_and_mul_ref(gu).to(dt)
  dn = lin(act, w["down"])
  return (x1.float() + dn.float()).to(dt).float()


def gemma2_layer_ref_fp32(x, w, cfg, head_chunk=2):
  """The same layer evaluated in fp32 end to end: the stored (16-bit) values of x and of the weights are upcast once
  and NOTHING is rounded afterwards -- the fp32 reference that a 16-bit pipeline is held against at
  rtol = atol = 2e-2.  Computes on the device of x.  Returns fp32 [B, S, hidden]."""
  B, S, hidden = x.shape
  H, Hk, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
  xf = x.float()
  wf = {k: t.float() for k, t in w.items()}

  def norm(t, weight):                                    # csrc/norm.cu:42-55 without the two roundings to T
    return t * torch.rsqrt(t.pow(2).mean(dim=-1, keepdim=True) + cfg["eps"]) * weight

  h = norm(xf, wf["ln1"])
  qkv = h @ wf["qkv"].t()
  q, k, v = qkv.split([H * D, Hk * D, Hk * D], dim=-1)
  pos = torch.arange(S, dtype=torch.int32, device=x.device).repeat(B)
  qr, kr = rotary_online_ref(pos, q.reshape(B * S, H * D), k.reshape(B * S, Hk * D), D, cfg["rope_theta"])
  a = attention_ref(qr.view(B, S, H, D), kr.view(B, S, Hk, D), v.reshape(B, S, Hk, D), causal=True,
                    window=cfg["window"], softcap=cfg["softcap"], want=("out",), head_chunk=head_chunk)["out"]
  x1 = xf + a.reshape(B, S, H * D) @ wf["o"].t()
  gu = norm(x1, wf["ln2"]) @ wf["gate_up"].t()
  d = gu.shape[-1] // 2
  act = F.gelu(gu[..., :d], approximate="tanh") * gu[..., d:]
  return x1 + act @ wf["down"].t()
