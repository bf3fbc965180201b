"""Fused attention core modules on BSHD tensors.

  attn_fwd(q, k, v, causal=True, window=-1, softcap=0.0, scale=None) -> out
  attn_score_fwd(q, k, v, want_sq=False, ...)                       -> (out, colsum[, colsum_sq])
  attn_kf_fwd(q, k, v, exp_rand | None, tau, ..., seed)             -> (out, kf_score)
  kf_noise(seed, batch, heads, q_len, kv_len, device)               -> exp_rand of the in-kernel generator
  attn_snapkv_fwd(q, k, v, kernel_size=5, ...)                      -> (out, pooled colsum)
  attn_corm_fwd(q, k, v, ...)                                       -> (out, bool flags)

q [B, Sq, H, D], k/v [B, Skv, Hk, D] (fp16 or bf16, contiguous); outputs are freshly allocated
on every call like the kernels the reference generates (to_triton.cpp:579-590): out [B, Sq, H, D]
in the input dtype, score vectors float32 [B, Hk, Skv].

The same three functions are registered as torch custom ops under the `b200attn` namespace
(torch.ops.b200attn.attn_fwd, ...) with fake implementations, so that they can sit inside
traced / compiled graphs.
"""
import math

import torch

from .tracing import traced

from . import _lib
from .native_ops import _dtype_code, _on_device, _require_cuda, _stream_ptr


def _row_strided(t):
  """True for a [B, S, H, D] view whose heads are packed (stride D) inside token rows that may be wider than
  H * D -- e.g. the q / k / v slices of a fused QKV projection output."""
  B, S, H, D = t.shape
  sb, ss, sh, sd = t.stride()
  return (sd == 1 and sh == D and ss >= H * D and ss % 8 == 0 and (B == 1 or (sb >= S * ss and sb % 8 == 0))
          and t.data_ptr() % 16 == 0)


def _check_qkv(where, q, k, v, allow_row_strided=False):
  dev = _require_cuda(where, q, k, v)
  if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
    raise ValueError(f"{where}: q, k, v must be [batch, seq, heads, head_dim]")
  if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
    raise TypeError(f"{where}: q, k, v must share dtype float16 or bfloat16 (got {q.dtype}, {k.dtype}, {v.dtype})")
  if k.shape != v.shape or k.size(0) != q.size(0) or k.size(3) != q.size(3):
    raise ValueError(f"{where}: shape mismatch q={tuple(q.shape)} k={tuple(k.shape)} v={tuple(v.shape)}")
  if q.size(2) % k.size(2) != 0:
    raise ValueError(f"{where}: heads ({q.size(2)}) not a multiple of kv heads ({k.size(2)})")
  if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
    if not (allow_row_strided and _row_strided(q) and _row_strided(k) and _row_strided(v)):
      raise ValueError(f"{where}: q, k, v must be contiguous" +
                       (" or row-strided views (packed heads, 16-byte aligned strides)" if allow_row_strided else ""))
  return dev


def _attn_fwd_impl(q, k, v, causal, window, softcap, scale, want_lse=False):
  where = "attn_fwd"
  dev = _check_qkv(where, q, k, v, allow_row_strided=True)
  B, Sq, H, D = q.shape
  Skv, Hk = k.size(1), k.size(2)
  if scale is None or scale <= 0:
    scale = 1.0 / math.sqrt(D)
  out = torch.empty((B, Sq, H, D), dtype=q.dtype, device=dev)
  lse = torch.empty((B, H, Sq), dtype=torch.float32, device=dev) if want_lse else None
  if B == 0 or Sq == 0:   # empty batch / no queries: nothing to launch (the torch reference returns empty tensors)
    return (out, lse) if want_lse else out
  with _on_device(dev):
    if q.is_contiguous() and k.is_contiguous() and v.is_contiguous():
      st = _lib.load().b200_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                     lse.data_ptr() if want_lse else None, B, Sq, Skv, H, Hk, D,
                                     _dtype_code(q, where), int(bool(causal)), int(window), float(softcap),
                                     float(scale), _stream_ptr(dev))
    else:
      # views into a wider buffer (fused QKV projection output): no copy, the strides go to the TMA descriptors
      def strides(t):
        return t.stride(1), (t.stride(0) if t.size(0) > 1 else t.size(1) * t.stride(1))
      (qt, qb), (kt, kb), (vt, vb) = strides(q), strides(k), strides(v)
      st = _lib.load().b200_attn_fwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                             lse.data_ptr() if want_lse else None, B, Sq, Skv, H, Hk, D,
                                             _dtype_code(q, where), qt, qb, kt, kb, vt, vb, int(bool(causal)),
                                             int(window), float(softcap), float(scale), _stream_ptr(dev))
  _lib.check(st, where)
  return (out, lse) if want_lse else out


def _workspace(dev, B, Sq, Skv, H):
  nbytes = _lib.load().b200_attn_score_workspace_bytes(B, Sq, Skv, H)
  return torch.empty(nbytes, dtype=torch.uint8, device=dev), nbytes


def _attn_score_impl(q, k, v, want_sq, causal, window, softcap, scale):
  where = "attn_score_fwd"
  dev = _check_qkv(where, q, k, v)
  B, Sq, H, D = q.shape
  Skv, Hk = k.size(1), k.size(2)
  if scale is None or scale <= 0:
    scale = 1.0 / math.sqrt(D)
  out = torch.empty_like(q)
  score = torch.empty((B, Hk, Skv), dtype=torch.float32, device=dev)
  score_sq = torch.empty((B, Hk, Skv), dtype=torch.float32, device=dev) if want_sq else None
  if B == 0 or Sq == 0:   # no queries: every column sum is an empty sum
    score.zero_()
    if want_sq:
      score_sq.zero_()
    return (out, score, score_sq) if want_sq else (out, score)
  ws, nbytes = _workspace(dev, B, Sq, Skv, H)
  if H != Hk:
    # grouped-query attention: mean over the query heads of a K/V head, then the sums (kernels/roco.py:39-46)
    with _on_device(dev):
      st = _lib.load().b200_attn_score_gqa(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                           score.data_ptr(), score_sq.data_ptr() if want_sq else None, None,
                                           ws.data_ptr(), nbytes, B, Sq, Skv, H, Hk, D, _dtype_code(q, where),
                                           int(bool(causal)), int(window), float(softcap), float(scale),
                                           _stream_ptr(dev))
    _lib.check(st, where)
    return (out, score, score_sq) if want_sq else (out, score)
  with _on_device(dev):
    st = _lib.load().b200_attn_score(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), score.data_ptr(),
                                     score_sq.data_ptr() if want_sq else None, ws.data_ptr(), nbytes, B, Sq, Skv, H,
                                     D, _dtype_code(q, where), int(bool(causal)), int(window), float(softcap),
                                     float(scale), _stream_ptr(dev))
  _lib.check(st, where)
  return (out, score, score_sq) if want_sq else (out, score)


def _attn_snapkv_impl(q, k, v, kernel_size, causal, scale):
  out, score = _attn_score_impl(q, k, v, False, causal, -1, 0.0, scale)
  pooled = torch.empty_like(score)
  dev = q.device
  with _on_device(dev):
    st = _lib.load().b200_avg_pool1d_f32(score.data_ptr(), pooled.data_ptr(), score.size(0) * score.size(1),
                                         score.size(2), int(kernel_size), _stream_ptr(dev))
  _lib.check(st, "attn_snapkv_fwd")
  return out, pooled


def _attn_corm_impl(q, k, v, causal, scale):
  where = "attn_corm_fwd"
  dev = _check_qkv(where, q, k, v)
  B, Sq, H, D = q.shape
  Skv, Hk = k.size(1), k.size(2)
  if scale is None or scale <= 0:
    scale = 1.0 / math.sqrt(D)
  out = torch.empty_like(q)
  score = torch.empty((B, Hk, Skv), dtype=torch.float32, device=dev)
  flags = torch.empty((B, Hk, Skv), dtype=torch.uint8, device=dev)
  if B == 0 or Sq == 0:   # no queries: `any` over an empty set
    flags.zero_()
    return out, flags.view(torch.bool)
  ws, nbytes = _workspace(dev, B, Sq, Skv, H)
  with _on_device(dev):
    if H != Hk:   # thresholds applied to the group-mean probabilities
      st = _lib.load().b200_attn_score_gqa(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                           score.data_ptr(), None, flags.data_ptr(), ws.data_ptr(), nbytes, B, Sq,
                                           Skv, H, Hk, D, _dtype_code(q, where), int(bool(causal)), 0, 0.0,
                                           float(scale), _stream_ptr(dev))
    else:
      st = _lib.load().b200_attn_corm(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), score.data_ptr(),
                                      flags.data_ptr(), ws.data_ptr(), nbytes, B, Sq, Skv, H, D,
                                      _dtype_code(q, where), int(bool(causal)), float(scale), _stream_ptr(dev))
  _lib.check(st, where)
  return out, flags.view(torch.bool)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
  """Philox4x32-10 (Salmon et al., SC'11) on int64 tensors that hold 32-bit words; k0, k1 are Python ints.
  Returns the four output words.  The same function as philox4x32_10 in csrc/attn_sweep.cuh."""
  m32 = 0xFFFFFFFF
  for _ in range(10):
    p0, p1 = c0 * 0xD2511F53, c2 * 0xCD9E8D57       # 64-bit products; int64 wrap-around keeps the bit pattern
    c0, c1, c2, c3 = ((p1 >> 32) & m32) ^ c1 ^ k0, p1 & m32, ((p0 >> 32) & m32) ^ c3 ^ k1, p0 & m32
    k0, k1 = (k0 + 0x9E3779B9) & m32, (k1 + 0xBB67AE85) & m32
  return c0, c1, c2, c3


def kf_noise(seed, batch, heads, q_len, kv_len, device="cpu"):
  """The exp_rand tensor float32 [batch, heads, q_len, kv_len] that attn_kf_fwd(..., exp_rand=None, seed=seed)
  generates inside its kernels: element (b, h, i, j) is word j & 3 of Philox4x32-10 at counter (j >> 2, i, b * heads +
  h, 0) under key (seed & 0xffffffff, seed >> 32), mapped to u = ((word >> 9) + 1/2) * 2^-23 and exp_rand = -ln(u)
  (so -ln(exp_rand) is Gumbel(0, 1) noise).  Plain torch integer arithmetic: runs on any device, so a CPU reference
  of the reference's KeyFormer module (kernels/kf.py:19-42) can be fed exactly the noise the kernels use."""
  dev = torch.device(device)
  nq = (kv_len + 3) // 4
  jq = torch.arange(nq, dtype=torch.int64, device=dev).view(1, 1, nq)
  i = torch.arange(q_len, dtype=torch.int64, device=dev).view(1, q_len, 1)
  bh = torch.arange(batch * heads, dtype=torch.int64, device=dev).view(batch * heads, 1, 1)
  shape = (batch * heads, q_len, nq)
  words = philox4x32_10(jq.expand(shape), i.expand(shape), bh.expand(shape), torch.zeros(shape, dtype=torch.int64, device=dev),
                        int(seed) & 0xFFFFFFFF, (int(seed) >> 32) & 0xFFFFFFFF)
  r = torch.stack(words, dim=-1).reshape(batch * heads, q_len, nq * 4)[:, :, :kv_len]
  u = ((r >> 9).double() + 0.5) * (1.0 / 8388608.0)
  return (-torch.log(u)).float().view(batch, heads, q_len, kv_len)


def kf_noise_fill(seed, batch, heads, q_len, kv_len, device):
  """kf_noise evaluated by the library's own fill kernel (b200_kf_noise_fill): same tensor, on the GPU."""
  dev = torch.device(device)
  out = torch.empty((batch, heads, q_len, kv_len), dtype=torch.float32, device=dev)
  with _on_device(dev):
    st = _lib.load().b200_kf_noise_fill(out.data_ptr(), int(seed) & 0xFFFFFFFFFFFFFFFF, batch, heads, q_len, kv_len,
                                        _stream_ptr(dev))
  _lib.check(st, "kf_noise_fill")
  return out


def _attn_kf_seeded_impl(q, k, v, seed, tau, causal, scale):
  where = "attn_kf_fwd"
  dev = _check_qkv(where, q, k, v)
  B, Sq, H, D = q.shape
  Skv, Hk = k.size(1), k.size(2)
  if scale is None or scale <= 0:
    scale = 1.0 / math.sqrt(D)
  out = torch.empty_like(q)
  score = torch.empty((B, Hk, Skv), dtype=torch.float32, device=dev)
  if B == 0 or Sq == 0:
    return out, score.zero_()
  ws, nbytes = _workspace(dev, B, Sq, Skv, H)
  with _on_device(dev):
    st = _lib.load().b200_attn_kf_score_seeded(q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                               int(seed) & 0xFFFFFFFFFFFFFFFF, out.data_ptr(), score.data_ptr(),
                                               ws.data_ptr(), nbytes, B, Sq, Skv, H, Hk, D, _dtype_code(q, where),
                                               int(bool(causal)), float(tau), float(scale), _stream_ptr(dev))
  _lib.check(st, where)
  return out, score


def _attn_kf_impl(q, k, v, exp_rand, tau, causal, scale):
  where = "attn_kf_fwd"
  dev = _check_qkv(where, q, k, v)
  B, Sq, H, D = q.shape
  Skv, Hk = k.size(1), k.size(2)
  _require_cuda(where, q, exp_rand)
  if exp_rand.dtype != torch.float32 or tuple(exp_rand.shape) != (B, H, Sq, Skv) or not exp_rand.is_contiguous():
    raise ValueError(f"{where}: exp_rand must be contiguous float32 [batch, heads, q_len, kv_len]")
  if scale is None or scale <= 0:
    scale = 1.0 / math.sqrt(D)
  out = torch.empty_like(q)
  score = torch.empty((B, Hk, Skv), dtype=torch.float32, device=dev)
  if B == 0 or Sq == 0:
    return out, score.zero_()
  ws, nbytes = _workspace(dev, B, Sq, Skv, H)
  with _on_device(dev):
    if H != Hk:   # score of a K/V head = mean over its query heads (figure/membound/attn.py:162-165)
      st = _lib.load().b200_attn_kf_score_gqa(q.data_ptr(), k.data_ptr(), v.data_ptr(), exp_rand.data_ptr(),
                                              out.data_ptr(), score.data_ptr(), ws.data_ptr(), nbytes, B, Sq, Skv, H,
                                              Hk, D, _dtype_code(q, where), int(bool(causal)), float(tau),
                                              float(scale), _stream_ptr(dev))
    else:
      st = _lib.load().b200_attn_kf_score(q.data_ptr(), k.data_ptr(), v.data_ptr(), exp_rand.data_ptr(),
                                          out.data_ptr(), score.data_ptr(), ws.data_ptr(), nbytes, B, Sq, Skv, H, D,
                                          _dtype_code(q, where), int(bool(causal)), float(tau), float(scale),
                                          _stream_ptr(dev))
  _lib.check(st, where)
  return out, score


# ----------------------------------------------------------------------------------------------
# torch custom ops (namespace b200attn) with fake kernels for tracing
# ----------------------------------------------------------------------------------------------
@torch.library.custom_op("b200attn::attn_fwd", mutates_args=())
def _op_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, window: int, softcap: float,
                 scale: float) -> torch.Tensor:
  return _attn_fwd_impl(q, k, v, causal, window, softcap, scale)


@_op_attn_fwd.register_fake
def _(q, k, v, causal, window, softcap, scale):
  return torch.empty_like(q)


@torch.library.custom_op("b200attn::attn_score_fwd", mutates_args=())
def _op_attn_score_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, window: int, softcap: float,
                       scale: float) -> tuple[torch.Tensor, torch.Tensor]:
  return _attn_score_impl(q, k, v, False, causal, window, softcap, scale)


@_op_attn_score_fwd.register_fake
def _(q, k, v, causal, window, softcap, scale):
  return torch.empty_like(q), q.new_empty((q.size(0), k.size(2), k.size(1)), dtype=torch.float32)


@torch.library.custom_op("b200attn::attn_score_sq_fwd", mutates_args=())
def _op_attn_score_sq_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, window: int,
                          softcap: float, scale: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
  return _attn_score_impl(q, k, v, True, causal, window, softcap, scale)


@_op_attn_score_sq_fwd.register_fake
def _(q, k, v, causal, window, softcap, scale):
  s = q.new_empty((q.size(0), k.size(2), k.size(1)), dtype=torch.float32)
  return torch.empty_like(q), s, torch.empty_like(s)


@torch.library.custom_op("b200attn::attn_kf_fwd", mutates_args=())
def _op_attn_kf_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, exp_rand: torch.Tensor, tau: float,
                    causal: bool, scale: float) -> tuple[torch.Tensor, torch.Tensor]:
  return _attn_kf_impl(q, k, v, exp_rand, tau, causal, scale)


@_op_attn_kf_fwd.register_fake
def _(q, k, v, exp_rand, tau, causal, scale):
  return torch.empty_like(q), q.new_empty((q.size(0), k.size(2), k.size(1)), dtype=torch.float32)


@torch.library.custom_op("b200attn::attn_kf_seeded_fwd", mutates_args=())
def _op_attn_kf_seeded_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seed: int, tau: float, causal: bool,
                           scale: float) -> tuple[torch.Tensor, torch.Tensor]:
  return _attn_kf_seeded_impl(q, k, v, seed, tau, causal, scale)


@_op_attn_kf_seeded_fwd.register_fake
def _(q, k, v, seed, tau, causal, scale):
  return torch.empty_like(q), q.new_empty((q.size(0), k.size(2), k.size(1)), dtype=torch.float32)


@torch.library.custom_op("b200attn::attn_snapkv_fwd", mutates_args=())
def _op_attn_snapkv_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel_size: int, causal: bool,
                        scale: float) -> tuple[torch.Tensor, torch.Tensor]:
  return _attn_snapkv_impl(q, k, v, kernel_size, causal, scale)


@_op_attn_snapkv_fwd.register_fake
def _(q, k, v, kernel_size, causal, scale):
  return torch.empty_like(q), q.new_empty((q.size(0), k.size(2), k.size(1)), dtype=torch.float32)


@torch.library.custom_op("b200attn::attn_corm_fwd", mutates_args=())
def _op_attn_corm_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool,
                      scale: float) -> tuple[torch.Tensor, torch.Tensor]:
  return _attn_corm_impl(q, k, v, causal, scale)


@_op_attn_corm_fwd.register_fake
def _(q, k, v, causal, scale):
  return torch.empty_like(q), q.new_empty((q.size(0), k.size(2), k.size(1)), dtype=torch.bool)


# ----------------------------------------------------------------------------------------------
# public functions
# ----------------------------------------------------------------------------------------------
def _tracing_graph():
  """True while torch.compile / export traces the caller: only then do the public functions go through the
  registered custom ops (which carry the fake kernels a tracer needs).  In eager mode they call the implementation
  directly -- the dispatcher round trip of a Python custom op costs ~17 us of host time per call, more than the
  kernel takes for a short sequence."""
  return torch.compiler.is_compiling()


@traced
def attn_fwd(q, k, v, causal=True, window=-1, softcap=0.0, scale=None):
  """softmax(mask(softcap(q k^T * scale))) v   (kernels/attn.py:18-34, kernels/gemma2.py:19-38)."""
  if not _tracing_graph():
    return _attn_fwd_impl(q, k, v, causal, window, softcap, scale)
  return _op_attn_fwd(q, k, v, bool(causal), int(window), float(softcap), float(scale or 0.0))


@traced
def attn_fwd_with_lse(q, k, v, causal=True, window=-1, softcap=0.0, scale=None):
  """attn_fwd plus the base-2 log-sum-exp of every row of scaled logits, float32 [B, H, Sq]."""
  return _attn_fwd_impl(q, k, v, causal, window, softcap, scale, want_lse=True)


@traced
def attn_score_fwd(q, k, v, want_sq=False, causal=True, window=-1, softcap=0.0, scale=None):
  """Attention output + per-key column sums of the fp32 probabilities (kernels/h2o.py:35-38);
  want_sq adds the column sums of the squared probabilities (kernels/roco.py:42-48)."""
  if not _tracing_graph():
    return _attn_score_impl(q, k, v, bool(want_sq), causal, window, softcap, scale)
  op = _op_attn_score_sq_fwd if want_sq else _op_attn_score_fwd
  return op(q, k, v, bool(causal), int(window), float(softcap), float(scale or 0.0))


@traced
def attn_kf_fwd(q, k, v, exp_rand=None, tau=1.5, causal=True, scale=None, seed=0):
  """Attention output + KeyFormer score: column sums of softmax((logits - log(exp_rand)) / tau)
  (kernels/kf.py:36-42).  exp_rand float32 [B, H, Sq, Skv] as the reference passes it -- or None: the kernels then
  generate the noise themselves from `seed` (the tensor kf_noise(seed, ...) describes), and nothing of size
  Sq x Skv is read or stored."""
  if not _tracing_graph():
    if exp_rand is None:
      return _attn_kf_seeded_impl(q, k, v, int(seed), float(tau), causal, scale)
    return _attn_kf_impl(q, k, v, exp_rand, float(tau), causal, scale)
  if exp_rand is None:
    return _op_attn_kf_seeded_fwd(q, k, v, int(seed), float(tau), bool(causal), float(scale or 0.0))
  return _op_attn_kf_fwd(q, k, v, exp_rand, float(tau), bool(causal), float(scale or 0.0))


@traced
def attn_snapkv_fwd(q, k, v, kernel_size=5, causal=True, scale=None):
  """Attention output + column sums average-pooled over a window of `kernel_size` keys, zero padded
  (kernels/snapkv.py:36-38)."""
  if not _tracing_graph():
    return _attn_snapkv_impl(q, k, v, int(kernel_size), causal, scale)
  return _op_attn_snapkv_fwd(q, k, v, int(kernel_size), bool(causal), float(scale or 0.0))


@traced
def attn_corm_fwd(q, k, v, causal=True, scale=None):
  """Attention output + bool [B, H, Skv]: does any query i attend to the key with probability >= 1 / (i + 1)
  (kernels/corm.py:35-37; the thresholds of Corm.prepare, kernels/corm.py:47-49, are evaluated in the kernel)."""
  if not _tracing_graph():
    return _attn_corm_impl(q, k, v, causal, scale)
  return _op_attn_corm_fwd(q, k, v, bool(causal), float(scale or 0.0))


@traced
def kv_evict_topk(score, k, v, budget, return_indices=False):
  """KV-cache eviction step of the reference's model glue (models/h2o.py:51-57, models/kf.py:54-60): per (batch,
  head) keep the `budget` keys with the largest score, in position order.
  score float32 [B, H, S]; k, v [B, S, H, D].  Returns kv_cache [B, 2, budget, H, D] (plane 0 keys, plane 1
  values) and, if asked, the selected positions int32 [B, H, budget]."""
  where = "kv_evict_topk"
  dev = _require_cuda(where, score, k, v)
  if score.dtype != torch.float32 or score.dim() != 3 or not score.is_contiguous():
    raise ValueError(f"{where}: score must be contiguous float32 [batch, heads, seq]")
  if k.dim() != 4 or k.shape != v.shape or k.dtype != v.dtype or not (k.is_contiguous() and v.is_contiguous()):
    raise ValueError(f"{where}: k, v must be contiguous [batch, seq, heads, head_dim] of one dtype")
  B, S, H, D = k.shape
  if tuple(score.shape) != (B, H, S):
    raise ValueError(f"{where}: score shape {tuple(score.shape)} does not match k {tuple(k.shape)}")
  kv_cache = torch.empty((B, 2, int(budget), H, D), dtype=k.dtype, device=dev)
  idx = torch.empty((B, H, int(budget)), dtype=torch.int32, device=dev) if return_indices else None
  with _on_device(dev):
    st = _lib.load().b200_kv_evict_topk(score.data_ptr(), k.data_ptr(), v.data_ptr(), kv_cache.data_ptr(),
                                        idx.data_ptr() if return_indices else None, B, S, H, D, int(budget),
                                        _dtype_code(k, where), _stream_ptr(dev))
  _lib.check(st, where)
  return (kv_cache, idx) if return_indices else kv_cache


@traced
def kv_evict_roco(score, score_sq, k, v, q_len, budget, recent, return_indices=False):
  """RoCo's KV-cache eviction (models/roco.py:52-66): keep the `recent` keys whose attention probabilities vary
  most over the queries (largest std, from the column sums of p and p^2) and, of the rest, the `budget` keys with
  the largest mean probability; position order.
  score, score_sq float32 [B, H, S] (from attn_score_fwd(want_sq=True)); k, v [B, S, H, D].  Returns kv_cache
  [B, 2, budget + recent, H, D] and, if asked, the selected positions int32 [B, H, budget + recent]."""
  where = "kv_evict_roco"
  dev = _require_cuda(where, score, score_sq, k, v)
  for name, t in (("score", score), ("score_sq", score_sq)):
    if t.dtype != torch.float32 or t.dim() != 3 or not t.is_contiguous():
      raise ValueError(f"{where}: {name} must be contiguous float32 [batch, heads, seq]")
  if k.dim() != 4 or k.shape != v.shape or k.dtype != v.dtype or not (k.is_contiguous() and v.is_contiguous()):
    raise ValueError(f"{where}: k, v must be contiguous [batch, seq, heads, head_dim] of one dtype")
  B, S, H, D = k.shape
  if tuple(score.shape) != (B, H, S) or score_sq.shape != score.shape:
    raise ValueError(f"{where}: score shapes {tuple(score.shape)}, {tuple(score_sq.shape)} do not match k {tuple(k.shape)}")
  keep = int(budget) + int(recent)
  kv_cache = torch.empty((B, 2, keep, H, D), dtype=k.dtype, device=dev)
  idx = torch.empty((B, H, keep), dtype=torch.int32, device=dev) if return_indices else None
  with _on_device(dev):
    st = _lib.load().b200_kv_evict_roco(score.data_ptr(), score_sq.data_ptr(), k.data_ptr(), v.data_ptr(),
                                        kv_cache.data_ptr(), idx.data_ptr() if return_indices else None, B, S, H, D,
                                        int(q_len), int(budget), int(recent), _dtype_code(k, where), _stream_ptr(dev))
  _lib.check(st, where)
  return (kv_cache, idx) if return_indices else kv_cache
