"""KERNEL_ZOO-compatible core modules (reference: deepgengraph_exp/cases/kernels/__init__.py:10-18).

Each class keeps the reference's constructor arguments, its `prepare(batch_size, q_len, kv_len, dtype,
device)` input factory (same distributions, same names, same `{'input': ..., 'output': [...]}` record) and
its forward signature and output order -- but `forward` runs the fused sm_100a kernels instead of
materialising the [B, H, S, S] score matrix.  Inputs and outputs are BSHD like the reference's.

Extensions over the reference (which asserts group_size == 1 and has no window): Attn and Gemma2 accept
kv_head_num < head_num (grouped-query attention), head_dim 256 and a sliding `window`.
"""
from collections import OrderedDict

import torch
import torch.nn as nn

from . import attention as _att


def _default_device():
  return torch.device("cuda", torch.cuda.current_device())


def check_corm_mask(corm_mask, q_len, kv_len):
  """The Corm kernel evaluates the thresholds of Corm.prepare (row i = 1 / (i + 1), kernels/corm.py:47-49) itself.
  The reference compares against whatever [q_len, kv_len] tensor the caller passes (kernels/corm.py:35-37), so a
  mask with other values cannot be honoured: it is refused instead of being ignored."""
  if corm_mask is None:
    return
  tag = (corm_mask.data_ptr(), corm_mask._version, tuple(corm_mask.shape), q_len, kv_len)
  if tag == _checked_corm_mask[0]:     # the same tensor, unmodified since it was checked: no second device round trip
    return
  if tuple(corm_mask.shape) != (q_len, kv_len):
    raise NotImplementedError(f"corm_mask must be [q_len, kv_len] = [{q_len}, {kv_len}], got {tuple(corm_mask.shape)}")
  want = 1.0 / torch.arange(1, q_len + 1, dtype=torch.float32, device=corm_mask.device)
  # row i is constant: its first and last columns and one full diagonal sample pin the whole tensor cheaply
  cols = corm_mask[:, [0, kv_len - 1]].float()
  diag = corm_mask[torch.arange(q_len, device=corm_mask.device), torch.arange(q_len, device=corm_mask.device) % kv_len].float()
  if not (torch.equal(cols[:, 0], want) and torch.equal(cols[:, 1], want) and torch.equal(diag, want)):
    raise NotImplementedError("corm_mask differs from the thresholds 1 / (i + 1) that the fused Corm kernel evaluates")
  _checked_corm_mask[0] = tag


_checked_corm_mask = [None]


class _CoreModule(nn.Module):
  def __init__(self, kv_head_num=32, head_num=32, head_dim=128):
    super().__init__()
    self.kv_head_num = kv_head_num
    self.head_num = head_num
    self.head_dim = head_dim
    self.hidden_size = head_num * head_dim
    self.kv_hidden_size = kv_head_num * head_dim
    assert head_num % kv_head_num == 0
    self.group_size = head_num // kv_head_num

  def _qkv(self, batch_size, q_len, kv_len, dtype, device, gen):
    device = device if device is not None else _default_device()
    q = gen(batch_size, q_len, self.head_num, self.head_dim, dtype=dtype, device=device)
    k = gen(batch_size, kv_len, self.kv_head_num, self.head_dim, dtype=dtype, device=device)
    v = gen(batch_size, kv_len, self.kv_head_num, self.head_dim, dtype=dtype, device=device)
    return q, k, v, device


class Attn(_CoreModule):
  """Causal attention (kernels/attn.py:18-34)."""

  def __init__(self, kv_head_num=32, head_num=32, head_dim=128, window=-1):
    super().__init__(kv_head_num, head_num, head_dim)
    self.window = window

  def forward(self, q, k, v):
    return _att.attn_fwd(q, k, v, causal=True, window=self.window)

  def prepare(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None):
    # the reference draws Attn's inputs from U[0, 1) (kernels/attn.py:38-40), every other module from N(0, 1)
    q, k, v, _ = self._qkv(batch_size, q_len, kv_len, dtype, device, torch.rand)
    return {'input': OrderedDict(q=q, k=k, v=v), 'output': ['out']}


class Gemma2(_CoreModule):
  """Causal attention with tanh logit soft-capping (kernels/gemma2.py:19-38)."""

  def __init__(self, logit_softcapping=50.0, kv_head_num=32, head_num=32, head_dim=128, window=-1):
    super().__init__(kv_head_num, head_num, head_dim)
    self.logit_softcapping = logit_softcapping
    self.window = window

  def forward(self, q, k, v):
    return _att.attn_fwd(q, k, v, causal=True, window=self.window, softcap=self.logit_softcapping)

  def prepare(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None):
    q, k, v, _ = self._qkv(batch_size, q_len, kv_len, dtype, device, torch.randn)
    return {'input': OrderedDict(q=q, k=k, v=v), 'output': ['out']}


class H2O(_CoreModule):
  """Attention + accumulated attention score per key (kernels/h2o.py:18-38)."""

  def __init__(self, kv_head_num=32, head_num=32, head_dim=128):
    super().__init__(kv_head_num, head_num, head_dim)
    assert self.group_size == 1

  def forward(self, q, k, v):
    return _att.attn_score_fwd(q, k, v, want_sq=False, causal=True)

  def prepare(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None):
    q, k, v, _ = self._qkv(batch_size, q_len, kv_len, dtype, device, torch.randn)
    return {'input': OrderedDict(q=q, k=k, v=v), 'output': ['out', 'h2o_score']}


class RoCo(_CoreModule):
  """Attention + per-key sums of the probabilities and of their squares (kernels/roco.py:18-48)."""

  def __init__(self, kv_head_num=32, head_num=32, head_dim=128):
    super().__init__(kv_head_num, head_num, head_dim)
    assert self.group_size == 1

  def forward(self, q, k, v):
    return _att.attn_score_fwd(q, k, v, want_sq=True, causal=True)

  def prepare(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None):
    q, k, v, _ = self._qkv(batch_size, q_len, kv_len, dtype, device, torch.randn)
    return {'input': OrderedDict(q=q, k=k, v=v), 'output': ['out', 'roco_score', 'roco_sq_score']}


class KeyFormer(_CoreModule):
  """Attention + column sums of a second softmax over logits perturbed by -log(exp_rand) at temperature
  tau (kernels/kf.py:19-42)."""

  def __init__(self, tau=1.5, kv_head_num=32, head_num=32, head_dim=128):
    super().__init__(kv_head_num, head_num, head_dim)
    self.tau = tau
    assert self.group_size == 1

  def forward(self, q, k, v, exp_rand):
    return _att.attn_kf_fwd(q, k, v, exp_rand, tau=self.tau, causal=True)

  def prepare(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None, gumbel=False):
    q, k, v, device = self._qkv(batch_size, q_len, kv_len, dtype, device, torch.randn)
    shape = (batch_size, self.head_num, q_len, kv_len)
    if gumbel:
      # exp_rand = -log(U), U ~ U(0, 1): then -log(exp_rand) is exactly Gumbel(0, 1) noise
      exp_rand = -torch.log(torch.rand(shape, dtype=torch.float32, device=device).clamp_min_(1e-10))
    else:
      exp_rand = 1 + torch.randn(shape, dtype=torch.float32, device=device).abs()   # kernels/kf.py:48
    return {'input': OrderedDict(q=q, k=k, v=v, exp_rand=exp_rand), 'output': ['out', 'kf_score']}


class SnapKV(_CoreModule):
  """Attention + column sums smoothed by a 1-D average pool over the keys (kernels/snapkv.py:18-38)."""

  def __init__(self, kernel_size=5, kv_head_num=32, head_num=32, head_dim=128):
    super().__init__(kv_head_num, head_num, head_dim)
    self.kernel_size = kernel_size
    assert self.group_size == 1

  def forward(self, q, k, v):
    return _att.attn_snapkv_fwd(q, k, v, kernel_size=self.kernel_size, causal=True)

  def prepare(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None):
    q, k, v, _ = self._qkv(batch_size, q_len, kv_len, dtype, device, torch.randn)
    return {'input': OrderedDict(q=q, k=k, v=v), 'output': ['out', 'snapkv_score']}


class Corm(_CoreModule):
  """Attention + per-key flag: some query i attends to the key with probability >= 1 / (i + 1)
  (kernels/corm.py:18-37).  `corm_mask` keeps the reference's signature: it must be the tensor Corm.prepare
  builds (row i filled with 1 / (i + 1), kernels/corm.py:47-49); the kernel evaluates those thresholds itself."""

  def __init__(self, kv_head_num=32, head_num=32, head_dim=128):
    super().__init__(kv_head_num, head_num, head_dim)
    assert self.group_size == 1

  def forward(self, q, k, v, corm_mask=None):
    check_corm_mask(corm_mask, q.shape[1], k.shape[1])
    return _att.attn_corm_fwd(q, k, v, causal=True)

  def prepare(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None):
    q, k, v, device = self._qkv(batch_size, q_len, kv_len, dtype, device, torch.randn)
    rows = 1.0 / torch.arange(1, q_len + 1, dtype=torch.float32, device=device)
    corm_mask = rows[:, None].expand(q_len, kv_len).contiguous()
    return {'input': OrderedDict(q=q, k=k, v=v, corm_mask=corm_mask), 'output': ['out', 'corm_score']}


KERNEL_ZOO = {
    'attn': Attn,
    'corm': Corm,
    'gemma2': Gemma2,
    'h2o': H2O,
    'kf': KeyFormer,
    'roco': RoCo,
    'snapkv': SnapKV,
}
