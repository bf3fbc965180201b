"""Host-side mirror of the reference's native-op module (csrc/ffi.cpp:4-8, csrc/op.h:2-6).

Same function names, argument order and in-place contracts:
  rms_norm(out, input, weight, epsilon)
  silu_and_mul(out, input)
  rotary_embedding_online(positions, query, key, head_size, rope_theta)
plus the two ops the reference has in source but does not export or lacks:
  fused_add_rms_norm(input, residual, weight, epsilon)     (csrc/norm.cu:100-113)
  gelu_tanh_and_mul(out, input)                            (GeGLU sibling of silu_and_mul)

All ops enqueue on the current CUDA stream of the tensors' device and never synchronise,
like the reference (csrc/norm.cu:94).  Unlike the reference they validate their arguments and
raise instead of launching on bad input.
"""
import torch

from .tracing import traced

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def _dtype_code(t, where):
  try:
    return _DTYPES[t.dtype]
  except KeyError:
    raise TypeError(f"{where}: unsupported dtype {t.dtype}") from None


def _require_cuda(where, *tensors):
  dev = tensors[0].device
  for t in tensors:
    if not t.is_cuda:
      raise RuntimeError(f"{where}: expected CUDA tensors, got {t.device} (there is no CPU path)")
    if t.device != dev:
      raise RuntimeError(f"{where}: tensors on different devices ({t.device} vs {dev})")
  return dev


def _stream_ptr(dev):
  return torch.cuda.current_stream(dev).cuda_stream


class _on_device:
  """`with _on_device(dev):` makes `dev` the current CUDA device for the enclosed library call.  When it already is
  (the usual case: one process per GPU) nothing is switched -- torch.cuda.device costs several microseconds per
  entry, which is as much host time as a whole launch."""
  __slots__ = ("dev", "ctx")

  def __init__(self, dev):
    self.dev = dev
    self.ctx = None

  def __enter__(self):
    idx = self.dev.index
    if idx is not None and idx != torch.cuda.current_device():
      self.ctx = torch.cuda.device(self.dev)
      self.ctx.__enter__()
    return self

  def __exit__(self, *exc):
    if self.ctx is not None:
      return self.ctx.__exit__(*exc)
    return False


@traced
def rms_norm(out, input, weight, epsilon):
  """out = T(input * rsqrt(mean(input^2, -1) + epsilon)) * weight   (csrc/norm.cu:34-56)."""
  where = "rms_norm"
  dev = _require_cuda(where, out, input, weight)
  hidden = input.size(-1)
  if out.shape != input.shape or weight.numel() != hidden:
    raise ValueError(f"{where}: shape mismatch out={tuple(out.shape)} input={tuple(input.shape)} weight={tuple(weight.shape)}")
  if out.dtype != input.dtype or weight.dtype != input.dtype:
    raise TypeError(f"{where}: dtype mismatch")
  if not (out.is_contiguous() and input.is_contiguous() and weight.is_contiguous()):
    raise ValueError(f"{where}: tensors must be contiguous")
  tokens = input.numel() // hidden if hidden else 0
  with _on_device(dev):
    st = _lib.load().b200_rms_norm(out.data_ptr(), input.data_ptr(), weight.data_ptr(), float(epsilon), tokens,
                                   hidden, _dtype_code(input, where), _stream_ptr(dev))
  _lib.check(st, where)


@traced
def fused_add_rms_norm(input, residual, weight, epsilon):
  """residual += input; input = rms_norm(residual) * weight, both in place (csrc/norm.cu:59-83)."""
  where = "fused_add_rms_norm"
  dev = _require_cuda(where, input, residual, weight)
  hidden = input.size(-1)
  if residual.shape != input.shape or weight.numel() != hidden:
    raise ValueError(f"{where}: shape mismatch")
  if residual.dtype != input.dtype or weight.dtype != input.dtype:
    raise TypeError(f"{where}: dtype mismatch")
  if not (residual.is_contiguous() and input.is_contiguous() and weight.is_contiguous()):
    raise ValueError(f"{where}: tensors must be contiguous")
  tokens = input.numel() // hidden if hidden else 0
  with _on_device(dev):
    st = _lib.load().b200_fused_add_rms_norm(input.data_ptr(), residual.data_ptr(), weight.data_ptr(),
                                             float(epsilon), tokens, hidden, _dtype_code(input, where),
                                             _stream_ptr(dev))
  _lib.check(st, where)


def _act_and_mul(fn_name, out, input):
  dev = _require_cuda(fn_name, out, input)
  d = input.size(-1) // 2
  if input.size(-1) != 2 * d or out.size(-1) != d or out.shape[:-1] != input.shape[:-1]:
    raise ValueError(f"{fn_name}: expected input [..., 2*d] and out [..., d], got {tuple(input.shape)} / {tuple(out.shape)}")
  if out.dtype != input.dtype:
    raise TypeError(f"{fn_name}: dtype mismatch")
  if not (out.is_contiguous() and input.is_contiguous()):
    raise ValueError(f"{fn_name}: tensors must be contiguous")
  tokens = input.numel() // (2 * d) if d else 0
  with _on_device(dev):
    st = getattr(_lib.load(), "b200_" + fn_name)(out.data_ptr(), input.data_ptr(), tokens, d,
                                                 _dtype_code(input, fn_name), _stream_ptr(dev))
  _lib.check(st, fn_name)


@traced
def silu_and_mul(out, input):
  """out[..., i] = T(silu(input[..., i])) * input[..., d + i]   (csrc/activation.cu:6-34)."""
  _act_and_mul("silu_and_mul", out, input)


@traced
def gelu_tanh_and_mul(out, input):
  """out[..., i] = T(gelu_tanh(input[..., i])) * input[..., d + i] (GeGLU gate)."""
  _act_and_mul("gelu_tanh_and_mul", out, input)


@traced
def rotary_embedding_online(positions, query, key, head_size, rope_theta):
  """In-place NeoX rotary embedding of query [T, H*D] and key [T, Hk*D] (csrc/pos_encoding.cu:64-113,180-199).

  positions: int32 [T].  The reference asserts head_size == 128; 64 and 256 are accepted too.
  """
  where = "rotary_embedding_online"
  dev = _require_cuda(where, positions, query, key)
  if positions.dtype != torch.int32:
    raise TypeError(f"{where}: positions must be int32")
  if query.dtype != key.dtype:
    raise TypeError(f"{where}: dtype mismatch")
  if query.dim() < 2 or key.dim() < 2 or query.stride(-1) != 1 or key.stride(-1) != 1:
    raise ValueError(f"{where}: query/key must be [..., tokens, heads*head_size] with unit inner stride")
  if query.size(-1) % head_size or key.size(-1) % head_size:
    raise ValueError(f"{where}: last dimension is not a multiple of head_size")
  tokens = query.numel() // query.size(-1)
  if key.numel() // key.size(-1) != tokens or positions.numel() != tokens or not positions.is_contiguous():
    raise ValueError(f"{where}: token count mismatch")
  # rows must be uniformly strided (the reference reads stride(-2) only, csrc/pos_encoding.cu:189-190)
  for name, t in (("query", query), ("key", key)):
    flat = t.reshape(-1, t.size(-1)) if t.dim() > 2 else t
    if flat.data_ptr() != t.data_ptr() or (flat.size(0) > 1 and flat.stride(0) != t.stride(-2)):
      raise ValueError(f"{where}: {name} rows are not uniformly strided")
  with _on_device(dev):
    st = _lib.load().b200_rotary_embedding_online(
        positions.data_ptr(), query.data_ptr(), key.data_ptr(), tokens, query.size(-1) // head_size,
        key.size(-1) // head_size, int(head_size), query.stride(-2), key.stride(-2), float(rope_theta),
        _dtype_code(query, where), _stream_ptr(dev))
  _lib.check(st, where)
