"""The C-ABI library loads, exports every symbol that include/b200attn.h declares, and rejects bad
arguments with status codes before touching the GPU.  Runs without a CUDA device."""
import ctypes
import os
import re

from deepgengraph_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
  text = open(os.path.join(ROOT, "include", "b200attn.h")).read()
  text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
  return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
  lib = _lib.load()
  names = header_functions()
  assert len(names) >= 12
  for n in names:
    assert hasattr(lib, n), f"{n} declared in include/b200attn.h but not exported"
  # and the ctypes table binds exactly the declared set
  assert sorted(_lib.SIGNATURES) == names


def test_status_strings_and_version():
  lib = _lib.load()
  assert lib.b200_abi_version() == 2
  assert lib.b200_status_string(0) == b"ok"
  assert b"unsupported" in lib.b200_status_string(4)


def test_bad_arguments_are_rejected_without_a_gpu():
  lib = _lib.load()
  buf = (ctypes.c_char * 4096)()
  p = ctypes.addressof(buf)
  p = (p + 255) // 256 * 256
  assert lib.b200_rms_norm(None, p, p, 1e-6, 4, 128, _lib.BF16, None) == 1
  assert lib.b200_rms_norm(p, p, p, 1e-6, 4, 128, 99, None) == 2
  assert lib.b200_rms_norm(p, p, p, 1e-6, 0, 128, _lib.BF16, None) == 0      # empty input: nothing to do
  assert lib.b200_silu_and_mul(p, p, 4, 0, _lib.BF16, None) == 1
  assert lib.b200_rotary_embedding_online(p, p, p, 4, 2, 2, 128, 128, 256, 1e4, _lib.BF16, None) == 1  # stride < row
  # attention: dtype / head_dim / shape checks come before any CUDA call
  args = lambda **kw: [kw.get(k, d) for k, d in (("batch", 1), ("q_len", 128), ("kv_len", 128), ("heads", 2),
                                                  ("kv_heads", 2), ("head_dim", 128), ("dtype", _lib.BF16),
                                                  ("causal", 1), ("window", 0))]
  call = lambda **kw: lib.b200_attn_fwd(p, p, p, p, None, *args(**kw), 0.0, 0.088, None)
  assert call(dtype=_lib.F32) == 2
  assert call(head_dim=96) == 4
  assert call(q_len=256, kv_len=128) == 4      # queries without any visible key
  assert call(heads=3, kv_heads=2) == 1
  assert call(causal=0, window=64) == 4
  assert lib.b200_attn_fwd(None, p, p, p, None, *args(), 0.0, 0.088, None) == 1
  assert lib.b200_attn_fwd(p + 2, p, p, p, None, *args(), 0.0, 0.088, None) == 3
  # score entry points: workspace checks
  need = lib.b200_attn_score_workspace_bytes(1, 128, 128, 2)
  assert need > 0 and need % 256 == 0
  assert lib.b200_attn_score(p, p, p, p, p, None, None, 0, 1, 128, 128, 2, 128, _lib.BF16, 1, 0, 0.0, 0.088, None) == 5
  assert lib.b200_attn_score(p, p, p, p, p, None, p, need - 1, 1, 128, 128, 2, 128, _lib.BF16, 1, 0, 0.0, 0.088, None) == 5
  assert lib.b200_attn_kf_score(p, p, p, p, p, p, p, need, 1, 128, 128, 2, 256, _lib.BF16, 1, 1.0, 0.088, None) == 4


def test_tracing_wrapper_is_transparent_when_off():
  from deepgengraph_b200 import attention, native_ops, tracing
  assert attention.attn_fwd.__name__ == "attn_fwd" and native_ops.rms_norm.__name__ == "rms_norm"
  calls = []

  @tracing.traced
  def probe(x, y=2):
    calls.append((x, y))
    return x + y

  tracing.enable(False)
  assert probe(1, y=3) == 4 and calls == [(1, 3)]
