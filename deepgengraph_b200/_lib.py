"""ctypes binding of libb200attn.so (the C ABI declared in include/b200attn.h).

The library is built in-tree by deepgengraph_b200/build.py.  There is no fallback: if the
shared object is missing and cannot be built, importing the ops raises.
"""
import ctypes
import os

from . import build as _build

_LIB = None

F32, F16, BF16 = 0, 1, 2

STATUS_NAMES = {
    0: "ok", 1: "bad argument", 2: "unsupported dtype", 3: "misaligned pointer or stride",
    4: "unsupported shape", 5: "workspace missing or too small", 6: "CUDA call failed",
    7: "device-side wait expired",
}

_vp, _i, _i64, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

# name -> (restype, argtypes); mirrors include/b200attn.h one to one
SIGNATURES = {
    "b200_status_string": (ctypes.c_char_p, [_i]),
    "b200_last_cuda_error": (_i, []),
    "b200_abi_version": (_i, []),
    "b200_device_status": (_i, [ctypes.POINTER(_i)]),
    "b200_selftest_bounded_wait": (_i, [_i, _vp, _vp]),
    "b200_rms_norm": (_i, [_vp, _vp, _vp, _f, _i64, _i, _i, _vp]),
    "b200_fused_add_rms_norm": (_i, [_vp, _vp, _vp, _f, _i64, _i, _i, _vp]),
    "b200_silu_and_mul": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "b200_gelu_tanh_and_mul": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "b200_rotary_embedding_online": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _i64, _i64, _f, _i, _vp]),
    "b200_attn_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp]),
    "b200_attn_fwd_strided": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64,
                                   _i, _i, _f, _f, _vp]),
    "b200_attn_score_workspace_bytes": (_i64, [_i, _i, _i, _i]),
    "b200_attn_score": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp]),
    "b200_attn_score_gqa": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f,
                                 _vp]),
    "b200_attn_kf_score_seeded": (_i, [_vp, _vp, _vp, ctypes.c_uint64, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, _i, _i, _i, _f,
                                       _f, _vp]),
    "b200_kf_noise_fill": (_i, [_vp, ctypes.c_uint64, _i, _i, _i, _i, _vp]),
    "b200_attn_kf_score_gqa": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp]),
    "b200_attn_score_static": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp]),
    "b200_attn_corm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "b200_avg_pool1d_f32": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "b200_kv_evict_topk": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "b200_kv_evict_roco": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "b200_attn_kf_score": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp]),
}


def lib_path():
  return _build.LIB


def load():
  """Loads (building first if needed) the native library and declares its signatures."""
  global _LIB
  if _LIB is not None:
    return _LIB
  path = _build.LIB
  if _build.needs_build():
    try:
      _build.build()
    except Exception as e:  # a present library is still usable where no compiler is installed
      if not os.path.exists(path):
        raise RuntimeError(f"libb200attn.so is missing and could not be built: {e}") from e
  lib = ctypes.CDLL(path)
  for name, (res, args) in SIGNATURES.items():
    fn = getattr(lib, name)  # AttributeError here = header / library mismatch
    fn.restype = res
    fn.argtypes = args
  _LIB = lib
  return lib


class B200Error(RuntimeError):
  def __init__(self, status, where):
    self.status = status
    lib = load()
    detail = ""
    if status == 6:
      detail = f" (cudaError {lib.b200_last_cuda_error()})"
    super().__init__(f"{where}: {STATUS_NAMES.get(status, status)}{detail}")


def check(status, where):
  if status != 0:
    raise B200Error(status, where)
