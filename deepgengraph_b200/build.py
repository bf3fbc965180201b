"""Builds the native library in-tree: deepgengraph_b200/csrc/libb200attn.so (sm_100a only).

The library is one translation unit (csrc/b200attn.cu) compiled with nvcc; it links only the
CUDA runtime (the driver's tensor-map encoder is looked up at run time), so it can be loaded
with ctypes from any host language.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(CSRC, "libb200attn.so")
SOURCES = ["b200attn.cu"]
DEPS = ["b200attn.cu", "common.cuh", "elementwise.cuh", "attn_fwd.cuh", "attn_fwd_persist.cuh", "attn_sweep.cuh", "kv_evict.cuh",
        os.path.join("..", "..", "include", "b200attn.h")]


def _nvcc():
  for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
    if cand and os.path.exists(cand):
      return cand
  raise RuntimeError("nvcc not found (set NVCC or install the CUDA toolkit)")


def needs_build():
  if not os.path.exists(LIB):
    return True
  t = os.path.getmtime(LIB)
  return any(os.path.getmtime(os.path.join(CSRC, d)) > t for d in DEPS)


def build(force=False, verbose=False):
  """Compile the library if it is missing or older than its sources. Returns its path."""
  if not force and not needs_build():
    return LIB
  cmd = [
      _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
      "-shared", "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v" if verbose else "-O3",
      "-o", LIB + ".tmp",
  ] + [os.path.join(CSRC, s) for s in SOURCES] + ["-lcudart"]
  res = subprocess.run(cmd, capture_output=True, text=True)
  if res.returncode != 0:
    sys.stderr.write(res.stdout + res.stderr)
    raise RuntimeError("nvcc failed building libb200attn.so")
  if verbose:
    sys.stderr.write(res.stdout + res.stderr)
  os.replace(LIB + ".tmp", LIB)
  return LIB


if __name__ == "__main__":
  print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
