"""Builds the REFERENCE's own native ops (csrc/norm.cu, activation.cu, pos_encoding.cu, ffi.cpp) for sm_100a
straight from the reference tree into oracle/_ref/_csrc_ref.so -- test infrastructure only.

The GPU tests use it, when present, to compare this package's RMSNorm / SiLU-gate / RoPE kernels with the
reference kernels themselves on the same device.  No reference source is copied: nvcc reads the files where
they lie.  Flags follow the reference's setup.py:20-38 (-O3 --use_fast_math -std=c++17, half/bf16 operators
enabled); only the architecture differs (the reference builds for 8.0/8.6/9.0).

    python oracle/build_ref.py [<reference tree>]      (default: $B200_REFERENCE_ROOT)
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "_csrc_ref.so")


DEFAULT_REF_ROOT = os.environ.get("B200_REFERENCE_ROOT", os.path.join(os.sep, "root", "reference"))


def build(ref_root=DEFAULT_REF_ROOT, force=False):
  srcs = [os.path.join(ref_root, "csrc", f) for f in ("norm.cu", "activation.cu", "pos_encoding.cu", "ffi.cpp")]
  if not all(os.path.exists(s) for s in srcs):
    return None
  if os.path.exists(OUT) and not force:
    return OUT
  import torch
  from torch.utils import cpp_extension
  os.makedirs(OUT_DIR, exist_ok=True)
  inc = cpp_extension.include_paths("cuda") + [sysconfig.get_paths()["include"]]
  torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
  flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math", "-std=c++17",
           "-Xcompiler", "-fPIC", "-DTORCH_EXTENSION_NAME=_csrc_ref", "-DFLASHINFER_ENABLE_BF16",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)),
           "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
           "-U__CUDA_NO_HALF2_OPERATORS__", "-x", "cu"]
  for i in inc:
    flags += ["-I", i]
  # one nvcc per source in parallel (the torch headers dominate the compile time), then one link step
  objs, procs = [], []
  for src in srcs:
    obj = os.path.join(OUT_DIR, os.path.basename(src) + ".o")
    objs.append(obj)
    procs.append(subprocess.Popen(["nvcc", "-c"] + flags + [src, "-o", obj], stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True))
  for pr in procs:
    log, _ = pr.communicate()
    if pr.returncode != 0:
      sys.stderr.write(log[-4000:])
      return None
  link = ["nvcc", "-shared", "-o", OUT] + objs + ["-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu",
                                                   "-ltorch_cuda", "-ltorch", "-ltorch_python", "-Xlinker",
                                                   "-rpath," + torch_lib]
  res = subprocess.run(link, capture_output=True, text=True)
  for obj in objs:
    if os.path.exists(obj):
      os.remove(obj)
  if res.returncode != 0:
    sys.stderr.write(res.stdout[-4000:] + res.stderr[-4000:])
    return None
  return OUT


if __name__ == "__main__":
  print(build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REF_ROOT, force=True))
