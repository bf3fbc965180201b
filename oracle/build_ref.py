"""Builds the REFERENCE's own native ops (csrc/norm.cu, activation.cu, pos_encoding.cu, ffi.cpp) for sm_100a
straight from the reference tree into oracle/_ref/ -- test infrastructure only.

  oracle/_ref/_csrc_ref.so        the reference's module as its ffi.cpp defines it (rms_norm, silu_and_mul,
                                  rotary_embedding_online)
  oracle/_ref/_csrc_ref_extra.so  the reference's fused_add_rms_norm (csrc/norm.cu:59-83,100-113), which ffi.cpp does
                                  not register: norm.cu compiled again next to oracle/ref_extra_binding.cpp

The GPU tests use them, when present, to compare this package's RMSNorm / SiLU-gate / RoPE kernels with the
reference kernels themselves on the same device.  No reference source is copied: nvcc reads the files where
they lie.  Flags follow the reference's setup.py:20-38 (-O3 --use_fast_math -std=c++17, half/bf16 operators
enabled); only the architecture differs (the reference builds for 8.0/8.6/9.0).

    python oracle/build_ref.py [<reference tree>]    (default: $B200_REFERENCE_ROOT, else ../reference beside the repository)
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "_csrc_ref.so")
OUT_EXTRA = os.path.join(OUT_DIR, "_csrc_ref_extra.so")
EXTRA_BINDING = os.path.join(HERE, "ref_extra_binding.cpp")


def reference_root():
  """The reference tree: $B200_REFERENCE_ROOT, else a directory named `reference` beside this repository; None when
  neither holds a csrc/ folder."""
  repo = os.path.dirname(HERE)
  for root in (os.environ.get("B200_REFERENCE_ROOT"), os.path.join(os.path.dirname(repo), "reference")):
    if root and os.path.isdir(os.path.join(root, "csrc")):
      return root
  return None


def _flags(module_name):
  import torch
  from torch.utils import cpp_extension
  inc = cpp_extension.include_paths("cuda") + [sysconfig.get_paths()["include"]]
  flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math", "-std=c++17",
           "-Xcompiler", "-fPIC", "-DTORCH_EXTENSION_NAME=" + module_name, "-DFLASHINFER_ENABLE_BF16",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)),
           "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
           "-U__CUDA_NO_HALF2_OPERATORS__", "-x", "cu"]
  for i in inc:
    flags += ["-I", i]
  return flags


def _compile_and_link(srcs, out, module_name):
  """One nvcc per source in parallel (the torch headers dominate the compile time), then one link step."""
  import torch
  torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
  flags = _flags(module_name)
  objs, procs = [], []
  for src in srcs:
    obj = os.path.join(OUT_DIR, module_name + "." + os.path.basename(src) + ".o")
    objs.append(obj)
    procs.append(subprocess.Popen(["nvcc", "-c"] + flags + [src, "-o", obj], stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True))
  ok = True
  for pr in procs:
    log, _ = pr.communicate()
    if pr.returncode != 0:
      sys.stderr.write(log[-4000:])
      ok = False
  if ok:
    link = ["nvcc", "-shared", "-o", out] + objs + ["-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu",
                                                     "-ltorch_cuda", "-ltorch", "-ltorch_python", "-Xlinker",
                                                     "-rpath," + torch_lib]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
      sys.stderr.write(res.stdout[-4000:] + res.stderr[-4000:])
      ok = False
  for obj in objs:
    if os.path.exists(obj):
      os.remove(obj)
  return out if ok else None


def build(ref_root, force=False):
  """Builds both libraries from the reference tree at `ref_root`.  Returns the path of _csrc_ref.so, or None
  when the tree is absent or a compile fails."""
  if not ref_root:
    return None
  csrc = os.path.join(ref_root, "csrc")
  srcs = [os.path.join(csrc, f) for f in ("norm.cu", "activation.cu", "pos_encoding.cu", "ffi.cpp")]
  if not all(os.path.exists(s) for s in srcs):
    return None
  os.makedirs(OUT_DIR, exist_ok=True)
  main = OUT
  if force or not os.path.exists(OUT):
    main = _compile_and_link(srcs, OUT, "_csrc_ref")
  if force or not os.path.exists(OUT_EXTRA):
    _compile_and_link([os.path.join(csrc, "norm.cu"), EXTRA_BINDING], OUT_EXTRA, "_csrc_ref_extra")
  return main


if __name__ == "__main__":
  root = sys.argv[1] if len(sys.argv) > 1 else reference_root()
  if not root:
    sys.exit("no reference tree: pass its path, or set B200_REFERENCE_ROOT")
  print(build(root, force=True))
