"""Generates tests/golden/*.npz by RUNNING THE REFERENCE's own PyTorch modules
(deepgengraph_exp/cases/kernels/*.py) on the seeded inputs of cases.py, in fp32 on CPU.

Needs the reference tree:
    python tests/golden/make_golden.py [<reference tree> [case names ...]]   (default tree: as oracle/build_ref.py finds it)
The tests only read the committed .npz files, so they run where the reference tree is absent.

Each file holds: `out_rows` (every ROW_STRIDE-th query row of the attention output, fp32),
`out_sum` / `out_abssum` (fp64 checksums over the whole output) and, per variant, the full
score vectors.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def load_reference(ref_root):
  # kernels/attn.py:36 evaluates torch.cuda.current_device() as a default argument at class-definition
  # time; on a CPU-only box that raises, so it is stubbed for the duration of the import.
  if not torch.cuda.is_available():
    torch.cuda.current_device = lambda: "cpu"
  sys.path.insert(0, ref_root)
  from deepgengraph_exp.cases.kernels import KERNEL_ZOO
  return KERNEL_ZOO


def load_reference_gqa(ref_root):
  """The reference's grouped-query variants of the same modules (deepgengraph_exp/figure/membound/attn.py:11-247).
  That file imports flashinfer for a comparison path that is not used here; a stub stands in when the import fails."""
  import importlib.util
  import types
  try:
    import flashinfer  # noqa: F401
  except Exception:
    sys.modules["flashinfer"] = types.ModuleType("flashinfer")
  path = os.path.join(ref_root, "deepgengraph_exp", "figure", "membound", "attn.py")
  spec = importlib.util.spec_from_file_location("_ref_membound_attn", path)
  m = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(m)
  return {"attn": m.Attn, "h2o": m.H2O, "roco": m.RoCo, "snapkv": m.Snapkv}


def main():
  sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
  from oracle import build_ref
  ref_root = sys.argv[1] if len(sys.argv) > 1 else build_ref.reference_root()
  if not ref_root:
    sys.exit("no reference tree: pass its path, or set B200_REFERENCE_ROOT")
  zoo = load_reference(ref_root)
  zoo_gqa = load_reference_gqa(ref_root)
  only = set(sys.argv[2:])          # optional: names of the cases to (re)generate
  for name, c in cases.CASES.items():
    if only and name not in only:
      continue
    inp = cases.make_inputs(name, torch.float32)
    kwargs = dict(kv_head_num=c.get("Hk", c["H"]), head_num=c["H"], head_dim=c["D"])
    if c["model"] == "kf":
      kwargs["tau"] = c["tau"]
    if c.get("source") == "membound":
      if c["model"] == "snapkv":
        kwargs["kernel_size"] = 5
      model = zoo_gqa[c["model"]](**kwargs).eval()
    else:
      model = zoo[c["model"]](**kwargs).eval()
    args = [inp["q"], inp["k"], inp["v"]]
    if c["model"] == "kf":
      args.append(inp["exp_rand"])
    if c["model"] == "corm":
      # Corm.prepare builds the [Sq, Skv] threshold 1/(i+1) (kernels/corm.py:47-49)
      thr = torch.ones(c["Sq"], c["Skv"], dtype=torch.float32)
      for i in range(c["Sq"]):
        thr[i] /= i + 1
      args.append(thr)
    with torch.no_grad():
      outs = model(*args)
    if not isinstance(outs, (tuple, list)):
      outs = (outs,)
    out = outs[0].double()
    blob = {
        "out_rows": outs[0][:, ::cases.ROW_STRIDE].contiguous().numpy().astype(np.float32),
        "out_sum": np.float64(out.sum().item()),
        "out_abssum": np.float64(out.abs().sum().item()),
    }
    for i, extra in enumerate(outs[1:]):
      blob[f"score{i}"] = extra.numpy()
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **blob)
    print(name, {k: getattr(v, "shape", v) for k, v in blob.items()}, os.path.getsize(path), "bytes")


if __name__ == "__main__":
  main()
