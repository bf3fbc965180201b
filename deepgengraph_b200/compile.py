"""Drop-in for the reference's system dispatch (compile.py:6-296): one more `system`, 'b200'.

    f = compile(model, input_names, inputs, output_names, system='b200')
    outs = f(*inputs)          # a tensor, or a tuple in `output_names` order; fresh tensors every call

`model` may be one of this package's core modules (deepgengraph_b200.kernels) or an instance of the
REFERENCE's own classes (deepgengraph_exp.cases.kernels.{Attn,Gemma2,H2O,RoCo,KeyFormer}): they are
recognised by class name and by the attributes their constructors set, so run_kernel.py's flow
(`KERNEL_ZOO[m]()` -> prepare -> compile -> f) works unchanged.  Where the reference spends minutes in
ONNX export, partition search and Triton autotuning, this lookup is immediate: the kernels are prebuilt.
"""
from . import attention as _att

SYSTEM = 'b200'

_OUTPUTS = {
    'Attn': ['out'], 'Gemma2': ['out'], 'H2O': ['out', 'h2o_score'],
    'RoCo': ['out', 'roco_score', 'roco_sq_score'], 'KeyFormer': ['out', 'kf_score'],
    'SnapKV': ['out', 'snapkv_score'], 'Corm': ['out', 'corm_score'],
}


def compile(model, input_names, inputs, output_names, system=SYSTEM):
  if system != SYSTEM:
    raise NotImplementedError(f"system {system} not implemented (this package provides '{SYSTEM}' only)")
  name = model.__class__.__name__
  if name not in _OUTPUTS:
    raise NotImplementedError(f"no fused sm_100a kernel for core module {name}")
  if list(output_names) != _OUTPUTS[name]:
    raise ValueError(f"{name}: expected outputs {_OUTPUTS[name]}, got {list(output_names)}")
  expect_inputs = ['q', 'k', 'v'] + {'KeyFormer': ['exp_rand'], 'Corm': ['corm_mask']}.get(name, [])
  if list(input_names) != expect_inputs:
    raise ValueError(f"{name}: expected inputs {expect_inputs}, got {list(input_names)}")
  window = getattr(model, 'window', -1)

  if name == 'Attn':
    def f(q, k, v):
      return _att.attn_fwd(q, k, v, causal=True, window=window)
  elif name == 'Gemma2':
    cap = float(model.logit_softcapping)

    def f(q, k, v):
      return _att.attn_fwd(q, k, v, causal=True, window=window, softcap=cap)
  elif name == 'H2O':
    def f(q, k, v):
      return _att.attn_score_fwd(q, k, v, want_sq=False, causal=True)
  elif name == 'RoCo':
    def f(q, k, v):
      return _att.attn_score_fwd(q, k, v, want_sq=True, causal=True)
  elif name == 'SnapKV':
    ks = int(model.kernel_size)

    def f(q, k, v):
      return _att.attn_snapkv_fwd(q, k, v, kernel_size=ks, causal=True)
  elif name == 'Corm':
    from .kernels import check_corm_mask

    def f(q, k, v, corm_mask=None):
      check_corm_mask(corm_mask, q.shape[1], k.shape[1])   # only the thresholds of Corm.prepare are implemented
      return _att.attn_corm_fwd(q, k, v, causal=True)
  else:
    tau = float(model.tau)

    def f(q, k, v, exp_rand):
      return _att.attn_kf_fwd(q, k, v, exp_rand, tau=tau, causal=True)
  return f
