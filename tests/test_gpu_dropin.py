"""The reference's operator flow -- KERNEL_ZOO[name]() -> prepare -> compile(..., system) -> f(*inputs) --
with system='b200' (run_kernel.py:44-78,100-107), checked the way run_kernel.py checks (`compare`, rtol =
atol = 1e-2 on fp16, utils.py:121-133) against the CPU oracle standing in for the torch module."""
import pytest
import torch

from deepgengraph_b200.compile import compile as b200_compile
from deepgengraph_b200.kernels import KERNEL_ZOO
from oracle import reference_math as rm

pytestmark = pytest.mark.gpu

WANT = {"attn": ("out",), "gemma2": ("out",), "h2o": ("out", "colsum"), "roco": ("out", "colsum", "colsum_sq"),
        "kf": ("out", "kf"), "snapkv": ("out", "snapkv"), "corm": ("out", "corm")}


@pytest.mark.parametrize("name", sorted(KERNEL_ZOO))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_run_kernel_flow(cuda_device, name, dtype):
  torch.manual_seed(0)
  model = KERNEL_ZOO[name](kv_head_num=4, head_num=4, head_dim=128).eval().cuda()
  specs = model.prepare(batch_size=1, q_len=512, kv_len=512, dtype=dtype)
  input_names = list(specs['input'].keys())
  inputs = [specs['input'][n] for n in input_names]
  output_names = specs['output']
  f = b200_compile(model=model, input_names=input_names, inputs=inputs, output_names=output_names, system='b200')
  outs = f(*inputs)
  outs2 = model(*inputs)           # the module itself runs the same kernels
  if not isinstance(outs, tuple):
    outs, outs2 = (outs,), (outs2,)
  assert len(outs) == len(output_names)
  cpu = [t.cpu() for t in inputs]
  ref = rm.attention_ref(cpu[0], cpu[1], cpu[2], causal=True, softcap=50.0 if name == "gemma2" else 0.0,
                         exp_rand=cpu[3] if name == "kf" else None, tau=getattr(model, "tau", 1.0), want=WANT[name])
  assert outs[0].dtype == dtype and outs[0].shape == inputs[0].shape and outs[0].is_cuda
  tol = 1e-2 if dtype == torch.float16 else 2e-2
  torch.testing.assert_close(outs[0].float().cpu(), ref["out"], rtol=tol, atol=tol)
  for o, key in zip(outs[1:], WANT[name][1:]):
    assert tuple(o.shape) == (1, 4, 512)
    if key == "corm":
      assert o.dtype == torch.bool and (o.cpu() != ref[key]).float().mean().item() <= 0.01
    else:
      assert o.dtype == torch.float32
      torch.testing.assert_close(o.cpu(), ref[key], rtol=1e-3, atol=1e-6)
  for a, b in zip(outs, outs2):
    assert torch.equal(a, b)
  assert f(*inputs)[0].data_ptr() != outs[0].data_ptr() or len(outs) == 1   # fresh outputs on every call


def test_compile_accepts_reference_style_modules_by_class_name(cuda_device):
  # an object shaped like the reference's own class (same class name, same attributes) is accepted
  class Gemma2(torch.nn.Module):
    logit_softcapping = 30.0
  q = torch.randn(1, 256, 2, 128, device=cuda_device, dtype=torch.float16)
  f = b200_compile(Gemma2(), ['q', 'k', 'v'], [q, q, q], ['out'], system='b200')
  ref = rm.attention_ref(q.cpu(), q.cpu(), q.cpu(), softcap=30.0)["out"]
  torch.testing.assert_close(f(q, q, q).float().cpu(), ref, rtol=1e-2, atol=1e-2)
  with pytest.raises(NotImplementedError):
    b200_compile(Gemma2(), ['q', 'k', 'v'], [q, q, q], ['out'], system='our')
  with pytest.raises(ValueError):
    b200_compile(Gemma2(), ['q', 'k', 'v'], [q, q, q], ['out', 'extra'], system='b200')


def test_custom_ops_are_registered_with_fake_kernels(cuda_device):
  q = torch.randn(1, 128, 2, 128, device=cuda_device, dtype=torch.bfloat16)
  out = torch.ops.b200attn.attn_fwd(q, q, q, True, -1, 0.0, 0.0)
  assert out.shape == q.shape
  from torch._subclasses.fake_tensor import FakeTensorMode
  with FakeTensorMode():
    fq = torch.empty(1, 128, 2, 128, device="cuda", dtype=torch.bfloat16)
    o, s = torch.ops.b200attn.attn_score_fwd(fq, fq, fq, True, -1, 0.0, 0.0)
    assert tuple(o.shape) == (1, 128, 2, 128) and tuple(s.shape) == (1, 2, 128) and s.dtype == torch.float32


def test_nvtx_ranges_do_not_change_results(cuda_device):
  from deepgengraph_b200 import attention as att, tracing
  g = torch.Generator().manual_seed(0)
  q, k, v = (torch.randn(1, 256, 2, 128, generator=g).to(torch.bfloat16).to(cuda_device) for _ in range(3))
  want = att.attn_fwd(q, k, v)
  tracing.enable(True)
  try:
    got = att.attn_fwd(q, k, v)
  finally:
    tracing.enable(False)
  assert torch.equal(got, want)


def test_prepare_draws_the_reference_distributions(cuda_device):
  # Attn draws q, k, v from U[0, 1) (kernels/attn.py:38-40); every other module from N(0, 1); KeyFormer's exp_rand is
  # 1 + |N(0, 1)| (kernels/kf.py:48); Corm's mask holds 1 / (i + 1) in row i (kernels/corm.py:47-49)
  torch.manual_seed(0)
  for name, cls in KERNEL_ZOO.items():
    spec = cls(kv_head_num=2, head_num=2, head_dim=128).prepare(batch_size=1, q_len=1024, kv_len=1024, dtype=torch.float16)
    for key in ("q", "k", "v"):
      t = spec["input"][key].float()
      assert t.is_cuda and tuple(t.shape) == (1, 1024, 2, 128)
      if name == "attn":
        assert t.min().item() >= 0.0 and t.max().item() < 1.0 and abs(t.mean().item() - 0.5) < 0.01
        assert abs(t.var().item() - 1.0 / 12.0) < 0.01
      else:
        assert abs(t.mean().item()) < 0.02 and abs(t.std().item() - 1.0) < 0.02 and t.min().item() < -3.0
    if name == "kf":
      er = spec["input"]["exp_rand"]
      assert er.dtype == torch.float32 and tuple(er.shape) == (1, 2, 1024, 1024) and er.min().item() >= 1.0
      assert abs((er - 1).mean().item() - (2.0 / 3.141592653589793) ** 0.5) < 0.01      # mean of |N(0, 1)|
    if name == "corm":
      m = spec["input"]["corm_mask"]
      assert tuple(m.shape) == (1024, 1024)
      torch.testing.assert_close(m[:, 0].cpu(), 1.0 / torch.arange(1, 1025, dtype=torch.float32))


def test_corm_with_foreign_thresholds_is_refused(cuda_device):
  # the kernel evaluates the thresholds 1 / (i + 1) itself; a caller that passes any other corm_mask must hear about it
  model = KERNEL_ZOO["corm"](kv_head_num=2, head_num=2, head_dim=128)
  spec = model.prepare(batch_size=1, q_len=256, kv_len=256, dtype=torch.float16)
  names = list(spec["input"].keys())
  inputs = [spec["input"][n] for n in names]
  f = b200_compile(model, names, inputs, spec["output"], system="b200")
  f(*inputs)
  with pytest.raises(NotImplementedError):
    f(inputs[0], inputs[1], inputs[2], inputs[3] * 0.5)
  with pytest.raises(NotImplementedError):
    model(inputs[0], inputs[1], inputs[2], inputs[3][:, :128].contiguous())
