#!/usr/bin/env python
"""Benchmark of the hot path: causal attention, bf16, seq 4096, head_dim 128 (BASELINE config 2:
batch 4, 32 heads) on N GPUs of one node, batch x head sharded (every rank owns a config-2-sized shard:
weak scaling, no data-path collective).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Prints ONE JSON line (rank 0).  `value` is the whole-job TFLOP/s with inputs resident in HBM, timed with
CUDA events on the launching stream, max over ranks; `e2e` is the same metric through the public operator
call with HOST (pinned) inputs and the result copied back, copies inside the timed region, next to the time
of the same copies without the kernel (the limit the host link sets); `roofline` relates the kernel to the
measured dense bf16 tensor peak; `cpu_baseline` is the CPU oracle (a port of the reference's PyTorch module,
fp32) timed on a bounded sample of the same workload.

Further records on the same line:
  strong_scaling   the FIXED config 2 (128 (batch, head) units) cut into 128 / N units per rank
  multi_gpu_check  (N > 1) sharded score run + NCCL gather of the score vectors == the one-GPU result, bit for bit
  sub              (N = 1) one record per other configuration: config 3 (H2O, RoCo), config 4 (KeyFormer), config 5
                   (attention, whole layer), the reference's Llama-shaped H2O layer, the five bandwidth ops, the
                   reference's default shape (batch 1, 32 heads, seq 4096, fp16) and the seq-length sweep:
                   median and min per launch over batches of launches (CUDA events around a batch) that rotate over
                   buffer sets whose total footprint is several times L2; every record starts from a GPU left idle for
                   0.3 s (as the headline's timed region does); kernels of a few tens of microseconds are also
                   replayed from a CUDA graph (`us_graph_*`: GPU time without the host's launch cost)

--impl reference times the CPU port alone (all host threads) and prints the same line shape.
FLOPs follow the reference's own formula 4*B*H*S*S*D/2 (run_kernel.py:24).
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B, H, S, D = 4, 32, 4096, 128
METRIC = "causal attn bf16 seq4k d128 TFLOP/s"
WORKLOAD = "config2: causal MHA bf16, batch 4, 32 heads, seq 4096, head_dim 128 (per GPU)"
# dram__bytes_read.sum + dram__bytes_write.sum per attn_fwd_persist_kernel launch: one ncu capture of the same kernel
# on 16 of the 128 (batch, head) units (53.0 MB) scaled by 8 -- traffic grows in proportion to the units, every unit
# reads its q, k, v once from DRAM.  A profiler figure carried as a constant: it cannot be measured in a timed run.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 8 * 53.0e6


def causal_flops(batch, heads, s, d):
  return 4.0 * batch * heads * s * s * d / 2.0


def window_flops(heads, s, d, window):
  """Visible (query, key) pairs under a causal sliding window, times 4 * d flops per pair and head."""
  w = min(window, s)
  pairs = w * (w + 1) / 2.0 + (s - w) * w
  return 4.0 * d * pairs * heads


def load_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  try:
    with open(path) as f:
      p = json.load(f)
    return {"tflops": float(p["bf16_tflops"]), "tflops_sustained": float(p.get("bf16_tflops_sustained", 0.0)),
            "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
  except Exception:
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
  """Samples SM clock and throttle reasons of one GPU while the timed regions run (NVML, read-only)."""

  def __init__(self, index):
    self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
    self._stop = threading.Event()
    self._thread = None
    self._nvml = None

  def start(self):
    try:
      import pynvml
      pynvml.nvmlInit()
      self._nvml = pynvml
      self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
      self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
      self._thread = threading.Thread(target=self._loop_nvml, daemon=True)
    except Exception:
      self._thread = threading.Thread(target=self._loop_smi, daemon=True)
    self._thread.start()

  def _loop_nvml(self):
    n = self._nvml
    names = {
        getattr(n, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
        getattr(n, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
        getattr(n, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
        getattr(n, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
    }
    while not self._stop.is_set():
      try:
        self.samples.append(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM))
        mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
        for bit, name in names.items():
          if mask & bit:
            self.reasons.add(name)
      except Exception:
        pass
      self._stop.wait(0.02)

  def _loop_smi(self):
    q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    while not self._stop.is_set():
      try:
        out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout.strip().split(",")
        self.samples.append(int(float(out[0])))
        self.max_mhz = int(float(out[1]))
        for name, v in zip(names, out[2:]):
          if v.strip().lower().startswith("active"):
            self.reasons.add(name)
      except Exception:
        pass
      self._stop.wait(0.2)

  def stop(self):
    self._stop.set()
    if self._thread is not None:
      self._thread.join(timeout=6)
    s = sorted(self.samples)
    return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
            "samples": len(s)}


# ----------------------------------------------------------------------------------------------------------
# CPU legs (the oracle port of the reference's PyTorch module; nothing else in this file touches oracle/)
# ----------------------------------------------------------------------------------------------------------
def cpu_reference_sample(budget_s, threads=None):
  """Times the CPU oracle (fp32 port of the reference's Attn.forward) on whole heads of the workload, as many
  as fit in `budget_s`.  Returns (tflops, cores, description)."""
  from oracle import reference_math as rm
  if threads:
    torch.set_num_threads(threads)
  cores = torch.get_num_threads()
  g = torch.Generator().manual_seed(0)
  q = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
  k = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
  v = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
  t0 = time.perf_counter()
  rm.attention_ref(q, k, v, causal=True, head_chunk=1)
  t1 = time.perf_counter() - t0
  heads = max(1, min(16, int(budget_s / max(t1, 1e-3))))
  qh, kh, vh = (t.expand(1, S, heads, D).contiguous() for t in (q, k, v))
  passes, t0 = 0, time.perf_counter()
  while True:
    rm.attention_ref(qh, kh, vh, causal=True, head_chunk=2)
    passes += 1
    dt = time.perf_counter() - t0
    if dt >= budget_s or passes >= 64:
      break
  return (causal_flops(1, heads, S, D) * passes / dt / 1e12, cores,
          f"{passes} pass(es) over {heads} of {B * H} (batch, head) units of config2, fp32, {dt:.1f} s")


def cpu_config1_whole(reps=3):
  """BASELINE config 1 timed whole on the host cores: causal MHA fp32, batch 1, 32 heads, seq 1024, head_dim 128,
  q, k, v ~ N(0, 1) / sqrt(128) -- the reference's own CPU-runnable case.  Median of `reps` after one warm-up."""
  from oracle import reference_math as rm
  b1, h1, s1, d1 = 1, 32, 1024, 128
  g = torch.Generator().manual_seed(0)
  q, k, v = (torch.randn(b1, s1, h1, d1, generator=g) / math.sqrt(d1) for _ in range(3))
  rm.attention_ref(q, k, v, causal=True, head_chunk=8)
  ts = []
  for _ in range(reps):
    t0 = time.perf_counter()
    rm.attention_ref(q, k, v, causal=True, head_chunk=8)
    ts.append(time.perf_counter() - t0)
  med = sorted(ts)[len(ts) // 2]
  return {"name": "config1_cpu_whole", "workload": "config1: causal MHA fp32 on CPU, batch 1, 32 heads, seq 1024, head_dim 128",
          "ms_median": med * 1e3, "ms_min": min(ts) * 1e3, "tflops": causal_flops(b1, h1, s1, d1) / med / 1e12,
          "cores": torch.get_num_threads(), "kind": "port"}


def run_reference_arm(args, rank, world):
  """The reference's CPU path (its PyTorch module, restated in oracle/reference_math.py) on the host cores."""
  if rank != 0:
    return
  from oracle import reference_math as rm
  cores = os.cpu_count() or 1
  torch.set_num_threads(cores)
  g = torch.Generator().manual_seed(0)
  # bound the whole run to a few minutes: one step = `heads` whole heads of config 2
  q1 = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
  t0 = time.perf_counter()
  rm.attention_ref(q1, q1, q1, causal=True, head_chunk=1)
  t_head = time.perf_counter() - t0
  total = max(1, args.steps + args.warmup)
  heads = max(1, min(8, int(150.0 / total / max(t_head, 1e-3))))
  rows = S
  if heads == 1 and t_head * total > 200.0:
    # even one head per step is too slow for this many steps: keep the last `rows` query rows of one head
    rows = max(128, int(S * 200.0 / (t_head * total)) // 128 * 128)
  q = torch.randn(1, rows, heads, D, generator=g).to(torch.bfloat16)
  k = torch.randn(1, S, heads, D, generator=g).to(torch.bfloat16)
  v = torch.randn(1, S, heads, D, generator=g).to(torch.bfloat16)
  pairs = rows * (S - rows) + rows * (rows + 1) / 2.0          # visible (query, key) pairs per head
  flops = 4.0 * heads * pairs * D
  for _ in range(args.warmup):
    rm.attention_ref(q, k, v, causal=True, head_chunk=2)
  t0 = time.perf_counter()
  for _ in range(args.steps):
    rm.attention_ref(q, k, v, causal=True, head_chunk=2)
  dt = (time.perf_counter() - t0) / max(1, args.steps)
  tflops = flops / dt / 1e12
  sample = f"{heads} head(s) x last {rows} of {S} query rows of config2 per step, fp32 on CPU"
  print(json.dumps({
      "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
      "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
      "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
      "config": {"workload": WORKLOAD, "reference_path": "PyTorch CPU port of deepgengraph_exp/cases/kernels/attn.py "
                 "(oracle/reference_math.py)", "sample": sample},
      "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
      "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
      "gpu_launches": 0,
  }), flush=True)


# ----------------------------------------------------------------------------------------------------------
# GPU helpers
# ----------------------------------------------------------------------------------------------------------
L2_BYTES = 126 << 20


SUB_IDLE_S = 0.3   # idle time before each sub-record's warm-up


def time_op(fns, iters, warmup):
  """Median and minimum time per launch (microseconds).  `fns` are closures of the SAME operation on different buffer
  sets whose total footprint exceeds L2 several times over (or a single closure whose own inputs do): a timed batch
  walks the sets round robin, at least four launches per batch, between one pair of CUDA events on the current
  stream, so that a launch neither finds its inputs in L2 nor carries the ~5 us gap of an event pair of its own.
  At least `iters` launches are timed in all."""
  if callable(fns):
    fns = [fns]
  per_batch = max(len(fns), 4)
  for i in range(max(warmup, len(fns))):
    fns[i % len(fns)]()
  batches = max(10, -(-iters // per_batch))
  pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(batches)]
  k = 0
  for e0, e1 in pairs:
    e0.record()
    for _ in range(per_batch):
      fns[k % len(fns)]()
      k += 1
    e1.record()
  torch.cuda.synchronize()
  ts = sorted(e0.elapsed_time(e1) * 1e3 / per_batch for e0, e1 in pairs)
  return ts[len(ts) // 2], ts[0]


def time_graph(fns, iters):
  """The batches of `time_op` captured once into a CUDA graph and replayed: per-launch GPU time without the host's
  cost of issuing the launch (a Python call into the library costs 15-20 us, as much as the shortest kernels here
  run).  Returns (median, min) in microseconds, or None when the operation cannot be captured."""
  if callable(fns):
    fns = [fns]
  per_batch = max(len(fns), 4)
  side = torch.cuda.Stream()
  try:
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
      for i in range(max(3, len(fns))):
        fns[i % len(fns)]()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
      for k in range(per_batch):
        fns[k % len(fns)]()
  except Exception:  # noqa: BLE001 -- the eager figure stands alone
    torch.cuda.synchronize()
    return None
  for _ in range(3):
    graph.replay()
  batches = max(10, -(-iters // per_batch))
  pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(batches)]
  for e0, e1 in pairs:
    e0.record()
    graph.replay()
    e1.record()
  torch.cuda.synchronize()
  ts = sorted(e0.elapsed_time(e1) * 1e3 / per_batch for e0, e1 in pairs)
  return ts[len(ts) // 2], ts[0]


def buffer_sets(footprint_bytes, cap=12):
  """How many independent buffer sets of `footprint_bytes` make a rotation that outgrows L2 (4 x L2, at most `cap`)."""
  return int(max(1, min(cap, -(-4 * L2_BYTES // max(1, footprint_bytes)))))


def sub_records(dev, peaks, iters, warmup):
  """One record per configuration other than the headline one (N = 1 only): see the module docstring."""
  from deepgengraph_b200 import attention as att
  from deepgengraph_b200 import layer as L
  from deepgengraph_b200 import native_ops as ops
  recs = []
  gen = torch.Generator(device=dev).manual_seed(7)
  peak_tf, peak_bw = peaks["tflops"], peaks["hbm_gbs"]

  def randn(*shape, dtype=torch.bfloat16, scale=1.0):
    return (torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32) * scale).to(dtype)

  def record(name, workload, fns, bound, work, extra=None, graph=False):
    """work = algorithmic flops (tensor) or bytes (hbm) per launch.  graph=True (kernels of a few tens of
    microseconds): the same batches are also replayed from a CUDA graph; `us_graph_*` and `*_graph` are then the GPU's
    own time per launch, `us_median` stays the eager call through the Python API."""
    n_sets = len(fns) if isinstance(fns, list) else 1
    # Every record starts from an idle GPU, as the headline's timed region does: looping for seconds these kernels
    # run into the board's power cap and the SM clock settles 10-25 % lower.
    torch.cuda.synchronize()
    time.sleep(SUB_IDLE_S)
    med, mn = time_op(fns, iters, warmup)
    r = {"name": name, "workload": workload, "us_median": med, "us_min": mn, "bound": bound, "buffer_sets": n_sets}
    if bound == "tensor":
      r.update(tflops=work / med / 1e6, frac_of_measured_peak=work / med / 1e6 / peak_tf)
    else:
      r.update(gbs=work / med / 1e3, algorithmic_bytes=work, frac_of_measured_peak=work / med / 1e3 / peak_bw)
    if graph:
      torch.cuda.synchronize()
      time.sleep(SUB_IDLE_S)
      tg = time_graph(fns, iters)
      if tg is None:
        r["graph"] = "not capturable"
      else:
        r.update(us_graph_median=tg[0], us_graph_min=tg[1])
        if bound == "tensor":
          r.update(tflops_graph=work / tg[0] / 1e6, frac_of_measured_peak_graph=work / tg[0] / 1e6 / peak_tf)
        else:
          r.update(gbs_graph=work / tg[0] / 1e3, frac_of_measured_peak_graph=work / tg[0] / 1e3 / peak_bw)
    if extra:
      r.update(extra)
    recs.append(r)
    return r

  def qkv_sets(b, s, h, hk, d, dtype=torch.bfloat16, q_scale=1.0):
    n = buffer_sets((2 * b * s * h * d + 2 * b * s * hk * d) * 2)
    return [(randn(b, s, h, d, dtype=dtype, scale=q_scale), randn(b, s, hk, d, dtype=dtype), randn(b, s, hk, d, dtype=dtype))
            for _ in range(n)]

  def over(sets, f):
    return [(lambda t=t: f(*t)) for t in sets]

  # ---- config 3: H2O / RoCo (attention + per-key column sums) ----
  b3, h3, s3 = 2, 32, 4096
  sets = qkv_sets(b3, s3, h3, h3, D)
  f3 = causal_flops(b3, h3, s3, D)
  w3 = "config3: B2 H32 S4096 D128 bf16 causal"
  record("config3_h2o", w3 + ", out + sum_i p", over(sets, lambda q, k, v: att.attn_score_fwd(q, k, v)), "tensor", f3,
         {"credited_flops": "attention only (the second QK^T of the sweep is overhead)"})
  record("config3_roco", w3 + ", out + sum_i p + sum_i p^2",
         over(sets, lambda q, k, v: att.attn_score_fwd(q, k, v, want_sq=True)), "tensor", f3)
  record("config3_forward_only", w3 + ", out only", over(sets, lambda q, k, v: att.attn_fwd(q, k, v)), "tensor", f3)
  record("config2_shape_softcap50", "B2 H32 S4096 D128 bf16 causal, soft-cap 50",
         over(sets, lambda q, k, v: att.attn_fwd(q, k, v, softcap=50.0)), "tensor", f3)
  scores = [att.attn_score_fwd(*t)[1] for t in sets]
  record("config3_kv_evict_topk", w3 + ", budget 512: topk -> sort -> gather",
         [(lambda t=t, sc=sc: att.kv_evict_topk(sc, t[1], t[2], 512)) for t, sc in zip(sets, scores)], "hbm",
         scores[0].numel() * 4 + 4 * b3 * 512 * h3 * D * 2, graph=True)
  del sets, scores

  # the reference's default shape (run_kernel.py:20-24; the workload of its Fig. 14): batch 1, 32 heads, seq 4096, fp16
  sets = qkv_sets(1, 4096, 32, 32, D, dtype=torch.float16)
  record("reference_default_attn_fp16", "B1 H32 S4096 D128 fp16 causal (run_kernel.py defaults)",
         over(sets, lambda q, k, v: att.attn_fwd(q, k, v)), "tensor", causal_flops(1, 32, 4096, D),
         {"published_a100_ms": {"FlashTensor": 0.929, "FlashAttention-2": 0.980, "TensorRT": 2.01}})
  record("reference_default_gemma2_fp16", "B1 H32 S4096 D128 fp16 causal, soft-cap 50",
         over(sets, lambda q, k, v: att.attn_fwd(q, k, v, softcap=50.0)), "tensor", causal_flops(1, 32, 4096, D),
         {"published_a100_ms": {"FlashTensor": 0.937, "FlashAttention-2": 1.314, "TensorRT": 4.27}})
  del sets

  # ---- seq-length sweep at batch 1, 32 heads (the reference's fig13/run.sh:30) ----
  for s in (1024, 2048, 4096, 8192):
    sets = qkv_sets(1, s, 32, 32, D)
    record(f"sweep_attn_s{s}", f"B1 H32 S{s} D128 bf16 causal", over(sets, lambda q, k, v: att.attn_fwd(q, k, v)),
           "tensor", causal_flops(1, 32, s, D), graph=s <= 2048)
    record(f"sweep_h2o_s{s}", f"B1 H32 S{s} D128 bf16 causal, out + sum_i p",
           over(sets, lambda q, k, v: att.attn_score_fwd(q, k, v)), "tensor", causal_flops(1, 32, s, D))
    del sets

  # ---- config 4: KeyFormer with the [B, H, S, S] fp32 noise tensor as an input (HBM-bound) ----
  b4, h4, s4 = 2, 32, 2048
  q, k, v = (randn(b4, s4, h4, D) for _ in range(3))
  exp_rand = -torch.log(torch.rand(b4, h4, s4, s4, generator=gen, device=dev).clamp_min_(1e-7))
  bytes4 = exp_rand.numel() * 4 + 4 * q.numel() * 2 + b4 * h4 * s4 * 4
  record("config4_keyformer", "config4: B2 H32 S2048 D128 bf16 causal, tau 1.0, Gumbel noise tensor input (1.07 GB)",
         lambda: att.attn_kf_fwd(q, k, v, exp_rand, tau=1.0), "hbm", bytes4,
         {"tflops_credited": causal_flops(b4, h4, s4, D) / 1e12, "note": "noise counted once in the algorithmic bytes"})
  del exp_rand
  # the same scores with the noise generated inside the kernels (Philox4x32-10 keyed by seed and position): nothing of
  # size S x S is read; the sweeps are then bound by integer/issue throughput (about 35 instructions per element for
  # the generator, the Gumbel mapping and the quad exchange), so the tensor figure is the credited attention FLOPs
  record("config4_keyformer_generated_noise", "config4 shape, noise generated in the kernels from a seed (no 1.07 GB input)",
         lambda: att.attn_kf_fwd(q, k, v, None, tau=1.0, seed=11), "tensor", causal_flops(b4, h4, s4, D),
         {"note": "issue-bound: counter-based generator, two log2 and one exp2 per element and sweep"})
  del q, k, v

  # ---- config 5: attention, whole Gemma-2-style layer, bandwidth ops ----
  cfg = L.Gemma2LayerConfig()
  s5, T = 8192, 8192
  sets = qkv_sets(1, s5, cfg.heads, cfg.kv_heads, cfg.head_dim, q_scale=2.0)
  f5 = window_flops(cfg.heads, s5, cfg.head_dim, cfg.window)
  record("config5_attention", "config5: B1 S8192 16q/8kv heads D256 window 4096 soft-cap 50 bf16",
         over(sets, lambda q, k, v: att.attn_fwd(q, k, v, window=cfg.window, softcap=cfg.softcap)), "tensor", f5)
  del sets
  w = L.init_weights(cfg, torch.bfloat16, dev, seed=0)
  x = randn(1, s5, cfg.hidden)
  qkv_out = (cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim
  gemm_flops = 2.0 * T * (cfg.hidden * qkv_out + cfg.heads * cfg.head_dim * cfg.hidden +
                          cfg.hidden * 2 * cfg.intermediate + cfg.intermediate * cfg.hidden)
  record("config5_layer", "config5: Gemma-2-style decoder layer, hidden 3584, GeGLU 14336 (4 cuBLAS GEMMs + this library's ops)",
         lambda: L.gemma2_layer(x, w, cfg), "tensor", gemm_flops + f5, {"gemm_tflop": gemm_flops / 1e12})
  del w, x
  sz, hid = 2, cfg.hidden
  wn = (1 + 0.02 * randn(hid).float()).to(torch.bfloat16)
  n = buffer_sets(2 * T * hid * sz)
  xs = [(randn(T, hid), torch.empty(T, hid, dtype=torch.bfloat16, device=dev)) for _ in range(n)]
  record("rms_norm", f"[{T}, {hid}] bf16", [(lambda t=t: ops.rms_norm(t[1], t[0], wn, cfg.eps)) for t in xs], "hbm",
         2 * T * hid * sz + hid * sz, graph=True)
  record("fused_add_rms_norm", f"[{T}, {hid}] bf16, in place",
         [(lambda t=t: ops.fused_add_rms_norm(t[0], t[1], wn, cfg.eps)) for t in xs], "hbm", 4 * T * hid * sz, graph=True)
  del xs
  n = buffer_sets(3 * T * cfg.intermediate * sz, cap=4)
  gs = [(randn(T, 2 * cfg.intermediate), torch.empty(T, cfg.intermediate, dtype=torch.bfloat16, device=dev)) for _ in range(n)]
  record("gelu_tanh_and_mul", f"[{T}, 2x{cfg.intermediate}] bf16", [(lambda t=t: ops.gelu_tanh_and_mul(t[1], t[0])) for t in gs],
         "hbm", 3 * T * cfg.intermediate * sz)
  record("silu_and_mul", f"[{T}, 2x{cfg.intermediate}] bf16", [(lambda t=t: ops.silu_and_mul(t[1], t[0])) for t in gs],
         "hbm", 3 * T * cfg.intermediate * sz)
  del gs
  pos = torch.arange(T, dtype=torch.int32, device=dev)
  n = buffer_sets(2 * T * (cfg.heads + cfg.kv_heads) * cfg.head_dim * sz)
  rs = [(randn(T, cfg.heads * cfg.head_dim), randn(T, cfg.kv_heads * cfg.head_dim)) for _ in range(n)]
  record("rotary_embedding_online", f"q [{T}, {cfg.heads}x{cfg.head_dim}], k [{T}, {cfg.kv_heads}x{cfg.head_dim}] bf16",
         [(lambda t=t: ops.rotary_embedding_online(pos, t[0], t[1], cfg.head_dim, cfg.rope_theta)) for t in rs], "hbm",
         2 * T * (cfg.heads + cfg.kv_heads) * cfg.head_dim * sz + 4 * T, graph=True)
  del rs

  # ---- the reference's Llama-shaped layer with a score variant and the eviction fused in (models/h2o.py:34-86),
  #      random weights as in run_e2e.py:48-66: hidden 4096, 32 heads, intermediate 11008, fp16, seq 4096 ----
  lc = L.LlamaLayerConfig()
  lw = L.init_llama_weights(lc, torch.float16, dev, seed=0)
  sl = 4096
  xl = randn(1, sl, lc.hidden, dtype=torch.float16)
  lg = 2.0 * sl * (lc.hidden * 3 * lc.hidden + lc.hidden * lc.hidden + lc.hidden * 2 * lc.intermediate +
                   lc.intermediate * lc.hidden)
  for variant in ("h2o", "roco"):
    record(f"llama_layer_{variant}", f"Llama-7B-shaped layer fp16, seq 4096, {variant} scores + KV eviction to 512 keys",
           lambda: L.llama_score_layer(xl, lw, lc, variant), "tensor", lg + causal_flops(1, lc.heads, sl, lc.head_dim),
           {"gemm_tflop": lg / 1e12})
  return recs


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=100)
  ap.add_argument("--warmup", type=int, default=10)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--e2e-steps", type=int, default=50)
  ap.add_argument("--sub-iters", type=int, default=100)
  ap.add_argument("--no-cpu-baseline", action="store_true")
  ap.add_argument("--no-sub", action="store_true", help="skip the per-configuration sub-records (N = 1)")
  args = ap.parse_args()
  args.warmup = max(args.warmup, 3)

  rank = int(os.environ.get("RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))

  if args.impl == "reference":
    run_reference_arm(args, rank, world)
    return

  import torch.distributed as dist
  from deepgengraph_b200 import attention as att
  from deepgengraph_b200 import sharding as sh

  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  if world > 1:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # keep NCCL's own messages off stdout (one JSON line)
    dist.init_process_group("nccl", device_id=dev)

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  def max_over_ranks(x):
    t = torch.tensor([x], dtype=torch.float64, device=dev)
    if world > 1:
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()

  # this rank's shard: B x H (batch, head) units, generated locally from seed + rank (no scatter is timed)
  gen = torch.Generator(device=dev).manual_seed(1234 + rank)
  q = torch.randn(B, S, H, D, generator=gen, device=dev, dtype=torch.bfloat16)
  k = torch.randn(B, S, H, D, generator=gen, device=dev, dtype=torch.bfloat16)
  v = torch.randn(B, S, H, D, generator=gen, device=dev, dtype=torch.bfloat16)
  flops_rank = causal_flops(B, H, S, D)

  sampler = ClockSampler(local_rank)
  for _ in range(args.warmup):
    out = att.attn_fwd(q, k, v, causal=True)
  barrier()
  sampler.start()

  # ---- device-resident timing: K steps, CUDA events on the launching (current) stream ----
  evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
  barrier()
  evs[0].record()
  for i in range(args.steps):
    out = att.attn_fwd(q, k, v, causal=True)
    evs[i + 1].record()
  barrier()
  ms_step = max_over_ranks(evs[0].elapsed_time(evs[-1])) / args.steps
  value = world * flops_rank / (ms_step * 1e-3) / 1e12
  per_step = sorted(evs[i].elapsed_time(evs[i + 1]) * 1e3 for i in range(args.steps))   # this rank, microseconds

  # ---- strong scaling: the FIXED config 2 (B x H = 128 units) cut into 128 / world units per rank ----
  lo, hi = sh.unit_range(B * H, world, rank)
  units = hi - lo
  if units % H == 0:
    shape = (units // H, S, H, D)          # whole batch elements
  else:
    shape = (1, S, units, D)               # part of one batch element's heads
  if world == 1:
    ms_strong = ms_step
  else:
    qs, ks, vs = (t.reshape(-1)[:shape[0] * S * shape[2] * D].view(shape) for t in (q, k, v))
    for _ in range(args.warmup):
      att.attn_fwd(qs, ks, vs, causal=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
      att.attn_fwd(qs, ks, vs, causal=True)
    e1.record()
    barrier()
    ms_strong = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    del qs, ks, vs
  strong = {"workload": "config2 as ONE fixed problem (128 (batch, head) units), cut into equal unit ranges",
            "units_per_rank": units, "ms_per_step": ms_strong, "value": flops_rank / (ms_strong * 1e-3) / 1e12,
            "unit": "TFLOP/s", "scaling": "strong"}

  # ---- end to end: pinned host inputs -> H2D -> kernel -> D2H of the result, every step ----
  # Every step copies its own q, k, v from pinned host memory and copies its output back.  Copies and kernels run
  # on three streams with two device buffer sets, so that step i+1's upload and step i-1's download overlap step
  # i's kernel (the operator call itself is the public attention.attn_fwd on the current stream).  The same
  # schedule without the kernel ("copy only") is timed next to it: that is the limit the host link sets.
  qh, kh, vh = (x.cpu().pin_memory() for x in (q, k, v))
  oh = [torch.empty_like(qh).pin_memory() for _ in range(2)]
  dev_in = [tuple(torch.empty_like(t) for t in (q, k, v)) for _ in range(2)]
  dev_out = [torch.empty_like(q) for _ in range(2)]
  s_h2d, s_run, s_d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
  ev_in = [torch.cuda.Event() for _ in range(2)]      # upload of buffer set b finished
  ev_free = [torch.cuda.Event() for _ in range(2)]    # kernel that read buffer set b finished
  ev_out = [torch.cuda.Event() for _ in range(2)]     # output of slot b produced
  ev_done = [torch.cuda.Event() for _ in range(2)]    # download of slot b finished
  outs = [None, None]

  def e2e_step(i, with_kernel):
    b = i & 1
    with torch.cuda.stream(s_h2d):
      s_h2d.wait_event(ev_free[b])
      for dst, src in zip(dev_in[b], (qh, kh, vh)):
        dst.copy_(src, non_blocking=True)
      ev_in[b].record(s_h2d)
    with torch.cuda.stream(s_run):
      s_run.wait_event(ev_in[b])
      s_run.wait_event(ev_done[b])                     # the previous output in this slot has left the device
      outs[b] = att.attn_fwd(*dev_in[b], causal=True) if with_kernel else dev_out[b]
      ev_free[b].record(s_run)
      ev_out[b].record(s_run)
    with torch.cuda.stream(s_d2h):
      s_d2h.wait_event(ev_out[b])
      oh[b].copy_(outs[b], non_blocking=True)
      ev_done[b].record(s_d2h)

  def e2e_run(n, with_kernel):
    for i in range(n):
      e2e_step(i, with_kernel)
    for st in (s_h2d, s_run, s_d2h):
      torch.cuda.current_stream(dev).wait_stream(st)

  def e2e_timed(with_kernel):
    e2e_run(4, with_kernel)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    e2e_run(args.e2e_steps, with_kernel)
    e1.record()
    barrier()
    return max_over_ranks(e0.elapsed_time(e1)) / args.e2e_steps

  e2e_ms = e2e_timed(True)
  e2e_value = world * flops_rank / (e2e_ms * 1e-3) / 1e12
  if not torch.equal(oh[(args.e2e_steps - 1) & 1], out.cpu()):
    raise RuntimeError("end-to-end output differs from the device-resident run")
  clocks = sampler.stop()          # the copy-only leg below leaves the SMs idle: not part of the clock record
  copy_ms = e2e_timed(False)
  del qh, kh, vh, oh, dev_in, dev_out, outs

  # ---- multi-GPU correctness: sharded score run + NCCL gather == the one-GPU run, bit for bit ----
  multi_check = None
  if world > 1:
    bc, hc, sc = 2, 32, 4096                                        # config 3's shape; the same problem on every rank
    g3 = torch.Generator(device=dev).manual_seed(99)
    q3, k3, v3 = (torch.randn(bc, sc, hc, D, generator=g3, device=dev, dtype=torch.bfloat16) for _ in range(3))
    results = sh.run_sharded(lambda a, b_, c: att.attn_score_fwd(a, b_, c), q3, k3, v3, world, rank)
    full = sh.gather_scores(sh.scores_from_pieces(results, index=1), bc * hc, world, rank)
    ref_out, ref_score = att.attn_score_fwd(q3, k3, v3)
    ok = torch.equal(full, ref_score.reshape(bc * hc, sc))
    for piece, (o, _) in results:
      ok = ok and torch.equal(o[0], ref_out[piece.b, :, piece.hk_lo:piece.hk_hi])
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    multi_check = "ok" if flag.item() == 1 else "MISMATCH"
    del q3, k3, v3, results, full, ref_out, ref_score

  # no bounded device-side wait may have expired
  import ctypes
  from deepgengraph_b200 import _lib
  word = ctypes.c_int(0)
  st = _lib.load().b200_device_status(ctypes.byref(word))
  if st != 0:
    raise RuntimeError(f"device status word {word.value:#x}: a kernel wait expired, the numbers are void")
  if not torch.isfinite(out.float()).all():
    raise RuntimeError("non-finite attention output")
  if multi_check == "MISMATCH":
    raise RuntimeError("sharded run differs from the single-GPU run")

  if rank == 0:
    peaks = load_peaks()
    peak_burst = peaks["tflops"]
    achieved = flops_rank / (ms_step * 1e-3) / 1e12   # per GPU, per launch: one kernel per step
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": B * world, "heads": H, "seq_len": S, "head_dim": D,
                   "parallelism": f"batch x head sharded over {world} GPU(s), no collective",
                   "l2": "q,k,v,out = 537 MB per GPU, larger than the 126 MB L2",
                   "us_per_core_module": ms_step * 1e3, "us_median": per_step[len(per_step) // 2],
                   "us_min": per_step[0], "e2e_steps": args.e2e_steps},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_burst, "unit": "TFLOP/s",
                     "frac": achieved / peak_burst, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     "traffic_source": "ncu dram__bytes of a 16-unit capture x 8 (constant, not measured in this run)",
                     "peak_source": f"{peaks['source']} (cuBLAS bf16 burst; sustained {peaks['tflops_sustained']})",
                     "frac_of_datasheet_2250": achieved / 2250.0},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": 3 * q.numel() * 2,
                "d2h_bytes_per_step": q.numel() * 2, "ms_per_step": e2e_ms, "copy_only_ms_per_step": copy_ms,
                "frac_of_copy_limit": copy_ms / e2e_ms},
        "strong_scaling": strong,
        "gpu_launches": args.steps,
        "clocks": clocks,
    }
    if multi_check is not None:
      line["multi_gpu_check"] = multi_check
    del q, k, v, out
    torch.cuda.empty_cache()
    if world == 1 and not args.no_sub:
      line["sub"] = sub_records(dev, peaks, args.sub_iters, 8)
      line["config"]["sub_idle_s"] = SUB_IDLE_S
    if world == 1 and not args.no_cpu_baseline:
      tf, cores, sample = cpu_reference_sample(budget_s=15.0)
      line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample}
      line.setdefault("sub", []).append(cpu_config1_whole())
    print(json.dumps(line), flush=True)

  if world > 1:
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
