#!/usr/bin/env python
"""Benchmark of the hot path: causal attention, bf16, seq 4096, head_dim 128 (BASELINE config 2:
batch 4, 32 heads) on N GPUs of one node, batch x head sharded (every rank owns a config-2-sized shard:
weak scaling, no data-path collective).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Prints ONE JSON line (rank 0).  `value` is the whole-job TFLOP/s with inputs resident in HBM, timed with
CUDA events on the launching stream, max over ranks; `e2e` is the same metric through the public operator
call with HOST (pinned) inputs and the result copied back, copies inside the timed region; `roofline`
relates the kernel to the measured dense bf16 tensor peak; `cpu_baseline` is the CPU oracle (a port of the
reference's PyTorch module, fp32) timed on a bounded sample of the same workload.

--impl reference times that CPU port alone (all host threads) and prints the same line shape.
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
# dram__bytes_read.sum + dram__bytes_write.sum per attn_fwd_kernel launch: ncu capture of the same kernel on 16 of
# the 128 (batch, head) units (51.7 MB, profiles/attn_fwd_kernel_b1_h16_s4096.md) scaled by 8 -- traffic grows in
# proportion to the units, every unit reads its q, k, v once from DRAM.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 8 * 53.0e6


def causal_flops(batch, heads, s, d):
  return 4.0 * batch * heads * s * s * d / 2.0


def load_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  try:
    with open(path) as f:
      p = json.load(f)
    return float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", 0.0)), "measured"
  except Exception:
    return 1590.0, 1400.0, "fallback"


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


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=100)
  ap.add_argument("--warmup", type=int, default=10)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--e2e-steps", type=int, default=20)
  ap.add_argument("--no-cpu-baseline", action="store_true")
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

  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  if world > 1:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

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
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  barrier()
  e0.record()
  for _ in range(args.steps):
    out = att.attn_fwd(q, k, v, causal=True)
  e1.record()
  barrier()
  ms_total = e0.elapsed_time(e1)
  t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
  if world > 1:
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
  ms_step = t.item() / args.steps
  value = world * flops_rank / (ms_step * 1e-3) / 1e12

  # ---- end to end: pinned host inputs -> H2D -> kernel -> D2H of the result, every step ----
  # Every step copies its own q, k, v from pinned host memory and copies its output back.  Copies and kernels run
  # on three streams with two device buffer sets, so that step i+1's upload and step i-1's download overlap step
  # i's kernel (the operator call itself is the public attention.attn_fwd on the current stream).
  qh, kh, vh = (x.cpu().pin_memory() for x in (q, k, v))
  oh = [torch.empty_like(qh).pin_memory() for _ in range(2)]
  dev_in = [tuple(torch.empty_like(t) for t in (q, k, v)) for _ in range(2)]
  s_h2d, s_run, s_d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
  ev_in = [torch.cuda.Event() for _ in range(2)]      # upload of buffer set b finished
  ev_free = [torch.cuda.Event() for _ in range(2)]    # kernel that read buffer set b finished
  ev_out = [torch.cuda.Event() for _ in range(2)]     # output of slot b produced
  ev_done = [torch.cuda.Event() for _ in range(2)]    # download of slot b finished
  outs = [None, None]

  def e2e_step(i):
    b = i & 1
    with torch.cuda.stream(s_h2d):
      s_h2d.wait_event(ev_free[b])
      for dst, src in zip(dev_in[b], (qh, kh, vh)):
        dst.copy_(src, non_blocking=True)
      ev_in[b].record(s_h2d)
    with torch.cuda.stream(s_run):
      s_run.wait_event(ev_in[b])
      s_run.wait_event(ev_done[b])                     # the previous output in this slot has left the device
      outs[b] = att.attn_fwd(*dev_in[b], causal=True)
      ev_free[b].record(s_run)
      ev_out[b].record(s_run)
    with torch.cuda.stream(s_d2h):
      s_d2h.wait_event(ev_out[b])
      oh[b].copy_(outs[b], non_blocking=True)
      ev_done[b].record(s_d2h)

  def e2e_run(n):
    for i in range(n):
      e2e_step(i)
    for st in (s_h2d, s_run, s_d2h):
      torch.cuda.current_stream(dev).wait_stream(st)

  e2e_run(4)
  barrier()
  e0.record()
  e2e_run(args.e2e_steps)
  e1.record()
  barrier()
  t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
  if world > 1:
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
  e2e_ms = t.item() / args.e2e_steps
  e2e_value = world * flops_rank / (e2e_ms * 1e-3) / 1e12
  if not torch.equal(oh[(args.e2e_steps - 1) & 1], out.cpu()):
    raise RuntimeError("end-to-end output differs from the device-resident run")
  clocks = sampler.stop()

  # no bounded device-side wait may have expired
  import ctypes
  from deepgengraph_b200 import _lib
  word = ctypes.c_int(0)
  st = _lib.load().b200_device_status(ctypes.byref(word))
  if st != 0:
    raise RuntimeError(f"device status word {word.value:#x}: a kernel wait expired, the numbers are void")
  if not torch.isfinite(out.float()).all():
    raise RuntimeError("non-finite attention output")

  if rank == 0:
    peak_burst, peak_sustained, peak_src = load_peaks()
    achieved = flops_rank / (ms_step * 1e-3) / 1e12   # per GPU, per launch: one kernel per step
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": B * world, "heads": H, "seq_len": S, "head_dim": D,
                   "parallelism": f"batch x head sharded over {world} GPU(s), no collective",
                   "l2": "q,k,v,out = 537 MB per GPU, larger than the 126 MB L2",
                   "us_per_core_module": ms_step * 1e3, "e2e_steps": args.e2e_steps},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_burst, "unit": "TFLOP/s",
                     "frac": achieved / peak_burst, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     "peak_source": f"{peak_src} (cuBLAS bf16 burst; sustained {peak_sustained})",
                     "frac_of_datasheet_2250": achieved / 2250.0},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": 3 * q.numel() * 2,
                "d2h_bytes_per_step": q.numel() * 2, "ms_per_step": e2e_ms},
        "gpu_launches": args.steps,
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
      tf, cores, sample = cpu_reference_sample(budget_s=15.0)
      line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)

  if world > 1:
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
