"""Benchmark of the RG-LRU + Conv1D path at the 2B-dims prefill workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("cfg1"): the RG-LRU + Conv1D sub-path of RecurrentBlock prefill at RecurrentGemma-2B
dimensions - batch 8, 4096 tokens, lru_width 2560, 10 heads, conv width 4, bfloat16 activations and
parameters, float32 scan state, single segment per row.  A step is one pass of
out = RGLRU(Conv1D(xb)) * gelu(yb) over that batch (xb, yb = the outputs of linear_x / linear_y,
synthetic N(0,1)); `value` is tokens/s with inputs resident in HBM, `e2e` the same through the
public API with pinned host buffers (host->device and device->host copies inside the timed
region).  With N > 1 (torchrun, one process per GPU) every rank runs the whole workload on its own
GPU - the path shards by batch without any collective - and `value` is the sum (weak scaling).

`--impl reference` times the CPU restatement of the reference's own implementation of the same
sub-path (oracle/, OpenMP over all host cores) on the same workload, K steps after W warm-ups.

The default line also carries the other workloads as extra keys, each a few hundred milliseconds:
`long_scan` (RG-LRU at 9B dims, batch 4 x 65536 tokens, heads sharded over the N ranks, with and
without the all_gather that reassembles the output), `decode_step` (26 decode layers, batch 256)
and `rglru_fp32` (the float32 RG-LRU layer); `--headline-only` skips them.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "rglru_conv1d_prefill_tokens_per_s"
UNIT = "tokens/s"
CFG1 = dict(batch=8, seq=4096, lru_width=2560, heads=10, conv_width=4)


def _peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      d = json.load(f)
    return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
  return 6650.0, 1590.0, "fallback"


def _workload_name(cfg):
  return (f"cfg1: RG-LRU+Conv1D sub-path of RecurrentBlock prefill, B{cfg['batch']} T{cfg['seq']} "
          f"E{cfg['lru_width']} H{cfg['heads']} W{cfg['conv_width']} bf16 (fp32 scan state)")


# ------------------------------------------------------------------------------------------------
# synthetic inputs (seeded; shapes and distributions of the workload)
# ------------------------------------------------------------------------------------------------
def make_params(cfg, device, seed):
  g = torch.Generator(device="cpu").manual_seed(seed)
  e, h, w = cfg["lru_width"], cfg["heads"], cfg["conv_width"]
  bw = e // h
  dt = torch.bfloat16

  def n(shape, std):
    return (torch.randn(shape, generator=g) * std).to(dt).to(device)

  u = torch.rand((e,), generator=g).double() * (0.999 ** 2 - 0.9 ** 2) + 0.9 ** 2
  a_param = torch.log(torch.expm1(-0.5 * torch.log(u))).float().to(dt).to(device)
  return {
      "conv_1d.w": n((w, e), math.sqrt(1.0 / w)), "conv_1d.b": torch.zeros(e, dtype=dt, device=device),
      "rg_lru.a_param": a_param,
      "rg_lru.input_gate.w": n((h, bw, bw), math.sqrt(1.0 / bw)),
      "rg_lru.input_gate.b": torch.zeros((h, bw), dtype=dt, device=device),
      "rg_lru.a_gate.w": n((h, bw, bw), math.sqrt(1.0 / bw)),
      "rg_lru.a_gate.b": torch.zeros((h, bw), dtype=dt, device=device),
  }


def make_activations(cfg, device, seed, batch=None):
  b = batch or cfg["batch"]
  g = torch.Generator(device="cpu").manual_seed(seed + 1)
  shape = (b, cfg["seq"], cfg["lru_width"])
  xb = torch.randn(shape, generator=g).to(torch.bfloat16)
  yb = torch.randn(shape, generator=g).to(torch.bfloat16)
  pos = torch.arange(cfg["seq"], dtype=torch.int64).repeat(b, 1)
  if device != "cpu":
    return xb.pin_memory(), yb.pin_memory(), pos.to(device)
  return xb, yb, pos


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
  FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
            "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
            "clocks_event_reasons.sw_power_cap")

  def __init__(self, index: int):
    self.index = index
    self.proc = None
    self.path = f"/tmp/rgk_clocks_{os.getpid()}.csv"

  def start(self):
    try:
      self.out = open(self.path, "w")
      self.proc = subprocess.Popen(
          ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms",
           "20", "-i", str(self.index)], stdout=self.out, stderr=subprocess.DEVNULL)
    except OSError:
      self.proc = None

  def stop(self):
    res = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    if self.proc is None:
      return res
    time.sleep(0.12)
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
    self.out.close()
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    try:
      with open(self.path) as f:
        for line in f:
          parts = [p.strip() for p in line.split(",")]
          if len(parts) < 7:
            continue
          try:
            sm.append(float(parts[0])); mx.append(float(parts[1]))
          except ValueError:
            continue
          for nme, val in zip(names, parts[3:7]):
            if val == "Active":
              reasons.add(nme)
      os.remove(self.path)
    except OSError:
      pass
    if sm:
      res.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons),
                 samples=len(sm))
    return res


# ------------------------------------------------------------------------------------------------
# CPU legs (the oracle: the reference's algorithm restated in C, OpenMP over the host cores)
# ------------------------------------------------------------------------------------------------
def cpu_leg(cfg, steps, warmup, seed=1, gpu_out=None):
  """Times oracle.recurrent_path on the WHOLE workload (all batch rows) with every host core, and
  the linear scan alone in both reference forms (torch rnn_scan, JAX lru_linear_scan restated).
  gpu_out: the CUDA path's output on the same inputs (CPU tensor) - the oracle then also serves as
  the checker, and the leg reports the error and the share of elements whose bits differ."""
  from oracle import oracle
  oracle.lib()
  threads = oracle.set_threads(os.cpu_count() or 1)     # a launcher may have exported OMP_NUM_THREADS=1
  torch.set_num_threads(max(1, os.cpu_count() or 1))
  p = make_params(cfg, "cpu", seed)
  op = oracle.params_of(p)
  xb, yb, pos = make_activations(cfg, "cpu", seed)
  times = []
  out = None
  for i in range(warmup + steps):
    t0 = time.perf_counter()
    out, _, _ = oracle.recurrent_path(xb, yb, pos, op)
    if i >= warmup:
      times.append(time.perf_counter() - t0)
  tokens = cfg["batch"] * cfg["seq"]
  mean = sum(times) / len(times)
  leg = {
      "value": tokens / mean, "best": tokens / min(times), "unit": UNIT, "cores": threads,
      "kind": "port",
      "sample": (f"oracle/rglru_oracle.c recurrent_path (OpenMP, {threads} threads of "
                 f"{os.cpu_count()} host cores) on the whole workload: {cfg['batch']} batch rows x "
                 f"{cfg['seq']} tokens x {cfg['lru_width']} channels, mean of {steps} after {warmup} "
                 f"warm-up"),
      "seconds_per_sample": mean,
  }
  # The recurrence alone, h_t = a_t h_{t-1} + x_t over the same [B, T, E] shape, in the torch
  # reference's form (rnn_scan, torch/layers.py:140-191) and in the JAX reference's
  # (lru_linear_scan, jax/scan.py:74-120), both restated in C: jax itself is not installed.
  g = torch.Generator(device="cpu").manual_seed(seed + 7)
  a = (torch.rand(xb.shape, generator=g) * 0.4 + 0.6).to(xb.dtype)
  no_reset = torch.zeros(xb.shape[:2], dtype=torch.bool)
  scan = {}
  for name, fn in (("torch_rnn_scan_restatement", lambda: oracle.rnn_scan(xb, a, no_reset, None)),
                   ("jax_linear_scan_restatement", lambda: oracle.jax_linear_scan(xb, a, None))):
    fn()
    t0 = time.perf_counter()
    fn()
    scan[name] = tokens / (time.perf_counter() - t0)
  scan["unit"] = UNIT
  scan["note"] = ("the recurrence alone on [B, T, E] bfloat16 inputs; the JAX figure is a C restatement of "
                  "lru_linear_scan, the genuine JAX scan is unavailable on this box (jax is not installed)")
  leg["linear_scan_only"] = scan
  if gpu_out is not None:
    o, r = gpu_out.float(), out.float()
    leg["parity"] = {
        "what": "CUDA path output against the oracle on the whole workload",
        "normalised_max_error": float((o - r).abs().max() / r.abs().max().clamp_min(1e-30)),
        "tolerance": 2e-2,
        "fraction_of_elements_differing": float((gpu_out != out).float().mean()),
    }
  return leg


def run_reference(args, cfg):
  rank = int(os.environ.get("RANK", "0"))
  if rank != 0:
    return
  steps, warmup = max(1, args.steps), max(0, args.warmup)
  leg = cpu_leg(cfg, steps, warmup)
  line = {
      "impl": "reference", "metric": METRIC, "value": leg["value"], "unit": UNIT,
      "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
      "ms_per_step": leg["seconds_per_sample"] * 1e3, "higher_is_better": True, "scaling": "weak",
      "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
      "config": {"workload": _workload_name(cfg), "step": leg["sample"]},
      "cpu_baseline": {k: leg[k] for k in ("value", "unit", "cores", "kind", "sample",
                                            "linear_scan_only")},
      "e2e": {"value": leg["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
              "d2h_bytes_per_step": 0},
  }
  print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def _time_loop(fn, steps, stream):
  ev0 = torch.cuda.Event(enable_timing=True)
  ev1 = torch.cuda.Event(enable_timing=True)
  ev0.record(stream)
  for _ in range(steps):
    fn()
  ev1.record(stream)
  ev1.synchronize()
  return ev0.elapsed_time(ev1) / steps  # ms per call


def run_gpu(args, cfg):
  import torch.distributed as dist
  import recurrentgemma_b200 as rg
  from recurrentgemma_b200 import _lib

  rank = int(os.environ.get("RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  local = int(os.environ.get("LOCAL_RANK", "0"))
  if world != args.gpus:
    if world == 1 and args.gpus > 1:
      raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run, one rank per GPU")
  torch.cuda.set_device(local)
  dev = torch.device("cuda", local)
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)
  lib = _lib.load()
  _lib.check(lib.rgk_device_check())

  b, t, e, h = cfg["batch"], cfg["seq"], cfg["lru_width"], cfg["heads"]
  dt = torch.bfloat16
  p = make_params(cfg, dev, 1 + rank)
  conv = rg.Conv1D(e, 4, device=dev, dtype=dt)
  conv.load_state_dict({"w": p["conv_1d.w"], "b": p["conv_1d.b"]})
  lru = rg.RGLRU(e, h, device=dev, dtype=dt)
  lru.load_state_dict({k[len("rg_lru."):]: v for k, v in p.items() if k.startswith("rg_lru.")})
  xb_h, yb_h, pos = make_activations(cfg, dev, 1 + rank)
  xb, yb = xb_h.to(dev), yb_h.to(dev)
  out = torch.empty_like(xb)
  out_h = torch.empty_like(xb_h).pin_memory()
  stream = torch.cuda.current_stream(dev)

  def step():
    rg.recurrent_path(xb, yb, pos, conv, lru, out=out)

  from recurrentgemma_b200 import host
  pipe = host.HostPipeline(conv, lru, t, rows_per_group=1, device=dev)

  def step_e2e():
    # public host-buffer API: batch rows streamed through copy-in / compute / copy-out streams
    h_state, _ = pipe(xb_h, yb_h, pos, out_h)
    h_state[:1, :1].cpu()      # the step's state read back

  for _ in range(max(args.warmup, 3)):
    step()
  torch.cuda.synchronize()
  _lib.workspace_status(_lib.workspace(dev, 1))
  # A step is `passes` back-to-back passes of the path over the batch, so that the timed region of
  # K steps lasts at least a quarter of a second whatever K is.
  est_ms = _time_loop(step, 5, stream)
  passes = max(1, int(math.ceil(250.0 / (max(args.steps, 1) * est_ms))))
  if world > 1:
    pt = torch.tensor([passes], device=dev)
    dist.all_reduce(pt, op=dist.ReduceOp.MAX)
    passes = int(pt.item())

  def timed_step():
    for _ in range(passes):
      step()

  clocks = ClockSampler(local)
  if rank == 0:
    clocks.start()
  if world > 1:
    dist.barrier()
  torch.cuda.synchronize()
  ms = _time_loop(timed_step, args.steps, stream)
  torch.cuda.synchronize()
  _lib.workspace_status(_lib.workspace(dev, 1))
  if world > 1:
    tmax = torch.tensor([ms], device=dev)
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.barrier()
    ms = float(tmax.item())
  clk = clocks.stop() if rank == 0 else None
  ms_pass = ms / passes

  # end to end through the public API, host buffers
  e2e_ms = None
  if not args.no_e2e:
    e2e_steps = max(2, min(max(args.steps, 30), 60))
    for _ in range(2):
      step_e2e()
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
    t0 = time.perf_counter()
    ev_ms = _time_loop(step_e2e, e2e_steps, stream)
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    e2e_ms = max(ev_ms, wall_ms)
    if world > 1:
      tmax = torch.tensor([e2e_ms], device=dev)
      dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
      e2e_ms = float(tmax.item())

  # The long head-sharded scan: every rank takes part (heads split over the ranks).
  long_scan = None
  if not args.headline_only:
    del xb, yb, out
    torch.cuda.empty_cache()
    long_scan = long_scan_leg(dev, rank, world, steps=10, warmup=3)
    xb, yb = xb_h.to(dev), yb_h.to(dev)
    out = torch.empty_like(xb)
    step()

  # Per-kernel device times: each stage through its own C-ABI entry point on preallocated buffers,
  # CUDA events on the launch stream (torch's current stream is the stream the library is given).
  kernels = {}
  if rank == 0:
    import ctypes
    n_el = b * t * e
    es = 2
    ksteps = max(5, min(args.steps, 20))
    sp = stream.cuda_stream
    dtc = _lib.RGK_BF16
    c = torch.empty_like(xb)
    y2 = torch.empty_like(xb)
    h_last = torch.empty((b, e), dtype=torch.float32, device=dev)
    ws = _lib.workspace(dev, _lib.workspace_bytes(b, t, e, dt))
    prm = lru._params(conv)
    no_reset = torch.zeros((b, t), dtype=torch.uint8, device=dev)
    a_t = torch.rand((b, t, e), device=dev).mul_(0.4).add_(0.6).to(dt)

    def k_conv():
      _lib.check(lib.rgk_conv1d_prefill(xb.data_ptr(), pos.data_ptr(), _lib.RGK_I64,
                                        conv.w.data_ptr(), conv.b.data_ptr(), b, t, e, 4, dtc,
                                        c.data_ptr(), None, sp))

    def k_scan(mul):
      _lib.check(lib.rgk_linear_scan(c.data_ptr(), a_t.data_ptr(), no_reset.data_ptr(), None,
                                     yb.data_ptr() if mul else None, b, t, e, dtc, y2.data_ptr(),
                                     h_last.data_ptr(), ws.data_ptr(), ws.numel(), sp))

    def k_lru(impl):
      _lib.check(lib.rgk_rglru_forward(c.data_ptr(), pos.data_ptr(), _lib.RGK_I64,
                                       ctypes.byref(prm), None, b, t, e, h, dtc, impl,
                                       y2.data_ptr(), h_last.data_ptr(), ws.data_ptr(), ws.numel(),
                                       sp))

    def k_path():
      _lib.check(lib.rgk_recurrent_path_prefill(
          xb.data_ptr(), yb.data_ptr(), pos.data_ptr(), _lib.RGK_I64, ctypes.byref(prm), None, b, t,
          e, h, 4, dtc, lru.gates_impl, y2.data_ptr(), h_last.data_ptr(), None, ws.data_ptr(),
          ws.numel(), sp))

    for fn in (k_conv, lambda: k_scan(True), lambda: k_scan(False),
               lambda: k_lru(_lib.GATES_TCGEN05), k_path):
      fn()
    torch.cuda.synchronize()
    gw = p["rg_lru.input_gate.w"].numel() * es
    gate_flops = 2 * 2 * b * t * e * (e // h)
    t_conv = _time_loop(k_conv, ksteps, stream)
    t_path = _time_loop(k_path, ksteps, stream)
    kernels["conv1d_prefill"] = {"ms": t_conv, "bytes": 2 * n_el * es, "flops": 8 * n_el}
    # The rest of the step is ONE kernel: gate projections (tcgen05) + gate arithmetic + scan + join.
    # Its algorithmic bytes: conv output and y branch in, joined output out, gate weights.
    kernels["rglru_fused"] = {"ms": max(t_path - t_conv, 1e-6), "bytes": 3 * n_el * es + 2 * gw,
                              "flops": gate_flops + 20 * n_el}
    # For comparison, the two-kernel route the library takes when T is not a multiple of 128.
    t_scan = _time_loop(lambda: k_scan(True), ksteps, stream)
    t_lru_tc = _time_loop(lambda: k_lru(_lib.GATES_TCGEN05), ksteps, stream)
    t_scan_plain = _time_loop(lambda: k_scan(False), ksteps, stream)
    two_kernel = {"gates_tc_ms": max(t_lru_tc - t_scan_plain, 1e-6), "scan_join_ms": t_scan,
                  "gates_tc_GB/s": (3 * n_el * es + 2 * gw) / max(t_lru_tc - t_scan_plain, 1e-6) / 1e6,
                  "scan_join_GB/s": 4 * n_el * es / t_scan / 1e6}
    # And the route with the Conv1D inside the RG-LRU kernel (rgk_set_conv_fusion): one kernel, no
    # conv output in HBM, the same bits; timed for the record, it is the slower one.
    lib.rgk_set_conv_fusion(1)
    try:
      k_path()
      torch.cuda.synchronize()
      two_kernel["conv_fused_in_one_kernel_ms"] = _time_loop(k_path, ksteps, stream)
    finally:
      lib.rgk_set_conv_fusion(0)
    del a_t, c, y2

    # The whole RecurrentBlock at the same shapes: the three projections on the
    # tcgen05 GEMM around the sub-path, one library call.
    gb = torch.Generator(device="cpu").manual_seed(77)
    blk = rg.RecurrentBlock(e, h, e, device=dev, dtype=dt)
    sd = dict(p)
    for nm in ("linear_y", "linear_x", "linear_out"):
      sd[nm + ".weight"] = (torch.randn((e, e), generator=gb) * math.sqrt(1.0 / e)).to(dt).to(dev)
      sd[nm + ".bias"] = torch.zeros(e, dtype=dt, device=dev)
    blk.load_state_dict(sd)
    x_in = torch.randn((b, t, e), generator=gb).to(dt).to(dev)
    for _ in range(2):
      blk(x_in, pos)
    torch.cuda.synchronize()
    t_blk = _time_loop(lambda: blk(x_in, pos), ksteps, stream)
    t_lin = _time_loop(lambda: rg.dense_linear(x_in, sd["linear_x.weight"], sd["linear_x.bias"]),
                       ksteps, stream)
    block_info = {"ms": t_blk, "tokens_per_s": b * t / (t_blk * 1e-3),
                  "linear_ms": t_lin, "linear_TFLOP/s": 2 * b * t * e * e / (t_lin * 1e-3) / 1e12,
                  "what": "RecurrentBlock.forward prefill, same shapes, projections on the tcgen05 GEMM"}
    # One step further out: recurrent_block(temporal_pre_norm(x)) + x, the temporal half of the
    # reference's ResidualBlock, as one library call (RMSNorm kernel; residual in linear_out's
    # epilogue), and the RMSNorm kernel alone against its HBM roofline (read x, write x).
    norm = rg.RMSNorm(e, device=dev, dtype=dt)
    norm.load_state_dict({"scale": (torch.randn(e, generator=gb) * 0.3).to(dt).to(dev)})
    for _ in range(2):
      rg.recurrent_residual(x_in, pos, norm, blk)
    torch.cuda.synchronize()
    t_res = _time_loop(lambda: rg.recurrent_residual(x_in, pos, norm, blk), ksteps, stream)
    t_norm = _time_loop(lambda: norm(x_in), ksteps, stream)
    block_info["residual_ms"] = t_res
    block_info["rmsnorm_ms"] = t_norm
    block_info["rmsnorm_GB/s"] = 2 * b * t * e * 2 / (t_norm * 1e-3) / 1e9
    # ... and the channel half: mlp_block(channel_pre_norm(r)) + r with the 2B model's expanded
    # width, i.e. the whole residual block of the recurrent kind.
    xw = 3 * e
    mlp = rg.MLPBlock(e, xw, device=dev, dtype=dt)
    mlp.load_state_dict({
        "ffw_up.w": (torch.randn((2, e, xw), generator=gb) * math.sqrt(1.0 / e)).to(dt).to(dev),
        "ffw_up.b": torch.zeros((2, 1, 1, xw), dtype=dt, device=dev),
        "ffw_down.weight": (torch.randn((e, xw), generator=gb) * math.sqrt(1.0 / xw)).to(dt).to(dev),
        "ffw_down.bias": torch.zeros(e, dtype=dt, device=dev)})
    for _ in range(2):
      rg.residual_block(x_in, pos, norm, blk, norm, mlp)
    torch.cuda.synchronize()
    t_mlp = _time_loop(lambda: mlp(x_in, pre_norm=norm), ksteps, stream)
    t_full = _time_loop(lambda: rg.residual_block(x_in, pos, norm, blk, norm, mlp), ksteps, stream)
    block_info["mlp_channel_ms"] = t_mlp
    block_info["mlp_TFLOP/s"] = 6 * b * t * e * xw / (t_mlp * 1e-3) / 1e12
    block_info["residual_block_ms"] = t_full
    block_info["residual_block_tokens_per_s"] = b * t / (t_full * 1e-3)
    # The other temporal block of the model: local (sliding-window, multi-query) attention with the
    # 2B model's geometry (10 heads of 256, window 2048): the block, its attention kernel alone
    # (rotary embedding done), and the residual block of the attention kind.
    heads, hd, window = 10, 256, 2048
    att = rg.LocalAttentionBlock(e, heads, window, device=dev, dtype=dt)
    att.load_state_dict({
        "proj_q.weight": (torch.randn((e, e), generator=gb) * math.sqrt(1.0 / e)).to(dt).to(dev),
        "proj_k.weight": (torch.randn((hd, e), generator=gb) * math.sqrt(1.0 / e)).to(dt).to(dev),
        "proj_v.weight": (torch.randn((hd, e), generator=gb) * math.sqrt(1.0 / e)).to(dt).to(dev),
        "proj_final.weight": (torch.randn((e, e), generator=gb) * math.sqrt(1.0 / e)).to(dt).to(dev),
        "proj_final.bias": torch.zeros(e, dtype=dt, device=dev)})
    q = torch.randn((b, t, heads, hd), generator=gb).to(dt).to(dev)
    k = torch.randn((b, t, hd), generator=gb).to(dt).to(dev)
    v = torch.randn((b, t, hd), generator=gb).to(dt).to(dev)
    enc = torch.empty((b, t, heads * hd), dtype=dt, device=dev)
    aws = _lib.workspace(dev, int(lib.rgk_attention_workspace_bytes(b, t)))
    pos_i32 = 1 if pos.dtype == torch.int64 else 0

    def k_attn():
      _lib.check(lib.rgk_local_attention_prefill(
          q.data_ptr(), k.data_ptr(), v.data_ptr(), pos.data_ptr(), pos_i32, b, t, heads, hd,
          window, 1, enc.data_ptr(), aws.data_ptr(), aws.numel(), sp))

    for _ in range(2):
      rg.residual_block(x_in, pos, norm, att, norm, mlp)
      k_attn()
    torch.cuda.synchronize()
    t_att = _time_loop(lambda: att(x_in, pos), ksteps, stream)
    t_core = _time_loop(k_attn, ksteps, stream)
    t_full_att = _time_loop(lambda: rg.residual_block(x_in, pos, norm, att, norm, mlp), ksteps,
                            stream)
    # 4 * head_dim flops per visible (query, key) pair; the kernel computes the logits twice
    # (two-pass softmax), so its tensor work is 6 * head_dim per pair of every touched tile
    pairs = b * heads * sum(min(i, window) + 1 for i in range(t))
    block_info["attention"] = {
        "what": "LocalAttentionBlock.forward prefill, 10 heads x 256, window 2048, same B and T",
        "block_ms": t_att, "kernel_ms": t_core,
        "kernel_useful_TFLOP/s": pairs * 4 * hd / (t_core * 1e-3) / 1e12,
        "residual_block_ms": t_full_att,
        "residual_block_tokens_per_s": b * t / (t_full_att * 1e-3)}
    del blk, x_in, norm, mlp, att, q, k, v, enc
  if rank != 0:
    if world > 1:
      dist.destroy_process_group()
    return

  hbm_gbs, bf16_tf, which = _peaks()
  block_info["linear_frac_of_bf16_peak"] = block_info["linear_TFLOP/s"] / bf16_tf
  tokens = b * t
  value = world * tokens * passes / (ms * 1e-3)
  for k in kernels.values():
    k["gbs"] = k["bytes"] / (k["ms"] * 1e-3) / 1e9
    k["tflops"] = k["flops"] / (k["ms"] * 1e-3) / 1e12
  dom_name = max(kernels, key=lambda k: kernels[k]["ms"])
  dom = kernels[dom_name]
  path_bytes = 3 * b * t * e * 2 + 2 * p["rg_lru.input_gate.w"].numel() * 2
  sfu_ops = 5.5     # per element: tanh (input gate), ex2 + half a rcp (recurrence gate), ex2, sqrt, tanh (gelu)
  roofline = {
      "bound": "hbm", "kernel": dom_name, "achieved": dom["gbs"], "peak": hbm_gbs, "unit": "GB/s",
      "frac": dom["gbs"] / hbm_gbs, "peak_source": which,
      "traffic": _recorded_traffic(dom_name) if cfg["batch"] == CFG1["batch"] else None,
      "algorithmic_bytes": dom["bytes"],
      "path": {"algorithmic_bytes": path_bytes, "achieved": path_bytes / (ms_pass * 1e-3) / 1e9,
               "frac": path_bytes / (ms_pass * 1e-3) / 1e9 / hbm_gbs,
               "frac_of_nominal_8TBs": path_bytes / (ms_pass * 1e-3) / 1e9 / 8000.0},
      "kernels": {k: {"ms": round(v["ms"], 4), "GB/s": round(v["gbs"], 1),
                      "TFLOP/s": round(v["tflops"], 2)} for k, v in kernels.items()},
      "two_kernel_route": {k: round(v, 4) for k, v in two_kernel.items()},
      "sfu": {"ops_per_element": sfu_ops,
              "achieved_Gops": sfu_ops * b * t * e / (kernels["rglru_fused"]["ms"] * 1e-3) / 1e9,
              "peak_Gops": 148 * 16 * 1.965, "unit": "G special-function ops/s",
              "frac": (sfu_ops * b * t * e / (kernels["rglru_fused"]["ms"] * 1e-3) / 1e9) / (148 * 16 * 1.965)},
      "note": ("rglru_fused is bounded by instruction issue and the special-function pipe (about 55 "
               "instructions and 5.5 special-function operations per element), not by HBM; frac is "
               "its algorithmic bytes over its time against the measured copy bandwidth"),
  }
  cpu = None
  if not args.no_cpu:
    step()
    torch.cuda.synchronize()
    cpu = cpu_leg(cfg, 2, 1, seed=1 + rank, gpu_out=out.cpu())
  line = {
      "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
      "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
      "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
      "config": {"workload": _workload_name(cfg), "per_gpu_batch": b, "seq_len": t,
                 "passes_per_step": passes, "ms_per_pass": ms_pass,
                 "step": f"{passes} passes of the path over the batch (timed region {ms * args.steps / 1e3:.2f} s)",
                 "parallelism": f"batch-sharded x{world}, no collective",
                 "cache": "inputs (336 MB) larger than L2 (126 MB); no flush"},
      "roofline": roofline,
      "cpu_baseline": None if cpu is None else {k: cpu[k] for k in
                                                ("value", "unit", "cores", "kind", "sample",
                                                 "linear_scan_only", "parity")},
      "block_prefill": block_info,
      "clocks": clk,
      # per pass: the conv kernel, the per-channel constant kernel and the fused RG-LRU kernel
      "gpu_launches": 3 * passes * args.steps,
  }
  if long_scan is not None:
    line["long_scan"] = long_scan
  if not args.headline_only:
    line["decode_step"] = decode_leg(dev, steps=50)
    line["rglru_fp32"] = rglru_fp32_leg(dev, steps=50)
  if e2e_ms is not None:
    h2d = 2 * b * t * e * 2
    line["e2e"] = {"value": world * tokens / (e2e_ms * 1e-3), "unit": UNIT,
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": b * t * e * 2 + b * e * 4,
                   "ms_per_step": e2e_ms, "steps": e2e_steps,
                   # both copy directions overlap; the larger one, host to device, sets the time
                   "bound": "pcie_h2d", "h2d_GB/s_per_gpu": h2d / (e2e_ms * 1e-3) / 1e9}
  print(json.dumps(line), flush=True)
  if world > 1:
    dist.destroy_process_group()


def _recorded_traffic(kernel: str):
  """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of a kernel at the
  headline workload, from the record of ncu captures kept beside the summaries - but only if the
  kernel's source file still has the checksum it had when the capture was made; else None."""
  path = os.path.join(ROOT, "profiles", "dram_traffic.json")
  try:
    with open(path) as f:
      rec = json.load(f).get(kernel)
    if rec is None:
      return None
    with open(os.path.join(ROOT, rec["source"]), "rb") as f:
      sha = hashlib.sha256(f.read()).hexdigest()
    return float(rec["dram_bytes_per_launch"]) if sha == rec["source_sha256"] else None
  except (OSError, KeyError, ValueError):
    return None


# ------------------------------------------------------------------------------------------------
# secondary workloads carried as extra keys of the default line
# ------------------------------------------------------------------------------------------------
def long_scan_leg(dev, rank, world, steps, warmup, seq=65536, gather=True, shard_of=0):
  """RG-LRU forward (gate projections + gate arithmetic + scan) at 9B dims: lru_width 4096, 16
  heads, batch 4, `seq` tokens, bfloat16, documents of geometric length (mean 2048).  Rank r owns
  heads [16 r / N, 16 (r+1) / N): strong scaling with no collective inside the path.  Timed twice:
  the path alone, and with the all_gather that reassembles the [B, T, E] output on every rank inside
  the timed region.  shard_of = N > 0 (single process): time what ONE of N GPUs would run, with no
  collective - for development on one GPU.  Returns the dictionary on rank 0, None elsewhere."""
  import ctypes
  import torch.distributed as dist
  import recurrentgemma_b200 as rg
  from recurrentgemma_b200 import _lib, sharding, synthetic
  b, t, e, h = 4, seq, 4096, 16
  dt = torch.bfloat16
  if h % world != 0:
    return {"unavailable": f"16 heads do not split over {world} ranks"} if rank == 0 else None
  cfg = dict(batch=b, seq=t, lru_width=e, heads=h, conv_width=4)
  p = make_params(cfg, "cpu", 3)
  parts = shard_of if (shard_of and world == 1) else world
  h0, h1 = sharding.head_range(h, parts, rank)
  e_loc = (h1 - h0) * (e // h)
  pl = {k: v.to(dev) for k, v in sharding.shard_state_dict(p, e, h, parts, rank).items()}
  lru = rg.RGLRU(e_loc, h1 - h0, device=dev, dtype=dt)
  lru.load_state_dict({k[len("rg_lru."):]: v for k, v in pl.items() if k.startswith("rg_lru.")})
  gen = torch.Generator(device=dev).manual_seed(11 + rank)
  x = torch.randn((b, t, e_loc), generator=gen, device=dev, dtype=torch.float32).to(dt)
  pos = synthetic.geometric_segment_pos(b, t, 2048.0, 5).to(dev)
  y = torch.empty_like(x)
  full = torch.empty((world, b, t, e_loc), dtype=dt, device=dev) if world > 1 else None
  h_last = torch.empty((b, e_loc), dtype=torch.float32, device=dev)
  lib = _lib.load()
  ws = _lib.workspace(dev, _lib.workspace_bytes(b, t, e_loc, dt))
  prm = lru._params()
  stream = torch.cuda.current_stream(dev)

  def path():
    _lib.check(lib.rgk_rglru_forward(x.data_ptr(), pos.data_ptr(), _lib.RGK_I64, ctypes.byref(prm),
                                     None, b, t, e_loc, h1 - h0, _lib.RGK_BF16, lru.gates_impl,
                                     y.data_ptr(), h_last.data_ptr(), ws.data_ptr(), ws.numel(),
                                     stream.cuda_stream))

  def path_and_gather():
    path()
    if world > 1:
      dist.all_gather_into_tensor(full, y)     # [N, B, T, E/N]: slice r holds rank r's channels

  def timed(fn):
    for _ in range(warmup):
      fn()
    torch.cuda.synchronize()
    _lib.workspace_status(ws)
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()
    ms = _time_loop(fn, steps, stream)
    torch.cuda.synchronize()
    if world > 1:
      tmax = torch.tensor([ms], device=dev)
      dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
      ms = float(tmax.item())
    return ms

  ms_path = timed(path)
  ms_gather = timed(path_and_gather) if (gather and world > 1) else ms_path
  del x, y, full
  torch.cuda.empty_cache()
  if rank != 0:
    return None
  hbm, _, which = _peaks()
  alg = (2 * b * t * e * 2 + 2 * h * 256 * 256 * 2 + b * t * 8) / parts   # per GPU
  recv = (world - 1) * b * t * e_loc * 2                                   # bytes a rank receives
  return {
      "workload": f"cfg3: RG-LRU forward B{b} T{t} E{e} H{h} bf16, geometric documents (mean 2048), "
                  f"heads sharded x{parts}" + (" (one shard timed on one GPU)" if parts != world else ""),
      "scaling": "strong", "n_gpus": world, "steps": steps,
      "ms_per_step": ms_path, "tokens_per_s": b * t / (ms_path * 1e-3),
      "roofline": {"bound": "hbm", "algorithmic_bytes_per_gpu": alg,
                   "achieved": alg / (ms_path * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                   "frac": alg / (ms_path * 1e-3) / 1e9 / hbm, "peak_source": which},
      "with_gather": {
          "ms_per_step": ms_gather, "tokens_per_s": b * t / (ms_gather * 1e-3),
          "collective": "all_gather_into_tensor of the [B, T, E/N] outputs (NCCL), inside the timed region",
          "bytes_received_per_gpu": recv,
          # what the reassembly alone costs at the measured peer bandwidth of this pool (770 GB/s
          # per direction per GPU): the floor of this leg whatever the scan does
          "nvlink_floor_ms": recv / 770e9 * 1e3,
      },
  }


def rglru_fp32_leg(dev, steps):
  """The float32 RG-LRU layer (batch 2, 1024 tokens, lru_width 2560, 10 heads, document starts at 0
  and 512): microseconds per forward, against its HBM bound (x in, y out, gate weights) and against
  the gate contraction (three TF32 tensor-core products per float32 product) it is bound by."""
  import recurrentgemma_b200 as rg
  from recurrentgemma_b200 import synthetic
  b, t, e, h = 2, 1024, 2560, 10
  g = torch.Generator(device="cpu").manual_seed(0)
  p = synthetic.rglru_params(e, h, g, torch.float32)
  m = rg.RGLRU(e, h, device=dev, dtype=torch.float32)
  m.load_state_dict(p)
  x = torch.randn((b, t, e), generator=g).to(dev)
  pos = torch.arange(t, dtype=torch.int64)
  pos[512:] -= 512
  pos = pos.repeat(b, 1).to(dev)
  for _ in range(3):
    m(x, pos)
  torch.cuda.synchronize()
  ms = _time_loop(lambda: m(x, pos), steps, torch.cuda.current_stream(dev))
  hbm, _, which = _peaks()
  alg = 2 * b * t * e * 4 + 2 * h * 256 * 256 * 4
  flops = 2 * 2 * b * t * e * 256
  return {"workload": "cfg0: RGLRU.forward float32 B2 T1024 E2560 H10, resets at 0 and 512",
          "us_per_forward": ms * 1e3, "tokens_per_s": b * t / (ms * 1e-3),
          "roofline": {"bound": "hbm", "algorithmic_bytes": alg, "achieved": alg / (ms * 1e-3) / 1e9,
                       "peak": hbm, "unit": "GB/s", "frac": alg / (ms * 1e-3) / 1e9 / hbm,
                       "peak_source": which},
          "gate_contraction": {"flops": flops, "achieved_TFLOP/s": flops / (ms * 1e-3) / 1e12,
                               "note": "float32 products as three TF32 products on the tensor cores "
                                       "(hi/lo split of both operands, float32 accumulation); the "
                                       "figure counts each float32 multiply-add once"}}


# ------------------------------------------------------------------------------------------------
# cfg2: single-token decode step of the recurrent path through 26 layers (secondary workload)
# ------------------------------------------------------------------------------------------------
def decode_leg(dev, steps):
  """Per-step latency of 26 back-to-back RG-LRU + Conv1D decode steps at 2B dims (batch 256,
  lru_width 2560, 10 heads, bf16, cached conv window and fp32 state), layer i feeding layer i+1,
  replayed from a CUDA graph (one kernel per layer), and the same with the block's three dense
  projections around every step.  Returns the dictionary of results."""
  import recurrentgemma_b200 as rg
  from recurrentgemma_b200 import _lib, modules
  dt = torch.bfloat16
  b, e, h, n_layers = 256, CFG1["lru_width"], CFG1["heads"], 26
  layers = []
  for i in range(n_layers):
    p = make_params(CFG1, dev, 100 + i)
    conv = rg.Conv1D(e, 4, device=dev, dtype=dt)
    conv.load_state_dict({"w": p["conv_1d.w"], "b": p["conv_1d.b"]})
    lru = rg.RGLRU(e, h, device=dev, dtype=dt)
    lru.load_state_dict({k[len("rg_lru."):]: v for k, v in p.items() if k.startswith("rg_lru.")})
    g = torch.Generator(device="cpu").manual_seed(500 + i)
    cache = modules.RecurrentBlockCache(
        rg_lru_state=(torch.randn((b, e), generator=g) * 0.5).to(dev),
        conv1d_state=torch.randn((b, 3, e), generator=g).to(dt).to(dev))
    yb = torch.randn((b, 1, e), generator=g).to(dt).to(dev)
    layers.append((conv, lru, cache, yb))
  g = torch.Generator(device="cpu").manual_seed(7)
  x0 = torch.randn((b, 1, e), generator=g).to(dt).to(dev)
  pos = torch.randint(1, 4097, (b, 1), generator=g).to(dev)

  def step():
    x = x0
    for conv, lru, cache, yb in layers:
      x, _ = rg.recurrent_path(x, yb, pos, conv, lru, cache)
    return x

  for _ in range(3):
    step()
  torch.cuda.synchronize()
  t0 = time.perf_counter()
  for _ in range(steps):
    step()
  torch.cuda.synchronize()
  eager_ms = (time.perf_counter() - t0) * 1e3 / steps
  graph = torch.cuda.CUDAGraph()
  side = torch.cuda.Stream()
  with torch.cuda.stream(side):
    step()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph, stream=side):
      step()
  torch.cuda.synchronize()
  for _ in range(3):
    graph.replay()
  torch.cuda.synchronize()
  graph_ms = _time_loop(graph.replay, steps, torch.cuda.current_stream())

  # The full-RecurrentBlock variant of the same step: linear_x / linear_y / linear_out as library
  # GEMMs (M = batch is too small for the 128 x 256 tensor-core tiles) around the fused kernel,
  # 26 blocks captured in one CUDA graph.
  blocks = []
  for i, (conv, lru, cache, _) in enumerate(layers):
    blk = rg.RecurrentBlock(e, h, e, device=dev, dtype=dt)
    gb = torch.Generator(device="cpu").manual_seed(900 + i)
    sd = {"conv_1d.w": conv.w, "conv_1d.b": conv.b}
    sd.update({"rg_lru." + k: v for k, v in lru.state_dict().items()})
    for nm in ("linear_y", "linear_x", "linear_out"):
      sd[nm + ".weight"] = (torch.randn((e, e), generator=gb) * math.sqrt(1.0 / e)).to(dt).to(dev)
      sd[nm + ".bias"] = torch.zeros(e, dtype=dt, device=dev)
    blk.load_state_dict(sd)
    blocks.append((blk, cache))

  def block_step():
    x = x0
    for blk, cache in blocks:
      x, _ = blk(x, pos, cache)
    return x

  graph_b = torch.cuda.CUDAGraph()
  with torch.cuda.stream(side):
    block_step()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph_b, stream=side):
      block_step()
  torch.cuda.synchronize()
  for _ in range(3):
    graph_b.replay()
  torch.cuda.synchronize()
  block_ms = _time_loop(graph_b.replay, steps, torch.cuda.current_stream())

  # The same 26 blocks at a serving-sized batch (16 rows), where the projections are bound by
  # streaming their weights: on library GEMMs (SMALL_ROWS = 0) and on this library's few-row
  # tensor-core kernel (linear_y and linear_x in one launch), each as a CUDA graph.
  b_small = 16
  x_small, pos_small = x0[:b_small].contiguous(), pos[:b_small].contiguous()
  caches_small = [modules.RecurrentBlockCache(c.rg_lru_state[:b_small].clone(),
                                              c.conv1d_state[:b_small].clone()) for _, c in blocks]

  def small_step():
    x = x_small
    for (blk, _), cache in zip(blocks, caches_small):
      x, _ = blk(x, pos_small, cache)
    return x

  small_ms = {}
  rows_default = modules.SMALL_ROWS
  for name, rows in (("library_gemm", 0), ("few_row_kernel", max(rows_default, b_small))):
    modules.SMALL_ROWS = rows
    try:
      gs = torch.cuda.CUDAGraph()
      with torch.cuda.stream(side):
        small_step()
        torch.cuda.synchronize()
        with torch.cuda.graph(gs, stream=side):
          small_step()
      torch.cuda.synchronize()
      for _ in range(3):
        gs.replay()
      torch.cuda.synchronize()
      small_ms[name] = _time_loop(gs.replay, steps, torch.cuda.current_stream())
    finally:
      modules.SMALL_ROWS = rows_default
  _lib.check_status()
  small_bytes = n_layers * (3 * e * e * 2 + 2 * 256 * e * 2 + 2 * b_small * 3 * e * 2 +
                            2 * b_small * e * 4 + 6 * b_small * e * 2)

  block_bytes = n_layers * 3 * e * e * 2
  path_bytes = n_layers * (2 * b * e * 2 + b * e * 2 + 2 * b * 3 * e * 2 + 2 * b * e * 4 +
                           2 * 256 * e * 2)
  hbm, _, which = _peaks()
  return {
      "metric": "recurrent_path_decode_step_latency", "value": graph_ms, "unit": "ms",
      "higher_is_better": False, "n_gpus": 1, "steps": steps, "dtype": "bf16",
      "data": "synthetic",
      "config": {"workload": "cfg2: RG-LRU+Conv1D decode step x26 layers, B256 E2560 H10 bf16, "
                             "CUDA-graph replay, one fused kernel per layer"},
      "eager_python_ms": eager_ms, "tokens_per_s": b / (graph_ms * 1e-3),
      "full_block": {"ms": block_ms, "what": "RecurrentBlock.forward decode x26 (the three "
                     "projections around the fused kernel), CUDA-graph replay",
                     "algorithmic_bytes": path_bytes + block_bytes,
                     "GB/s": (path_bytes + block_bytes) / (block_ms * 1e-3) / 1e9,
                     "frac": (path_bytes + block_bytes) / (block_ms * 1e-3) / 1e9 / hbm},
      "full_block_b16": {"ms": small_ms["few_row_kernel"], "ms_library_gemm": small_ms["library_gemm"],
                         "what": "the same 26 blocks at batch 16: projections on the few-row "
                                 "tcgen05 kernel (linear_y | linear_x in one launch) against "
                                 "library GEMMs, CUDA-graph replay",
                         "algorithmic_bytes": small_bytes,
                         "GB/s": small_bytes / (small_ms["few_row_kernel"] * 1e-3) / 1e9,
                         "frac": small_bytes / (small_ms["few_row_kernel"] * 1e-3) / 1e9 / hbm},
      "roofline": {"bound": "hbm", "algorithmic_bytes": path_bytes,
                   "achieved": path_bytes / (graph_ms * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                   "frac": path_bytes / (graph_ms * 1e-3) / 1e9 / hbm, "peak_source": which},
      "gpu_launches": n_layers * steps}


def run_decode(args):
  dev = torch.device("cuda", 0)
  torch.cuda.set_device(dev)
  print(json.dumps(decode_leg(dev, args.steps)), flush=True)


# ------------------------------------------------------------------------------------------------
# cfg3: long-sequence RG-LRU at 9B dims, channels sharded by whole heads (secondary workload)
# ------------------------------------------------------------------------------------------------
def run_long_scan(args):
  """The long head-sharded scan alone (see long_scan_leg); one JSON line on rank 0."""
  import torch.distributed as dist
  rank = int(os.environ.get("RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  dev = torch.device("cuda", local)
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)
  leg = long_scan_leg(dev, rank, world, steps=args.steps, warmup=max(args.warmup, 3),
                      seq=args.seq or 65536, gather=True, shard_of=args.shard_of)
  if rank == 0:
    leg.update({"metric": "rglru_long_scan_tokens_per_s", "value": leg["tokens_per_s"],
                "unit": "tokens/s", "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                "gpu_launches": 3 * args.steps})
    print(json.dumps(leg), flush=True)
  if world > 1:
    dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# cfg4: the whole 2B model, prompt processing then greedy decoding (secondary workload)
# ------------------------------------------------------------------------------------------------
def run_griffin(args):
  """Griffin 2B with random weights (26 residual blocks: recurrent, recurrent, local attention;
  width 2560, 10 heads, MLP 7680, vocabulary 256000, bfloat16): 64 prompts of 2048 token ids drawn
  uniformly from a seed, then 512 greedy decode steps, through `GreedySampler` (prefill of all
  prompt tokens but the last, one step for the last, the decode step replayed as a CUDA graph,
  argmax on the device).  With N ranks (torchrun) the 64 sequences are split over the ranks
  (strong scaling, no collective).  A step is one whole generation.  Prints one JSON line."""
  import torch.distributed as dist
  import recurrentgemma_b200 as rg
  rank = int(os.environ.get("RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  dev = torch.device("cuda", local)
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)
  total_b, prompt, gen_steps = args.batch or 64, args.seq or 2048, args.gen_steps
  b = max(1, total_b // world)
  cfg = rg.GriffinConfig.recurrent_gemma_2b()
  torch.manual_seed(17)                        # the same weights on every rank
  model = rg.Griffin(cfg, device=dev, dtype=torch.bfloat16)
  g = torch.Generator(device="cpu").manual_seed(23 + rank)
  tokens_h = torch.randint(0, cfg.vocab_size, (b, prompt), generator=g, dtype=torch.int32).pin_memory()
  out_h = torch.empty((b, gen_steps), dtype=torch.int32).pin_memory()
  sampler = rg.GreedySampler(model)
  stream = torch.cuda.current_stream(dev)
  pos = torch.arange(prompt - 1, device=dev, dtype=torch.int32).repeat(b, 1)

  def generate():
    tokens = tokens_h.to(dev, non_blocking=True)
    out = sampler(tokens, gen_steps)
    out_h.copy_(out.tokens, non_blocking=True)

  def prefill():
    model(tokens_d[:, :-1], pos, None, return_logits=False, return_cache=True)

  for _ in range(max(1, min(args.warmup, 2))):
    generate()
  torch.cuda.synchronize()
  tokens_d = tokens_h.to(dev)
  steps = max(1, min(args.steps, 3))
  if world > 1:
    dist.barrier()
  torch.cuda.synchronize()
  sampler_clk = ClockSampler(local)
  if rank == 0:
    sampler_clk.start()
  ms = _time_loop(generate, steps, stream)
  torch.cuda.synchronize()
  clk = sampler_clk.stop() if rank == 0 else None
  ms_prefill = _time_loop(prefill, steps, stream)
  torch.cuda.synchronize()
  # one decode step alone: replays of the sampler's captured graph (state left by the last call)
  ms_replay = _time_loop(sampler._graph.replay, 100, stream) if sampler._graph is not None else None
  torch.cuda.synchronize()
  if world > 1:
    tmax = torch.tensor([ms, ms_prefill, ms_replay or 0.0], device=dev)
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms, ms_prefill, ms_replay = float(tmax[0].item()), float(tmax[1].item()), float(tmax[2].item())
  if rank == 0:
    n_tok = world * b * (prompt + gen_steps)
    decode_ms = ms_replay or (ms - ms_prefill) / gen_steps
    value = n_tok / (ms * 1e-3)
    params = sum(p.numel() for p in model.parameters())
    n_rec = sum(1 for t in cfg.block_types if t.name == "RECURRENT")
    n_att = len(cfg.block_types) - n_rec
    print(json.dumps({
        "metric": "griffin_2b_generation_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": max(1, min(args.warmup, 2)), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"cfg4: Griffin 2B random init, batch {world * b} (x{world} ranks), prompt "
                               f"{prompt} uniform token ids, {gen_steps} greedy decode steps",
                   "parameters": params, "per_gpu_batch": b,
                   "cache": "weights (5.4 GB) larger than L2; no flush"},
        "prefill": {"ms": ms_prefill, "tokens_per_s": world * b * (prompt - 1) / (ms_prefill * 1e-3)},
        "decode": {"ms_per_step": decode_ms, "tokens_per_s": world * b / (decode_ms * 1e-3),
                   "what": "100 replays of the captured step, event-timed",
                   "ms_per_step_in_generation": (ms - ms_prefill) / gen_steps,
                   # every step streams the weights once and the attention rings of 9 layers
                   "weight_GB/s": 2 * params / (decode_ms * 1e-3) / 1e9},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": b * prompt * 4,
                "d2h_bytes_per_step": b * gen_steps * 4,
                "note": "the timed region is the public call on pinned host token ids, copies included"},
        "clocks": clk,
        # this library's kernels per generation: a decode step launches 2 rmsnorm + geglu per block,
        # the fused recurrent step per recurrent block, 2 rope + 3 ring kernels per attention
        # block, the final rmsnorm, embed, logits and argmax; the prompt 8 per recurrent block
        # (2 rmsnorm, conv, RG-LRU, 4 GEMMs... ) and 12 per attention block, twice (prompt, last token)
        "gpu_launches": steps * (gen_steps * (3 * len(cfg.block_types) + n_rec + 5 * n_att + 4)
                                 + 2 * (9 * n_rec + 12 * n_att + 3))}), flush=True)
  if world > 1:
    dist.destroy_process_group()


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--workload", default="cfg1", choices=["cfg1", "cfg2", "cfg3", "cfg4"],
                  help="cfg1 (default, the headline prefill workload), cfg2 (decode step), cfg3 "
                       "(long head-sharded scan) or cfg4 (the whole 2B model: prompt + greedy decode)")
  ap.add_argument("--seq", type=int, default=None,
                  help="cfg3: sequence length (default 65536); cfg4: prompt length (default 2048)")
  ap.add_argument("--shard-of", type=int, default=0,
                  help="cfg3 on one GPU: time the shard one of this many GPUs would run (development)")
  ap.add_argument("--gen-steps", type=int, default=512, help="cfg4: greedy decode steps (default 512)")
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
  ap.add_argument("--batch", type=int, default=None, help="override the per-GPU batch (profiling)")
  ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
  ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
  ap.add_argument("--headline-only", action="store_true",
                  help="cfg1: skip the long_scan / decode_step / rglru_fp32 legs")
  args = ap.parse_args()
  cfg = dict(CFG1)
  if args.batch:
    cfg["batch"] = args.batch
  if args.workload == "cfg2":
    run_decode(args)
  elif args.workload == "cfg3":
    run_long_scan(args)
  elif args.workload == "cfg4":
    if args.impl == "reference":
      # the reference model lives in the recurrentgemma checkout, which a GPU box does not have,
      # and the scalar CPU restatement of a 2.7 B parameter model is not a bounded sample
      print(json.dumps({"impl": "reference", "unavailable":
                        "cfg4 needs the recurrentgemma checkout; only cfg1 has a timed CPU arm"}))
      return
    run_griffin(args)
  elif args.impl == "reference":
    run_reference(args, cfg)
  else:
    run_gpu(args, cfg)


if __name__ == "__main__":
  main()
