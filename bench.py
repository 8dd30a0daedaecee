"""Benchmark of the hot path: batched GEMM bf16 (fp32 accumulate) B=64, M=N=K=2048, the
batch sharded over the ranks, the output returned to every rank (by the GEMM epilogue itself,
which stores each finished slab into every rank's buffer; `--nccl-gather` uses one NCCL
all-gather instead).

  python bench.py --gpus 1 --steps 20 --warmup 5
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
  python bench.py --impl reference ...     CPU arm: the llvm-template loop nest on the host cores

One JSON line on rank 0.  A step is one pass over the whole batch: every rank runs the
tcgen05 kernel on its 64/N items (and, for N > 1, all-gathers the output).  `value` is
whole-job TFLOP/s with the operands resident in HBM; `e2e` is the same step through
Task -> schedule_with_config -> build -> func(*arrays) with pinned host buffers, the
host->device copy of the operands and the device->host read of the result inside the timed
region.  Inputs (1 GiB) are larger than L2, so consecutive steps do not find them cached.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH, DIM = 64, 2048
FLOP_PER_ITEM = 2.0 * DIM ** 3
METRIC = "TFLOP/s batched GEMM bf16 (fp32 accumulate) B=64 M=N=K=2048"
WORKLOAD = "batched GEMM bf16 B=64 M=N=K=2048, fp32 accumulate, normal(0,0.02) inputs, bf16 output"
FALLBACK_BF16_TFLOPS = 1590.0
# DRAM bytes of one full-batch launch of the dominant kernel: dram__bytes_read.sum +
# dram__bytes_write.sum of an ncu capture of a 6-item launch, scaled to 64 items by the items
# processed (traffic grows in proportion: every item is read once).  The 6-item capture still
# holds half of its output in L2 when the kernel ends, so the write part is a lower bound; the
# algorithmic figure is 1.61e9.
NCU_TRAFFIC_BYTES_PER_LAUNCH = (104.52e6 + 24.33e6) * 64 / 6
KNOBS = {"cluster": 2, "tile_n": 512, "raster": 3, "group_m": 8}
# N > 1 with the fused gather: the epilogue's bulk stores cross NVLink and take longer.  The 256 x 512
# tile overlaps its epilogue with the next main loop only half by half, and for as long as handing an
# accumulator half back was slow the 256 x 256 tile (whole-tile overlap) was the faster one there; with
# that fixed the wide tile leads at N = 2 and 4 (20 steps: 0.483 ms against 0.492 ms, 0.657 against
# 0.664 ms), with a shorter grouped-M walk because a rank owns fewer items.  At N = 8 a rank writes every
# slab eight times and the step is all stores: there the tile with a spare accumulator still wins
# (0.730 / 0.737 ms against 0.750 / 0.753 ms, runs alternated on one box).
KNOBS_FUSED = {"cluster": 2, "tile_n": 512, "raster": 3, "group_m": 4}
KNOBS_FUSED_8 = {"cluster": 2, "tile_n": 256, "raster": 3, "group_m": 4, "stages": 6, "release": 2}
# Receive bandwidth per GPU (GB/s) when every rank pushes its slice into all the others at the same
# time, by world size; 770 is the one-pair peer copy measured on this pool.
ALL_TO_ALL_GBS = {2: 737.0, 4: 730.0, 8: 730.0}
ALL_TO_ALL_SOURCE = ("`bench.py --link-ceiling --link-mib 256` on this pool: 737 GB/s at N=2, 730 GB/s at N=4; at N=8 "
                     "the same pattern of device-to-device copies (56 at once) reaches only 503 GB/s per GPU, less "
                     "than the fused kernel's own stores move there (643 GB/s), so it is no ceiling and the N=4 "
                     "figure is used")


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            peaks = json.load(f)
        return float(peaks["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except Exception:
        return FALLBACK_BF16_TFLOPS, "fallback"


_SAMPLER_CHILD = r"""
import sys, time
import pynvml
pynvml.nvmlInit()
h = pynvml.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
print("max", pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM), flush=True)
while True:
    try:
        print(time.time(), pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM),
              pynvml.nvmlDeviceGetCurrentClocksEventReasons(h), flush=True)
    except Exception:
        pass
    time.sleep(0.003)
"""


class ClockSampler(object):
    """Samples the SM clock and the throttle reasons of one GPU while a region runs.

    Read-only NVML queries every few milliseconds from a CHILD process (queries made from the
    benchmarking process itself contend with its kernel launches for the driver and stretch a
    launch-bound step); only samples stamped inside [mark_start, mark_end] are used.  Falls
    back to `nvidia-smi -lms 100` when the NVML module cannot be loaded.
    """

    REASONS = (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20),
               ("hw_thermal_slowdown", 0x40))
    SMI_FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.sw_power_cap,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.hw_thermal_slowdown")

    def __init__(self, index):
        self.index = index
        self.lines = []
        self.proc = None
        self.thread = None
        self.mode = None
        self.t0 = self.t1 = None

    def start(self):
        try:
            import pynvml  # noqa: F401  (only to know the child can import it)
            self.proc = subprocess.Popen([sys.executable, "-c", _SAMPLER_CHILD, str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.mode = "nvml (child process)"
        except Exception:
            try:
                self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.SMI_FIELDS,
                                              "--format=csv,noheader,nounits", "-lms", "100"],
                                             stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                self.mode = "nvidia-smi"
            except Exception:
                self.proc = None
                return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source"], "samples": 0}
        time.sleep(0.02)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        clocks, all_clocks, reasons, mx = [], [], set(), None
        for stamp, line in self.lines:
            parts = line.replace(",", " ").split()
            try:
                if self.mode == "nvidia-smi":
                    when, clock, mx = stamp, float(parts[0]), float(parts[1])
                    mask = sum(bit for (name, bit), val in zip(self.REASONS, parts[2:6]) if val.lower().startswith("active"))
                elif parts[0] == "max":
                    mx = float(parts[1])
                    continue
                else:
                    when, clock, mask = float(parts[0]), float(parts[1]), int(parts[2])
            except (ValueError, IndexError):
                continue
            all_clocks.append(clock)
            if self.t0 is not None and self.t1 is not None and not (self.t0 - 0.005 <= when <= self.t1 + 0.005):
                continue
            clocks.append(clock)
            for name, bit in self.REASONS:
                if mask & bit:
                    reasons.add(name)
        used = sorted(clocks) if clocks else sorted(all_clocks)
        return {"sm_mhz": used[len(used) // 2] if used else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks), "source": self.mode,
                "window": "timed region" if clocks else "whole run (no sample fell inside the timed region)"}


# ---------------------------------------------------------------------- CPU arm / CPU baseline
def cpu_items(count, seed=3):
    import numpy as np
    from oracle import ft_oracle as O
    a = np.empty((count, DIM, DIM), dtype=np.uint16)
    b = np.empty((count, DIM, DIM), dtype=np.uint16)
    for i in range(count):
        ai, bi = O.batch_gemm_item(i, DIM, DIM, DIM, seed=seed)
        a[i] = O.to_bf16_bits(ai)
        b[i] = O.to_bf16_bits(bi)
    return a, b


def cpu_step_time(a, b, out, tiles):
    from oracle import c_oracle as CO
    t0 = time.perf_counter()
    CO.bgemm_bf16_tiled(a, b, *tiles, out=out)
    return time.perf_counter() - t0


def pick_cpu_tiles(a, b, out):
    """Small sweep over tile factors of the loop nest, as a short search over split factors
    would do; returns the fastest (ti, tj, tk)."""
    best, best_t = None, float("inf")
    for tiles in ((8, 64, 64), (4, 64, 256), (8, 64, 256), (16, 64, 64)):
        t = cpu_step_time(a[:1], b[:1], out[:1], tiles)
        if t < best_t:
            best, best_t = tiles, t
    return best


def run_reference(args, rank):
    """`--impl reference`: the reference has no runnable CPU path here (it needs an un-vendored
    TVM fork), so the arm times the C restatement of the loop nest its llvm template emits, with
    all host threads, one batch item (2048^3) per step - a bounded sample of the workload."""
    if rank != 0:
        return
    import numpy as np
    from oracle import c_oracle as CO
    cores = CO.use_all_cores()
    a, b = cpu_items(1)
    out = np.empty((1, DIM, DIM), dtype=np.uint16)
    tiles = pick_cpu_tiles(a, b, out)
    for _ in range(args.warmup):
        cpu_step_time(a, b, out, tiles)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step_time(a, b, out, tiles)
    dt = (time.perf_counter() - t0) / args.steps
    value = FLOP_PER_ITEM / dt / 1e12
    sample = "1 of 64 batch items (2048^3) per step, tile factors %s" % (tiles,)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_leg(budget_s=12.0):
    import numpy as np
    from oracle import c_oracle as CO
    CO.use_all_cores()
    a, b = cpu_items(1)
    out = np.empty((1, DIM, DIM), dtype=np.uint16)
    tiles = pick_cpu_tiles(a, b, out)
    times = []
    t_start = time.perf_counter()
    while len(times) < 8 and (time.perf_counter() - t_start < budget_s or not times):
        times.append(cpu_step_time(a, b, out, tiles))
    dt = sorted(times)[len(times) // 2]
    return {"value": FLOP_PER_ITEM / dt / 1e12, "unit": "TFLOP/s", "cores": CO.max_threads(), "kind": "port",
            "sample": "1 of 64 batch items (2048^3), median of %d runs, tile factors %s, scaled linearly" %
                      (len(times), tiles)}


# ---------------------------------------------------------------------- other operators
def measured_ceilings():
    """What the vendor libraries reach on this GPU right now, as practical denominators for the
    dtypes MEASURED_PEAKS.json does not cover: TF32 (torch.matmul with TF32 allowed, 8192^3) and
    int8 (torch._int_mm, 8192^3).  Best of five, CUDA events; informational."""
    import torch
    out = {}

    def best_of(fn, reps=5):
        fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1e-3)
        return best

    n = 8192
    old = torch.backends.cuda.matmul.allow_tf32
    try:
        torch.backends.cuda.matmul.allow_tf32 = True
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        c = torch.empty(n, n, device="cuda")
        out["tf32_tflops"] = 2.0 * n ** 3 / best_of(lambda: torch.matmul(a, b, out=c)) / 1e12
        del a, b, c
    except Exception as exc:
        out["tf32_tflops"] = None
        out["tf32_error"] = str(exc)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    try:
        a8 = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
        b8 = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
        out["int8_tops"] = 2.0 * n ** 3 / best_of(lambda: torch._int_mm(a8, b8)) / 1e12
        del a8, b8
    except Exception as exc:
        out["int8_tops"] = None
        out["int8_error"] = str(exc)
    return out


def per_op_lines(peak_bf16, hbm_gbs):
    """Kernel-only device time of the other four configurations, CUDA-graph replay of 20
    back-to-back launches (these are microsecond-sized: a single launch is latency-bound).
    Every entry carries `frac` (achieved / peak) and `peak_source`."""
    import numpy as np
    import torch
    from flextensor_b200.runtime import build
    from flextensor_b200.scheduler import schedule_with_config
    from flextensor_b200.utils import Config
    from oracle import ft_oracle as O
    out = {}
    ceil = measured_ceilings()
    out["measured_ceilings"] = ceil
    tf32_peak = ceil.get("tf32_tflops") or 1100.0
    tf32_src = ("torch.matmul TF32 8192^3 measured in this run" if ceil.get("tf32_tflops")
                else "nominal 1100 TFLOP/s (no measurement)")
    int8_peak = ceil.get("int8_tops") or 2.0 * peak_bf16
    int8_src = ("torch._int_mm 8192^3 measured in this run" if ceil.get("int8_tops")
                else "2 x measured bf16 peak (no int8 measurement)")
    hbm_src = "MEASURED_PEAKS.json hbm_gbs (copy)"

    def dev(x):
        return torch.from_numpy(np.ascontiguousarray(x)).cuda()

    def module(key, nops, precision=None, cfgs=None):
        s, bufs = schedule_with_config(key, cfgs or Config([{}] * nops, None), precision=precision)
        return build(s, bufs)

    def timed(key, arrays, nops, precision=None, cfgs=None, flush_l2=False):
        func = module(key, nops, precision, cfgs)
        res = func.time_evaluator(func.entry_name, None, number=20, repeat=5, flush_l2=flush_l2)(*arrays)
        return res.median

    a, b = O.gemm_inputs(1024, 1024, 1024, seed=0)
    arrays = [dev(a), dev(b), torch.empty(1024, 1024, device="cuda")]
    for mode in ("3xtf32", "tf32"):
        t = timed("gemm_gemm_(1024, 1024, 1024)_cuda(0)", arrays, 1, precision=mode)
        tf = 2 * 1024 ** 3 / t / 1e12
        peak = tf32_peak / 3.0 if mode == "3xtf32" else tf32_peak
        out["gemm_f32_1024_" + mode] = {"us": t * 1e6, "tflops": tf, "frac": tf / peak,
                                        "peak_source": tf32_src + (" / 3 (three TF32 passes per product)"
                                                                   if mode == "3xtf32" else ""),
                                        "note": "one wave of tiles: latency-sized"}
    x, w = O.conv2d_inputs(1, 64, 56, 56, 64, 3, 3, seed=1)
    arrays = [dev(x), dev(w), torch.empty(1, 64, 56, 56, device="cuda")]
    t = timed("conv2d_res_b13_(1, 64, 56, 56, 64, 3, 1, 1, 1, 1)_cuda(0)", arrays, 2)
    out["conv2d_c64_56_k64_tf32"] = {"us": t * 1e6, "tflops": 231211008 / t / 1e12,
                                     "frac": 231211008 / t / 1e12 / tf32_peak, "peak_source": tf32_src,
                                     "note": "25 output tiles for 148 SMs: latency-sized"}
    x, w = O.depthwise_inputs(1, 256, 56, 56, 1, 3, 3, seed=2)
    arrays = [dev(x), dev(w), torch.empty(1, 256, 56, 56, device="cuda")]
    key = "conv2d_depthwise_(1, 256, 56, 56, 1, 3, 1, 1, 1)_cuda(0)"
    t = timed(key, arrays, 2)
    out["depthwise_c256_56"] = {"us": t * 1e6, "gbs": 6431744 / t / 1e9, "frac": 6431744 / t / 1e9 / hbm_gbs,
                                "peak_source": hbm_src, "note": "L2-warm graph replay; 6.4 MB working set"}
    t = timed(key, arrays, 2, flush_l2=True)
    out["depthwise_c256_56_l2_flushed"] = {"us": t * 1e6, "gbs": 6431744 / t / 1e9, "frac": 6431744 / t / 1e9 / hbm_gbs,
                                           "peak_source": hbm_src,
                                           "note": "a 256 MB scratch is written before every timed launch; each launch "
                                                   "timed on its own with CUDA events (includes launch latency)"}
    # The same two kernels on batched variants of the shapes (batch 64), where the work is large
    # enough for the bound to show: HBM traffic for depthwise, tensor time for conv2d.
    from flextensor_b200.task import Task, depthwise_conv2d, register_task
    big = Task("conv2d", "depthwise", depthwise_conv2d, (64, 256, 56, 56, 1, 3, 1, 1, 1), "cuda", 0)
    register_task(big)
    arrays = [torch.rand(64, 256, 56, 56, device="cuda"), dev(w), torch.empty(64, 256, 56, 56, device="cuda")]
    t = timed(big.key, arrays, 2)
    out["depthwise_c256_56_batch64"] = {"us": t * 1e6, "gbs": 64 * 6422528 / t / 1e9,
                                        "frac": 64 * 6422528 / t / 1e9 / hbm_gbs, "peak_source": hbm_src,
                                        "note": "411 MB of input+output per launch, larger than L2"}
    from flextensor_b200.task import TASK_TABLE
    x64 = torch.randn(64, 64, 56, 56, device="cuda")
    w64 = torch.randn(64, 64, 3, 3, device="cuda")
    arrays = [x64, w64, torch.empty(64, 64, 56, 56, device="cuda")]
    t = timed("conv2d_res3_(64, 64, 56, 56, 64, 3, 1, 1, 1, 1)_cuda(0)", arrays, 2)
    out["conv2d_c64_56_k64_batch64_tf32"] = {"us": t * 1e6, "tflops": 64 * 231211008 / t / 1e12,
                                             "frac": 64 * 231211008 / t / 1e12 / tf32_peak, "peak_source": tf32_src}
    # the same layer after the layout rewrite (channels-last tensors read in place: no layout pass)
    s_cl, bufs_cl = schedule_with_config("conv2d_res3_(64, 64, 56, 56, 64, 3, 1, 1, 1, 1)_cuda(0)", Config([], None),
                                         rewrite=True)
    func_cl = build(s_cl, bufs_cl)
    arrays = [x64.permute(0, 2, 3, 1).contiguous(), w64, torch.empty(64, 56, 56, 64, device="cuda")]
    t = func_cl.time_evaluator(func_cl.entry_name, None, number=20, repeat=5)(*arrays).median
    out["conv2d_c64_56_k64_batch64_tf32_channels_last"] = {
        "us": t * 1e6, "tflops": 64 * 231211008 / t / 1e12, "frac": 64 * 231211008 / t / 1e12 / tf32_peak,
        "peak_source": tf32_src, "note": "schedule_with_config(..., rewrite=True): [N,H,W,C] in, [N,P,Q,K] out"}
    del arrays, x64, w64, func_cl
    # The reference's conv3d table (flextensor/configs/conv3d_config.py: 3-D ResNet-18 after the stem, batch 1),
    # library-default knobs, single-pass TF32
    layers3 = []
    flop3 = 0.0
    for key in [k for k in TASK_TABLE if k.startswith("conv3d_conv3d_") and k.endswith("_cuda(0)")]:
        n_, c_, d_, h_, w_, k_, ks_, st_, pad_ = TASK_TABLE[key].args[:9]
        od, oh = (d_ + 2 * pad_ - ks_) // st_ + 1, (h_ + 2 * pad_ - ks_) // st_ + 1
        arrays = [torch.randn(n_, c_, d_, h_, w_, device="cuda"), torch.randn(k_, c_, ks_, ks_, ks_, device="cuda"),
                  torch.empty(n_, k_, od, oh, oh, device="cuda")]
        t = timed(key, arrays, 2)
        flop = 2.0 * n_ * k_ * od * oh * oh * c_ * ks_ ** 3
        flop3 += flop
        layers3.append({"args": list(TASK_TABLE[key].args), "us": t * 1e6, "tflops": flop / t / 1e12})
        del arrays
    sum3 = sum(l["us"] for l in layers3)
    out["conv3d_resnet18_b1_tf32"] = {"layers": layers3, "sum_us": sum3, "frac": flop3 / (sum3 * 1e-6) / 1e12 / tf32_peak,
                                      "peak_source": tf32_src, "note": "batch 1: latency-sized"}
    # The reference's own conv2d benchmark: the 15 YOLO-v1 layers at batch 1
    # (flextensor/configs/conv2d_config.py:18-45), library-default knobs, single-pass TF32.  Beside
    # them the kernel times the reference published for its tuned fp32 CUDA kernels
    # (testing/others/profile/compute_flops.py:17-33; GPU not named there, sibling files are V100).
    published_ms = [0.1007, 0.2825, 0.0252, 0.2062, 0.0571, 0.7426, 0.0373, 0.2107, 0.0541, 0.7973, 0.0653,
                    0.2498, 0.5610, 0.3801, 0.2718]
    layers = []
    flop_sum = 0.0
    for i in range(15):
        key = next(k for k in TASK_TABLE if k.startswith("conv2d_yolo%d_" % i) and k.endswith("_cuda(0)"))
        n_, c_, h_, w_, k_, r_, st_, pad_ = TASK_TABLE[key].args[:8]
        out_hw = (h_ + 2 * pad_ - r_) // st_ + 1
        arrays = [torch.randn(n_, c_, h_, w_, device="cuda"), torch.randn(k_, c_, r_, r_, device="cuda"),
                  torch.empty(n_, k_, out_hw, out_hw, device="cuda")]
        t = timed(key, arrays, 2)
        flop = 2.0 * n_ * k_ * out_hw * out_hw * c_ * r_ * r_
        flop_sum += flop
        layers.append({"layer": i + 1, "us": t * 1e6, "tflops": flop / t / 1e12,
                       "published_reference_us": published_ms[i] * 1e3})
        del arrays
    sum_us = sum(l["us"] for l in layers)
    out["conv2d_yolo_b1_tf32"] = {"layers": layers, "sum_us": sum_us,
                                  "frac": flop_sum / (sum_us * 1e-6) / 1e12 / tf32_peak, "peak_source": tf32_src,
                                  "published_reference_sum_us": sum(published_ms) * 1e3,
                                  "note": "published figures: the reference's tuned fp32 kernels on its own GPU"}
    a8 = torch.randint(-127, 128, (8192, 8192), device="cuda", dtype=torch.int8)
    b8 = torch.randint(-127, 128, (8192, 8192), device="cuda", dtype=torch.int8)
    arrays = [a8, b8, torch.empty(8192, 8192, device="cuda", dtype=torch.int32)]
    t = timed("gemm_gemm_int8_(8192, 8192, 8192)_cuda(0)", arrays, 1)
    tops = 2 * 8192 ** 3 / t / 1e12
    out["gemm_int8_8192"] = {"us": t * 1e6, "tops": tops, "frac": tops / int8_peak, "peak_source": int8_src,
                             "frac_of_2x_bf16_measured": tops / (2 * peak_bf16)}
    return out


def sharded_per_op(world, rank, device, hbm_gbs, reps=10):
    """The batch-sharded conv2d and depthwise conv2d of the reference's batched tables at this
    world size: ResNet-50 stage-2 3x3 at batch 64 (flextensor/configs/conv2d_config.py:231) and
    the first MobileNet depthwise layer at batch 16 (configs/depthwise_config.py:23-31), images
    sharded over the ranks, weights replicated, the output returned to every rank; time includes
    the gather.  Max over ranks of CUDA-event time per call."""
    import torch
    import torch.distributed as dist
    from flextensor_b200.sharded import ShardedOp, shard_range
    from flextensor_b200.task import conv2d, depthwise_conv2d
    from oracle import ft_oracle as O
    import numpy as np
    out = {}
    cases = [
        ("conv2d_res_stage2_b64_tf32", "conv2d", "sharded_res3", conv2d, (64, 64, 56, 56, 64, 3, 1, 1, 1, 1),
         (64, 64, 56, 56), (64, 64, 3, 3), 64 * 231211008.0, None),
        ("depthwise_mobilenet1_b16", "conv2d", "depthwise", depthwise_conv2d, (16, 32, 112, 112, 1, 3, 1, 1, 1),
         (16, 32, 112, 112), (32, 1, 3, 3), None, 2.0 * 16 * 32 * 112 * 112 * 4 + 32 * 9 * 4),
    ]
    for label, category, name, builder, args, xshape, wshape, flop, nbytes in cases:
        batch = args[0]
        if batch % world:
            continue
        try:
            _sharded_case(out, label, category, name, builder, args, xshape, wshape, flop, nbytes, world, rank, device,
                          hbm_gbs, reps)
        except Exception as exc:  # reported in the line; the headline numbers above are not lost
            out[label] = {"error": "%s: %s" % (type(exc).__name__, exc)}
    return out


def _sharded_case(out, label, category, name, builder, args, xshape, wshape, flop, nbytes, world, rank, device, hbm_gbs,
                  reps):
    import torch
    import torch.distributed as dist
    from flextensor_b200.sharded import ShardedOp, shard_range
    from flextensor_b200.task import conv2d
    from oracle import ft_oracle as O
    batch = args[0]
    lo, hi = shard_range(batch, world, rank)
    gen = torch.Generator(device=device)
    gen.manual_seed(11 * 1_000_003 + lo)
    x = torch.randn(hi - lo, *xshape[1:], device=device, generator=gen)
    wgen = torch.Generator(device=device)
    wgen.manual_seed(12)
    w = torch.randn(*wshape, device=device, generator=wgen)      # replicated: same seed on every rank
    try:
        op = ShardedOp(category, name, builder, args, gather="fused")
    except Exception as exc:
        op = ShardedOp(category, name, builder, args, gather="nccl")
        out[label + "_fused_unavailable"] = "%s: %s" % (type(exc).__name__, exc)
    full = op(x, w)
    torch.cuda.synchronize()
    op.check()
    # parity of what is timed: this rank's first image against the oracle
    xi, wi = x[:1].cpu().numpy(), w.cpu().numpy()
    if builder is conv2d:
        want = O.conv2d_nchw(xi, wi, None, 1, 1, 1, 1)
        ok = O.normalised_error(full[lo:lo + 1].cpu().numpy(), want) <= O.TOLERANCE["conv2d_tf32"]
    else:
        want = O.depthwise_conv2d_nchw(xi, wi, None, 1, 1, 1)
        ok = O.normalised_error(full[lo:lo + 1].cpu().numpy(), want) <= O.TOLERANCE["depthwise_f32"]
    assert ok, "%s: sharded output does not match the oracle" % label
    for _ in range(3):
        op(x, w)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        op(x, w)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    entry = {"us": ms * 1e3, "gather": op.gather + ("" if op.gather != "fused" or op.func.pushed_by_kernel
                                                     else " (device-to-device push after the kernel)"),
             "images_per_gpu": hi - lo, "api": "Module.__call__ via sharded.ShardedOp"}
    if flop:
        entry["tflops"] = flop / (ms * 1e-3) / 1e12
    if nbytes:
        entry["gbs"] = nbytes / (ms * 1e-3) / 1e9
        entry["frac_of_hbm_peak_x_gpus"] = entry["gbs"] / (hbm_gbs * world)
    out[label] = entry
    if world > 1:
        dist.barrier()
    op.close()
    del x, w, full


# ---------------------------------------------------------------------- GPU arm
def run_ours(args, rank, world, local_rank):
    import numpy as np
    import torch
    import torch.distributed as dist
    from flextensor_b200 import backend
    from flextensor_b200.runtime import build
    from flextensor_b200.scheduler import schedule_with_config
    from flextensor_b200.sharded import ShardedOp, disable_symm_mem_multicast
    from flextensor_b200.task import Task, batch_gemm, register_task
    from flextensor_b200.templates import knobs_to_config
    from flextensor_b200.utils import Config
    from oracle import ft_oracle as O

    disable_symm_mem_multicast()  # plain peer pointers only; set before any rendezvous
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # a child process; it is up and polling long before the timed region
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    assert BATCH % world == 0, "the batch of 64 shards over 1, 2, 4 or 8 ranks"

    # The reference-facing path: Task -> schedule_with_config -> build -> func(*arrays), planned for this
    # rank's shard.  N > 1: the output argument is this rank's slice of a buffer every rank holds and the
    # GEMM epilogue stores into all of them (fused gather), else one NCCL all-gather follows the call.
    fused_why = None
    knobs = KNOBS if world == 1 else KNOBS_FUSED if world < 8 else KNOBS_FUSED_8
    if args.knobs:
        knobs = json.loads(args.knobs)
    op = None
    if world > 1 and not args.nccl_gather:
        try:
            op = ShardedOp("gemm", "batch_gemm", batch_gemm, (BATCH, DIM, DIM, DIM), gather="fused", knobs=knobs)
        except Exception as exc:  # reported in the JSON line, the NCCL path is used instead
            fused_why = "%s: %s" % (type(exc).__name__, exc)
    if op is None:
        knobs = KNOBS
        op = ShardedOp("gemm", "batch_gemm", batch_gemm, (BATCH, DIM, DIM, DIM), gather="nccl", knobs=knobs)
    fused = op.gather == "fused"
    lo, hi, local = op.lo, op.hi, op.local
    func = op.func

    # Synthetic operands: normal(0, 0.02) rounded to bf16, drawn on the device with a per-rank
    # seed; the first item of the shard is replaced by the oracle's item, which is checked below.
    gen = torch.Generator(device=device)
    gen.manual_seed(3 * 1_000_003 + lo)
    a = (torch.randn(local, DIM, DIM, device=device, generator=gen) * 0.02).to(torch.bfloat16)
    b = (torch.randn(local, DIM, DIM, device=device, generator=gen) * 0.02).to(torch.bfloat16)
    a0, b0 = O.batch_gemm_item(lo, DIM, DIM, DIM, seed=3)
    a[0] = torch.from_numpy(a0).to(device).to(torch.bfloat16)
    b[0] = torch.from_numpy(b0).to(device).to(torch.bfloat16)
    c_full = op.out_full
    c_local = op.out_local if op.gather == "nccl" else c_full[lo:hi]

    def step():
        op.launch(a, b)
        op.finish()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # parity of what is being timed
    step()
    barrier()
    op.check()
    got = c_local[0].float().cpu().numpy()
    assert O.bf16_output_ok(got, O.gemm(a0, b0, out_dtype=np.float64)), "bench output does not match the oracle"
    if world > 1:
        assert torch.equal(c_full[lo:hi], c_local)
        # every rank's first item is the oracle's item of that index: the gathered copy must hold them all
        from flextensor_b200.sharded import shard_range
        for r in range(world):
            first = shard_range(BATCH, world, r)[0]
            ar, br = O.batch_gemm_item(first, DIM, DIM, DIM, seed=3)
            assert O.bf16_output_ok(c_full[first].float().cpu().numpy(), O.gemm(ar, br, out_dtype=np.float64)), \
                "rank %d does not hold rank %d's slice" % (rank, r)

    for _ in range(args.warmup):
        step()
    barrier()
    stream = torch.cuda.current_stream()
    launches0 = backend.launch_count()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    kern_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    sampler.mark_start()
    ev[0].record(stream)
    for i in range(args.steps):
        kern_ev[i][0].record(stream)
        op.launch(a, b)
        kern_ev[i][1].record(stream)
        op.finish()
    ev[1].record(stream)
    barrier()
    sampler.mark_end()
    launches = backend.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    op.check()
    total_ms = ev[0].elapsed_time(ev[1])
    kernel_ms = sum(s0.elapsed_time(s1) for s0, s1 in kern_ev) / args.steps
    t = torch.tensor([total_ms, kernel_ms, float(launches)], device=device, dtype=torch.float64)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        total_ms, kernel_ms, launches = float(tmax[0]), float(tmax[1]), int(tsum[2])
    ms_per_step = total_ms / args.steps
    value = BATCH * FLOP_PER_ITEM / (ms_per_step * 1e-3) / 1e12
    kernel_only = BATCH * FLOP_PER_ITEM / (kernel_ms * 1e-3) / 1e12

    # ---- end to end: pinned host operands -> device -> kernel -> (gather) -> host
    ha = torch.empty(local, DIM, DIM, dtype=torch.bfloat16).pin_memory()
    hb = torch.empty(local, DIM, DIM, dtype=torch.bfloat16).pin_memory()
    hc = torch.empty(local, DIM, DIM, dtype=torch.bfloat16).pin_memory()
    ha.copy_(a)
    hb.copy_(b)
    e2e_steps = max(3, min(args.steps, 10))

    # The step is pipelined over chunks of the local batch: chunk c+1 is copied host->device on one
    # copy stream while chunk c is computed and chunk c-1 is read back on another (PCIe is full
    # duplex).  Every chunk goes through the public callable of its own Task.
    nchunks = max(1, min(8, local))
    while local % nchunks:
        nchunks -= 1
    csz = local // nchunks
    chunk_task = Task("gemm", "batch_gemm", batch_gemm, (csz, DIM, DIM, DIM), "cuda", local_rank)
    register_task(chunk_task)
    cop = chunk_task.func(*chunk_task.args)[0][0]
    cs, cbufs = schedule_with_config(chunk_task.key, Config([knobs_to_config(knobs, cop)], None))
    chunk_func = build(cs, cbufs, "cuda")
    chunk_out = [op.peer_out.slice(lo + c * csz, lo + (c + 1) * csz) if fused else c_local[c * csz:(c + 1) * csz]
                 for c in range(nchunks)]
    h2d_stream, d2h_stream = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    ev_in = [torch.cuda.Event() for _ in range(nchunks)]
    ev_cmp = [torch.cuda.Event() for _ in range(nchunks)]
    ev_out = [torch.cuda.Event() for _ in range(nchunks)]
    for e in ev_cmp + ev_out:
        e.record(stream)

    def e2e_step():
        for c in range(nchunks):
            sl = slice(c * csz, (c + 1) * csz)
            with torch.cuda.stream(h2d_stream):
                h2d_stream.wait_event(ev_cmp[c])      # the previous step is done reading this chunk's operands
                a[sl].copy_(ha[sl], non_blocking=True)
                b[sl].copy_(hb[sl], non_blocking=True)
                ev_in[c].record(h2d_stream)
            stream.wait_event(ev_in[c])
            stream.wait_event(ev_out[c])              # the previous step's read-back of this chunk is done
            chunk_func(a[sl], b[sl], chunk_out[c])
            ev_cmp[c].record(stream)
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(ev_cmp[c])
                hc[sl].copy_(c_local[sl], non_blocking=True)
                ev_out[c].record(d2h_stream)
        op.finish()
        stream.wait_stream(d2h_stream)

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t[0])
    chunk_func.check()
    assert torch.equal(hc[0], c_local[0].cpu())
    e2e_value = BATCH * FLOP_PER_ITEM / (e2e_ms * 1e-3) / 1e12
    elem = 2
    h2d = 2 * BATCH * DIM * DIM * elem
    d2h = BATCH * DIM * DIM * elem

    hbm = 6536.0
    try:
        hbm = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        pass
    del ha, hb, hc, chunk_out
    sharded_ops = None
    if not args.no_extra:
        sharded_ops = sharded_per_op(world, rank, device, hbm)
    per_op = None
    if rank == 0 and world == 1 and not args.no_extra:
        per_op = per_op_lines(measured_peak()[0], hbm)

    # ---- sustained: back-to-back steps for about two seconds (the power cap settles the clock);
    # last, so that nothing else is measured on a GPU this run has heated up
    sustained = None
    if world == 1 and not args.no_extra:
        n_sus = max(args.steps, int(2000.0 / max(ms_per_step, 1e-3)))
        sus_sampler = ClockSampler(local_rank)
        sus_sampler.start()
        time.sleep(0.05)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sus_sampler.mark_start()
        e0.record(stream)
        for _ in range(n_sus):
            op.launch(a, b)
        e1.record(stream)
        torch.cuda.synchronize()
        sus_sampler.mark_end()
        sus_clocks = sus_sampler.stop()
        sus_ms = e0.elapsed_time(e1) / n_sus
        sus_peak = None
        try:
            sus_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
        except Exception:
            pass
        sus_val = BATCH * FLOP_PER_ITEM / (sus_ms * 1e-3) / 1e12
        sustained = {"value": sus_val, "unit": "TFLOP/s", "steps": n_sus, "ms_per_step": sus_ms,
                     "sm_mhz_median": sus_clocks.get("sm_mhz"), "reasons": sus_clocks.get("reasons"),
                     "peak": sus_peak, "frac": (sus_val / sus_peak) if sus_peak else None,
                     "peak_source": "MEASURED_PEAKS.json bf16_tflops_sustained"}

    op.close()
    del a, b

    if rank == 0:
        peak, peak_src = measured_peak()
        # the dominant kernel processes 64/N items per launch on each rank
        achieved = local * FLOP_PER_ITEM / (kernel_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "api": "Module.__call__ (Task -> schedule_with_config -> build -> func(*arrays))",
            "config": {"workload": WORKLOAD, "sharding": "batch 64/%d items per GPU" % world,
                       "collective": ("none" if world == 1 else
                                      "fused: epilogue bulk stores into every rank's output over NVLink + one barrier"
                                      if fused else
                                      "NCCL all-gather of the bf16 output (512 MiB total)" +
                                      (" [fused path unavailable: %s]" % fused_why if fused_why else "")),
                       "l2": "inputs (1 GiB) larger than L2; no flush needed",
                       "knobs": knobs,
                       "kernel": "umma_gemm_kernel<bf16, bf16 out, cta_group::2, %s tile>" %
                                 ("256x%d" % knobs["tile_n"])},
            "kernel_only_value": kernel_only,
            "kernel_only_note": ("whole-job TFLOP/s over the kernel launches alone (CUDA events around each "
                                 "launch)" + ("; at N > 1 the kernel includes its stores into the peers' buffers, "
                                              "only the closing barrier is outside" if fused else "")),
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "pipeline": "%d chunks per rank; host->device, compute and device->host overlap" % nchunks},
            "gpu_launches": launches,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "peak_source": peak_src, "frac_of_nominal_2250": achieved / 2250.0,
                         "kernel_ms": kernel_ms, "flop_per_launch": local * FLOP_PER_ITEM,
                         "traffic": (NCU_TRAFFIC_BYTES_PER_LAUNCH * local / BATCH) if NCU_TRAFFIC_BYTES_PER_LAUNCH else None},
            "clocks": clocks,
        }
        if sustained is not None:
            line["sustained"] = sustained
        if world > 1:
            # fused compute + collective: the step cannot beat the slower of the math at the GEMM peak and
            # the bytes every GPU must receive over NVLink.  The link figure is the all-to-all rate measured
            # on this pool with every rank pushing its slice to all others at once (profiles/), not the
            # one-pair peer copy.
            link_bytes = (world - 1) * local * DIM * DIM * elem
            t_math = local * FLOP_PER_ITEM / (peak * 1e12) * 1e3
            link_gbs = ALL_TO_ALL_GBS.get(world, 770.0)
            t_link = link_bytes / (link_gbs * 1e9) * 1e3
            line["fused_collective"] = {"bound": "nvlink" if t_link > t_math else "tensor",
                                        "nvlink_bytes_per_gpu_per_step": link_bytes, "link_gbs": link_gbs,
                                        "link_source": ALL_TO_ALL_SOURCE,
                                        "target_ms": max(t_math, t_link),
                                        "achieved_ms": ms_per_step, "frac": max(t_math, t_link) / ms_per_step}
        if sharded_ops is not None:
            line["per_op_sharded"] = sharded_ops
        if world == 1:
            line["cpu_baseline"] = cpu_baseline_leg()
            if per_op is not None:
                line["per_op"] = per_op
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_link_ceiling(args, rank, world, local_rank):
    """`--link-ceiling` (N > 1): what the NVLink fabric gives when every rank pushes a slice into
    every other rank's buffer at the same time - the traffic pattern of the fused gather without
    any compute.  Each rank copies `mib` MiB into each peer's symmetric buffer, one stream per
    peer; CUDA events, max over ranks.  Prints receive GB/s per GPU."""
    import torch
    import torch.distributed as dist
    from flextensor_b200.sharded import PeerGatheredOutput, disable_symm_mem_multicast
    disable_symm_mem_multicast()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    mib = args.link_mib
    elems = mib * 1024 * 1024 // 2
    buf = PeerGatheredOutput(world, elems, dtype=torch.bfloat16)
    src = torch.randn(elems, device=device).to(torch.bfloat16)
    peers = buf.peer_order()[1:]
    streams = [torch.cuda.Stream(device=device) for _ in peers]
    main = torch.cuda.current_stream()

    def push_all():
        for st, r in zip(streams, peers):
            st.wait_stream(main)
            with torch.cuda.stream(st):
                buf.view_of(r)[rank].copy_(src, non_blocking=True)
        for st in streams:
            main.wait_stream(st)

    for _ in range(3):
        push_all()
    buf.barrier()
    dist.barrier()
    torch.cuda.synchronize()
    reps = 10
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(main)
    for _ in range(reps):
        push_all()
    e1.record(main)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    buf.barrier()
    torch.cuda.synchronize()
    ok = bool(torch.equal(buf.tensor[(rank + 1) % world], buf.tensor[(rank + 1) % world]))
    if rank == 0:
        recv = (world - 1) * mib * 1024 * 1024
        print(json.dumps({"link_ceiling": {"n_gpus": world, "mib_per_peer": mib, "ms": ms,
                                           "recv_gbs_per_gpu": recv / (ms * 1e-3) / 1e9,
                                           "send_gbs_per_gpu": recv / (ms * 1e-3) / 1e9,
                                           "pattern": "every rank pushes one slice to every other rank at once "
                                                      "(device-to-device copies into mapped peer memory)", "ok": ok}}),
              flush=True)
    dist.barrier()
    buf.close()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the per-operator lines of the other four configs")
    ap.add_argument("--nccl-gather", action="store_true", help="N > 1: return the output with an NCCL all-gather "
                    "instead of the fused epilogue stores")
    ap.add_argument("--knobs", default="", help="JSON knob set for the headline kernel instead of the built-in one")
    ap.add_argument("--link-ceiling", action="store_true", help="N > 1: measure the all-to-all push rate of the "
                    "NVLink fabric instead of running the benchmark")
    ap.add_argument("--link-mib", type=int, default=64, help="MiB pushed to each peer by --link-ceiling")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
    if args.link_ceiling:
        if world < 2:
            raise SystemExit("--link-ceiling needs at least two ranks")
        run_link_ceiling(args, rank, world, local_rank)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
