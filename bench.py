#!/usr/bin/env python
"""Benchmark of the frisk.gemm hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg5] [--impl reference]

One step = one pass of the GEMM over one batch of synthetic input.  The default workload is the
row-sharded bf16 GEMM (M=65536, N=K=8192): rank r of N computes rows [r*M/N, (r+1)*M/N) of C with
B replicated, no collective on the data path (strong scaling: the total work is fixed).  Rank 0
prints ONE JSON line: whole-job TFLOP/s with inputs resident in HBM (`value`), the same metric
through the host-buffer C-ABI call with the copies inside the timed region (`e2e`), the roofline
of the dominant kernel, the CPU baseline (the oracle port on the host cores) and, at N=1, the
other benchmark configurations under `other_configs`.  At N > 1 the line also carries every
rank's time and SM clock (`clocks_per_rank`, `clock_normalised`) and the all-gather of C measured
two ways (`allgather`: NCCL after the GEMM, and folded into the GEMM's epilogue).

`--impl reference` times the CPU restatement of the op (the reference has no GEMM implementation
of its own to run) on a bounded sample of the same workload, with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from frisk_b200 import workloads as W  # noqa: E402

FULL_DIMS = {
    "cfg1": (512, 512, 512), "cfg2": (4096, 4096, 4096), "cfg3": (16, 8192, 8192),
    "cfg4": (8192, 8192, 8192), "cfg5": (65536, 8192, 8192), "bf16_8192": (8192, 8192, 8192),
    "fp32_4096": (4096, 4096, 4096),   # cfg1's layout and distribution at a size the 3xTF32 plan takes
    "bf16_short_k": (8192, 8192, 256),  # cfg5's distributions with a short K: the epilogue is the kernel's time
    "bf16_deep_k": (512, 512, 65536),   # ... with four tiles of C against a deep K: the K-planes plan
}
AB_TYPE = {"cfg1": W.F32, "cfg2": W.F16, "cfg4": W.E4M3, "fp32_4096": W.F32}
C_TYPE = {"cfg1": W.F32, "cfg2": W.F16, "fp32_4096": W.F32}
TRANS_B = {"cfg2", "cfg4"}
BOUND = {"cfg3": "hbm", "bf16_short_k": "hbm", "bf16_deep_k": "hbm"}  # everything else is measured against the tensor-core peak
# DRAM bytes per launch of the dominant kernel (ncu: dram__bytes_read.sum + dram__bytes_write.sum
# of one captured launch, `--clock-control none`); None where no capture exists.
NCU_TRAFFIC_BYTES = {
    # CTA-pair kernel, bf16 8192^3, bands of 8 tile rows: 1060.3 MB read + 127.3 MB written
    "bf16_8192": 1187610032,
    # cfg5: see CFG5_SLAB_TRAFFIC below
    # few-row cluster plan, cfg3: 134.57 MB read + 4.01 MB written
    "cfg3": 138584832,
    # frisk.reduce, 8192 x 8192: read + written per step (the column reduce: both of its launches)
    "row_max_f16": 134233088 + 3560960,
    "row_sum_f32": 268450048 + 3368960,
    "col_min_f16": 134231040 + 3605248 + 1222144,
}
# cfg5's launch (2.1 GB resident, 6 ms) is beyond what a multi-pass capture should hold, so its
# DRAM traffic is measured on a slab of CFG5_SLAB_ROWS rows of the same problem (same B, same
# band walk) and scaled by the rows a rank holds: the bands are walked one after the other, each
# streaming all of B past its own rows of A, so the bytes grow in proportion to the rows.
CFG5_SLAB_ROWS = 16384
CFG5_SLAB_TRAFFIC = 2893966763   # mean of three captured launches: 2633.5 MB read + 260.5 MB written


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs.

    NVML is read directly from a thread every 2 ms (a timed region can be a few milliseconds long
    at 8 GPUs, far shorter than one round of `nvidia-smi`); when the NVML binding is missing the
    sampler falls back to an `nvidia-smi -lms` child process.  Reading only: no setting is touched.
    """

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, uuid=None):
        self.index, self.uuid = index, uuid
        self.proc = None
        self.lines: list[str] = []
        self.samples: list[tuple] = []   # (sm MHz, max MHz, reasons bit mask)
        self.nvml = None
        self._stop = threading.Event()
        self._thread = None

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        if self.uuid is not None:
            try:
                return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(self.uuid)).encode())
            except Exception:
                pass
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def start(self):
        try:
            self.nvml, handle = self._nvml_handle()
            mx = self.nvml.nvmlDeviceGetMaxClockInfo(handle, self.nvml.NVML_CLOCK_SM)
            # the first query of a kind can take tens of milliseconds: make it here, not in the loop
            self.nvml.nvmlDeviceGetClockInfo(handle, self.nvml.NVML_CLOCK_SM)
            self.nvml.nvmlDeviceGetCurrentClocksEventReasons(handle)

            def loop():
                while not self._stop.is_set():
                    try:
                        sm = self.nvml.nvmlDeviceGetClockInfo(handle, self.nvml.NVML_CLOCK_SM)
                        why = self.nvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                        self.samples.append((float(sm), float(mx), int(why)))
                    except Exception:
                        pass
                    time.sleep(0.002)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.nvml is not None:
            self._stop.set()
            self._thread.join(timeout=1.0)
            if not self.samples:
                return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
            n = self.nvml
            names = (("hw_slowdown", n.nvmlClocksEventReasonHwSlowdown),
                     ("hw_thermal_slowdown", n.nvmlClocksEventReasonHwThermalSlowdown),
                     ("sw_thermal_slowdown", n.nvmlClocksEventReasonSwThermalSlowdown),
                     ("sw_power_cap", n.nvmlClocksEventReasonSwPowerCap))
            mask = 0
            for _, _, why in self.samples:
                mask |= why
            sm = [x[0] for x in self.samples]
            busy = [x for x in sm if x > 0.5 * max(sm)] or sm
            return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": self.samples[0][1],
                    "reasons": sorted(k for k, bit in names if mask & bit), "samples": len(sm),
                    "how": "NVML every 2 ms"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s in sm if s > 0.5 * max(sm)] or sm
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": float(max(mx)),
                "reasons": sorted(reasons), "samples": len(sm), "how": "nvidia-smi -lms 20"}


TORCH_BITS = {W.F32: "float32", W.F16: "float16", W.BF16: "bfloat16", W.E4M3: "float8_e4m3fn"}


def device_inputs(torch, name, M, N, K, dev, seed):
    """Synthetic inputs of the workload's shapes and distributions.

    cfg1, cfg2 and cfg3 at their full sizes are the bits the parity tests run on: drawn on the
    host with the pinned generator (numpy default_rng(seed); A, then B, as float32 in C order,
    rounded to nearest even) and copied up.  The large problems (cfg4, cfg5, bf16 8192^3, and any
    row shard) are drawn on the device from a torch generator with the same distributions and,
    for cfg4, the same quantisation: q = sat_e4m3(rne(X / s)), so the operands sit where the real
    ones sit (most of the e4m3 range in use, part of it saturated), not near +-1.
    """
    ab = AB_TYPE.get(name, W.BF16)
    if name in ("cfg1", "cfg2", "cfg3") and (M, N, K) == FULL_DIMS[name]:
        w = W.make_workload(name)
        tdt = getattr(torch, TORCH_BITS[ab])
        view = {W.F32: np.float32, W.F16: np.float16, W.BF16: np.int16}[ab]
        A = torch.from_numpy(np.ascontiguousarray(w.A).view(view)).to(dev).view(tdt)
        B = torch.from_numpy(np.ascontiguousarray(w.B).view(view)).to(dev).view(tdt)
        return A, B, None, None
    g = torch.Generator(device=dev).manual_seed(seed)
    a_shape = (M, K)
    b_shape = (N, K) if name in TRANS_B else (K, N)
    sa = sb = None
    if ab == W.E4M3:
        sa = (torch.rand(M, generator=g, device=dev) * 1.5 + 0.5) / 448.0
        sb = (torch.rand(N, generator=g, device=dev) * 1.5 + 0.5) / 448.0
        # B is stored [N, K] (K-inner): row n is column n of the logical B, scaled by 1 / sb[n]
        A = (torch.randn(a_shape, generator=g, device=dev) / sa[:, None]).clamp_(-448, 448).to(torch.float8_e4m3fn)
        B = (torch.randn(b_shape, generator=g, device=dev) / sb[:, None]).clamp_(-448, 448).to(torch.float8_e4m3fn)
    elif ab == W.F32:
        A = torch.rand(a_shape, generator=g, device=dev) * 2 - 1
        B = torch.rand(b_shape, generator=g, device=dev) * 2 - 1
    else:
        tdt = torch.float16 if ab == W.F16 else torch.bfloat16
        a_scale = K ** -0.5 if name == "cfg2" else 1.0
        b_scale = K ** -0.5 if name == "cfg2" else 0.02
        A = (torch.randn(a_shape, generator=g, device=dev) * a_scale).to(tdt)
        B = (torch.randn(b_shape, generator=g, device=dev) * b_scale).to(tdt)
    return A, B, sa, sb


def out_dtype(torch, name):
    ct = C_TYPE.get(name, W.BF16)
    return {W.F32: torch.float32, W.F16: torch.float16, W.BF16: torch.bfloat16}[ct]


L2_BYTES = 126 * 1024 * 1024


def time_device(torch, R, name, M, N, K, steps, warmup, dev, seed, rotate=False, graph=False, **plan_kw):
    """`steps` back-to-back launches of the plan on device-resident inputs.

    Returns (ms_per_step, plan info, l2 note).  With `rotate` (workloads whose operands would
    stay in L2 from one launch to the next) the launches cycle through enough copies of A, B and
    C that more than two L2 sizes of other data pass between two uses of the same copy.
    With `graph` the same rotation is also captured into one CUDA graph and replayed
    (info["cuda_graph_ms"], per launch): what a caller with a launch-bound loop would do.
    """
    A, B, sa, sb = device_inputs(torch, name, M, N, K, dev, seed)
    C = torch.empty((M, N), device=dev, dtype=out_dtype(torch, name))
    per_set = A.numel() * A.element_size() + B.numel() * B.element_size() + C.numel() * C.element_size()
    copies = 1
    if rotate:
        copies = min(64, max(2, -(-2 * L2_BYTES // per_set) + 1))
    sets = [(A, B, C)] + [(A.clone(), B.clone(), torch.empty_like(C)) for _ in range(copies - 1)]
    plan = R.GemmPlan(M, N, K, AB_TYPE.get(name, W.BF16), C_TYPE.get(name, W.BF16),
                      transB=name in TRANS_B, scales=sa is not None, **plan_kw)
    ws = torch.empty(max(plan.workspace_bytes, 16), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for i in range(max(warmup, copies if rotate else 0)):
        a, b, c = sets[i % copies]
        plan.run(a, b, c, sa, sb, ws, status, stream)
    torch.cuda.synchronize()
    R.check_status(status, stream)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        a, b, c = sets[i % copies]
        plan.run(a, b, c, sa, sb, ws, status, stream)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    R.check_status(status, stream)
    info = plan.info
    if graph:
        per_replay = copies * max(1, 24 // copies)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            cs = torch.cuda.current_stream().cuda_stream
            for i in range(per_replay):
                a, b, c = sets[i % copies]
                plan.run(a, b, c, sa, sb, ws, status, cs)
        g.replay()
        torch.cuda.synchronize()
        replays = max(1, steps // per_replay)
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        R.check_status(status, stream)
        info["cuda_graph_ms"] = e0.elapsed_time(e1) / (replays * per_replay)
        info["cuda_graph_launches"] = per_replay
        del g
    plan.close()
    note = ("inputs larger than L2" if copies == 1 else
            f"{copies} rotating copies of A, B, C ({copies * per_set >> 20} MiB) so no launch finds its operands in L2")
    return ms, info, note


def measure_tensor_peaks(torch, R, dev, like_ms):
    """Tensor-pipe denominators measured on this device in this run, for the operand types the
    driver-written peaks file does not cover (it holds a cuBLAS bf16 figure only):

    * ``mma_only``: every SM pair issuing tcgen05.mma back to back from resident shared memory
      (frisk_b200_measure_mma_peak), launch length matched to `like_ms` per type because the
      clock under the power cap depends on how long the pipes stay busy;
    * ``cublaslt_e4m3``: torch._scaled_mm (cuBLASLt) on e4m3 8192^3, best of 10 -- the library
      figure of the same kind as the bf16 one in the peaks file.
    """
    out = {}
    for key, ab in (("e4m3", W.E4M3), ("bf16", W.BF16), ("tf32", W.F32)):
        try:
            probe = R.measure_mma_peak(ab, pair=True, k_blocks=1024, reps=5)
            want = like_ms.get(key, probe["ms_per_launch"])
            kb = int(max(32, round(1024 * want / probe["ms_per_launch"] / 32) * 32))
            best = max((R.measure_mma_peak(ab, pair=True, k_blocks=kb, reps=10) for _ in range(3)),
                       key=lambda r: r["tflops"])
            out["mma_only_" + key] = {"tflops": round(best["tflops"], 1), "ms_per_launch": round(best["ms_per_launch"], 4),
                                      "k_blocks": kb, "shape": "256x256x(32 bytes) two-SM MMAs, 74 pairs"}
        except Exception as e:  # the figure is reported, never required
            out["mma_only_" + key] = {"error": str(e)}
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).clamp_(-448, 448).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).clamp_(-448, 448).to(torch.float8_e4m3fn)
        one = torch.ones((), device=dev)
        for _ in range(3):
            torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        out["cublaslt_e4m3"] = {"tflops": round(2.0 * n ** 3 / (best * 1e-3) / 1e12, 1), "ms": round(best, 4),
                                "how": "torch._scaled_mm e4m3 8192^3 -> bf16, best of 10, CUDA events"}
        del a, b
    except Exception as e:
        out["cublaslt_e4m3"] = {"error": str(e)}
    return out


def roofline_for(name, M, N, K, ms, peaks, sustained, tensor_peaks=None):
    ab, ct = AB_TYPE.get(name, W.BF16), C_TYPE.get(name, W.BF16)
    extra = {}
    if BOUND.get(name) == "hbm":
        alg = M * K * W.ELEM_SIZE[ab] + K * N * W.ELEM_SIZE[ab] + M * N * W.ELEM_SIZE[ct]
        achieved = alg / (ms * 1e-3) / 1e9
        peak = peaks["hbm_gbs"]
        unit = "GB/s"
        source = peaks["source"]
    else:
        achieved = 2.0 * M * N * K / (ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
        source = peaks["source"] + (" (sustained)" if sustained else " (burst)")
        unit = "TFLOP/s"
        if ab == W.E4M3:
            # no e4m3 figure in the peaks file: the denominator is the tensor pipes' own rate
            # measured in this run; the library figure and the nominal one are given beside it
            tp = tensor_peaks or {}
            mma = tp.get("mma_only_e4m3", {}).get("tflops")
            lib = tp.get("cublaslt_e4m3", {}).get("tflops")
            if mma:
                peak, source = mma, "measured mma-only"
            else:
                peak, source = 2.0 * peak, "2 x " + source + " (no e4m3 peak could be measured)"
            extra = {"frac_of_cublaslt_e4m3": None if not lib else round(achieved / lib, 4),
                     "frac_of_nominal_4500": round(achieved / 4500.0, 4),
                     "frac_of_2x_cublas_bf16": round(achieved / (2.0 * peaks["bf16_tflops"]), 4)}
        if ab == W.F32:
            # the 3xTF32 plan spends three tf32 products per fp32 product: its ceiling is a third
            # of the tensor pipes' tf32 rate measured in this run; the CUDA-core kernel (small
            # problems) has no tensor roofline
            mma = (tensor_peaks or {}).get("mma_only_tf32", {}).get("tflops")
            if mma and name != "cfg1":
                peak, source = mma / 3.0, "measured mma-only tf32 / 3"
            else:
                peak = None
    out = {"bound": BOUND.get(name, "tensor"), "achieved": round(achieved, 2),
           "peak": None if peak is None else round(peak, 1), "unit": unit,
           "frac": None if peak is None else round(achieved / peak, 4),
           "traffic": (CFG5_SLAB_TRAFFIC * M // CFG5_SLAB_ROWS if name == "cfg5"
                       else NCU_TRAFFIC_BYTES.get(name)),
           "peak_source": source}
    out.update(extra)
    return out


REDUCE_CASES = (
    # name, shape, dim, element type, kind: the two reduces of the reference's online-softmax sketch
    # (tmp/ir.mlir:21-78: row maximum of fp16 activations, row sum of fp32 exponentials) and the
    # same matrix reduced the other way
    ("row_max_f16", (8192, 8192), 1, W.F16, "max"),
    ("row_sum_f32", (8192, 8192), 1, W.F32, "add"),
    ("col_min_f16", (8192, 8192), 0, W.F16, "min"),
)


def time_reduce(torch, R, dev, steps, warmup, peaks, with_cpu):
    """frisk.reduce on whole buffers: GB/s of algorithmic bytes (source read once + destination
    written) against the measured copy bandwidth.  Three source copies are rotated so that no
    launch finds its input in L2."""
    out = {}
    tdt = {W.F16: torch.float16, W.F32: torch.float32}
    for name, shape, dim, dtype, kind in REDUCE_CASES:
        n = shape[0] * shape[1]
        g = torch.Generator(device=dev).manual_seed(17)
        srcs = [torch.randn(n, generator=g, device=dev, dtype=torch.float32).to(tdt[dtype]) for _ in range(3)]
        desc = R.reduce_desc(shape, dim, dtype, kind)
        info = R.reduce_info(desc)
        dst = torch.empty(desc.outer * desc.inner, device=dev, dtype=tdt[dtype])
        ws = torch.empty(max(R.reduce_workspace_bytes(desc), 16), dtype=torch.uint8, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        for i in range(warmup):
            R.reduce_run(desc, srcs[i % 3], dst, ws, stream)
        torch.cuda.synchronize()
        k = steps
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(k):
            R.reduce_run(desc, srcs[i % 3], dst, ws, stream)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / k
        alg = (n + desc.outer * desc.inner) * W.ELEM_SIZE[dtype]
        achieved = alg / (ms * 1e-3) / 1e9
        entry = {"shape": list(shape), "dim": dim, "dtype": W.DTYPE_NAMES[dtype], "kind": kind,
                 "ms": round(ms, 5), "launches_per_step": info["launches"], "ctas": info["ctas"],
                 "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                              "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                              "traffic": NCU_TRAFFIC_BYTES.get(name),
                              "peak_source": peaks["source"]},
                 "l2": "three sources rotated (0.4 - 0.8 GB)"}
        if with_cpu:  # the float64 restatement on a row sample, beside the kernel
            from oracle import ref
            rows = 256
            sample = srcs[0].view(*shape)[:rows].cpu().numpy()
            t0 = time.perf_counter()
            ref.ref_reduce(sample, dim, dtype, kind)
            dt = time.perf_counter() - t0
            entry["cpu_baseline"] = {"value": round(sample.nbytes / dt / 1e9, 3), "unit": "GB/s", "cores": 1,
                                     "kind": "port", "sample": f"{rows} rows of the source, {dt * 1e3:.0f} ms"}
        out[name] = entry
        del srcs, dst, ws
    return out


def host_threads() -> int:
    """All cores this process may use (torchrun sets OMP_NUM_THREADS=1; the CPU legs ignore that)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_baseline(name, target_s=12.0):
    """The oracle port (naive fp32 loop, OpenMP over rows) on a bounded sample of the workload."""
    from oracle import ref

    M, N, K = FULL_DIMS[name]
    threads = host_threads()
    rows = min(M, 16)
    w = W.make_workload(name, rows, N, K)
    t0 = time.perf_counter()
    ref.ref_gemm(w, num_threads=threads)
    dt = time.perf_counter() - t0
    # grow the sample towards the target time
    rows2 = int(min(M, max(rows, rows * target_s / max(dt, 1e-3))))
    rows2 = max(threads, rows2 // threads * threads)
    if rows2 > rows:
        w = W.make_workload(name, rows2, N, K)
        t0 = time.perf_counter()
        ref.ref_gemm(w, num_threads=threads)
        dt = time.perf_counter() - t0
        rows = rows2
    tflops = 2.0 * rows * N * K / dt / 1e12
    out = {"value": round(tflops, 5), "unit": "TFLOP/s", "cores": threads, "kind": "port",
           "sample": f"rows [0, {rows}) of {name} ({rows}x{N}x{K}), {dt:.1f} s, per-FLOP rate of the full problem assumed equal"}
    try:
        import torch

        torch.set_num_threads(threads)
        a = torch.from_numpy(w.a_logical().astype(np.float32))
        b = torch.from_numpy(np.ascontiguousarray(w.b_logical().astype(np.float32)))
        a @ b
        t0 = time.perf_counter()
        for _ in range(3):
            a @ b
        dt2 = (time.perf_counter() - t0) / 3
        out["torch_matmul_cpu_tflops"] = round(2.0 * rows * N * K / dt2 / 1e12, 4)
    except Exception:  # torch CPU matmul is an extra, never required
        pass
    return out


def run_reference(args):
    """`--impl reference`: the CPU restatement timed on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref

    name = args.workload
    M, N, K = FULL_DIMS[name]
    threads = host_threads()
    rows = max(threads, min(M, 8 * threads))
    w = W.make_workload(name, rows, N, K)
    for _ in range(max(args.warmup, 0)):
        ref.ref_gemm(w, num_threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ref.ref_gemm(w, num_threads=threads)
    dt = (time.perf_counter() - t0) / args.steps
    tflops = 2.0 * rows * N * K / dt / 1e12
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": round(tflops, 5), "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": W.DTYPE_NAMES[AB_TYPE.get(name, W.BF16)], "data": "synthetic",
        "config": {"workload": name, "M": M, "N": N, "K": K,
                   "note": "the reference has no executable GEMM; this is its op restated as a "
                           "naive fp32 loop (oracle/frisk_ref_gemm.c) on a row sample"},
        "cpu_baseline": {"value": round(tflops, 5), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"rows [0, {rows}) of {name} per step"},
        "e2e": {"value": round(tflops, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg5", choices=sorted(FULL_DIMS))
    ap.add_argument("--impl", default="frisk_b200", choices=["frisk_b200", "reference"])
    ap.add_argument("--no-others", action="store_true", help="skip the other configurations")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer measurement")
    ap.add_argument("--no-allgather", action="store_true", help="skip the all-gather measurements (N > 1)")
    ap.add_argument("--reduce-only", action="store_true",
                    help="time only the frisk.reduce cases, with exactly --warmup and --steps launches each "
                         "(a small run for a profiler), and print their JSON")
    ap.add_argument("--band", type=int, default=0,
                    help="tile rows the rasterisation walks together (0: the plan's choice)")
    ap.add_argument("--panel", type=int, default=0,
                    help="walk the tiles in panels of this many tile columns (0: the plan's choice)")
    ap.add_argument("--l2-hints", type=int, default=0,
                    help="bit 0: A loads evict-first, bit 1: B loads evict-last (0: the plan's choice)")
    ap.add_argument("--epilogue", type=int, default=0,
                    help="1: per-thread row stores, 2: rows staged through swizzled shared memory, 3: staged through "
                         "linear rows, 4: TMA tensor stores (0: the plan's choice)")
    ap.add_argument("--k-split", type=int, default=0,
                    help="-1: never split K, 1: over clusters or stream-K, 2: K planes (0: the plan's choice)")
    ap.add_argument("--rows", type=int, default=0,
                    help="run the workload on this many rows only (a small case for a profiler)")
    args = ap.parse_args()
    asked_warmup = args.warmup
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)

    import torch
    from frisk_b200 import runtime as R
    from frisk_b200 import sharding as S

    R.lib()  # fail loudly when the CUDA library is missing: there is no other path
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a); none is visible")
    if args.reduce_only:
        torch.cuda.set_device(0)
        print(json.dumps(time_reduce(torch, R, torch.device("cuda:0"), max(args.steps, 1), asked_warmup,
                                     load_peaks(), False)), flush=True)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    name = args.workload
    M, N, K = FULL_DIMS[name]
    if args.rows:
        M = args.rows
        args.warmup = asked_warmup   # a profiler's small case: exactly the launches asked for
    row0, rows = S.local_rows(M, world, rank)
    peaks = load_peaks()
    ab, ct = AB_TYPE.get(name, W.BF16), C_TYPE.get(name, W.BF16)

    # ---- device-resident timing: K steps, barrier + synchronize on both sides, max over ranks
    A, B, sa, sb = device_inputs(torch, name, rows, N, K, dev, seed=4 + 1000 * rank)
    if world > 1:  # B is replicated: every rank holds rank 0's B
        dist.broadcast(B, 0)
    C = torch.empty((rows, N), device=dev, dtype=out_dtype(torch, name))
    plan = R.GemmPlan(rows, N, K, ab, ct, transB=name in TRANS_B, scales=sa is not None,
                      band_tiles=args.band, epilogue=args.epilogue, panel_tiles=args.panel,
                      l2_hints=args.l2_hints,
                      # (the peer stores of the fused all-gather live in the whole-tile epilogue)
                      k_split=args.k_split if world == 1 or args.k_split else -1)
    ws = torch.empty(max(plan.workspace_bytes, 16), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    small_inputs = (A.numel() * A.element_size() + B.numel() * B.element_size()) < 256 * 2 ** 20
    # Operands that would stay in the 126 MB L2 from one launch to the next are rotated: enough
    # copies of A, B and C that more than two L2 sizes of other data pass between two uses of one
    sets = [(A, B, C)]
    if small_inputs:
        per_set = sum(t.numel() * t.element_size() for t in (A, B, C))
        copies = min(64, max(2, -(-2 * L2_BYTES // per_set) + 1))
        sets += [(A.clone(), B.clone(), torch.empty_like(C)) for _ in range(copies - 1)]
    for i in range(max(args.warmup, len(sets) if small_inputs else 0)):
        a_, b_, c_ = sets[i % len(sets)]
        plan.run(a_, b_, c_, sa, sb, ws, status, stream)
    torch.cuda.synchronize()
    R.check_status(status, stream)

    sampler_index, sampler_uuid = local, getattr(torch.cuda.get_device_properties(local), "uuid", None)
    sampler = ClockSampler(sampler_index, sampler_uuid)   # every rank its own GPU
    sampler.start()
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        a_, b_, c_ = sets[i % len(sets)]
        plan.run(a_, b_, c_, sa, sb, ws, status, stream)
    e1.record()
    torch.cuda.synchronize()
    my_ms = e0.elapsed_time(e1)
    if dist:
        dist.barrier()
    R.check_status(status, stream)
    my_clocks = sampler.stop()
    elapsed_ms = S.max_over_ranks(dist, my_ms, dev)
    ms_per_step = elapsed_ms / args.steps
    total_flops = 2.0 * M * N * K
    value = total_flops / (ms_per_step * 1e-3) / 1e12
    # per rank: time and the clock it ran at.  The product ms x MHz is the time in SM cycles: it
    # separates what the sharding does from what the power cap does to the clock (a long 1-GPU step
    # is pulled down by the cap, the short per-rank steps at 8 GPUs are not).
    per_rank = [{"rank": rank, "ms_per_step": round(my_ms / args.steps, 4), "sm_mhz": my_clocks.get("sm_mhz"),
                 "reasons": my_clocks.get("reasons")}]
    if dist:
        gathered = [None] * world
        dist.all_gather_object(gathered, per_rank[0])
        per_rank = gathered
    slowest = max(per_rank, key=lambda r: r["ms_per_step"])
    clock_note = None
    if slowest.get("sm_mhz"):
        clock_note = {"slowest_rank": slowest["rank"], "slowest_rank_sm_mhz": slowest["sm_mhz"],
                      "rank0_sm_mhz": per_rank[0].get("sm_mhz"),
                      "mcycles_per_step": round(ms_per_step * slowest["sm_mhz"] * 1e-3, 3),
                      "note": "ms_per_step x median SM MHz of the slowest rank = SM cycles per step (millions); "
                              "compare this across N, not ms, to judge the sharding apart from the power cap"}

    # ---- the all-gather of C over NVLink (not on the data path; never inside `value`)
    allgather = None
    if dist and world > 1 and M % world == 0 and not args.no_allgather:
        allgather = time_allgather(torch, R, S, dist, plan, A, B, C, sa, sb, ws, status, stream, M, N, world, rank,
                                   dev, ms_per_step, 20, gpu_index=sampler_index, gpu_uuid=sampler_uuid)

    # ---- end to end: host buffers through the C-ABI call, copies inside the timed region
    e2e = None
    if not args.no_e2e:
        hA = torch.empty(A.shape, dtype=A.dtype, pin_memory=True).copy_(A)
        hB = torch.empty(B.shape, dtype=B.dtype, pin_memory=True).copy_(B)
        hC = torch.empty(C.shape, dtype=C.dtype, pin_memory=True)
        hsa = None if sa is None else sa.cpu()
        hsb = None if sb is None else sb.cpu()
        e2e_steps = max(1, min(args.steps, 5))
        L = R.lib()

        def host_step():
            rc = L.frisk_b200_gemm_run_host(plan._h, hA.data_ptr(), hB.data_ptr(), hC.data_ptr(),
                                            None if hsa is None else hsa.data_ptr(),
                                            None if hsb is None else hsb.data_ptr())
            if rc != 0:
                raise SystemExit(f"frisk_b200_gemm_run_host failed: {rc}")

        host_step()
        if dist:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host_step()  # synchronous: returns after C is back in host memory
        dt = (time.perf_counter() - t0) / e2e_steps
        dt = S.max_over_ranks(dist, dt, dev)
        h2d = hA.numel() * hA.element_size() + hB.numel() * hB.element_size()
        if sa is not None:
            h2d += 4 * (rows + N)
        d2h = hC.numel() * hC.element_size()
        e2e = {"value": round(total_flops / dt / 1e12, 3), "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": round(dt * 1e3, 3), "steps": e2e_steps,
               "api": "frisk_b200_gemm_run_host (pinned host buffers, per rank)"}
        del hA, hB, hC
    info = plan.info
    plan.close()
    del A, B, C

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return

    sustained = elapsed_ms > 500.0
    tensor_peaks = None
    if ab == W.E4M3:
        tensor_peaks = measure_tensor_peaks(torch, R, dev, {"e4m3": ms_per_step})
    roof = roofline_for(name, rows, N, K, ms_per_step, peaks, sustained, tensor_peaks)
    line = {
        "metric": "gemm_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": W.DTYPE_NAMES[ab], "data": "synthetic",
        "config": {"workload": name, "M": M, "N": N, "K": K, "rows_per_gpu": rows,
                   "sharding": f"rows of A and C over {world} GPU(s), B replicated, no collective",
                   "accumulate": "fp32", "kernel": info["kernel_name"],
                   "tile": f"{info['tile_m']}x{info['tile_n']}x{info['tile_k']}",
                   "stages": info["stages"], "ctas": info["num_ctas"],
                   "l2": "inputs larger than L2" if len(sets) == 1 else
                         f"{len(sets)} rotating copies of A, B, C so no launch finds its operands in L2"},
        "roofline": roof,
        "clocks": {k: my_clocks.get(k) for k in ("sm_mhz", "sm_max_mhz", "reasons", "samples", "how")},
        "clocks_per_rank": per_rank,
        "clock_normalised": clock_note,
        "gpu_launches": info["launches"] * args.steps,
        "e2e": e2e,
    }
    if allgather:
        line["allgather"] = allgather

    if world == 1 and not args.no_others and not args.rows:
        others = {}
        tensor_peaks = measure_tensor_peaks(torch, R, dev, {"e4m3": 0.37, "bf16": 0.70, "tf32": 0.45})
        line["tensor_peaks_measured"] = tensor_peaks
        for other in ("cfg1", "cfg2", "cfg3", "cfg4", "bf16_8192", "fp32_4096", "bf16_short_k", "bf16_deep_k"):
            if other == name:
                continue
            m, n, k = FULL_DIMS[other]
            # operands (nearly) fit in L2: rotate copies
            small = other in ("cfg1", "cfg2", "cfg3", "bf16_short_k", "bf16_deep_k")
            ms, oinfo, l2_note = time_device(torch, R, other, m, n, k,
                                             max(args.steps, 200 if small else 10), args.warmup, dev,
                                             seed=int(other[-1]) if other.startswith("cfg") else 5,
                                             rotate=small, graph=other in ("cfg1", "cfg3"))
            r = roofline_for(other, m, n, k, ms, peaks, False, tensor_peaks)
            others[other] = {"ms": round(ms, 5), "kernel": oinfo["kernel_name"],
                             "tflops": round(2.0 * m * n * k / (ms * 1e-3) / 1e12, 2),
                             "launches_per_step": oinfo["launches"], "roofline": r,
                             "l2": l2_note}
            if "cuda_graph_ms" in oinfo:   # the same launches replayed from one captured CUDA graph
                others[other]["cuda_graph"] = {"ms": round(oinfo["cuda_graph_ms"], 5),
                                               "launches_per_graph": oinfo["cuda_graph_launches"]}
            if other == "cfg2":
                others[other]["library_same_shape"] = library_matmul(torch, dev, m, n, k, torch.float16)
            if other in ("bf16_short_k", "bf16_deep_k"):   # planner rules made for shapes like these
                others[other]["library_same_shape"] = library_matmul(torch, dev, m, n, k, torch.bfloat16,
                                                                     b_row_major=True)
            if other == "cfg1":   # the same problem forced onto the 3xTF32 plan (three launches)
                ms3, _, _ = time_device(torch, R, other, m, n, k, 200, args.warmup, dev, seed=1, rotate=True,
                                        force_kernel="tf32x3")
                others[other]["tf32x3_forced_ms"] = round(ms3, 5)
            if other == "fp32_4096":   # ... and the large one on the CUDA-core kernel
                ms1, _, _ = time_device(torch, R, other, m, n, k, 3, 1, dev, seed=5, force_kernel="simt")
                others[other]["cuda_core_ms"] = round(ms1, 3)
        line["other_configs"] = others
        line["reduce"] = time_reduce(torch, R, dev, max(args.steps, 30), max(args.warmup, 3), peaks,
                                     not args.no_cpu)
        line["gemm_with_row_reduce"] = time_fused_row_reduce(torch, R, dev, 10, 3)

    if world == 1 and not args.no_cpu and not args.rows:
        line["cpu_baseline"] = cpu_baseline(name)
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


def time_fused_row_reduce(torch, R, dev, steps, warmup):
    """bf16 8192^3 followed by the row maxima of its result (the gemm + reduce pair of the
    reference's attention sketch, tmp/ir.mlir:112-116), two ways: the fold in the GEMM's epilogue
    (`desc.row_reduce`: the rows are folded as they leave tensor memory, a small second launch folds
    the per-tile results), and the GEMM followed by the separate reduce kernel reading C again."""
    M = N = K = 8192
    A, B, _, _ = device_inputs(torch, "bf16_8192", M, N, K, dev, 5)
    C = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
    rowmax = torch.empty(M, device=dev, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    fused = R.GemmPlan(M, N, K, W.BF16, row_reduce="max")
    plain = R.GemmPlan(M, N, K, W.BF16)
    ws = torch.empty(max(fused.workspace_bytes, 16), dtype=torch.uint8, device=dev)
    rdesc = R.reduce_desc((M, N), 1, W.BF16, "max")

    def fold_in_epilogue():
        fused.run_ex(A, B, C, workspace=ws, status=status, stream=stream, row_reduce_dst=rowmax)

    def two_launches():
        plain.run(A, B, C, None, None, None, status, stream)
        R.reduce_run(rdesc, C, rowmax, None, stream)

    out = {}
    for key, fn in (("fold_in_epilogue", fold_in_epilogue), ("gemm_then_reduce", two_launches)):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out[key + "_ms"] = round(e0.elapsed_time(e1) / steps, 4)
        out[key + "_rowmax_checksum"] = float(rowmax.float().sum().item())
    R.check_status(status, stream)
    out["same_result"] = out.pop("fold_in_epilogue_rowmax_checksum") == out.pop("gemm_then_reduce_rowmax_checksum")
    out["shape"] = "bf16 8192^3, max over the 8192 columns of each row of C"
    fused.close()
    plain.close()
    return out


def library_matmul(torch, dev, m, n, k, dtype, b_row_major=False):
    """torch.matmul (cuBLAS) on the same shape with rotating operands, for context beside a
    configuration whose roofline denominator was measured on another shape.  B is stored [N, K]
    (cfg2's order) unless `b_row_major` ([K, N], the order of the bf16 workloads)."""
    copies = 4
    a = [torch.randn(m, k, device=dev).to(dtype) * k ** -0.5 for _ in range(copies)]
    if b_row_major:
        b = [torch.randn(k, n, device=dev).to(dtype) * k ** -0.5 for _ in range(copies)]
    else:
        b = [(torch.randn(n, k, device=dev).to(dtype) * k ** -0.5).t() for _ in range(copies)]
    c = [torch.empty(m, n, device=dev, dtype=dtype) for _ in range(copies)]
    for i in range(copies):
        torch.matmul(a[i], b[i], out=c[i])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = 200
    e0.record()
    for i in range(steps):
        torch.matmul(a[i % copies], b[i % copies], out=c[i % copies])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"ms": round(ms, 5), "tflops": round(2.0 * m * n * k / (ms * 1e-3) / 1e12, 2),
            "how": "torch.matmul, four rotating copies of A, B and C, 200 launches"}


def time_allgather(torch, R, S, dist, plan, A, B, C, sa, sb, ws, status, stream, M, N, world, rank, dev,
                   gemm_ms, steps, gpu_index=0, gpu_uuid=None):
    """The optional all-gather of the C shards, two ways, each timed on the device (max over ranks):

    * ``nccl_after``: the GEMM, then ncclAllGather of the finished shards (the library baseline),
      timed as the sequence a caller would run, step after step;
    * ``fused``: the GEMM itself stores every tile into every rank's copy of C
      (frisk_b200_gemm_run_ex with peer pointers; plain stores over NVLink, nothing loaded from a
      peer), so the transfer runs under the math.

    Every loop runs the same number of steps after its own warm-up with the SM clock sampled
    beside it, and the plain GEMM is timed once more directly behind the fused loop: a B200 under
    its power cap runs a GEMM that follows tens of milliseconds of GEMMs slower than one that
    follows an idle GPU, so only loops in the same state compare.  `hidden` is the share of the
    all-gather's own time that the fused form no longer adds to a GEMM in that state.
    """
    rows = C.shape[0]
    es = C.element_size()
    out = {"steps_per_loop": steps}

    def loop(step, warm=3):
        dist.barrier()
        for _ in range(warm):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        sampler = ClockSampler(gpu_index, gpu_uuid)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        clk = sampler.stop()
        ms = S.max_over_ranks(dist, e0.elapsed_time(e1) / steps, dev)
        return ms, clk.get("sm_mhz")

    def gemm_only():
        plan.run(A, B, C, sa, sb, ws, status, stream)

    keep = {}

    def nccl_only():
        keep["full"] = S.allgather_rows(dist, C, M, world, rank)

    def gemm_then_nccl():
        gemm_only()
        nccl_only()

    ag_ms, _ = loop(nccl_only, warm=2)
    seq_ms, seq_mhz = loop(gemm_then_nccl)
    recv = (world - 1) * rows * N * es
    out["nccl_after"] = {"allgather_alone_ms": round(ag_ms, 3),
                         "recv_GBps_per_gpu": round(recv / (ag_ms * 1e-3) / 1e9, 1),
                         "gemm_plus_allgather_ms": round(seq_ms, 3), "sm_mhz": seq_mhz,
                         "how": "GEMM, then all_gather_into_tensor, step after step on one stream"}
    want = keep["full"][:: max(1, M // 64)].clone()   # a sample of rows of the NCCL result, to check the fused one
    keep.clear()
    try:
        pg = S.PeerGather(dist, M, N, es, world, rank)
    except Exception as e:  # no peer access between these GPUs: report it, keep the NCCL figure
        out["fused"] = {"error": str(e)}
        return out
    try:
        def fused():
            plan.run_ex(A, B, pg.local_c, scale_a=sa, scale_b=sb, workspace=ws, status=status, stream=stream,
                        peers=pg.peer_dsts)

        fused_ms, fused_mhz = loop(fused)
        again_ms, again_mhz = loop(gemm_only, warm=0)   # the plain GEMM in the state the fused loop left
        dist.barrier()   # every rank's stores have landed
        R.check_status(status, stream)
        got = pg.as_tensor(C.dtype)[:: max(1, M // 64)]
        same = bool(torch.equal(got.view(torch.int16) if es == 2 else got, want.view(torch.int16) if es == 2 else want))
        sent = (world - 1) * rows * N * es
        out["fused"] = {"gemm_plus_allgather_ms": round(fused_ms, 3), "sm_mhz": fused_mhz,
                        "sent_GBps_per_gpu": round(sent / (fused_ms * 1e-3) / 1e9, 1),
                        "gemm_alone_right_after_ms": round(again_ms, 3), "gemm_alone_right_after_sm_mhz": again_mhz,
                        "hidden": round(1.0 - max(0.0, fused_ms - again_ms) / ag_ms, 3),
                        "vs_nccl_after": round(seq_ms / fused_ms, 3),
                        "equals_nccl_result_on_sampled_rows": same,
                        "how": f"the epilogue stores each C tile to the local shard and to the {world - 1} peer cop{'y' if world == 2 else 'ies'}"}
    finally:
        torch.cuda.synchronize()
        pg.close(dist)
    return out


if __name__ == "__main__":
    main()
