#!/usr/bin/env python
"""Benchmark of the dense-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload auto|c1..c5|s16|i32|moe]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

A step is one pass of the hot path over one synthetic batch: one fused GEMM + epilogue call.
Workloads are the five synthetic configurations the metric is quoted on:
  c1  F32 1024^3 + bias + GELU (exact-F32 mode)          c2  BF16 4096^3, transposed-B, + bias + ReLU
  c3  I8 x I8 -> I32 4096^3                               c4  FP8-E4M3 8192^3 scaled + bias + SiLU + residual -> BF16
  c5  BF16 X[16384,4096] @ W[4096,14336] + SiLU, W split along N over the ranks (no reduction)
`auto` runs c5 at every GPU count (the N-sharded configuration: the 1 -> 8 curve is one workload); on
one GPU the line also carries the kernel-only figures of c1..c4, each against its roofline.
Three more, outside numr's headline configurations: s16 (decode shape, HBM-bound), i32 (the
integer widths without a tensor-core form) and moe (grouped matmul, offsets on the device).

Rank 0 prints ONE JSON line: `value` is whole-job TFLOPS with inputs resident in HBM (CUDA-event
timed, max over ranks); `e2e` is the same metric through the client call with pinned host buffers,
host<->device copies inside the timed region; `roofline` and `cpu_baseline` explain the numbers.
`--impl reference` times the CPU restatement of numr's own path for the same workload instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL_TFLOPS = {"bf16": 2250.0, "f8": 4500.0, "i8": 4500.0, "tf32": 1125.0}


# ----------------------------------------------------------------------------- workloads
class Workload:
    """One configuration: host inputs (numpy -> torch CPU tensors), op call, flop count."""

    def __init__(self, name, world=1, rank=0):
        self.name = name
        self.world, self.rank = world, rank
        build = getattr(self, "_build_" + name)
        build()

    # inputs are generated on the host with numpy's default_rng(seed), as the configs state
    def _build_c1(self):
        rng = np.random.default_rng(0)
        m = n = k = 1024
        self.a = torch.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32))
        self.b = torch.from_numpy(rng.uniform(-1, 1, (k, n)).astype(np.float32))
        self.bias = torch.from_numpy(rng.uniform(-1, 1, n).astype(np.float32))
        self.m, self.n, self.k = m, n, k
        self.dtype, self.peak_key = "f32", "tf32"
        self.desc = "c1: F32 matmul_bias_activation(GELU) 1024x1024x1024, exact-F32 mode (3xTF32)"
        # exact mode issues three TF32 MMAs per product term
        self.hw_flop_factor = 3.0
        self.graph = True     # tens of microseconds per step: timed as a CUDA-graph replay

    def _build_c2(self):
        rng = np.random.default_rng(1)
        m = n = k = 4096
        s = 1.0 / np.sqrt(4096.0)
        self.a = torch.from_numpy((rng.standard_normal((m, k)) * s).astype(np.float32)).to(torch.bfloat16)
        self.w_nk = torch.from_numpy((rng.standard_normal((n, k)) * s).astype(np.float32)).to(torch.bfloat16)
        self.bias = torch.from_numpy((rng.standard_normal(n) * s).astype(np.float32)).to(torch.bfloat16)
        self.m, self.n, self.k = m, n, k
        self.dtype, self.peak_key = "bf16", "bf16"
        self.desc = "c2: BF16 matmul_bias_activation(ReLU) 4096x4096x4096, B = transposed view of W[N,K]"

    def _build_c3(self):
        rng = np.random.default_rng(2)
        m = n = k = 4096
        self.a = torch.from_numpy(rng.integers(-127, 128, (m, k)).astype(np.int8))
        self.b = torch.from_numpy(rng.integers(-127, 128, (k, n)).astype(np.int8))
        self.m, self.n, self.k = m, n, k
        self.dtype, self.peak_key = "i8", "i8"
        self.desc = "c3: I8 x I8 -> I32 matmul 4096x4096x4096"

    def _build_c4(self):
        rng = np.random.default_rng(3)
        m = n = k = 8192
        a0 = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32))
        b0 = torch.from_numpy(rng.standard_normal((k, n)).astype(np.float32))
        self.scale_a = float(a0.abs().max() / 448.0)
        self.scale_b = float(b0.abs().max() / 448.0)
        self.a = (a0 / self.scale_a).to(torch.float8_e4m3fn)
        self.b = (b0 / self.scale_b).to(torch.float8_e4m3fn)
        del a0, b0
        self.bias = torch.from_numpy((rng.standard_normal(n) * 0.02).astype(np.float32)).to(torch.bfloat16)
        self.residual = torch.from_numpy((rng.standard_normal((m, n)) * 0.02).astype(np.float32)).to(torch.bfloat16)
        self.m, self.n, self.k = m, n, k
        self.dtype, self.peak_key = "f8e4m3", "f8"
        self.desc = "c4: FP8-E4M3 scaled GEMM + bias + SiLU + residual -> BF16, 8192x8192x8192"

    def _build_c5(self):
        rng = np.random.default_rng(4)
        m, k, n = 16384, 4096, 14336
        assert n % self.world == 0
        shard = n // self.world
        self.a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(torch.bfloat16)
        # Every rank draws the same full W stream, then keeps its own column block re-packed
        # contiguous as [K, N/g]; only the shard is kept to bound host memory.
        from numr_b200.sharding import column_range
        cols = column_range(n, self.world, self.rank)
        w = np.empty((k, shard), dtype=np.float32)
        for r0 in range(0, k, 512):
            block = rng.standard_normal((512, n)).astype(np.float32) * 0.02
            w[r0:r0 + 512] = block[:, cols]
        self.b = torch.from_numpy(w).to(torch.bfloat16)
        self.m, self.n, self.k = m, shard, k
        self.n_total = n
        self.dtype, self.peak_key = "bf16", "bf16"
        self.desc = "c5: BF16 X[16384,4096] @ W[4096,14336] + SiLU, W split along N over the GPUs, no reduction"

    def _build_s16(self):
        # decode shape of numr's own small-M benches (M in 1..64 against a [4096,4096] weight given
        # as [N,K]): bound by reading the weight once from HBM
        rng = np.random.default_rng(5)
        m, n, k = 16, 4096, 4096
        self.a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(torch.bfloat16)
        self.w_nk = torch.from_numpy((rng.standard_normal((n, k)) * 0.02).astype(np.float32)).to(torch.bfloat16)
        self.m, self.n, self.k = m, n, k
        self.dtype, self.peak_key = "bf16", "bf16"
        self.bound = "hbm"
        self.graph = True     # a 16 us kernel: the timed steps are replayed from one CUDA graph
        self.desc = "s16: BF16 matmul 16x4096x4096 against W[N,K] (decode shape; reads the weight once)"

    def _build_moe(self):
        # grouped matmul (numr GroupedMatmulOps): 16384 token rows routed to 8 experts of uneven load,
        # the row boundaries on the device; each expert's weight [K, N] = [4096, 4096]
        rng = np.random.default_rng(7)
        m, k, n, groups = 16384, 4096, 4096, 8
        counts = np.array([3100, 0, 1500, 4097, 129, 2047, 3511, 2000])
        assert counts.sum() == m
        self.a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(torch.bfloat16)
        self.b = torch.from_numpy((rng.standard_normal((groups, k, n)) * 0.02).astype(np.float32)).to(torch.bfloat16)
        self.offsets = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32))
        self.m, self.n, self.k = m, n, k
        self.dtype, self.peak_key = "bf16", "bf16"
        self.desc = ("moe: BF16 grouped_matmul_activation(SiLU), 16384 rows over 8 experts "
                     "(3100/0/1500/4097/129/2047/3511/2000), K = N = 4096, offsets on the device")

    def _build_i32(self):
        # what numr's integer benches time: I32 1024^2, values in [-64, 64), 128-bit accumulation
        rng = np.random.default_rng(6)
        m = n = k = 1024
        self.a = torch.from_numpy(rng.integers(-64, 64, (m, k)).astype(np.int32))
        self.b = torch.from_numpy(rng.integers(-64, 64, (k, n)).astype(np.int32))
        self.m, self.n, self.k = m, n, k
        self.dtype, self.peak_key = "i32", None
        self.desc = "i32: I32 x I32 -> I32 matmul 1024x1024x1024 (CUDA cores, 128-bit accumulator)"

    bound = "tensor"
    graph = False

    @property
    def flops(self) -> float:
        """Algorithmic flops of this rank's step."""
        return 2.0 * self.m * self.n * self.k

    def host_inputs(self):
        names = {"c1": ["a", "b", "bias"], "c2": ["a", "w_nk", "bias"], "c3": ["a", "b"],
                 "c4": ["a", "b", "bias", "residual"], "c5": ["a", "b"], "s16": ["a", "w_nk"],
                 "i32": ["a", "b"], "moe": ["a", "b", "offsets"]}[self.name]
        return {nm: getattr(self, nm) for nm in names}

    def run(self, client, t):
        """One step on device tensors `t` (same keys as host_inputs)."""
        from numr_b200 import GemmActivation
        if self.name == "c1":
            return client.matmul_bias_activation(t["a"], t["b"], t["bias"], GemmActivation.GELU)
        if self.name == "c2":
            return client.matmul_bias_activation(t["a"], t["w_nk"].t(), t["bias"], GemmActivation.RELU)
        if self.name in ("c3", "i32"):
            return client.matmul(t["a"], t["b"])
        if self.name == "moe":
            return client.grouped_matmul_activation(t["a"], t["b"], t["offsets"], GemmActivation.SILU)
        if self.name == "s16":
            return client.matmul(t["a"], t["w_nk"].t())
        if self.name == "c4":
            return client.fp8_matmul_fused(t["a"], t["b"], self.scale_a, self.scale_b, torch.bfloat16,
                                           bias=t["bias"], activation=GemmActivation.SILU,
                                           residual=t["residual"])
        return client.matmul_activation(t["a"], t["b"], GemmActivation.SILU)

    def kernels_per_step(self) -> int:
        # c1 prepares both F32 operands (one split kernel for the two) before the GEMM kernel; the grouped
        # matmul runs its plan kernel first
        return {"c1": 2, "moe": 2}.get(self.name, 1)


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Polls NVML for the SM clock and the clock-event reasons while a region runs."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake", 0x2: "applications_clocks"}

    def __init__(self, device_index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception as e:   # NVML missing: report that instead of clocks
            self._nv = None
            self.error = f"{type(e).__name__}: {e}"

    def _poll(self):
        nv, h = self._nv, self._h
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if self._nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": self.error}
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ----------------------------------------------------------------------------- helpers
def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text()), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def ncu_traffic(name):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if present."""
    p = ROOT / "profiles" / "traffic.json"
    if p.exists():
        try:
            entry = json.loads(p.read_text()).get(name)
            return entry.get("total") if isinstance(entry, dict) else entry
        except Exception:
            return None
    return None


def dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


def host_threads() -> int:
    """Host cores this process may run on (not OMP_NUM_THREADS, which torchrun sets to 1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def config_of(wl, world):
    """The `config` object: identical in the GPU arm and the reference arm of one run."""
    return {"workload": wl.desc, "m": wl.m, "n": getattr(wl, "n_total", wl.n), "k": wl.k,
            "sharding": f"N split over {world} GPU(s)" if wl.name == "c5" else "none"}


def time_region(fn, steps, stream):
    """CUDA-event time of `steps` calls of fn(i) on `stream`, in ms."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        fn(i)
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1)


class Harness:
    """Device-side timing of one workload: rotating input sets, repeated timed regions."""

    def __init__(self, wl, client, dev, world=1, dist=None, set_budget=400e6):
        self.wl, self.client, self.dev, self.world, self.dist = wl, client, dev, world, dist
        self.stream = torch.cuda.current_stream(dev)
        self.host = {k: v.pin_memory() for k, v in wl.host_inputs().items()}
        self.in_bytes = sum(v.numel() * v.element_size() for v in self.host.values())
        probe = wl.run(client, {k: v.to(dev) for k, v in self.host.items()})
        self.out_bytes = probe.numel() * probe.element_size()
        del probe
        # Rotating input sets larger than the 126 MB L2, so no timed step finds its operands cached.
        self.n_sets = max(2, min(16, -(-int(set_budget) // (self.in_bytes + self.out_bytes))))
        self.sets = [{k: v.to(dev, non_blocking=True) for k, v in self.host.items()} for _ in range(self.n_sets)]
        torch.cuda.synchronize()
        self.regions = 0

    def step(self, i):
        return self.wl.run(self.client, self.sets[i % self.n_sets])

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def _max_over_ranks(self, values):
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def timed_regions(self, steps, warmup, min_total_ms=250.0, min_regions=10, max_regions=120):
        """Warm up, then time regions of exactly `steps` steps (barrier + synchronize on both sides of
        each, CUDA events on the launching stream, max over ranks) until at least `min_regions`
        regions and `min_total_ms` of device time have been timed. Returns the per-region times.
        (A quarter of a second of back-to-back regions at every GPU count: the 1000 W power cap then
        acts on the 0.2 ms steps of 8 GPUs as it does on the 1.3 ms steps of one, so the N-GPU
        figures compare like with like.)"""
        for i in range(warmup):
            self.step(i)
        self.barrier()
        graph = None
        if self.wl.graph:
            # Launch-bound workload: the K steps (each on its own input set) are captured once and a
            # region is one replay, so the events bracket kernels, not the host's call overhead.
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(steps):
                    self.step(i)
            graph.replay()
            self.barrier()

        def one_region():
            self.barrier()
            if graph is not None:
                ms = time_region(lambda i: graph.replay() if i == 0 else None, 1, self.stream)
            else:
                ms = time_region(self.step, steps, self.stream)
            torch.cuda.synchronize()
            return ms

        first = self._max_over_ranks([one_region()])[0]
        n = int(min(max_regions, max(min_regions, -(-min_total_ms // max(first, 1e-3)))))
        local = [one_region() for _ in range(n)]
        self.barrier()
        self.regions = n
        self.timed_as = "CUDA-graph replays of the K steps" if graph is not None else "stream of launches"
        return self._max_over_ranks(local)

    def sustained(self, seconds, ms_per_step, device_index):
        """Back-to-back launches for about `seconds`, with the clocks sampled: the power-capped steady state."""
        steps = int(max(10, min(20000, seconds * 1e3 / max(ms_per_step, 1e-3))))
        self.barrier()
        with ClockSampler(device_index) as clocks:
            ms = time_region(self.step, steps, self.stream)
            torch.cuda.synchronize()
        self.barrier()
        ms = self._max_over_ranks([ms])[0]
        return steps, ms, clocks.summary()


def library_yardsticks(dev):
    """Vendor-library GEMMs on this very GPU, as roofline denominators only (never on the product
    path): torch.matmul bf16, torch._scaled_mm fp8-e4m3 and torch._int_mm int8 at 8192^3, best of 10."""
    out = {}
    n = 8192
    flops = 2.0 * n * n * n
    stream = torch.cuda.current_stream(dev)

    def best(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        return min(time_region(lambda i: fn(), 1, stream) for _ in range(10))

    try:
        a = torch.randn(n, n, device=dev, dtype=torch.bfloat16)
        b = torch.randn(n, n, device=dev, dtype=torch.bfloat16)
        out["bf16"] = round(flops / (best(lambda: torch.matmul(a, b)) * 1e-3) / 1e12, 1)
    except Exception as e:
        out["bf16_error"] = f"{type(e).__name__}: {e}"[:120]
    try:
        a8 = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b8 = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        out["f8"] = round(flops / (best(lambda: torch._scaled_mm(a8, b8, scale_a=one, scale_b=one,
                                                                   out_dtype=torch.bfloat16)) * 1e-3) / 1e12, 1)
    except Exception as e:
        out["f8_error"] = f"{type(e).__name__}: {e}"[:120]
    try:
        ai = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
        bi = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
        out["i8"] = round(flops / (best(lambda: torch._int_mm(ai, bi)) * 1e-3) / 1e12, 1)
    except Exception as e:
        out["i8_error"] = f"{type(e).__name__}: {e}"[:120]
    torch.cuda.empty_cache()
    return out


def roofline_of(wl, ms_per_step, in_bytes, out_bytes, peaks, peak_src, yard, burst=True):
    """The `roofline` object of one workload from its device time per step."""
    tflops = wl.flops / (ms_per_step * 1e-3) / 1e12
    if wl.bound == "hbm":
        gbs = (in_bytes + out_bytes) / (ms_per_step * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": round(gbs, 1), "unit": "GB/s", "kernel": "gemm_tcgen05_kernel",
                "bytes_per_launch": in_bytes + out_bytes, "peak": peaks["hbm_gbs"],
                "peak_source": f"{peak_src} copy bandwidth"}
    else:
        roof = {"bound": "tensor", "achieved": round(tflops, 2), "unit": "TFLOP/s", "kernel": "gemm_tcgen05_kernel",
                "flops_per_launch": wl.flops}
        if wl.peak_key is None:
            roof["kernel"] = "matmul_int_kernel"
            roof["peak"] = None
            roof["peak_source"] = "no tensor-core form; bound by the software 128-bit multiply-add"
        elif wl.peak_key == "bf16":
            roof["peak"] = peaks["bf16_tflops"] if burst else peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
            roof["peak_source"] = f"{peak_src} cuBLAS bf16 8192^3 ({'burst' if burst else 'sustained'})"
        elif yard.get(wl.peak_key):
            roof["peak"] = yard[wl.peak_key]
            roof["peak_source"] = ("vendor-library GEMM of this operand type at 8192^3 timed in this run "
                                   "(torch._scaled_mm / torch._int_mm, best of 10)")
        else:
            roof["peak"] = NOMINAL_TFLOPS[wl.peak_key]
            roof["peak_source"] = "nominal dense peak (no measured figure for this type)"
        if wl.peak_key:
            roof["frac_of_nominal"] = round(tflops / NOMINAL_TFLOPS[wl.peak_key], 4)
    roof["frac"] = round(roof["achieved"] / roof["peak"], 4) if roof.get("peak") else None
    roof["traffic"] = ncu_traffic(wl.name if getattr(wl, "world", 1) == 1 else f"{wl.name}@{wl.world}")
    return roof


# ----------------------------------------------------------------------------- oracle legs
def _bits16(t):
    return t.view(torch.int16).numpy().view(np.uint16)


def oracle_rows(wl: Workload, rows, threads: int):
    """The CPU restatement of numr's path on the given rows of A (a count n = the first n rows, or an
    index array) against the whole B. Returns the oracle's output rows (storage arrays)."""
    from oracle import oracle as O   # only the checker / CPU-baseline legs of the benchmark execute the oracle

    idx = slice(0, rows) if isinstance(rows, int) else torch.as_tensor(rows)
    a = wl.a[idx]
    if wl.name == "c1":
        return O.gemm(O.F32, a.numpy(), wl.b.numpy(), bias=wl.bias.numpy(), act=O.ACT_GELU, threads=threads)
    if wl.name == "c2":
        return O.gemm(O.BF16, _bits16(a), _bits16(wl.w_nk), bias=_bits16(wl.bias), act=O.ACT_RELU,
                      b_transposed=True, threads=threads)
    if wl.name == "c3":
        return O.gemm(O.I8, a.numpy(), wl.b.numpy(), threads=threads)
    if wl.name == "c4":
        return O.fp8_matmul(a.view(torch.uint8).numpy(), wl.b.view(torch.uint8).numpy(), wl.scale_a,
                            wl.scale_b, O.BF16, bias=_bits16(wl.bias), residual=_bits16(wl.residual[idx]),
                            act=O.ACT_SILU, threads=threads)
    if wl.name == "s16":
        return O.gemm(O.BF16, _bits16(a), _bits16(wl.w_nk), b_transposed=True, threads=threads)
    if wl.name == "i32":
        return O.matmul_wide_int(a.numpy(), wl.b.numpy())
    if wl.name == "moe":
        # the first `rows` rows, each group's share of them against its own weight
        assert isinstance(rows, int)
        off = wl.offsets.numpy()
        outs = []
        for g in range(len(off) - 1):
            s, e = int(off[g]), min(int(off[g + 1]), rows)
            if e > s:
                outs.append(O.gemm(O.BF16, _bits16(wl.a[s:e]), _bits16(wl.b[g]), act=O.ACT_SILU, threads=threads))
        return np.concatenate(outs)
    return O.gemm(O.BF16, _bits16(a), _bits16(wl.b), act=O.ACT_SILU, threads=threads)


def parity_check(wl: Workload, client, dev_inputs, threads: int, n_rows: int = 64):
    """Outside every timed region: `n_rows` rows of this rank's output, spread over all row tiles,
    against the oracle on the same rows. Integers must be equal; 16-bit float outputs within one unit
    in the last place (the same f32 sums added in another order). Returns a summary or raises."""
    from oracle import oracle as O
    if wl.name == "moe":
        rows = n_rows
        idx = np.arange(n_rows)
    else:
        rng = np.random.default_rng(1234 + wl.rank)
        block = max(1, wl.m // n_rows)
        idx = np.unique(np.minimum(wl.m - 1, np.arange(min(n_rows, wl.m)) * block + rng.integers(0, block, min(n_rows, wl.m))))
        rows = idx
    out = wl.run(client, dev_inputs)
    got_t = out[torch.as_tensor(idx, device=out.device)].cpu()
    want = oracle_rows(wl, rows, threads)
    if got_t.dtype in (torch.int32, torch.int64):
        ok = np.array_equal(got_t.numpy(), want)
        return {"rows": int(len(idx)), "rule": "bit exact", "ok": bool(ok)}
    if got_t.dtype == torch.float32:
        g, w = got_t.numpy().astype(np.float64), want.astype(np.float64)
        err = float(np.linalg.norm(g - w) / max(np.linalg.norm(w), 1e-30))
        return {"rows": int(len(idx)), "rule": "relative Frobenius error vs the CPU f32 path <= 1e-5", "rel": err,
                "ok": bool(err <= 1e-5)}
    dt = O.BF16 if got_t.dtype == torch.bfloat16 else O.F16
    g = got_t.to(torch.float64).numpy()
    w = O.decode(want, dt).astype(np.float64)
    mag = np.maximum(np.abs(g), np.abs(w))
    ulp = np.exp2(np.floor(np.log2(np.where(mag > 0, mag, 1.0))) - (7 if dt == O.BF16 else 10))
    diff = np.abs(g - w)
    floor = 1e-6 * max(1.0, float(np.abs(w).max()))
    worst = float((np.maximum(diff - floor, 0) / ulp).max())
    frac = float((diff > floor).mean())
    return {"rows": int(len(idx)), "rule": "<= 1 ulp of the output type vs the CPU path, <= 5% of elements differing",
            "max_ulp": round(worst, 3), "differing": round(frac, 5), "ok": bool(worst <= 1.0 and frac <= 0.05)}


def cpu_run(wl: Workload, rows: int, threads: int) -> float:
    """Seconds the CPU path takes for the first `rows` rows of A."""
    t0 = time.perf_counter()
    oracle_rows(wl, rows, threads)
    return time.perf_counter() - t0


def cpu_sample(wl: Workload, budget_s: float, threads: int):
    """Times a bounded row-sample of the workload: grows the sample until it fills the budget."""
    rows = min(wl.m, 128)
    t = cpu_run(wl, rows, threads)           # also warms the library and the page cache
    t = cpu_run(wl, rows, threads)
    while rows < wl.m and t < budget_s / 4:
        grow = max(2, min(8, int(budget_s / 2 / max(t, 1e-4))))
        rows = min(wl.m, rows * grow)
        t = cpu_run(wl, rows, threads)
    flops = 2.0 * rows * wl.n * wl.k
    return rows, t, flops / t / 1e12


CPU_NOTE = ("C++ restatement of numr's CPU path (widen to f32, blocked GEMM in 128-column chunks over the host "
            "threads, epilogue, one narrowing); numr itself is Rust and cannot be built with the available toolchains")


def cpu_baseline(wl: Workload, budget_s: float):
    threads = host_threads()
    rows, secs, tflops = cpu_sample(wl, budget_s, threads)
    return {"value": round(tflops, 5), "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"first {rows} of {wl.m} rows of A against the whole B ({secs:.2f} s); {CPU_NOTE}"}


# ----------------------------------------------------------------------------- our arm
def summarise(region_ms, steps):
    per_step = sorted(ms / steps for ms in region_ms)
    return statistics.median(per_step), per_step[0]


def run_ours(args, world, rank, local):
    import torch.distributed as dist
    from numr_b200 import CudaClient

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback (use --impl reference)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    wl_name = args.workload if args.workload != "auto" else "c5"
    if world > 1 and wl_name != "c5":
        raise SystemExit("bench.py: only c5 shards over several GPUs")
    wl = Workload(wl_name, world, rank)
    client = CudaClient(local, f32_mode="exact")
    stream = torch.cuda.current_stream(dev)
    h = Harness(wl, client, dev, world, dist)
    status0 = client.device_status()

    # ---- kernel-only throughput: regions of exactly K steps, inputs resident in HBM
    with ClockSampler(local) as clocks:
        region_ms = h.timed_regions(args.steps, args.warmup)
    ms_per_step, ms_best = summarise(region_ms, args.steps)
    total_flops = wl.flops * world                      # every rank computes an equal column block
    value = total_flops / (ms_per_step * 1e-3) / 1e12
    clock_summary = clocks.summary()

    # ---- sustained leg: seconds of back-to-back launches (power-capped steady state)
    sustained = None
    if args.sustained_seconds > 0:
        s_steps, s_ms, s_clocks = h.sustained(args.sustained_seconds, ms_per_step, local)
        sustained = (s_steps, s_ms, s_clocks)

    # ---- end to end: every step copies its inputs from pinned host memory, runs the op through the
    # client, and reads the result back into pinned host memory. As a caller streaming batches would,
    # the three stages run on their own streams and overlap across steps (two buffers each).
    host = h.host
    sample_out = wl.run(client, h.sets[0])
    out_host = [torch.empty(sample_out.shape, dtype=sample_out.dtype).pin_memory() for _ in range(2)]
    dev_in = [{k: torch.empty_like(v, device=dev) for k, v in host.items()} for _ in range(2)]
    del sample_out
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def e2e_region(steps):
        """Runs `steps` pipelined steps; returns the CUDA-event time from first copy to last read-back."""
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_comp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        outs = [None, None]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record(stream)
        s_in.wait_stream(stream)
        s_out.wait_stream(stream)
        for i in range(steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_comp[b])          # the step that last read this input buffer is done
                for k, v in host.items():
                    dev_in[b][k].copy_(v, non_blocking=True)
                ev_in[b].record(s_in)
            stream.wait_event(ev_in[b])
            if i >= 2:
                stream.wait_event(ev_out[b])             # its output has been read back (frees the old output)
            outs[b] = wl.run(client, dev_in[b])
            ev_comp[b].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[b])
                outs[b].record_stream(s_out)
                out_host[b].copy_(outs[b], non_blocking=True)
                ev_out[b].record(s_out)
        stream.wait_stream(s_in)
        stream.wait_stream(s_out)
        stop.record(stream)
        stop.synchronize()
        return start.elapsed_time(stop)

    e2e_steps = args.steps
    e2e_region(min(args.warmup, 4))
    h.barrier()
    e2e_ms = e2e_region(e2e_steps)
    torch.cuda.synchronize()
    h.barrier()
    e2e_ms = h._max_over_ranks([e2e_ms])[0]
    e2e_value = total_flops / (e2e_ms / e2e_steps * 1e-3) / 1e12
    del dev_in, out_host

    # ---- optional all-gather of the output shards (c5, several GPUs), timed apart from the GEMM:
    # the collective plus the re-interleave of its [g, M, N/g] staging buffer into row-major [M, N]
    allgather_ms = None
    if world > 1:
        from numr_b200.sharding import all_gather_columns
        shard = wl.run(client, h.sets[0])
        for _ in range(3):
            full = all_gather_columns(shard)
        assert tuple(full.shape) == (wl.m, wl.n * world)
        del full
        h.barrier()
        ag = time_region(lambda i: all_gather_columns(shard), 10, stream)
        torch.cuda.synchronize()
        allgather_ms = h._max_over_ranks([ag / 10])[0]
        del shard

    # ---- the same step with the all-gather fused into the GEMM's epilogue: every finished tile is
    # stored into all ranks' row-major [M, N] buffers over NVLink (peer stores), followed by a
    # device-side barrier across the ranks; checked against the NCCL path's result
    fused = None
    if world > 1 and wl.name == "c5":
        try:
            from numr_b200 import GemmActivation
            from numr_b200.sharding import GatheredOutput, all_gather_columns
            gathered = GatheredOutput(wl.m, wl.n * world, torch.bfloat16, dev)

            def fused_step(i):
                t_in = h.sets[i % h.n_sets]
                client.matmul_activation_allgather(t_in["a"], t_in["b"], GemmActivation.SILU, gathered)
                gathered.barrier()

            fused_step(0)
            want_full = all_gather_columns(wl.run(client, h.sets[0]))
            h.barrier()
            same = bool(torch.equal(gathered.tensor.view(torch.int16), want_full.view(torch.int16)))
            del want_full
            for i in range(3):
                fused_step(i)
            h.barrier()
            f_steps = max(10, args.steps)
            f_ms = time_region(fused_step, f_steps, stream)
            torch.cuda.synchronize()
            h.barrier()
            f_ms = h._max_over_ranks([f_ms / f_steps])[0]
            same = h._max_over_ranks([0.0 if same else 1.0])[0] == 0.0
            out_bytes_peer = h.out_bytes * (world - 1)
            fused = {"ms_per_step": round(f_ms, 4), "equals_nccl_path": same,
                     "nvlink_bytes_out_per_gpu": out_bytes_peer,
                     "achieved_gbs_per_gpu": round(out_bytes_peer / (f_ms * 1e-3) / 1e9, 1),
                     "peak_gbs_per_gpu": 770.0, "peak_source": "measured peer copy per direction on this pool (900 nominal)",
                     "frac": round(out_bytes_peer / (f_ms * 1e-3) / 1e9 / 770.0, 4),
                     "what": "GEMM + SiLU with the epilogue storing every tile into all ranks' [M, N] buffers (peer "
                             "stores over NVLink), then a device-side barrier over the ranks"}
            del gathered
        except Exception as e:   # symmetric memory unavailable: the NCCL path above stands
            fused = {"error": f"{type(e).__name__}: {e}"[:300]}

    # ---- parity, outside every timed region: sampled rows of this rank's output against the oracle
    parity = parity_check(wl, client, h.sets[0], host_threads() // max(1, min(world, host_threads())) or 1)
    flags = h._max_over_ranks([0.0 if parity["ok"] else 1.0])
    status1 = client.device_status()
    if status0 != 0 or status1 != 0:
        raise SystemExit(f"bench.py: device status word {status0}/{status1}: a bounded wait ran out; number invalid")
    if not parity["ok"]:
        raise SystemExit(f"bench.py: rank {rank}: result differs from the oracle: {parity}")
    if flags[0] != 0.0:
        raise SystemExit("bench.py: another rank's result differs from the oracle; number invalid")

    line = None
    if rank == 0:
        peaks, peak_src = measured_peaks()
        yard = library_yardsticks(dev) if (world == 1 and not args.no_yardsticks) else {}
        roof = roofline_of(wl, ms_per_step, h.in_bytes, h.out_bytes, peaks, peak_src, yard, burst=True)
        line = {
            "metric": "GEMM+epilogue TFLOPS (whole job)", "value": round(value, 2), "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": config_of(wl, world),
            "timing": {"regions": h.regions, "steps_per_region": args.steps, "ms_per_step_median": round(ms_per_step, 5),
                       "ms_per_step_min": round(ms_best, 5), "timed_ms_total": round(sum(region_ms), 2),
                       "timed_as": h.timed_as,
                       "l2": f"{h.n_sets} rotating input sets + fresh outputs "
                             f"({h.n_sets * (h.in_bytes + h.out_bytes) / 1e6:.0f} MB) > 126 MB L2"},
            "clocks": clock_summary,
            "e2e": {"value": round(e2e_value, 3), "unit": "TFLOP/s", "h2d_bytes_per_step": h.in_bytes,
                    "d2h_bytes_per_step": h.out_bytes},
            "gpu_launches": wl.kernels_per_step() * args.steps * h.regions,
            "roofline": roof,
            "parity_checked": True, "parity": parity,
        }
        if clock_summary.get("sm_mhz"):
            line["timing"]["ms_x_mhz"] = round(ms_per_step * clock_summary["sm_mhz"], 2)
        if sustained is not None:
            s_steps, s_ms, s_clocks = sustained
            s_per = s_ms / s_steps
            s_tflops = wl.flops / (s_per * 1e-3) / 1e12
            sus = {"seconds": round(s_ms / 1e3, 2), "steps": s_steps, "ms_per_step": round(s_per, 5),
                   "value": round(s_tflops * world, 2), "per_gpu": round(s_tflops, 2), "unit": "TFLOP/s",
                   "clocks": s_clocks}
            if wl.peak_key == "bf16" and wl.bound == "tensor":
                sp = peaks.get("bf16_tflops_sustained")
                if sp:
                    sus["frac_of_sustained_peak"] = round(s_tflops / sp, 4)
                    sus["peak"] = sp
                    sus["peak_source"] = f"{peak_src} cuBLAS bf16 8192^3 back to back for seconds"
            if s_clocks.get("sm_mhz"):
                sus["ms_x_mhz"] = round(s_per * s_clocks["sm_mhz"], 2)
            line["sustained"] = sus
        if yard:
            line["yardsticks_tflops"] = yard
        if allgather_ms is not None:
            line["allgather_ms"] = round(allgather_ms, 4)
            line["allgather_includes"] = "NCCL all-gather + re-interleave of the [g, M, N/g] staging buffer to row-major [M, N]"
        if fused is not None:
            line["fused_allgather"] = fused
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(wl, budget_s=args.cpu_seconds)
    del h
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_other_configs and args.workload == "auto":
        line["configs"] = other_configs(client, wl_name, dev, local, peaks, peak_src, yard)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def other_configs(client, skip, dev, local, peaks, peak_src, yard):
    """Kernel-only figures of the single-GPU configurations next to the headline one, each timed like
    it (rotating sets, repeated regions, CUDA events), checked against the oracle on sampled rows, and
    set against its roofline."""
    out = {}
    steps_of = {"c1": 200, "c2": 50, "c3": 50, "c4": 20}
    for name in ("c1", "c2", "c3", "c4"):
        if name == skip:
            continue
        wl = Workload(name)
        h = Harness(wl, client, dev, set_budget=300e6)
        steps = steps_of[name]
        with ClockSampler(local) as clocks:
            region_ms = h.timed_regions(steps, 5, min_total_ms=30.0, min_regions=5, max_regions=20)
        ms, best = summarise(region_ms, steps)
        parity = parity_check(wl, client, h.sets[0], host_threads())
        if not parity["ok"]:
            raise SystemExit(f"bench.py: {name}: result differs from the oracle: {parity}")
        entry = {"workload": wl.desc, "dtype": wl.dtype, "ms_per_step": round(ms, 5), "ms_per_step_min": round(best, 5),
                 "value": round(wl.flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "steps": steps,
                 "regions": h.regions, "timed_as": h.timed_as, "gpu_launches": wl.kernels_per_step() * steps * h.regions,
                 "clocks": clocks.summary(), "parity": parity,
                 "roofline": roofline_of(wl, ms, h.in_bytes, h.out_bytes, peaks, peak_src, yard)}
        if wl.graph:
            # the same steps as a stream of launches through the client: what a caller without a graph sees
            for i in range(5):
                h.step(i)
            torch.cuda.synchronize()
            entry["ms_per_step_client"] = round(time_region(h.step, steps, h.stream) / steps, 5)
        out[name] = entry
        del h
        torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------- reference arm
def run_reference(args, world, rank):
    """numr's own CPU implementation of the path (its C++ restatement) on the host cores, on rank 0."""
    if rank != 0:
        return
    wl_name = args.workload if args.workload != "auto" else "c5"
    wl = Workload(wl_name, 1, 0)            # the CPU arm runs the whole problem on the host
    threads = host_threads()
    for _ in range(args.warmup):
        cpu_run(wl, min(wl.m, 64), threads)
    # Each step is a bounded row-sample sized so that all steps together take about a minute.
    rows, secs, tflops = cpu_sample(wl, min(10.0, 60.0 / max(args.steps + args.warmup, 1)), threads)
    times = [secs]
    for _ in range(args.steps - 1):
        times.append(cpu_run(wl, rows, threads))
    per_step = sum(times) / len(times)
    value = 2.0 * rows * wl.n * wl.k / per_step / 1e12
    sample = (f"each step = first {rows} of {wl.m} rows of A against the whole B on {threads} host threads "
              f"({per_step:.2f} s/step)")
    line = {
        "impl": "reference", "metric": "GEMM+epilogue TFLOPS (whole job)", "value": round(value, 5),
        "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(per_step * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": config_of(wl, world),
        "cpu_baseline": {"value": round(value, 5), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": sample + "; " + CPU_NOTE},
        "e2e": {"value": round(value, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["auto", "c1", "c2", "c3", "c4", "c5", "s16", "i32", "moe"], default="auto")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the CPU-baseline sample")
    ap.add_argument("--sustained-seconds", type=float, default=2.0, help="length of the sustained leg (0 = skip)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the c1..c4 figures of the default run")
    ap.add_argument("--no-yardsticks", action="store_true", help="skip timing the vendor-library GEMMs")
    args = ap.parse_args()
    world, rank, local = dist_env()
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("bench.py: --gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 3
        args.warmup = args.warmup if args.warmup is not None else 1
        run_reference(args, world, rank)
        return
    args.steps = args.steps if args.steps is not None else 20
    args.warmup = max(3, args.warmup if args.warmup is not None else 5)
    run_ours(args, world, rank, local)


if __name__ == "__main__":
    main()
