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
`auto` runs c2 on one GPU (the BF16 GEMM+epilogue configuration) and c5 on several.
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
        self.desc = (f"c5: BF16 X[16384,4096] @ W[4096,14336] + SiLU, W split along N over {self.world} "
                     f"GPU(s) ({shard} columns each), no reduction")

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
        # c1 prepares both F32 operands (one split kernel each) before the GEMM kernel; the grouped
        # matmul runs its plan kernel first
        return {"c1": 3, "moe": 2}.get(self.name, 1)


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


def time_region(fn, steps, stream):
    """CUDA-event time of `steps` calls of fn(i) on `stream`, in ms."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        fn(i)
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1)


# ----------------------------------------------------------------------------- our arm
def run_ours(args, world, rank, local):
    import torch.distributed as dist
    from numr_b200 import CudaClient

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback (use --impl reference)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    wl_name = args.workload if args.workload != "auto" else ("c2" if world == 1 else "c5")
    if world > 1 and wl_name != "c5":
        raise SystemExit("bench.py: only c5 shards over several GPUs")
    wl = Workload(wl_name, world, rank)
    client = CudaClient(local, f32_mode="exact")
    stream = torch.cuda.current_stream(dev)

    host = {k: v.pin_memory() for k, v in wl.host_inputs().items()}
    in_bytes = sum(v.numel() * v.element_size() for v in host.values())
    # Rotating input sets larger than the 126 MB L2, so no timed step finds its operands cached.
    out_probe = wl.run(client, {k: v.to(dev) for k, v in host.items()})
    out_bytes = out_probe.numel() * out_probe.element_size()
    n_sets = max(2, -(-int(400e6) // (in_bytes + out_bytes)))
    sets = [{k: v.to(dev, non_blocking=True) for k, v in host.items()} for _ in range(n_sets)]
    del out_probe
    torch.cuda.synchronize()
    status0 = client.device_status()

    def step(i):
        return wl.run(client, sets[i % n_sets])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    graph = None
    if wl.graph:
        # Launch-bound workload: the K timed steps (each on its own input set) are captured once and
        # replayed, so the CUDA events bracket kernels, not the Python call overhead.
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(args.steps):
                step(i)
        graph.replay()
        torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        if graph is not None:
            ms = time_region(lambda i: graph.replay() if i == 0 else None, args.steps, stream)
        else:
            ms = time_region(step, args.steps, stream)
        torch.cuda.synchronize()
    barrier()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    ms_per_step = ms_max / args.steps
    total_flops = wl.flops * world                      # every rank computes an equal column block
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end: every step copies its inputs from pinned host memory, runs the op through the
    # client, and reads the result back into pinned host memory. As a caller streaming batches would,
    # the three stages run on their own streams and overlap across steps (two buffers each).
    sample_out = wl.run(client, sets[0])
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
    barrier()
    e2e_ms = e2e_region(e2e_steps)
    torch.cuda.synchronize()
    barrier()
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = total_flops / (float(t.item()) / e2e_steps * 1e-3) / 1e12

    # ---- optional all-gather of the output shards (c5, several GPUs), timed apart from the GEMM
    allgather_ms = None
    if world > 1:
        shard = wl.run(client, sets[0])
        gathered = torch.empty((world * shard.shape[0], shard.shape[1]), dtype=shard.dtype, device=dev)
        for _ in range(3):
            dist.all_gather_into_tensor(gathered, shard)
        barrier()
        ag = time_region(lambda i: dist.all_gather_into_tensor(gathered, shard), 10, stream)
        torch.cuda.synchronize()
        t = torch.tensor([ag / 10], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        allgather_ms = float(t.item())

    status1 = client.device_status()
    if status0 != 0 or status1 != 0:
        raise SystemExit(f"bench.py: device status word {status0}/{status1}: a bounded wait ran out; number invalid")

    line = None
    if rank == 0:
        peaks, peak_src = measured_peaks()
        # A short timed region (tens of ms) is a burst; a long one runs under the power cap.
        burst = ms_max < 1500.0
        peak_bf16 = peaks["bf16_tflops"] if burst else peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        per_gpu_tflops = wl.flops / (ms_per_step * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": round(per_gpu_tflops, 2), "unit": "TFLOP/s",
                "kernel": "gemm_tcgen05_kernel", "flops_per_launch": wl.flops,
                "traffic": ncu_traffic(wl_name)}
        if wl.bound == "hbm":
            gbs = (in_bytes + out_bytes) / (ms_per_step * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": round(gbs, 1), "unit": "GB/s", "kernel": "gemm_tcgen05_kernel",
                    "bytes_per_launch": in_bytes + out_bytes, "traffic": ncu_traffic(wl_name),
                    "peak": peaks["hbm_gbs"], "peak_source": f"{peak_src} copy bandwidth"}
        elif wl.peak_key is None:
            roof["kernel"] = "matmul_int_kernel"
            roof["peak"] = None
            roof["peak_source"] = "no tensor-core form; bound by the software 128-bit multiply-add"
        elif wl.peak_key == "bf16":
            roof["peak"] = peak_bf16
            roof["peak_source"] = f"{peak_src} cuBLAS bf16 ({'burst' if burst else 'sustained'})"
        else:
            # no measured yardstick exists for this operand type: nominal dense peak
            roof["peak"] = NOMINAL_TFLOPS[wl.peak_key]
            roof["peak_source"] = "nominal dense peak (no measured figure for this type)"
        roof["frac"] = round(roof["achieved"] / roof["peak"], 4) if roof["peak"] else None
        if wl.bound == "tensor" and wl.peak_key:
            roof["frac_of_nominal"] = round(per_gpu_tflops / NOMINAL_TFLOPS[wl.peak_key], 4)
        line = {
            "metric": "GEMM+epilogue TFLOPS (whole job)", "value": round(value, 2), "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": {"workload": wl.desc, "m": wl.m, "n_per_gpu": wl.n, "k": wl.k,
                       "l2": f"{n_sets} rotating input/output sets ({n_sets * (in_bytes + out_bytes) / 1e6:.0f} MB) "
                             f"> 126 MB L2"},
            "clocks": clocks.summary(),
            "e2e": {"value": round(e2e_value, 3), "unit": "TFLOP/s", "h2d_bytes_per_step": in_bytes,
                    "d2h_bytes_per_step": out_bytes},
            "gpu_launches": wl.kernels_per_step() * args.steps,
            "timed_as": "one CUDA graph of the K steps" if graph is not None else "stream of launches",
            "roofline": roof,
        }
        if allgather_ms is not None:
            line["allgather_ms"] = round(allgather_ms, 4)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(wl, budget_s=args.cpu_seconds)
        if world == 1 and args.all_configs:
            line["other_configs"] = other_configs(client, wl_name, dev)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def other_configs(client, skip, dev):
    """Kernel-only TFLOPS of the remaining single-GPU configurations (short runs, rotating sets)."""
    out = {}
    stream = torch.cuda.current_stream(dev)
    for name in ("c1", "c3", "c4", "c5"):
        if name == skip:
            continue
        wl = Workload(name)
        host = wl.host_inputs()
        in_bytes = sum(v.numel() * v.element_size() for v in host.values())
        n_sets = max(2, min(8, -(-int(300e6) // in_bytes)))
        sets = [{k: v.to(dev) for k, v in host.items()} for _ in range(n_sets)]
        steps = 200 if name == "c1" else 20
        for i in range(3):
            wl.run(client, sets[i % n_sets])
        torch.cuda.synchronize()
        ms = time_region(lambda i: wl.run(client, sets[i % n_sets]), steps, stream) / steps
        tf = wl.flops / (ms * 1e-3) / 1e12
        out[name] = {"workload": wl.desc, "ms_per_step": round(ms, 5), "tflops": round(tf, 2),
                     "frac_of_nominal": round(tf / NOMINAL_TFLOPS[wl.peak_key], 4)}
        del sets
        torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------- CPU baseline / reference arm
def cpu_run(wl: Workload, rows: int, threads: int) -> float:
    """Runs the CPU restatement of numr's path on the first `rows` rows of A; returns seconds."""
    from oracle import oracle as O   # the one place the benchmark executes the oracle: as the CPU baseline

    def bits16(t):
        return t.view(torch.int16).numpy().view(np.uint16)

    t0 = time.perf_counter()
    if wl.name == "c1":
        O.gemm(O.F32, wl.a[:rows].numpy(), wl.b.numpy(), bias=wl.bias.numpy(), act=O.ACT_GELU, threads=threads)
    elif wl.name == "c2":
        O.gemm(O.BF16, bits16(wl.a[:rows]), bits16(wl.w_nk), bias=bits16(wl.bias), act=O.ACT_RELU,
               b_transposed=True, threads=threads)
    elif wl.name == "c3":
        O.gemm(O.I8, wl.a[:rows].numpy(), wl.b.numpy(), threads=threads)
    elif wl.name == "c4":
        O.fp8_matmul(wl.a[:rows].view(torch.uint8).numpy(), wl.b.view(torch.uint8).numpy(), wl.scale_a,
                     wl.scale_b, O.BF16, bias=bits16(wl.bias), residual=bits16(wl.residual[:rows]),
                     act=O.ACT_SILU, threads=threads)
    elif wl.name == "s16":
        O.gemm(O.BF16, bits16(wl.a[:rows]), bits16(wl.w_nk), b_transposed=True, threads=threads)
    elif wl.name == "i32":
        O.matmul_wide_int(wl.a[:rows].numpy(), wl.b.numpy())
    elif wl.name == "moe":
        # the first `rows` rows, each group's share of them against its own weight
        off = wl.offsets.numpy()
        for g in range(len(off) - 1):
            s, e = int(off[g]), min(int(off[g + 1]), rows)
            if e > s:
                O.gemm(O.BF16, bits16(wl.a[s:e]), bits16(wl.b[g]), act=O.ACT_SILU, threads=threads)
    else:
        O.gemm(O.BF16, bits16(wl.a[:rows]), bits16(wl.b), act=O.ACT_SILU, threads=threads)
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


def cpu_baseline(wl: Workload, budget_s: float):
    from oracle import oracle as O
    threads = O.max_threads()
    rows, secs, tflops = cpu_sample(wl, budget_s, threads)
    return {"value": round(tflops, 5), "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"first {rows} of {wl.m} rows of A against the whole B ({secs:.2f} s); C++ restatement of "
                      f"numr's CPU path (widen to f32, blocked GEMM in 128-column chunks over all threads, "
                      f"epilogue, one narrowing); numr itself is Rust and cannot be built here"}


def run_reference(args, world, rank):
    if rank != 0:
        return
    wl_name = args.workload if args.workload != "auto" else ("c2" if world == 1 else "c5")
    wl = Workload(wl_name, 1, 0)            # the CPU arm runs the whole problem on the host
    from oracle import oracle as O
    threads = O.max_threads()
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
        "config": {"workload": wl.desc, "m": wl.m, "n_per_gpu": wl.n, "k": wl.k},
        "cpu_baseline": {"value": round(value, 5), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": sample + "; C++ restatement of numr's CPU path (numr is Rust and cannot be "
                                            "built with the available toolchains)"},
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
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--all-configs", action="store_true", help="also time the other single-GPU configurations")
    args = ap.parse_args()
    world, rank, local = dist_env()
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("bench.py: --gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 3
        args.warmup = args.warmup if args.warmup is not None else 1
        run_reference(args, world, rank)
        return
    args.steps = args.steps if args.steps is not None else 200
    args.warmup = max(3, args.warmup if args.warmup is not None else 10)
    run_ours(args, world, rank, local)


if __name__ == "__main__":
    main()
