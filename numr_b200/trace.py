"""Timeline of one GEMM launch: where the first CTAs of gemm_tcgen05_kernel spend their time.

Needs the trace build of the library (`python -m numr_b200.build --trace`), whose kernel writes the
global timer and the SM cycle counter of its first 8 CTAs at fixed points of their life. This script
loads that build, runs the problem a few thousand times to bring the clocks up, then prints the marks
of the last of four back-to-back launches (operands rotate over four sets), in microseconds after the
earliest CTA's entry:

    python -m numr_b200.trace bf16 1024 1024 1024 kn --act gelu --bias
    python -m numr_b200.trace f32 1024 1024 1024 kn --act gelu --bias
    python -m numr_b200.trace bf16 16 4096 4096 nk --act gelu --bias
    python -m numr_b200.trace bf16 4096 4096 4096 nk --act gelu --bias --warm 300

Columns: entry, set-up done, dependencies met (producer), first load issued, first stage full (MMA
issuer), last MMA issued, first accumulator seen (epilogue warp of TMEM lanes 0-31), its last store
issued, stores read, TMEM freed, then the start of the issuer's first six work units.
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

MARKS = ["entry", "setup", "deps", "1st_load", "1st_full", "last_mma", "1st_acc", "last_store", "stores_read",
         "done", "unit0", "unit1", "unit2", "unit3", "unit4", "unit5"]


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("dtype", choices=["bf16", "f16", "f32", "i8"])
    ap.add_argument("m", type=int)
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int)
    ap.add_argument("layout", choices=["kn", "nk"], help="B as [K,N], or as [N,K] read through its transposed view")
    ap.add_argument("--act", choices=["none", "relu", "gelu", "silu"], default="none")
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--warm", type=int, default=3000, help="untimed launches before the traced ones")
    ap.add_argument("--tf32", action="store_true", help="F32 operands in TF32 mode instead of the exact mode")
    args = ap.parse_args()

    from . import build as _build
    if "NUMR_B200_LIBRARY" not in os.environ:
        if not _build.TRACE_LIB_PATH.exists():
            _build.build(trace=True)
        os.environ["NUMR_B200_LIBRARY"] = str(_build.TRACE_LIB_PATH)
    import torch
    from . import CudaClient, GemmActivation, _lib

    if not torch.cuda.is_available():
        print("numr_b200.trace needs a CUDA device", file=sys.stderr)
        return 2
    dev = torch.device("cuda:0")
    lib = _lib.load()
    client = CudaClient(0, "tf32" if args.tf32 else "exact")
    trace = torch.zeros(256, dtype=torch.int64, device=dev)
    os.environ["NUMR_B200_TRACE_PTR"] = hex(trace.data_ptr())
    lib.numr_b200_reload_tuning()

    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "i8": torch.int8}[args.dtype]
    act = {"none": GemmActivation.NONE, "relu": GemmActivation.RELU, "gelu": GemmActivation.GELU,
           "silu": GemmActivation.SILU}[args.act]
    m, n, k = args.m, args.n, args.k
    sets = []
    for _ in range(4):
        if dt == torch.int8:
            a = torch.randint(-127, 128, (m, k), device=dev, dtype=torch.int8)
            b = torch.randint(-127, 128, (k, n), device=dev, dtype=torch.int8)
            sets.append((a, b, None))
            continue
        a = torch.randn((m, k), device=dev).to(dt)
        if args.layout == "nk":
            b = (torch.randn((n, k), device=dev) * 0.05).to(dt).t()
        else:
            b = (torch.randn((k, n), device=dev) * 0.05).to(dt)
        sets.append((a, b, torch.randn(n, device=dev).to(dt) if args.bias else None))

    def step(i):
        a, b, bias = sets[i % 4]
        if bias is not None:
            return client.matmul_bias_activation(a, b, bias, act)
        if act != GemmActivation.NONE:
            return client.matmul_activation(a, b, act)
        return client.matmul(a, b)

    for i in range(args.warm):
        step(i)
    torch.cuda.synchronize()
    trace.zero_()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(4):
        step(i)
    e1.record()
    e1.synchronize()
    marks = trace.cpu().numpy().reshape(8, 16, 2)
    ns, cyc = marks[:, :, 0], marks[:, :, 1]
    seen = ns[:, 0] > 0
    if not seen.any():
        print("no marks were written: is NUMR_B200_LIBRARY the trace build?", file=sys.stderr)
        return 1
    base = ns[seen, 0].min()
    print(f"{args.dtype} {m} x {n} x {k} {args.layout} act={args.act} bias={int(args.bias)}: 4 launches in "
          f"{e0.elapsed_time(e1) * 1e3:.1f} us; marks of the last one, us after the earliest CTA's entry")
    if ns[0, 7] > ns[0, 1]:
        print(f"SM clock of CTA 0 between set-up and last store: "
              f"{(cyc[0, 7] - cyc[0, 1]) / (ns[0, 7] - ns[0, 1]) * 1e3:.0f} MHz")
    print("cta " + " ".join(f"{x:>11s}" for x in MARKS))
    for c in range(8):
        if not seen[c]:
            continue
        print(f"{c:3d} " + " ".join(f"{(ns[c, e] - base) / 1e3:11.2f}" if ns[c, e] else f"{'-':>11s}"
                                    for e in range(16)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
