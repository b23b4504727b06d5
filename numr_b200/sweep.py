"""BF16 matmul over a grid of shapes, CUDA-graph replays, beside torch.matmul (the vendor library) on the same
operands: finds the shapes where this library's heuristics or fixed costs lose.

    python -m numr_b200.sweep nk      # B given as [N, K] and read through its transposed view
    python -m numr_b200.sweep kn      # B given as [K, N]

Prints, per (N, K) and per M, microseconds per call of this library / of torch.matmul and their ratio. The
vendor library is only the yardstick here; nothing in the library calls it."""
import sys, time
import torch
from . import CudaClient
dev = torch.device("cuda:0"); client = CudaClient(0)
def graph_time(fn, nsets, steps=20, reps=5):
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for i in range(max(nsets,3)): fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(steps): fn(i)
        g.replay(); torch.cuda.synchronize()
        ts=[]
        for r in range(reps):
            e0,e1=torch.cuda.Event(enable_timing=True),torch.cuda.Event(enable_timing=True)
            e0.record(s); g.replay(); e1.record(s); e1.synchronize(); ts.append(e0.elapsed_time(e1)/steps)
    ts.sort(); return ts[len(ts)//2]*1e3
layout = sys.argv[1] if len(sys.argv) > 1 else "nk"
print(f"bf16, B as {layout}; us per call in a CUDA graph: ours / torch.matmul (ratio)")
for (n,k) in [(4096,4096),(4096,14336),(14336,4096),(8192,8192),(1024,1024),(2048,2048),(512,4096),(4096,512)]:
    nsets = max(2, min(8, int(300e6 // (n*k*2)) + 1))
    if layout == "nk": ws = [(torch.randn((n,k),device=dev)*0.05).to(torch.bfloat16).t() for _ in range(nsets)]
    else: ws = [(torch.randn((k,n),device=dev)*0.05).to(torch.bfloat16) for _ in range(nsets)]
    row=[]
    for m in (1,16,33,64,128,256,512,1024,2048,4096):
        a = torch.randn((m,k),device=dev).to(torch.bfloat16)
        t1 = graph_time(lambda i: client.matmul(a, ws[i % nsets]), nsets)
        t2 = graph_time(lambda i: torch.matmul(a, ws[i % nsets]), nsets)
        row.append(f"M={m}: {t1:.1f}/{t2:.1f} ({t1/t2:.2f})")
    print(f"N={n} K={k}: " + "  ".join(row), flush=True)
