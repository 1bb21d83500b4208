"""Micro-benchmark of one routed-MoE FFN (router, CSR, quantize, grouped gate|up, quantize,
grouped down, reduce) through the C ABI: CUDA graph of back-to-back calls over rotating expert
banks (larger than L2 in total), CUDA-event timing.

    python bench_moe.py [--tokens 16] [--experts 256] [--topk 8] [--embd 2048] [--ff 512]
"""
import argparse, sys, os, numpy as np, torch
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import __graft_entry__ as g
pkg = g.load_package()
from sycl_infer_b200.moe import MoeScratch, make_synthetic_moe, moe_call
ap = argparse.ArgumentParser()
ap.add_argument("--tokens", type=int, default=16); ap.add_argument("--experts", type=int, default=256)
ap.add_argument("--topk", type=int, default=8); ap.add_argument("--embd", type=int, default=2048)
ap.add_argument("--ff", type=int, default=512); ap.add_argument("--type", type=int, default=12)
ap.add_argument("--copies", type=int, default=2); ap.add_argument("--iters", type=int, default=20)
a = ap.parse_args()
be = pkg.make_cuda_backend(0)
banks = [make_synthetic_moe(a.experts, a.topk, a.embd, a.ff, (a.type,) * 3, seed=i, with_router=True)[1]
         for i in range(a.copies)]
S = MoeScratch(banks[0], a.tokens)
x = torch.from_numpy(pkg.synth.make_activation(a.tokens, a.embd, 5)).cuda()
out = torch.zeros(a.tokens, a.embd, device="cuda")
st = torch.cuda.Stream()
be._stream = st
graph = torch.cuda.CUDAGraph()
with torch.cuda.stream(st):
    for i in range(2): moe_call(be, banks[i % a.copies], S, x, a.tokens, out)
    st.synchronize()
    with torch.cuda.graph(graph, stream=st):
        for i in range(a.iters): moe_call(be, banks[i % a.copies], S, x, a.tokens, out)
    graph.replay(); st.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    graph.replay()
    e1.record(st); st.synchronize()
us = 1e3 * e0.elapsed_time(e1) / a.iters
n_active = int(S.n_active.cpu()[0])
per_expert = sum(int(pkg.synth.row_bytes(a.type, K)) * rows for rows, K in ((a.ff, a.embd), (a.ff, a.embd), (a.embd, a.ff)))
nbytes = n_active * per_expert
print(f"moe tokens={a.tokens} experts={a.experts} top{a.topk} embd={a.embd} ff={a.ff} type={a.type}: {us:.1f} us/call  "
      f"{n_active} active experts  {nbytes/1e6:.1f} MB  {nbytes/us/1e3:.0f} GB/s  ({100*nbytes/us/1e3/6537:.1f}% of measured)  "
      f"status={be.device_status()}")
