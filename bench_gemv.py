"""Micro-benchmark of one GEMV shape through the C ABI: rotating weight copies (larger than L2
in total), a CUDA graph of back-to-back launches, CUDA-event timing.

    python bench_gemv.py --type 12 --rows 17408 --K 5120 [--TB 1] [--fused 1]
"""
import argparse, sys, os, numpy as np, torch
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import __graft_entry__ as g
pkg = g.load_package()
from sycl_infer_b200.backend import gemv_seg, alloc_act
ap = argparse.ArgumentParser()
ap.add_argument("--type", type=int, default=12); ap.add_argument("--rows", type=int, default=17408)
ap.add_argument("--K", type=int, default=5120); ap.add_argument("--TB", type=int, default=1)
ap.add_argument("--copies", type=int, default=4); ap.add_argument("--iters", type=int, default=50)
ap.add_argument("--warm", type=int, default=3); ap.add_argument("--fused", type=int, default=0)
a = ap.parse_args()
be = pkg.make_cuda_backend(0)
w0 = pkg.synth.make_weight(a.type, a.rows, a.K, 1)
ws = [torch.from_numpy(w0).cuda() for _ in range(a.copies)]
for i, w in enumerate(ws): w[:64] = i  # distinct content irrelevant; distinct addresses matter
x = torch.from_numpy(pkg.synth.make_activation(a.TB, a.K, 2)).cuda()
x8, xm, xs = alloc_act(a.TB, a.K)
be.xq(x, None, a.K, a.K, x8, xm, xs, None, a.TB, a.K)
out = torch.zeros(a.TB * a.rows, dtype=torch.float32, device="cuda")
segs = [gemv_seg(w=w, type=a.type, K=a.K, n_rows=a.rows, x=x, x_stride=a.K, out=out, out_stride=a.rows, x8=x8, xmeta=xm, xsumq=xs) for w in ws]
def run(i):
    if a.fused: be.quant_gemv([segs[i % a.copies]], a.TB)
    elif a.TB == 1: be.i8_gemv(segs[i % a.copies])
    else: be.i8_gemm(segs[i % a.copies], a.TB)
for i in range(a.warm): run(i)
torch.cuda.synchronize()
st = torch.cuda.Stream()
be._stream = st
graph = torch.cuda.CUDAGraph()
with torch.cuda.stream(st):
    for i in range(2): run(i)
    st.synchronize()
    with torch.cuda.graph(graph, stream=st):
        for i in range(a.iters): run(i)
    graph.replay(); st.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    graph.replay()
    e1.record(st); st.synchronize()
us = 1e3 * e0.elapsed_time(e1) / a.iters
nbytes = w0.size
print(f"type={a.type} rows={a.rows} K={a.K} TB={a.TB} fused={a.fused}: {us:.2f} us/launch  {nbytes/us/1e3:.0f} GB/s  ({100*nbytes/us/1e3/6537:.1f}% of measured)  status={be.device_status()}")
