"""Micro-benchmark of one routed-MoE FFN (router, CSR, quantize, grouped gate|up, quantize,
grouped down, reduce) through the C ABI: CUDA graph of back-to-back calls over rotating expert
banks (larger than L2 in total), CUDA-event timing.

    python bench_moe.py [--tokens 16] [--experts 256] [--topk 8] [--embd 2048] [--ff 512] [--parts]

--parts also times every stage of the call on its own (a graph of back-to-back launches of that
stage alone, same rotating banks): where a call's time goes.
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
ap.add_argument("--parts", action="store_true")
ap.add_argument("--fused-hq", action="store_true", help="gate|up quantizes h in its epilogue (one launch less)")
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
    for i in range(2): moe_call(be, banks[i % a.copies], S, x, a.tokens, out, fused_hq=a.fused_hq)
    st.synchronize()
    with torch.cuda.graph(graph, stream=st):
        for i in range(a.iters): moe_call(be, banks[i % a.copies], S, x, a.tokens, out, fused_hq=a.fused_hq)
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

if a.parts:
    from sycl_infer_b200 import moe as M

    def timed(fn):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.stream(st):
            fn(0)
            st.synchronize()
            with torch.cuda.graph(gr, stream=st):
                for i in range(a.iters):
                    fn(i)
            gr.replay(); st.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(st); gr.replay(); t1.record(st); st.synchronize()
        return 1e3 * t0.elapsed_time(t1) / a.iters

    n_pairs = a.tokens * a.topk
    nmax = min(a.experts, n_pairs)
    B = lambda i: banks[i % a.copies]  # noqa: E731
    parts = [
        ("router + CSR (2 launches)", lambda i: M.moe_router_csr_launch(be, B(i).gate_inp, 0, x, x.shape[1], a.tokens, a.embd,
                                                                        a.experts, a.topk, S.logits, S.ids, S.wts, S.off,
                                                                        S.pair, S.active, S.n_active)),
        ("softmax/top-k + CSR from given logits", lambda i: M.moe_router_csr_launch(be, None, 0, x, x.shape[1], a.tokens, a.embd,
                                                                                    a.experts, a.topk, S.logits, S.ids, S.wts,
                                                                                    S.off, S.pair, S.active, S.n_active)),
        ("quantize tokens", lambda i: M.moe_actq_launch(be, x, x.shape[1], a.tokens, a.embd, *S.xq)),
        ("gate|up + quantize h (1 launch)", lambda i: M.moe_grp_gate_up_q_launch(be, B(i), S.off, S.pair, S.active, S.n_active,
                                                                               nmax, *S.xq, a.tokens, S.h, a.ff, *S.hq)),
        ("gate|up", lambda i: M.moe_grp_gate_up_launch(be, B(i), S.off, S.pair, S.active, S.n_active, nmax, *S.xq, a.tokens,
                                                       S.h, a.ff)),
        ("quantize h", lambda i: M.moe_actq_launch(be, S.h, a.ff, n_pairs, a.ff, *S.hq)),
        ("down", lambda i: M.moe_grp_down_launch(be, B(i), S.off, S.pair, S.active, S.n_active, nmax, *S.hq, n_pairs, S.acc,
                                                 a.embd)),
        ("reduce", lambda i: M.moe_reduce_launch(be, S.acc, S.wts, a.topk, a.tokens, a.embd, a.embd, out, out.shape[1])),
    ]
    for name, fn in parts:
        print(f"  {name:34s} {timed(fn):7.2f} us")
    # the same stages in call order, cumulatively: what each one adds when it has to wait for the one before
    seq = [parts[2], parts[0], parts[4], parts[5], parts[6], parts[7]]
    prev = 0.0
    for n in range(1, len(seq) + 1):
        t = timed(lambda i: [fn(i) for _, fn in seq[:n]])
        print(f"  in sequence, up to {seq[n - 1][0]:30s} {t:7.2f} us  (+{t - prev:.2f})")
        prev = t
    print(f"  status={be.device_status()}")
