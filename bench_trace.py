"""Timeline of the single-token GEMV kernel inside a dense layer step.

Builds a variant of the library with -DB200Q_TUNING (kernels then stamp %globaltimer at their
milestones into a buffer named by B200Q_TRACE_PTR; the product build has none of this), replays
CUDA graphs of the layer's four launches and prints, per launch, when its CTAs entered, passed
griddepcontrol.wait, had their activation in registers, got their first tile, finished consuming,
and stored their last output - microseconds from the first CTA's entry, mean over CTAs.

    python bench_trace.py [chain|fused|plain|chain1]
    python bench_trace.py router [tokens]    # phases of the MoE router kernel (softmax, top-k, CSR)
        chain:  q|k|v, then o -> gate|up -> down as one launch (the default of a one-GPU layer)
        fused:  four launches, the quantizers inside them
        plain:  separate quantizer launch for down
        chain1: as chain, with q|k|v through the chain kernel too (one kernel image in the stream)

For a chained launch every call has its own line: "entry" is when the CTA's consumers reached the
call, "wait_done" when they saw every CTA's rows of the previous call stored.
"""
import importlib.util
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
spec = importlib.util.spec_from_file_location("b200q_build", os.path.join(ROOT, "sycl-infer_b200", "build.py"))
build = importlib.util.module_from_spec(spec)
spec.loader.exec_module(build)
os.environ["B200Q_LIB"] = build.build_tuning()
import torch  # noqa: E402

if len(sys.argv) > 1 and sys.argv[1] == "router":
    # MoE router: config 3's shape, host launches (router, then the token quantizer), stamps of the last call
    rt = torch.zeros(64 * 16, dtype=torch.int64, device="cuda")
    os.environ["B200Q_ROUTE_TRACE_PTR"] = str(rt.data_ptr())
    import __graft_entry__ as graft
    pkg = graft.load_package()
    from sycl_infer_b200 import moe as M
    be = pkg.make_cuda_backend(0)
    tokens = int(sys.argv[2]) if len(sys.argv) > 2 else 16
    _, bank = M.make_synthetic_moe(256, 8, 2048, 512, (12, 12, 12), seed=0, with_router=True)
    S = M.MoeScratch(bank, tokens)
    x = torch.from_numpy(pkg.synth.make_activation(tokens, 2048, 5)).cuda()
    for _ in range(6):
        rt.zero_()
        M.moe_router_csr_launch(be, bank.gate_inp, 0, x, x.shape[1], tokens, 2048, 256, 8, S.logits, S.ids, S.wts, S.off,
                                S.pair, S.active, S.n_active)
        M.moe_actq_launch(be, x, x.shape[1], tokens, 2048, *S.xq)
    be.synchronize()
    t = rt.cpu().numpy().reshape(64, 16)[:tokens].astype(np.float64)
    t0 = t[:, 0].min()
    print(f"moe_route_kernel, {tokens} tokens: microseconds from the first CTA's entry (mean / latest over the CTAs)")
    for k, nm in enumerate(["entry", "previous kernel done", "maximum", "exp", "sequential sum", "scaled", "rank count",
                            "ids written", "counted in", "CSR done (last CTA)"]):
        col = t[:, k][t[:, k] > 0]
        if col.size:
            print(f"  {nm:22s} {(col.mean() - t0) / 1e3:7.2f} {(col.max() - t0) / 1e3:7.2f}")
    sys.exit(0)

trace = torch.zeros(64 * 160 * 8, dtype=torch.int64, device="cuda")
os.environ["B200Q_TRACE_PTR"] = str(trace.data_ptr())
import __graft_entry__ as graft  # noqa: E402

pkg = graft.load_package()
from sycl_infer_b200.layer import DenseLayer  # noqa: E402

be = pkg.make_cuda_backend(0)
L = 4
layers = [DenseLayer(be, "Q4_K_M", seed=100 + i, TB=1) for i in range(L)]
xs = [torch.from_numpy(pkg.synth.make_activation(1, 5120, 10 + i)).cuda() for i in range(L)]
out = torch.zeros(1, 5120, device="cuda")
mode = sys.argv[1] if len(sys.argv) > 1 else "chain"
if mode == "chain1":
    os.environ["B200Q_CHAIN1"] = "1"
for ly in layers:
    ly.chain = mode in ("chain", "chain1")
    if mode == "plain":
        ly.fused_h = False
st = torch.cuda.Stream()
be._stream = st
with torch.cuda.stream(st):
    for i in range(L):
        layers[i].forward(xs[i], out)
    st.synchronize()
    graphs = []
    for i in range(L):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            layers[i].forward(xs[i], out)
        graphs.append(gr)
    st.synchronize()
    trace.zero_()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    for i in range(8):
        graphs[i % L].replay()
    e1.record(st)
    st.synchronize()
    print(f"{e0.elapsed_time(e1) / 8 * 1e3:.2f} us per layer step (tuning build, stamps on)")
t = trace.cpu().numpy().reshape(64, 160, 8).astype(np.float64)
if os.environ.get("B200Q_TRACE_SAVE"):  # the raw stamps, for a closer look than the means below
    np.save(os.environ["B200Q_TRACE_SAVE"], t)
idx = [i for i in range(64) if (t[i, :, 0] > 0).any()]  # a graph's kernel nodes keep the launch index of their capture
names = ["entry", "wait_done", "act_ready", "first_tile", "cons_done", "epi_done", "pre_wait", "act_landed"]
t0 = min(t[i, :, 0][t[i, :, 0] > 0].min() for i in idx)
rows = []
for i in idx:
    n = int((t[i, :, 0] > 0).sum())
    rows.append((t[i, :n, 0].min(), i, n, t[i, :n]))
rows.sort(key=lambda r: r[0])
print(f"mode={mode}: last replay of every captured launch; microseconds from the earliest entry (mean over CTAs)")
for _, i, n, c in rows:
    cells = []
    for k, nm in enumerate(names):
        col = c[:, k][c[:, k] > 0]
        cells.append(f"{nm}={((col.mean() - t0) / 1e3) if col.size else float('nan'):7.2f}")
    last = c[:, 5][c[:, 5] > 0]
    print(f"launch {i:2d} ctas={n:3d} " + "  ".join(cells) + f"  last_store={((last.max() - t0) / 1e3) if last.size else float('nan'):7.2f}")
