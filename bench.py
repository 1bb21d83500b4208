"""Benchmark of the quantized-GEMV hot path.

Headline workload = benchmark configuration 1, batch 1: hidden 5120, 40 query / 8 KV heads of
dim 128, FFN 17408, Q/K/O/gate/up in Q4_K, V/down in Q6_K (the "Q4_K_M" mix), seeded synthetic
blocks.  One step = one layer pass = four calls (q|k|v, o, gate|up, down), each ONE launch that
quantizes its activation and streams its weights.  Steps rotate over `--layers` distinct weight
sets of 210 MB each, so every step streams weights that are not in the 126 MB L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-cells]

Prints ONE JSON line (rank 0).  `value` is weight-stream GB/s with all inputs resident in HBM;
`e2e` is the same through the host-buffer call sequence (pinned H2D of the step's activations,
D2H of its output, every step); `roofline` is the GEMV kernel alone against the measured HBM copy
bandwidth; `cpu_baseline` is the reference's own CPU path on this machine's cores; `cells` holds
the other configurations (config 0, config 1 batch 16, config 2, config 3 on one GPU; batch 1 and
32 x three type mixes x {peer-store, NCCL all-gather, layer split} on several).  `--impl
reference` times the CPU path as the headline instead.
"""
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
import __graft_entry__ as graft  # noqa: E402

METRIC = "quant_gemv_effective_hbm_gbs"
WORKLOAD = "dense layer GEMV set, Q4_K_M mix (hidden 5120, 40q/8kv x128, ffn 17408), batch 1"
LAYERS_PER_TOKEN = 64
DTYPE = "int8xu4/u6->int32, fp32 scales"
# dram__bytes_read.sum + dram__bytes_write.sum per GEMV launch of one layer step: from the ncu capture
# summarised in profiles/gemv_pinned_layer_q4km_batch1.md (not re-measured by this program)
TRAFFIC_NOTE = "profiles/gemv_pinned_layer_q4km_batch1.md"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def ncu_traffic_per_launch():
    """The figure the profile summary records, if it is there: 'traffic_bytes_per_launch: N'."""
    p = os.path.join(ROOT, TRAFFIC_NOTE)
    try:
        for line in open(p):
            if line.startswith("traffic_bytes_per_launch:"):
                return float(line.split(":", 1)[1])
    except OSError:
        pass
    return None


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.stop_flag = index, [], threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                self.rows.append([c.strip() for c in out.strip().split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.05)

    def summary(self):
        self.stop_flag.set()
        self.join(timeout=6)
        sm = [float(r[0]) for r in self.rows if len(r) == 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) == 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) == 6 for n, v in zip(names, r[2:]) if v == "Active"})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------ CPU reference arm
def cpu_layer_pass(ref, pkg, weights, x, attn):
    """One layer pass on the reference's CPU integer path (cpu_xq + cpu_i8_gemv)."""
    sh = {n: (t, r, k) for n, t, r, k in pkg.synth.dense_layer_shapes("Q4_K_M")}
    a = ref.xq(x)
    q = [ref.gemv(sh[n][0], weights[n], sh[n][2], sh[n][1], a) for n in ("q", "k", "v")]
    o = ref.gemv(sh["o"][0], weights["o"], sh["o"][2], sh["o"][1], ref.xq(attn))
    a2 = ref.xq(o)
    g = ref.gemv(sh["gate"][0], weights["gate"], sh["gate"][2], sh["gate"][1], a2)
    u = ref.gemv(sh["up"][0], weights["up"], sh["up"][2], sh["up"][1], a2)
    y = ref.gemv(sh["down"][0], weights["down"], sh["down"][2], sh["down"][1], ref.xq(g, u), residual=x[0].copy())
    return y, q


def cpu_arm(steps, warmup, budget_s=25.0):
    pkg, po = graft.load_package(), graft.load_oracle()
    if po.Ref.available():
        ref, kind = po.Ref(), "reference"
        cores = ref.threads()
    else:  # the C restatement stands in where the reference's sources were never compiled
        orc = po.Oracle()
        kind, cores = "port", 1

        class _R:
            xq = staticmethod(lambda x, up=None: orc.xq(x, up))

            @staticmethod
            def gemv(t, w, K, n, a, residual=None):
                return orc.gemm(t, w, K, n, a, residual=None if residual is None else residual[None, :])[0]
        ref = _R()
    weights = {n: pkg.synth.make_weight(t, r, k, i) for i, (n, t, r, k) in
               enumerate(pkg.synth.dense_layer_shapes("Q4_K_M"))}
    nbytes = sum(w.size for w in weights.values())
    x, attn = pkg.synth.make_activation(1, 5120, 1), pkg.synth.make_activation(1, 5120, 2)
    t_begin = time.perf_counter()
    for _ in range(warmup):
        cpu_layer_pass(ref, pkg, weights, x, attn)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_layer_pass(ref, pkg, weights, x, attn)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    ms = 1e3 * float(np.mean(times))
    return {"value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"{len(times)} full layer passes (210 MB of weights each, one weight set, host-resident)",
            "ms_per_step": ms, "steps": len(times)}


# ------------------------------------------------------------------------ GPU helpers
class Ctx:
    """What every cell needs: package, backend, ranks, peaks, a side stream for graph capture."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank, self.world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
        self.local = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        self.pkg = graft.load_package()
        self.be = self.pkg.make_cuda_backend(self.local)
        self.side = torch.cuda.Stream()
        self.peaks, self.peak_source = measured_peaks()
        self.args = args
        self.ceilings = {}

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, vals):
        if self.world == 1:
            return [float(v) for v in vals]
        t = self.torch.tensor(list(vals), device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.cpu()]

    def capture(self, fn):
        """Record fn() into a CUDA graph (the backend launches on the side stream meanwhile)."""
        torch = self.torch
        self.be._stream = self.side
        try:
            with torch.cuda.stream(self.side):
                fn()
                self.side.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.side):
                    fn()
        finally:
            self.be._stream = None
        torch.cuda.synchronize()
        return g

    def time_ms(self, run, n, warm=3):
        """Device time of n calls of run(i): warm-up, barrier, CUDA events, barrier; max over ranks."""
        torch = self.torch
        for i in range(warm):
            run(i)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            run(i)
        e1.record()
        self.barrier()
        return self.max_over_ranks([e0.elapsed_time(e1)])[0]

    def frac(self, gbs):
        return gbs / self.peaks["hbm_gbs"]


def clocked(ctx, fn):
    """Run fn() with a clock sampler around it; returns (result, clocks summary)."""
    s = ClockSampler(ctx.local)
    s.start()
    r = fn()
    return r, s.summary()


def make_layers(ctx, mix, TB, L, rank, world, arena=None, seed0=100):
    from sycl_infer_b200.layer import DenseLayer
    torch, pkg = ctx.torch, ctx.pkg
    layers = [DenseLayer(ctx.be, mix, seed=seed0 + i, TB=TB, rank=rank, world=world, arena=arena,
                         group=None) for i in range(L)]
    hidden, q_dim = layers[0].hidden, layers[0].q_dim
    # a step's two inputs (hidden state and attention output) share one device buffer per weight
    # set, so the end-to-end loop moves them with ONE host-to-device copy
    xin = [torch.zeros(TB * (hidden + q_dim), dtype=torch.float32, device="cuda") for _ in range(L)]
    xs = [b[:TB * hidden].view(TB, hidden) for b in xin]
    for i, ly in enumerate(layers):
        xs[i].copy_(torch.from_numpy(pkg.synth.make_activation(TB, hidden, 10 + i)))
        ly.attn = xin[i][TB * hidden:].view(TB, q_dim)
        ly.attn.copy_(torch.from_numpy(pkg.synth.make_activation(TB, q_dim, 3)))
    return layers, xin, xs


def layer_bytes(pkg, mix, TB, ly):
    """Algorithmic bytes of one layer pass: raw weight blocks once + fp32 activations in and out."""
    vec = 2 * ly.hidden + ly.q_dim + 2 * ly.n_ff + (ly.q_dim + 2 * ly.kv_dim) + 2 * ly.hidden + 2 * ly.n_ff
    return pkg.synth.layer_weight_bytes(mix) + 4 * TB * vec


# ------------------------------------------------------------------------ cells, one GPU
def cell_single_matrix(ctx, name, qtype, rows, K, copies=16, iters=64):
    """One quantize + GEMV call per iteration over rotating copies of one matrix (config 0)."""
    torch, pkg, be = ctx.torch, ctx.pkg, ctx.be
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    w0 = pkg.synth.make_weight(qtype, rows, K, 0xB200)
    ws = [torch.from_numpy(w0).cuda() for _ in range(copies)]
    x = torch.from_numpy(pkg.synth.make_activation(1, K, 0xB201)).cuda()
    x8, xm, xs = alloc_act(1, K)
    out = torch.zeros(rows, dtype=torch.float32, device="cuda")
    segs = [gemv_seg(w=w, type=qtype, K=K, n_rows=rows, x=x, x_stride=K, out=out, out_stride=rows, x8=x8, xmeta=xm,
                     xsumq=xs) for w in ws]
    g = ctx.capture(lambda: [be.quant_gemv([segs[i % copies]], 1) for i in range(iters)])
    (ms, clocks) = clocked(ctx, lambda: ctx.time_ms(lambda i: g.replay(), 20))
    us = 1e3 * ms / (20 * iters)
    nbytes = w0.size + 8 * K
    gbs = nbytes / us / 1e3
    return {"cell": name, "us": us, "bytes": nbytes, "GB/s": gbs, "frac_of_measured_hbm": ctx.frac(gbs),
            "l2": f"{copies} rotating copies ({copies * w0.size / 1e6:.0f} MB)", "launches_per_iter": 1, "clocks": clocks}


def cell_layer(ctx, name, mix, TB, L=4, steps=40):
    """One dense layer per step on ONE GPU (config 1 at another batch or mix)."""
    layers, xin, xs = make_layers(ctx, mix, TB, L, 0, 1)
    torch, be = ctx.torch, ctx.be
    out = torch.zeros(TB, layers[0].hidden, dtype=torch.float32, device="cuda")
    graphs = [ctx.capture(lambda i=i: layers[i].forward(xs[i], out)) for i in range(L)]
    (ms, clocks) = clocked(ctx, lambda: ctx.time_ms(lambda i: graphs[i % L].replay(), steps))
    us = 1e3 * ms / steps
    nbytes = layer_bytes(ctx.pkg, mix, TB, layers[0])
    gbs = nbytes / us / 1e3
    return {"cell": name, "us": us, "bytes": nbytes, "GB/s": gbs, "frac_of_measured_hbm": ctx.frac(gbs),
            "tok_s_64_layers": TB * 1e6 / (us * LAYERS_PER_TOKEN), "launches_per_iter": layers[0].launches_per_step(),
            "l2": f"{L} rotating weight sets", "clocks": clocks}


def measure_ceilings(ctx):
    """The two ceilings a copy benchmark and a bf16 GEMM do not give (library instruments): one pass of
    16-byte loads over 2 GiB, and tcgen05 kind::i8 products with shared-memory-resident operands."""
    import ctypes as C
    torch, be = ctx.torch, ctx.be
    nbytes = 2 << 30
    buf = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    buf.fill_(7)
    sink = torch.zeros(1, dtype=torch.int32, device="cuda")
    bp, sp = C.c_void_p(buf.data_ptr()), C.c_void_p(sink.data_ptr())
    ms = ctx.time_ms(lambda i: be.lib.check(be.lib.probe_hbm_read(be._s(), bp, C.c_size_t(nbytes), sp)), 5, warm=2)
    read_gbs = 5 * nbytes / (ms * 1e-3) / 1e9
    iters = 20000
    ms2 = ctx.time_ms(lambda i: be.lib.check(be.lib.probe_i8_mma(be._s(), iters, sp)), 3, warm=1)
    sms = torch.cuda.get_device_properties(ctx.local).multi_processor_count
    tops = 3.0 * sms * iters * 2 * 128 * 256 * 32 / (ms2 * 1e-3) / 1e12
    ok = int(sink.cpu()[0]) == 0 and be.device_status() == 0
    del buf
    return {"hbm_read_gbs": read_gbs if ok else None, "i8_mma_tops": tops if ok else None,
            "how": "b200q_probe_hbm_read over 2 GiB; b200q_probe_i8_mma, 128x256x32 kind::i8, 20000 per SM; CUDA events"}


def cell_token(ctx, layers, n_layers=LAYERS_PER_TOKEN, iters=10):
    """A whole decode token as one replayed graph: n_layers layer steps, each layer's input the
    previous layer's output, the weight sets of `layers` cycled (1.7 GB in total: a set is evicted
    from L2 long before its next use)."""
    torch = ctx.torch
    L, hidden = len(layers), layers[0].hidden
    a = torch.from_numpy(ctx.pkg.synth.make_activation(1, hidden, 77)).cuda()
    bufs = [a.clone(), torch.zeros(1, hidden, device="cuda")]

    def token():
        bufs[0].copy_(a)
        for i in range(n_layers):
            layers[i % L].forward(bufs[i & 1], bufs[(i + 1) & 1])
    g = ctx.capture(token)
    (ms, clocks) = clocked(ctx, lambda: ctx.time_ms(lambda i: g.replay(), iters))
    us = 1e3 * ms / iters
    ok = bool(torch.isfinite(bufs[n_layers & 1]).all()) and ctx.be.device_status() == 0
    nbytes = n_layers * layer_bytes(ctx.pkg, "Q4_K_M", 1, layers[0])
    gbs = nbytes / us / 1e3
    return {"cell": f"config 1: one decode token = {n_layers} chained layer steps in one graph, Q4_K_M, batch 1",
            "us": us, "us_per_layer": us / n_layers, "bytes": nbytes, "GB/s": gbs, "frac_of_measured_hbm": ctx.frac(gbs),
            "tok_s": 1e6 / us, "finite_and_status_clean": ok, "launches_per_iter": n_layers * layers[0].launches_per_step(),
            "l2": f"{L} weight sets of 210 MB cycled", "clocks": clocks}


def cell_layer_norm(ctx, L=4, steps=96):
    """The layer step with the two RMSNorms a decoder layer has (ahead of q|k|v and of gate|up) folded
    into those calls' quantizers: still four launches."""
    from sycl_infer_b200.layer import DenseLayer
    torch, pkg = ctx.torch, ctx.pkg
    layers = [DenseLayer(ctx.be, "Q4_K_M", seed=500 + i, TB=1, norm=True) for i in range(L)]
    xs = [torch.from_numpy(pkg.synth.make_activation(1, layers[0].hidden, 20 + i)).cuda() for i in range(L)]
    for ly in layers:
        ly.attn.copy_(torch.from_numpy(pkg.synth.make_activation(1, ly.q_dim, 3)))
    out = torch.zeros(1, layers[0].hidden, device="cuda")
    g = ctx.capture(lambda: [layers[i].forward(xs[i], out) for i in range(L)])
    (ms, clocks) = clocked(ctx, lambda: ctx.time_ms(lambda i: g.replay(), steps // L))
    us = 1e3 * ms / (steps // L * L)
    nbytes = layer_bytes(pkg, "Q4_K_M", 1, layers[0]) + 2 * 4 * layers[0].hidden
    gbs = nbytes / us / 1e3
    return {"cell": "config 1 + RMSNorm ahead of q|k|v and gate|up folded into their quantizers, batch 1", "us": us,
            "bytes": nbytes, "GB/s": gbs, "frac_of_measured_hbm": ctx.frac(gbs), "launches_per_iter": 4,
            "status_clean": ctx.be.device_status() == 0, "l2": f"{L} rotating weight sets", "clocks": clocks}


def cell_lm_head(ctx, rows=152064, K=5120, iters=20):
    """The LM head of a greedy decode step: Q6_K rows x K GEMV whose launch also leaves the argmax of
    the logits, against the same GEMV followed by the argmax launch.  One weight copy: 639 MB, five
    times the L2."""
    torch, pkg, be = ctx.torch, ctx.pkg, ctx.be
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    w = torch.from_numpy(pkg.synth.make_weight(14, rows, K, 0xB209)).cuda()
    x = torch.from_numpy(pkg.synth.make_activation(1, K, 0xB20A)).cuda()
    x8, xm, xs = alloc_act(1, K)
    out = torch.zeros(rows, dtype=torch.float32, device="cuda")
    idx, val = torch.zeros(1, dtype=torch.int32, device="cuda"), torch.zeros(1, device="cuda")
    seg = gemv_seg(w=w, type=14, K=K, n_rows=rows, x=x, x_stride=K, out=out, out_stride=rows, x8=x8, xmeta=xm, xsumq=xs)
    g1 = ctx.capture(lambda: [be.quant_gemv_ex([seg], 1, argmax=(idx, val)) for _ in range(iters)])
    (ms1, clocks) = clocked(ctx, lambda: ctx.time_ms(lambda i: g1.replay(), 5))
    fused_idx = int(idx.cpu()[0])
    g2 = ctx.capture(lambda: [(be.quant_gemv_ex([seg], 1), be.mtp_argmax(out, rows, idx, val, 1)) for _ in range(iters)])
    ms2 = ctx.time_ms(lambda i: g2.replay(), 5)
    us1, us2 = 1e3 * ms1 / (5 * iters), 1e3 * ms2 / (5 * iters)
    nbytes = w.numel() + 4 * K + 4 * rows
    return {"cell": f"LM head: Q6_K {rows}x{K} GEMV + argmax in one launch, batch 1", "us": us1, "us_two_launches": us2,
            "bytes": nbytes, "GB/s": nbytes / us1 / 1e3, "frac_of_measured_hbm": ctx.frac(nbytes / us1 / 1e3),
            "same_token": fused_idx == int(idx.cpu()[0]) == int(out.argmax().cpu()), "launches_per_iter": 1,
            "l2": "one 639 MB weight", "clocks": clocks}


def cell_prefill(ctx, name, M, rows=17408, K=5120, iters=3):
    """Config 2: M tokens x (Q4_K weight of `rows` x K); quantizer + tensor-core GEMM per iteration."""
    torch, pkg, be = ctx.torch, ctx.pkg, ctx.be
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    w = torch.from_numpy(pkg.synth.make_weight(12, rows, K, 0xB202)).cuda()
    x = torch.from_numpy(pkg.synth.make_activation(M, K, 0xB203)).cuda()
    x8, xm, xs = alloc_act(M, K)
    out = torch.zeros(M * rows, dtype=torch.float32, device="cuda")
    seg = gemv_seg(w=w, type=12, K=K, n_rows=rows, x=x, x_stride=K, out=out, out_stride=rows, x8=x8, xmeta=xm, xsumq=xs)
    (ms, clocks) = clocked(ctx, lambda: ctx.time_ms(lambda i: be.quant_gemv([seg], M), iters, warm=1))
    us = 1e3 * ms / iters
    ops = 2.0 * M * K * rows
    nbytes = w.numel() + 4 * M * K + 4 * M * rows
    return {"cell": name, "us": us, "int8_ops": ops, "Tops": ops / us / 1e6, "bytes": nbytes, "GB/s": nbytes / us / 1e3,
            "frac_of_measured_hbm": ctx.frac(nbytes / us / 1e3),
            "frac_of_i8_mma_peak": (ops / us / 1e6) / ctx.ceilings["i8_mma_tops"] if ctx.ceilings.get("i8_mma_tops") else None,
            "clocks": clocks}


def cell_moe(ctx, name, tokens=16, experts=256, topk=8, embd=2048, ff=512, copies=2, iters=20):
    """Config 3: router -> CSR -> quantize -> grouped gate|up -> quantize -> grouped down -> reduce."""
    torch, pkg, be = ctx.torch, ctx.pkg, ctx.be
    from sycl_infer_b200.moe import MoeScratch, make_synthetic_moe, moe_call
    banks = [make_synthetic_moe(experts, topk, embd, ff, (12, 12, 12), seed=i, with_router=True)[1]
             for i in range(copies)]
    S = MoeScratch(banks[0], tokens)
    x = torch.from_numpy(pkg.synth.make_activation(tokens, embd, 5)).cuda()
    out = torch.zeros(tokens, embd, device="cuda")
    g = ctx.capture(lambda: [moe_call(be, banks[i % copies], S, x, tokens, out) for i in range(iters)])
    (ms, clocks) = clocked(ctx, lambda: ctx.time_ms(lambda i: g.replay(), 10))
    us = 1e3 * ms / (10 * iters)
    n_active = int(S.n_active.cpu()[0])
    per_expert = sum(int(pkg.synth.row_bytes(12, K)) * r for r, K in ((ff, embd), (ff, embd), (embd, ff)))
    nbytes = n_active * per_expert
    gbs = nbytes / us / 1e3
    cell = {"cell": name, "us": us, "bytes": nbytes, "active_experts": n_active, "GB/s": gbs,
            "frac_of_measured_hbm": ctx.frac(gbs), "l2": f"{copies} rotating expert banks", "clocks": clocks}
    if tokens * topk > 4 * min(experts, tokens * topk):  # the grouped tensor-core form: arithmetic, not the weight stream
        tops = 2.0 * tokens * topk * 3 * embd * ff / us / 1e6
        cell["T_int8_op/s"] = tops
        if ctx.ceilings.get("i8_mma_tops"):
            cell["frac_of_i8_mma_peak"] = tops / ctx.ceilings["i8_mma_tops"]
    return cell


# ------------------------------------------------------------------------ cells, several GPUs
def cell_sharded(ctx, mix, TB, arm, L=2, steps=30):
    """Row-sharded layer: `peer` = GEMV epilogue stores rows on every GPU (flag barrier folded into
    the kernels), `nccl` = NCCL all-gather after each call (host launches)."""
    torch, be, rank, world = ctx.torch, ctx.be, ctx.rank, ctx.world
    arena = None
    if arm == "peer":
        from sycl_infer_b200.sharding import PeerArena
        arena = PeerArena(L * TB * 65536 + 8192, rank, world)
    layers, xin, xs = make_layers(ctx, mix, TB, L, rank, world, arena=arena, seed0=300)
    out = arena.alloc(TB, layers[0].hidden) if arena is not None else torch.zeros(TB, layers[0].hidden, device="cuda")
    graphs = None
    if arm == "peer":
        graphs = [ctx.capture(lambda i=i: layers[i].forward(xs[i], out)) for i in range(L)]
    run = (lambda i: graphs[i % L].replay()) if graphs else (lambda i: layers[i % L].forward(xs[i % L], out))
    ms = ctx.time_ms(run, steps)
    # the same step with the exchange left out (wrong results, timing only): its share is the difference
    for ly in layers:
        ly.exchange = False
    if arm == "peer":
        graphs = [ctx.capture(lambda i=i: layers[i].forward(xs[i], out)) for i in range(L)]
        run = lambda i: graphs[i % L].replay()  # noqa: E731
    ms_noex = ctx.time_ms(run, steps)
    us, us_noex = 1e3 * ms / steps, 1e3 * ms_noex / steps
    nbytes = layer_bytes(ctx.pkg, mix, TB, layers[0])
    gbs = nbytes / us / 1e3
    return {"cell": f"{mix} batch {TB} row-sharded x{world} ({arm})", "us": us, "bytes": nbytes, "GB/s": gbs,
            "frac_of_P_x_measured_hbm": gbs / (world * ctx.peaks["hbm_gbs"]),
            "tok_s_64_layers": TB * 1e6 / (us * LAYERS_PER_TOKEN),
            "exchange_share": max(0.0, 1.0 - us_noex / us), "launch": "cuda graph" if arm == "peer" else "host launches"}


def cell_layer_split(ctx, mix, TB, n_layers=8, steps=10):
    """The reference's contiguous layer split (--layer-map): n_layers layers over the ranks, the
    hidden state handed on at each boundary (NCCL send/recv).  One step = one token batch through
    all n_layers; a rank idles while the others compute (no pipelining across steps here)."""
    from sycl_infer_b200.layer import DenseLayer
    from sycl_infer_b200.sharding import even_layer_map, parse_layer_map, run_layer_split
    torch, be, rank, world = ctx.torch, ctx.be, ctx.rank, ctx.world
    ranges = parse_layer_map(even_layer_map(n_layers, world), n_layers)
    mine = ranges[rank] if rank < len(ranges) else None
    layers = {}
    if mine is not None:
        for l in range(mine.l0, mine.l1):
            layers[l] = DenseLayer(be, mix, seed=500 + l, TB=TB)
            layers[l].attn.copy_(torch.from_numpy(ctx.pkg.synth.make_activation(TB, layers[l].q_dim, 3)))
    hidden = 5120
    x = torch.from_numpy(ctx.pkg.synth.make_activation(TB, hidden, 11)).cuda()

    def run_layer(l, xx):
        layers[l].forward(xx, xx)  # residual add in place: the layer's output is the next layer's input

    ms = ctx.time_ms(lambda i: run_layer_split(ranges, rank, x, run_layer), steps)
    us = 1e3 * ms / steps
    proto = next(iter(layers.values())) if layers else DenseLayer(be, mix, seed=1, TB=TB, hidden=256, n_head=2,
                                                                  n_kv=2, head_dim=128, n_ff=256)
    nbytes = n_layers * (ctx.pkg.synth.layer_weight_bytes(mix) + 4 * TB * 4 * hidden)
    del proto
    gbs = nbytes / us / 1e3
    return {"cell": f"{mix} batch {TB} layer split x{world} ({n_layers} layers, {even_layer_map(n_layers, world)})",
            "us": us, "us_per_layer": us / n_layers, "bytes": nbytes, "GB/s": gbs,
            "frac_of_P_x_measured_hbm": gbs / (world * ctx.peaks["hbm_gbs"]),
            "tok_s_64_layers": TB * 1e6 / (us / n_layers * LAYERS_PER_TOKEN), "launch": "host launches",
            "note": "consecutive steps overlap across ranks (rank 0 starts step s+1 while rank 1 runs step s): a pipelined figure, not a per-token latency"}


def safe(cells, fn, *a, **kw):
    try:
        cells.append(fn(*a, **kw))
    except Exception as e:  # a cell that cannot run is reported, not hidden
        cells.append({"cell": getattr(fn, "__name__", "cell") + str(a[1:]), "error": f"{type(e).__name__}: {e}"[:300]})


# ------------------------------------------------------------------------ GPU arm
def gpu_arm(args):
    ctx = Ctx(args)
    torch, pkg, be, rank, world = ctx.torch, ctx.pkg, ctx.be, ctx.rank, ctx.world
    L = args.layers
    arena = None
    if world > 1 and args.gather == "peer":
        from sycl_infer_b200.sharding import PeerArena
        arena = PeerArena(L * 65536 + 8192, rank, world)
    layers, xin, xs = make_layers(ctx, "Q4_K_M", 1, L, rank, world, arena=arena)
    hidden, q_dim = layers[0].hidden, layers[0].q_dim
    out = arena.alloc(1, hidden) if arena is not None else torch.zeros(1, hidden, dtype=torch.float32, device="cuda")
    step_bytes = layer_bytes(pkg, "Q4_K_M", 1, layers[0])  # whole-job bytes per step however rows are sharded

    # One CUDA graph per weight set: the engine this path plugs into replays a recorded graph
    # per decode step too, so a step is one graph launch, not four host launches.
    graphs = []
    if (world == 1 or arena is not None) and not args.no_graph:
        graphs = [ctx.capture(lambda i=i: layers[i].forward(xs[i], out)) for i in range(L)]

    def step(i):
        if graphs:
            graphs[i % L].replay()
        else:
            layers[i % L].forward(xs[i % L], out)

    # The engine this path plugs into replays one recorded graph per decode TOKEN (all its layers),
    # not one per layer: the timed K steps therefore run as graphs of L consecutive layer steps
    # (K // L replays) plus K % L single-step graphs - the same K steps, the same launches, without a
    # graph-launch gap after every layer.
    span = None
    if graphs and not args.step_graphs:
        span = ctx.capture(lambda: [layers[i].forward(xs[i], out) for i in range(L)])

    def run_steps(n):
        """Device time (ms) of exactly n layer steps."""
        if span is None:
            return ctx.time_ms(step, n, warm=max(args.warmup, 3))
        q, r = divmod(n, L)
        for i in range(max(args.warmup, 3)):
            step(i)
        return ctx.time_ms(lambda j: span.replay() if j < q else graphs[j - q].replay(), q + r, warm=1)

    sampler = ClockSampler(ctx.local)
    sampler.start()
    ms = run_steps(args.steps)

    # ---- e2e: host buffers, pinned H2D of the step's activations, D2H of its output, every step
    hx = [xin[i].cpu().pin_memory() for i in range(L)]
    hout = torch.zeros(1, hidden, dtype=torch.float32).pin_memory()

    # A decode step as an engine would replay it: ONE graph holding the pinned-host -> device copy of
    # the step's inputs, the layer's launches and the device -> pinned-host copy of its output; the
    # host waits for the result every step (the next token depends on it).
    e2e_graphs = []
    if graphs and world == 1:
        def whole(i):
            xin[i].copy_(hx[i], non_blocking=True)
            layers[i].forward(xs[i], out)
            hout.copy_(out, non_blocking=True)
        e2e_graphs = [ctx.capture(lambda i=i: whole(i)) for i in range(L)]

    def e2e_step(i):
        if e2e_graphs:
            e2e_graphs[i % L].replay()
        else:
            xin[i % L].copy_(hx[i % L], non_blocking=True)
            step(i)
            hout.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    ms_e2e = ctx.time_ms(e2e_step, args.steps)

    # ---- roofline of the dominant kernel: the four GEMV launches of a layer alone, activations
    # pre-quantized, in one CUDA graph over all weight sets
    calls = [ly.calls(xs[i], out) for i, ly in enumerate(layers)]
    for i, ly in enumerate(layers):  # make sure the quantized views are valid
        ly.forward(xs[i], out)
    torch.cuda.synchronize()
    reps = max(1, args.steps // L)
    n_launch = 4 * L * reps
    gemv_only = lambda: [be.i8_gemv(segs) for i in range(L) for segs, _ in calls[i]]  # noqa: E731
    if world == 1 or arena is not None:
        gg = ctx.capture(gemv_only)
        ms_gemv = ctx.time_ms(lambda i: gg.replay(), reps)
    else:
        ms_gemv = ctx.time_ms(lambda i: gemv_only(), reps)
    clocks = sampler.summary()

    ctx.ceilings = measure_ceilings(ctx) if world == 1 and not args.no_ceilings else {}
    cells = []
    if not args.no_cells:
        if world == 1:
            safe(cells, cell_token, ctx, layers)
            safe(cells, cell_lm_head, ctx)
            safe(cells, cell_single_matrix, ctx, "config 0: Q4_K 4096x4096 GEMV, batch 1", 12, 4096, 4096)
            safe(cells, cell_layer, ctx, "config 1: dense layer Q4_K_M, batch 16", "Q4_K_M", 16)
            safe(cells, cell_prefill, ctx, "config 2: prefill GEMM M=512 x 5120 x 17408 Q4_K", 512)
            safe(cells, cell_prefill, ctx, "config 2: prefill GEMM M=2048 x 5120 x 17408 Q4_K", 2048)
            safe(cells, cell_prefill, ctx, "config 2: prefill GEMM M=8192 x 5120 x 17408 Q4_K", 8192, iters=2)
            safe(cells, cell_moe, ctx, "config 3: routed MoE, 256 experts top-8, 16 tokens, Q4_K")
            safe(cells, cell_moe, ctx, "config 3 (prefill): routed MoE, 256 experts top-8, 512 tokens, Q4_K", tokens=512, iters=4)
            safe(cells, cell_layer, ctx, "config 4 (1 GPU): dense layer IQ4_XS, batch 1", "IQ4_XS", 1)
            safe(cells, cell_layer, ctx, "config 4 (1 GPU): dense layer Q5_K, batch 1", "Q5_K", 1)
            safe(cells, cell_layer, ctx, "config 4 (1 GPU): dense layer Q4_K_M, batch 32", "Q4_K_M", 32)
            # last: from the first call with a norm on, the library launches its norm-capable kernel image
            safe(cells, cell_layer_norm, ctx)
        else:
            for mix in ("Q4_K_M", "IQ4_XS", "Q5_K"):
                for TB in (1, 32):
                    for arm in ("peer", "nccl"):
                        safe(cells, cell_sharded, ctx, mix, TB, arm)
                    safe(cells, cell_layer_split, ctx, mix, TB)

    if rank == 0:
        per_step = ms / args.steps
        gbs = step_bytes * args.steps / (ms * 1e-3) / 1e9
        alg_launch = step_bytes / 4.0 / world
        achieved = alg_launch * n_launch / (ms_gemv * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": per_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": WORKLOAD, "launch": (f"cuda graph of {L} consecutive layer steps" if span is not None else "cuda graph per step") if graphs else "host launches",
                       "l2": f"inputs larger than L2: {L} rotating weight sets of 210 MB", "bytes_per_step": step_bytes,
                       "parallelism": (f"row-sharded x{world}, " + ("peer-store epilogue, flag exchange inside the GEMV kernels"
                                                                   if arena is not None else "NCCL all-gather"))
                       if world > 1 else "1 GPU",
                       "decode_tok_s_64_layers": 1e3 / (per_step * LAYERS_PER_TOKEN),
                       "pct_of_measured_hbm": 100.0 * gbs / ctx.peaks["hbm_gbs"], "pct_of_8TBs": 100.0 * gbs / 8000.0},
            "e2e": {"value": step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": 4 * (hidden + q_dim), "d2h_bytes_per_step": 4 * hidden,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": args.steps * layers[0].launches_per_step(),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": ctx.peaks["hbm_gbs"] , "unit": "GB/s",
                         "frac": achieved / ctx.peaks["hbm_gbs"],
                         "frac_of_read_ceiling": achieved / ctx.ceilings["hbm_read_gbs"] if ctx.ceilings.get("hbm_read_gbs") else None,
                         "traffic": ncu_traffic_per_launch() if world == 1 else None, "traffic_source": TRAFFIC_NOTE,
                         "peak_source": ctx.peak_source,
                         "kernel": "gemv_pinned_kernel (one launch per call, 4 per layer), CUDA graph, pre-quantized activations",
                         "bytes_per_launch": alg_launch,
                         "weight_bytes_per_launch": pkg.synth.layer_weight_bytes("Q4_K_M") / 4.0 / world,
                         "us_per_launch": 1e3 * ms_gemv / n_launch},
            "ceilings": ctx.ceilings,
            "cells": cells,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = {k: v for k, v in cpu_arm(6, 1, budget_s=20.0).items()
                                    if k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        ctx.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--layers", type=int, default=8, help="distinct weight sets rotated through (L2 defeat)")
    ap.add_argument("--impl", default="b200q", choices=["b200q", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-cells", action="store_true", help="headline only: skip the other configurations")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="N > 1: GEMV epilogue stores rows on every GPU (peer), or NCCL all-gather")
    ap.add_argument("--no-graph", action="store_true", help="launch kernels from the host instead of CUDA graphs")
    ap.add_argument("--no-ceilings", action="store_true", help="skip the read-only HBM and int8 tensor-core probes")
    ap.add_argument("--step-graphs", action="store_true", help="one CUDA graph per layer step instead of one per L steps")
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", 0)) != 0:
            return
        r = cpu_arm(args.steps, max(args.warmup, 1), budget_s=150.0)
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "GB/s", "n_gpus": args.gpus,
            "steps": r["steps"], "warmup": max(args.warmup, 1), "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": DTYPE,
            "data": "synthetic", "config": {"workload": WORKLOAD, "device": "host CPU"},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    gpu_arm(args)


if __name__ == "__main__":
    main()
