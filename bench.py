"""Benchmark of the quantized-GEMV hot path: one dense layer's GEMV calls, batch 1.

Workload = benchmark configuration 1: hidden 5120, 40 query / 8 KV heads of dim 128, FFN
17408, Q/K/O/gate/up in Q4_K, V/down in Q6_K (the "Q4_K_M" mix), seeded synthetic blocks.
One step = one layer pass = four calls (q|k|v, o, gate|up, down), each an activation
quantize + one GEMV launch.  Steps rotate over `--layers` distinct weight sets of 210 MB
each, so every step streams weights that are not in the 126 MB L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line (rank 0).  `value` is weight-stream GB/s with all inputs resident in
HBM; `e2e` is the same through the host-buffer call sequence (pinned H2D of the step's
activations, D2H of its output, every step); `roofline` is the GEMV kernel alone against
the measured HBM copy bandwidth; `cpu_baseline` is the reference's own CPU path on this
machine's cores.  `--impl reference` times that CPU path as the headline instead.
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

# dram__bytes_read.sum + dram__bytes_write.sum of the four GEMV launches of one layer step, from an
# ncu capture of this workload on one B200 (215.6 MB per layer against 210.1 MB of weights): per launch
NCU_DRAM_BYTES_PER_LAUNCH = 53.9e6
METRIC = "quant_gemv_effective_hbm_gbs"
WORKLOAD = "dense layer GEMV set, Q4_K_M mix (hidden 5120, 40q/8kv x128, ffn 17408), batch 1"
LAYERS_PER_TOKEN = 64


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


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
            self.stop_flag.wait(0.1)

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
def cpu_layer_pass(ref, po, pkg, weights, x, attn):
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
        kind, cores = "port", os.cpu_count() or 1

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
        cpu_layer_pass(ref, po, pkg, weights, x, attn)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_layer_pass(ref, po, pkg, weights, x, attn)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    ms = 1e3 * float(np.mean(times))
    return {"value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"{len(times)} full layer passes (210 MB of weights each, one weight set, host-resident)",
            "ms_per_step": ms, "steps": len(times)}


# ------------------------------------------------------------------------ GPU arm
def gpu_arm(args):
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = graft.load_package()
    from sycl_infer_b200.layer import DenseLayer
    be = pkg.make_cuda_backend(local)
    L = args.layers
    arena = None
    if world > 1 and args.gather == "peer":
        from sycl_infer_b200.sharding import PeerArena
        arena = PeerArena(L * 65536 + 8192, rank, world)
    layers = [DenseLayer(be, "Q4_K_M", seed=100 + i, TB=1, rank=rank, world=world, arena=arena) for i in range(L)]
    hidden = layers[0].hidden
    # a step's two inputs (hidden state and attention output) share one device buffer per weight
    # set, so the end-to-end loop moves them with ONE host-to-device copy
    q_dim = layers[0].q_dim
    xin = [torch.zeros(hidden + q_dim, dtype=torch.float32, device="cuda") for _ in range(L)]
    xs = [b[:hidden].view(1, hidden) for b in xin]
    attn = torch.from_numpy(pkg.synth.make_activation(1, q_dim, 3)).cuda()
    for i, ly in enumerate(layers):
        xs[i].copy_(torch.from_numpy(pkg.synth.make_activation(1, hidden, 10 + i)))
        ly.attn = xin[i][hidden:].view(1, q_dim)
        ly.attn.copy_(attn)
    out = arena.alloc(1, hidden) if arena is not None else torch.zeros(1, hidden, dtype=torch.float32, device="cuda")
    full_bytes = pkg.synth.layer_weight_bytes("Q4_K_M") + 4 * (
        2 * hidden + layers[0].q_dim + 2 * layers[0].n_ff + (layers[0].q_dim + 2 * layers[0].kv_dim)
        + 2 * hidden + 2 * layers[0].n_ff)
    step_bytes = full_bytes  # whole-job bytes per step regardless of how rows are sharded

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # One CUDA graph per weight set: the engine this path plugs into replays a recorded graph
    # per decode step too, so a step is one graph launch (8 kernels), not 8 host launches.
    graphs = []
    if (world == 1 or arena is not None) and not args.no_graph:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for i in range(L):
                layers[i].forward(xs[i], out)
            side.synchronize()
            for i in range(L):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    layers[i].forward(xs[i], out)
                graphs.append(g)
        torch.cuda.synchronize()

    def run_steps(n, first=0):
        for i in range(n):
            if graphs:
                graphs[(first + i) % L].replay()
            else:
                j = (first + i) % L
                layers[j].forward(xs[j], out, cached[j])

    cached = [ly.calls(xs[i], out) for i, ly in enumerate(layers)]
    run_steps(max(args.warmup, 3))
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_steps(args.steps)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # the device-resident loop is short; keep sampling clocks through the e2e loop as well
    # ---- e2e: host buffers, pinned H2D of the step's activations, D2H of its output
    hx = [torch.cat([torch.from_numpy(pkg.synth.make_activation(1, hidden, 10 + i)).view(-1), attn.cpu().view(-1)]).pin_memory()
          for i in range(L)]
    hout = torch.zeros(1, hidden, dtype=torch.float32).pin_memory()
    dx = torch.zeros(1, hidden, dtype=torch.float32, device="cuda")

    def e2e_step(i):
        ly = layers[i % L]
        xin[i % L].copy_(hx[i % L], non_blocking=True)
        if graphs:
            graphs[i % L].replay()
        else:
            ly.forward(xs[i % L], out)
        hout.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    barrier()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for i in range(args.steps):
        e2e_step(i)
    g1.record()
    barrier()
    ms_e2e = g0.elapsed_time(g1)
    # ---- roofline of the dominant kernel: GEMV launches alone (activations pre-quantized)
    from sycl_infer_b200.backend import gemv_seg  # noqa: F401
    calls = [ly.calls(xs[i], out) for i, ly in enumerate(layers)]
    for i, ly in enumerate(layers):  # make sure the quantized views are valid
        ly.forward(xs[i], out)
    torch.cuda.synchronize()
    n_launch = 4 * args.steps
    if world == 1 and not args.no_graph:
        side = torch.cuda.Stream()
        gg = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(gg, stream=side):
                for i in range(L):
                    for segs, _ in calls[i]:
                        be.i8_gemv(segs)
        torch.cuda.synchronize()
        reps = max(1, args.steps // L)
        n_launch = 4 * L * reps
        gg.replay()
        torch.cuda.synchronize()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(reps):
            gg.replay()
        r1.record()
    else:
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for i in range(args.steps):
            for segs, _ in calls[i % L]:
                be.i8_gemv(segs)
        r1.record()
    barrier()
    ms_gemv = r0.elapsed_time(r1)
    clocks = sampler.summary()
    if world > 1:
        t = torch.tensor([ms, ms_e2e, ms_gemv], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e, ms_gemv = (float(v) for v in t.cpu())
    peaks, how = measured_peaks()
    if rank == 0:
        per_step = ms / args.steps
        gbs = step_bytes * args.steps / (ms * 1e-3) / 1e9
        wbytes_launch = pkg.synth.layer_weight_bytes("Q4_K_M") / 4.0 / world
        alg_launch = step_bytes / 4.0 / world
        achieved = alg_launch * n_launch / (ms_gemv * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": per_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "int8xu4/u6->int32, fp32 scales",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "launch": "cuda graph per step" if graphs else "host launches", "l2": f"inputs larger than L2: {L} rotating weight sets of 210 MB",
                       "bytes_per_step": step_bytes, "parallelism": (f"row-sharded x{world}, " + ("peer-store epilogue + flag barrier" if arena is not None
                                                                 else "NCCL all-gather")) if world > 1 else "1 GPU",
                       "decode_tok_s_64_layers": 1e3 / (per_step * LAYERS_PER_TOKEN),
                       "pct_of_measured_hbm": 100.0 * gbs / peaks["hbm_gbs"], "pct_of_8TBs": 100.0 * gbs / 8000.0},
            "e2e": {"value": step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": 4 * (hidden + layers[0].q_dim), "d2h_bytes_per_step": 4 * hidden,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": args.steps * layers[0].launches_per_step(),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_DRAM_BYTES_PER_LAUNCH if world == 1 else None,
                         "peak_source": how,
                         "kernel": "gemv (one launch per call, 4 per layer)", "bytes_per_launch": alg_launch,
                         "weight_bytes_per_launch": wbytes_launch, "us_per_launch": 1e3 * ms_gemv / n_launch},
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = {k: v for k, v in cpu_arm(6, 1, budget_s=20.0).items()
                                    if k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--layers", type=int, default=8, help="distinct weight sets rotated through (L2 defeat)")
    ap.add_argument("--impl", default="b200q", choices=["b200q", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="N > 1: GEMV epilogue stores rows on every GPU + flag barrier (peer), or NCCL all-gather")
    ap.add_argument("--no-graph", action="store_true", help="launch kernels from the host instead of CUDA graphs")
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", 0)) != 0:
            return
        r = cpu_arm(args.steps, max(args.warmup, 1), budget_s=150.0)
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "GB/s", "n_gpus": args.gpus,
            "steps": r["steps"], "warmup": max(args.warmup, 1), "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xu4/u6->int32, fp32 scales",
            "data": "synthetic", "config": {"workload": WORKLOAD, "device": "host CPU"},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    gpu_arm(args)


if __name__ == "__main__":
    main()
