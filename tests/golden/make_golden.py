"""Generate tests/golden/ref_vectors.npz by RUNNING the reference's own CPU code.

Needs oracle/_ref/libsiref.so and libsiref_nofma.so (built by `make -C oracle ref` where
the reference tree is mounted).  The committed .npz lets the CPU test-suite pin the C
restatement (oracle/oracle.c) against the reference on machines where the reference
cannot be built.  Inputs are seeded synthetic blocks plus the procedural inputs of the
reference's own hermetic test (tests/backend/cpu/kernels/test_cpu_gemv_units.cpp:40-55:
the `rnd` hash and `make_q4k` blocks).

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import __graft_entry__ as graft  # noqa: E402

pkg = graft.load_package()
po = graft.load_oracle()
synth = pkg.synth
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz")


def ref_test_rnd(i, scale=2.0):
    """The reference unit test's input hash (test_cpu_gemv_units.cpp:40-43)."""
    h = (np.uint32(i) * np.uint32(2654435761) + np.uint32(1013904223)).astype(np.uint32)
    return (((h >> 8) & 0xFFFF).astype(np.float32) / np.float32(32768.0) - np.float32(1.0)) * np.float32(scale)


def ref_test_q4k(n_rows, f2h):
    """The reference unit test's one-superblock-per-row Q4_K tensor (test_cpu_gemv_units.cpp:46-55)."""
    b = np.zeros((n_rows, 144), np.uint8)
    for n in range(n_rows):
        d = f2h(np.float32(0.004) * np.float32(n + 1))
        dm = f2h(np.float32(0.001) * np.float32(n + 1))
        b[n, 0], b[n, 1], b[n, 2], b[n, 3] = d & 0xFF, d >> 8, dm & 0xFF, dm >> 8
        b[n, 4:16] = [(0x11 + 7 * i) & 0xFF for i in range(12)]
        b[n, 16:144] = [(n * 37 + i * 11) & 0xFF for i in range(128)]
    return b.reshape(-1)


def main():
    R, RS = po.Ref(), po.Ref(strict=True)
    g = {}
    rng = np.random.default_rng(20240)
    # f16 conversions
    fs = np.concatenate([rng.normal(0, 1, 200), rng.normal(0, 1e-5, 200), rng.normal(0, 1e-7, 60),
                         [0.0, -0.0, 65504.0, 70000.0, 1e-8, 6.1e-5, 5.9e-8, 1e30]]).astype(np.float32)
    g["f16_in"] = fs
    g["f16_bits"] = np.array([R.f2h(f) for f in fs], np.uint16)
    hs = np.concatenate([np.arange(0, 0x0420), rng.integers(0, 65536, 512)]).astype(np.uint16)
    g["h_in"] = hs
    g["h_f32"] = np.array([R.h2f(h) for h in hs], np.float32)
    # activation quantizer, with and without the fused silu(x)*up, plus a zero group
    TB, K = 3, 512
    x = synth.make_activation(TB, K, 101)
    x[1, 64:96] = 0.0
    up = synth.make_activation(TB, K, 102)
    g["xq_x"], g["xq_up"] = x, up
    for tag, u in (("", None), ("_up", up)):
        a = R.xq(x, u, TB)
        g["xq_x8" + tag], g["xq_meta" + tag], g["xq_sum" + tag] = a.x8, a.xmeta, a.xsumq
    # integer GEMV/GEMM per K-quant type
    N = 5
    act1, act3 = R.xq(x[0], None, 1), R.xq(x, None, 3)
    res = synth.make_activation(3, N, 103)
    g["res"] = res
    for t in (po.Q4_K, po.Q5_K, po.Q6_K):
        w = synth.make_weight(t, N, K, 200 + t)
        g[f"w_{t}"] = w
        g[f"gemv_{t}"] = R.gemv(t, w, K, N, act1, residual=res[0], alpha=0.75)
        g[f"gemv_strict_{t}"] = RS.gemv(t, w, K, N, act1, residual=res[0], alpha=0.75)
        g[f"gemm3_{t}"] = R.gemm(t, w, K, N, act3, residual=res, alpha=0.75)
        g[f"gemm3_strict_{t}"] = RS.gemm(t, w, K, N, act3, residual=res, alpha=0.75)
        g[f"deq_{t}"] = RS.dequantize(t, w, N, K)
    # Q8_0: the reference's only integer kernel for it (expert down), and IQ4_XS: dequant only
    w8 = synth.make_weight(po.Q8_0, N, K, 208)
    g["w_8"], g["deq_8"] = w8, RS.dequantize(po.Q8_0, w8, N, K)
    g["q8down_1"] = RS.q8_0_down(w8, K, N, act1)
    g["q8down_3"] = RS.q8_0_down(w8, K, N, act3)
    wi = synth.make_weight(po.IQ4_XS, N, K, 223)
    g["w_23"], g["deq_23"] = wi, RS.dequantize(po.IQ4_XS, wi, N, K)
    g["f32gemv_23"] = R.gemv_f32(po.IQ4_XS, wi, K, N, x[0])
    g["f32gemv_8"] = R.gemv_f32(po.Q8_0, w8, K, N, x[0])
    # the reference unit test's own procedural case
    wq = ref_test_q4k(3, R.f2h)
    xt = ref_test_rnd(np.arange(256) + 100)
    g["ut_w"], g["ut_x"] = wq, xt
    at = R.xq(xt, None, 1)
    g["ut_gemv"] = R.gemv(po.Q4_K, wq, 256, 3, at)
    g["ut_gemv_strict"] = RS.gemv(po.Q4_K, wq, 256, 3, at)
    xm = ref_test_rnd(np.arange(3 * 256) + 700).reshape(3, 256)
    g["ut_xm"] = xm
    g["ut_gemm3_strict"] = RS.gemm(po.Q4_K, wq, 256, 3, R.xq(xm, None, 3))
    # routed MoE: router, experts (Q4_K gate/up, Q8_0 down: the combination the reference's
    # cpu_moe_experts_i8 implements), reduce
    E, top_k, n_embd, n_ff, n_tok = 4, 2, 256, 256, 3
    gate_inp = rng.normal(0, 1, (E, n_embd)).astype(np.float32)
    xt2 = synth.make_activation(n_tok, n_embd, 104)
    logits, ids, wts = R.moe_route(xt2, gate_inp, top_k)
    g["moe_gate_inp"], g["moe_x"], g["moe_logits"], g["moe_ids"], g["moe_wts"] = gate_inp, xt2, logits, ids, wts
    gw = synth.make_weight(po.Q4_K, E * n_ff, n_embd, 301)
    uw = synth.make_weight(po.Q4_K, E * n_ff, n_embd, 302)
    dw = synth.make_weight(po.Q8_0, E * n_embd, n_ff, 303)
    g["moe_gw"], g["moe_uw"], g["moe_dw"] = gw, uw, dw
    acc = np.concatenate([RS.moe_experts_q8down(gw, uw, dw, po.Q4_K, E, n_embd, n_ff, xt2[t], ids[t])
                          for t in range(n_tok)])
    g["moe_acc_strict"] = acc
    base = synth.make_activation(n_tok, n_embd, 105)
    g["moe_base"] = base
    g["moe_out_strict"] = RS.moe_reduce(acc, wts, base)
    # RMSNorm rows.  The reference sums the squares in the order of the host's vector width; the
    # width of the host that wrote these vectors is recorded beside them (16 = AVX-512).
    r2 = np.random.default_rng(777)
    g["rms_lanes"] = np.array([R.isa_lanes()], np.int32)
    for n in (256, 1000, 5120):
        xr, wr = r2.normal(0, 1, n).astype(np.float32), r2.normal(1, 0.2, n).astype(np.float32)
        g[f"rms_x_{n}"], g[f"rms_w_{n}"], g[f"rms_out_{n}"] = xr, wr, R.rmsnorm(xr, wr, 1e-6)
    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
