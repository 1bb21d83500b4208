"""GPU parity: every operator is called through the C ABI and compared with the oracle
on the same seeded inputs.  Integer results are bit-exact; fp32 outputs are within 1e-5
of the row's sum of |terms| (the tolerance the benchmark's north star states; the
yardstick is the one the reference's own tests use for cancelling dot products,
tests/backend/gpu/kernels/test_moe_grp_q6.cpp:184-206 of the reference)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL = 1e-5
TYPES = (12, 13, 14, 8, 23)
G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_vectors.npz"))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def gpu_xq(be, x, up=None, TB=1):
    from sycl_infer_b200.backend import alloc_act
    x = np.ascontiguousarray(x, np.float32).reshape(TB, -1)
    K = x.shape[1]
    x8, xm, xs = alloc_act(TB, K)
    dx = dev(x)
    dup = None if up is None else dev(np.ascontiguousarray(up, np.float32).reshape(TB, -1))
    be.xq(dx, dup, K, K, x8, xm, xs, None, TB, K)
    be.synchronize()
    return x8, xm, xs


def gpu_gemm(be, t, w, K, N, act, TB, residual=None, alpha=1.0, out_stride=None, alias=False):
    from sycl_infer_b200.backend import gemv_seg
    out_stride = out_stride or N
    out = torch.full((TB * out_stride,), 7.0, dtype=torch.float32, device="cuda")
    res = None
    if residual is not None:
        if alias:
            out.view(TB, out_stride)[:, :N] = dev(residual)
            res = out
        else:
            r = np.zeros((TB, out_stride), np.float32)
            r[:, :N] = residual
            res = dev(r)
    s = gemv_seg(w=dev(w), type=t, K=K, n_rows=N, out=out, out_stride=out_stride, residual=res, alpha=alpha,
                 x8=dev(act.x8), xmeta=dev(act.xmeta), xsumq=dev(act.xsumq))
    if TB == 1:
        be.i8_gemv(s)
    else:
        be.i8_gemm(s, TB)
    be.synchronize()
    return out.cpu().numpy().reshape(TB, out_stride)


def rel_err(got, ref, ab):
    return float(np.max(np.abs(got.astype(np.float64) - ref) / np.maximum(ab, 1e-30)))


@pytest.mark.parametrize("TB,K", [(1, 256), (1, 4096), (3, 5120), (16, 2048), (33, 512)])
def test_xq_bit_exact(be, orc, pkg, TB, K):
    x = pkg.synth.make_activation(TB, K, 300 + TB)
    x[0, 32:64] = 0.0  # an all-zero group must encode as scale 0
    a = orc.xq(x, None, TB)
    x8, xm, xs = gpu_xq(be, x, None, TB)
    assert np.array_equal(x8.cpu().numpy(), a.x8)
    assert np.array_equal(xm.cpu().numpy().view(np.uint32), a.xmeta.view(np.uint32))
    assert np.array_equal(xs.cpu().numpy(), a.xsumq)


def test_xq_golden_from_reference(be):
    x8, xm, xs = gpu_xq(be, G["xq_x"], None, 3)
    assert np.array_equal(x8.cpu().numpy(), G["xq_x8"])
    assert np.array_equal(xm.cpu().numpy().view(np.uint32), G["xq_meta"].view(np.uint32))
    assert np.array_equal(xs.cpu().numpy(), G["xq_sum"])


@pytest.mark.parametrize("TB,K", [(1, 512), (4, 17408)])
def test_xq_fused_silu(be, orc, pkg, TB, K):
    """silu(x)*up goes through exp: the device evaluates it in double and rounds once.
    Codes may differ from the host's expf only where a product lands on a rounding tie."""
    x, up = pkg.synth.make_activation(TB, K, 310), pkg.synth.make_activation(TB, K, 311)
    a = orc.xq(x, up, TB)
    x8, xm, xs = gpu_xq(be, x, up, TB)
    d = np.abs(x8.cpu().numpy().astype(np.int32) - a.x8.astype(np.int32))
    assert d.max() <= 1 and np.count_nonzero(d) <= 1e-4 * d.size
    sm = xm.cpu().numpy()
    assert np.count_nonzero(sm.view(np.uint32) != a.xmeta.view(np.uint32)) <= 1e-3 * sm.size
    assert np.max(np.abs(sm - a.xmeta)) <= 2.0 ** -10 * np.max(a.xmeta)


def test_xq_fused_silu_golden(be):
    x8, xm, _ = gpu_xq(be, G["xq_x"], G["xq_up"], 3)
    d = np.abs(x8.cpu().numpy().astype(np.int32) - G["xq_x8_up"].astype(np.int32))
    assert d.max() <= 1 and np.count_nonzero(d) <= 2


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("K,N,TB,tok", [(256, 3, 1, 0), (1024, 37, 1, 0), (5120, 7, 1, 0), (4352, 9, 3, 2), (512, 5, 9, 4)])
def test_block_dots_bit_exact(be, orc, po, pkg, t, K, N, TB, tok):
    w = pkg.synth.make_weight(t, N, K, 400 + t)
    a = orc.xq(pkg.synth.make_activation(TB, K, 401), None, TB)
    want = orc.block_dots(t, w, K, N, a, tok)
    wd = torch.empty(want.shape, dtype=torch.int32, device="cuda")
    be.i8_block_dots(dev(w), t, K, N, dev(a.x8), TB, tok, wd)
    be.synchronize()
    assert np.array_equal(wd.cpu().numpy(), want)


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("K,N", [(256, 1), (512, 5), (1024, 37), (5120, 64), (17408, 11)])
def test_gemv_parity(be, orc, pkg, t, K, N):
    w = pkg.synth.make_weight(t, N, K, 500 + t)
    a = orc.xq(pkg.synth.make_activation(1, K, 501))
    ref, ab = orc.gemm(t, w, K, N, a), orc.gemm_abs(t, w, K, N, a)
    got = gpu_gemm(be, t, w, K, N, a, 1)
    assert rel_err(got, ref, ab) <= TOL


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("TB", [2, 3, 5, 8, 16, 33])
def test_gemm_parity(be, orc, pkg, t, TB):
    K, N = 1024, 45
    w = pkg.synth.make_weight(t, N, K, 600 + t)
    a = orc.xq(pkg.synth.make_activation(TB, K, 601), None, TB)
    res = pkg.synth.make_activation(TB, N, 602)
    ref = orc.gemm(t, w, K, N, a, residual=res.copy(), alpha=0.5)
    ab = orc.gemm_abs(t, w, K, N, a, alpha=0.5) + np.abs(res)
    got = gpu_gemm(be, t, w, K, N, a, TB, residual=res, alpha=0.5)
    assert rel_err(got, ref, ab) <= TOL


@pytest.mark.parametrize("t", (12, 14, 8))
@pytest.mark.parametrize("TB,K", [(2, 17408), (4, 17408), (3, 8192), (4, 5120)])
def test_small_batch_long_k(be, orc, pkg, t, TB, K):
    """Two to four tokens with long rows: activation packs that fill half of shared memory
    (2 x 17408), packs that do not fit (4 x 17408: the tensor-core kernel takes the call), and
    the three- and four-token instantiations of the streaming kernel."""
    N = 70
    w = pkg.synth.make_weight(t, N, K, 650 + t)
    a = orc.xq(pkg.synth.make_activation(TB, K, 651), None, TB)
    ref = orc.gemm(t, w, K, N, a, alpha=0.25)
    ab = orc.gemm_abs(t, w, K, N, a, alpha=0.25)
    got = gpu_gemm(be, t, w, K, N, a, TB, alpha=0.25)
    assert be.device_status() == 0
    assert rel_err(got, ref, ab) <= TOL


@pytest.mark.parametrize("t", (12, 14))
def test_residual_alias_and_wide_stride(be, orc, pkg, t):
    """residual may alias out (in-place residual add, src/engine/graph.cpp:299,355 of the
    reference) and out_stride may exceed n_rows (gate|up halves, graph.cpp:342-343);
    columns beyond n_rows must stay untouched."""
    K, N, TB, stride = 512, 19, 3, 50
    w = pkg.synth.make_weight(t, N, K, 700 + t)
    a = orc.xq(pkg.synth.make_activation(TB, K, 701), None, TB)
    res = pkg.synth.make_activation(TB, N, 702)
    ref = orc.gemm(t, w, K, N, a, residual=res.copy(), alpha=2.0)
    ab = orc.gemm_abs(t, w, K, N, a, alpha=2.0) + np.abs(res)
    got = gpu_gemm(be, t, w, K, N, a, TB, residual=res, alpha=2.0, out_stride=stride, alias=True)
    assert rel_err(got[:, :N], ref, ab) <= TOL
    assert np.all(got[:, N:] == 7.0)


def test_multi_segment_call_mixed_types(be, orc, pkg):
    """q|k|v of one call: three segments, two types, one shared activation, one launch."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    K, TB = 1024, 2
    shapes = [(12, 96), (12, 24), (14, 24)]
    x = pkg.synth.make_activation(TB, K, 801)
    a = orc.xq(x, None, TB)
    x8, xm, xs = alloc_act(TB, K)
    dx = dev(x)
    segs, outs, ws = [], [], []
    for i, (t, n) in enumerate(shapes):
        w = pkg.synth.make_weight(t, n, K, 810 + i)
        ws.append(w)
        o = torch.zeros(TB * n, dtype=torch.float32, device="cuda")
        outs.append(o)
        segs.append(gemv_seg(w=dev(w), type=t, K=K, n_rows=n, x=dx, x_stride=K, out=o, out_stride=n, x8=x8,
                             xmeta=xm, xsumq=xs))
    be.quant_gemv(segs, TB)
    be.synchronize()
    assert np.array_equal(x8.cpu().numpy(), a.x8)
    for (t, n), w, o in zip(shapes, ws, outs):
        ref, ab = orc.gemm(t, w, K, n, a), orc.gemm_abs(t, w, K, n, a)
        assert rel_err(o.cpu().numpy().reshape(TB, n), ref, ab) <= TOL


@pytest.mark.parametrize("t", (12, 13, 14))
def test_golden_reference_outputs(be, orc, t):
    """Outputs of the reference's own compiled CPU path (default build), from the fixture."""
    K, N = 512, 5
    a1 = orc.xq(G["xq_x"][0])
    a3 = orc.xq(G["xq_x"], None, TB=3)
    got1 = gpu_gemm(be, t, G[f"w_{t}"], K, N, a1, 1, residual=G["res"][:1], alpha=0.75)
    got3 = gpu_gemm(be, t, G[f"w_{t}"], K, N, a3, 3, residual=G["res"], alpha=0.75)
    ab1 = orc.gemm_abs(t, G[f"w_{t}"], K, N, a1, alpha=0.75) + np.abs(G["res"][:1])
    ab3 = orc.gemm_abs(t, G[f"w_{t}"], K, N, a3, alpha=0.75) + np.abs(G["res"])
    assert rel_err(got1, G[f"gemv_{t}"][None, :], ab1) <= TOL
    assert rel_err(got3, G[f"gemm3_{t}"], ab3) <= TOL


def test_reference_unit_test_case(be, orc):
    a = orc.xq(G["ut_x"])
    got = gpu_gemm(be, 12, G["ut_w"], 256, 3, a, 1)
    ab = orc.gemm_abs(12, G["ut_w"], 256, 3, a)
    assert rel_err(got, G["ut_gemv"][None, :], ab) <= TOL


def test_config0_full_size(be, orc, pkg):
    """Benchmark configuration 0 at full size: 4096x4096 Q4_K, batch 1."""
    K = N = 4096
    w = pkg.synth.make_weight(12, N, K, 0xB200)
    x = pkg.synth.make_activation(1, K, 0xB201)
    a = orc.xq(x)
    x8, xm, xs = gpu_xq(be, x)
    assert np.array_equal(x8.cpu().numpy(), a.x8)
    ref, ab = orc.gemm(12, w, K, N, a), orc.gemm_abs(12, w, K, N, a)
    assert rel_err(gpu_gemm(be, 12, w, K, N, a, 1), ref, ab) <= TOL


@pytest.mark.parametrize("name", ["k", "v", "gate", "down"])
def test_config1_layer_shapes_full_size(be, orc, pkg, name):
    """Dense-layer projections of benchmark configuration 1 at full size (batch 1), plus
    size-independent properties: alpha-linearity is exact, and a row slice computed as its own
    call agrees with the same rows of the full call (the two may tile differently, so the
    fp32 summation order may differ)."""
    shape = {n: (t, r, k) for n, t, r, k in pkg.synth.dense_layer_shapes("Q4_K_M")}[name]
    t, N, K = shape
    w = pkg.synth.make_weight(t, N, K, 900)
    a = orc.xq(pkg.synth.make_activation(1, K, 901))
    ref, ab = orc.gemm(t, w, K, N, a), orc.gemm_abs(t, w, K, N, a)
    got = gpu_gemm(be, t, w, K, N, a, 1)
    assert rel_err(got, ref, ab) <= TOL
    got2 = gpu_gemm(be, t, w, K, N, a, 1, alpha=2.0)
    assert np.array_equal(got2, 2.0 * got)  # scaling by a power of two is exact
    rb = pkg.synth.row_bytes(t, K)
    r0, r1 = N // 3, N // 3 + 100
    part = gpu_gemm(be, t, w[r0 * rb:r1 * rb], K, r1 - r0, a, 1)
    assert rel_err(part, got[:, r0:r1].astype(np.float64), ab[:, r0:r1]) <= 1e-6


def test_errors_are_reported_not_swallowed(be, pkg):
    from sycl_infer_b200.backend import gemv_seg
    from sycl_infer_b200.capi import B200QError
    w = torch.zeros(144 * 4, dtype=torch.uint8, device="cuda")
    o = torch.zeros(4, dtype=torch.float32, device="cuda")
    with pytest.raises(B200QError) as e:
        be.i8_gemv(gemv_seg(w=w, type=2, K=256, n_rows=4, out=o, x8=w, xmeta=o, xsumq=o))
    assert e.value.code == 2
    with pytest.raises(B200QError):
        be.i8_gemv(gemv_seg(w=w, type=12, K=256, n_rows=4, out=o))  # no activation views


def test_zy_no_device_side_wait_ran_out(be):
    """Every mbarrier wait in the streaming kernel is bounded; none may have expired."""
    assert be.device_status() == 0


@pytest.mark.parametrize("t,K,N", [(12, 1024, 300), (14, 5120, 77), (23, 2048, 64), (13, 8192, 40)])
def test_quant_gemv_single_token_quantizes_in_kernel(be, orc, pkg, t, K, N):
    """One token, plain activation, short K: the GEMV kernel quantizes in its prologue (one
    launch).  Outputs against the oracle; the scratch views must hold the quantizer's exact
    codes, scales and sums all the same."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    x = pkg.synth.make_activation(1, K, 900 + t)
    res = pkg.synth.make_activation(1, N, 901)
    w = pkg.synth.make_weight(t, N, K, 902 + t)
    a = orc.xq(x)
    x8, xm, xs = alloc_act(1, K)
    o = torch.zeros(N, dtype=torch.float32, device="cuda")
    seg = gemv_seg(w=dev(w), type=t, K=K, n_rows=N, x=dev(x), x_stride=K, out=o, out_stride=N, residual=dev(res),
                   alpha=0.5, x8=x8, xmeta=xm, xsumq=xs)
    be.quant_gemv([seg], 1)
    be.synchronize()
    assert be.device_status() == 0
    assert np.array_equal(x8.cpu().numpy(), a.x8)
    assert np.array_equal(xm.cpu().numpy(), a.xmeta)
    assert np.array_equal(xs.cpu().numpy(), a.xsumq)
    ref = orc.gemm(t, w, K, N, a, residual=res.copy(), alpha=0.5)
    ab = orc.gemm_abs(t, w, K, N, a, alpha=0.5) + np.abs(res)
    assert rel_err(o.cpu().numpy().reshape(1, N), ref, ab) <= TOL


def test_quant_gemv_misaligned_activation_pointer(be, orc, pkg):
    """An fp32 activation that starts 4 bytes off a 16-byte boundary is legal (the reference's
    gemv_seg.x is any float pointer): the call must take the separate quantizer (scalar loads)
    instead of the in-kernel one (128-bit loads) and give the same results."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    t, K, N = 12, 2048, 70
    x = pkg.synth.make_activation(1, K, 930)
    w = pkg.synth.make_weight(t, N, K, 931)
    a = orc.xq(x)
    buf = torch.zeros(K + 4, dtype=torch.float32, device="cuda")
    dx = buf[1:K + 1]
    dx.copy_(torch.from_numpy(x[0]))
    assert dx.data_ptr() % 16 == 4
    x8, xm, xs = alloc_act(1, K)
    o = torch.zeros(N, dtype=torch.float32, device="cuda")
    be.quant_gemv([gemv_seg(w=dev(w), type=t, K=K, n_rows=N, x=dx, x_stride=K, out=o, out_stride=N, x8=x8, xmeta=xm,
                            xsumq=xs)], 1)
    be.synchronize()
    assert be.device_status() == 0
    assert np.array_equal(x8.cpu().numpy(), a.x8)
    ref, ab = orc.gemm(t, w, K, N, a), orc.gemm_abs(t, w, K, N, a)
    assert rel_err(o.cpu().numpy().reshape(1, N), ref, ab) <= TOL


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("K,N", [(256, 700), (2560, 333), (4096, 4096), (8704, 50), (32768, 9)])
def test_gemv_parity_row_slot_shapes(be, orc, pkg, t, K, N):
    """Single-token shapes that exercise the pinned kernel's geometry: many row slots per step
    (short K), a partly filled last step, unit counts that do not divide the lanes, long rows."""
    w = pkg.synth.make_weight(t, N, K, 940 + t)
    a = orc.xq(pkg.synth.make_activation(1, K, 941))
    res = pkg.synth.make_activation(1, N, 942)
    ref = orc.gemm(t, w, K, N, a, residual=res.copy(), alpha=0.5)
    ab = orc.gemm_abs(t, w, K, N, a, alpha=0.5) + np.abs(res)
    got = gpu_gemm(be, t, w, K, N, a, 1, residual=res, alpha=0.5)
    assert be.device_status() == 0
    assert rel_err(got, ref, ab) <= TOL


@pytest.mark.parametrize("K,n_ff", [(1024, 1280), (5120, 17408)])
def test_gate_up_emits_next_activation(be, orc, pkg, K, n_ff):
    """gate|up with the next-activation option: besides gate and up, the launch leaves
    quantize(silu(gate)*up) for the down call.  Codes, scales and sums must be exactly what the
    standalone quantizer makes of the SAME gate and up values (same device arithmetic), and agree
    with the host quantizer up to rounding ties of expf; a second call gives the same; the down call on that activation (no quantizer) matches the oracle."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    t = 12
    x = pkg.synth.make_activation(1, K, 950)
    wg, wu = pkg.synth.make_weight(t, n_ff, K, 951), pkg.synth.make_weight(t, n_ff, K, 952)
    a = orc.xq(x)
    alpha = 1.0 / (3.0 * K ** 0.5)
    gu = torch.zeros(1, 2 * n_ff, dtype=torch.float32, device="cuda")
    x8, xm, xs = alloc_act(1, K)
    h8, hm, hs = alloc_act(1, n_ff)
    dx, dwg, dwu = dev(x), dev(wg), dev(wu)
    segs = [gemv_seg(w=dwg, type=t, K=K, n_rows=n_ff, x=dx, x_stride=K, out=gu.view(-1), out_stride=2 * n_ff,
                     alpha=alpha, x8=x8, xmeta=xm, xsumq=xs),
            gemv_seg(w=dwu, type=t, K=K, n_rows=n_ff, x=dx, x_stride=K, out=gu.view(-1)[n_ff:], out_stride=2 * n_ff,
                     alpha=alpha, x8=x8, xmeta=xm, xsumq=xs)]
    for _ in range(2):
        h8.zero_()
        be.quant_gemv_ex(segs, 1, next_act=(h8, hm, hs))
        be.synchronize()
        assert be.device_status() == 0
        g = gu.cpu().numpy()
        for wq, lo in ((wg, 0), (wu, n_ff)):
            rows = slice(0, n_ff) if n_ff <= 2048 else slice(n_ff - 300, n_ff)
            rb = pkg.synth.row_bytes(t, K)
            sub = wq[rows.start * rb:rows.stop * rb]
            ref = orc.gemm(t, sub, K, rows.stop - rows.start, a, alpha=alpha)
            ab = orc.gemm_abs(t, sub, K, rows.stop - rows.start, a, alpha=alpha)
            assert rel_err(g[:, lo + rows.start:lo + rows.stop], ref, ab) <= TOL
        q8, qm, qs = gpu_xq(be, g[:, :n_ff], g[:, n_ff:], 1)  # the standalone quantizer on the same values
        assert np.array_equal(h8.cpu().numpy(), q8.cpu().numpy())
        assert np.array_equal(hm.cpu().numpy().view(np.uint32), qm.cpu().numpy().view(np.uint32))
        assert np.array_equal(hs.cpu().numpy(), qs.cpu().numpy())
        host = orc.xq(g[:, :n_ff], g[:, n_ff:], 1)
        d = np.abs(h8.cpu().numpy().astype(np.int32) - host.x8.astype(np.int32))
        assert d.max() <= 1 and np.count_nonzero(d) <= 1e-4 * d.size + 1
    # down on the emitted activation, quantizer skipped
    N = 64
    wd_ = pkg.synth.make_weight(14, N, n_ff, 953)
    o = torch.zeros(N, dtype=torch.float32, device="cuda")
    be.quant_gemv_ex([gemv_seg(w=dev(wd_), type=14, K=n_ff, n_rows=N, out=o, out_stride=N, x8=h8, xmeta=hm, xsumq=hs)],
                     1, prequantized=True)
    be.synchronize()
    act = orc.xq(g[:, :n_ff], g[:, n_ff:], 1)
    act.x8, act.xmeta, act.xsumq = h8.cpu().numpy(), hm.cpu().numpy(), hs.cpu().numpy()
    ref, ab = orc.gemm(14, wd_, n_ff, N, act), orc.gemm_abs(14, wd_, n_ff, N, act)
    assert rel_err(o.cpu().numpy().reshape(1, N), ref, ab) <= TOL


@pytest.mark.parametrize("t,K,N", [(12, 5120, 5120), (14, 2048, 1024), (13, 1024, 96)])
def test_single_segment_emits_next_activation(be, orc, pkg, t, K, N):
    """A one-segment call (the o projection, or down with its residual) that also leaves its
    output quantized for the next call: the emitted codes, scales and sums are exactly the
    standalone quantizer's on the stored output, and the host quantizer's too (no exp involved:
    the arithmetic is the reference's, bit for bit)."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    x = pkg.synth.make_activation(1, K, 970)
    res = pkg.synth.make_activation(1, N, 971)
    w = pkg.synth.make_weight(t, N, K, 972)
    a = orc.xq(x)
    alpha = 1.0 / (3.0 * K ** 0.5)
    x8, xm, xs = alloc_act(1, K)
    n8, nm, ns = alloc_act(1, N)
    out = torch.zeros(N, dtype=torch.float32, device="cuda")
    seg = gemv_seg(w=dev(w), type=t, K=K, n_rows=N, x=dev(x), x_stride=K, out=out, out_stride=N, residual=dev(res),
                   alpha=alpha, x8=x8, xmeta=xm, xsumq=xs)
    for _ in range(2):
        n8.zero_()
        be.quant_gemv_ex([seg], 1, next_act=(n8, nm, ns))
        be.synchronize()
        assert be.device_status() == 0
        got = out.cpu().numpy().reshape(1, N)
        ref = orc.gemm(t, w, K, N, a, residual=res.copy(), alpha=alpha)
        ab = orc.gemm_abs(t, w, K, N, a, alpha=alpha) + np.abs(res)
        assert rel_err(got, ref, ab) <= TOL
        host = orc.xq(got)
        assert np.array_equal(n8.cpu().numpy(), host.x8)
        assert np.array_equal(nm.cpu().numpy().view(np.uint32), host.xmeta.view(np.uint32))
        assert np.array_equal(ns.cpu().numpy(), host.xsumq)


def test_moe_rejects_misaligned_activation(be):
    """The expert kernels read the quantized activation with 128-bit loads: a misaligned view is
    refused with EINVAL before any launch."""
    from sycl_infer_b200.capi import B200QError
    import ctypes as C
    z = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = z.data_ptr()
    i32 = torch.zeros(64, dtype=torch.int32, device="cuda")
    f32 = torch.zeros(4096, dtype=torch.float32, device="cuda")
    lib = be.lib
    rc = lib.moe_gate_up(None, p, p, 12, 12, 144 * 8 * 8, 144 * 8 * 8, i32.data_ptr(), i32.data_ptr(), i32.data_ptr(),
                         i32.data_ptr(), 1, p + 4, f32.data_ptr(), i32.data_ptr(), 1, f32.data_ptr(), 8, 2048, 8, 1)
    assert rc == 1 and "16-byte aligned" in lib.last_error()
    rc = lib.moe_down(None, p, 12, 144 * 2 * 8, i32.data_ptr(), i32.data_ptr(), i32.data_ptr(), i32.data_ptr(), 1,
                      p + 8, f32.data_ptr(), i32.data_ptr(), 1, f32.data_ptr(), 2048, 2048, 512)
    assert rc == 1 and "16-byte aligned" in lib.last_error()
    del B200QError, C


def test_second_device_in_one_process(pkg, orc):
    """One process, two GPUs (the reference's layer split runs this way): kernels that opt in to
    large dynamic shared memory must be configured on the second device too."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    for d in (0, 1):
        with torch.cuda.device(d):
            be_d = pkg.make_cuda_backend(d)
            for TB, t, K, N in ((1, 12, 5120, 300), (3, 14, 2048, 70), (16, 12, 1024, 200)):
                w = pkg.synth.make_weight(t, N, K, 960)
                x = pkg.synth.make_activation(TB, K, 961)
                a = orc.xq(x, None, TB)
                x8, xm, xs = alloc_act(TB, K, device=f"cuda:{d}")
                o = torch.zeros(TB * N, dtype=torch.float32, device=f"cuda:{d}")
                seg = gemv_seg(w=torch.from_numpy(w).to(f"cuda:{d}"), type=t, K=K, n_rows=N,
                               x=torch.from_numpy(x).to(f"cuda:{d}"), x_stride=K, out=o, out_stride=N, x8=x8,
                               xmeta=xm, xsumq=xs)
                be_d.quant_gemv([seg], TB)
                be_d.synchronize()
                ref, ab = orc.gemm(t, w, K, N, a), orc.gemm_abs(t, w, K, N, a)
                assert rel_err(o.cpu().numpy().reshape(TB, N), ref, ab) <= TOL
            assert be_d.device_status() == 0


@pytest.mark.parametrize("t,K,N", [(12, 1024, 96), (12, 5120, 640), (14, 2048, 128)])
def test_rmsnorm_folded_into_the_quantizer(be, orc, pkg, t, K, N):
    """b200q_call_opts.norm: the call consumes quantize(rmsnorm(x)).  The codes, scales and sums the
    launch leaves in the scratch views are the host quantizer's on the oracle's rmsnorm row (the
    reference's rmsnorm_row in its AVX-512 summation order), bit for bit; outputs against the oracle
    GEMV on exactly that activation."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    x = pkg.synth.make_activation(1, K, 1201)
    g = (1.0 + 0.2 * pkg.synth.make_activation(1, K, 1202)).astype(np.float32)
    w = pkg.synth.make_weight(t, N, K, 1203)
    eps = 1e-6
    x8, xm, xs = alloc_act(1, K)
    out = torch.zeros(N, dtype=torch.float32, device="cuda")
    alpha = 1.0 / (3.0 * K ** 0.5)
    seg = gemv_seg(w=dev(w), type=t, K=K, n_rows=N, x=dev(x), x_stride=K, out=out, out_stride=N, alpha=alpha,
                   x8=x8, xmeta=xm, xsumq=xs)
    for _ in range(2):
        x8.zero_()
        be.quant_gemv_ex([seg], 1, norm=(dev(g), eps))
        be.synchronize()
        assert be.device_status() == 0
        a = orc.xq(orc.rmsnorm(x, g, eps, 16))
        assert np.array_equal(x8.cpu().numpy(), a.x8)
        assert np.array_equal(xm.cpu().numpy().view(np.uint32), a.xmeta.view(np.uint32))
        assert np.array_equal(xs.cpu().numpy(), a.xsumq)
        ref, ab = orc.gemm(t, w, K, N, a, alpha=alpha), orc.gemm_abs(t, w, K, N, a, alpha=alpha)
        assert rel_err(out.cpu().numpy().reshape(1, N), ref, ab) <= TOL


def test_rmsnorm_with_gate_up_next_activation(be, orc, pkg):
    """norm -> quantize -> gate|up -> silu(gate)*up -> quantize in ONE launch."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    K, n_ff, t = 1024, 1280, 12
    x = pkg.synth.make_activation(1, K, 1301)
    g = (1.0 + 0.2 * pkg.synth.make_activation(1, K, 1302)).astype(np.float32)
    wg, wu = pkg.synth.make_weight(t, n_ff, K, 1303), pkg.synth.make_weight(t, n_ff, K, 1304)
    alpha = 1.0 / (3.0 * K ** 0.5)
    gu = torch.zeros(1, 2 * n_ff, dtype=torch.float32, device="cuda")
    x8, xm, xs = alloc_act(1, K)
    h8, hm, hs = alloc_act(1, n_ff)
    dx = dev(x)
    segs = [gemv_seg(w=dev(wg), type=t, K=K, n_rows=n_ff, x=dx, x_stride=K, out=gu.view(-1), out_stride=2 * n_ff,
                     alpha=alpha, x8=x8, xmeta=xm, xsumq=xs),
            gemv_seg(w=dev(wu), type=t, K=K, n_rows=n_ff, x=dx, x_stride=K, out=gu.view(-1)[n_ff:], out_stride=2 * n_ff,
                     alpha=alpha, x8=x8, xmeta=xm, xsumq=xs)]
    be.quant_gemv_ex(segs, 1, next_act=(h8, hm, hs), norm=(dev(g), 1e-5))
    be.synchronize()
    assert be.device_status() == 0
    a = orc.xq(orc.rmsnorm(x, g, 1e-5, 16))
    assert np.array_equal(x8.cpu().numpy(), a.x8)
    got = gu.cpu().numpy()
    for wq, lo in ((wg, 0), (wu, n_ff)):
        ref, ab = orc.gemm(t, wq, K, n_ff, a, alpha=alpha), orc.gemm_abs(t, wq, K, n_ff, a, alpha=alpha)
        assert rel_err(got[:, lo:lo + n_ff], ref, ab) <= TOL
    q8, qm, qs = gpu_xq(be, got[:, :n_ff], got[:, n_ff:], 1)
    assert np.array_equal(h8.cpu().numpy(), q8.cpu().numpy()) and np.array_equal(hs.cpu().numpy(), qs.cpu().numpy())


def test_rmsnorm_option_refused_where_it_cannot_be_folded(be, pkg):
    """Several tokens, or a pre-quantized activation: B200Q_EUNSUPPORTED, nothing launched."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    from sycl_infer_b200.capi import B200QError
    K, N = 1024, 64
    w = dev(pkg.synth.make_weight(12, N, K, 1401))
    g = dev(np.ones(K, np.float32))
    for TB, preq in ((3, False), (1, True)):
        x = dev(pkg.synth.make_activation(TB, K, 1402))
        x8, xm, xs = alloc_act(TB, K)
        out = torch.zeros(TB * N, dtype=torch.float32, device="cuda")
        seg = gemv_seg(w=w, type=12, K=K, n_rows=N, x=x, x_stride=K, out=out, out_stride=N, x8=x8, xmeta=xm, xsumq=xs)
        with pytest.raises(B200QError) as ei:
            be.quant_gemv_ex([seg], TB, prequantized=preq, norm=(g, 1e-6))
        assert ei.value.code == 2
