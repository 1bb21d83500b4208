"""Tensor-core GEMM path (five tokens and more: one tcgen05 int8 MMA per 32-value group) against
the oracle.  The int32 group dots are compared bit for bit: b200q_i8_block_dots with five or
more tokens runs the tensor-core kernel itself and stores the accumulators its epilogue read
from tensor memory.  fp32 outputs are within 1e-5 of the sum of |terms| of the oracle's
tiled-GEMM order."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
TOL = 1e-5


def _gemm(be, t, w, K, N, act, TB, residual=None, alpha=1.0):
    from sycl_infer_b200.backend import gemv_seg
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
    out = torch.full((TB * N,), 5.0, dtype=torch.float32, device="cuda")
    s = gemv_seg(w=dev(w), type=t, K=K, n_rows=N, out=out, out_stride=N, alpha=alpha,
                 residual=None if residual is None else dev(residual), x8=dev(act.x8), xmeta=dev(act.xmeta),
                 xsumq=dev(act.xsumq))
    be.i8_gemm(s, TB)
    be.synchronize()
    assert be.device_status() == 0
    return out.cpu().numpy().reshape(TB, N)


@pytest.mark.parametrize("t", (12, 13, 14, 8, 23))
@pytest.mark.parametrize("TB,N,K", [(16, 128, 256), (32, 200, 512), (9, 37, 1024), (130, 260, 512), (256, 128, 768),
                                    (4, 300, 512), (8, 129, 1280), (5, 64, 256)])
def test_mma_gemm_parity(be, orc, pkg, t, TB, N, K):
    w = pkg.synth.make_weight(t, N, K, 1200 + t)
    a = orc.xq(pkg.synth.make_activation(TB, K, 1201), None, TB)
    res = pkg.synth.make_activation(TB, N, 1202)
    ref = orc.gemm(t, w, K, N, a, residual=res.copy(), alpha=0.5)
    ab = orc.gemm_abs(t, w, K, N, a, alpha=0.5) + np.abs(res)
    got = _gemm(be, t, w, K, N, a, TB, residual=res, alpha=0.5)
    assert float(np.max(np.abs(got - ref) / ab)) <= TOL


def test_batched_decode_config1_batch16(be, orc, pkg):
    """gate projection of benchmark configuration 1 at batch 16 (full size)."""
    t, N, K, TB = 12, 17408, 5120, 16
    w = pkg.synth.make_weight(t, N, K, 1300)
    a = orc.xq(pkg.synth.make_activation(TB, K, 1301), None, TB)
    ref, ab = orc.gemm(t, w, K, N, a), orc.gemm_abs(t, w, K, N, a)
    got = _gemm(be, t, w, K, N, a, TB)
    assert float(np.max(np.abs(got - ref) / ab)) <= TOL


def test_prefill_config2_slice(be, orc, pkg):
    """Prefill GEMM of configuration 2 (M = 512 tokens, K = 5120) on a 1024-row slice of the
    17408-row gate weight: the oracle finishes this in seconds; the full N is covered by the
    batch-16 case and by linearity in rows (every row is independent)."""
    t, N, K, TB = 12, 1024, 5120, 512
    w = pkg.synth.make_weight(t, N, K, 1400)
    a = orc.xq(pkg.synth.make_activation(TB, K, 1401), None, TB)
    ref, ab = orc.gemm(t, w, K, N, a), orc.gemm_abs(t, w, K, N, a)
    got = _gemm(be, t, w, K, N, a, TB)
    assert float(np.max(np.abs(got - ref) / ab)) <= TOL


def _dots(be, t, w, K, N, act, TB, tok):
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
    D = K // 16 if t == 14 else K // 32
    wd = torch.full((N, D), -77, dtype=torch.int32, device="cuda")
    be.i8_block_dots(dev(w), t, K, N, dev(act.x8), TB, tok, wd)
    be.synchronize()
    assert be.device_status() == 0
    return wd.cpu().numpy()


@pytest.mark.parametrize("t", (12, 13, 14, 8, 23))
@pytest.mark.parametrize("TB,N,K", [(5, 64, 256), (8, 130, 512), (16, 128, 1280), (32, 200, 512), (33, 129, 768),
                                    (64, 37, 512), (100, 260, 256)])
def test_mma_int32_dots_bit_exact(be, orc, pkg, t, TB, N, K):
    """Token tiles of 8 / 16 / 32 / 64 columns, ragged last row tile and last token tile: the
    accumulators the tensor core produced are the reference's int32 sums
    (src/backend/cpu/kernels/i8.cpp:57,117,149 of the reference), bit for bit, for the first, a
    middle and the last token."""
    w = pkg.synth.make_weight(t, N, K, 1500 + t)
    a = orc.xq(pkg.synth.make_activation(TB, K, 1501), None, TB)
    for tok in sorted({0, TB // 2, TB - 1}):
        want = orc.block_dots(t, w, K, N, a, tok)
        got = _dots(be, t, w, K, N, a, TB, tok)
        assert np.array_equal(got, want), f"token {tok}"


def _saturated(pkg, t, N, K):
    """Weights whose every quant code is the largest in magnitude the format holds (scales stay
    random): 15 / 31 / 63 for Q4_K / Q5_K / Q6_K, +127 and -128 on alternating rows for Q8_0,
    codebook entry 0 (-127) for IQ4_XS."""
    sbb = pkg.synth.SUPERBLOCK_BYTES[t]
    w = pkg.synth.make_weight(t, N, K, 1600 + t).reshape(N, K // 256, sbb).copy()
    if t == 12:
        w[:, :, 16:] = 0xFF
    elif t == 13:
        w[:, :, 16:] = 0xFF
    elif t == 14:
        w[:, :, :192] = 0xFF
    elif t == 23:
        w[:, :, 8:] = 0x00
    else:
        b = w.reshape(N, K // 32, 34)
        b[0::2, :, 2:] = 0x7F
        b[1::2, :, 2:] = 0x80
    return w.reshape(-1)


@pytest.mark.parametrize("t", (12, 13, 14, 8, 23))
@pytest.mark.parametrize("TB", (8, 48))
def test_mma_saturated_operands(be, orc, pkg, t, TB):
    """Every activation code +-127 against the largest weight codes: the int32 sums reach their
    extreme (32*127*128 = 520192 for Q8_0), far inside the 2^22 range the epilogue's
    integer-to-float conversion relies on; both the raw sums and the fp32 outputs must hold."""
    N, K = 130, 512
    w = _saturated(pkg, t, N, K)
    x = np.ones((TB, K), np.float32)
    x[1::2] = -1.0
    x[:, 5::7] *= -1.0  # mixed signs inside a group as well
    a = orc.xq(x, None, TB)
    assert np.all(np.abs(a.x8) == 127)
    for tok in (0, TB - 1):
        want = orc.block_dots(t, w, K, N, a, tok)
        assert np.array_equal(_dots(be, t, w, K, N, a, TB, tok), want)
    all_pos = orc.xq(np.ones((TB, K), np.float32), None, TB)
    assert np.max(np.abs(orc.block_dots(t, w, K, N, all_pos, 0))) >= {12: 60960, 13: 125984, 14: 128016, 8: 516128,
                                                                       23: 516128}[t]
    assert np.array_equal(_dots(be, t, w, K, N, all_pos, TB, 0), orc.block_dots(t, w, K, N, all_pos, 0))
    for act in (a, all_pos):
        ref, ab = orc.gemm(t, w, K, N, act), orc.gemm_abs(t, w, K, N, act)
        got = _gemm(be, t, w, K, N, act, TB)
        assert float(np.max(np.abs(got - ref) / ab)) <= TOL


def test_prefill_config2_m2048_sampled_rows(be, orc, pkg):
    """Prefill GEMM of configuration 2 at M = 2048 tokens, K = 5120: the GPU computes a 256-row
    slice of the gate weight for all 2048 tokens (two full row tiles, 32 token tiles of 64); the
    oracle checks 64 sampled rows x all tokens."""
    t, N, K, TB = 12, 256, 5120, 2048
    w = pkg.synth.make_weight(t, N, K, 1700)
    a = orc.xq(pkg.synth.make_activation(TB, K, 1701), None, TB)
    got = _gemm(be, t, w, K, N, a, TB)
    rb = pkg.synth.row_bytes(t, K)
    rows = np.random.default_rng(5).choice(N, 64, replace=False)
    sub = np.concatenate([w[r * rb:(r + 1) * rb] for r in rows])
    ref, ab = orc.gemm(t, sub, K, 64, a), orc.gemm_abs(t, sub, K, 64, a)
    assert float(np.max(np.abs(got[:, rows] - ref) / ab)) <= TOL


@pytest.mark.parametrize("t,N,K", [(23, 17408, 5120), (13, 17408, 5120), (23, 5120, 17408), (13, 5120, 17408)])
def test_batch32_layer_shapes_iq4xs_q5k(be, orc, pkg, t, N, K):
    """Configuration 4's batch 32 on the real layer shapes in IQ4_XS and Q5_K (one gate-shaped and
    one down-shaped matrix each): the GPU computes the full matrix, the oracle 96 sampled rows."""
    TB = 32
    w = pkg.synth.make_weight(t, N, K, 1800 + t)
    a = orc.xq(pkg.synth.make_activation(TB, K, 1801), None, TB)
    got = _gemm(be, t, w, K, N, a, TB)
    rb = pkg.synth.row_bytes(t, K)
    rows = np.sort(np.random.default_rng(6).choice(N, 96, replace=False))
    sub = np.concatenate([w[r * rb:(r + 1) * rb] for r in rows])
    ref, ab = orc.gemm(t, sub, K, 96, a), orc.gemm_abs(t, sub, K, 96, a)
    assert float(np.max(np.abs(got[:, rows] - ref) / ab)) <= TOL


@pytest.mark.parametrize("t", (12, 13, 14, 8, 23))
@pytest.mark.parametrize("TB,N,K", [(2, 16, 256), (7, 45, 768), (9, 130, 1024), (16, 700, 512), (17, 300, 2560),
                                    (32, 129, 768), (4, 5120, 1024), (24, 96, 4352)])
def test_fragment_kernel_geometry(be, orc, pkg, t, TB, N, K):
    """2..32 tokens (the register-fragment MMA kernel): one and two token halves, 8- and 16-column
    warps, row tiles from 16 to 128 rows with 1..8 K slices, ragged rows and tokens, and row pitches
    that need 1, 2, 4 or 8 alignment classes (Q6_K with 1, 3, 4, 10, 17 superblocks per row).
    Outputs against the oracle, and the raw int32 sums of one token bit for bit."""
    w = pkg.synth.make_weight(t, N, K, 1900 + t)
    a = orc.xq(pkg.synth.make_activation(TB, K, 1901), None, TB)
    res = pkg.synth.make_activation(TB, N, 1902)
    ref = orc.gemm(t, w, K, N, a, residual=res.copy(), alpha=0.5)
    ab = orc.gemm_abs(t, w, K, N, a, alpha=0.5) + np.abs(res)
    got = _gemm(be, t, w, K, N, a, TB, residual=res, alpha=0.5)
    assert float(np.max(np.abs(got - ref) / ab)) <= TOL
    tok = TB - 1
    assert np.array_equal(_dots(be, t, w, K, N, a, TB, tok), orc.block_dots(t, w, K, N, a, tok))


def test_fragment_kernel_mixed_segments(be, orc, pkg):
    """q|k|v at batch 8: three segments, two weight types (Q4_K rows of pitch 16k, Q6_K rows in
    two alignment classes), one launch."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
    K, TB = 5120, 8
    shapes = [(12, 640), (12, 128), (14, 128)]
    x = pkg.synth.make_activation(TB, K, 2001)
    a = orc.xq(x, None, TB)
    x8, xm, xs = alloc_act(TB, K)
    dx = dev(x)
    segs, outs, ws = [], [], []
    for i, (t, n) in enumerate(shapes):
        w = pkg.synth.make_weight(t, n, K, 2010 + i)
        ws.append(w)
        o = torch.zeros(TB * n, dtype=torch.float32, device="cuda")
        outs.append(o)
        segs.append(gemv_seg(w=dev(w), type=t, K=K, n_rows=n, x=dx, x_stride=K, out=o, out_stride=n, x8=x8, xmeta=xm,
                             xsumq=xs))
    be.quant_gemv(segs, TB)
    be.synchronize()
    assert be.device_status() == 0
    for (t, n), w, o in zip(shapes, ws, outs):
        ref, ab = orc.gemm(t, w, K, n, a), orc.gemm_abs(t, w, K, n, a)
        assert float(np.max(np.abs(o.cpu().numpy().reshape(TB, n) - ref) / ab)) <= TOL
