"""Row argmax on the device (compute_backend::mtp_argmax) and as the tail of the single-token GEMV:
the index of the largest value, the LOWEST index among equals, as the reference's host scan
`best = 0; if (row[i] > row[best]) best = i` (src/backend/cpu/cpu_backend.cpp:117-128)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def host_scan(row):
    best = 0
    for i in range(1, len(row)):
        if row[i] > row[best]:
            best = i
    return best


@pytest.mark.parametrize("M,n", [(1, 248320), (5, 248320), (70, 1000), (3, 1), (2, 33)])
def test_argmax_rows(be, M, n):
    rng = np.random.default_rng(M * 1000 + n)
    x = rng.normal(0, 1, (M, n)).astype(np.float32)
    if n > 40:
        x[0, [n - 1, 17, n // 2]] = 9.0       # three equal maxima: the lowest index wins
        x[-1, :] = -np.abs(x[-1, :]) - 1.0     # all negative
    d = torch.from_numpy(x).cuda()
    idx = torch.full((M,), -7, dtype=torch.int32, device="cuda")
    val = torch.zeros(M, dtype=torch.float32, device="cuda")
    for _ in range(2):  # the device-side words return to zero between calls
        be.mtp_argmax(d, n, idx, val, M)
        be.synchronize()
        assert be.device_status() == 0
        want = x.argmax(axis=1)  # numpy's argmax returns the first maximum
        assert np.array_equal(idx.cpu().numpy(), want.astype(np.int32))
        assert np.array_equal(val.cpu().numpy(), x[np.arange(M), want])
    if n <= 1000:
        assert [host_scan(r) for r in x[:4]] == list(want[:4])
    be.mtp_argmax(d, n, idx, None, M)  # the value is optional
    be.synchronize()
    assert np.array_equal(idx.cpu().numpy(), want.astype(np.int32))


def test_argmax_zero_signs_tie(be):
    """-0.0 and +0.0 compare equal under the host's `>`: the lower index wins whatever the sign."""
    x = np.full((2, 300), -1.0, np.float32)
    x[0, 40], x[0, 200] = -0.0, 0.0
    x[1, 40], x[1, 200] = 0.0, -0.0
    idx = torch.zeros(2, dtype=torch.int32, device="cuda")
    be.mtp_argmax(torch.from_numpy(x).cuda(), 300, idx, None, 2)
    be.synchronize()
    assert list(idx.cpu().numpy()) == [40, 40]


@pytest.mark.parametrize("t,K,N", [(14, 1024, 4096), (12, 5120, 40000), (13, 1024, 77)])
def test_gemv_with_argmax_tail(be, orc, pkg, t, K, N):
    """The LM-head form: logits = W x stored as usual, and the argmax of exactly those stored values
    from the same launch.  Some rows are copies of others, so their logits tie bit for bit."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    w = pkg.synth.make_weight(t, N, K, 1501).copy()
    rb = pkg.synth.row_bytes(t, K)
    x = pkg.synth.make_activation(1, K, 1502)
    x8, xm, xs = alloc_act(1, K)
    out = torch.zeros(N, dtype=torch.float32, device="cuda")
    idx = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    val = torch.zeros(1, dtype=torch.float32, device="cuda")
    seg = gemv_seg(w=None, type=t, K=K, n_rows=N, x=torch.from_numpy(x).cuda(), x_stride=K, out=out, out_stride=N,
                   x8=x8, xmeta=xm, xsumq=xs)
    for rnd in range(2):
        if rnd == 1:  # plant the winning row again at a higher and at a lower index
            win = int(out.cpu().numpy().argmax())
            for dst in (N - 1, max(0, win - 3)):
                w[dst * rb:(dst + 1) * rb] = w[win * rb:(win + 1) * rb]
        seg.w = torch.from_numpy(w).cuda()
        be.quant_gemv_ex([seg], 1, argmax=(idx, val))
        be.synchronize()
        assert be.device_status() == 0
        got = out.cpu().numpy()
        assert int(idx.cpu()[0]) == int(got.argmax())
        assert float(val.cpu()[0]) == float(got[got.argmax()])
    a = orc.xq(x)
    rows = slice(0, min(N, 256))
    ref = orc.gemm(t, w[:rows.stop * rb], K, rows.stop, a)
    ab = orc.gemm_abs(t, w[:rows.stop * rb], K, rows.stop, a)
    assert float(np.max(np.abs(got[rows] - ref[0]) / ab[0])) <= 1e-5
