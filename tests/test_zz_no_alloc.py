"""b200q_quant_gemv_static: the fused quantize + GEMV for hosts that cannot allocate.

An embedder that has no device allocator to offer (all memory already committed to its
weight blob and arena, or a host process whose allocator a plugin must not touch) cannot
hand b200q_quant_gemv the int8 activation scratch it needs.  The static variant keeps that
scratch inside the library image.  Here it is called through the C ABI twice in a row, on
different inputs, and each result is compared with b200q_quant_gemv on caller-owned scratch:
the second call proves that whatever the first left in the shared array is not consumed.
This file sorts last so that a run stopping at the first failure has run everything else.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL = 1e-5  # of the row's sum of |terms|, the tolerance of the parity tests


def _run(be, orc, pkg, qtype, K, N, seed, use_up):
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    w = pkg.synth.make_weight(qtype, N, K, seed)
    x = pkg.synth.make_activation(1, K, seed + 1)
    up = pkg.synth.make_activation(1, K, seed + 2) if use_up else None
    dw, dx = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    dup = None if up is None else torch.from_numpy(up).cuda()
    res = torch.from_numpy(pkg.synth.make_activation(1, N, seed + 3)).cuda()
    outs = []
    for static in (False, True):
        out = torch.full((N,), -3.0, dtype=torch.float32, device="cuda")
        x8, xm, xs = alloc_act(1, K)
        seg = gemv_seg(w=dw, type=qtype, K=K, n_rows=N, x=dx, x_stride=K, act_up=dup, out=out, out_stride=N,
                       residual=res, alpha=0.5, x8=None if static else x8, xmeta=None if static else xm,
                       xsumq=None if static else xs)
        if static:
            be.quant_gemv_static([seg])
        else:
            be.quant_gemv([seg], 1)
        be.synchronize()
        outs.append(out.cpu().numpy())
    act = orc.xq(x, up)
    ab = orc.gemm_abs(qtype, w, K, N, act, alpha=0.5)[0] + np.abs(res.cpu().numpy()[0])
    ref = orc.gemm(qtype, w, K, N, act, residual=res.cpu().numpy().copy(), alpha=0.5)[0]
    return outs[0], outs[1], ref, ab


def test_static_scratch_matches_caller_scratch_twice_in_a_row(be, orc, pkg):
    # call 1: long K, so the shared array is left full of a previous activation
    a, b, ref, ab = _run(be, orc, pkg, 12, 17408, 40, 7001, use_up=True)
    assert np.max(np.abs(a.astype(np.float64) - b) / ab) <= TOL
    assert np.max(np.abs(b.astype(np.float64) - ref) / ab) <= 5e-4  # silu through expf: codes may differ at rounding ties
    # call 2: another type, a shorter K and other values, straight after
    a2, b2, ref2, ab2 = _run(be, orc, pkg, 14, 5120, 64, 7011, use_up=False)
    assert np.max(np.abs(a2.astype(np.float64) - b2) / ab2) <= TOL
    assert np.max(np.abs(b2.astype(np.float64) - ref2) / ab2) <= TOL
    assert be.device_status() == 0


@pytest.mark.parametrize("qtype", (12, 14))
def test_static_scratch_at_its_size_limit(be, orc, pkg, qtype):
    """K = B200Q_STATIC_MAX_K: the whole built-in array is in use (codes, scales and sums of
    32768 values); the result is checked against the oracle as well as against caller scratch."""
    a, b, ref, ab = _run(be, orc, pkg, qtype, 32768, 6, 7021, use_up=False)
    assert np.max(np.abs(a.astype(np.float64) - b) / ab) <= TOL
    assert np.max(np.abs(b.astype(np.float64) - ref) / ab) <= TOL
    assert be.device_status() == 0


def test_static_scratch_refuses_what_does_not_fit(be, pkg):
    from sycl_infer_b200.backend import gemv_seg
    from sycl_infer_b200.capi import B200QError
    K = 32768 + 256
    w = torch.zeros(144 * (K // 256), dtype=torch.uint8, device="cuda")
    x = torch.zeros(K, dtype=torch.float32, device="cuda")
    o = torch.zeros(1, dtype=torch.float32, device="cuda")
    with pytest.raises(B200QError) as e:
        be.quant_gemv_static([gemv_seg(w=w, type=12, K=K, n_rows=1, x=x, x_stride=K, out=o)])
    assert e.value.code == 2 and "exceeds the built-in scratch" in str(e.value)
