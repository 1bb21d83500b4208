"""Tensor-core GEMM path (more than 8 tokens: tcgen05 int8 MMA per 32-value group) against the
oracle's tiled-GEMM order.  fp32 outputs within 1e-5 of the sum of |terms|; the int32 group
dots come out of the tensor core exact, which the fp32 agreement at this tolerance on
cancelling sums already demands."""
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
