"""The measurement instruments run, leave the device status clean and do not report a wait that
ran out (their numbers are taken by bench.py; here only that they work)."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_probes_run_clean(be):
    buf = torch.full((64 << 20,), 3, dtype=torch.uint8, device="cuda")
    sink = torch.zeros(1, dtype=torch.int32, device="cuda")
    be.lib.check(be.lib.probe_hbm_read(be._s(), C.c_void_p(buf.data_ptr()), C.c_size_t(buf.numel()), C.c_void_p(sink.data_ptr())))
    for iters in (1, 32, 33, 100, 4096):  # fewer than one batch, exactly one, ragged, many
        be.lib.check(be.lib.probe_i8_mma(be._s(), iters, C.c_void_p(sink.data_ptr())))
    be.synchronize()
    assert be.device_status() == 0
    assert int(sink.cpu()[0]) == 0
    # a GEMV right after: tensor memory was given back, shared memory configuration is intact
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    import __graft_entry__ as graft
    pkg = graft.load_package()
    K, N = 1024, 256
    w = torch.from_numpy(pkg.synth.make_weight(12, N, K, 5)).cuda()
    x = torch.from_numpy(pkg.synth.make_activation(40, K, 6)).cuda()
    x8, xm, xs = alloc_act(40, K)
    out = torch.zeros(40 * N, device="cuda")
    be.quant_gemv([gemv_seg(w=w, type=12, K=K, n_rows=N, x=x, x_stride=K, out=out, out_stride=N, x8=x8, xmeta=xm, xsumq=xs)], 40)
    be.synchronize()
    assert be.device_status() == 0
