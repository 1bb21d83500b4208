"""Row-sharded dense layer on 2 and 4 GPUs, both exchange forms, checked call by call against the
oracle: after every call the oracle recomputes that call on the full (unsharded) weight from the
activation the GPUs really consumed (their own gathered output of the previous call), and every
output value must lie within 1e-5 of its sum of |terms|.  A wrong, stale or missing row from any
rank fails this bound.  Skipped on a single-GPU box; the host logic is covered on CPU by
test_sharding_cpu.py."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

KW = dict(hidden=1024, n_head=8, n_kv=2, head_dim=128, n_ff=2048)
SEED = 9
TOL = 1e-5


def _worker(rank, world, port, TB, ret, fused):
    import sys
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import __graft_entry__ as graft
    pkg = graft.load_package()
    from sycl_infer_b200.layer import DenseLayer
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        be = pkg.make_cuda_backend(rank)
        x = torch.from_numpy(pkg.synth.make_activation(TB, KW["hidden"], 5)).cuda()
        attn = torch.from_numpy(pkg.synth.make_activation(TB, KW["n_head"] * KW["head_dim"], 6)).cuda()
        arena = None
        if fused:
            from sycl_infer_b200.sharding import PeerArena
            arena = PeerArena(TB * 16384, rank, world)
        ly = DenseLayer(be, "Q4_K_M", seed=SEED, TB=TB, rank=rank, world=world, arena=arena, **KW)
        ly.attn.copy_(attn)
        out = ly.out if fused else torch.zeros(TB, KW["hidden"], device="cuda")
        for _ in range(3):  # several steps: the flag sequence and buffer reuse across steps
            ly.forward(x, out)
        torch.cuda.synchronize()
        dist.barrier()
        assert be.device_status() == 0
        ret[rank] = dict(out=out.cpu().numpy(), qkv=ly.qkv.cpu().numpy(), o=ly.o_out.cpu().numpy(), gu=ly.gu.cpu().numpy(),
                         act_f=tuple(t.cpu().numpy() for t in ly.act_f))
    finally:
        dist.destroy_process_group()


def _check_rank(orc, pkg, r, TB):
    """Every call of the layer against the oracle on the full weights, from the GPU's own inputs."""
    shapes = {n: (t, rows, K) for n, t, rows, K in pkg.synth.dense_layer_shapes("Q4_K_M", **KW)}
    w = {n: pkg.synth.make_weight(t, rows, K, SEED * 16 + i) for i, (n, (t, rows, K)) in enumerate(shapes.items())}
    x, attn = pkg.synth.make_activation(TB, KW["hidden"], 5), pkg.synth.make_activation(TB, 1024, 6)

    def call(name, act, got, residual=None):
        t, rows, K = shapes[name]
        alpha = 1.0 / (3.0 * K ** 0.5)
        ref = orc.gemm(t, w[name], K, rows, act, residual=None if residual is None else residual.copy(), alpha=alpha)
        ab = orc.gemm_abs(t, w[name], K, rows, act, alpha=alpha) + (0 if residual is None else np.abs(residual))
        err = float(np.max(np.abs(got.astype(np.float64) - ref) / ab))
        assert err <= TOL, f"{name}: {err}"

    qd, kd, nf = 1024, 256, KW["n_ff"]
    ax = orc.xq(x, None, TB)
    call("q", ax, r["qkv"][:, :qd])
    call("k", ax, r["qkv"][:, qd:qd + kd])
    call("v", ax, r["qkv"][:, qd + kd:])
    call("o", orc.xq(attn, None, TB), r["o"])
    ao = orc.xq(r["o"], None, TB)
    call("gate", ao, r["gu"][:, :nf])
    call("up", ao, r["gu"][:, nf:])
    # down consumes quantize(silu(gate)*up): the GPU's own codes (they may differ from the host's
    # expf at rounding ties only), then the oracle GEMV on exactly those
    host = orc.xq(r["gu"][:, :nf], r["gu"][:, nf:], TB)
    d = np.abs(r["act_f"][0].astype(np.int32) - host.x8.astype(np.int32))
    assert d.max() <= 1 and np.count_nonzero(d) <= 1e-4 * d.size + 1
    host.x8, host.xmeta, host.xsumq = r["act_f"]
    call("down", host, r["out"], residual=x)


@pytest.mark.parametrize("fused", [False, True], ids=["nccl_allgather", "peer_store"])
@pytest.mark.parametrize("TB", [1, 3, 8])
@pytest.mark.parametrize("world", [2, 4])
def test_row_sharded_layer_every_call_against_oracle(orc, pkg, world, TB, fused):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, TB, ret, fused), nprocs=world, join=True)
    for rank in range(world):
        _check_rank(orc, pkg, ret[rank], TB)
    for rank in range(1, world):  # all ranks hold the same gathered buffers, bit for bit
        for k in ("qkv", "o", "gu", "out"):
            assert np.array_equal(ret[rank][k], ret[0][k]), k


def test_peer_barrier_times_out_instead_of_hanging(be):
    """A peer that never signals: the bounded wait gives up after about a second and reports
    through the device status word; the context stays usable.  The 'peer' is a second flag
    array on this same GPU that nothing ever writes to this rank's slot of."""
    import ctypes as C
    import time
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    other = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags = (C.c_void_p * 2)(mine.data_ptr(), other.data_ptr())
    t0 = time.time()
    be.peer_barrier(flags, 2, 0, 1)
    be.synchronize()
    assert time.time() - t0 < 10
    assert int(other[0]) == 1          # this rank's signal landed at the peer
    assert be.device_status() == 4     # B200Q_ETIMEOUT, and the word is cleared by the read
    assert be.device_status() == 0
    mine[1] = 1                        # the peer "arrives": the same barrier now passes
    be.peer_barrier(flags, 2, 0, 1)
    be.synchronize()
    assert be.device_status() == 0


def test_in_kernel_peer_wait_times_out_and_signal_lands(be, orc, pkg):
    """The exchange folded into the GEMV launch, on one GPU with a stand-in peer array: the
    launch signals the 'peer' when its last CTA is done, and a launch told to wait for a signal
    that never comes gives up after about a second with B200Q_ETIMEOUT instead of hanging."""
    import ctypes as C
    import time
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    from sycl_infer_b200.capi import Peers
    t, K, N = 12, 1024, 300
    w = torch.from_numpy(pkg.synth.make_weight(t, N, K, 77)).cuda()
    x = torch.from_numpy(pkg.synth.make_activation(1, K, 78)).cuda()
    x8, xm, xs = alloc_act(1, K)
    out = torch.zeros(N, dtype=torch.float32, device="cuda")
    seg = gemv_seg(w=w, type=t, K=K, n_rows=N, x=x, x_stride=K, out=out, out_stride=N, x8=x8, xmeta=xm, xsumq=xs)
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    other = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags = (C.c_void_p * 2)(mine.data_ptr(), other.data_ptr())
    peers = Peers()  # no peer outputs: only the flag protocol is exercised here
    be.quant_gemv_ex([seg], 1, peers=peers, sync=(flags, 2, 0), wait=True, signal=True)
    be.synchronize()
    assert be.device_status() == 0          # nothing signalled yet, nothing expected yet
    assert int(other[0]) == 1 and int(mine[32]) == 1 and int(mine[33]) == 0
    t0 = time.time()
    be.quant_gemv_ex([seg], 1, peers=peers, sync=(flags, 2, 0), wait=True, signal=True)
    be.synchronize()
    assert time.time() - t0 < 10
    assert be.device_status() == 4          # the peer never signalled call 1
    assert be.device_status() == 0
    mine[1] = 2                             # the peer catches up
    be.quant_gemv_ex([seg], 1, peers=peers, sync=(flags, 2, 0), wait=True, signal=True)
    be.synchronize()
    assert be.device_status() == 0 and int(other[0]) == 3
    a = orc.xq(x.cpu().numpy())
    wn = w.cpu().numpy()
    ref, ab = orc.gemm(t, wn, K, N, a), orc.gemm_abs(t, wn, K, N, a)
    assert float(np.max(np.abs(out.cpu().numpy() - ref[0]) / ab[0])) <= TOL
