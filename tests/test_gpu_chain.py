"""Dependent single-token calls in one launch (b200q_quant_gemv_chain): o -> gate|up -> down of a
dense layer.  The chained launch must give, bit for bit, what the same calls give as separate
launches (same per-row arithmetic, only the launch structure differs), and every call is
checked against the oracle on the activation the GPU really consumed."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL = 1e-5
SMALL = dict(hidden=1024, n_head=8, n_kv=2, head_dim=128, n_ff=2048)
FULL = dict(hidden=5120, n_head=40, n_kv=8, head_dim=128, n_ff=17408)


def _run(pkg, be, mix, kw, chain, steps, seed=21):
    from sycl_infer_b200.layer import DenseLayer
    ly = DenseLayer(be, mix, seed=seed, TB=1, **kw)
    ly.chain = chain  # the layer's default is separate launches
    x = torch.from_numpy(pkg.synth.make_activation(1, kw["hidden"], 31)).cuda()
    ly.attn.copy_(torch.from_numpy(pkg.synth.make_activation(1, kw["n_head"] * kw["head_dim"], 32)).cuda())
    out = torch.zeros(1, kw["hidden"], device="cuda")
    for _ in range(steps):
        for buf in (ly.qkv, ly.o_out, ly.gu, out, *ly.act_f):
            buf.zero_()
        ly.forward(x, out)
        be.synchronize()
        assert be.device_status() == 0
    got = dict(qkv=ly.qkv, o=ly.o_out, gu=ly.gu, out=out, f8=ly.act_f[0], fm=ly.act_f[1], fs=ly.act_f[2])
    return ly, {k: v.cpu().numpy().copy() for k, v in got.items()}


@pytest.mark.parametrize("mix,kw", [("Q4_K_M", SMALL), ("Q5_K", SMALL), ("IQ4_XS", SMALL), ("Q4_K_M", FULL)],
                         ids=["q4km_small", "q5k_small", "iq4xs_small", "q4km_config1"])
def test_chain_equals_separate_launches_and_oracle(be, orc, pkg, mix, kw):
    ly, sep = _run(pkg, be, mix, kw, chain=False, steps=1)
    assert ly.launches_per_step() == 4
    ly2, ch = _run(pkg, be, mix, kw, chain=True, steps=3)  # several launches: the device-side count returns to zero
    assert ly2.launches_per_step() == 2
    for k in sep:
        assert np.array_equal(sep[k].view(np.uint8), ch[k].view(np.uint8)), k
    # the chained results against the oracle, call by call, from the GPU's own intermediate values
    shapes = {n: (t, rows, K) for n, t, rows, K in pkg.synth.dense_layer_shapes(mix, **kw)}
    w = {n: pkg.synth.make_weight(t, rows, K, 21 * 16 + i) for i, (n, (t, rows, K)) in enumerate(shapes.items())}
    x = pkg.synth.make_activation(1, kw["hidden"], 31)
    attn = pkg.synth.make_activation(1, kw["n_head"] * kw["head_dim"], 32)
    nf = kw["n_ff"]

    def call(name, act, got, residual=None, rows=None):
        t, n, K = shapes[name]
        rows = rows or slice(0, n)
        rb = pkg.synth.row_bytes(t, K)
        sub = w[name][rows.start * rb:rows.stop * rb]
        alpha = 1.0 / (3.0 * K ** 0.5)
        m = rows.stop - rows.start
        res = None if residual is None else residual[:, rows].copy()
        ref = orc.gemm(t, sub, K, m, act, residual=res, alpha=alpha)
        ab = orc.gemm_abs(t, sub, K, m, act, alpha=alpha) + (0 if res is None else np.abs(res))
        err = float(np.max(np.abs(got[:, rows].astype(np.float64) - ref) / ab))
        assert err <= TOL, f"{name}: {err}"

    tail = None if nf <= 2048 else slice(nf - 400, nf)  # the oracle is a scalar port: sample the big matrices
    call("o", orc.xq(attn), ch["o"])
    ao = orc.xq(ch["o"])
    call("gate", ao, ch["gu"][:, :nf], rows=tail)
    call("up", ao, ch["gu"][:, nf:], rows=tail)
    host = orc.xq(ch["gu"][:, :nf], ch["gu"][:, nf:], 1)
    d = np.abs(ch["f8"].astype(np.int32) - host.x8.astype(np.int32))
    assert d.max() <= 1 and np.count_nonzero(d) <= 1e-4 * d.size + 1
    host.x8, host.xmeta, host.xsumq = ch["f8"], ch["fm"], ch["fs"]
    call("down", host, ch["out"], residual=x, rows=None if nf <= 2048 else slice(0, 256))


def test_chain_of_two_and_of_four(be, orc, pkg):
    """Chains of other lengths: y1 = W1 x; y2 = W2 y1 (+ y3 = W3 y2, y4 = W4 y3), every call
    quantizing its input inside the launch, against the same calls made one by one."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    dims = [1024, 768, 2048, 512, 1280]  # K of call i = dims[i], rows = dims[i + 1]
    types = [12, 14, 13, 8]
    x = torch.from_numpy(pkg.synth.make_activation(1, dims[0], 41)).cuda()
    ws = [torch.from_numpy(pkg.synth.make_weight(t, dims[i + 1], dims[i], 50 + i)).cuda() for i, t in enumerate(types)]

    def build(n):
        bufs = [x] + [torch.zeros(1, dims[i + 1], device="cuda") for i in range(n)]
        acts = [alloc_act(1, dims[i]) for i in range(n)]
        calls = []
        for i in range(n):
            K = dims[i]
            calls.append(([gemv_seg(w=ws[i], type=types[i], K=K, n_rows=dims[i + 1], x=bufs[i], x_stride=K,
                                    out=bufs[i + 1].view(-1), out_stride=dims[i + 1], alpha=1.0 / (3.0 * K ** 0.5),
                                    x8=acts[i][0], xmeta=acts[i][1], xsumq=acts[i][2])], False, None))
        return bufs, calls

    for n in (2, 4):
        b1, c1 = build(n)
        for segs, _, _ in c1:
            be.quant_gemv_ex(segs, 1)
        b2, c2 = build(n)
        for _ in range(2):
            be.quant_gemv_chain(c2)
        be.synchronize()
        assert be.device_status() == 0
        for i in range(1, n + 1):
            assert torch.equal(b1[i], b2[i]), (n, i)
        a = orc.xq(b2[n - 1].cpu().numpy())
        wn = ws[n - 1].cpu().numpy()
        alpha = 1.0 / (3.0 * dims[n - 1] ** 0.5)
        ref = orc.gemm(types[n - 1], wn, dims[n - 1], dims[n], a, alpha=alpha)
        ab = orc.gemm_abs(types[n - 1], wn, dims[n - 1], dims[n], a, alpha=alpha)
        assert float(np.max(np.abs(b2[n].cpu().numpy() - ref) / ab)) <= TOL


def test_chain_falls_back_to_separate_launches(be, pkg):
    """A chain the fused form cannot take (five calls; a K the single-token kernel does not
    serve) still runs, launch by launch, with the same results."""
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    K = 1024
    x = torch.from_numpy(pkg.synth.make_activation(1, K, 61)).cuda()
    w = torch.from_numpy(pkg.synth.make_weight(12, K, K, 62)).cuda()

    def build(n):
        bufs = [x] + [torch.zeros(1, K, device="cuda") for _ in range(n)]
        acts = [alloc_act(1, K) for _ in range(n)]
        return bufs, [([gemv_seg(w=w, type=12, K=K, n_rows=K, x=bufs[i], x_stride=K, out=bufs[i + 1].view(-1),
                                 out_stride=K, alpha=1.0 / (3.0 * K ** 0.5), x8=acts[i][0], xmeta=acts[i][1],
                                 xsumq=acts[i][2])], False, None) for i in range(n)]

    b1, c1 = build(5)
    for segs, _, _ in c1:
        be.quant_gemv_ex(segs, 1)
    b2, c2 = build(5)
    be.quant_gemv_chain(c2)
    be.synchronize()
    assert be.device_status() == 0
    assert torch.equal(b1[5], b2[5])
