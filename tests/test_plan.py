"""Forward plan (seg_plan mirror) and its replay as one CUDA graph: lowering decisions on CPU, and
on the GPU the whole chain model file -> loader -> device blob -> plan -> graph -> replay, every
call checked against the oracle on the values the GPU really consumed."""
import numpy as np
import pytest

import __graft_entry__ as graft

pkg = graft.load_package()
torch = pytest.importorskip("torch")
from sycl_infer_b200 import gguf as G  # noqa: E402
from sycl_infer_b200.backend import gemv_seg  # noqa: E402
from sycl_infer_b200.plan import PlanBuckets, SegPlan  # noqa: E402

H, QD, KD, FF, V, L = 512, 512, 128, 1024, 1024, 2
EPS = 1e-6


def _act(K, dev):
    return (torch.zeros(K, dtype=torch.int8, device=dev), torch.zeros(K // 16, dtype=torch.float32, device=dev),
            torch.zeros(K // 16, dtype=torch.int32, device=dev))


def build_plan(w, bufs, dev, tb=1):
    """w(name) -> uint8 weight tensor; bufs: activations and outputs of one token."""
    p = SegPlan()
    act_h, act_q, act_f = _act(H, dev), _act(QD, dev), _act(FF, dev)
    h = bufs["h0"]
    for i in range(L):
        qkv, o, gu, nxt = bufs[f"qkv{i}"], bufs[f"o{i}"], bufs[f"gu{i}"], bufs[f"h{i + 1}"]
        seg = lambda name, t, K, n, act, out, col, res=None: gemv_seg(  # noqa: E731
            w=w(f"blk.{i}.{name}.weight"), type=t, K=K, n_rows=n, out=out.view(-1)[col:], out_stride=out.shape[-1],
            residual=None if res is None else res.view(-1), alpha=1.0 / (3.0 * K ** 0.5), x8=act[0], xmeta=act[1], xsumq=act[2])
        p.begin_call(tb)
        p.add(seg("attn_q", 12, H, QD, act_h, qkv, 0))
        p.add(seg("attn_k", 12, H, KD, act_h, qkv, QD))
        p.add(seg("attn_v", 14, H, KD, act_h, qkv, QD + KD))
        p.set_xq(h)
        p.set_norm(w(f"blk.{i}.attn_norm.weight").view(torch.float32), EPS)
        p.begin_call(tb)
        p.add(seg("attn_output", 12, QD, H, act_q, o, 0, res=h))
        p.set_xq(bufs[f"attn{i}"])
        p.begin_call(tb)
        p.add(seg("ffn_gate", 12, H, FF, act_h, gu, 0))
        p.add(seg("ffn_up", 12, H, FF, act_h, gu, FF))
        p.set_xq(o)
        p.set_norm(w(f"blk.{i}.ffn_norm.weight").view(torch.float32), EPS)
        p.begin_call(tb)
        p.add(seg("ffn_down", 14, FF, H, act_f, nxt, 0, res=o))
        p.set_xq(gu, gu[:, FF:])
        h = nxt
    p.begin_call(tb)
    p.add(gemv_seg(w=w("output.weight"), type=14, K=H, n_rows=V, out=bufs["logits"].view(-1), out_stride=V, x8=act_h[0],
                   xmeta=act_h[1], xsumq=act_h[2]))
    p.set_xq(h)
    p.set_norm(w("output_norm.weight").view(torch.float32), EPS)
    p.set_argmax(bufs["tok"], bufs["tokv"])
    return p


def make_bufs(dev):
    f = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)  # noqa: E731
    b = {"h0": f(1, H), "logits": f(1, V), "tok": torch.zeros(1, dtype=torch.int32, device=dev), "tokv": f(1)}
    for i in range(L):
        b.update({f"qkv{i}": f(1, QD + 2 * KD), f"attn{i}": f(1, QD), f"o{i}": f(1, H), f"gu{i}": f(1, 2 * FF), f"h{i + 1}": f(1, H)})
    return b


def model_tensors():
    ts, seed = [], 700
    for i in range(L):
        for name, t, K, n in (("attn_q", 12, H, QD), ("attn_k", 12, H, KD), ("attn_v", 14, H, KD), ("attn_output", 12, QD, H),
                              ("ffn_gate", 12, H, FF), ("ffn_up", 12, H, FF), ("ffn_down", 14, FF, H)):
            ts.append((f"blk.{i}.{name}.weight", t, (K, n), pkg.synth.make_weight(t, n, K, seed).tobytes()))
            seed += 1
        for name in ("attn_norm", "ffn_norm"):
            ts.append((f"blk.{i}.{name}.weight", 0, (H,), (1.0 + 0.1 * pkg.synth.make_activation(1, H, seed)).astype(np.float32).tobytes()))
            seed += 1
    ts.append(("output_norm.weight", 0, (H,), (1.0 + 0.1 * pkg.synth.make_activation(1, H, seed)).astype(np.float32).tobytes()))
    ts.append(("output.weight", 14, (H, V), pkg.synth.make_weight(14, V, H, seed + 1).tobytes()))
    return ts


def test_lowering_pairs_gate_up_with_down():
    cpu = torch.device("cpu")
    ws = {}
    w = lambda name: ws.setdefault(name, torch.zeros(64, dtype=torch.uint8))  # noqa: E731
    p = build_plan(w, make_bufs(cpu), cpu).finalize()
    assert len(p.calls) == 4 * L + 1
    for i in range(L):
        qkv, o, gu, dn = p.calls[4 * i:4 * i + 4]
        assert gu.next_act is not None and dn.prequantized and not gu.prequantized and qkv.next_act is None
        assert gu.next_act[0].data_ptr() == dn.segs[0].x8.data_ptr()
        assert qkv.norm is not None and o.norm is None
    assert p.calls[-1].argmax is not None
    assert p.launches() == 4 * L + 1  # one launch per call: no quantizer launch anywhere
    # several tokens: nothing is paired, every call is quantizer + GEMM
    p3 = build_plan(w, make_bufs(cpu), cpu, tb=1)
    for c in p3.calls:
        c.tb, c.norm, c.argmax = 3, None, None
    p3.finalize()
    assert all(c.next_act is None and not c.prequantized for c in p3.calls) and p3.launches() == 2 * (4 * L + 1)


def test_validate_names_the_violation():
    cpu = torch.device("cpu")
    w = lambda name: torch.zeros(64, dtype=torch.uint8)  # noqa: E731
    p = build_plan(w, make_bufs(cpu), cpu)
    p.calls[2].segs[1].K = 768
    with pytest.raises(ValueError, match="call 2: segment 1"):
        p.finalize()
    p = build_plan(w, make_bufs(cpu), cpu)
    p.calls[1].x = None
    with pytest.raises(ValueError, match="call 1: no activation"):
        p.finalize()
    p = SegPlan()
    p.begin_call(1)
    with pytest.raises(ValueError, match="call 0: 0 segments"):
        p.finalize()


@pytest.mark.gpu
def test_model_file_to_replayed_token(tmp_path, orc):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    be = pkg.make_cuda_backend(0)
    ts = model_tensors()
    F = G.GgufFile(G.write_gguf(tmp_path / "m.gguf", {"general.architecture": (G.STR, "synthetic")}, ts, shards=2)[0])
    F.upload()
    dev = torch.device("cuda")
    bufs = make_bufs(dev)
    x0 = pkg.synth.make_activation(1, H, 801)
    attn = [pkg.synth.make_activation(1, QD, 802 + i) for i in range(L)]
    plan = build_plan(F.weight, bufs, dev).finalize()
    assert plan.launches() == 4 * L + 1
    st = torch.cuda.Stream()
    plan.record(be, st)
    for rnd in range(2):
        for b in bufs.values():
            b.zero_()
        bufs["h0"].copy_(torch.from_numpy(x0))
        for i in range(L):
            bufs[f"attn{i}"].copy_(torch.from_numpy(attn[i]))
        torch.cuda.synchronize()
        with torch.cuda.stream(st):
            plan.replay()
        st.synchronize()
        assert be.device_status() == 0
    got = {k: v.cpu().numpy() for k, v in bufs.items()}
    raw = {name: (t, dims, np.frombuffer(data, np.uint8)) for name, t, dims, data in ts}

    def check(name, act, out, residual=None):
        t, (K, n), wb = raw[name]
        alpha = 1.0 / (3.0 * K ** 0.5) if name != "output.weight" else 1.0
        ref = orc.gemm(t, wb, K, n, act, residual=None if residual is None else residual.copy(), alpha=alpha)
        ab = orc.gemm_abs(t, wb, K, n, act, alpha=alpha) + (0 if residual is None else np.abs(residual))
        err = float(np.max(np.abs(out.astype(np.float64) - ref) / ab))
        assert err <= 1e-5, f"{name}: {err}"

    nw = lambda name: raw[name][2].view(np.float32)  # noqa: E731
    h = got["h0"]
    for i in range(L):
        a = orc.xq(orc.rmsnorm(h, nw(f"blk.{i}.attn_norm.weight"), EPS, 16))
        check(f"blk.{i}.attn_q.weight", a, got[f"qkv{i}"][:, :QD])
        check(f"blk.{i}.attn_k.weight", a, got[f"qkv{i}"][:, QD:QD + KD])
        check(f"blk.{i}.attn_v.weight", a, got[f"qkv{i}"][:, QD + KD:])
        check(f"blk.{i}.attn_output.weight", orc.xq(attn[i]), got[f"o{i}"], residual=h)
        a2 = orc.xq(orc.rmsnorm(got[f"o{i}"], nw(f"blk.{i}.ffn_norm.weight"), EPS, 16))
        check(f"blk.{i}.ffn_gate.weight", a2, got[f"gu{i}"][:, :FF])
        check(f"blk.{i}.ffn_up.weight", a2, got[f"gu{i}"][:, FF:])
        q8, qm, qs = be_xq(be, got[f"gu{i}"][:, :FF], got[f"gu{i}"][:, FF:])  # the device quantizer on the same values
        af = orc.xq(got[f"gu{i}"][:, :FF], got[f"gu{i}"][:, FF:], 1)
        d = np.abs(q8.astype(np.int32) - af.x8.astype(np.int32))
        assert d.max() <= 1 and np.count_nonzero(d) <= 1e-4 * d.size + 1
        af.x8, af.xmeta, af.xsumq = q8, qm, qs
        check(f"blk.{i}.ffn_down.weight", af, got[f"h{i + 1}"], residual=got[f"o{i}"])
        h = got[f"h{i + 1}"]
    check("output.weight", orc.xq(orc.rmsnorm(h, nw("output_norm.weight"), EPS, 16)), got["logits"])
    assert int(got["tok"][0]) == int(got["logits"].argmax()) and float(got["tokv"][0]) == float(got["logits"].max())


def be_xq(be, x, up):
    from sycl_infer_b200.backend import alloc_act
    K = x.shape[1]
    x8, xm, xs = alloc_act(1, K)
    be.xq(torch.from_numpy(np.ascontiguousarray(x)).cuda(), torch.from_numpy(np.ascontiguousarray(up)).cuda(), K, K, x8, xm,
          xs, None, 1, K)
    be.synchronize()
    return x8.cpu().numpy(), xm.cpu().numpy(), xs.cpu().numpy()


@pytest.mark.gpu
def test_moe_call_inside_a_plan(orc):
    """A dense call and a routed-MoE call recorded into one graph: the replay gives what the same
    launches give when made directly."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from sycl_infer_b200.moe import MoeScratch, make_synthetic_moe, moe_call
    be = pkg.make_cuda_backend(0)
    dev = torch.device("cuda")
    n_tok, E, top_k, n_embd, n_ff = 4, 16, 2, 512, 256
    _, M = make_synthetic_moe(E, top_k, n_embd, n_ff, (12, 12, 12), seed=3, with_router=True)
    x = torch.from_numpy(pkg.synth.make_activation(n_tok, n_embd, 901)).cuda()
    wq = torch.from_numpy(pkg.synth.make_weight(12, n_embd, n_embd, 902)).cuda()

    def build(S, hbuf, out):
        p = SegPlan()
        p.begin_call(n_tok)
        a8 = torch.zeros(n_tok * n_embd, dtype=torch.int8, device=dev)
        am = torch.zeros(n_tok * n_embd // 16, dtype=torch.float32, device=dev)
        asq = torch.zeros(n_tok * n_embd // 16, dtype=torch.int32, device=dev)
        p.add(gemv_seg(w=wq, type=12, K=n_embd, n_rows=n_embd, out=hbuf.view(-1), out_stride=n_embd,
                       alpha=1.0 / (3.0 * n_embd ** 0.5), x8=a8, xmeta=am, xsumq=asq))
        p.set_xq(x)
        p.begin_moe_call(M, S, hbuf, out, n_tok)
        return p.finalize()

    S1, h1, o1 = MoeScratch(M, n_tok), torch.zeros(n_tok, n_embd, device=dev), torch.zeros(n_tok, n_embd, device=dev)
    plan = build(S1, h1, o1)
    assert plan.launches() == 2 + 7
    st = torch.cuda.Stream()
    plan.record(be, st)
    o1.zero_()
    with torch.cuda.stream(st):
        plan.replay()
    st.synchronize()
    S2, h2, o2 = MoeScratch(M, n_tok), torch.zeros(n_tok, n_embd, device=dev), torch.zeros(n_tok, n_embd, device=dev)
    build(S2, h2, o2).run(be)
    be.synchronize()
    assert be.device_status() == 0
    assert torch.equal(h1, h2) and torch.equal(o1, o2) and torch.equal(S1.ids, S2.ids)
    assert float(o1.abs().max()) > 0


# ---- decode buckets: a plan per row count ------------------------------------------------------------
def _two_call_plan(w_qkv, w_o, x, mid, out, act_h, act_q, tb):
    """q|k|v-like call (two segments) and an o-like call with a residual, tb rows each."""
    p = SegPlan()
    p.begin_call(tb)
    p.add(gemv_seg(w=w_qkv[0], type=12, K=H, n_rows=QD, out=mid.view(-1), out_stride=mid.shape[-1], x8=act_h[0],
                   xmeta=act_h[1], xsumq=act_h[2]))
    p.add(gemv_seg(w=w_qkv[1], type=14, K=H, n_rows=KD, out=mid.view(-1)[QD:], out_stride=mid.shape[-1], x8=act_h[0],
                   xmeta=act_h[1], xsumq=act_h[2]))
    p.set_xq(x[:tb])
    p.begin_call(tb)
    p.add(gemv_seg(w=w_o, type=12, K=QD, n_rows=H, out=out.view(-1), out_stride=H, residual=x.view(-1), x8=act_q[0],
                   xmeta=act_q[1], xsumq=act_q[2]))
    p.set_xq(mid[:tb, :QD])
    return p


class _CountingBackend:
    def __init__(self):
        self.calls = []

    def quant_gemv_ex(self, segs, tb, **kw):
        self.calls.append(("ex", tb, len(segs)))

    def quant_gemv(self, segs, tb):
        self.calls.append(("gemv", tb, len(segs)))


def test_buckets_build_one_plan_per_row_count():
    dev = "cpu"
    x, mid, out = torch.zeros(6, H), torch.zeros(6, QD + KD), torch.zeros(6, H)
    dummy = torch.zeros(16, dtype=torch.uint8)
    built = []

    def build(tb):
        built.append(tb)
        return _two_call_plan((dummy, dummy), dummy, x, mid, out, _act(H * 6, dev), _act(QD * 6, dev), tb)

    B = PlanBuckets(build, 6)
    assert [B.graph_rows(t) for t in range(1, 7)] == [True, True, False, True, False, True]
    be = _CountingBackend()
    B.run(be, 3)
    B.run(be, 3)
    B.run(be, 1)
    assert built == [3, 1]  # built on first use, once
    assert be.calls == [("gemv", 3, 2), ("gemv", 3, 1)] * 2 + [("ex", 1, 2), ("ex", 1, 1)]
    assert B.launches(3) == 4 and B.launches(1) == 2  # several rows take a quantizer launch per call
    with pytest.raises(ValueError):
        B.run(be, 7)
    with pytest.raises(ValueError):
        PlanBuckets(lambda tb: _two_call_plan((dummy, dummy), dummy, x, mid, out, _act(H, dev), _act(QD, dev), 1), 4).run(be, 2)
    assert sorted(PlanBuckets(build, 6).build_all().plans) == [1, 2, 3, 4, 5, 6]


@pytest.mark.gpu
def test_buckets_graph_and_direct_replay_agree_with_plain_calls():
    """Row counts 1..5 through the buckets (graphs for 1, 2, 4 and 5 = max, direct replay for 3) against
    the same calls issued one by one: identical outputs."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    be = pkg.make_cuda_backend(0)
    dev, R = "cuda", 5
    w_qkv = (torch.from_numpy(pkg.synth.make_weight(12, QD, H, 1)).cuda(), torch.from_numpy(pkg.synth.make_weight(14, KD, H, 2)).cuda())
    w_o = torch.from_numpy(pkg.synth.make_weight(12, H, QD, 3)).cuda()
    x = torch.from_numpy(pkg.synth.make_activation(R, H, 4)).cuda()
    mid, out = torch.zeros(R, QD + KD, device=dev), torch.zeros(R, H, device=dev)
    from sycl_infer_b200.backend import alloc_act
    acts = {}

    def build(tb):
        acts[tb] = (alloc_act(tb, H), alloc_act(tb, QD))
        return _two_call_plan(w_qkv, w_o, x, mid, out, acts[tb][0], acts[tb][1], tb)

    B = PlanBuckets(build, R)
    st = torch.cuda.Stream()
    for n in (1, 2, 3, 4, 5, 3, 1):
        mid.zero_()
        out.zero_()
        torch.cuda.synchronize()
        p = B.run(be, n, st)
        st.synchronize()
        assert (p.graph is not None) == (n != 3)
        got_mid, got_out = mid.clone(), out.clone()
        mid.zero_()
        out.zero_()
        _two_call_plan(w_qkv, w_o, x, mid, out, acts[n][0], acts[n][1], n).finalize().run(be)
        be.synchronize()
        assert be.device_status() == 0
        assert torch.equal(got_mid, mid) and torch.equal(got_out, out)
        assert torch.count_nonzero(out[:n]).item() > 0 and torch.count_nonzero(out[n:]).item() == 0
