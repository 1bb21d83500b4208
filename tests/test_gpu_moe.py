"""Routed-MoE parity through the C ABI (benchmark configuration 3 and small cases).

Stage by stage against the oracle, because each stage re-quantizes the previous one's output:
router ids exact and weights within 1e-6 (tests/backend/cpu/kernels/test_cpu_moe_qsa_units.cpp:59-105
of the reference); gate|up within 1e-5 of the sum of |terms|; down and reduce are checked on the
intermediate the GPU itself produced (the oracle is run on those bytes), so a one-ulp difference
in h cannot masquerade as a down-projection error.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
TOL = 1e-5
G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_vectors.npz"))


def test_router_golden_from_reference(be):
    from sycl_infer_b200.moe import moe_router_launch
    x, gate = torch.from_numpy(G["moe_x"]).cuda(), torch.from_numpy(G["moe_gate_inp"]).cuda()
    n_tok, n_embd = x.shape
    E, top_k = gate.shape[0], 2
    logits = torch.zeros(n_tok, E, device="cuda")
    ids = torch.zeros(n_tok, top_k, dtype=torch.int32, device="cuda")
    wts = torch.zeros(n_tok, top_k, device="cuda")
    moe_router_launch(be, gate, 0, x, n_embd, n_tok, n_embd, E, top_k, logits, ids, wts)
    be.synchronize()
    assert np.array_equal(ids.cpu().numpy(), G["moe_ids"])
    assert np.max(np.abs(wts.cpu().numpy() - G["moe_wts"])) <= 1e-6
    assert np.max(np.abs(logits.cpu().numpy() - G["moe_logits"])) <= 1e-6


@pytest.mark.parametrize("n_tok,E,top_k", [(1, 8, 2), (16, 256, 8), (5, 64, 6)])
def test_router_from_logits(be, orc, pkg, n_tok, E, top_k):
    from sycl_infer_b200.moe import moe_router_launch
    lg = pkg.synth.make_router_logits(n_tok, E, 77 + E)
    lg[0, :4] = lg[0, 0]  # ties go to the lower index
    p, ids_o, wts_o = orc.moe_route_logits(lg, top_k)
    logits = torch.from_numpy(lg.copy()).cuda()
    ids = torch.zeros(n_tok, top_k, dtype=torch.int32, device="cuda")
    wts = torch.zeros(n_tok, top_k, device="cuda")
    moe_router_launch(be, None, 0, None, 0, n_tok, 0, E, top_k, logits, ids, wts)
    be.synchronize()
    assert np.array_equal(ids.cpu().numpy(), ids_o)
    assert np.max(np.abs(wts.cpu().numpy() - wts_o)) <= 1e-6
    assert np.max(np.abs(logits.cpu().numpy() - p)) <= 1e-7


def _run_moe(be, orc, pkg, E, top_k, n_embd, n_ff, n_tok, types, seed, fused_hq=False):
    from sycl_infer_b200.moe import MoeScratch, make_synthetic_moe, moe_call
    host, dev = make_synthetic_moe(E, top_k, n_embd, n_ff, types, seed)
    x = pkg.synth.make_activation(n_tok, n_embd, seed + 50)
    lg = pkg.synth.make_router_logits(n_tok, E, seed + 51)
    base = pkg.synth.make_activation(n_tok, n_embd, seed + 52)
    S = MoeScratch(dev, n_tok)
    S.logits.copy_(torch.from_numpy(lg))
    out = torch.from_numpy(base.copy()).cuda()
    moe_call(be, dev, S, torch.from_numpy(x).cuda(), n_tok, out, logits_given=True, fused_hq=fused_hq)
    be.synchronize()
    assert be.device_status() == 0
    # router
    _, ids_o, wts_o = orc.moe_route_logits(lg, top_k)
    ids = S.ids.cpu().numpy()
    assert np.array_equal(ids, ids_o)
    # CSR: every pair listed once under its expert, in increasing pair order
    off, pair = S.off.cpu().numpy(), S.pair.cpu().numpy()
    flat = ids.reshape(-1)
    assert off[0] == 0 and off[-1] == n_tok * top_k
    for e in range(E):
        assert list(pair[off[e]:off[e + 1]]) == list(np.nonzero(flat == e)[0])
    assert int(S.n_active.cpu()[0]) == len(np.unique(flat))
    # gate|up: h vs the oracle's h (same activation codes on both sides)
    a = orc.xq(x, None, n_tok)
    assert np.array_equal(S.xq[0].cpu().numpy(), a.x8)
    gw, uw, dw = host.gate_exps.numpy(), host.up_exps.numpy(), host.down_exps.numpy()
    h_o, acc_o = orc.moe_experts(gw, uw, dw, types, n_embd, n_ff, x, ids_o)
    h = S.h.cpu().numpy()
    scale = np.max(np.abs(h_o)) + 1e-30
    assert np.max(np.abs(h - h_o)) <= 2e-5 * scale  # product of two dots of ~1e-7 relative error each
    # down on the GPU's own h: oracle quantizes those bytes and runs the down rows
    rb = pkg.synth.row_bytes(types[2], n_ff) * n_embd
    acc = S.acc.cpu().numpy()
    hq = orc.xq(h, None, n_tok * top_k)
    assert np.array_equal(S.hq[0].cpu().numpy(), hq.x8)
    for p in range(0, n_tok * top_k, max(1, n_tok * top_k // 12)):  # a dozen pairs, full rows
        e = flat[p]
        one = orc.xq(h[p])
        ref = orc.gemm(types[2], dw[e * rb:(e + 1) * rb], n_ff, n_embd, one)[0]
        ab = orc.gemm_abs(types[2], dw[e * rb:(e + 1) * rb], n_ff, n_embd, one)[0]
        assert np.max(np.abs(acc[p] - ref) / np.maximum(ab, 1e-30)) <= TOL
    # reduce on the GPU's acc
    ref_out = orc.moe_reduce(acc, S.wts.cpu().numpy(), base)
    got = out.cpu().numpy()
    assert np.max(np.abs(got - ref_out)) <= 1e-6 * max(1.0, np.max(np.abs(ref_out)))
    # end to end against the all-oracle pipeline (loose: h is re-quantized on both sides)
    full = orc.moe_reduce(acc_o, wts_o, base)
    assert np.max(np.abs(got - full)) <= 2e-2 * np.max(np.abs(full))
    return len(np.unique(flat))


@pytest.mark.parametrize("types", [(12, 12, 12), (12, 12, 8), (13, 13, 14), (23, 23, 23)])
def test_moe_small(be, orc, pkg, types):
    _run_moe(be, orc, pkg, E=8, top_k=2, n_embd=512, n_ff=256, n_tok=5, types=types, seed=3)


def test_moe_many_tokens_per_expert(be, orc, pkg):
    """More than four routed tokens per expert on average: the grouped tensor-core expert kernel
    (10 tokens per expert: 16-token tiles, the busier experts take two)."""
    _run_moe(be, orc, pkg, E=8, top_k=2, n_embd=512, n_ff=256, n_tok=40, types=(12, 12, 12), seed=7)


@pytest.mark.parametrize("n_tok,types", [(40, (13, 13, 14)), (100, (12, 12, 12)), (100, (14, 14, 8)), (100, (23, 23, 13)),
                                         (300, (12, 12, 14)), (300, (8, 8, 23))])
def test_moe_grouped_tensor_core_tiles(be, orc, pkg, n_tok, types):
    """Prefill-sized calls on the grouped tcgen05 kernel: 16-, 32- and 64-token tiles (10, 25 and 75
    routed tokens per expert on average), every block format on either side."""
    _run_moe(be, orc, pkg, E=8, top_k=2, n_embd=512, n_ff=256, n_tok=n_tok, types=types, seed=31 + n_tok)


def test_moe_many_tokens_mixed_gate_up_types(be, orc, pkg):
    """gate and up planes of different types with many tokens per expert: the grouped kernel pairs
    gate and up rows of one format only, this shape stays on the warp-per-row kernel."""
    _run_moe(be, orc, pkg, E=8, top_k=2, n_embd=512, n_ff=256, n_tok=40, types=(12, 14, 12), seed=8)


def test_moe_config3_prefill_512_tokens(be, orc, pkg):
    """Configuration 3 with 512 tokens (16 routed tokens per expert on average)."""
    n = _run_moe(be, orc, pkg, E=256, top_k=8, n_embd=2048, n_ff=512, n_tok=512, types=(12, 12, 12), seed=0xC3)
    assert n >= 250


@pytest.mark.parametrize("types", [(12, 14, 12), (14, 14, 14)])
def test_moe_mixed_gate_up_types(be, orc, pkg, types):
    """gate and up planes of different types (separate row passes), and Q6_K planes whose rows are
    16-byte multiples only when K is a multiple of 2048."""
    _run_moe(be, orc, pkg, E=8, top_k=2, n_embd=2048, n_ff=256, n_tok=3, types=types, seed=9)


@pytest.mark.parametrize("cfg", [dict(E=8, top_k=2, n_embd=512, n_ff=256, n_tok=5, types=(12, 12, 12), seed=3),
                                 dict(E=8, top_k=2, n_embd=512, n_ff=256, n_tok=5, types=(13, 13, 8), seed=4),
                                 dict(E=16, top_k=4, n_embd=256, n_ff=256, n_tok=1, types=(12, 12, 12), seed=5),
                                 dict(E=8, top_k=2, n_embd=2048, n_ff=256, n_tok=3, types=(12, 14, 12), seed=9),
                                 dict(E=8, top_k=2, n_embd=512, n_ff=256, n_tok=40, types=(12, 12, 12), seed=7),
                                 dict(E=256, top_k=8, n_embd=2048, n_ff=512, n_tok=16, types=(12, 12, 12), seed=0xB3)],
                         ids=["q4k", "q5k_q8", "one_token", "mixed_types_two_launches", "many_tokens_two_launches", "config3"])
def test_moe_gate_up_also_quantizes_h(be, orc, pkg, cfg):
    """b200q_moe_gate_up_q: h and its quantization from one call - inside the expert kernel's
    epilogue where the pinned kernel serves the shape, else as the two launches.  The harness holds
    the emitted codes to the host quantizer of the SAME h, bit for bit, and runs down on them."""
    _run_moe(be, orc, pkg, fused_hq=True, **cfg)


def test_moe_gate_up_q_rejects_ragged_ffn(be, pkg):
    """n_ff_exp not a multiple of 32: no whole quantization groups, EINVAL."""
    from sycl_infer_b200.capi import B200QError
    from sycl_infer_b200.moe import MoeScratch, make_synthetic_moe, moe_grp_gate_up_q_launch
    host, dev = make_synthetic_moe(4, 2, 256, 256, (12, 12, 12), 1)
    S = MoeScratch(dev, 2)
    import dataclasses
    dev = dataclasses.replace(dev, n_ff_exp=250)
    with pytest.raises(B200QError) as ei:
        moe_grp_gate_up_q_launch(be, dev, S.off, S.pair, S.active, S.n_active, 4, *S.xq, 2, S.h, 256, *S.hq)
    assert ei.value.code == 1


def test_moe_many_pairs_per_share(be, orc, pkg):
    """600 routed pairs on short expert planes: a CTA's share of the expert kernel spans several
    pairs (its down launch gives every CTA four or five whole pairs), each with its own activation."""
    n = _run_moe(be, orc, pkg, E=256, top_k=4, n_embd=256, n_ff=256, n_tok=150, types=(12, 12, 12), seed=11)
    assert n >= 150


def test_moe_single_token(be, orc, pkg):
    _run_moe(be, orc, pkg, E=16, top_k=4, n_embd=256, n_ff=256, n_tok=1, types=(12, 12, 12), seed=5)


def test_moe_config3_full_size(be, orc, pkg):
    """256 experts, top-8, hidden 2048, expert FFN 512, Q4_K, 16 tokens."""
    n = _run_moe(be, orc, pkg, E=256, top_k=8, n_embd=2048, n_ff=512, n_tok=16, types=(12, 12, 12), seed=0xB3)
    assert 60 <= n <= 128


@pytest.mark.parametrize("n_tok,E,n_embd", [(100, 40, 520), (300, 40, 520), (256, 256, 2048), (257, 33, 96)])
def test_router_logits_many_tokens(be, orc, pkg, n_tok, E, n_embd):
    """256 tokens and more take the tiled logits kernel (ragged token, expert and K tiles included),
    fewer the kernel of two experts per CTA in several passes of 16 tokens: logits within 1e-6 of the
    oracle's fp64 sums, same ids."""
    from sycl_infer_b200.moe import moe_router_launch
    rng = np.random.default_rng(n_tok + E)
    x = pkg.synth.make_activation(n_tok, n_embd, 900 + n_tok)
    gate = (rng.standard_normal((E, n_embd)) / np.sqrt(n_embd)).astype(np.float32)
    top_k = 4
    lg_o, ids_o, wts_o = orc.moe_route(x, gate, top_k)
    logits = torch.zeros(n_tok, E, device="cuda")
    ids = torch.zeros(n_tok, top_k, dtype=torch.int32, device="cuda")
    wts = torch.zeros(n_tok, top_k, device="cuda")
    moe_router_launch(be, torch.from_numpy(gate).cuda(), 0, torch.from_numpy(x).cuda(), n_embd, n_tok, n_embd, E, top_k,
                      logits, ids, wts)
    be.synchronize()
    assert be.device_status() == 0
    assert np.max(np.abs(logits.cpu().numpy() - lg_o)) <= 1e-6 * max(1.0, np.max(np.abs(lg_o)))
    assert np.array_equal(ids.cpu().numpy(), ids_o)
    assert np.max(np.abs(wts.cpu().numpy() - wts_o)) <= 1e-6


@pytest.mark.parametrize("n_tok,E,top_k", [(16, 256, 8), (3, 32, 4), (600, 64, 4), (2100, 8, 4), (2048, 512, 4),
                                           (1024, 2048, 4)])
def test_csr_separate_and_fused_agree(be, pkg, n_tok, E, top_k):
    """Router + CSR as two entry points and as the fused one (the router's last CTA builds the
    lists): identical ids, offsets, pair lists and active experts; the lists are checked against a
    host construction as well."""
    from sycl_infer_b200.moe import moe_csr_launch, moe_router_csr_launch, moe_router_launch
    lg = pkg.synth.make_router_logits(n_tok, E, 123 + E)
    i32 = dict(dtype=torch.int32, device="cuda")
    res = []
    for fused in (False, True):
        logits = torch.from_numpy(lg.copy()).cuda()
        ids, wts = torch.zeros(n_tok, top_k, **i32), torch.zeros(n_tok, top_k, device="cuda")
        off, pair = torch.zeros(E + 1, **i32), torch.zeros(n_tok * top_k, **i32)
        active, n_active = torch.zeros(E, **i32), torch.zeros(1, **i32)
        for rep in range(2):  # twice: the fused form's completion counter must return to zero
            if fused:
                moe_router_csr_launch(be, None, 0, None, 0, n_tok, 0, E, top_k, logits, ids, wts, off, pair, active, n_active)
            else:
                moe_router_launch(be, None, 0, None, 0, n_tok, 0, E, top_k, logits, ids, wts)
                moe_csr_launch(be, ids, n_tok * top_k, E, off, pair, active, n_active)
            be.synchronize()
            if rep == 0:
                logits.copy_(torch.from_numpy(lg))  # the router leaves probabilities in its logits scratch
        na = int(n_active.cpu()[0])
        res.append((ids.cpu().numpy(), off.cpu().numpy(), pair.cpu().numpy(), active.cpu().numpy()[:na], na))
    for a, b in zip(res[0], res[1]):
        assert np.array_equal(a, b)
    ids, off, pair, active, na = res[0]
    flat = ids.reshape(-1)
    assert na == len(np.unique(flat)) and np.array_equal(active, np.unique(flat))
    for e in range(E):
        assert np.array_equal(pair[off[e]:off[e + 1]], np.nonzero(flat == e)[0])


def test_pairs_with_invalid_expert_ids_are_left_out(be, pkg):
    """Expert ids outside 0..n_expert-1 (a caller's own router may emit -1 for "no expert"): the CSR
    builder leaves those pairs out of every list, the expert kernels never touch their rows of h and
    acc, and every other pair's rows are bit-identical to a run on the same lists with the bad pairs
    routed to a valid expert."""
    from sycl_infer_b200.moe import (MoeScratch, make_synthetic_moe, moe_actq_launch, moe_csr_launch,
                                     moe_grp_down_launch, moe_grp_gate_up_launch)
    E, top_k, n_embd, n_ff, n_tok = 8, 2, 512, 256, 6
    _, dev = make_synthetic_moe(E, top_k, n_embd, n_ff, (12, 12, 14), 21)
    x = torch.from_numpy(pkg.synth.make_activation(n_tok, n_embd, 77)).cuda()
    n_pairs, n_act_max = n_tok * top_k, min(E, n_tok * top_k)
    good = np.array([[0, 3], [3, 5], [7, 0], [2, 3], [5, 6], [1, 7]], np.int32)
    bad = good.copy()
    bad[1, 0], bad[3, 1], bad[5, 0] = -1, E, 1 << 20
    res = []
    for ids in (good, bad):
        S = MoeScratch(dev, n_tok)
        S.ids.copy_(torch.from_numpy(ids))
        S.h.fill_(7.0)
        S.acc.fill_(7.0)
        moe_actq_launch(be, x, n_embd, n_tok, n_embd, *S.xq)
        moe_csr_launch(be, S.ids, n_pairs, E, S.off, S.pair, S.active, S.n_active)
        moe_grp_gate_up_launch(be, dev, S.off, S.pair, S.active, S.n_active, n_act_max, *S.xq, n_tok, S.h, n_ff)
        moe_actq_launch(be, S.h, n_ff, n_pairs, n_ff, *S.hq)
        moe_grp_down_launch(be, dev, S.off, S.pair, S.active, S.n_active, n_act_max, *S.hq, n_pairs, S.acc, n_embd)
        be.synchronize()
        assert be.device_status() == 0
        res.append((S.off.cpu().numpy().copy(), S.h.cpu().numpy().copy(), S.acc.cpu().numpy().copy()))
    (off_g, h_g, acc_g), (off_b, h_b, acc_b) = res
    assert off_g[-1] == n_pairs and off_b[-1] == n_pairs - 3
    left_out = np.nonzero((bad.reshape(-1) < 0) | (bad.reshape(-1) >= E))[0]
    kept = np.setdiff1d(np.arange(n_pairs), left_out)
    assert np.all(h_b[left_out] == 7.0) and np.all(acc_b[left_out] == 7.0)
    assert np.array_equal(h_b[kept], h_g[kept]) and np.array_equal(acc_b[kept], acc_g[kept])
    assert not np.any(h_g[left_out] == 7.0)


@pytest.mark.parametrize("t", [12, 14])
def test_grouped_expert_tiles_with_ragged_rows(be, orc, pkg, t):
    """The grouped tensor-core kernel on planes whose row count is not a multiple of its tiles (200 rows:
    64-pair tiles of gate|up, 128-row tiles of down), experts with more tokens than one 32-token tile,
    called through b200q_moe_gate_up / b200q_moe_down directly; every pair against the oracle's rows."""
    from sycl_infer_b200.backend import alloc_act
    from sycl_infer_b200.moe import (moe_actq_launch, moe_csr_launch, moe_grp_down_launch, moe_grp_gate_up_launch,
                                     moe_t)
    E, top_k, K, rows, n_tok = 4, 2, 512, 200, 48
    n_pairs = n_tok * top_k
    rng = np.random.default_rng(5 + t)
    ids = rng.integers(0, E, (n_tok, top_k)).astype(np.int32)
    ids[:40, 0] = 1  # expert 1 gets more than 32 tokens: two tiles of tokens
    i32 = dict(dtype=torch.int32, device="cuda")
    off, pair = torch.zeros(E + 1, **i32), torch.zeros(n_pairs, **i32)
    active, n_active = torch.zeros(E, **i32), torch.zeros(1, **i32)
    moe_csr_launch(be, torch.from_numpy(ids).cuda(), n_pairs, E, off, pair, active, n_active)
    flat = ids.reshape(-1)

    # gate|up: h[p] = silu(gate_e . x_t) * (up_e . x_t)
    gate = [pkg.synth.make_weight(t, rows, K, 100 + e) for e in range(E)]
    up = [pkg.synth.make_weight(t, rows, K, 200 + e) for e in range(E)]
    M = moe_t(gate_exps=torch.from_numpy(np.concatenate(gate)).cuda(), up_exps=torch.from_numpy(np.concatenate(up)).cuda(),
              down_exps=None, gate_type=t, up_type=t, down_type=t, n_expert=E, top_k=top_k, n_embd=K, n_ff_exp=rows)
    x = pkg.synth.make_activation(n_tok, K, 61)
    xq = alloc_act(n_tok, K)
    moe_actq_launch(be, torch.from_numpy(x).cuda(), K, n_tok, K, *xq)
    h = torch.full((n_pairs, rows), 7.0, device="cuda")
    moe_grp_gate_up_launch(be, M, off, pair, active, n_active, E, *xq, n_tok, h, rows)
    be.synchronize()
    assert be.device_status() == 0
    got = h.cpu().numpy()
    for p in range(n_pairs):
        e, one = flat[p], orc.xq(x[p // top_k])
        g = orc.gemm(t, gate[e], K, rows, one)[0]
        u = orc.gemm(t, up[e], K, rows, one)[0]
        with np.errstate(over="ignore"):  # exp(-g) may overflow to inf: silu is then -0, on both sides
            ref = (g / (np.float32(1) + np.exp(-g, dtype=np.float32))) * u
        assert np.max(np.abs(got[p] - ref)) <= 2e-5 * (np.max(np.abs(ref)) + 1e-30), p

    # down: acc[p] = down_e . h_p, 200 output rows, K = 256
    Kd = 256
    down = [pkg.synth.make_weight(t, rows, Kd, 300 + e) for e in range(E)]
    D = moe_t(gate_exps=None, up_exps=None, down_exps=torch.from_numpy(np.concatenate(down)).cuda(), gate_type=t, up_type=t,
              down_type=t, n_expert=E, top_k=top_k, n_embd=rows, n_ff_exp=Kd)
    hv = pkg.synth.make_activation(n_pairs, Kd, 62)
    hq = alloc_act(n_pairs, Kd)
    moe_actq_launch(be, torch.from_numpy(hv).cuda(), Kd, n_pairs, Kd, *hq)
    acc = torch.full((n_pairs, rows), 7.0, device="cuda")
    moe_grp_down_launch(be, D, off, pair, active, n_active, E, *hq, n_pairs, acc, rows)
    be.synchronize()
    assert be.device_status() == 0
    got = acc.cpu().numpy()
    for p in range(n_pairs):
        e, one = flat[p], orc.xq(hv[p])
        ref = orc.gemm(t, down[e], Kd, rows, one)[0]
        ab = orc.gemm_abs(t, down[e], Kd, rows, one)[0]
        assert np.max(np.abs(got[p] - ref) / np.maximum(ab, 1e-30)) <= TOL, p
