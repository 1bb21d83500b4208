"""Routed mixture-of-experts FFN on raw GGUF expert banks: host-side mirror of the reference's
MoE launchers for this path.

The reference calls these as free functions on its queue, not through `compute_backend`
(src/engine/graph.cpp:905-1122 of the reference): `moe_router_launch`, the `moe_csr_*` launchers,
`moe_actq_launch`, `moe_grp_gate_up_launch`, `moe_grp_down_launch`, `moe_reduce_launch`
(src/backend/gpu/kernels/kernels.h:595-792).  Same names and argument meaning here; the queue
argument is a `cuda_backend` (one device + one stream).  `moe_call` strings them together the way
the engine's `moe_call` does (graph.cpp:787-1122).  All scratch is caller-owned (`MoeScratch`),
as in the reference, so the sequence can be recorded into a CUDA graph.
"""
import ctypes as C
from dataclasses import dataclass

import torch

from .backend import _ptr, alloc_act
from . import synth


@dataclass
class moe_t:
    """Expert banks of one layer (reference: moe_t / cpu_moe, src/backend/cpu/cpu_types.h:195-211)."""
    gate_exps: object  # uint8 [n_expert][n_ff_exp rows][n_embd] raw blocks
    up_exps: object
    down_exps: object  # uint8 [n_expert][n_embd rows][n_ff_exp]
    gate_type: int
    up_type: int
    down_type: int
    n_expert: int
    top_k: int
    n_embd: int
    n_ff_exp: int
    gate_inp: object = None  # F32 router [n_expert][n_embd] or None (logits supplied)

    @property
    def slot_gb(self):
        return synth.row_bytes(self.gate_type, self.n_embd) * self.n_ff_exp

    @property
    def slot_ub(self):
        return synth.row_bytes(self.up_type, self.n_embd) * self.n_ff_exp

    @property
    def slot_db(self):
        return synth.row_bytes(self.down_type, self.n_ff_exp) * self.n_embd


class MoeScratch:
    """Caller-owned device scratch of one MoE call (the engine's d_moe_* buffers)."""

    def __init__(self, M: moe_t, n_tok, device="cuda"):
        n_pairs = n_tok * M.top_k
        i32 = dict(dtype=torch.int32, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.logits = torch.zeros(n_tok, M.n_expert, **f32)
        self.ids = torch.zeros(n_tok, M.top_k, **i32)
        self.wts = torch.zeros(n_tok, M.top_k, **f32)
        self.off = torch.zeros(M.n_expert + 1, **i32)
        self.pair = torch.zeros(n_pairs, **i32)
        self.active = torch.zeros(M.n_expert, **i32)
        self.n_active = torch.zeros(1, **i32)
        self.xq = alloc_act(n_tok, M.n_embd, device)
        self.h = torch.zeros(n_pairs, M.n_ff_exp, **f32)
        self.hq = alloc_act(n_pairs, M.n_ff_exp, device)
        self.acc = torch.zeros(n_pairs, M.n_embd, **f32)


def moe_router_launch(be, gate_inp, gp_type, x, x_stride, n_tok, n_embd, n_expert, top_k, logits, ids, wts):
    if gate_inp is not None and gp_type != 0:
        raise RuntimeError("moe_router_launch: only an F32 router (ggml type 0) is implemented")
    be.lib.check(be.lib.moe_route(be._s(), _ptr(gate_inp), _ptr(x), x_stride, n_tok, n_embd, n_expert, top_k,
                                  _ptr(logits), _ptr(ids), _ptr(wts)))


def moe_router_csr_launch(be, gate_inp, gp_type, x, x_stride, n_tok, n_embd, n_expert, top_k, logits, ids, wts, off,
                          pair, active, n_active):
    """moe_router_launch + moe_csr_launch; the router's last CTA builds the CSR (one kernel less)."""
    if gate_inp is not None and gp_type != 0:
        raise RuntimeError("moe_router_csr_launch: only an F32 router (ggml type 0) is implemented")
    be.lib.check(be.lib.moe_route_csr(be._s(), _ptr(gate_inp), _ptr(x), x_stride, n_tok, n_embd, n_expert, top_k,
                                      _ptr(logits), _ptr(ids), _ptr(wts), _ptr(off), _ptr(pair), _ptr(active),
                                      _ptr(n_active)))


def moe_csr_launch(be, ids, n_pairs, n_expert, off, pair, active, n_active):
    """moe_csr_clear/count/prefix/scatter_launch of the reference in one launch."""
    be.lib.check(be.lib.moe_csr(be._s(), _ptr(ids), n_pairs, n_expert, _ptr(off), _ptr(pair), _ptr(active),
                                _ptr(n_active)))


def moe_actq_launch(be, x, x_stride, n_rows, K, x8, xmeta, xsumq):
    """Per-row int8 quantization of an activation tile.  The reference's device variant writes a
    row-major layout with an f16-rounded (RNE) scale; this path keeps the host quantizer's
    layout and rounding (cpu_xq: group-major, truncated f16 scale), the one the oracle defines."""
    be.xq(x, None, x_stride, x_stride, x8, xmeta, xsumq, None, n_rows, K)


def moe_grp_gate_up_launch(be, M, off, pair, active, n_active, n_act_max, x8, xmeta, xsumq, n_tok, h, h_stride):
    be.lib.check(be.lib.moe_gate_up(be._s(), _ptr(M.gate_exps), _ptr(M.up_exps), M.gate_type, M.up_type,
                                    C.c_size_t(M.slot_gb), C.c_size_t(M.slot_ub), _ptr(off), _ptr(pair),
                                    _ptr(active), _ptr(n_active), n_act_max, _ptr(x8), _ptr(xmeta), _ptr(xsumq),
                                    n_tok, _ptr(h), h_stride, M.n_embd, M.n_ff_exp, M.top_k))
    return True


def moe_grp_gate_up_q_launch(be, M, off, pair, active, n_active, n_act_max, x8, xmeta, xsumq, n_tok, h, h_stride, h8,
                             hmeta, hsumq):
    """moe_grp_gate_up_launch that also leaves h quantized for the down launch (no quantizer launch
    in between where the expert kernel can do it in its epilogue)."""
    be.lib.check(be.lib.moe_gate_up_q(be._s(), _ptr(M.gate_exps), _ptr(M.up_exps), M.gate_type, M.up_type,
                                      C.c_size_t(M.slot_gb), C.c_size_t(M.slot_ub), _ptr(off), _ptr(pair),
                                      _ptr(active), _ptr(n_active), n_act_max, _ptr(x8), _ptr(xmeta), _ptr(xsumq),
                                      n_tok, _ptr(h), h_stride, M.n_embd, M.n_ff_exp, M.top_k, _ptr(h8), _ptr(hmeta),
                                      _ptr(hsumq)))
    return True


def moe_grp_down_launch(be, M, off, pair, active, n_active, n_act_max, h8, hmeta, hsumq, n_pairs, acc, acc_stride):
    be.lib.check(be.lib.moe_down(be._s(), _ptr(M.down_exps), M.down_type, C.c_size_t(M.slot_db), _ptr(off),
                                 _ptr(pair), _ptr(active), _ptr(n_active), n_act_max, _ptr(h8), _ptr(hmeta),
                                 _ptr(hsumq), n_pairs, _ptr(acc), acc_stride, M.n_embd, M.n_ff_exp))
    return True


def moe_reduce_launch(be, acc, wts, top_k, n_tok, n_embd, acc_stride, out, out_stride):
    be.lib.check(be.lib.moe_reduce(be._s(), _ptr(acc), _ptr(wts), top_k, n_tok, n_embd, acc_stride, _ptr(out),
                                   out_stride))


def moe_call(be, M: moe_t, S: MoeScratch, x, n_tok, out, logits_given=False, fused_hq=False):
    """One routed-MoE FFN: out[t] += sum_j w[t,j] * expert_{ids[t,j]}(x[t]).
    fused_hq: gate|up also quantizes h (one launch less; measured slower than the quantizer launch
    at config 3's size, so off by default)."""
    n_pairs = n_tok * M.top_k
    n_act_max = min(M.n_expert, n_pairs)
    # the token quantizer does not depend on the router: it goes first
    moe_actq_launch(be, x, x.shape[1], n_tok, M.n_embd, *S.xq)
    moe_router_csr_launch(be, None if logits_given else M.gate_inp, 0, x, x.shape[1], n_tok, M.n_embd, M.n_expert,
                          M.top_k, S.logits, S.ids, S.wts, S.off, S.pair, S.active, S.n_active)
    if fused_hq and M.n_ff_exp % 32 == 0:
        moe_grp_gate_up_q_launch(be, M, S.off, S.pair, S.active, S.n_active, n_act_max, *S.xq, n_tok, S.h, M.n_ff_exp,
                                 *S.hq)
    else:
        moe_grp_gate_up_launch(be, M, S.off, S.pair, S.active, S.n_active, n_act_max, *S.xq, n_tok, S.h, M.n_ff_exp)
        moe_actq_launch(be, S.h, M.n_ff_exp, n_pairs, M.n_ff_exp, *S.hq)
    moe_grp_down_launch(be, M, S.off, S.pair, S.active, S.n_active, n_act_max, *S.hq, n_pairs, S.acc, M.n_embd)
    moe_reduce_launch(be, S.acc, S.wts, M.top_k, n_tok, M.n_embd, M.n_embd, out, out.shape[1])
    return out


def make_synthetic_moe(n_expert=256, top_k=8, n_embd=2048, n_ff_exp=512, types=(12, 12, 12), seed=0, device="cuda",
                       with_router=False):
    """Benchmark configuration 3: 256 experts, top-8, hidden 2048, expert FFN 512, Q4_K banks."""
    import numpy as np
    gt, ut, dt = types
    mk = lambda t, rows, K, s: torch.from_numpy(synth.make_weight(t, rows, K, s))  # noqa: E731
    g = mk(gt, n_expert * n_ff_exp, n_embd, seed * 8 + 1)
    u = mk(ut, n_expert * n_ff_exp, n_embd, seed * 8 + 2)
    d = mk(dt, n_expert * n_embd, n_ff_exp, seed * 8 + 3)
    r = None
    if with_router:
        r = torch.from_numpy(np.random.default_rng(seed * 8 + 4).normal(0, 1, (n_expert, n_embd)).astype(np.float32))
    host = moe_t(g, u, d, gt, ut, dt, n_expert, top_k, n_embd, n_ff_exp, r)
    dev = moe_t(g.to(device), u.to(device), d.to(device), gt, ut, dt, n_expert, top_k, n_embd, n_ff_exp,
                None if r is None else r.to(device))
    return host, dev
