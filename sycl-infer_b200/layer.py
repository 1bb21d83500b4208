"""One dense transformer layer's GEMV calls over raw GGUF blocks: the benchmark workload.

A layer is four *calls* in the reference engine's sense (seg_plan::call_t,
src/engine/engine_types.h:46-61 of the reference): q|k|v (three segments sharing the
quantized hidden state), o, gate|up (two segments writing the halves of one 2*n_ff
buffer, src/engine/graph.cpp:342-343) and down (activation silu(gate)*up, residual add
in place, graph.cpp:355-357).  Attention itself is outside this path: the o call reads
a fixed device vector.  With world > 1 every weight is sharded by output rows
(sharding.shard_rows) and each call's outputs are all-gathered before the next call
consumes them.
"""
import torch

from . import synth
from .backend import alloc_act, gemv_seg
from .sharding import gather_rows, shard_rows


class DenseLayer:
    def __init__(self, be, mix="Q4_K_M", seed=0, TB=1, rank=0, world=1, hidden=5120, n_head=40, n_kv=8,
                 head_dim=128, n_ff=17408, group=None, arena=None, norm=False):
        """`arena` (sharding.PeerArena): outputs live in memory every rank maps, each call's GEMV
        stores its rows on all ranks and a flag barrier replaces the all-gather."""
        self.be, self.TB, self.rank, self.world, self.group = be, TB, rank, world, group
        self.arena = arena if world > 1 else None
        self.hidden, self.n_ff, self.q_dim, self.kv_dim = hidden, n_ff, n_head * head_dim, n_kv * head_dim
        dev = be.device
        self.shapes = {n: (t, r, k) for n, t, r, k in
                       synth.dense_layer_shapes(mix, hidden=hidden, n_head=n_head, n_kv=n_kv, head_dim=head_dim,
                                                n_ff=n_ff)}
        self.w, self.rows = {}, {}
        for i, (name, (t, n, K)) in enumerate(self.shapes.items()):
            r0, r1 = shard_rows(n, rank, world)
            rb = synth.row_bytes(t, K)
            full = synth.make_weight(t, n, K, seed * 16 + i)
            self.w[name] = torch.from_numpy(full[r0 * rb:r1 * rb].copy()).to(dev)
            self.rows[name] = (r0, r1)
        f32 = dict(dtype=torch.float32, device=dev)
        new = (lambda *sh: self.arena.alloc(*sh)) if self.arena else (lambda *sh: torch.zeros(*sh, **f32))
        self.qkv = new(TB, self.q_dim + 2 * self.kv_dim)
        self.attn = torch.zeros(TB, self.q_dim, **f32)
        self.o_out = new(TB, hidden)
        self.gu = new(TB, 2 * n_ff)
        self.out = new(TB, hidden)  # the layer's output when the caller passes none
        self.exchange = True  # False: leave the cross-GPU exchange out (timing of the compute alone; wrong results)
        if self.arena:
            self._peers, self._flags = self.arena.peers(), self.arena.flag_ptrs()
            self._sync = (self._flags, world, rank)
        self.act_h = alloc_act(TB, hidden, dev)
        self.act_q = alloc_act(TB, self.q_dim, dev)
        self.act_f = alloc_act(TB, n_ff, dev)
        # one token on one GPU: the gate|up GEMV leaves the quantized silu(gate)*up for the down call
        # norm: RMSNorm of the layer input ahead of q|k|v and of o's output ahead of gate|up, folded into
        # those calls' quantizers (one token on one GPU)
        self.norm = None
        if norm:
            rng_w = lambda s: torch.from_numpy((1.0 + 0.1 * synth.make_activation(1, hidden, s)).astype("float32")).to(dev)  # noqa: E731
            self.norm = (rng_w(seed * 16 + 14).view(-1), rng_w(seed * 16 + 15).view(-1), 1e-6)
        self.fused_h = TB == 1 and world == 1
        # True: o, gate|up and down (each consumes the previous one's output) go out as ONE launch
        # (quant_gemv_chain).  Off by default: measured equal to three launches on its own (47.9 us
        # against ~49) and slower in a step where it alternates with the q|k|v launch (73.7 us against
        # 58.3): two large kernel images taking turns on the SMs cost more than the boundaries save.
        self.chain = False
        self._staging = {}

    def weight_bytes(self):
        return sum(int(w.numel()) for w in self.w.values())

    def _seg(self, name, x, act, out, col0, act_up=None, residual=None):
        t, n, K = self.shapes[name]
        r0, r1 = self.rows[name]
        stride = out.shape[1]
        # synthetic blocks have weights of magnitude ~3; alpha keeps every call's output O(1) so the
        # chain stays inside the f16 range of the activation scales (a real model's weights do)
        seg = gemv_seg(w=self.w[name], type=t, K=K, n_rows=r1 - r0, x=x, x_stride=x.shape[1], act_up=act_up,
                       alpha=1.0 / (3.0 * K ** 0.5),
                       out=out.view(-1)[col0 + r0:], out_stride=stride,
                       residual=None if residual is None else residual.view(-1)[col0 + r0:], x8=act[0],
                       xmeta=act[1], xsumq=act[2])
        return seg, (out, n, col0)

    def calls(self, x, out):
        """The four calls: (segments, [(buffer, full rows, first column)] to gather afterwards)."""
        qd, kd, nf = self.q_dim, self.kv_dim, self.n_ff
        up = self.gu[:, nf:]
        plan = [
            [self._seg("q", x, self.act_h, self.qkv, 0), self._seg("k", x, self.act_h, self.qkv, qd),
             self._seg("v", x, self.act_h, self.qkv, qd + kd)],
            [self._seg("o", self.attn, self.act_q, self.o_out, 0)],
            [self._seg("gate", self.o_out, self.act_h, self.gu, 0), self._seg("up", self.o_out, self.act_h, self.gu, nf)],
            [self._seg("down", self.gu, self.act_f, out, 0, act_up=up, residual=x)],
        ]
        return [([s for s, _ in call], [g for _, g in call]) for call in plan]

    def forward(self, x, out, calls=None):
        calls = calls or self.calls(x, out)
        if self.fused_h and self.chain:
            self.be.quant_gemv_ex(calls[0][0], 1)
            self.be.quant_gemv_chain([(calls[1][0], False, None), (calls[2][0], False, self.act_f),
                                      (calls[3][0], True, None)])
            return out
        for i, (segs, gathers) in enumerate(calls):
            if self.fused_h:
                # one launch per call: q|k|v and o quantize in the GEMV's prologue, gate|up emits down's
                # quantized activation
                nm = None if self.norm is None or i not in (0, 2) else (self.norm[0 if i == 0 else 1], self.norm[2])
                self.be.quant_gemv_ex(segs, 1, prequantized=(i == 3), next_act=self.act_f if i == 2 else None, norm=nm)
                continue
            if self.arena and self.exchange:
                if self.TB == 1:
                    # the launch waits for the peers' rows of the previous call, stores its own rows on
                    # every GPU and signals: no barrier kernel between two calls
                    self.be.quant_gemv_ex(segs, 1, peers=self._peers, sync=self._sync, wait=True, signal=True)
                else:
                    self.be.quant_gemv_scatter(segs, self.TB, self._peers)
                    self.be.peer_barrier(self._flags, self.world, self.rank, 0)  # device-numbered: graph-safe
                continue
            self.be.quant_gemv(segs, self.TB)
            if self.world > 1 and self.exchange:
                for buf, n, col0 in gathers:
                    key = (n, self.TB)
                    if self.TB > 1 and key not in self._staging:
                        self._staging[key] = torch.empty(self.world, self.TB, n // self.world, dtype=buf.dtype,
                                                         device=buf.device)
                    gather_rows(buf, n, col0, self.rank, self.world, self.group, self._staging.get(key))
        return out

    def launches_per_step(self):
        # single token on one GPU: q|k|v, o and gate|up quantize in the GEMV's prologue and gate|up
        # also emits down's quantized activation: one launch per call; otherwise a quantizer + GEMV per call
        if self.arena is not None:  # GEMV with peer stores; down keeps its silu(gate)*up quantizer launch
            return 5 if self.TB == 1 else 12
        if self.fused_h:
            return 2 if self.chain else 4
        return 5 if self.TB == 1 else 8
