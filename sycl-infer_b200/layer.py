"""One dense transformer layer's GEMV calls over raw GGUF blocks: the benchmark workload.

A layer is four *calls* in the reference engine's sense (seg_plan::call_t,
src/engine/engine_types.h:46-61 of the reference): q|k|v (three segments sharing the
quantized hidden state), o, gate|up (two segments writing the halves of one 2*n_ff
buffer, src/engine/graph.cpp:342-343) and down (activation silu(gate)*up, residual add
in place, graph.cpp:355-357).  Attention itself is outside this path: the o call reads
a fixed device vector.  With world_size > 1 every weight is sharded by output rows and
each call's output is all-gathered (NCCL) before the next call consumes it.
"""
import numpy as np
import torch

from . import synth
from .backend import alloc_act, gemv_seg


def _shard(n_rows, rank, world):
    """Contiguous row range of `rank`; boundaries are multiples of 8 rows."""
    per = -(-n_rows // world)
    per = -(-per // 8) * 8
    r0 = min(n_rows, rank * per)
    return r0, min(n_rows, r0 + per)


class DenseLayer:
    def __init__(self, be, mix="Q4_K_M", seed=0, TB=1, rank=0, world=1, hidden=5120, n_head=40, n_kv=8,
                 head_dim=128, n_ff=17408):
        self.be, self.TB, self.rank, self.world = be, TB, rank, world
        self.hidden, self.n_ff, self.q_dim, self.kv_dim = hidden, n_ff, n_head * head_dim, n_kv * head_dim
        dev = be.device
        self.shapes = {n: (t, r, k) for n, t, r, k in
                       synth.dense_layer_shapes(mix, hidden=hidden, n_head=n_head, n_kv=n_kv, head_dim=head_dim,
                                                n_ff=n_ff)}
        self.w, self.rows = {}, {}
        for i, (name, (t, n, K)) in enumerate(self.shapes.items()):
            r0, r1 = _shard(n, rank, world)
            rb = synth.row_bytes(t, K)
            full = synth.make_weight(t, n, K, seed * 16 + i)
            self.w[name] = torch.from_numpy(full[r0 * rb:r1 * rb].copy()).to(dev)
            self.rows[name] = (r0, r1)
        f32 = dict(dtype=torch.float32, device=dev)
        self.qkv = torch.zeros(TB, self.q_dim + 2 * self.kv_dim, **f32)
        self.attn = torch.zeros(TB, self.q_dim, **f32)
        self.o_out = torch.zeros(TB, hidden, **f32)
        self.gu = torch.zeros(TB, 2 * n_ff, **f32)
        self.act_h = alloc_act(TB, hidden, dev)
        self.act_q = alloc_act(TB, self.q_dim, dev)
        self.act_f = alloc_act(TB, n_ff, dev)

    def weight_bytes(self):
        return sum(int(w.numel()) for w in self.w.values())

    def algorithmic_bytes(self):
        """Raw weight blocks read once + fp32 activations read + fp32 outputs written."""
        vec = 4 * self.TB * (self.hidden + self.q_dim + 2 * self.n_ff  # inputs of qkv, o, down(gate, up)
                             + self.hidden  # gate|up input
                             + (self.q_dim + 2 * self.kv_dim) + self.hidden + 2 * self.n_ff + self.hidden)
        return self.weight_bytes() + vec

    def _seg(self, name, x, act, out, col0, out_stride, act_up=None, residual=None):
        t, n, K = self.shapes[name]
        r0, r1 = self.rows[name]
        o = out.view(-1)[col0 + r0:]
        return gemv_seg(w=self.w[name], type=t, K=K, n_rows=r1 - r0, x=x, x_stride=x.shape[1], act_up=act_up,
                        out=o, out_stride=out_stride, residual=None if residual is None else
                        residual.view(-1)[col0 + r0:], x8=act[0], xmeta=act[1], xsumq=act[2])

    def calls(self, x, out):
        """The four calls as lists of segments (x: [TB, hidden] in, out: [TB, hidden])."""
        qd, kd, nf, h = self.q_dim, self.kv_dim, self.n_ff, self.hidden
        wq = qd + 2 * kd
        gate, up = self.gu[:, :nf], self.gu[:, nf:]
        return [
            ([self._seg("q", x, self.act_h, self.qkv, 0, wq), self._seg("k", x, self.act_h, self.qkv, qd, wq),
              self._seg("v", x, self.act_h, self.qkv, qd + kd, wq)], self.qkv),
            ([self._seg("o", self.attn, self.act_q, self.o_out, 0, h)], self.o_out),
            ([self._seg("gate", self.o_out, self.act_h, self.gu, 0, 2 * nf),
              self._seg("up", self.o_out, self.act_h, self.gu, nf, 2 * nf)], self.gu),
            ([self._seg("down", self.gu, self.act_f, out, 0, h, act_up=up, residual=x)], out),
        ]

    def gather(self, buf, segs):
        """All-gather the row shards the call just wrote (in place, NCCL)."""
        import torch.distributed as dist
        for s in segs:
            name = next(n for n, w in self.w.items() if w is s.w)
            t, n, K = self.shapes[name]
            per = self.rows[name][1] - self.rows[name][0]
            if per * self.world != n:
                raise ValueError("row sharding must be even for the in-place all-gather")
        for tok in range(self.TB):
            for s in segs:
                name = next(n for n, w in self.w.items() if w is s.w)
                n = self.shapes[name][1]
                off = s.out.data_ptr() - buf.data_ptr()
                col0 = (off // 4) % buf.shape[1] - self.rows[name][0]
                full = buf[tok, col0:col0 + n]
                dist.all_gather_into_tensor(full, full[self.rows[name][0]:self.rows[name][1]])

    def forward(self, x, out, graph_safe=True):
        for segs, buf in self.calls(x, out):
            self.be.quant_gemv(segs, self.TB)
            if self.world > 1:
                self.gather(buf, segs)
        return out

    def launches_per_step(self):
        return 8  # 4 calls x (activation quantizer + GEMV)


def layer_numpy_inputs(TB, hidden, q_dim, seed):
    rng = np.random.default_rng(seed)
    return (rng.normal(0, 1, (TB, hidden)).astype(np.float32), rng.normal(0, 1, (TB, q_dim)).astype(np.float32))
