"""The caller's side of the GEMV path: a forward plan and its replay as one CUDA graph.

The reference engine describes a forward pass as a `seg_plan` - a flat list of GEMV segments cut
into calls, each call with the activation its quantizer reads (src/engine/engine_types.h:11-133) -
and replays it with `record_forward` into a command graph per token (src/engine/engine.h:1269,
src/engine/graph.cpp:145-429).  `SegPlan` mirrors that structure (begin_call / add / set_xq /
finalize, same meaning) and adds what this library can do with it: `finalize()` lowers the calls to
launches, pairing a gate|up call with the down call that consumes silu(gate)*up (the former emits
the latter's quantized activation, the latter runs without a quantizer), folding a call's RMSNorm
into its quantizer and hanging the argmax on the head call; `record()` captures the launches of a
whole token into ONE CUDA graph and `replay()` runs it.

`PlanBuckets` mirrors the engine's decode buckets (src/engine/engine.h:770-782, src/engine/graph.cpp:
2824-2835 and 3146-3194): one plan per row count 1..max_rows, so that a decode step of n sequences runs
exactly n rows, with a recorded graph for the coarse row counts only and direct replay of the plan for
the others.
"""
from dataclasses import dataclass, field

from .backend import gemv_seg

MAX_SEGS = 8


@dataclass
class Call:
    """One call of the plan: segments sharing one quantized activation (seg_plan::call_t)."""
    tb: int
    segs: list = field(default_factory=list)
    x: object = None          # fp32 activation the call's quantizer reads (xq_t.x)
    up: object = None         # non-None: the activation is silu(x) * up (xq_t.up)
    norm: tuple = None        # (weight, eps): RMSNorm of x ahead of the quantizer
    argmax: tuple = None      # (idx, val or None): argmax of the outputs (the head call)
    # a routed-MoE call has no segments: it dispatches the MoE launch sequence (call_t::moe_routed)
    moe: tuple = None         # (moe_t, MoeScratch, out): out[t] += sum_j w[t,j] * expert(x[t])
    # set by finalize()
    prequantized: bool = False
    next_act: tuple = None

    @property
    def total_rows(self):
        return sum(s.n_rows for s in self.segs)


def _same(a, b):
    return a is not None and b is not None and a.data_ptr() == b.data_ptr()


class SegPlan:
    def __init__(self):
        self.calls = []
        self.lowered = None
        self.graph = None

    # ---- building (names and meaning of seg_plan's builders) ---------------------------------
    def begin_call(self, tb=1):
        self.calls.append(Call(tb=tb))
        self.lowered = None

    def add(self, seg: gemv_seg):
        self.calls[-1].segs.append(seg)

    def set_xq(self, x, up=None):
        self.calls[-1].x, self.calls[-1].up = x, up

    def set_norm(self, weight, eps):
        self.calls[-1].norm = (weight, float(eps))

    def set_argmax(self, idx, val=None):
        self.calls[-1].argmax = (idx, val)

    def begin_moe_call(self, M, scratch, x, out, tb):
        """A routed-MoE FFN in the call sequence (seg_plan::begin_moe_call): router, CSR, quantizers,
        grouped gate|up and down, reduce - recorded into the same graph as the dense calls."""
        self.calls.append(Call(tb=tb, x=x, moe=(M, scratch, out)))
        self.lowered = None

    # ---- validation + lowering ------------------------------------------------------------------
    def validate(self):
        """Structural self-check (seg_plan::validate): raises ValueError naming the first violation."""
        for ci, c in enumerate(self.calls):
            if c.moe is not None:
                if c.segs or c.x is None or c.norm or c.argmax:
                    raise ValueError(f"call {ci}: a MoE call has an activation and nothing else")
                continue
            if not 1 <= len(c.segs) <= MAX_SEGS:
                raise ValueError(f"call {ci}: {len(c.segs)} segments (1..{MAX_SEGS})")
            if c.x is None:
                raise ValueError(f"call {ci}: no activation (set_xq)")
            s0 = c.segs[0]
            for si, s in enumerate(c.segs):
                if s.K != s0.K or not _same(s.x8, s0.x8) or not _same(s.xmeta, s0.xmeta) or not _same(s.xsumq, s0.xsumq):
                    raise ValueError(f"call {ci}: segment {si} does not share the call's K and activation scratch")
                if s.n_rows < 1 or s.K % 256:
                    raise ValueError(f"call {ci}: segment {si} has no rows or a K that is not a multiple of 256")
            if c.tb < 1:
                raise ValueError(f"call {ci}: tb < 1")
            if c.tb != 1 and (c.norm or c.argmax):
                raise ValueError(f"call {ci}: norm / argmax are single-token options")

    def finalize(self):
        """Validate, then decide the launches.  A single-token call whose activation is silu(g)*u of
        the two segments of the call right before it (equal rows, a multiple of 32, one type) is
        paired with it: no quantizer runs between them."""
        self.validate()
        for c in self.calls:
            c.prequantized, c.next_act = False, None
        for p, c in zip(self.calls, self.calls[1:]):
            if (p.moe is None and c.moe is None and c.tb == 1 and p.tb == 1 and c.up is not None and c.norm is None and p.argmax is None and len(p.segs) == 2 and
                    _same(p.segs[0].out, c.x) and _same(p.segs[1].out, c.up) and p.segs[0].type == p.segs[1].type and
                    p.segs[0].n_rows == p.segs[1].n_rows and p.segs[0].n_rows % 32 == 0 and
                    p.segs[0].n_rows == c.segs[0].K):
                s0 = c.segs[0]
                p.next_act, c.prequantized = (s0.x8, s0.xmeta, s0.xsumq), True
        self.lowered = True
        return self

    def launches(self):
        """Kernel launches of one replay (the single-token kernel quantizes plain activations itself;
        silu(x)*up outside a pairing and several tokens take a quantizer launch)."""
        assert self.lowered, "finalize() first"
        n = 0
        for c in self.calls:
            if c.moe is not None:
                n += 7  # token quantizer, router logits, softmax/top-k + CSR, gate|up, quantizer of h, down, reduce
            else:
                n += 1 if c.prequantized or (c.tb == 1 and c.up is None) else 2
        return n

    # ---- execution ------------------------------------------------------------------------------
    def run(self, be):
        assert self.lowered, "finalize() first"
        from .moe import moe_call
        for c in self.calls:
            if c.moe is not None:
                M, scratch, out = c.moe
                moe_call(be, M, scratch, c.x, c.tb, out)
                continue
            segs = []
            # the segments carry the call's activation, as the C ABI wants it; a 2-D activation may be a
            # column slice of a wider buffer: its row stride, not its width, separates the rows
            x_stride = c.x.stride(0) if c.x.dim() > 1 else c.x.shape[-1]
            for s in c.segs:
                s.x, s.act_up, s.x_stride = c.x, c.up, x_stride
                segs.append(s)
            if c.tb == 1:
                be.quant_gemv_ex(segs, 1, prequantized=c.prequantized, next_act=c.next_act, norm=c.norm, argmax=c.argmax)
            else:
                be.quant_gemv(segs, c.tb)

    def record(self, be, stream):
        """Capture one pass over the plan into a CUDA graph on `stream` (record_forward)."""
        import torch
        prev = be._stream
        be._stream = stream
        try:
            with torch.cuda.stream(stream):
                self.run(be)  # warm-up: attributes, lazy state
                stream.synchronize()
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, stream=stream):
                    self.run(be)
        finally:
            be._stream = prev
        torch.cuda.synchronize()
        return self.graph

    def replay(self):
        self.graph.replay()


class PlanBuckets:
    """Decode plans by row count.  `build(tb)` returns the (unfinalized or finalized) SegPlan of a step
    with tb rows; plans are built on first use (`build_all()` builds every one up front, as the engine
    does).  `run(be, n_rows, stream)` replays the bucket's CUDA graph when n_rows is one of the graphed
    row counts (1, 2, 4, 8, 16 and max_rows: dec_graph_rows) and a stream is given, else it issues the
    plan's launches directly."""

    def __init__(self, build, max_rows):
        if max_rows < 1:
            raise ValueError("max_rows < 1")
        self.build, self.max_rows = build, int(max_rows)
        self.plans = {}

    def graph_rows(self, tb):
        return tb in (1, 2, 4, 8, 16, self.max_rows)

    def bucket(self, n_rows):
        if not 1 <= n_rows <= self.max_rows:
            raise ValueError(f"{n_rows} rows: buckets cover 1..{self.max_rows}")
        p = self.plans.get(n_rows)
        if p is None:
            p = self.build(n_rows)
            for ci, c in enumerate(p.calls):
                if c.tb != n_rows:
                    raise ValueError(f"bucket {n_rows}: call {ci} was built for {c.tb} rows")
            if not p.lowered:
                p.finalize()
            self.plans[n_rows] = p
        return p

    def build_all(self):
        for tb in range(1, self.max_rows + 1):
            self.bucket(tb)
        return self

    def launches(self, n_rows):
        return self.bucket(n_rows).launches()

    def run(self, be, n_rows, stream=None):
        p = self.bucket(n_rows)
        if stream is not None and self.graph_rows(n_rows):
            if p.graph is None:
                p.record(be, stream)
            p.replay()
        else:
            p.run(be)
        return p
