"""Multi-GPU placement of the GEMV path: row sharding with an all-gather, and the reference's
contiguous layer split as the pipeline-parallel alternative.

Row sharding is new relative to the reference (it has no tensor parallelism): output rows are
independent and contiguous byte ranges of a GGUF tensor, so rank r of P owns a zero-copy slice
[r0, r1) of every weight; the quantized activation is replicated; one exchange step per call
gathers the row shards of its outputs.  The layer split keeps the reference's `--layer-map`
semantics (src/engine/engine.cpp:3505-3570 of the reference): comma-separated inclusive ranges
`begin-end:device` that must cover [0, n_layer) in order, each device computing its range and
handing the hidden state to the next (engine::handoff_x, src/engine/engine.cpp:2424-2468 - a
host-staged copy there, a peer send/recv here).

Everything in this file is host logic on torch tensors and `torch.distributed`; it runs
unchanged on CPU tensors with the gloo backend, which is how it is tested without GPUs.
"""
from dataclasses import dataclass
from typing import List

import torch
import torch.distributed as dist


def shard_rows(n_rows: int, rank: int, world: int, align: int = 16):
    """Contiguous, equal-size row range of `rank`.  The in-place all-gather needs equal
    shards, so n_rows must split into `world` multiples of `align` rows (a tile of the
    streaming kernel); anything else is an error, not a silent imbalance."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    if n_rows % (world * align):
        raise ValueError(f"{n_rows} rows do not split into {world} shards of a multiple of {align} rows")
    per = n_rows // world
    return rank * per, (rank + 1) * per


def gather_rows(full: torch.Tensor, n_rows: int, col0: int, rank: int, world: int, group=None, staging=None):
    """All-gather the row shards of one segment's output, in place.

    `full` is the [TB, stride] output buffer; the segment occupies columns col0..col0+n_rows and
    this rank has just written its shard.  One token: the shards are contiguous, the collective
    runs in place.  Several tokens: the shards go through `staging` ([world, TB, per]) and are
    copied back, because a token-major buffer interleaves the ranks."""
    if world == 1:
        return
    TB = full.shape[0]
    per = n_rows // world
    if TB == 1:
        seg = full[0, col0:col0 + n_rows]
        dist.all_gather_into_tensor(seg, seg[rank * per:(rank + 1) * per].clone() if seg.device.type == "cpu"
                                    else seg[rank * per:(rank + 1) * per], group=group)
        return
    if staging is None:
        staging = torch.empty(world, TB, per, dtype=full.dtype, device=full.device)
    local = full[:, col0 + rank * per:col0 + (rank + 1) * per].contiguous()
    dist.all_gather_into_tensor(staging.view(-1), local.view(-1), group=group)
    full[:, col0:col0 + n_rows].view(TB, world, per).copy_(staging.permute(1, 0, 2))


@dataclass
class LayerRange:
    l0: int  # first layer
    l1: int  # one past the last layer
    device: str  # "gpu.N" or "cpu"


def parse_layer_map(layer_map: str, n_layer: int) -> List[LayerRange]:
    """The reference's --layer-map grammar and checks, error for error."""
    ents: List[LayerRange] = []
    for tok in layer_map.split(","):
        if not tok:
            continue
        if ":" not in tok:
            raise ValueError("bad --layer-map entry (expect begin-end:device): " + tok)
        rng, dev = tok.split(":", 1)
        if "-" not in rng:
            raise ValueError("bad --layer-map range: " + rng)
        a, b = rng.split("-", 1)
        try:
            l0, l1 = int(a), int(b) + 1  # begin-end is inclusive
        except ValueError:
            raise ValueError("bad --layer-map range: " + rng) from None
        if dev in ("cpu", "host", "1"):
            device = "cpu"
        elif dev.startswith("gpu."):
            device = "gpu." + str(int(dev[4:]))
        elif dev == "gpu":
            device = "gpu.0"
        else:
            raise ValueError("bad --layer-map device (expect gpu[.N] or cpu): " + dev)
        if l0 < 0 or l1 <= l0:
            raise ValueError("bad --layer-map range: " + rng)
        ents.append(LayerRange(l0, l1, device))
    if not ents:
        raise ValueError("empty --layer-map")
    expect = 0
    for e in ents:
        if e.l0 != expect:
            raise ValueError("--layer-map must cover every layer without gaps")
        expect = e.l1
    if expect != n_layer:
        raise ValueError("--layer-map must end at the model's layer count")
    return ents


def even_layer_map(n_layer: int, world: int) -> str:
    """`world` contiguous ranges of (almost) equal length, one per GPU."""
    cuts = [n_layer * r // world for r in range(world + 1)]
    return ",".join(f"{cuts[r]}-{cuts[r + 1] - 1}:gpu.{r}" for r in range(world) if cuts[r + 1] > cuts[r])


def rank_of_layer(ranges: List[LayerRange], layer: int) -> int:
    for i, e in enumerate(ranges):
        if e.l0 <= layer < e.l1:
            return i
    raise ValueError(f"layer {layer} is not in the layer map")


def handoff_x(x: torch.Tensor, src: int, dst: int, rank: int, group=None):
    """Hidden-state hand-off at a partition boundary: only the live rows travel (x is [TB, hidden])."""
    if src == dst:
        return
    if rank == src:
        dist.send(x, dst, group=group)
    elif rank == dst:
        dist.recv(x, src, group=group)


def run_layer_split(ranges: List[LayerRange], rank: int, x: torch.Tensor, run_layer, group=None):
    """Walk all layers in order; each rank runs the layers of its range (`run_layer(l, x)` updates
    x in place) and passes x on at the boundary.  Returns x on the rank that ran the last layer."""
    for i, e in enumerate(ranges):
        if rank == i:
            for layer in range(e.l0, e.l1):
                run_layer(layer, x)
        if i + 1 < len(ranges):
            handoff_x(x, i, i + 1, rank, group)
    return x


class PeerArena:
    """One fp32 output arena that every rank of the group maps at the same layout (torch
    symmetric memory: CUDA IPC / fabric handles underneath), plus the flag words of the
    cross-GPU barrier.  Buffers carved from it can be the `out` of a scattered call: the GEMV
    epilogue stores each value into every rank's copy, so no collective follows the GEMV."""

    def __init__(self, n_floats: int, rank: int, world: int, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        self.rank, self.world = rank, world
        self.buf = symm_mem.empty(n_floats + 64, dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.used = 64  # the first 64 words are the barrier flags (one word per source rank)
        self.seq = 0
        dist.barrier(group)

    def alloc(self, *shape):
        n = 1
        for d in shape:
            n *= d
        n_al = -(-n // 64) * 64
        t = self.buf[self.used:self.used + n].view(*shape)
        self.used += n_al
        if self.used > self.buf.numel():
            raise MemoryError("PeerArena exhausted")
        return t

    def peers(self):
        """b200q_peers for this rank: byte distances to the other ranks' mappings."""
        from .capi import Peers
        p = Peers()
        others = [r for r in range(self.world) if r != self.rank]
        p.n_peers = len(others)
        for i, r in enumerate(others):
            p.out_delta[i] = self.ptrs[r] - self.ptrs[self.rank]
        return p

    def flag_ptrs(self):
        import ctypes as C
        return (C.c_void_p * self.world)(*self.ptrs)  # flags live at the start of every mapping
