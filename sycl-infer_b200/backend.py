"""Host-side mirror of the reference engine's backend-operator interface for the
integer GEMV/GEMM path.

`cuda_backend` carries the same operator names, argument order and meaning as the
reference's `compute_backend` (src/backend/backend.h:33-124 of the reference) for the
operators on this path - `xq`, `i8_gemv`, `i8_gemm`, `gemv_group`, `synchronize` - and
`gemv_seg` mirrors its segment descriptor (src/backend/gpu/kernels/kernels.h:44-81).
Like the reference's backends it is one device + one in-order queue (a CUDA stream),
owns no memory, and raises (RuntimeError subclass) instead of falling back when an
operator is not available.  Buffers are torch CUDA tensors (device memory plumbing
only); every operator goes through the C ABI of libb200q.so.
"""
import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from .capi import MAX_SEGS, Seg, load_lib


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    assert t.is_cuda, "device tensor expected"
    return t.data_ptr()


@dataclass
class gemv_seg:
    """One GEMV output segment (reference: gemv_seg / cpu_gemv_seg)."""
    w: object = None            # uint8 tensor: raw GGUF blocks [n_rows][K]
    type: int = 0               # ggml type id
    K: int = 0
    n_rows: int = 0
    x: object = None            # fp32 activations (fused-quantize operators)
    x_stride: int = 0
    act_up: object = None       # non-None: activation is silu(x)*act_up
    out: object = None          # fp32, out[t*out_stride + row]
    out_stride: int = 0
    residual: object = None
    alpha: float = 1.0
    x8: object = None           # int8 codes, group-major
    xmeta: object = None        # fp32 (scale, 0) pairs
    xsumq: object = None        # int32 pairs of 16-value sums
    i8: bool = True

    def to_c(self):
        return Seg(_ptr(self.w), self.type, self.K, self.n_rows, _ptr(self.x), self.x_stride, _ptr(self.act_up),
                   _ptr(self.out), self.out_stride or self.n_rows, _ptr(self.residual), self.alpha, _ptr(self.x8),
                   _ptr(self.xmeta), _ptr(self.xsumq))


def _pack(segs):
    if isinstance(segs, gemv_seg):
        segs = [segs]
    if not 1 <= len(segs) <= MAX_SEGS:
        raise ValueError(f"a call holds 1..{MAX_SEGS} segments")
    arr = (Seg * len(segs))(*[s.to_c() for s in segs])
    return arr, len(segs)


class cuda_backend:
    """One B200 + one stream.  Mirrors compute_backend for the int8 GEMV/GEMM path."""

    def __init__(self, device=0, stream: Optional[torch.cuda.Stream] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("cuda_backend needs a CUDA device; this library has no CPU path")
        self.lib = load_lib()
        self.device = torch.device("cuda", device)
        self._stream = stream

    def name(self):
        return "b200q-cuda"

    def is_cpu(self):
        return False

    def kind(self):
        return "gpu"

    @property
    def stream(self):
        return self._stream if self._stream is not None else torch.cuda.current_stream(self.device)

    def _s(self):
        return C.c_void_p(self.stream.cuda_stream)

    # compute_backend::xq (backend.h:104-105): x8/xmeta/xsumq are caller-owned outputs
    def xq(self, x, up, x_stride, up_stride, x8, xmeta, xsumq, info, TB, K):
        del info  # the reference's host quantizer ignores it as well (xq.cpp:12)
        self.lib.check(self.lib.xq(self._s(), _ptr(x), _ptr(up), x_stride, up_stride, _ptr(x8), _ptr(xmeta),
                                   _ptr(xsumq), TB, K))

    # compute_backend::i8_gemv (backend.h:113); a list runs the segments of one call in one launch
    def i8_gemv(self, s):
        arr, n = _pack(s)
        self.lib.check(self.lib.i8_gemv(self._s(), arr, n))

    # compute_backend::i8_gemm (backend.h:114)
    def i8_gemm(self, s, TB):
        arr, n = _pack(s)
        self.lib.check(self.lib.i8_gemm(self._s(), arr, n, TB))

    # compute_backend::gemv_group (backend.h:61-62): every segment of one type-group of a
    # call, activation given as fp32.  Here the group is quantized into the scratch the
    # segments carry (x8/xmeta/xsumq, engine-owned as in src/engine/graph.cpp:218-220)
    # and run on the integer path; total_rows/nsb/n_tok_blocks are implied by the
    # segments and accepted for signature parity.
    def gemv_group(self, type, segs, n_segs, total_rows, TB, nsb=0, n_tok_blocks=0):
        segs = list(segs)[:n_segs]
        if any(s.type != type for s in segs):
            raise ValueError("gemv_group: every segment must have the group's type")
        if total_rows != sum(s.n_rows for s in segs):
            raise ValueError("gemv_group: total_rows does not match the segments")
        self.quant_gemv(segs, TB)

    # fused decode launch (reference: i8_grp_quant_gemv_launch, kernels.h:216-219)
    def quant_gemv(self, segs, TB=1):
        arr, n = _pack(segs)
        s0 = segs[0] if not isinstance(segs, gemv_seg) else segs
        self.lib.check(self.lib.quant_gemv(self._s(), arr, n, TB, _ptr(s0.x8), _ptr(s0.xmeta), _ptr(s0.xsumq)))

    def quant_gemv_ex(self, segs, TB=1, prequantized=False, peers=None, next_act=None, sync=None, wait=False,
                      signal=False, norm=None, argmax=None):
        """quant_gemv with options: `prequantized` skips the quantizer (the segments' scratch holds
        the activation already); `peers` scatters the outputs; `next_act` = (x8, xmeta, xsumq) makes
        the call emit its output (gate|up: silu(gate)*up) quantized as the following call's activation;
        `sync` = (flag pointer array, world, rank) with `wait` / `signal` folds the cross-GPU flag
        exchange of a row-sharded call into the launch; `norm` = (weight, eps) folds the RMSNorm of
        the activation into the call's quantizer; `argmax` = (idx, val or None) also leaves the row
        index of the largest output (lowest among equals): the LM head of a greedy step."""
        from .capi import ArgmaxOut, CallOpts, NextAct, Norm, PeerSync, OPT_PREQUANTIZED, OPT_SIGNAL_PEERS, OPT_WAIT_PEERS
        arr, n = _pack(segs)
        s0 = segs[0]
        opts = CallOpts()
        opts.flags = (OPT_PREQUANTIZED if prequantized else 0) | (OPT_WAIT_PEERS if wait else 0) | \
            (OPT_SIGNAL_PEERS if signal else 0)
        keep = []
        if peers is not None:
            opts.peers = C.pointer(peers)
        if next_act is not None:
            na = NextAct(_ptr(next_act[0]), _ptr(next_act[1]), _ptr(next_act[2]))
            keep.append(na)
            opts.next = C.pointer(na)
        if argmax is not None:
            am = ArgmaxOut(_ptr(argmax[0]), _ptr(argmax[1]))
            keep.append(am)
            opts.argmax = C.pointer(am)
        if norm is not None:
            nm = Norm(_ptr(norm[0]), float(norm[1]))
            keep.append(nm)
            opts.norm = C.pointer(nm)
        if sync is not None:
            ps = PeerSync(C.cast(sync[0], C.POINTER(C.c_void_p)), sync[1], sync[2])
            keep.append(ps)
            opts.sync = C.pointer(ps)
        self.lib.check(self.lib.quant_gemv_ex(self._s(), arr, n, TB, _ptr(s0.x8), _ptr(s0.xmeta), _ptr(s0.xsumq),
                                              C.byref(opts)))

    def quant_gemv_chain(self, calls):
        """Several dependent one-token calls as one launch where the kernels allow it (same results
        as quant_gemv_ex call by call).  `calls`: a list of (segs, prequantized, next_act)."""
        from .capi import ChainCall, NextAct, OPT_PREQUANTIZED
        arr = (ChainCall * len(calls))()
        keep = []
        for cc, (segs, prequantized, next_act) in zip(arr, calls):
            sa, n = _pack(segs)
            keep.append(sa)
            s0 = segs[0]
            cc.segs, cc.n_segs = sa, n
            cc.x8, cc.xmeta, cc.xsumq = _ptr(s0.x8), _ptr(s0.xmeta), _ptr(s0.xsumq)
            cc.flags = OPT_PREQUANTIZED if prequantized else 0
            if next_act is not None:
                na = NextAct(_ptr(next_act[0]), _ptr(next_act[1]), _ptr(next_act[2]))
                keep.append(na)
                cc.next = C.pointer(na)
        self.lib.check(self.lib.quant_gemv_chain(self._s(), arr, len(calls)))

    # compute_backend::mtp_argmax (backend.h:47-48)
    def mtp_argmax(self, logits, n, out_idx, out_val, M):
        self.lib.check(self.lib.argmax(self._s(), _ptr(logits), n, _ptr(out_idx), _ptr(out_val), M))

    def quant_gemv_scatter(self, segs, TB, peers):
        """quant_gemv whose outputs are also stored into the peers' copies of the output arena."""
        arr, n = _pack(segs)
        s0 = segs[0]
        self.lib.check(self.lib.quant_gemv_scatter(self._s(), arr, n, TB, _ptr(s0.x8), _ptr(s0.xmeta), _ptr(s0.xsumq),
                                                   C.byref(peers)))

    def peer_barrier(self, flag_ptrs, world, rank, seq):
        """Signal every peer that this rank's stores are done and wait for theirs (bounded)."""
        self.lib.check(self.lib.peer_barrier(self._s(), flag_ptrs, world, rank, seq))

    def quant_gemv_static(self, segs):
        """One-token quant_gemv on the library's built-in scratch: for hosts that cannot
        allocate the activation scratch themselves (K <= 32768; calls must not overlap)."""
        arr, n = _pack(segs)
        self.lib.check(self.lib.quant_gemv_static(self._s(), arr, n))

    # parity instrument (no reference operator: the reference never exposes these sums)
    def i8_block_dots(self, w, type, K, n_rows, x8, TB, t, wd):
        self.lib.check(self.lib.i8_block_dots(self._s(), _ptr(w), type, K, n_rows, _ptr(x8), TB, t, _ptr(wd)))

    def device_status(self, clear=True):
        """Error word set by a kernel whose bounded wait ran out (0 = none)."""
        st = C.c_int(0)
        self.lib.check(self.lib.device_status(C.byref(st), 1 if clear else 0))
        return st.value

    # compute_backend::synchronize (backend.h:123): must truly block
    def synchronize(self):
        self.lib.check(self.lib.synchronize(self._s()))


def make_cuda_backend(device=0, stream=None):
    """Counterpart of make_gpu_backend(queue&) (backend.h:126)."""
    return cuda_backend(device, stream)


def alloc_act(TB, K, device="cuda"):
    """Caller-owned quantized-activation scratch of one call (x8, xmeta, xsumq)."""
    G = K // 32
    return (torch.empty(G * TB * 32, dtype=torch.int8, device=device),
            torch.empty(G * TB * 2, dtype=torch.float32, device=device),
            torch.empty(G * TB * 2, dtype=torch.int32, device=device))
