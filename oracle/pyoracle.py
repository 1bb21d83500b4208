"""TEST INFRASTRUCTURE ONLY: ctypes bindings of the two CPU checkers.

* ``Oracle``  - liboracle.so, this repository's plain-C restatement (oracle.c).
* ``Ref``     - _ref/libsiref*.so, the reference's own CPU sources compiled
  unmodified behind ref_shim.cpp (present only where it was built).

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this module; the product package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS = 8, 12, 13, 14, 23
TYPES = (Q4_K, Q5_K, Q6_K, Q8_0, IQ4_XS)
TYPE_NAMES = {Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", IQ4_XS: "IQ4_XS"}

_vp = C.c_void_p


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_vp)


def build(ref=True):
    """Compile liboracle.so (and _ref/ when the reference tree is mounted)."""
    subprocess.run(["make", "-s", "-C", HERE, os.path.join(HERE, "liboracle.so")], check=True)
    if ref:
        subprocess.run(["make", "-s", "-C", HERE, "ref"], check=True)


class OrcSeg(C.Structure):
    _fields_ = [("w", _vp), ("type", C.c_uint32), ("K", C.c_int32), ("n_rows", C.c_int32), ("out", _vp),
                ("out_stride", C.c_int32), ("residual", _vp), ("alpha", C.c_float), ("x8", _vp), ("xmeta", _vp),
                ("xsumq", _vp)]


def row_bytes(t, K):
    return {Q4_K: 144, Q5_K: 176, Q6_K: 210, IQ4_XS: 136}[t] * (K // 256) if t != Q8_0 else 34 * (K // 32)


def dots_per_row(t, K):
    return K // 16 if t == Q6_K else K // 32


class Act:
    """Quantized activation of TB tokens (group-major, see orc_xq)."""

    def __init__(self, x8, xmeta, xsumq, TB, K):
        self.x8, self.xmeta, self.xsumq, self.TB, self.K = x8, xmeta, xsumq, TB, K


def _alloc_act(TB, K):
    G = K // 32
    return Act(np.zeros(G * TB * 32, np.int8), np.zeros(G * TB * 2, np.float32), np.zeros(G * TB * 2, np.int32), TB, K)


class Oracle:
    def __init__(self, path=None):
        path = path or os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build(ref=False)
        L = self.L = C.CDLL(path)
        L.orc_f2h.restype = C.c_uint16
        L.orc_f2h.argtypes = [C.c_float]
        L.orc_h2f.restype = C.c_float
        L.orc_h2f.argtypes = [C.c_uint16]
        L.orc_row_bytes.restype = C.c_size_t
        L.orc_row_bytes.argtypes = [C.c_uint32, C.c_int64]
        L.orc_dequantize_row.argtypes = [C.c_uint32, _vp, _vp, C.c_int64]
        L.orc_xq.argtypes = [_vp, _vp, C.c_int, C.c_int, _vp, _vp, _vp, C.c_int, C.c_int]
        L.orc_rmsnorm.argtypes = [_vp, _vp, _vp, C.c_int, C.c_float, C.c_int]
        L.orc_block_dots.argtypes = [C.c_uint32, _vp, C.c_int, C.c_int, _vp, C.c_int, C.c_int, _vp]
        L.orc_i8_gemm.argtypes = [C.POINTER(OrcSeg), C.c_int]
        L.orc_i8_gemm_abs.argtypes = [C.POINTER(OrcSeg), C.c_int, _vp]
        L.orc_moe_route.argtypes = [_vp, C.c_int, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp]
        L.orc_moe_route_logits.argtypes = [C.c_int, C.c_int, C.c_int, _vp, _vp, _vp]
        L.orc_moe_experts_i8.argtypes = [_vp, _vp, _vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_size_t, C.c_size_t,
                                         C.c_size_t, C.c_int, C.c_int, _vp, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp,
                                         C.c_int]
        L.orc_moe_reduce.argtypes = [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, C.c_int]

    def f2h(self, f):
        return int(self.L.orc_f2h(float(f)))

    def h2f(self, h):
        return float(self.L.orc_h2f(int(h)))

    def dequantize(self, t, w, n_rows, K):
        y = np.zeros(n_rows * K, np.float32)
        self.L.orc_dequantize_row(t, _p(w), _p(y), n_rows * K)
        return y.reshape(n_rows, K)

    def rmsnorm(self, x, w, eps, lanes=16):
        """One row; lanes 1 / 8 / 16 = the reference's portable, AVX2 or AVX-512 order of the sum of squares."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1)
        w = np.ascontiguousarray(w, np.float32).reshape(-1)
        out = np.zeros_like(x)
        self.L.orc_rmsnorm(_p(x), _p(w), _p(out), x.size, float(eps), int(lanes))
        return out

    def xq(self, x, up=None, TB=1, K=None):
        x = np.ascontiguousarray(x, np.float32).reshape(TB, -1)
        K = K or x.shape[1]
        a = _alloc_act(TB, K)
        upc = None if up is None else np.ascontiguousarray(up, np.float32).reshape(TB, -1)
        self.L.orc_xq(_p(x), _p(upc), x.shape[1], 0 if upc is None else upc.shape[1], _p(a.x8), _p(a.xmeta),
                      _p(a.xsumq), TB, K)
        return a

    def block_dots(self, t, w, K, n_rows, act, tok=0):
        wd = np.zeros((n_rows, dots_per_row(t, K)), np.int32)
        self.L.orc_block_dots(t, _p(w), K, n_rows, _p(act.x8), act.TB, tok, _p(wd))
        return wd

    def _seg(self, t, w, K, n_rows, act, out, out_stride, residual, alpha):
        return OrcSeg(_p(w), t, K, n_rows, _p(out), out_stride, _p(residual), alpha, _p(act.x8), _p(act.xmeta),
                      _p(act.xsumq))

    def gemm(self, t, w, K, n_rows, act, residual=None, alpha=1.0, out_stride=None):
        """out[t*out_stride + row]; TB == 1 is the GEMV."""
        TB = act.TB
        out_stride = out_stride or n_rows
        out = np.zeros(TB * out_stride, np.float32)
        s = self._seg(t, w, K, n_rows, act, out, out_stride, residual, alpha)
        self.L.orc_i8_gemm(C.byref(s), TB)
        return out.reshape(TB, out_stride)

    def gemm_abs(self, t, w, K, n_rows, act, alpha=1.0):
        TB = act.TB
        ab = np.zeros(TB * n_rows, np.float64)
        s = self._seg(t, w, K, n_rows, act, None, n_rows, None, alpha)
        self.L.orc_i8_gemm_abs(C.byref(s), TB, _p(ab))
        return ab.reshape(TB, n_rows)

    def moe_route(self, x, gate_inp, top_k):
        n_tok, n_embd = x.shape
        n_expert = gate_inp.shape[0]
        logits = np.zeros((n_tok, n_expert), np.float32)
        ids = np.zeros((n_tok, top_k), np.int32)
        wts = np.zeros((n_tok, top_k), np.float32)
        self.L.orc_moe_route(_p(x), n_embd, _p(gate_inp), n_tok, n_embd, n_expert, top_k, _p(logits), _p(ids),
                             _p(wts))
        return logits, ids, wts

    def moe_route_logits(self, logits, top_k):
        p = np.array(logits, np.float32, copy=True)
        n_tok, n_expert = p.shape
        ids = np.zeros((n_tok, top_k), np.int32)
        wts = np.zeros((n_tok, top_k), np.float32)
        self.L.orc_moe_route_logits(n_tok, n_expert, top_k, _p(p), _p(ids), _p(wts))
        return p, ids, wts

    def moe_experts(self, gate, up, down, types, n_embd, n_ff, x, ids):
        n_tok, top_k = ids.shape
        gt, ut, dt = types
        gp, upb, dp = row_bytes(gt, n_embd) * n_ff, row_bytes(ut, n_embd) * n_ff, row_bytes(dt, n_ff) * n_embd
        h = np.zeros((n_tok * top_k, n_ff), np.float32)
        acc = np.zeros((n_tok * top_k, n_embd), np.float32)
        xx = np.ascontiguousarray(x, np.float32)
        self.L.orc_moe_experts_i8(_p(gate), _p(up), _p(down), gt, ut, dt, gp, upb, dp, n_embd, n_ff, _p(xx), n_embd,
                                  n_tok, top_k, _p(np.ascontiguousarray(ids, np.int32)), _p(h), _p(acc), n_embd)
        return h, acc

    def moe_reduce(self, acc, wts, out):
        n_tok, top_k = wts.shape
        n_embd = out.shape[1]
        o = np.array(out, np.float32, copy=True)
        self.L.orc_moe_reduce(_p(acc), _p(np.ascontiguousarray(wts, np.float32)), top_k, n_tok, n_embd, acc.shape[1],
                              _p(o), n_embd)
        return o


class Ref:
    """The reference's own compiled CPU path.  `strict=True` loads the build with
    -ffp-contract=off (the fp32 order the C restatement reproduces bit for bit)."""

    @staticmethod
    def available(strict=False):
        return os.path.exists(os.path.join(HERE, "_ref", "libsiref_nofma.so" if strict else "libsiref.so"))

    def __init__(self, strict=False):
        L = self.L = C.CDLL(os.path.join(HERE, "_ref", "libsiref_nofma.so" if strict else "libsiref.so"))
        L.siref_threads.restype = C.c_int
        L.siref_set_threads.argtypes = [C.c_int]
        L.siref_f2h.restype = C.c_uint16
        L.siref_f2h.argtypes = [C.c_float]
        if hasattr(L, "siref_rmsnorm_row"):  # builds of the shim made before it forwarded this
            L.siref_isa.restype = C.c_int
            L.siref_rmsnorm_row.argtypes = [_vp, _vp, _vp, C.c_int, C.c_float]
        L.siref_h2f.restype = C.c_float
        L.siref_h2f.argtypes = [C.c_uint16]
        L.siref_row_bytes.restype = C.c_uint64
        L.siref_row_bytes.argtypes = [C.c_uint32, C.c_int64]
        L.siref_dequantize_row.argtypes = [C.c_uint32, _vp, _vp, C.c_int64]
        L.siref_xq.argtypes = [_vp, _vp, C.c_int, C.c_int, _vp, _vp, _vp, C.c_int, C.c_int]
        L.siref_i8_gemv.argtypes = [_vp, C.c_uint32, C.c_int, C.c_int, _vp, _vp, C.c_float, _vp, _vp, _vp]
        L.siref_i8_gemv1_chunked.argtypes = [_vp, C.c_uint32, C.c_int, C.c_int, _vp, _vp, C.c_float, _vp, _vp, _vp,
                                             C.c_int]
        L.siref_i8_gemm.argtypes = [_vp, C.c_uint32, C.c_int, C.c_int, _vp, C.c_int, _vp, C.c_float, _vp, _vp, _vp,
                                    C.c_int]
        L.siref_i8_expert_gemm.argtypes = [C.c_uint32, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp, C.c_int]
        L.siref_gemv_f32.argtypes = [_vp, C.c_uint32, C.c_int, C.c_int, _vp, C.c_int, _vp, _vp, C.c_int, _vp,
                                     C.c_float, C.c_int]
        L.siref_q8_0_down_grouped.argtypes = [_vp, C.c_uint64, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int,
                                              _vp, C.c_int]
        L.siref_moe_route.argtypes = [_vp, C.c_int, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp]
        L.siref_moe_experts_i8_q8down.argtypes = [_vp, _vp, _vp, C.c_uint32, C.c_uint64, C.c_uint64, C.c_uint64,
                                                  C.c_int, C.c_int, C.c_int, _vp, C.c_int, _vp, _vp, C.c_int]
        L.siref_moe_reduce.argtypes = [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, C.c_int]
        L.siref_silu.restype = C.c_float
        L.siref_silu.argtypes = [C.c_float]

    def threads(self):
        return int(self.L.siref_threads())

    def isa_lanes(self):
        """Accumulators of the sum-of-squares helper this host selects: 1, 8 or 16."""
        return {0: 1, 1: 8, 2: 16}[int(self.L.siref_isa())]

    def rmsnorm(self, x, w, eps):
        x = np.ascontiguousarray(x, np.float32).reshape(-1)
        w = np.ascontiguousarray(w, np.float32).reshape(-1)
        out = np.zeros_like(x)
        self.L.siref_rmsnorm_row(_p(x), _p(w), _p(out), x.size, float(eps))
        return out

    def f2h(self, f):
        return int(self.L.siref_f2h(float(f)))

    def h2f(self, h):
        return float(self.L.siref_h2f(int(h)))

    def row_bytes(self, t, K):
        return int(self.L.siref_row_bytes(t, K))

    def dequantize(self, t, w, n_rows, K):
        y = np.zeros(n_rows * K, np.float32)
        self.L.siref_dequantize_row(t, _p(w), _p(y), n_rows * K)
        return y.reshape(n_rows, K)

    def xq(self, x, up=None, TB=1, K=None):
        x = np.ascontiguousarray(x, np.float32).reshape(TB, -1)
        K = K or x.shape[1]
        a = _alloc_act(TB, K)
        upc = None if up is None else np.ascontiguousarray(up, np.float32).reshape(TB, -1)
        self.L.siref_xq(_p(x), _p(upc), x.shape[1], 0 if upc is None else upc.shape[1], _p(a.x8), _p(a.xmeta),
                        _p(a.xsumq), TB, K)
        return a

    def gemv(self, t, w, K, n_rows, act, residual=None, alpha=1.0, chunks=0):
        out = np.zeros(n_rows, np.float32)
        if chunks:
            self.L.siref_i8_gemv1_chunked(_p(w), t, K, n_rows, _p(out), _p(residual), alpha, _p(act.x8),
                                          _p(act.xmeta), _p(act.xsumq), chunks)
        else:
            self.L.siref_i8_gemv(_p(w), t, K, n_rows, _p(out), _p(residual), alpha, _p(act.x8), _p(act.xmeta),
                                 _p(act.xsumq))
        return out

    def gemm(self, t, w, K, n_rows, act, residual=None, alpha=1.0, out_stride=None):
        TB = act.TB
        out_stride = out_stride or n_rows
        out = np.zeros(TB * out_stride, np.float32)
        self.L.siref_i8_gemm(_p(w), t, K, n_rows, _p(out), out_stride, _p(residual), alpha, _p(act.x8),
                             _p(act.xmeta), _p(act.xsumq), TB)
        return out.reshape(TB, out_stride)

    def expert_gemm(self, t, w, K, n_rows, act):
        out = np.zeros((act.TB, n_rows), np.float32)
        self.L.siref_i8_expert_gemm(t, _p(w), _p(act.x8), _p(act.xmeta), _p(act.xsumq), K, n_rows, act.TB, _p(out),
                                    n_rows)
        return out

    def gemv_f32(self, t, w, K, n_rows, x, act_up=None, residual=None, alpha=1.0):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
        TB = x.shape[0]
        out = np.zeros((TB, n_rows), np.float32)
        self.L.siref_gemv_f32(_p(w), t, K, n_rows, _p(x), K, _p(act_up), _p(out), n_rows, _p(residual), alpha, TB)
        return out

    def q8_0_down(self, w, K, n_rows, act):
        acc = np.zeros((act.TB, n_rows), np.float32)
        self.L.siref_q8_0_down_grouped(_p(w), row_bytes(Q8_0, K), _p(act.x8), _p(act.xmeta), _p(act.xsumq), act.TB,
                                       act.TB, n_rows, K, _p(acc), n_rows)
        return acc

    def moe_route(self, x, gate_inp, top_k):
        n_tok, n_embd = x.shape
        n_expert = gate_inp.shape[0]
        logits = np.zeros((n_tok, n_expert), np.float32)
        ids = np.zeros((n_tok, top_k), np.int32)
        wts = np.zeros((n_tok, top_k), np.float32)
        self.L.siref_moe_route(_p(x), n_embd, _p(gate_inp), n_tok, n_embd, n_expert, top_k, _p(logits), _p(ids),
                               _p(wts))
        return logits, ids, wts

    def moe_experts_q8down(self, gate, up, down, gu_type, n_expert, n_embd, n_ff, x_row, ids_row):
        n_pairs = len(ids_row)
        acc = np.zeros((n_pairs, n_embd), np.float32)
        self.L.siref_moe_experts_i8_q8down(_p(gate), _p(up), _p(down), gu_type, row_bytes(gu_type, n_embd) * n_ff,
                                           row_bytes(Q8_0, n_ff) * n_embd, row_bytes(Q8_0, n_ff), n_expert, n_embd,
                                           n_ff, _p(np.ascontiguousarray(x_row, np.float32)), n_pairs,
                                           _p(np.ascontiguousarray(ids_row, np.int32)), _p(acc), n_embd)
        return acc

    def moe_reduce(self, acc, wts, out):
        n_tok, top_k = wts.shape
        n_embd = out.shape[1]
        o = np.array(out, np.float32, copy=True)
        self.L.siref_moe_reduce(_p(acc), _p(np.ascontiguousarray(wts, np.float32)), top_k, n_tok, n_embd,
                                acc.shape[1], _p(o), n_embd)
        return o
