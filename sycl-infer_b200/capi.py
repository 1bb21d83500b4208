"""ctypes binding of libb200q.so (the C ABI declared in include/b200q.h).

There is no fallback: if the library is missing or fails to load, importing code gets
an exception that says how to build it.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# B200Q_LIB selects another build of the same library (bench_trace.py loads one compiled with
# -DB200Q_TUNING, whose kernels record timeline stamps); the default is the in-tree product build.
LIB_PATH = os.environ.get("B200Q_LIB") or os.path.join(HERE, "libb200q.so")

_vp = C.c_void_p
OK, EINVAL, EUNSUPPORTED, ECUDA, ETIMEOUT = 0, 1, 2, 3, 4
MAX_SEGS = 8


class B200QError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"b200q status {code}: {msg}")
        self.code = code


class Peers(C.Structure):
    """struct b200q_peers."""
    _fields_ = [("n_peers", C.c_int32), ("out_delta", C.c_int64 * 7)]


class NextAct(C.Structure):
    """struct b200q_next_act."""
    _fields_ = [("x8", _vp), ("xmeta", _vp), ("xsumq", _vp)]


class PeerSync(C.Structure):
    """struct b200q_peer_sync."""
    _fields_ = [("flags", C.POINTER(_vp)), ("world", C.c_int32), ("rank", C.c_int32)]


class Norm(C.Structure):
    """struct b200q_norm."""
    _fields_ = [("weight", _vp), ("eps", C.c_float)]


class ArgmaxOut(C.Structure):
    """struct b200q_argmax_out."""
    _fields_ = [("idx", _vp), ("val", _vp)]


class CallOpts(C.Structure):
    """struct b200q_call_opts."""
    _fields_ = [("flags", C.c_uint32), ("peers", C.POINTER(Peers)), ("next", C.POINTER(NextAct)),
                ("sync", C.POINTER(PeerSync)), ("norm", C.POINTER(Norm)), ("argmax", C.POINTER(ArgmaxOut))]


OPT_PREQUANTIZED, OPT_WAIT_PEERS, OPT_SIGNAL_PEERS = 1, 2, 4


class Seg(C.Structure):
    """struct b200q_seg, field for field."""
    _fields_ = [("w", _vp), ("type", C.c_uint32), ("K", C.c_int32), ("n_rows", C.c_int32), ("x", _vp),
                ("x_stride", C.c_int32), ("act_up", _vp), ("out", _vp), ("out_stride", C.c_int32),
                ("residual", _vp), ("alpha", C.c_float), ("x8", _vp), ("xmeta", _vp), ("xsumq", _vp)]


class ChainCall(C.Structure):
    """struct b200q_chain_call."""
    _fields_ = [("segs", C.POINTER(Seg)), ("n_segs", C.c_int32), ("x8", _vp), ("xmeta", _vp), ("xsumq", _vp),
                ("flags", C.c_uint32), ("next", C.POINTER(NextAct))]


class GgufTensor(C.Structure):
    """struct b200q_gguf_tensor."""
    _fields_ = [("name", C.c_char_p), ("type", C.c_uint32), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4),
                ("n_rows", C.c_uint64), ("row_bytes", C.c_uint64), ("nbytes", C.c_uint64), ("blob_offset", C.c_uint64),
                ("shard", C.c_int32), ("host_data", _vp)]


_SIGS = {
    "b200q_last_error": (C.c_char_p, []),
    "b200q_version": (C.c_int, []),
    "b200q_row_bytes": (C.c_size_t, [C.c_uint32, C.c_int64]),
    "b200q_xq": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, _vp, _vp, _vp, C.c_int, C.c_int]),
    "b200q_i8_gemv": (C.c_int, [_vp, C.POINTER(Seg), C.c_int]),
    "b200q_i8_gemm": (C.c_int, [_vp, C.POINTER(Seg), C.c_int, C.c_int]),
    "b200q_quant_gemv": (C.c_int, [_vp, C.POINTER(Seg), C.c_int, C.c_int, _vp, _vp, _vp]),
    "b200q_quant_gemv_ex": (C.c_int, [_vp, C.POINTER(Seg), C.c_int, C.c_int, _vp, _vp, _vp, C.POINTER(CallOpts)]),
    "b200q_quant_gemv_chain": (C.c_int, [_vp, C.POINTER(ChainCall), C.c_int]),
    "b200q_quant_gemv_scatter": (C.c_int, [_vp, C.POINTER(Seg), C.c_int, C.c_int, _vp, _vp, _vp, C.POINTER(Peers)]),
    "b200q_peer_barrier": (C.c_int, [_vp, C.POINTER(_vp), C.c_int, C.c_int, C.c_uint32]),
    "b200q_moe_route": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp]),
    "b200q_moe_route_csr": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp, _vp,
                                      _vp, _vp]),
    "b200q_moe_csr": (C.c_int, [_vp, _vp, C.c_int, C.c_int, _vp, _vp, _vp, _vp]),
    "b200q_moe_gate_up": (C.c_int, [_vp, _vp, _vp, C.c_uint32, C.c_uint32, C.c_size_t, C.c_size_t, _vp, _vp, _vp, _vp,
                                    C.c_int, _vp, _vp, _vp, C.c_int, _vp, C.c_int, C.c_int, C.c_int, C.c_int]),
    "b200q_moe_gate_up_q": (C.c_int, [_vp, _vp, _vp, C.c_uint32, C.c_uint32, C.c_size_t, C.c_size_t, _vp, _vp, _vp, _vp,
                                      C.c_int, _vp, _vp, _vp, C.c_int, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp,
                                      _vp]),
    "b200q_moe_down": (C.c_int, [_vp, _vp, C.c_uint32, C.c_size_t, _vp, _vp, _vp, _vp, C.c_int, _vp, _vp, _vp,
                                 C.c_int, _vp, C.c_int, C.c_int, C.c_int]),
    "b200q_moe_reduce": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, C.c_int]),
    "b200q_quant_gemv_static": (C.c_int, [_vp, C.POINTER(Seg), C.c_int]),
    "b200q_i8_block_dots": (C.c_int, [_vp, _vp, C.c_uint32, C.c_int, C.c_int, _vp, C.c_int, C.c_int, _vp]),
    "b200q_device_status": (C.c_int, [C.POINTER(C.c_int), C.c_int]),
    "b200q_argmax": (C.c_int, [_vp, _vp, C.c_int, _vp, _vp, C.c_int]),
    "b200q_gguf_open": (C.c_int, [C.c_char_p, C.POINTER(_vp)]),
    "b200q_gguf_close": (None, [_vp]),
    "b200q_gguf_n_tensors": (C.c_int, [_vp]),
    "b200q_gguf_n_shards": (C.c_int, [_vp]),
    "b200q_gguf_version": (C.c_uint32, [_vp]),
    "b200q_gguf_tensor_at": (C.c_int, [_vp, C.c_int, C.POINTER(GgufTensor)]),
    "b200q_gguf_find": (C.c_int, [_vp, C.c_char_p]),
    "b200q_gguf_blob_bytes": (C.c_uint64, [_vp]),
    "b200q_gguf_upload": (C.c_int, [_vp, _vp, _vp]),
    "b200q_gguf_meta_type": (C.c_int, [_vp, C.c_char_p]),
    "b200q_gguf_meta_u64": (C.c_int, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "b200q_gguf_meta_f64": (C.c_int, [_vp, C.c_char_p, C.POINTER(C.c_double)]),
    "b200q_gguf_meta_str": (C.c_char_p, [_vp, C.c_char_p]),
    "b200q_gguf_meta_arr": (C.c_int, [_vp, C.c_char_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]),
    "b200q_gguf_meta_arr_str": (C.c_char_p, [_vp, C.c_char_p, C.c_uint64]),
    "b200q_gguf_meta_arr_data": (_vp, [_vp, C.c_char_p]),
    "b200q_probe_hbm_read": (C.c_int, [_vp, _vp, C.c_size_t, _vp]),
    "b200q_probe_i8_mma": (C.c_int, [_vp, C.c_int, _vp]),
    "b200q_synchronize": (C.c_int, [_vp]),
}


class Lib:
    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; "
                              "g.build()'` (needs nvcc); there is no CPU fallback")
        self.path = path
        self.dll = C.CDLL(path)
        for name, (res, args) in _SIGS.items():
            fn = getattr(self.dll, name)
            fn.restype = res
            fn.argtypes = args

    def last_error(self):
        return self.dll.b200q_last_error().decode()

    def check(self, rc):
        if rc != OK:
            raise B200QError(rc, self.last_error())

    def __getattr__(self, name):
        return getattr(self.dll, "b200q_" + name)


_lib = None


def load_lib():
    global _lib
    if _lib is None:
        _lib = Lib()
    return _lib
