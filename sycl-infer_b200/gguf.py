"""GGUF files on the input side of the path: a reader over the library's loader (b200q_gguf_*,
csrc/gguf.cu) and a writer for model files made of this repository's synthetic tensors.

The reference maps a model file, binds tensors by name and uploads the whole data section into one
device blob (src/model/gguf.{h,cpp}, src/backend/weight_store.h:28-62); `GgufFile.upload` does the
same into a torch uint8 tensor, and `GgufFile.weight(name)` returns the zero-copy view of a tensor in
that blob, ready to be a `gemv_seg.w`.
"""
import ctypes as C
import struct

import numpy as np

from .capi import GgufTensor, load_lib as load

# GGUF metadata value types
U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q",
        F64: "<d"}


class GgufFile:
    """One model file (all shards of a split one), parsed by the native loader."""

    def __init__(self, path):
        self.lib = load()
        h = C.c_void_p()
        self.lib.check(self.lib.gguf_open(str(path).encode(), C.byref(h)))
        self.h = h
        self.tensors = {}
        for i in range(self.lib.gguf_n_tensors(h)):
            t = GgufTensor()
            self.lib.check(self.lib.gguf_tensor_at(h, i, C.byref(t)))
            self.tensors[t.name.decode()] = dict(type=int(t.type), dims=tuple(int(d) for d in t.dims[:t.n_dims]),
                                                 n_rows=int(t.n_rows), row_bytes=int(t.row_bytes), nbytes=int(t.nbytes),
                                                 blob_offset=int(t.blob_offset), shard=int(t.shard),
                                                 host_data=int(t.host_data or 0))
        self.blob = None

    @property
    def version(self):
        return int(self.lib.gguf_version(self.h))

    @property
    def n_shards(self):
        return int(self.lib.gguf_n_shards(self.h))

    @property
    def blob_bytes(self):
        return int(self.lib.gguf_blob_bytes(self.h))

    def close(self):
        if self.h:
            self.lib.gguf_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def host_bytes(self, name):
        """The tensor's raw bytes as they lie in the file mapping (a copy)."""
        t = self.tensors[name]
        return np.ctypeslib.as_array((C.c_uint8 * t["nbytes"]).from_address(t["host_data"])).copy()

    def meta(self, key):
        """Metadata value of `key` as a Python value (None when absent)."""
        k = key.encode()
        ty = self.lib.gguf_meta_type(self.h, k)
        if ty < 0:
            return None
        if ty == STR:
            return self.lib.gguf_meta_str(self.h, k).decode()
        if ty == ARR:
            et, n = C.c_uint32(), C.c_uint64()
            self.lib.check(self.lib.gguf_meta_arr(self.h, k, C.byref(et), C.byref(n)))
            if et.value == STR:
                return [self.lib.gguf_meta_arr_str(self.h, k, i).decode() for i in range(n.value)]
            w = struct.calcsize(_FMT[et.value])
            raw = C.string_at(self.lib.gguf_meta_arr_data(self.h, k), w * n.value) if n.value else b""
            return [struct.unpack_from(_FMT[et.value], raw, w * i)[0] for i in range(n.value)]
        if ty in (F32, F64):
            v = C.c_double()
            self.lib.check(self.lib.gguf_meta_f64(self.h, k, C.byref(v)))
            return v.value
        v = C.c_uint64()
        self.lib.check(self.lib.gguf_meta_u64(self.h, k, C.byref(v)))
        if ty in (I8, I16, I32, I64):
            return C.c_int64(v.value).value
        return bool(v.value) if ty == BOOL else v.value

    def upload(self, device="cuda", stream=None):
        """Allocate the device blob (torch uint8) and copy every shard's data section into it."""
        import torch
        self.blob = torch.empty(max(self.blob_bytes, 256), dtype=torch.uint8, device=device)
        s = C.c_void_p(stream.cuda_stream if stream is not None else torch.cuda.current_stream().cuda_stream)
        self.lib.check(self.lib.gguf_upload(self.h, C.c_void_p(self.blob.data_ptr()), s))
        torch.cuda.current_stream().synchronize()
        return self.blob

    def weight(self, name):
        """The tensor as a zero-copy uint8 view of the device blob: a gemv_seg.w (rows of dims[0] values)."""
        t = self.tensors[name]
        return self.blob[t["blob_offset"]:t["blob_offset"] + t["nbytes"]]


# ---- writer -------------------------------------------------------------------------------------
def _pack_str(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _pack_value(ty, v, elem=None):
    if ty == STR:
        return _pack_str(v)
    if ty == ARR:
        out = struct.pack("<IQ", elem, len(v))
        for e in v:
            out += _pack_str(e) if elem == STR else struct.pack(_FMT[elem], e)
        return out
    return struct.pack(_FMT[ty], v)


def _one_file(path, kv, tensors, alignment):
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kv))
    for key, (ty, v, *elem) in kv.items():
        head += _pack_str(key) + struct.pack("<I", ty) + _pack_value(ty, v, elem[0] if elem else None)
    off, offs = 0, []
    for _, _, _, data in tensors:
        offs.append(off)
        off = (off + len(data) + alignment - 1) // alignment * alignment
    for (name, ty, dims, _), o in zip(tensors, offs):
        head += _pack_str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", ty, o)
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for (_, _, _, data), o in zip(tensors, offs):
            f.write(bytes(data))
            f.write(b"\0" * ((-len(data)) % alignment))


def write_gguf(path, kv, tensors, alignment=32, shards=1):
    """Write a GGUF v3 file.  kv: {key: (type, value)} or {key: (ARR, values, elem_type)}; tensors:
    [(name, ggml_type, dims (dims[0] = row length), raw bytes)].  shards > 1 writes a split file
    "<stem>-0000i-of-0000N.gguf" (path must end in .gguf): tensors dealt round-robin, the model's
    metadata in the first shard, split.no / split.count / split.tensors.count in each; returns the
    paths written."""
    kv = dict(kv)
    if alignment != 32:
        kv["general.alignment"] = (U32, alignment)
    if shards == 1:
        _one_file(path, kv, tensors, alignment)
        return [str(path)]
    stem = str(path)[:-5]
    paths = []
    for s in range(shards):
        p = f"{stem}-{s + 1:05d}-of-{shards:05d}.gguf"
        skv = dict(kv) if s == 0 else ({"general.alignment": kv["general.alignment"]} if "general.alignment" in kv else {})
        skv.update({"split.no": (U16, s), "split.count": (U16, shards), "split.tensors.count": (I32, len(tensors))})
        _one_file(p, skv, tensors[s::shards], alignment)
        paths.append(p)
    return paths
