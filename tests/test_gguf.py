"""GGUF files -> tensor table and device blob (b200q_gguf_*).  Files written by this repository's
writer are read back by the library's loader and - where the reference tree was present at build
time - by the reference's own loader (src/model/gguf.cpp, compiled unmodified into
oracle/_ref/libsigguf.so): both must see the same tensors, shapes, types, bytes and metadata.
Malformed files must be refused, not crash."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

import __graft_entry__ as graft

pkg = graft.load_package()
from sycl_infer_b200 import gguf as G  # noqa: E402
from sycl_infer_b200.capi import B200QError  # noqa: E402

REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libsigguf.so")


def model(n_layers=2):
    kv = {"general.architecture": (G.STR, "qwen3"), "general.name": (G.STR, "synthetic"),
          "qwen3.block_count": (G.U32, n_layers), "qwen3.embedding_length": (G.U32, 512),
          "qwen3.attention.layer_norm_rms_epsilon": (G.F32, 1e-6), "qwen3.expert_count": (G.U32, 4),
          "tokenizer.ggml.tokens": (G.ARR, ["<s>", "a", "bc", ""], G.STR),
          "tokenizer.ggml.token_type": (G.ARR, [3, 1, 1, -1], G.I32), "general.file_type": (G.U32, 15),
          "x.flag": (G.BOOL, 1), "x.big": (G.U64, 1 << 40), "x.neg": (G.I64, -5), "x.f64": (G.F64, 0.25)}
    ts = []
    for i in range(n_layers):
        ts.append((f"blk.{i}.attn_q.weight", 12, (512, 8), pkg.synth.make_weight(12, 8, 512, 10 + i).tobytes()))
        ts.append((f"blk.{i}.ffn_down.weight", 14, (256, 6), pkg.synth.make_weight(14, 6, 256, 20 + i).tobytes()))
        ts.append((f"blk.{i}.ffn_gate_exps.weight", 12, (256, 4, 4), pkg.synth.make_weight(12, 16, 256, 30 + i).tobytes()))
        ts.append((f"blk.{i}.attn_norm.weight", 0, (512,), np.arange(512, dtype=np.float32).tobytes()))
    ts.append(("output.weight", 8, (512, 3), pkg.synth.make_weight(8, 3, 512, 40).tobytes()))
    ts.append(("iq.weight", 23, (256, 5), pkg.synth.make_weight(23, 5, 256, 41).tobytes()))
    return kv, ts


class RefGguf:
    def __init__(self, path):
        L = self.L = C.CDLL(REF_LIB)
        L.sigguf_load.restype = C.c_void_p
        L.sigguf_load.argtypes = [C.c_char_p]
        for f in ("sigguf_close", "sigguf_n_tensors", "sigguf_n_shards", "sigguf_version"):
            getattr(L, f).argtypes = [C.c_void_p]
        L.sigguf_version.restype = C.c_uint32
        L.sigguf_tensor.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32),
                                    C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.POINTER(C.c_void_p)]
        for f, rt in (("sigguf_has", C.c_int), ("sigguf_u32", C.c_uint32), ("sigguf_f32", C.c_float), ("sigguf_str", C.c_char_p),
                      ("sigguf_arr_len", C.c_int)):
            getattr(L, f).restype = rt
            getattr(L, f).argtypes = [C.c_void_p, C.c_char_p]
        L.sigguf_arr_str.restype = C.c_char_p
        L.sigguf_arr_str.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        L.sigguf_arr_i64.restype = C.c_longlong
        L.sigguf_arr_i64.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        self.h = L.sigguf_load(str(path).encode())

    def tensors(self):
        out = {}
        for i in range(self.L.sigguf_n_tensors(self.h)):
            buf = C.create_string_buffer(256)
            dims, ty, nd, nb, data = (C.c_uint64 * 4)(), C.c_uint32(), C.c_uint32(), C.c_uint64(), C.c_void_p()
            assert self.L.sigguf_tensor(self.h, i, buf, 256, dims, C.byref(ty), C.byref(nd), C.byref(nb), C.byref(data)) == 0
            raw = np.ctypeslib.as_array((C.c_uint8 * nb.value).from_address(data.value)).copy()
            out[buf.value.decode()] = (ty.value, tuple(dims[:nd.value]), nb.value, raw)
        return out


def check_against_written(F, kv, ts):
    assert set(F.tensors) == {t[0] for t in ts}
    for name, ty, dims, data in ts:
        t = F.tensors[name]
        assert (t["type"], t["dims"], t["nbytes"]) == (ty, tuple(dims), len(data))
        assert t["blob_offset"] % 32 == 0 and t["n_rows"] * t["row_bytes"] == t["nbytes"]
        assert F.host_bytes(name).tobytes() == data
    for key, (ty, v, *_) in kv.items():
        got = F.meta(key)
        if ty in (G.F32,):
            assert got == np.float32(v)
        else:
            assert got == (bool(v) if ty == G.BOOL else v), key
    assert F.meta("no.such.key") is None
    # tensors do not overlap in the blob and fit it
    spans = sorted((t["blob_offset"], t["blob_offset"] + t["nbytes"]) for t in F.tensors.values())
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:])) and spans[-1][1] <= F.blob_bytes


@pytest.mark.parametrize("alignment,shards", [(32, 1), (64, 1), (32, 3), (128, 2)])
def test_round_trip_and_reference_loader(tmp_path, alignment, shards):
    kv, ts = model()
    paths = G.write_gguf(tmp_path / "m.gguf", kv, ts, alignment=alignment, shards=shards)
    F = G.GgufFile(paths[-1])  # any shard of a split file names the whole
    assert F.version == 3 and F.n_shards == shards
    check_against_written(F, kv, ts)
    if shards > 1:
        assert {t["shard"] for t in F.tensors.values()} == set(range(shards))
        assert F.meta("split.count") == shards and F.meta("general.architecture") == "qwen3"
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libsigguf.so not built (reference tree absent)")
    R = RefGguf(paths[0])
    assert R.h, "the reference's loader refused the file"
    rt = R.tensors()
    assert set(rt) == set(F.tensors) and R.L.sigguf_version(R.h) == 3
    for name, (ty, dims, nb, raw) in rt.items():
        t = F.tensors[name]
        assert (ty, dims, nb) == (t["type"], t["dims"], t["nbytes"])
        assert np.array_equal(raw, F.host_bytes(name))
    assert R.L.sigguf_u32(R.h, b"qwen3.block_count") == F.meta("qwen3.block_count")
    assert R.L.sigguf_f32(R.h, b"qwen3.attention.layer_norm_rms_epsilon") == np.float32(F.meta("qwen3.attention.layer_norm_rms_epsilon"))
    assert R.L.sigguf_str(R.h, b"general.architecture").decode() == F.meta("general.architecture")
    n = R.L.sigguf_arr_len(R.h, b"tokenizer.ggml.tokens")
    assert [R.L.sigguf_arr_str(R.h, b"tokenizer.ggml.tokens", i).decode() for i in range(n)] == F.meta("tokenizer.ggml.tokens")
    assert [R.L.sigguf_arr_i64(R.h, b"tokenizer.ggml.token_type", i) for i in range(4)] == F.meta("tokenizer.ggml.token_type")
    R.L.sigguf_close(R.h)


def test_expert_bank_planes(tmp_path):
    """A [K][N][E] bank: plane e starts e * N * row_bytes into the tensor."""
    kv, ts = model(1)
    F = G.GgufFile(G.write_gguf(tmp_path / "e.gguf", kv, ts)[0])
    t = F.tensors["blk.0.ffn_gate_exps.weight"]
    assert t["dims"] == (256, 4, 4) and t["n_rows"] == 16 and t["row_bytes"] == 144
    whole = pkg.synth.make_weight(12, 16, 256, 30)
    plane = t["dims"][1] * t["row_bytes"]
    for e in range(4):
        assert np.array_equal(F.host_bytes("blk.0.ffn_gate_exps.weight")[e * plane:(e + 1) * plane], whole[e * plane:(e + 1) * plane])


def _bytes_of(tmp_path):
    kv, ts = model(1)
    p = G.write_gguf(tmp_path / "ok.gguf", kv, ts)[0]
    return bytearray(open(p, "rb").read())


@pytest.mark.parametrize("case", ["magic", "version", "truncated_header", "truncated_data", "huge_counts", "string_overrun",
                                  "unknown_type", "misaligned_tensor", "short"])
def test_malformed_files_are_refused(tmp_path, case):
    b = _bytes_of(tmp_path)
    if case == "magic":
        b[0:4] = b"GGUX"
    elif case == "version":
        b[4:8] = struct.pack("<I", 9)
    elif case == "truncated_header":
        b = b[:200]
    elif case == "truncated_data":
        b = b[:len(b) - 4096]
    elif case == "huge_counts":
        b[8:16] = struct.pack("<Q", 1 << 60)
    elif case == "string_overrun":
        b[24:32] = struct.pack("<Q", 1 << 50)  # the first key's length
    elif case == "unknown_type":
        i = bytes(b).index(b"iq.weight") + len(b"iq.weight") + 4 + 16
        assert struct.unpack_from("<I", b, i)[0] == 23
        b[i:i + 4] = struct.pack("<I", 77)
    elif case == "misaligned_tensor":
        i = bytes(b).index(b"iq.weight") + len(b"iq.weight") + 4 + 16 + 4
        b[i:i + 8] = struct.pack("<Q", struct.unpack_from("<Q", b, i)[0] + 8)
    elif case == "short":
        b = b[:10]
    p = tmp_path / "bad.gguf"
    p.write_bytes(bytes(b))
    with pytest.raises(B200QError) as ei:
        G.GgufFile(p)
    assert ei.value.code in (1, 2)


def test_missing_shard_is_refused(tmp_path):
    kv, ts = model(1)
    paths = G.write_gguf(tmp_path / "m.gguf", kv, ts, shards=3)
    os.remove(paths[1])
    with pytest.raises(B200QError):
        G.GgufFile(paths[0])


@pytest.mark.gpu
def test_upload_and_gemv_from_the_blob(tmp_path, orc):
    """The device blob holds the tensors byte for byte, and a GEMV on a view of it equals the GEMV
    on the same weight uploaded on its own (zero-copy: the blob IS the weight store)."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from sycl_infer_b200.backend import alloc_act, gemv_seg
    be = pkg.make_cuda_backend(0)
    kv, ts = model(2)
    F = G.GgufFile(G.write_gguf(tmp_path / "m.gguf", kv, ts, shards=2)[0])
    F.upload()
    for name, _, _, data in ts:
        assert bytes(F.weight(name).cpu().numpy().tobytes()) == data
    K, N, t = 512, 8, 12
    x = torch.from_numpy(pkg.synth.make_activation(1, K, 99)).cuda()
    outs = []
    for w in (F.weight("blk.1.attn_q.weight"), torch.from_numpy(pkg.synth.make_weight(12, 8, 512, 11)).cuda()):
        x8, xm, xs = alloc_act(1, K)
        out = torch.zeros(N, device="cuda")
        be.quant_gemv([gemv_seg(w=w, type=t, K=K, n_rows=N, x=x, x_stride=K, out=out, out_stride=N, x8=x8, xmeta=xm, xsumq=xs)], 1)
        be.synchronize()
        outs.append(out.cpu().numpy())
    assert np.array_equal(outs[0], outs[1]) and be.device_status() == 0
    a = orc.xq(x.cpu().numpy())
    wn = pkg.synth.make_weight(12, 8, 512, 11)
    ref, ab = orc.gemm(t, wn, K, N, a), orc.gemm_abs(t, wn, K, N, a)
    assert float(np.max(np.abs(outs[0] - ref[0]) / ab[0])) <= 1e-5
