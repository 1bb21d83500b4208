"""The C-ABI library loads and exports every entry point include/b200q.h declares.
No compute call is made here (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "b200q.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_the_path():
    syms = declared_symbols()
    for need in ("b200q_xq", "b200q_i8_gemv", "b200q_i8_gemm", "b200q_quant_gemv", "b200q_i8_block_dots",
                 "b200q_synchronize", "b200q_last_error"):
        assert need in syms


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.load_lib()
    for s in declared_symbols():
        assert hasattr(lib.dll, s), f"{s} declared in include/b200q.h but not exported"
    assert lib.dll.b200q_version() == 1


def test_header_is_plain_c_and_structs_match_the_binding(tmp_path, pkg):
    """include/b200q.h compiles as C11 (a host in C, cgo or any FFI generator reads it as such), and
    the struct sizes a C compiler derives from it are the sizes of the ctypes mirrors."""
    import shutil
    import subprocess
    from sycl_infer_b200 import capi
    if not shutil.which("gcc"):
        pytest.skip("no gcc")
    names = [("b200q_seg", capi.Seg), ("b200q_peers", capi.Peers), ("b200q_next_act", capi.NextAct),
             ("b200q_peer_sync", capi.PeerSync), ("b200q_norm", capi.Norm), ("b200q_argmax_out", capi.ArgmaxOut),
             ("b200q_call_opts", capi.CallOpts), ("b200q_chain_call", capi.ChainCall), ("b200q_gguf_tensor", capi.GgufTensor)]
    src = '#include <stdio.h>\n#include "b200q.h"\nint main(void) {\n'
    src += "".join(f'  printf("%zu\\n", sizeof({n}));\n' for n, _ in names) + "  return 0;\n}\n"
    c = tmp_path / "sizes.c"
    c.write_text(src)
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(ROOT, "include"), str(c),
                    "-o", str(exe)], check=True)
    sizes = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    for (n, ct), sz in zip(names, sizes):
        assert ctypes.sizeof(ct) == sz, f"{n}: C says {sz}, the ctypes mirror {ctypes.sizeof(ct)}"


def test_cpp_host_links_against_the_library(tmp_path, pkg):
    """A host written in C++ (the reference's language) links libb200q.so through the header alone and
    gets statuses and messages where the reference throws: no Python, no torch in between."""
    import shutil
    import subprocess
    if not shutil.which("g++"):
        pytest.skip("no g++")
    lib_dir = os.path.dirname(pkg.load_lib().path)
    src = tmp_path / "host.cpp"
    src.write_text('''
#include <cstdio>
#include "b200q.h"
int main() {
    b200q_seg s{};
    s.w = (const void *)0x1000; s.type = B200Q_Q4_K; s.K = 300; s.n_rows = 4; s.out = (float *)0x2000; s.out_stride = 4;
    const int rc = b200q_i8_gemv(nullptr, &s, 1);
    std::printf("%d|%s|%zu|%d\\n", rc, b200q_last_error(), b200q_row_bytes(B200Q_Q6_K, 4096), b200q_version());
    b200q_gguf * g = nullptr;
    std::printf("%d|%d\\n", b200q_gguf_open("/no/such/file.gguf", &g), g == nullptr);
    return 0;
}
''')
    exe = tmp_path / "host"
    subprocess.run(["g++", "-std=c++17", "-Wall", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe), "-L", lib_dir,
                    "-lb200q", f"-Wl,-rpath,{lib_dir}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines()
    assert out[0] == "1|K must be a positive multiple of 256 (got 300)|3360|1"
    assert out[1] == "1|1"


def test_row_bytes_table(pkg, po):
    # quant_row_bytes of the reference (src/common/quant.h:1177-1198; tests/model/test_quant_synth.cpp:106-111)
    lib = pkg.load_lib()
    for t, per256 in ((12, 144), (13, 176), (14, 210), (8, 272), (23, 136)):
        assert lib.dll.b200q_row_bytes(t, 4096) == per256 * 16 == po.row_bytes(t, 4096)
    assert lib.dll.b200q_row_bytes(2, 4096) == 0


def test_argument_errors_need_no_gpu(pkg):
    """Validation happens before any CUDA call and reports through status + last_error."""
    from sycl_infer_b200.capi import Seg, EINVAL, EUNSUPPORTED
    lib = pkg.load_lib()
    seg = (Seg * 1)(Seg(0x1000, 12, 300, 4, None, 0, None, 0x2000, 4, None, 1.0, 0x3000, 0x4000, 0x5000))
    assert lib.dll.b200q_i8_gemv(None, seg, 1) == EINVAL and "multiple of 256" in lib.last_error()
    seg[0].K = 512
    seg[0].type = 2
    assert lib.dll.b200q_i8_gemv(None, seg, 1) == EUNSUPPORTED and "unsupported ggml type" in lib.last_error()
    seg[0].type = 12
    seg[0].w = 0x1001
    assert lib.dll.b200q_i8_gemv(None, seg, 1) == EINVAL and "16-byte aligned" in lib.last_error()
    assert lib.dll.b200q_i8_gemv(None, seg, 0) == EINVAL
    assert lib.dll.b200q_xq(None, None, None, 0, 0, None, None, None, 1, 256) == EINVAL


def test_no_cpu_fallback_without_device(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(RuntimeError):
        pkg.make_cuda_backend(0)
