"""In-tree build of libb200q.so with nvcc for sm_100a (no JIT cache, no torch headers)."""
import hashlib
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200q.so")
STAMP = os.path.join(HERE, "build", "libb200q.stamp")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libb200q.so")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest():
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    inc = os.path.join(HERE, "..", "include", "b200q.h")
    for f in sorted(os.listdir(CSRC)):
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode() + fh.read())
    with open(inc, "rb") as fh:
        h.update(fh.read())
    return h.hexdigest()


def build_native(force=False, verbose=False, extra=(), out=None):
    """Compile every .cu under csrc/ into libb200q.so; skipped when sources are unchanged.
    `out` builds a variant (e.g. with -DB200Q_TUNING in `extra`) under another name."""
    lib = out or LIB
    stamp = STAMP if out is None else os.path.join(HERE, "build", os.path.basename(out) + ".stamp")
    dig = _digest() + " ".join(extra)
    if not force and os.path.exists(lib) and os.path.exists(stamp) and open(stamp).read() == dig:
        return lib
    os.makedirs(os.path.dirname(stamp), exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-o", lib, *sources()]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    with open(stamp, "w") as fh:
        fh.write(dig)
    return lib


TUNING_LIB = os.path.join(HERE, "libb200q_tuning.so")


def build_tuning(force=False, verbose=False):
    """The A/B variant (-DB200Q_TUNING: timeline stamps and kernel-selection knobs read from the
    environment) beside the product library; select it with B200Q_LIB=<path>."""
    return build_native(force=force, verbose=verbose, extra=["-DB200Q_TUNING"], out=TUNING_LIB)


if __name__ == "__main__":
    import sys
    if "--tuning" in sys.argv:
        print(build_tuning(force="--force" in sys.argv, verbose=True))
    else:
        build_native(force="--force" in sys.argv, verbose=True,
                     extra=["-Xptxas", "-v"] if "--ptxas" in sys.argv else [])
