"""Build ``libpf_refpath.so``: the reference's transfer path restated for timing (ref_path.cu).

TEST / BENCHMARK INFRASTRUCTURE ONLY.

Two flavours:

* ``oracle/_ref/libpf_refpath.so`` — when the reference checkout is present
  (``PEGAFLOW_REFERENCE``, default: a ``reference`` directory beside this repository): the reference's only CUDA kernel, which it
  keeps as a source string inside ``pegaflow-core/src/transfer/kernel.rs`` and compiles with
  NVRTC at run time, is extracted from where it lies, compiled unchanged into the library, and
  the extracted text is deleted again.  Only the binary stays (``oracle/_ref/`` is git-ignored).
* ``oracle/libpf_refpath.so`` — without the checkout: the direct (memcpy loop) path only.

The rest of the reference is Rust (cudarc, tokio, tonic); there is no Rust toolchain in this
image and the crates are not vendored, so nothing else of it can be compiled here.
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("PEGAFLOW_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
KERNEL_RS = os.path.join(REF, "pegaflow-core", "src", "transfer", "kernel.rs")
REF_DIR = os.path.join(HERE, "_ref")
LIB_WITH_KERNEL = os.path.join(REF_DIR, "libpf_refpath.so")
LIB_PORT_ONLY = os.path.join(HERE, "libpf_refpath.so")


def _nvcc():
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _compile(out, extra):
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
           "-I", HERE, "-o", out, os.path.join(HERE, "ref_path.cu"), os.path.join(HERE, "pf_oracle.c"), "-lpthread"] + extra
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout)


def lib_path():
    """The library to load: the one carrying the reference's kernel when it was built."""
    if os.path.exists(LIB_WITH_KERNEL):
        return LIB_WITH_KERNEL
    if os.path.exists(LIB_PORT_ONLY):
        return LIB_PORT_ONLY
    return None


def build(force: bool = False) -> str:
    srcs = [os.path.join(HERE, f) for f in ("ref_path.cu", "pf_oracle.c", "pf_oracle.h")]
    newest = max(os.path.getmtime(p) for p in srcs)
    if os.path.exists(KERNEL_RS):
        if not force and os.path.exists(LIB_WITH_KERNEL) and os.path.getmtime(LIB_WITH_KERNEL) >= newest:
            return LIB_WITH_KERNEL
        text = open(KERNEL_RS).read()
        m = re.search(r'const KERNEL_SRC: &str = r#"(.*?)"#;', text, re.S)
        if not m:
            raise RuntimeError("could not find KERNEL_SRC in " + KERNEL_RS)
        os.makedirs(REF_DIR, exist_ok=True)
        inc = os.path.join(REF_DIR, "pega_batch_copy.inc")
        with open(inc, "w") as f:
            f.write(m.group(1))
        try:
            _compile(LIB_WITH_KERNEL, ['-DPF_REF_KERNEL_INC="%s"' % inc])
        finally:
            os.remove(inc)
        return LIB_WITH_KERNEL
    existing = lib_path()
    if existing and not force and os.path.getmtime(existing) >= newest:
        return existing
    if existing == LIB_WITH_KERNEL and not force:
        return existing  # prebuilt with the reference's kernel; sources are not available to rebuild it
    _compile(LIB_PORT_ONLY, [])
    return LIB_PORT_ONLY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
