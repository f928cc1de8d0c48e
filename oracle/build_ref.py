"""Builds oracle/_ref/libref_kernels.so: the reference's own device kernels behind C entry points (test
infrastructure; see ref_wrap.cu).  Needs the reference checkout and nvcc; where either is missing the function
returns None and the GPU tests that use the library skip.

    python oracle/build_ref.py path/to/reference      (or QW3_REFERENCE_DIR=path/to/reference)

The reference is one file, Inference.cu.  Only its first 292 lines (includes, constants, macros and the six
kernels) compile with this toolkit; they are cut into a temporary file, compiled together with ref_wrap.cu, and
the temporary file is deleted.  Nothing of the reference is written into the repository."""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "libref_kernels.so")
PREFIX_LINES = 292   # up to, not including, readBinaryFileToDevice (Inference.cu:297)


def build(reference_dir=None, force=False):
    """reference_dir: the reference checkout (default: $QW3_REFERENCE_DIR, else a directory `reference` beside this
    repository).  Returns the library path, or None when neither the checkout nor a prebuilt library is there."""
    if reference_dir is None:
        reference_dir = os.environ.get("QW3_REFERENCE_DIR") or os.path.join(HERE, "..", "..", "reference")
    src = os.path.join(reference_dir, "Inference.cu")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(src) or not os.path.exists(nvcc):
        return OUT if os.path.exists(OUT) else None
    wrap = os.path.join(HERE, "ref_wrap.cu")
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= max(os.path.getmtime(src), os.path.getmtime(wrap)):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        prefix = os.path.join(tmp, "reference_kernels_prefix.cu")
        with open(src) as f, open(prefix, "w") as g:
            for i, line in enumerate(f):
                if i >= PREFIX_LINES:
                    break
                g.write(line)
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
               "-diag-suppress", "177", f'-DQW3_REF_PREFIX="{prefix}"', wrap, "-o", OUT, "-lcublas"]
        subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), force=True))
