"""Builds oracle/_ref/libbruce_ref.so: the reference engine's own kernels behind a small C harness
(oracle/ref_harness.cu), for tests that pin this repository against the reference itself.

Only possible where the reference tree is mounted (REF_ROOT); elsewhere the prebuilt library is used
if present and the tests that need it are skipped if not.  The reference sources are compiled where
they lie, through a temporary copy that receives one portability fix (its JSON value type lacks a
`long long` constructor, which gcc on LP64 needs: engine/src/json.h:30-36 vs server.h:808 ff.);
nothing is written into the repository except the built library under oracle/_ref/.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference tree: BRUCE_REFERENCE_ROOT, else a checkout named "reference" beside this repository
REF_ROOT = os.environ.get("BRUCE_REFERENCE_ROOT",
                          os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
OUT = os.path.join(HERE, "_ref", "libbruce_ref.so")
HARNESS = os.path.join(HERE, "ref_harness.cu")


def available() -> bool:
    return os.path.exists(OUT)


def build_if_possible(force: bool = False, verbose: bool = False):
    src = os.path.join(REF_ROOT, "engine", "src")
    if not os.path.exists(os.path.join(src, "bruce.cu")):
        return OUT if available() else None
    if not force and available() and os.path.getmtime(OUT) >= os.path.getmtime(HARNESS):
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="bruce_ref_") as tmp:
        for f in os.listdir(src):
            shutil.copy(os.path.join(src, f), os.path.join(tmp, f))
            os.chmod(os.path.join(tmp, f), 0o644)
        jp = os.path.join(tmp, "json.h")
        text = open(jp).read()
        anchor = "Value(int64_t v) : type(Type::Number), number((double)v) {}"
        if anchor not in text:
            raise RuntimeError("json.h changed: portability patch does not apply")
        text = text.replace(anchor, anchor + "\n    Value(long long v) : type(Type::Number), number((double)v) {}")
        open(jp, "w").write(text)
        cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC,-O2",
               "-shared", "-I", tmp, "-o", OUT, HARNESS, os.path.join(tmp, "unicode.cpp"),
               os.path.join(tmp, "unicode-data.cpp")]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if verbose or res.returncode:
            sys.stderr.write(res.stdout[-4000:])
        if res.returncode:
            raise RuntimeError("building the reference harness failed")
    return OUT


if __name__ == "__main__":
    print(build_if_possible(force="--force" in sys.argv, verbose=True))
