"""The C-ABI library builds, loads without a GPU, and exports exactly what include/battn.h
declares.  No compute calls here."""
import ctypes as C
import os
import re

import pytest

import bruce_engine_b200  # noqa: F401
from bruce_engine_b200 import build, capi
from bruce_engine_b200.layout import G_B, G_R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "battn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(battn_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    assert os.path.exists(path)
    lib = C.CDLL(path)
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in battn.h but not exported"
    assert set(names) == set(capi.SIGNATURES), "ctypes binding and header disagree"
    assert capi.load().battn_version() == 4


def test_argument_errors_without_a_device():
    lib = capi.load()
    h = C.c_void_p()
    assert lib.battn_init(None, 0, C.byref(h)) == capi.ERR_ARG
    bad = capi.CGeom(32, 8, 96, 4096, 8192, 1, 1, 1, 0.0)            # head_dim 96 unsupported
    assert lib.battn_init(C.byref(bad), 0, C.byref(h)) == capi.ERR_ARG
    bad = capi.CGeom(32, 8, 128, 1000, 8192, 1, 1, 1, 0.0)           # window not a power of two
    assert lib.battn_init(C.byref(bad), 0, C.byref(h)) == capi.ERR_ARG
    bad = capi.CGeom(32, 8, 128, 4096, 8191, 1, 1, 1, 0.0)           # odd slot_ctx
    assert lib.battn_init(C.byref(bad), 0, C.byref(h)) == capi.ERR_ARG
    bad = capi.CGeom(30, 8, 128, 4096, 8192, 1, 1, 1, 0.0)           # heads not divisible
    assert lib.battn_init(C.byref(bad), 0, C.byref(h)) == capi.ERR_ARG
    assert lib.battn_destroy(None) == capi.ERR_ARG
    assert lib.battn_launch_count(None) == 0


def test_engine_refuses_to_run_without_cuda():
    import torch
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    from bruce_engine_b200.engine import AttnEngine
    with pytest.raises(RuntimeError):
        AttnEngine(G_B)


def test_layout_constants_match_reference():
    # bruce.cu:56-61: 272 B per kv head per position, 1088 B per position (4 kv heads), K or V
    assert G_R.rec == 272 and G_R.n_kv * G_R.rec == 1088
    assert G_B.rec == 136
    assert G_B.pos_bytes == G_R.pos_bytes == 2176
    g = G_B.with_(slot_ctx=262144)
    assert g.layer_bytes(False) == 262144 * 1088 and g.layer_bytes(True) == 8192 * 1088
    g8 = G_R.with_(slot_ctx=4096, n_slots=8)
    assert g8.slot_offset(3, False) == 3 * 4096 * 1088 and g8.slot_offset(3, True) == 3 * 2048 * 1088


def test_reference_shim_header_compiles():
    """include/battn_bruce_shim.h re-creates the reference's call surface over the C ABI."""
    import shutil
    import subprocess
    import tempfile
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "shim_check.cu")
        with open(src, "w") as f:
            f.write('#include "battn_bruce_shim.h"\n'
                    "void use(float* o, const float* q, const uint8_t* k, const uint8_t* v, const int* p, float* part,\n"
                    "         cudaStream_t st) { launch_attn_m(o, q, k, v, p, part, 1, 56, 0, st);\n"
                    "  launch_attn_ms(o, q, k, v, p, p, p, part, 8, 7, 1, st); launch_attn_exact(o, q, k, v, p, part, 4, 8, 0, st);\n"
                    "  launch_attn_m(o, q, k, v, p, part, 8, 28, 0, st); launch_attn_m(o, q, k, v, p, part, 512, 2, 1, st);\n"
                    "  gate_norm_rows(nullptr, o, q, q, (int8_t*)o, o, (int*)o, 4, st);\n"
                    "  attn_gate_norm_rows(q, k, v, p, part, q, q, (int8_t*)o, o, (int*)o, 512, 0, st); }\n")
        r = subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                            os.path.join(ROOT, "include"), "-c", src, "-o", os.path.join(d, "shim_check.o")],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr


def test_workspace_covers_every_shorter_call():
    """battn_workspace_bytes(n_seq, R) must serve calls of 1..R rows: a prompt's last chunk is shorter than the
    chunk `part` was sized for, and shorter chunks take MORE key splits.  battn_call_workspace_bytes is the
    per-shape need on a device with the given SM count; the handle-based size is its maximum over r <= R (the
    maximisation itself runs in tests/test_gpu_prefill.py, which has a handle); here the handle-free function is
    checked for the shapes that once overflowed."""
    lib = capi.load()
    for geom, sms in ((G_R, 148), (G_B, 148), (G_B, 132)):
        cg = capi.CGeom(geom.n_head, geom.n_kv, geom.head_dim, geom.window, 65536, 1, geom.q_dtype, geom.out_dtype, 0.0)
        need = {}
        for r in range(1, 513):
            n = C.c_size_t()
            assert lib.battn_call_workspace_bytes(C.byref(cg), sms, 1, r, C.byref(n)) == capi.OK
            need[r] = n.value
        rec = (geom.head_dim + 2) * 4 * geom.n_head
        # a prompt chunk of r rows with s key splits writes r * s records of n_head * (HD + 2) floats
        for r in (40, 96, 160, 192, 384, 512):
            if r * geom.group > 32:
                assert need[r] % (r * rec) == 0 and 1 <= need[r] // (r * rec) <= 8
        # the shapes of the old overflow: a 512-row buffer sized by its own split count alone is too small
        worst = max(need.values())
        assert worst >= need[512]
        if geom is G_R:
            assert max(need[r] for r in range(147, 385)) > need[512]
    bad = C.c_size_t()
    cg = capi.CGeom(32, 8, 128, 4096, 8192, 1, 1, 1, 0.0)
    assert lib.battn_call_workspace_bytes(C.byref(cg), 0, 1, 1, C.byref(bad)) == capi.ERR_ARG
    assert lib.battn_call_workspace_bytes(C.byref(cg), 148, 1, 513, C.byref(bad)) == capi.ERR_CAPACITY
