"""Pins this repository against the REFERENCE'S OWN KERNELS (engine/src/bruce.cu compiled unmodified
into oracle/_ref/libbruce_ref.so by oracle/ref_build.py), in the reference's native geometry
(16 q-heads / 4 KV heads / head_dim 256 / window 1024):

  * KV bytes: the V records written by the reference's append kernel k_qkv_prep_fast (which quantises v
    raw, bruce.cu:1886, 1910-1915) must equal battn_kv_append's and the CPU oracle's, byte for byte.
    (K goes through the reference's model-specific L2-norm/RoPE prologue first and is compared through
    attention instead.)
  * Attention: on the cache the REFERENCE wrote and the query IT normalised, the reference's exact
    fp32 path (k_attn_rows + k_attn_combine_rows) must agree with the CPU oracle (tight) and with
    every fast path here (decode, verify, prompt chunk, exact) within the test tolerance.

Skipped when the reference library was not built (the reference tree is not available on the box)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import dev_i32, new_out, to_np
from tests.util import assert_close, errors, oracle_geom

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libbruce_ref.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(LIB):
        pytest.skip("oracle/_ref/libbruce_ref.so not built (reference tree unavailable)")
    lib = C.CDLL(LIB)
    geo = (C.c_int * 7)()
    lib.ref_geometry(geo)
    assert list(geo)[:6] == [16, 4, 256, 1024, 2048, 272]
    return lib


def _p(t):
    return C.c_void_p(t.data_ptr())


class RefCase:
    """A sequence appended by the reference's own kernel."""

    def __init__(self, lib, n, is_swa, seed):
        from bruce_engine_b200.engine import AttnEngine
        from bruce_engine_b200.layout import G_R
        self.lib, self.n, self.is_swa = lib, n, is_swa
        self.g = G_R.with_(slot_ctx=max(n, 2048))
        self.eng = AttnEngine(self.g)
        g = self.g
        rng = np.random.default_rng(seed)
        self.k = rng.standard_normal((n, g.n_kv, g.head_dim), dtype=np.float32)
        self.v = rng.standard_normal((n, g.n_kv, g.head_dim), dtype=np.float32)
        self.kvk, self.kvv = self.eng.alloc_kv_layer(is_swa, fill=0)
        kd, vd = torch.from_numpy(self.k).cuda(), torch.from_numpy(self.v).cuda()
        sqk = torch.ones((g.n_head, g.head_dim), device="cuda")
        for a in range(0, n, 512):                     # identity RoPE: cos = 1, sin = 0
            rows = min(512, n - a)
            cs = torch.ones((rows, 256), device="cuda")
            sn = torch.zeros((rows, 256), device="cuda")
            qd = torch.zeros((rows, g.n_head, g.head_dim), device="cuda")
            rc = lib.ref_kv_append(_p(qd), _p(kd[a:a + rows].contiguous()), _p(vd[a:a + rows].contiguous()), _p(sqk),
                                   _p(self.kvk), _p(self.kvv), _p(dev_i32([a], "cuda")), rows, int(is_swa),
                                   g.slot_ctx, _p(cs), _p(sn))
            assert rc == 0

    def ref_query(self, rows, seed):
        """Queries as the reference's prologue leaves them (L2-normalised, bruce.cu:1845-1865)."""
        g = self.g
        rng = np.random.default_rng(seed)
        q = torch.from_numpy(rng.standard_normal((rows, g.n_head, g.head_dim), dtype=np.float32)).cuda()
        scratch_k = torch.zeros((rows, g.n_kv, g.head_dim), device="cuda")
        sk, sv = self.eng.alloc_kv_layer(self.is_swa, fill=0)       # throw-away cache for the prologue call
        rc = self.lib.ref_kv_append(_p(q), _p(scratch_k), _p(scratch_k), _p(torch.ones((g.n_head, g.head_dim), device="cuda")),
                                    _p(sk), _p(sv), _p(dev_i32([0], "cuda")), rows, int(self.is_swa), g.slot_ctx,
                                    _p(torch.ones((rows, 256), device="cuda")), _p(torch.zeros((rows, 256), device="cuda")))
        assert rc == 0
        return q * 384.0                                # unit-norm q and k rows: scale up so that scores have std ~1.5

    def ref_exact(self, q, p0, rows, ns=8):
        g = self.g
        out = torch.zeros((rows, g.n_head, g.head_dim), device="cuda")
        part = torch.zeros(rows * g.n_kv * ns * 4 * (g.head_dim + 2), device="cuda")
        rc = self.lib.ref_attn_exact(_p(out), _p(q), _p(self.kvk), _p(self.kvv), _p(dev_i32([p0], "cuda")), _p(part),
                                     rows, ns, int(self.is_swa), g.slot_ctx)
        assert rc == 0
        return out


@pytest.mark.parametrize("is_swa", [False, True])
def test_v_bytes_equal_the_reference_kernels(ref, is_swa):
    n = 2500 if is_swa else 1300                       # the ring (2048) wraps
    c = RefCase(ref, n, is_swa, seed=41)
    g, eng = c.g, c.eng
    # this repository's append kernel on the same V rows (K rows too, into a scratch cache)
    kvk2, kvv2 = eng.alloc_kv_layer(is_swa, fill=0)
    vd = torch.from_numpy(c.v).cuda()
    for a in range(0, n, 512):
        rows = min(512, n - a)
        eng.qkv_prep_store(vd[a:a + rows], vd[a:a + rows], kvk2, kvv2, dev_i32([a], "cuda"), rows=rows, is_swa=is_swa)
    torch.cuda.synchronize()
    assert torch.equal(kvv2, c.kvv), "V cache bytes differ from the reference kernel's"
    og = oracle_geom(g)
    okvk, okvv = O.new_cache(og, is_swa), O.new_cache(og, is_swa)
    O.kv_append(og, c.v[None], c.v[None], okvk, okvv, [0], rows=n, is_swa=is_swa)
    assert (c.kvv.cpu().numpy() == okvv).all(), "oracle V bytes differ from the reference kernel's"


@pytest.mark.parametrize("is_swa", [False, True])
def test_attention_agrees_with_the_reference_exact_kernels(ref, is_swa):
    n = 2300 if is_swa else 1500
    c = RefCase(ref, n, is_swa, seed=42)
    g, eng = c.g, c.eng
    og = oracle_geom(g)
    okvk, okvv = c.kvk.cpu().numpy(), c.kvv.cpu().numpy()          # the cache the reference wrote
    for rows in (1, 4, 8, 96):
        p0 = n - rows
        q = c.ref_query(rows, seed=100 + rows)
        want = to_np(c.ref_exact(q, p0, rows))[None]                # the reference's own exact kernels
        # the CPU oracle restates that arithmetic: tight agreement
        orc = O.attend(og, to_np(q)[None], okvk, okvv, [p0], rows=rows, is_swa=is_swa)
        mabs, rel, _, _ = errors(orc, want)
        assert mabs < 2e-5 and rel < 2e-5, f"oracle vs reference exact kernels: {mabs:.2e} {rel:.2e}"
        # every path of this repository on the reference's cache
        out = new_out(eng, 1, rows, g.n_head, g.head_dim)
        part = eng.alloc_part(1, rows)
        eng.launch_attn_m(out, q[None].contiguous(), c.kvk, c.kvv, dev_i32([p0], "cuda"), part, rows, is_swa)
        torch.cuda.synchronize()
        assert_close(to_np(out), want, f"fast path vs reference exact kernel rows={rows} swa={is_swa}")
        ex = new_out(eng, 1, rows, g.n_head, g.head_dim)
        ws = torch.empty(eng.exact_workspace_bytes(1, rows, 8), dtype=torch.uint8, device="cuda")
        eng.attn_exact(ex, q[None].contiguous(), c.kvk, c.kvv, dev_i32([p0], "cuda"), ws, 1, rows, 8, is_swa)
        torch.cuda.synchronize()
        mabs, rel, _, _ = errors(to_np(ex), want)
        assert mabs < 2e-5 and rel < 2e-5, f"exact path vs reference exact kernels: {mabs:.2e} {rel:.2e}"
    assert eng.device_status() == 0


def test_reference_shipping_kernels_for_context(ref):
    """The reference's shipping tensor-core kernels accumulate in fp16 (bruce.cu:2998-3095): their
    distance from the reference's own exact path is recorded here next to this repository's, as context
    for the tolerance (no assertion on the reference's error beyond sanity)."""
    n = 4096
    c = RefCase(ref, n, False, seed=43)
    g = c.g
    q = c.ref_query(1, seed=7)
    want = to_np(c.ref_exact(q, n - 1, 1))
    out = torch.zeros((1, g.n_head, g.head_dim), device="cuda")
    part = torch.zeros(g.n_kv * 56 * 4 * (g.head_dim + 2), device="cuda")
    ms = C.c_float()
    rc = ref.ref_attn_shipping(_p(out), _p(q), _p(c.kvk), _p(c.kvv), _p(dev_i32([n - 1], "cuda")), _p(part), 1, 56, 0,
                               g.slot_ctx, 5, C.byref(ms))
    assert rc == 0
    mabs, rel, relmax, _ = errors(to_np(out), want)
    print(f"[reference shipping decode kernel vs its exact path] max-abs {mabs:.2e} rel-l2 {rel:.2e} rel-max {relmax:.2e}")
    assert mabs < 5e-2


def test_reference_shipping_prompt_kernel_for_context(ref):
    """The reference's shipping prompt-chunk dispatch (launch_attn_m with rows = 512 -> k_attn_tc_rs_opt, fp16
    accumulation, bruce.cu:4021-4078) compiled for sm_100a, timed on this GPU next to this repository's kernel on
    the same cache and queries (512 rows against 16,384 cached keys, the reference's geometry), and both compared
    with the reference's exact path.  Context for the measurements; the only assertions are on this
    repository's result."""
    n, rows = 16384, 512
    c = RefCase(ref, n, False, seed=47)
    g, eng = c.g, c.eng
    p0 = n - rows
    q = c.ref_query(rows, seed=11)
    pos = dev_i32([p0], "cuda")
    want = to_np(c.ref_exact(q, p0, rows, ns=4))[None]
    flops = 4.0 * g.head_dim * g.n_head * (rows * p0 + rows * (rows + 1) // 2)
    # reference shipping kernels: split counts around its own rule (3 at this shape, bruce.cu:7703-7706)
    best = None
    for ns in (1, 3, 8):
        out_r = torch.zeros((rows, g.n_head, g.head_dim), device="cuda")
        part = torch.zeros(rows * ns * g.n_kv * 4 * (g.head_dim + 2), device="cuda")
        ms = C.c_float()
        rc = ref.ref_attn_shipping(_p(out_r), _p(q), _p(c.kvk), _p(c.kvv), _p(pos), _p(part), rows, ns, 0, g.slot_ctx, 5,
                                   C.byref(ms))
        assert rc == 0
        us = ms.value * 1e3 / 5
        if best is None or us < best[0]:
            best = (us, ns, out_r)
    mabs_r, rel_r, _, _ = errors(to_np(best[2])[None], want)
    # this repository
    out = new_out(eng, 1, rows, g.n_head, g.head_dim)
    part = eng.alloc_part(1, rows)
    for _ in range(3):
        eng.launch_attn_m(out, q[None].contiguous(), c.kvk, c.kvv, pos, part, rows, False)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        eng.launch_attn_m(out, q[None].contiguous(), c.kvk, c.kvv, pos, part, rows, False)
    e1.record()
    torch.cuda.synchronize()
    us_here = e0.elapsed_time(e1) * 1e3 / 5
    from tests.util import PROMPT_HEAD_REL_TOL
    mabs, rel = assert_close(to_np(out), want, "prompt kernel vs reference exact kernels at depth 16K",
                             head_tol=PROMPT_HEAD_REL_TOL)
    print(f"[reference shipping prompt kernel, sm_100a build] {best[0]:.0f} us (ns={best[1]}) = {flops / best[0] / 1e6:.0f} TFLOPS,"
          f" max-abs {mabs_r:.2e} rel {rel_r:.2e} vs its exact path;"
          f" this repository {us_here:.0f} us = {flops / us_here / 1e6:.0f} TFLOPS, max-abs {mabs:.2e} rel {rel:.2e}")
    assert eng.device_status() == 0


def test_reference_shipping_decode_kernel_timing_for_context(ref):
    """The reference's shipping decode dispatch (launch_attn_m with rows = 1 + k_attn_combine_rows) compiled for
    sm_100a, timed on this GPU next to battn_decode on the same 65,536-position cache (the reference's geometry).
    Its split count is tuned for a 28-SM GPU (56, bruce.cu:3926); the largest it supports (128) is tried as well."""
    n = 65536
    c = RefCase(ref, n, False, seed=53)
    g, eng = c.g, c.eng
    q = c.ref_query(1, seed=3)
    pos = dev_i32([n - 1], "cuda")
    want = to_np(c.ref_exact(q, n - 1, 1))[None]
    nbytes = n * g.n_kv * (g.head_dim + g.head_dim // 16) * 2
    best = None
    for ns in (56, 128):
        out_r = torch.zeros((1, g.n_head, g.head_dim), device="cuda")
        part = torch.zeros(g.n_kv * ns * 4 * (g.head_dim + 2), device="cuda")
        ms = C.c_float()
        rc = ref.ref_attn_shipping(_p(out_r), _p(q), _p(c.kvk), _p(c.kvv), _p(pos), _p(part), 1, ns, 0, g.slot_ctx, 20,
                                   C.byref(ms))
        assert rc == 0
        us = ms.value * 1e3 / 20
        if best is None or us < best[0]:
            best = (us, ns)
    out = new_out(eng, 1, 1, g.n_head, g.head_dim)
    part = eng.alloc_part(1, 1)
    for _ in range(3):
        eng.launch_attn_m(out, q[None].contiguous(), c.kvk, c.kvv, pos, part, 1, False)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        eng.launch_attn_m(out, q[None].contiguous(), c.kvk, c.kvv, pos, part, 1, False)
    e1.record()
    torch.cuda.synchronize()
    us_here = e0.elapsed_time(e1) * 1e3 / 20
    assert_close(to_np(out), want, "decode vs reference exact kernels at 64K")
    print(f"[reference shipping decode kernel, sm_100a build, 64K] {best[0]:.1f} us (ns={best[1]}) = "
          f"{nbytes / best[0] / 1e6:.2f} TB/s; this repository {us_here:.1f} us = {nbytes / us_here / 1e6:.2f} TB/s")
    assert eng.device_status() == 0
