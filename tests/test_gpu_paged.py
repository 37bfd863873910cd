"""Paged cache of a full-causal layer, through the C ABI.

The same seeded K/V go into a contiguous cache (whose bytes the other tests pin to the oracle's) and, through
battn_kv_append_paged, into a pool whose page table is a random permutation.  Checked: every page holds the bytes
of the contiguous cache; decode, verify (2..8 rows), prompt-chunk and exact attention over the pages equal the
contiguous calls bit for bit and the CPU oracle within the usual tolerances; two sequences sharing prefix pages;
a table entry outside the pool sets the status bit without a fault."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import dev_i32, dev_q, gpu_fill, new_out, to_np
from tests.util import assert_close, draw_qkv, oracle_fill, oracle_geom

pytestmark = pytest.mark.gpu


def _geom(name, **kw):
    from bruce_engine_b200.layout import F32, G_B, G_R
    base = {"B": G_B, "B32": G_B.with_(out_dtype=F32), "R": G_R}[name]
    return base.with_(**kw)


def _engine(g):
    from bruce_engine_b200.engine import AttnEngine
    return AttnEngine(g)


class PagedSeqs:
    """n_seq sequences of ragged lengths, cached twice: contiguous partitions and scrambled pages."""

    def __init__(self, name, lens, page_len, seed, rows_q=8, spare_pages=3):
        self.lens = lens
        n_seq = len(lens)
        cap = max(lens) + 16
        cap += (-cap) % page_len
        self.g = g = _geom(name, slot_ctx=cap, n_slots=n_seq)
        self.eng = eng = _engine(g)
        self.og = oracle_geom(g)
        self.page_len, self.max_pages = page_len, cap // page_len
        rng = np.random.default_rng(seed)
        need = [(n + 16 + page_len - 1) // page_len for n in lens]
        self.n_pages = sum(need) + spare_pages
        perm = rng.permutation(self.n_pages)
        table = np.full((n_seq, self.max_pages), -1, dtype=np.int32)     # unused entries are invalid on purpose
        at = 0
        for i, c in enumerate(need):
            table[i, :c] = perm[at:at + c]
            at += c
        self.table_np = table
        self.table = torch.from_numpy(table).to(eng.device)
        self.pages, self.pool_k, self.pool_v = eng.alloc_pages(self.n_pages, page_len, self.table, fill=0x7F)
        self.kvk, self.kvv = eng.alloc_kv_layer(False, fill=0x7F)
        self.okvk, self.okvv = O.new_cache(self.og, False, fill=0x7F), O.new_cache(self.og, False, fill=0x7F)
        self.q = []
        for i, n in enumerate(lens):
            q, k, v = draw_qkv(g, n, rows_q, seed * 100 + i, q_f16=(g.q_dtype == 1))
            self.q.append(q[0])
            gpu_fill(eng, k, v, self.kvk, self.kvv, False, slot=i)
            oracle_fill(self.og, k, v, False, slot=i, kvk=self.okvk, kvv=self.okvv)
            kd = torch.from_numpy(k).to(eng.device)
            vd = torch.from_numpy(v).to(eng.device)
            for a in range(0, n, 512):
                b = min(n, a + 512)
                eng.kv_append_paged(self.pages, kd[a:b], vd[a:b], dev_i32([a], eng.device),
                                    ktab=dev_i32([i], eng.device), rows=b - a)
        torch.cuda.synchronize()
        assert (self.kvk.cpu().numpy() == self.okvk).all() and (self.kvv.cpu().numpy() == self.okvv).all()
        self.part = eng.alloc_part(n_seq, 8)
        self.q = np.stack(self.q)                 # [n_seq][rows_q][n_head][head_dim]

    def check_page_bytes(self):
        g = self.g
        rec = g.rec
        for pool, cache in ((self.pool_k, self.kvk), (self.pool_v, self.kvv)):
            pool = pool.cpu().numpy().reshape(self.n_pages, g.n_kv, self.page_len, rec)
            cache = cache.cpu().numpy().reshape(g.n_slots, g.n_kv, g.slot_ctx, rec)
            for i, n in enumerate(self.lens):
                for lp in range((n + self.page_len - 1) // self.page_len):
                    a, b = lp * self.page_len, min(n, (lp + 1) * self.page_len)
                    assert (pool[self.table_np[i, lp], :, :b - a] == cache[i, :, a:b]).all(), (i, lp)

    def both(self, pos, rows):
        """(paged output, contiguous output, oracle) for `rows` query rows per sequence at positions pos[i].."""
        g, eng = self.g, self.eng
        n_seq = len(self.lens)
        q = self.q[:, :rows]
        qd = dev_q(eng, q)
        posd, slots = dev_i32(pos, eng.device), dev_i32(list(range(n_seq)), eng.device)
        got = new_out(eng, n_seq, rows, g.n_head, g.head_dim)
        ref = new_out(eng, n_seq, rows, g.n_head, g.head_dim)
        eng.attn_paged(got, qd, self.pages, posd, self.part, rows=rows, ktab=slots)
        eng.launch_attn_ms(ref, qd, self.kvk, self.kvv, posd, slots, None, self.part, n_seq, rows_per_seq=rows)
        torch.cuda.synchronize()
        want = O.attend(self.og, q, self.okvk, self.okvv, list(pos), kslot=list(range(n_seq)), rows=rows)
        return to_np(got), to_np(ref), want


@pytest.mark.parametrize("name", ["B32", "R"])
@pytest.mark.parametrize("page_len", [128, 512])
def test_paged_append_and_decode(name, page_len):
    s = PagedSeqs(name, [3000, 129, 1, 1025, 640], page_len, seed=3)
    s.check_page_bytes()
    pos = [n - 1 for n in s.lens]
    got, ref, want = s.both(pos, 1)
    assert np.array_equal(got, ref), "paged decode differs from the contiguous call"
    assert_close(got, want, f"paged decode {name} page {page_len}")
    # earlier positions: tiles that end inside a page, on a page boundary, one past it
    pos = [min(n - 1, p) for n, p in zip(s.lens, [page_len - 1, page_len, 0, page_len + 1, 2 * page_len - 1])]
    got, ref, want = s.both(pos, 1)
    assert np.array_equal(got, ref)
    assert_close(got, want, f"paged decode edges {name} page {page_len}")
    assert s.eng.device_status() == 0


def test_paged_decode_with_early_kv_streaming():
    """Early KV streaming reads the page table before the preceding kernel has finished; with the table uploaded by a
    copy (as here) the paged decode still equals the contiguous call bit for bit."""
    s = PagedSeqs("B32", [2000, 700, 4100], 256, seed=9)
    s.eng.set_early_kv_stream(True)
    for step in range(3):
        pos = [n - 1 - step for n in s.lens]
        got, ref, want = s.both(pos, 1)
        assert np.array_equal(got, ref)
        assert_close(got, want, f"paged decode, early streaming, step {step}")
    assert s.eng.device_status() == 0


@pytest.mark.parametrize("name,rows", [("B32", 2), ("B32", 4), ("B32", 8), ("B", 8), ("R", 3), ("R", 8)])
def test_paged_verify(name, rows):
    s = PagedSeqs(name, [2500, 300, 1100], 256, seed=4)
    pos = [n - rows for n in s.lens]
    got, ref, want = s.both(pos, rows)
    assert np.array_equal(got, ref), "paged verify differs from the contiguous call"
    assert_close(got, want, f"paged verify {name} rows {rows}")
    assert s.eng.device_status() == 0


@pytest.mark.parametrize("name", ["B32", "R"])
def test_paged_prompt_chunk_and_exact(name):
    """A 200-row chunk at depth ~1.9K of table row 1 (row 0 holds another sequence), against the contiguous prompt
    kernel (bit-identical), the paged exact path and the oracle."""
    s = PagedSeqs(name, [700, 2100], 256, seed=5, rows_q=200)
    g, eng = s.g, s.eng
    rows, p0 = 200, 2100 - 200
    q = s.q[1:2, :rows]
    qd = dev_q(eng, q)
    posd = dev_i32([p0], eng.device)
    part = eng.alloc_part(1, rows)
    got = new_out(eng, 1, rows, g.n_head, g.head_dim)
    ref = new_out(eng, 1, rows, g.n_head, g.head_dim)
    eng.attn_paged(got, qd, s.pages, posd, part, rows=rows, table_row=1)
    layer = g.layer_bytes(False) // g.n_slots
    eng.launch_attn_m(ref, qd, s.kvk[layer:], s.kvv[layer:], posd, part, rows)
    torch.cuda.synchronize()
    assert np.array_equal(to_np(got), to_np(ref)), "paged prompt chunk differs from the contiguous call"
    want = O.attend(s.og, q, s.okvk, s.okvv, [p0], kslot=[1], rows=rows)
    assert_close(to_np(got), want, f"paged prompt chunk {name}")
    # exact path over the pages
    nsplit = 4
    ws = torch.empty(eng.exact_workspace_bytes(1, rows, nsplit), dtype=torch.uint8, device=eng.device)
    ex = new_out(eng, 1, rows, g.n_head, g.head_dim)
    eng.attn_exact_paged(ex, qd, s.pages, posd, ws, 1, rows, nsplit, ktab=dev_i32([1], eng.device))
    torch.cuda.synchronize()
    assert_close(to_np(ex), want, f"paged exact {name}")
    assert eng.device_status() == 0


def test_paged_prefix_sharing():
    """Two table rows point at the same physical pages for a 512-position prefix and at their own pages after it;
    each decodes exactly what a private copy of the prefix gives."""
    name, page_len, pre = "B32", 256, 512
    g = _geom(name, slot_ctx=2048, n_slots=2)
    eng, og = _engine(g), oracle_geom(g)
    lens = [900, 1300]
    _, kp, vp = draw_qkv(g, pre, 1, 70)
    tails = [draw_qkv(g, n - pre, 1, 71 + i) for i, n in enumerate(lens)]
    table = np.full((2, 8), -1, dtype=np.int32)
    table[0, :4] = [5, 2, 7, 0]
    table[1, :6] = [5, 2, 1, 3, 6, 4]               # pages 5 and 2 are shared
    td = torch.from_numpy(table).to(eng.device)
    pages, pool_k, pool_v = eng.alloc_pages(8, page_len, td, fill=0x7F)
    okvk, okvv = O.new_cache(og, False, fill=0x7F), O.new_cache(og, False, fill=0x7F)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(eng.device)
    eng.kv_append_paged(pages, up(kp), up(vp), dev_i32([0], eng.device), ktab=dev_i32([0], eng.device), rows=pre)
    qs = []
    for i, (q, kt, vt) in enumerate(tails):
        for a in range(0, kt.shape[0], 512):
            b = min(kt.shape[0], a + 512)
            eng.kv_append_paged(pages, up(kt[a:b]), up(vt[a:b]), dev_i32([pre + a], eng.device),
                                ktab=dev_i32([i], eng.device), rows=b - a)
        oracle_fill(og, np.concatenate([kp, kt]), np.concatenate([vp, vt]), False, slot=i, kvk=okvk, kvv=okvv)
        qs.append(q[0])
    q = np.stack(qs).astype(np.float16).astype(np.float32)
    pos = [n - 1 for n in lens]
    out = new_out(eng, 2, 1, g.n_head, g.head_dim)
    part = eng.alloc_part(2, 1)
    eng.attn_paged(out, dev_q(eng, q), pages, dev_i32(pos, eng.device), part, rows=1, ktab=dev_i32([0, 1], eng.device))
    torch.cuda.synchronize()
    want = O.attend(og, q, okvk, okvv, pos, kslot=[0, 1], rows=1)
    assert_close(to_np(out), want, "shared prefix pages")
    assert eng.device_status() == 0


def test_paged_copy_on_write():
    """Row 1 shares row 0's two pages, then overwrites position 300 (inside the second shared page) after taking a
    private copy of that page: row 0 still decodes its own records, row 1 the changed ones."""
    name, page_len = "B32", 256
    g = _geom(name, slot_ctx=1024, n_slots=2)
    eng, og = _engine(g), oracle_geom(g)
    q, k, v = draw_qkv(g, 512, 1, 90, n_seq=2)
    _, k2, v2 = draw_qkv(g, 1, 1, 91)
    table = np.full((2, 4), -1, dtype=np.int32)
    table[0, :2] = [3, 1]
    table[1, :2] = [3, 1]
    td = torch.from_numpy(table).to(eng.device)
    pages, pool_k, pool_v = eng.alloc_pages(5, page_len, td, fill=0x7F)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(eng.device)
    eng.kv_append_paged(pages, up(k), up(v), dev_i32([0], eng.device), ktab=dev_i32([0], eng.device), rows=512)
    # copy on write of logical page 1 of row 1: physical 1 -> 4, then the table entry, then the append
    eng.pages_copy(pages, 1, 4)
    td[1, 1] = 4
    eng.kv_append_paged(pages, up(k2), up(v2), dev_i32([300], eng.device), ktab=dev_i32([1], eng.device), rows=1)
    okvk, okvv = O.new_cache(og, False, fill=0x7F), O.new_cache(og, False, fill=0x7F)
    oracle_fill(og, k, v, False, slot=0, kvk=okvk, kvv=okvv)
    kb, vb = k.copy(), v.copy()
    kb[300], vb[300] = k2[0], v2[0]
    oracle_fill(og, kb, vb, False, slot=1, kvk=okvk, kvv=okvv)
    out = new_out(eng, 2, 1, g.n_head, g.head_dim)
    part = eng.alloc_part(2, 1)
    eng.attn_paged(out, dev_q(eng, q), pages, dev_i32([511, 511], eng.device), part, rows=1, ktab=dev_i32([0, 1], eng.device))
    torch.cuda.synchronize()
    want = O.attend(og, q, okvk, okvv, [511, 511], kslot=[0, 1], rows=1)
    assert_close(to_np(out), want, "copy on write")
    assert not np.array_equal(to_np(out)[0], to_np(out)[1])
    assert eng.device_status() == 0


def test_paged_bad_table_entry_sets_status():
    """A page number outside the pool: the status bit is set and nothing outside the pool is touched."""
    s = PagedSeqs("B32", [600], 128, seed=6)
    bad = s.table.clone()
    bad[0, 2] = s.n_pages + 7
    from bruce_engine_b200 import capi
    pages = capi.CPages(s.pool_k.data_ptr(), s.pool_v.data_ptr(), bad.data_ptr(), s.n_pages, 1, s.max_pages, 128)
    g, eng = s.g, s.eng
    out = new_out(eng, 1, 1, g.n_head, g.head_dim)
    eng.attn_paged(out, dev_q(eng, s.q[:, :1]), pages, dev_i32([599], eng.device), s.part, rows=1)
    torch.cuda.synchronize()
    assert eng.device_status(clear=True) & capi.DEV_BAD_POSITION
    # the library refuses malformed descriptors before any launch
    for page_len in (64, 192):
        d = capi.CPages(s.pool_k.data_ptr(), s.pool_v.data_ptr(), s.table.data_ptr(), s.n_pages, 1, s.max_pages, page_len)
        with pytest.raises(capi.BattnError):
            eng.attn_paged(out, dev_q(eng, s.q[:, :1]), d, dev_i32([599], eng.device), s.part, rows=1)


@pytest.mark.parametrize("name", ["B32", "R"])
def test_paged_fused_prologue_writes_the_same_bytes(name):
    """battn_qkv_prep_paged against battn_qkv_prep on the same inputs: the same q, and every page holds the bytes of
    the contiguous partition (the contiguous form is pinned to the oracle and the reference's kernel elsewhere)."""
    page_len, n_seq, rows = 128, 3, 5
    g = _geom(name, slot_ctx=1024, n_slots=n_seq)
    eng = _engine(g)
    rng = np.random.default_rng(11)
    HD = g.head_dim
    q = rng.standard_normal((n_seq, rows, g.n_head, HD), dtype=np.float32)
    k = rng.standard_normal((n_seq, rows, g.n_kv, HD), dtype=np.float32) * 3.0
    v = rng.standard_normal((n_seq, rows, g.n_kv, HD), dtype=np.float32)
    sqk = (1.0 + 0.2 * rng.standard_normal((g.n_head, HD))).astype(np.float32)
    pos = np.array([125, 640, 3], dtype=np.int32)                    # the first sequence's rows cross a page boundary
    cs, sn = O.rope_tables(HD, (pos[:, None] + np.arange(rows)[None]).reshape(-1))
    table = np.array([[7, 2, -1, -1, -1, -1, -1, -1], [0, 1, 3, 4, 5, 6, -1, -1], [8, -1, -1, -1, -1, -1, -1, -1]], dtype=np.int32)
    td = torch.from_numpy(table).to(eng.device)
    pages, pool_k, pool_v = eng.alloc_pages(9, page_len, td, fill=0)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(eng.device)
    qd, kd, vd, sq, csd, snd = up(q), up(k), up(v), up(sqk), up(cs), up(sn)
    posd, rowsd = dev_i32(pos, eng.device), dev_i32([0, 1, 2], eng.device)
    q_a = torch.empty_like(qd, dtype=eng.q_torch)
    q_b = torch.empty_like(qd, dtype=eng.q_torch)
    eng.qkv_prep(q_a, qd, kd, vd, sq, csd, snd, kvk, kvv, posd, kslot=rowsd, rows=rows)
    eng.qkv_prep_paged(q_b, qd, kd, vd, sq, csd, snd, pages, posd, ktab=rowsd, rows=rows)
    torch.cuda.synchronize()
    assert torch.equal(q_a, q_b)
    rec = g.rec
    for pool, cache in ((pool_k, kvk), (pool_v, kvv)):
        pool = pool.cpu().numpy().reshape(9, g.n_kv, page_len, rec)
        cache = cache.cpu().numpy().reshape(n_seq, g.n_kv, g.slot_ctx, rec)
        assert cache.any()
        for i in range(n_seq):
            for p in range(int(pos[i]), int(pos[i]) + rows):
                assert (pool[table[i, p // page_len], :, p % page_len] == cache[i, :, p]).all(), (i, p)
    assert eng.device_status() == 0
