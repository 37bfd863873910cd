"""Host-side mirror of the reference engine's attention call surface, over the C ABI.

Method names follow the reference's launches (engine/src/bruce.cu): `qkv_prep_store` is the
quantise-and-store half of k_qkv_prep / k_qkv_prep_fast / k_qkv_prep_fast_ms (:644, :1732, :1835),
`launch_attn_m` is launch_attn_m + the merge (:3942, :928, :1999), `launch_attn_ms` is
launch_attn_ms + the merge (:4158), `attn_combine` is k_attn_combine (:992).  Arguments keep the
reference's meaning: device buffers owned by the caller, device-resident positions, `part` scratch.

torch is used only for device memory and streams; every computation is a call into libbattn.so.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi
from .layout import F16, Geom


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class AttnEngine:
    """One attention context (geometry + device), the replacement of the reference's lazily-set
    kernel attributes and its g_kv_nctx symbol (bruce.cu:65, 3948-3955, 5482)."""

    def __init__(self, geom: Geom, device: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("AttnEngine needs a CUDA device (sm_100a); there is no CPU path")
        self.lib = capi.load()
        self.geom = geom
        self.device = torch.device("cuda", device)
        cg = capi.CGeom(geom.n_head, geom.n_kv, geom.head_dim, geom.window, geom.slot_ctx,
                        geom.n_slots, geom.q_dtype, geom.out_dtype, geom.softmax_scale)
        h = C.c_void_p()
        rc = self.lib.battn_init(C.byref(cg), device, C.byref(h))
        if rc:
            raise capi.BattnError("battn_init", rc, self.lib.battn_last_cuda_error(None))
        self.h = h
        self.q_torch = torch.float16 if geom.q_dtype == F16 else torch.float32
        self.out_torch = torch.float16 if geom.out_dtype == F16 else torch.float32

    def close(self):
        if getattr(self, "h", None):
            self.lib.battn_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- sizes and allocation (alloc_buffers, bruce.cu:5460-5507, 5564) --------------------------
    def _check(self, fn: str, rc: int):
        if rc:
            raise capi.BattnError(fn, rc, self.lib.battn_last_cuda_error(self.h))

    def kv_layer_bytes(self, is_swa: bool) -> int:
        n = C.c_size_t()
        self._check("battn_kv_layer_bytes", self.lib.battn_kv_layer_bytes(self.h, int(is_swa), C.byref(n)))
        return n.value

    def alloc_kv_layer(self, is_swa: bool, fill: int | None = None):
        """One layer's K and V buffers for all slots."""
        n = self.kv_layer_bytes(is_swa)
        mk = (lambda: torch.empty(n, dtype=torch.uint8, device=self.device)) if fill is None else \
             (lambda: torch.full((n,), fill, dtype=torch.uint8, device=self.device))
        return mk(), mk()

    def workspace_bytes(self, n_seq: int, rows: int) -> int:
        n = C.c_size_t()
        self._check("battn_workspace_bytes", self.lib.battn_workspace_bytes(self.h, n_seq, rows, C.byref(n)))
        return n.value

    def exact_workspace_bytes(self, n_seq: int, rows: int, nsplit: int) -> int:
        n = C.c_size_t()
        self._check("battn_exact_workspace_bytes",
                    self.lib.battn_exact_workspace_bytes(self.h, n_seq, rows, nsplit, C.byref(n)))
        return n.value

    def alloc_part(self, n_seq: int, rows: int) -> torch.Tensor:
        """The split-K scratch (`part`, bruce.cu:5564)."""
        return torch.empty(self.workspace_bytes(n_seq, rows), dtype=torch.uint8, device=self.device)

    @staticmethod
    def _stream():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    # ---- KV append ---------------------------------------------------------------------------------
    def qkv_prep_store(self, k, v, kvk, kvv, pos, kslot=None, act=None, rows: int = 1, is_swa: bool = False):
        """k, v: fp32 [n_seq][rows][n_kv][head_dim]; pos/kslot/act: int32 device tensors."""
        n_seq = pos.numel()
        self._check("battn_kv_append", self.lib.battn_kv_append(
            self.h, _ptr(k), _ptr(v), _ptr(kvk), _ptr(kvv), _ptr(pos), _ptr(kslot), _ptr(act),
            n_seq, rows, int(is_swa), self._stream()))

    def kv_copy_prefix(self, kvk, kvv, src_slot: int, dst_slot: int, n_pos: int, is_swa: bool = False):
        """Prefix sharing between slots: the first n_pos cached positions of src_slot copied into dst_slot."""
        self._check("battn_kv_copy_prefix", self.lib.battn_kv_copy_prefix(
            self.h, _ptr(kvk), _ptr(kvv), src_slot, dst_slot, n_pos, int(is_swa), self._stream()))

    def qkv_prep(self, q_out, q, k, v, sqk, cs, sn, kvk, kvv, pos, kslot=None, act=None, rows: int = 1,
                 is_swa: bool = False, theta_sel: int = 1):
        """The whole k_qkv_prep_fast / k_qkv_prep_fast_ms step (bruce.cu:1732-1812, 1835-1918): L2 scale + RoPE
        (+ sqk on q) and the quantised append, one launch.  q_out: the geometry's q dtype (fp32 may be q itself)."""
        n_seq = pos.numel()
        self._check("battn_qkv_prep", self.lib.battn_qkv_prep(
            self.h, _ptr(q_out), _ptr(q), _ptr(k), _ptr(v), _ptr(sqk), _ptr(cs), _ptr(sn), int(theta_sel),
            _ptr(kvk), _ptr(kvv), _ptr(pos), _ptr(kslot), _ptr(act), n_seq, rows, int(is_swa), self._stream()))

    def rope_tables(self, cs, sn, pos, rows: int = 1):
        """k_rope_tables_rows / _ms (bruce.cu:1641-1654, 1821-1833): cs, sn fp32 [n_seq*rows][head_dim]."""
        self._check("battn_rope_tables", self.lib.battn_rope_tables(
            self.h, _ptr(cs), _ptr(sn), _ptr(pos), pos.numel(), rows, self._stream()))

    # ---- attention ---------------------------------------------------------------------------------
    def launch_attn_m(self, out, q, kvk, kvv, pos, part, rows: int, is_swa: bool = False):
        """Single-sequence attention: rows == 1 decode, 2..8 speculative verify, > 8 prompt chunk
        (the dispatch of launch_attn_m, bruce.cu:3942-4122), merge included."""
        st = self._stream()
        if rows == 1:
            rc = self.lib.battn_decode(self.h, _ptr(out), _ptr(q), _ptr(kvk), _ptr(kvv), _ptr(pos), None, None,
                                       _ptr(part), 1, int(is_swa), st)
            self._check("battn_decode", rc)
        elif rows <= 8 and rows * self.geom.group <= 32:
            rc = self.lib.battn_verify(self.h, _ptr(out), _ptr(q), _ptr(kvk), _ptr(kvv), _ptr(pos), None, None,
                                       _ptr(part), rows, 1, int(is_swa), st)
            self._check("battn_verify", rc)
        else:
            rc = self.lib.battn_prefill(self.h, _ptr(out), _ptr(q), _ptr(kvk), _ptr(kvv), _ptr(pos), _ptr(part),
                                        rows, int(is_swa), st)
            self._check("battn_prefill", rc)

    def launch_attn_ms(self, out, q, kvk, kvv, pos, kslot, act, part, rows: int, is_swa: bool = False,
                       rows_per_seq: int = 1):
        """Multi-slot attention: `rows` independent sequences (launch_attn_ms, bruce.cu:4158-4177);
        rows_per_seq > 1 runs a batched speculative verify."""
        st = self._stream()
        if rows_per_seq == 1:
            rc = self.lib.battn_decode(self.h, _ptr(out), _ptr(q), _ptr(kvk), _ptr(kvv), _ptr(pos), _ptr(kslot),
                                       _ptr(act), _ptr(part), rows, int(is_swa), st)
            self._check("battn_decode", rc)
        else:
            rc = self.lib.battn_verify(self.h, _ptr(out), _ptr(q), _ptr(kvk), _ptr(kvv), _ptr(pos), _ptr(kslot),
                                       _ptr(act), _ptr(part), rows_per_seq, rows, int(is_swa), st)
            self._check("battn_verify", rc)

    def decode_append(self, out, q, k, v, kvk, kvv, pos, part, kslot=None, act=None, is_swa: bool = False):
        """One row per sequence: append k, v ([n_seq][n_kv][head_dim] fp32) at pos[i] and attend, the append done by
        the decode kernel itself (battn_decode_append)."""
        rc = self.lib.battn_decode_append(self.h, _ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(kvk), _ptr(kvv), _ptr(pos),
                                          _ptr(kslot), _ptr(act), _ptr(part), pos.numel(), int(is_swa), self._stream())
        self._check("battn_decode_append", rc)

    def qkv_decode(self, out, q, k, v, sqk, cs, sn, kvk, kvv, pos, part, kslot=None, act=None, is_swa: bool = False,
                   theta_sel: int = 1):
        """One row per sequence: the QKV prologue (as qkv_prep), the append and the attention in one call whose decode
        kernel does all three (battn_qkv_decode); q, k, v are the raw fp32 rows."""
        rc = self.lib.battn_qkv_decode(self.h, _ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(sqk), _ptr(cs), _ptr(sn),
                                       int(theta_sel), _ptr(kvk), _ptr(kvv), _ptr(pos), _ptr(kslot), _ptr(act),
                                       _ptr(part), pos.numel(), int(is_swa), self._stream())
        self._check("battn_qkv_decode", rc)

    def decode_append_paged(self, out, q, k, v, pages, pos, part, ktab=None, act=None):
        rc = self.lib.battn_decode_append_paged(self.h, _ptr(out), _ptr(q), _ptr(k), _ptr(v), C.byref(pages), _ptr(pos),
                                                _ptr(ktab), _ptr(act), _ptr(part), pos.numel(), self._stream())
        self._check("battn_decode_append_paged", rc)

    def qkv_decode_paged(self, out, q, k, v, sqk, cs, sn, pages, pos, part, ktab=None, act=None, theta_sel: int = 1):
        rc = self.lib.battn_qkv_decode_paged(self.h, _ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(sqk), _ptr(cs), _ptr(sn),
                                             int(theta_sel), C.byref(pages), _ptr(pos), _ptr(ktab), _ptr(act), _ptr(part),
                                             pos.numel(), self._stream())
        self._check("battn_qkv_decode_paged", rc)

    def set_early_kv_stream(self, enable: bool):
        """Whether decode calls stream the cache tiles below their first position before the preceding kernel of
        the stream has finished (battn_set_early_kv_stream; off by default: the host must not let a kernel that
        writes positions or older cache rows directly precede an attention call)."""
        self._check("battn_set_early_kv_stream", self.lib.battn_set_early_kv_stream(self.h, int(enable)))

    def decode_noalloc(self, out, q, kvk, kvv, pos, kslot=None, act=None, is_swa: bool = False):
        """Decode attention without a caller-provided `part` buffer: the scratch is a fixed array
        inside the library (for hosts that cannot allocate device memory while serving)."""
        rc = self.lib.battn_decode_noalloc(self.h, _ptr(out), _ptr(q), _ptr(kvk), _ptr(kvv), _ptr(pos),
                                           _ptr(kslot), _ptr(act), pos.numel(), int(is_swa), self._stream())
        self._check("battn_decode_noalloc", rc)

    def attn_exact(self, out, q, kvk, kvv, pos, part, n_seq: int, rows: int, nsplit: int, is_swa: bool = False,
                   kslot=None, act=None):
        """The exact fp32 path (k_attn / k_attn_rows / k_attn_m + k_attn_combine_rows)."""
        rc = self.lib.battn_attend_exact(self.h, _ptr(out), _ptr(q), _ptr(kvk), _ptr(kvv), _ptr(pos), _ptr(kslot),
                                         _ptr(act), _ptr(part), n_seq, rows, nsplit, int(is_swa), self._stream())
        self._check("battn_attend_exact", rc)

    def attn_partials(self, rec, q, kvk, kvv, pos, part, rows: int = 1, batch: int = 1, is_swa: bool = False,
                      kslot=None, act=None):
        """Split records (o, m, l) instead of the normalised output (bruce.cu:781-783)."""
        rc = self.lib.battn_partials(self.h, _ptr(rec), _ptr(q), _ptr(kvk), _ptr(kvv), _ptr(pos), _ptr(kslot),
                                     _ptr(act), _ptr(part), rows, batch, int(is_swa), self._stream())
        self._check("battn_partials", rc)

    def attn_combine(self, out, parts, n_parts: int, n_rows: int):
        """k_attn_combine over records gathered from several devices (bruce.cu:992-1007)."""
        rc = self.lib.battn_merge(self.h, _ptr(out), _ptr(parts), n_parts, n_rows, self._stream())
        self._check("battn_merge", rc)

    # ---- paged cache of a full-causal layer ------------------------------------------------------------
    def alloc_pages(self, n_pages: int, page_len: int, table: torch.Tensor, fill: int | None = None):
        """A pool of `n_pages` pages of `page_len` positions (K and V) and its `battn_pages` descriptor; `table` is
        the int32 device tensor [n_tables][max_pages] the kernels read the page numbers from (the host may edit it
        between launches).  Returns (descriptor, pool_k, pool_v); keep the tensors alive with the descriptor."""
        n = C.c_size_t()
        self._check("battn_pages_pool_bytes", self.lib.battn_pages_pool_bytes(self.h, n_pages, page_len, C.byref(n)))
        mk = (lambda: torch.empty(n.value, dtype=torch.uint8, device=self.device)) if fill is None else \
             (lambda: torch.full((n.value,), fill, dtype=torch.uint8, device=self.device))
        pk, pv = mk(), mk()
        assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
        desc = capi.CPages(pk.data_ptr(), pv.data_ptr(), table.data_ptr(), n_pages, table.shape[0], table.shape[1],
                           page_len)
        return desc, pk, pv

    def pages_copy(self, pages, from_page: int, to_page: int):
        """Copy on write: one physical page's K and V records into another page."""
        self._check("battn_pages_copy", self.lib.battn_pages_copy(self.h, C.byref(pages), from_page, to_page,
                                                                  self._stream()))

    def kv_append_paged(self, pages, k, v, pos, ktab=None, act=None, rows: int = 1):
        self._check("battn_kv_append_paged", self.lib.battn_kv_append_paged(
            self.h, C.byref(pages), _ptr(k), _ptr(v), _ptr(pos), _ptr(ktab), _ptr(act), pos.numel(), rows,
            self._stream()))

    def qkv_prep_paged(self, q_out, q, k, v, sqk, cs, sn, pages, pos, ktab=None, act=None, rows: int = 1,
                       theta_sel: int = 1):
        """The fused prologue (qkv_prep) storing its K/V rows into a paged cache."""
        self._check("battn_qkv_prep_paged", self.lib.battn_qkv_prep_paged(
            self.h, _ptr(q_out), _ptr(q), _ptr(k), _ptr(v), _ptr(sqk), _ptr(cs), _ptr(sn), int(theta_sel),
            C.byref(pages), _ptr(pos), _ptr(ktab), _ptr(act), pos.numel(), rows, self._stream()))

    def attn_paged(self, out, q, pages, pos, part, rows: int = 1, ktab=None, act=None, table_row: int = 0):
        """Attention over a paged cache: one row per sequence (decode), 2..8 rows (verify) or a prompt chunk of the
        sequence with table row `table_row`; the dispatch of launch_attn_m / launch_attn_ms."""
        st = self._stream()
        n_seq = pos.numel()
        if rows == 1:
            rc = self.lib.battn_decode_paged(self.h, _ptr(out), _ptr(q), C.byref(pages), _ptr(pos), _ptr(ktab),
                                             _ptr(act), _ptr(part), n_seq, st)
            self._check("battn_decode_paged", rc)
        elif rows * self.geom.group <= 32:
            rc = self.lib.battn_verify_paged(self.h, _ptr(out), _ptr(q), C.byref(pages), _ptr(pos), _ptr(ktab),
                                             _ptr(act), _ptr(part), rows, n_seq, st)
            self._check("battn_verify_paged", rc)
        else:
            rc = self.lib.battn_prefill_paged(self.h, _ptr(out), _ptr(q), C.byref(pages), table_row, _ptr(pos),
                                              _ptr(part), rows, st)
            self._check("battn_prefill_paged", rc)

    def attn_exact_paged(self, out, q, pages, pos, part, n_seq: int, rows: int, nsplit: int, ktab=None, act=None):
        rc = self.lib.battn_attend_exact_paged(self.h, _ptr(out), _ptr(q), C.byref(pages), _ptr(pos), _ptr(ktab),
                                               _ptr(act), _ptr(part), n_seq, rows, nsplit, self._stream())
        self._check("battn_attend_exact_paged", rc)

    # ---- the step after attention ------------------------------------------------------------------------
    def gate_norm(self, dst, aout, gate, sgate, xq, xd, xsum, rows: int):
        """k_gate_norm_vec4 (bruce.cu:1526): sigmoid gate, L2 norm, q8 activation copy; dst may be None."""
        rc = self.lib.battn_gate_norm(self.h, _ptr(dst), _ptr(aout), _ptr(gate), _ptr(sgate), _ptr(xq), _ptr(xd),
                                      _ptr(xsum), rows, self._stream())
        self._check("battn_gate_norm", rc)

    def prefill_gate_norm(self, dst, q, kvk, kvv, pos, part, gate, sgate, xq, xd, xsum, rows: int, is_swa: bool = False):
        """Prompt-chunk attention fused with the gate-norm step (k_combine_gate_norm_rows_opt, bruce.cu:1577)."""
        rc = self.lib.battn_prefill_gate_norm(self.h, _ptr(dst), _ptr(q), _ptr(kvk), _ptr(kvv), _ptr(pos), _ptr(part),
                                              _ptr(gate), _ptr(sgate), _ptr(xq), _ptr(xd), _ptr(xsum), rows, int(is_swa),
                                              self._stream())
        self._check("battn_prefill_gate_norm", rc)

    # ---- one sequence split by position range across devices ----------------------------------------
    def xchg_create(self, rank: int, world: int, max_rows: int = 8):
        """This device's receive area for the cross-device exchange of split records.  Returns (exchange, its
        IPC handle as bytes) -- the handle goes to the other processes."""
        x = C.c_void_p()
        buf = C.create_string_buffer(capi.IPC_HANDLE_BYTES)
        self._check("battn_xchg_create", self.lib.battn_xchg_create(self.h, rank, world, max_rows, C.byref(x), buf))
        return x, bytes(buf.raw)

    def xchg_connect(self, x, all_handles: bytes):
        self._check("battn_xchg_connect", self.lib.battn_xchg_connect(x, all_handles))

    def xchg_area(self, x):
        ptr, n = C.c_void_p(), C.c_size_t()
        self._check("battn_xchg_area", self.lib.battn_xchg_area(x, C.byref(ptr), C.byref(n)))
        return ptr.value, n.value

    def xchg_connect_ptrs(self, x, ptrs):
        arr = (C.c_void_p * len(ptrs))(*ptrs)
        self._check("battn_xchg_connect_ptrs", self.lib.battn_xchg_connect_ptrs(x, arr))

    def xchg_set_wait_polls(self, x, polls: int):
        self._check("battn_xchg_set_wait_polls", self.lib.battn_xchg_set_wait_polls(x, polls))

    def xchg_destroy(self, x):
        self.lib.battn_xchg_destroy(x)

    def attn_partials_push(self, x, out, q, kvk, kvv, pos, part, epoch, rows: int = 1, batch: int = 1,
                           is_swa: bool = False, kslot=None, act=None, epoch_advance: int = 1):
        """Decode on this device's shard, push the merged (o, m, l) records to every device of the group and --
        when `out` is given -- wait for the peers' records of the same step and merge them (one decode launch + one
        merge launch).  `epoch`: int32 device tensor holding this device's step counter (advanced on the device)."""
        rc = self.lib.battn_partials_push(self.h, x, _ptr(out), _ptr(q), _ptr(kvk), _ptr(kvv), _ptr(pos), _ptr(kslot),
                                          _ptr(act), _ptr(part), rows, batch, int(is_swa), _ptr(epoch),
                                          int(epoch_advance), self._stream())
        self._check("battn_partials_push", rc)

    def attn_merge_wait(self, x, out, n_rows: int, epoch):
        rc = self.lib.battn_merge_wait(self.h, x, _ptr(out), n_rows, _ptr(epoch), self._stream())
        self._check("battn_merge_wait", rc)

    # ---- diagnostics -------------------------------------------------------------------------------
    def device_status(self, clear: bool = True) -> int:
        bits = C.c_int()
        self._check("battn_device_status", self.lib.battn_device_status(self.h, C.byref(bits), int(clear)))
        return bits.value

    def profile_start(self, max_launches: int):
        """Bracket the main kernel of every following attention call with CUDA events."""
        self._check("battn_profile_start", self.lib.battn_profile_start(self.h, max_launches))
        self._prof_cap = max_launches

    def profile_stop(self):
        """Elapsed milliseconds of each bracketed launch since profile_start, in call order."""
        buf = (C.c_float * self._prof_cap)()
        n = C.c_int()
        self._check("battn_profile_stop", self.lib.battn_profile_stop(self.h, buf, self._prof_cap, C.byref(n)))
        return [buf[i] for i in range(min(n.value, self._prof_cap))]

    def launch_count(self) -> int:
        return int(self.lib.battn_launch_count(self.h))
