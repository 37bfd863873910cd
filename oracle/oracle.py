"""ctypes front end of the CPU oracle (battn_oracle.c) plus an independent numpy restatement.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's CPU
baseline leg.  The product package never imports this module and has no CPU path.

The numpy functions (`np_quant_records`, `np_attend`) restate the same reference arithmetic
(engine/src/bruce.cu:698-710 quantiser, :713-785 attention) a second time, independently of the C
file, so that the two can be checked against each other.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libbattn_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile battn_oracle.c with the Makefile beside it (gcc, -O2, no fast-math)."""
    src = os.path.join(_HERE, "battn_oracle.c")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
        return _LIB_PATH
    subprocess.run(["make", "-C", _HERE, "-B", "libbattn_oracle.so"], check=True,
                   stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


class _Geom(C.Structure):
    _fields_ = [("n_head", C.c_int), ("n_kv", C.c_int), ("head_dim", C.c_int),
                ("window", C.c_int), ("slot_ctx", C.c_int), ("n_slots", C.c_int),
                ("softmax_scale", C.c_float)]


@dataclass(frozen=True)
class Geom:
    """Attention geometry.  G_B is the graded one (32/8/128, window 4096); G_R is the reference's
    native one (16/4/256, window 1024; bruce.cu:43-53)."""
    n_head: int = 32
    n_kv: int = 8
    head_dim: int = 128
    window: int = 4096
    slot_ctx: int = 8192
    n_slots: int = 1
    softmax_scale: float = 0.0

    @property
    def rec(self) -> int:
        return self.head_dim + 2 * (self.head_dim // 32)

    @property
    def group(self) -> int:
        return self.n_head // self.n_kv

    def pstride(self, is_swa: bool) -> int:
        return 2 * self.window if is_swa else self.slot_ctx

    def layer_bytes(self, is_swa: bool) -> int:
        return self.n_slots * self.pstride(is_swa) * self.n_kv * self.rec

    def c(self) -> _Geom:
        return _Geom(self.n_head, self.n_kv, self.head_dim, self.window, self.slot_ctx,
                     self.n_slots, self.softmax_scale)


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.oracle_f32_to_f16.restype = C.c_uint16
        L.oracle_f32_to_f16.argtypes = [C.c_float]
        L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.oracle_kv_layer_bytes.restype = C.c_size_t
        L.oracle_kv_layer_bytes.argtypes = [C.POINTER(_Geom), C.c_int]
        L.oracle_quant_block32.restype = None
        L.oracle_quant_block32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.oracle_kv_append.restype = C.c_int
        L.oracle_kv_append.argtypes = [C.POINTER(_Geom)] + [C.c_void_p] * 7 + [C.c_int] * 3
        L.oracle_qkv_prep.restype = C.c_int
        L.oracle_qkv_prep.argtypes = ([C.POINTER(_Geom)] + [C.c_void_p] * 6 + [C.c_int] + [C.c_void_p] * 5 +
                                      [C.c_int] * 3)
        L.oracle_gate_norm.restype = C.c_int
        L.oracle_gate_norm.argtypes = [C.c_int, C.c_int] + [C.c_void_p] * 7
        L.oracle_attend.restype = C.c_int
        L.oracle_attend.argtypes = [C.POINTER(_Geom)] + [C.c_void_p] * 8 + [C.c_int] * 6
        L.oracle_attend_f32.restype = C.c_int
        L.oracle_attend_f32.argtypes = [C.POINTER(_Geom)] + [C.c_void_p] * 7 + [C.c_int] * 4
        L.oracle_merge.restype = None
        L.oracle_merge.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.oracle_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _ints(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def new_cache(g: Geom, is_swa: bool, fill: int = 0) -> np.ndarray:
    return np.full(g.layer_bytes(is_swa), fill, dtype=np.uint8)


def kv_append(g: Geom, k, v, kvk, kvv, pos, kslot=None, act=None, rows=1, is_swa=False):
    """k, v: float32 [n_seq][rows][n_kv][head_dim].  Writes into the uint8 caches in place."""
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    pos, kslot, act = _ints(pos), _ints(kslot), _ints(act)
    n_seq = pos.size
    gc = g.c()
    rc = lib().oracle_kv_append(C.byref(gc), _p(k), _p(v), _p(kvk), _p(kvv), _p(pos), _p(kslot),
                                _p(act), n_seq, rows, int(is_swa))
    if rc:
        raise ValueError(f"oracle_kv_append failed: {rc}")


def qkv_prep(g: Geom, q, k, v, sqk, cs, sn, kvk, kvv, pos, kslot=None, act=None, rows=1, is_swa=False,
             theta_sel=1):
    """The reference's QKV prologue + append (bruce.cu:1732-1812, 1835-1918).  q: float32
    [n_seq][rows][n_head][head_dim], k, v: [n_seq][rows][n_kv][head_dim], sqk: [n_head][head_dim],
    cs, sn: [n_seq*rows][head_dim] (two tables of head_dim/2).  Returns the prepared q; writes the caches."""
    q = np.array(q, dtype=np.float32, order="C", copy=True)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    sqk = np.ascontiguousarray(sqk, dtype=np.float32)
    cs = np.ascontiguousarray(cs, dtype=np.float32)
    sn = np.ascontiguousarray(sn, dtype=np.float32)
    pos, kslot, act = _ints(pos), _ints(kslot), _ints(act)
    n_seq = pos.size
    assert cs.size == n_seq * rows * g.head_dim and sn.size == cs.size
    gc = g.c()
    rc = lib().oracle_qkv_prep(C.byref(gc), _p(q), _p(k), _p(v), _p(sqk), _p(cs), _p(sn), int(theta_sel),
                               _p(kvk), _p(kvv), _p(pos), _p(kslot), _p(act), n_seq, rows, int(is_swa))
    if rc:
        raise ValueError(f"oracle_qkv_prep failed: {rc}")
    return q


def rope_tables(head_dim: int, positions) -> tuple:
    """cos/sin tables in the reference's layout (bruce.cu:1641-1654): per row [theta 1e7 | theta 1e4], head_dim/2
    entries each, computed in double and rounded once (the reference evaluates powf/cosf/sinf in fp32 on the
    device, so its tables differ from these in the last bits and, at large positions, by the fp32 error of the
    angle itself; the prologue takes the tables as an input for that reason)."""
    p = np.asarray(positions, dtype=np.float64).reshape(-1, 1)
    i = np.arange(head_dim // 2, dtype=np.float64)
    th1 = p * (1e7 ** (-2.0 * i / head_dim))
    th2 = p * (1e4 ** (-2.0 * i / head_dim))
    cs = np.concatenate([np.cos(th1), np.cos(th2)], axis=1).astype(np.float32)
    sn = np.concatenate([np.sin(th1), np.sin(th2)], axis=1).astype(np.float32)
    return cs, sn


def gate_norm(aout, gate, sgate):
    """k_gate_norm_vec4 (bruce.cu:1526) restated: aout, gate float32 [rows][n], sgate [n] ->
    (dst float32 [rows][n], xq int8 [rows][n], xd float32 [rows][n/32], xsum int32 [rows][n/32])."""
    aout = np.ascontiguousarray(aout, dtype=np.float32)
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    sgate = np.ascontiguousarray(sgate, dtype=np.float32)
    rows, n = aout.shape
    dst = np.zeros((rows, n), np.float32)
    xq = np.zeros((rows, n), np.int8)
    xd = np.zeros((rows, n // 32), np.float32)
    xsum = np.zeros((rows, n // 32), np.int32)
    rc = lib().oracle_gate_norm(n, rows, _p(aout), _p(gate), _p(sgate), _p(dst), _p(xq), _p(xd), _p(xsum))
    if rc:
        raise ValueError(f"oracle_gate_norm failed: {rc}")
    return dst, xq, xd, xsum


def attend(g: Geom, q, kvk, kvv, pos, kslot=None, act=None, rows=1, is_swa=False,
           key_lo=0, key_hi=2**31 - 1, records=False, nthreads=0):
    """q: float32 [n_seq][rows][n_head][head_dim] -> same-shape output (or [..., head_dim+2]
    split records when records=True).  Double accumulation."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    pos, kslot, act = _ints(pos), _ints(kslot), _ints(act)
    n_seq = pos.size
    HD = g.head_dim
    shape = (n_seq, rows, g.n_head, HD + 2 if records else HD)
    res = np.zeros(shape, dtype=np.float32)
    gc = g.c()
    rc = lib().oracle_attend(C.byref(gc), None if records else _p(res), _p(res) if records else None,
                             _p(q), _p(kvk), _p(kvv), _p(pos), _p(kslot), _p(act), n_seq, rows,
                             int(is_swa), int(key_lo), int(key_hi), int(nthreads))
    if rc:
        raise ValueError(f"oracle_attend failed: {rc}")
    return res


def attend_f32(g: Geom, q, kvk, kvv, pos, kslot=None, act=None, rows=1, is_swa=False, nsplit=1):
    q = np.ascontiguousarray(q, dtype=np.float32)
    pos, kslot, act = _ints(pos), _ints(kslot), _ints(act)
    n_seq = pos.size
    res = np.zeros((n_seq, rows, g.n_head, g.head_dim), dtype=np.float32)
    gc = g.c()
    rc = lib().oracle_attend_f32(C.byref(gc), _p(res), _p(q), _p(kvk), _p(kvv), _p(pos), _p(kslot),
                                 _p(act), n_seq, rows, int(is_swa), int(nsplit))
    if rc:
        raise ValueError(f"oracle_attend_f32 failed: {rc}")
    return res


def merge(parts: np.ndarray) -> np.ndarray:
    """parts: float32 [n_parts][..., head_dim+2] -> [..., head_dim]."""
    parts = np.ascontiguousarray(parts, dtype=np.float32)
    n_parts, HD = parts.shape[0], parts.shape[-1] - 2
    n_items = int(np.prod(parts.shape[1:-1]))
    out = np.zeros(parts.shape[1:-1] + (HD,), dtype=np.float32)
    lib().oracle_merge(_p(out), _p(parts), n_parts, n_items, HD)
    return out


def f32_to_f16_bits(x: float) -> int:
    return int(lib().oracle_f32_to_f16(C.c_float(x)))


# ----------------------------------------------------------------------------------------------
# Independent numpy restatement (no shared code with the C file)
# ----------------------------------------------------------------------------------------------

def np_quant_records(x: np.ndarray) -> np.ndarray:
    """x float32 [..., HD] -> uint8 [..., HD + HD/16] records, scales first (bruce.cu:698-710)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    HD = x.shape[-1]
    nblk = HD // 32
    xb = x.reshape(x.shape[:-1] + (nblk, 32))
    amax = np.max(np.abs(xb), axis=-1).astype(np.float32)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, (np.float32(1.0) / d).astype(np.float32), np.float32(0.0)).astype(np.float32)
    qv = np.rint((xb * inv[..., None]).astype(np.float32)).astype(np.int8)     # half-even, no clamp
    scales = d.astype(np.float16)                                              # RNE like __float2half
    rec = np.empty(x.shape[:-1] + (HD + 2 * nblk,), dtype=np.uint8)
    rec[..., :2 * nblk] = scales.view(np.uint8).reshape(x.shape[:-1] + (2 * nblk,))
    rec[..., 2 * nblk:] = qv.view(np.uint8).reshape(x.shape[:-1] + (HD,))
    return rec


def np_dequant_records(rec: np.ndarray, HD: int) -> np.ndarray:
    nblk = HD // 32
    scales = np.ascontiguousarray(rec[..., :2 * nblk]).view(np.float16).astype(np.float32)
    qv = np.ascontiguousarray(rec[..., 2 * nblk:]).view(np.int8).astype(np.float32)
    return (qv.reshape(rec.shape[:-1] + (nblk, 32)) * scales[..., None]).reshape(rec.shape[:-1] + (HD,))


def np_cache_view(g: Geom, cache: np.ndarray, is_swa: bool) -> np.ndarray:
    """uint8 cache -> view [slot][kvh][pstride][rec]."""
    return cache.reshape(g.n_slots, g.n_kv, g.pstride(is_swa), g.rec)


def np_attend(g: Geom, q, kvk, kvv, pos, kslot=None, rows=1, is_swa=False) -> np.ndarray:
    """Whole-softmax attention in float64, the style of tools/ref_np.py:237-250."""
    q = np.asarray(q, dtype=np.float64)
    pos = np.asarray(pos).reshape(-1)
    HD, G = g.head_dim, g.group
    scale = g.softmax_scale if g.softmax_scale else 1.0 / np.sqrt(HD)
    K = np_cache_view(g, kvk, is_swa)
    V = np_cache_view(g, kvv, is_swa)
    out = np.zeros((pos.size, rows, g.n_head, HD), dtype=np.float64)
    for i in range(pos.size):
        slot = 0 if kslot is None else int(kslot[i])
        for r in range(rows):
            p = int(pos[i]) + r
            lo = max(0, p + 1 - g.window) if is_swa else 0
            keys = np.arange(lo, p + 1)
            idx = keys & (2 * g.window - 1) if is_swa else keys
            for h in range(g.n_head):
                kh = h // G
                ks = np_dequant_records(K[slot, kh, idx], HD).astype(np.float64)
                vs = np_dequant_records(V[slot, kh, idx], HD).astype(np.float64)
                sc = (ks @ q[i, r, h]) * scale
                w = np.exp(sc - sc.max())
                out[i, r, h] = (w / w.sum()) @ vs
    return out.astype(np.float32)


def _np_fma(a, b, c):
    """fp32 fused multiply-add through float64 (the product of two floats is exact in double)."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def np_qkv_prologue(x: np.ndarray, c: np.ndarray, s: np.ndarray, extra=None) -> np.ndarray:
    """Independent numpy restatement of the prologue of one tensor of heads: x [..., HD] float32, c, s
    broadcastable [..., HD/2].  Same fp32 operation order as oracle_qkv_prep (see battn_oracle.c)."""
    f32 = np.float32
    x = np.asarray(x, dtype=f32)
    HD = x.shape[-1]
    H2, VEC = HD // 2, HD // 64
    def partial(y):                                   # y [..., 32, VEC]
        t = _np_fma(y[..., 0], y[..., 0], (y[..., 1] * y[..., 1]).astype(f32))
        for j in range(2, VEC):
            t = _np_fma(y[..., j], y[..., j], t)
        return t
    lane = (partial(x[..., :H2].reshape(x.shape[:-1] + (32, VEC))) +
            partial(x[..., H2:].reshape(x.shape[:-1] + (32, VEC)))).astype(f32)
    for o in (16, 8, 4, 2, 1):
        nxt = lane.copy()
        nxt[..., :32 - o] = (lane[..., :32 - o] + lane[..., o:]).astype(f32)
        lane = nxt
    ss = lane[..., 0]
    a = ((ss / f32(HD)).astype(f32) + f32(f32(1e-6) / f32(HD))).astype(f32)
    norm = ((f32(1.0) / np.sqrt(a).astype(f32)).astype(f32) * f32(f32(1.0) / np.sqrt(f32(HD)))).astype(f32)[..., None]
    x0, x1 = x[..., :H2], x[..., H2:]
    lo = (_np_fma(x0, c, -(x1 * s).astype(f32)) * norm).astype(f32)
    hi = (_np_fma(x0, s, (x1 * c).astype(f32)) * norm).astype(f32)
    if extra is not None:
        lo = (lo * extra[..., :H2]).astype(f32)
        hi = (hi * extra[..., H2:]).astype(f32)
    return np.concatenate([lo, hi], axis=-1)
