// The work cut of the split-K attention kernels (flash-decode, both verify kernels) and the matching record ranges of
// the merge kernel: plain integer logic, shared by device code and by a host test (tests/host/cut_test.cpp).
//
// Work unit = (sequence, kv head, tile); `cum[i]` = tiles per kv head of the sequences before i.  Tiles are numbered
// g = Hkv * cum[i] + kvh * nt_i + t.  A CTA owns tiles [g0, g1); the tiles of one (sequence, kv head) item inside a
// share are a piece; a CTA writes the split record of its piece of item `it` at slot `cta + it`.
#pragma once

#ifdef __CUDACC__
#define BATTN_HD __host__ __device__ __forceinline__
#else
#define BATTN_HD inline
#endif

namespace battn {
namespace fd {

struct Piece {
    int i, kvh, tl, n;   // sequence, kv head, first tile (relative to the item), tiles in this piece
};

// The piece that starts at global tile index g (g < g1): every thread of the CTA computes the same.
BATTN_HD Piece locate(int g, int g1, const int* cum, int n_seq, int Hkv) {
    int lo = 0, hi = n_seq - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (Hkv * cum[mid] <= g) lo = mid; else hi = mid - 1;
    }
    Piece pc;
    pc.i = lo;
    const int nt = cum[lo + 1] - cum[lo];
    const int rem = g - Hkv * cum[lo];
    pc.kvh = rem / nt;
    pc.tl = rem - pc.kvh * nt;
    const int left = nt - pc.tl, room = g1 - g;
    pc.n = left < room ? left : room;
    return pc;
}

// The share of CTA `cta` of `n_cta`: tiles [g0, g1), `per` tiles per CTA; g0 == g1: no work.  One sequence (cph > 0):
// the CTAs are dealt to the kv heads in groups of cph and no share crosses a head -- a CTA whose share straddles two
// heads runs two pieces (Q staging, in-CTA merge and record twice) and is the last to finish.  Several sequences: one
// cut through the whole order.
struct Share {
    int per, g0, g1;
};
BATTN_HD Share cut_share(const int* cum, int n_seq, int Hkv, int cph, int cta, int n_cta) {
    Share sh;
    const int total = Hkv * cum[n_seq];
    if (cph > 0) {
        const int nt = cum[1], kvh = cta / cph, c = cta - kvh * cph;
        sh.per = (nt + cph - 1) / cph;
        if (sh.per < 1) sh.per = 1;
        const bool none = kvh >= Hkv || c * sh.per >= nt;
        const int end = (c + 1) * sh.per < nt ? (c + 1) * sh.per : nt;
        sh.g0 = none ? total : kvh * nt + c * sh.per;
        sh.g1 = none ? total : kvh * nt + end;
    } else {
        sh.per = (int)(((long long)total + n_cta - 1) / n_cta);
        if (sh.per < 1) sh.per = 1;
        const long long g0l = (long long)cta * sh.per;
        sh.g0 = (int)(g0l < total ? g0l : total);
        sh.g1 = sh.g0 + sh.per < total ? sh.g0 + sh.per : total;
    }
    return sh;
}

// The merge side: the CTAs clo..chi that hold a piece of the item (kv head `kvh` of a sequence whose tiles start at
// cum value c0 and count nt > 0), given the cut's `per`.
BATTN_HD void item_ctas(int cph, int per, int Hkv, int c0, int nt, int kvh, int& clo, int& chi) {
    if (cph > 0) {
        clo = kvh * cph;
        chi = clo + (nt + per - 1) / per - 1;
    } else {
        const long long t0 = (long long)Hkv * c0 + (long long)kvh * nt, t1 = t0 + nt;
        clo = (int)(t0 / per);
        chi = (int)((t1 - 1) / per);
    }
}

}  // namespace fd
}  // namespace battn
