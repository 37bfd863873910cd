// The exact fp32 attention path and the log-sum-exp merge.
//
// k_attn_exact restates, for run-time geometry, what k_attn / k_attn_rows / k_attn_m compute
// (engine/src/bruce.cu:713-785, 1921-1997, 2087-2143): per-key online softmax in fp32, one warp per
// query head, the reference's key-split rule (:724-729) and its split record (o[HD], m, l).
// It is the slow, tensor-core-free path used to validate the fast kernels at sizes the CPU oracle
// cannot reach, and the reference's own "--prefill-tc 0" behaviour.
//
// k_merge is the merge of k_attn_combine / k_attn_combine_rows (bruce.cu:992-1007, 1999-2016) for the
// reference's regular [row][kvh][split][head] record layout and for records gathered from several
// devices; k_merge_balanced merges the work-balanced records of the flash-decode kernels.
#pragma once
#include "common.cuh"
#include "work_cut.h"

namespace battn {

struct ExactParams {
    const void* q;
    const uint8_t* kvk;
    const uint8_t* kvv;
    const int* pos;
    const int* kslot;
    const int* act;
    float* part;          // [(seq*rows + r)][kvh][split][head-in-group][HD+2]
    int n_seq, rows, Hq, Hkv, G;
    int W, pstride, ring_mask, slot_ctx, n_slots, is_swa;
    int q_f16;
    float scale;
    int* status;
    Paging pg;
};

template <int HD>
__global__ void __launch_bounds__(256) k_attn_exact(const ExactParams P) {
    constexpr int NBLK = HD / 32, REC = HD + 2 * NBLK, DPL = HD / 32;   // dims per lane
    const int item = blockIdx.x, i = item / P.Hkv, kvh = item % P.Hkv;
    const int split = blockIdx.y, ns = gridDim.y, r = blockIdx.z;
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const SeqRange sr = seq_range(P.pos, P.kslot, P.act, i, P.rows, P.is_swa, P.W, P.slot_ctx, P.n_slots, P.status);
    if (!sr.active) return;

    const int p = sr.p0 + r, kend = p + 1;
    const int kstart = P.is_swa ? max(0, kend - P.W) : 0;
    const int nkeys = kend - kstart, per = (nkeys + ns - 1) / ns;      // bruce.cu:727-729
    const int a0 = kstart + split * per, a1 = min(kend, a0 + per);

    const size_t rowidx = (size_t)i * P.rows + r;
    const int hq = kvh * P.G + h;
    float qv[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
        const size_t qi = (rowidx * P.Hq + hq) * HD + lane * DPL + j;
        qv[j] = P.q_f16 ? __half2float(reinterpret_cast<const __half*>(P.q)[qi])
                        : reinterpret_cast<const float*>(P.q)[qi];
    }
    const int blk = (lane * DPL) >> 5;
    const size_t hb = P.pg.table ? 0 : ((size_t)sr.slot * P.Hkv + kvh) * P.pstride * (size_t)REC;
    const uint8_t* kb = P.kvk + hb;
    const uint8_t* vb = P.kvv + hb;
    const int off = 2 * NBLK + lane * DPL;

    float m = NEG_BIG, l = 0.f, o[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) o[j] = 0.f;

    for (int key = a0; key < a1; ++key) {
        const size_t ro = (P.pg.table ? kv_rec_index(P.pg, sr.slot, kvh, P.Hkv, P.pstride, key, P.status)
                                      : (size_t)(key & P.ring_mask)) * REC;   // ring slot (bruce.cu:740)
        const uint8_t* kk = kb + ro;
        const uint8_t* vv = vb + ro;
        const float d = __half2float(reinterpret_cast<const __half*>(kk)[blk]);
        const float dv = __half2float(reinterpret_cast<const __half*>(vv)[blk]);
        uint32_t kw[DPL / 4], vw[DPL / 4];
        if (DPL == 4) {
            kw[0] = *reinterpret_cast<const uint32_t*>(kk + off);
            vw[0] = *reinterpret_cast<const uint32_t*>(vv + off);
        } else {
            const uint2 a = *reinterpret_cast<const uint2*>(kk + off);
            const uint2 b = *reinterpret_cast<const uint2*>(vv + off);
            kw[0] = a.x; kw[DPL / 4 - 1] = a.y;
            vw[0] = b.x; vw[DPL / 4 - 1] = b.y;
        }
        float kq[DPL], vq[DPL];
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
            kq[j] = (float)(int)(int8_t)((kw[j >> 2] >> (8 * (j & 3))) & 0xffu);   // bruce.cu:748
            vq[j] = (float)(int)(int8_t)((vw[j >> 2] >> (8 * (j & 3))) & 0xffu);
        }
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < DPL; ++j) dot = fmaf(qv[j], d * kq[j], dot);   // bruce.cu:749
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
        dot *= P.scale;
        const float mnew = fmaxf(m, dot);
        const float pw = __expf(dot - mnew), corr = __expf(m - mnew);   // bruce.cu:757-761
        l = l * corr + pw;
        m = mnew;
#pragma unroll
        for (int j = 0; j < DPL; ++j) o[j] = fmaf(o[j], corr, pw * dv * vq[j]);   // :769
    }
    float* base = P.part + ((((rowidx * P.Hkv + kvh) * ns + split) * P.G + h) * (size_t)(HD + 2));
#pragma unroll
    for (int j = 0; j < DPL; ++j) base[lane * DPL + j] = o[j];
    if (lane == 0) { base[HD] = m; base[HD + 1] = l; }                 // bruce.cu:781-783
}

// ------------------------------------------------------------------------------------------------

enum { MERGE_REGULAR = 0, MERGE_GATHERED = 1 };

// Exchange of split records between the devices that hold the position shards of ONE sequence.
// Every device owns a receive area, mapped into all peers: records [2 parities][world][max_items], a record being
// HD + 2 payload words (o[HD], m in log2 units, l) EACH PAIRED WITH THE STEP NUMBER: 16-byte units
// {word, step, word, step}.  Device `rank` pushes its merged record of item (row, head) for step `epoch` into slot
// [epoch & 1][rank][item] of EVERY device (its own included) with plain 16-byte stores and nothing else: no fence and
// no separate flag.  A reader polls the units it needs until their step numbers have reached its epoch -- an 8-byte
// half of a unit arrives whole, so a word that carries the step's number is the step's word (the low-latency
// protocol of collective libraries for small messages).  One trip over the link instead of store, fence round trip
// and flag store.  Two record buffers suffice: a device cannot push step e + 2 before its own merge of step e + 1
// completed, which needed every peer's push of e + 1, which those peers issue after their merge of step e.
constexpr int XCHG_MAX_WORLD = 8;
struct XchgView {
    uint8_t* area[XCHG_MAX_WORLD];  // receive area of device d as mapped HERE (area[rank] is the local one), or null
    int world, rank, max_items;
    const int* epoch_ptr;           // device-resident step number, advanced by the decode kernel of the same call
    unsigned wait_polls;            // bound of the spin (polls of ~100 ns)
    int push, wait;                 // which halves of the exchange this launch performs
};

template <int HD>
__host__ __device__ constexpr size_t xchg_record_bytes() { return (size_t)(HD + 2) * 8; }

__device__ __forceinline__ void st_unit(uint8_t* p, float a, float b, int epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(p), "r"(__float_as_uint(a)), "r"(epoch),
                 "r"(__float_as_uint(b)) : "memory");
}
__device__ __forceinline__ uint4 ld_unit(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool unit_ready(const uint4& v, int epoch) {
    return (int)v.y - epoch >= 0 && (int)v.w - epoch >= 0;
}

// Pushes float4 `dq` of this device's record of `item` (and, with_ml, its (m, l)) into device `d`'s receive area.
template <int HD>
__device__ __forceinline__ void xchg_push(const XchgView& X, int epoch, int item, int d, int dq, const float4& o,
                                          bool with_ml, float m, float l) {
    uint8_t* dst = X.area[d] + (((size_t)(epoch & 1) * X.world + X.rank) * X.max_items + item) * xchg_record_bytes<HD>();
    st_unit(dst + 32 * dq, o.x, o.y, epoch);
    st_unit(dst + 32 * dq + 16, o.z, o.w, epoch);
    if (with_ml) st_unit(dst + 8 * HD, m, l, epoch);
}

// Polls (bounded) the local receive area until float4 `dq` and (m, l) of device `r`'s record of `item` for the step
// have landed, and returns them.  False when the wait ran out.
template <int HD>
__device__ __forceinline__ bool xchg_poll(const XchgView& X, int epoch, int item, int r, int dq, float4& o, float2& ml) {
    const uint8_t* src = X.area[X.rank] + (((size_t)(epoch & 1) * X.world + r) * X.max_items + item) * xchg_record_bytes<HD>();
    for (unsigned it = 0; it < X.wait_polls; ++it) {
        const uint4 a = ld_unit(src + 32 * dq), b = ld_unit(src + 32 * dq + 16), c = ld_unit(src + 8 * HD);
        if (unit_ready(a, epoch) && unit_ready(b, epoch) && unit_ready(c, epoch)) {
            o = make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
            ml = make_float2(__uint_as_float(c.x), __uint_as_float(c.z));
            return true;
        }
        __nanosleep(100);
    }
    return false;
}

// One step of the merge of the devices' records, in device order (both callers run exactly this sequence).
struct XchgAcc {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    float L = 0.f;
    __device__ __forceinline__ void add(const float4& o, float m, float l, float M) {
        const float w = fast_exp2(m - M);
        L = fmaf(l, w, L);
        a.x = fmaf(o.x, w, a.x); a.y = fmaf(o.y, w, a.y); a.z = fmaf(o.z, w, a.z); a.w = fmaf(o.w, w, a.w);
    }
    __device__ __forceinline__ void store(void* out, int out_f16, size_t oi) const {
        const float il = L > 0.f ? 1.f / L : 0.f;
        if (out_f16) {
            const __half2 x = __floats2half2_rn(a.x * il, a.y * il), y = __floats2half2_rn(a.z * il, a.w * il);
            *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + oi) =
                make_uint2(*reinterpret_cast<const uint32_t*>(&x), *reinterpret_cast<const uint32_t*>(&y));
        } else {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + oi) = make_float4(a.x * il, a.y * il, a.z * il, a.w * il);
        }
    }
};

struct MergeParams {
    int mode;              // k_merge only: MERGE_REGULAR or MERGE_GATHERED
    const float* part;     // records
    void* out;             // normalised output (out_f16 ? half : float), or null
    float* rec_out;        // merged record [row][head][HD+2] in natural-log units, or null
    int n_rows;            // total rows = n_seq * rows
    int rows;              // rows per sequence
    int Hq, Hkv, G;
    int count;             // REGULAR: splits; GATHERED: parts
    int log2_domain;       // records carry m in log2 units (flash-decode partials)
    int out_f16;
    // REGULAR only: skip rows of inactive sequences
    const int* pos; const int* kslot; const int* act;
    int is_swa, W, slot_ctx, n_slots;
    int* status;
    // k_merge_balanced only: header written by the flash-decode kernel: {tiles_per_cta, total, cum[n_seq+1]}
    const int* hdr;
    // k_merge_balanced, single sequence behind an early-streaming decode kernel: the work cut is recomputed from the
    // positions before the wait (pre_grid CTAs, pre_tile keys per tile) instead of read from the header after it
    int pre_grid, pre_tile;
    int cph;               // the decode kernel's cut: > 0: one sequence, cph CTAs per kv head; 0: linear
    // sequence split across devices (k_merge_balanced as the pushing epilogue, k_merge_wait): see XchgView
    XchgView xchg;
};

constexpr int MERGE_THREADS = 256;
constexpr int MERGE_MAX_COUNT = 1024;     // records merged per (row, head)

// One block per (row, head).  The records are read in three block-wide phases (max, weights and
// denominator, weighted sum) with every load independent of the others, so the latency of the record
// reads is paid a few times per block instead of once per split.
template <int HD>
__global__ void __launch_bounds__(MERGE_THREADS) k_merge(const MergeParams P) {
    __shared__ float s_m[MERGE_MAX_COUNT];       // m_s, then the weight w_s
    __shared__ float s_l[MERGE_MAX_COUNT];
    __shared__ float s_red[MERGE_THREADS / 32];
    __shared__ float2 s_acc[MERGE_THREADS];
    const int hq = blockIdx.x % P.Hq, rowidx = blockIdx.x / P.Hq;
    const int i = rowidx / P.rows;
    const int kvh = hq / P.G, h = hq % P.G;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_wait();                                  // (a no-op unless launched with programmatic stream serialisation)
    pdl_trigger();
    const float* base;
    size_t stride;
    int count;
    if (P.mode == MERGE_REGULAR) {
        const SeqRange sr = seq_range(P.pos, P.kslot, P.act, i, P.rows, P.is_swa, P.W, P.slot_ctx, P.n_slots, P.status);
        if (!sr.active) return;
        count = P.count;
        base = P.part + (((size_t)rowidx * P.Hkv + kvh) * count * P.G + h) * (size_t)(HD + 2);
        stride = (size_t)P.G * (HD + 2);
    } else {                                     // MERGE_GATHERED
        count = P.count;
        base = P.part + ((size_t)rowidx * P.Hq + hq) * (size_t)(HD + 2);
        stride = (size_t)P.n_rows * P.Hq * (HD + 2);
    }
    count = min(count, MERGE_MAX_COUNT);

    // phase 1: (m, l) of every record, block max of m
    float mx = NEG_BIG;
    for (int s = tid; s < count; s += MERGE_THREADS) {
        const float2 ml = *reinterpret_cast<const float2*>(base + s * stride + HD);
        s_m[s] = ml.x; s_l[s] = ml.y;
        mx = fmaxf(mx, ml.x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    float M = s_red[0];
#pragma unroll
    for (int w = 1; w < MERGE_THREADS / 32; ++w) M = fmaxf(M, s_red[w]);
    __syncthreads();
    // phase 2: weights w_s = e^(m_s - M) and the denominator sum w_s l_s   (bruce.cu:1000-1001)
    float ls = 0.f;
    for (int s = tid; s < count; s += MERGE_THREADS) {
        const float w = P.log2_domain ? fast_exp2(s_m[s] - M) : __expf(s_m[s] - M);
        s_m[s] = w;
        ls = fmaf(s_l[s], w, ls);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
    if (lane == 0) s_red[warp] = ls;
    __syncthreads();
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < MERGE_THREADS / 32; ++w) L += s_red[w];
    // phase 3: weighted sum of o; HD/2 dim pairs x NG interleaved groups of records
    constexpr int NDP = HD / 2, NG = MERGE_THREADS / NDP;
    const int dp = tid % NDP, grp = tid / NDP;
    float a0 = 0.f, a1 = 0.f;
#pragma unroll 4
    for (int s = grp; s < count; s += NG) {
        const float2 o = *reinterpret_cast<const float2*>(base + s * stride + 2 * dp);
        const float w = s_m[s];
        a0 = fmaf(o.x, w, a0);
        a1 = fmaf(o.y, w, a1);
    }
    s_acc[tid] = make_float2(a0, a1);
    __syncthreads();
    if (grp != 0) return;
#pragma unroll
    for (int g2 = 1; g2 < NG; ++g2) { a0 += s_acc[g2 * NDP + dp].x; a1 += s_acc[g2 * NDP + dp].y; }
    const int d2 = 2 * dp;
    if (P.out) {
        const float il = L > 0.f ? 1.f / L : 0.f;
        const size_t oi = ((size_t)rowidx * P.Hq + hq) * HD + d2;
        if (P.out_f16) reinterpret_cast<__half2*>(P.out)[oi >> 1] = __floats2half2_rn(a0 * il, a1 * il);
        else *reinterpret_cast<float2*>(reinterpret_cast<float*>(P.out) + oi) = make_float2(a0 * il, a1 * il);
    }
    if (P.rec_out) {
        float* ro = P.rec_out + ((size_t)rowidx * P.Hq + hq) * (size_t)(HD + 2);
        *reinterpret_cast<float2*>(ro + d2) = make_float2(a0, a1);
        if (dp == 0) {
            ro[HD] = (P.log2_domain && M > -1e29f) ? M * LN2 : M;
            ro[HD + 1] = L;
        }
    }
}

// The merge behind the flash-decode kernels (their work-balanced records only).  Those records are padded to
// HD + 4 floats so that every record is 16-byte aligned.  The kernel is one latency chain (header -> records ->
// output) behind every decode call, so it is built to have as few dependent steps as possible: warp w owns the
// float4 lanes w, w + 32, ... of the output and lane s of every warp owns records s, s + 32, ...; each warp
// reads the (m, l) pairs itself, so the maximum, the weights, the denominator and the weighted sum are all
// butterfly shuffles inside a warp -- one round of independent loads (up to 128 records), no block barrier, no
// shared memory.  More records take further rounds with the running (M, L, acc) rescaled, in a fixed order.
// (Eight warps with four float4 lanes each would fit on an SM beside the next call's decode CTAs, but measured
// 1 us slower per call: the chain of loads and shuffles per lane is what counts here.)
constexpr int MERGE_B_THREADS = 1024;
constexpr int MERGE_B_KEEP = 4;           // records per lane and round

template <int HD>
__global__ void __launch_bounds__(MERGE_B_THREADS) k_merge_balanced(const MergeParams P) {
    constexpr int RS = HD + 4;                                   // floats per internal record
    constexpr int NWARP = MERGE_B_THREADS / 32, DPW = (HD / 4) / NWARP;   // float4 lanes per warp: 1 or 2
    static_assert(DPW >= 1 && DPW * NWARP * 4 == HD, "one float4 lane per warp and step");
    const int hq = blockIdx.x % P.Hq, rowidx = blockIdx.x / P.Hq;
    const int i = rowidx / P.rows, r = rowidx % P.rows;
    const int kvh = hq / P.G, h = hq % P.G;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // The successor may start at once: it is either a kernel of this library, which touches nothing this kernel
    // or its predecessors write before its own griddepcontrol.wait, or a launch without the programmatic attribute,
    // which waits for this grid to complete anyway.  The next decode call uses the head start to stream cache tiles.
    pdl_trigger();
    int per = 1, c0 = 0, c1 = 0;
    const bool pre = P.pre_grid > 0;
    if (pre) {
        // what the decode kernel derives from the same positions (flash_decode.cuh): one L2 round trip less behind the wait
        const SeqRange sr = seq_range(P.pos, P.kslot, P.act, 0, P.rows, P.is_swa, P.W, P.slot_ctx, P.n_slots, P.status);
        c1 = sr.active ? ((sr.hi + P.pre_tile - 1) / P.pre_tile - sr.lo / P.pre_tile) : 0;
        per = P.cph > 0 ? max(1, (c1 + P.cph - 1) / P.cph) : max(1, (P.Hkv * c1 + P.pre_grid - 1) / P.pre_grid);
    }
    pdl_wait();
    if (!pre) {
        per = P.hdr[0];
        c0 = P.hdr[2 + i];
        c1 = P.hdr[3 + i];
    }
    const int nt = c1 - c0;
    const bool xq = P.xchg.world > 0;                            // this launch feeds a cross-device exchange
    if (nt <= 0 && !xq) return;                                  // inactive sequence: no output
    const int item = i * P.Hkv + kvh;
    // the CTAs that hold pieces of this item: the decode kernel's cut (per-head groups of cph CTAs, or linear)
    int clo = 0, chi = -1;
    if (nt > 0) fd::item_ctas(P.cph, per, P.Hkv, c0, nt, kvh, clo, chi);
    const int RG = P.rows * P.G;
    // (an inactive shard of a split sequence contributes the empty record (0, -1e30, 0), bruce.cu:2319-2322)
    const int count = nt <= 0 ? 0 : min(chi - clo + 1, MERGE_MAX_COUNT);
    const float* base = P.part + ((size_t)(clo + item) * RG + r * P.G + h) * (size_t)RS;
    const size_t stride = (size_t)RG * RS;

    float M = NEG_BIG, L = 0.f;
    float4 acc[DPW];
#pragma unroll
    for (int j = 0; j < DPW; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < count; s0 += 32 * MERGE_B_KEEP) {
        float2 ml[MERGE_B_KEEP];
        float4 o[MERGE_B_KEEP][DPW];
#pragma unroll
        for (int k = 0; k < MERGE_B_KEEP; ++k) {                 // every load of the round is in flight at once
            const int s = s0 + 32 * k + lane;
            ml[k] = make_float2(NEG_BIG, 0.f);
#pragma unroll
            for (int j = 0; j < DPW; ++j) o[k][j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s < count) {
                const float* rp = base + s * stride;
                ml[k] = *reinterpret_cast<const float2*>(rp + HD);
#pragma unroll
                for (int j = 0; j < DPW; ++j) o[k][j] = *reinterpret_cast<const float4*>(rp + 4 * (warp + NWARP * j));
            }
        }
        float mk = ml[0].x;
#pragma unroll
        for (int k = 1; k < MERGE_B_KEEP; ++k) mk = fmaxf(mk, ml[k].x);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, d));
        const float Mn = fmaxf(M, mk);
        const float sc = fast_exp2(M - Mn);                      // records carry m in log2 units
        float ls = 0.f;
        float4 a[DPW];
#pragma unroll
        for (int j = 0; j < DPW; ++j) a[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < MERGE_B_KEEP; ++k) {
            const float w = fast_exp2(ml[k].x - Mn);
            ls = fmaf(ml[k].y, w, ls);
#pragma unroll
            for (int j = 0; j < DPW; ++j) {
                a[j].x = fmaf(o[k][j].x, w, a[j].x); a[j].y = fmaf(o[k][j].y, w, a[j].y);
                a[j].z = fmaf(o[k][j].z, w, a[j].z); a[j].w = fmaf(o[k][j].w, w, a[j].w);
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {                       // fixed-order butterfly: every lane ends with the sums
            ls += __shfl_xor_sync(0xffffffffu, ls, d);
#pragma unroll
            for (int j = 0; j < DPW; ++j) {
                a[j].x += __shfl_xor_sync(0xffffffffu, a[j].x, d); a[j].y += __shfl_xor_sync(0xffffffffu, a[j].y, d);
                a[j].z += __shfl_xor_sync(0xffffffffu, a[j].z, d); a[j].w += __shfl_xor_sync(0xffffffffu, a[j].w, d);
            }
        }
        L = fmaf(L, sc, ls);
#pragma unroll
        for (int j = 0; j < DPW; ++j) {
            acc[j].x = fmaf(acc[j].x, sc, a[j].x); acc[j].y = fmaf(acc[j].y, sc, a[j].y);
            acc[j].z = fmaf(acc[j].z, sc, a[j].z); acc[j].w = fmaf(acc[j].w, sc, a[j].w);
        }
        M = Mn;
    }

    const size_t obase = ((size_t)rowidx * P.Hq + hq) * HD;
    if (xq) {
        // ---- sequence split: push this device's record to every peer, then merge what the peers pushed ----
        // Every lane of a warp holds the warp's float4(s) of the record: lane d sends them to device d, lane r then
        // polls device r's record, and the merge over the devices runs on shuffled values in device order.
        const XchgView& X = P.xchg;
        const int xitem = rowidx * P.Hq + hq;
        const int epoch = *X.epoch_ptr;
        if (X.push && lane < X.world) {
#pragma unroll
            for (int j = 0; j < DPW; ++j)
                xchg_push<HD>(X, epoch, xitem, lane, warp + NWARP * j, acc[j], warp == 0 && j == 0, M, L);
        }
        if (!X.wait || !P.out) return;
        bool ok = true;
        float4 o[DPW];
        float2 ml = make_float2(NEG_BIG, 0.f);
#pragma unroll
        for (int j = 0; j < DPW; ++j) o[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (lane < X.world) {
#pragma unroll
            for (int j = 0; j < DPW; ++j) ok = ok && xchg_poll<HD>(X, epoch, xitem, lane, warp + NWARP * j, o[j], ml);
        }
        ok = __syncthreads_and(ok);
        if (!ok) {                                               // a peer's record never came: output untouched
            if (tid == 0) atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
            return;
        }
        float Mx = NEG_BIG;
#pragma unroll
        for (int r = 0; r < XCHG_MAX_WORLD; ++r) {
            const float m = __shfl_sync(0xffffffffu, ml.x, r);
            if (r < X.world) Mx = fmaxf(Mx, m);
        }
        XchgAcc xa[DPW];
#pragma unroll
        for (int r = 0; r < XCHG_MAX_WORLD; ++r) {
            const float m = __shfl_sync(0xffffffffu, ml.x, r), l = __shfl_sync(0xffffffffu, ml.y, r);
#pragma unroll
            for (int j = 0; j < DPW; ++j) {
                const float4 v = make_float4(__shfl_sync(0xffffffffu, o[j].x, r), __shfl_sync(0xffffffffu, o[j].y, r),
                                             __shfl_sync(0xffffffffu, o[j].z, r), __shfl_sync(0xffffffffu, o[j].w, r));
                if (r < X.world) xa[j].add(v, m, l, Mx);
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < DPW; ++j) xa[j].store(P.out, P.out_f16, obase + 4 * (warp + NWARP * j));
        }
        return;
    }
    if (lane != 0) return;
#pragma unroll
    for (int j = 0; j < DPW; ++j) {
        const int d4 = 4 * (warp + NWARP * j);
        const size_t oi = obase + d4;
        if (P.out) {
            const float il = L > 0.f ? 1.f / L : 0.f;
            if (P.out_f16) {
                const __half2 a = __floats2half2_rn(acc[j].x * il, acc[j].y * il), b = __floats2half2_rn(acc[j].z * il, acc[j].w * il);
                *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(P.out) + oi) =
                    make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
            } else {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(P.out) + oi) =
                    make_float4(acc[j].x * il, acc[j].y * il, acc[j].z * il, acc[j].w * il);
            }
        }
        if (P.rec_out) {                                         // public record: HD + 2 floats, natural-log m
            float* ro = P.rec_out + ((size_t)rowidx * P.Hq + hq) * (size_t)(HD + 2);
            *reinterpret_cast<float2*>(ro + d4) = make_float2(acc[j].x, acc[j].y);
            *reinterpret_cast<float2*>(ro + d4 + 2) = make_float2(acc[j].z, acc[j].w);
            if (d4 == 0) {
                ro[HD] = M > -1e29f ? M * LN2 : M;
                ro[HD + 1] = L;
            }
        }
    }
}

// The receiving half of the exchange on its own: one block per (row, head) waits for every device's record of the
// step and merges them (for hosts that put other work between the push and the merge).
template <int HD>
__global__ void __launch_bounds__(HD / 4 < 32 ? 32 : HD / 4) k_merge_wait(const MergeParams P) {
    pdl_wait();
    pdl_trigger();
    const XchgView& X = P.xchg;
    const int xitem = blockIdx.x, dq = threadIdx.x;
    const int epoch = *X.epoch_ptr;
    float4 o[XCHG_MAX_WORLD];
    float2 ml[XCHG_MAX_WORLD];
    bool ok = true;
    float M = NEG_BIG;
    if (dq < HD / 4) {
#pragma unroll
        for (int r = 0; r < XCHG_MAX_WORLD; ++r)
            if (r < X.world) {
                ok = ok && xchg_poll<HD>(X, epoch, xitem, r, dq, o[r], ml[r]);
                M = fmaxf(M, ml[r].x);
            }
    }
    ok = __syncthreads_and(ok);
    if (!ok) {
        if (threadIdx.x == 0) atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
        return;
    }
    if (dq >= HD / 4) return;
    XchgAcc xa;
#pragma unroll
    for (int r = 0; r < XCHG_MAX_WORLD; ++r)
        if (r < X.world) xa.add(o[r], ml[r].x, ml[r].y, M);
    xa.store(P.out, P.out_f16, (size_t)xitem * HD + 4 * dq);
}

}  // namespace battn
