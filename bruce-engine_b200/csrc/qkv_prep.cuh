// QKV prologue fused with the quantise-on-append: per head an L2 scale, NeoX rotate-half RoPE from
// per-row cos/sin tables and (q only) the per-head sqk scale; k is then quantised into the q8_0 cache,
// v is quantised raw.  Replaces k_qkv_prep / k_qkv_prep_rows / k_qkv_prep_fast / k_qkv_prep_fast_ms
// (engine/src/bruce.cu:645-710, 1656-1725, 1732-1812, 1835-1918) and the table kernels
// k_rope_tables / k_rope_tables_rows / k_rope_tables_rows_ms (:328-336, 1641-1654, 1821-1833).
//
// HBM-bound element-wise work: one warp per (row, head) with the whole head in the warp's registers
// (16-byte loads and stores), eight heads per CTA, no shared memory, no block barrier.  Every fp32 step is written
// with explicit round-to-nearest intrinsics in the order nvcc generates for the reference source (which
// fuses x0*c - x1*s into fma(x0, c, -(x1*s)) and the squares into a chain of fma), so q and the K/V
// records are bit-identical to the reference kernel's and do not depend on this file's compiler flags.
// q can be emitted as fp16 for the attention kernels in the same pass.
#pragma once
#include "common.cuh"

namespace battn {

struct PrepParams {
    const float* q;       // [n_seq*rows][Hq][HD]
    void* q_out;          // same shape, fp32 (may alias q) or fp16
    const float* k;       // [n_seq*rows][Hkv][HD]
    const float* v;
    const float* sqk;     // [Hq][HD]
    const float* cs;      // [n_seq*rows][HD]: two tables of HD/2 per row
    const float* sn;
    uint8_t* kvk;
    uint8_t* kvv;
    const int* pos;
    const int* kslot;     // null: single sequence, caches point at the slot base
    const int* act;       // null: every sequence active
    int n_seq, rows, Hq, Hkv;
    int table_off;        // 0 or HD/2 (second table)
    int q_out_f16;
    int pstride, ring_mask, n_slots;
    int* status;
    Paging pg;            // table != nullptr: paged cache (pstride = positions a table row can hold)
};

// The arithmetic of one head, one warp per head, lane l holding VEC consecutive values of the first half of the head
// (at VEC*l) and the VEC values HD/2 further on.  Used by k_qkv_prep below and by the decode kernel that runs the
// prologue itself (flash_decode.cuh), so both produce the same bits.
namespace prep {

template <int HD>
struct Cfg {
    static constexpr int VEC = HD / 64;                 // values per lane and half: 4 (float4) or 2 (float2)
    static constexpr int H2 = HD / 2;
    static constexpr int NBLK = HD / 32;
    static constexpr int REC = HD + 2 * NBLK;
    static constexpr int LPB = 32 / VEC;                // lanes per 32-value quantisation block
};

template <int VEC>
__device__ __forceinline__ void load(const float* p, float (&o)[VEC]) {
    if constexpr (VEC == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
    } else {
        const float2 t = *reinterpret_cast<const float2*>(p);
        o[0] = t.x; o[1] = t.y;
    }
}

// this lane's cos / sin entries of a row's table (cs_row, sn_row: the row's table, table offset included)
template <int HD>
__device__ __forceinline__ void tables(const float* cs_row, const float* sn_row, int lane, float (&c)[HD / 64],
                                       float (&s)[HD / 64]) {
    constexpr int VEC = HD / 64;
#pragma unroll
    for (int j = 0; j < VEC; ++j) { c[j] = cs_row[VEC * lane + j]; s[j] = sn_row[VEC * lane + j]; }
}

// L2 scale of one head held as e (first half) and f (second half): bruce.cu:305-307, 1751-1755
template <int HD>
__device__ __forceinline__ float l2_scale(const float (&e)[HD / 64], const float (&f)[HD / 64]) {
    constexpr int VEC = HD / 64;
    float a = __fmaf_rn(e[0], e[0], __fmul_rn(e[1], e[1]));
    float b = __fmaf_rn(f[0], f[0], __fmul_rn(f[1], f[1]));
#pragma unroll
    for (int j = 2; j < VEC; ++j) { a = __fmaf_rn(e[j], e[j], a); b = __fmaf_rn(f[j], f[j], b); }
    float ss = __fadd_rn(a, b);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, o));
    ss = __shfl_sync(0xffffffffu, ss, 0);
    const float arg = __fadd_rn(__fdiv_rn(ss, (float)HD), __fdiv_rn(1e-6f, (float)HD));
    return __fmul_rn(__fdiv_rn(1.0f, __fsqrt_rn(arg)), __fdiv_rn(1.0f, __fsqrt_rn((float)HD)));
}

// q head: scale, rotate, sqk (bruce.cu:1742-1766); qh, sqkh: the head's HD values
template <int HD>
__device__ __forceinline__ void q_head(const float* qh, const float* sqkh, const float (&c)[HD / 64],
                                       const float (&s)[HD / 64], int lane, float (&lo)[HD / 64], float (&hi)[HD / 64]) {
    constexpr int VEC = HD / 64, H2 = HD / 2;
    float e[VEC], f[VEC], s0[VEC], s1[VEC];
    load<VEC>(qh + VEC * lane, e); load<VEC>(qh + H2 + VEC * lane, f);
    load<VEC>(sqkh + VEC * lane, s0); load<VEC>(sqkh + H2 + VEC * lane, s1);
    const float norm = l2_scale<HD>(e, f);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        lo[j] = __fmul_rn(__fmul_rn(__fmaf_rn(e[j], c[j], -__fmul_rn(f[j], s[j])), norm), s0[j]);
        hi[j] = __fmul_rn(__fmul_rn(__fmaf_rn(e[j], s[j], __fmul_rn(f[j], c[j])), norm), s1[j]);
    }
}

// k head: scale and rotate (bruce.cu:1768-1795)
template <int HD>
__device__ __forceinline__ void k_head(const float* kh, const float (&c)[HD / 64], const float (&s)[HD / 64], int lane,
                                       float (&k0)[HD / 64], float (&k1)[HD / 64]) {
    constexpr int VEC = HD / 64, H2 = HD / 2;
    float e[VEC], f[VEC];
    load<VEC>(kh + VEC * lane, e); load<VEC>(kh + H2 + VEC * lane, f);
    const float norm = l2_scale<HD>(e, f);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        k0[j] = __fmul_rn(__fmaf_rn(e[j], c[j], -__fmul_rn(f[j], s[j])), norm);
        k1[j] = __fmul_rn(__fmaf_rn(e[j], s[j], __fmul_rn(f[j], c[j])), norm);
    }
}

// Quantises this lane's VEC values of 32-value block `blk` into the record `rec` (bruce.cu:1799-1802): one block =
// LPB neighbouring lanes.
template <int HD>
__device__ __forceinline__ void quant(uint8_t* rec, int blk, const float (&x)[HD / 64], int lane) {
    constexpr int VEC = HD / 64, NBLK = HD / 32, LPB = 32 / VEC;
    float amax = fmaxf(fabsf(x[0]), fabsf(x[1]));
#pragma unroll
    for (int j = 2; j < VEC; ++j) amax = fmaxf(amax, fabsf(x[j]));
#pragma unroll
    for (int o = LPB / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.f);                        // bruce.cu:1799
    const float id = d != 0.f ? __fdiv_rn(1.f, d) : 0.f;           // :1800
    if ((lane & (LPB - 1)) == 0) reinterpret_cast<__half*>(rec)[blk] = __float2half_rn(d);
    uint32_t pk = 0;
#pragma unroll
    for (int j = 0; j < VEC; ++j)                                    // lrintf(x * id), no clamp (:1802)
        pk |= (uint32_t)(uint8_t)(int8_t)__float2int_rn(__fmul_rn(x[j], id)) << (8 * j);
    uint8_t* dst = rec + 2 * NBLK + blk * 32 + (lane & (LPB - 1)) * VEC;
    if constexpr (VEC == 4) *reinterpret_cast<uint32_t*>(dst) = pk;
    else                    *reinterpret_cast<uint16_t*>(dst) = (uint16_t)pk;
}

// a head held as (first half, second half) quantised into one record: this lane's first-half values sit in block
// lane / LPB, its second-half values NBLK/2 blocks later
template <int HD>
__device__ __forceinline__ void quant_head(uint8_t* rec, const float (&x0)[HD / 64], const float (&x1)[HD / 64], int lane) {
    constexpr int NBLK = HD / 32, LPB = 32 / (HD / 64);
    quant<HD>(rec, lane / LPB, x0, lane);
    quant<HD>(rec, lane / LPB + NBLK / 2, x1, lane);
}

}  // namespace prep

template <int HD>
__global__ void __launch_bounds__(256) k_qkv_prep(const PrepParams P) {
    constexpr int VEC = HD / 64;                 // values per lane and half: 4 (float4) or 2 (float2)
    constexpr int H2 = HD / 2;
    constexpr int NBLK = HD / 32;
    constexpr int REC = HD + 2 * NBLK;
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x;                    // row of the launch: sequence m / rows, row m % rows
    const int i = m / P.rows, r = m - i * P.rows;
    const int lane = threadIdx.x & 31;
    const int hw = blockIdx.y * 8 + (threadIdx.x >> 5);   // q heads first, then kv heads
    if (hw >= P.Hq + P.Hkv) return;

    float c[VEC], s[VEC];
    prep::tables<HD>(P.cs + (size_t)m * HD + P.table_off, P.sn + (size_t)m * HD + P.table_off, lane, c, s);

    // ---- q heads: scale, rotate, sqk (bruce.cu:1742-1766) ----------------------------------------------
    if (hw < P.Hq) {
        const int h = hw;
        const size_t base = ((size_t)m * P.Hq + h) * HD + VEC * lane;
        float lo[VEC], hi[VEC];
        prep::q_head<HD>(P.q + ((size_t)m * P.Hq + h) * HD, P.sqk + (size_t)h * HD, c, s, lane, lo, hi);
        if (P.q_out_f16) {
            __half* o = reinterpret_cast<__half*>(P.q_out) + base;
#pragma unroll
            for (int j = 0; j < VEC; j += 2) {
                *reinterpret_cast<__half2*>(o + j) = __floats2half2_rn(lo[j], lo[j + 1]);
                *reinterpret_cast<__half2*>(o + H2 + j) = __floats2half2_rn(hi[j], hi[j + 1]);
            }
        } else {
            float* o = reinterpret_cast<float*>(P.q_out) + base;
            if constexpr (VEC == 4) {
                *reinterpret_cast<float4*>(o) = make_float4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<float4*>(o + H2) = make_float4(hi[0], hi[1], hi[2], hi[3]);
            } else {
                *reinterpret_cast<float2*>(o) = make_float2(lo[0], lo[1]);
                *reinterpret_cast<float2*>(o + H2) = make_float2(hi[0], hi[1]);
            }
        }
        return;
    }

    // ---- kv heads: k scale + rotate, then quantise k and raw v (bruce.cu:1768-1812, 1866-1918) ---------
    if (P.act && !P.act[i]) return;               // idle rows normalise q but never write KV (:1869)
    const int slot = P.kslot ? P.kslot[i] : 0;
    const int p = P.pos[i] + r;
    const bool bad = p < 0 || (P.ring_mask < 0 && p >= P.pstride) || slot < 0 || (P.kslot && slot >= P.n_slots);
    if (bad) {
        if (lane == 0) atomicOr(P.status, BATTN_DEV_BAD_POSITION);
        return;
    }
    const int pp = p & P.ring_mask;               // ring slot (bruce.cu:1796); identity when the mask is -1
    {
        const int h = hw - P.Hq;
        const size_t base = ((size_t)m * P.Hkv + h) * HD;
        float k0[VEC], k1[VEC], v0[VEC], v1[VEC];
        prep::k_head<HD>(P.k + base, c, s, lane, k0, k1);
        prep::load<VEC>(P.v + base + VEC * lane, v0); prep::load<VEC>(P.v + base + H2 + VEC * lane, v1);
        const size_t roff = kv_rec_index(P.pg, slot, h, P.Hkv, P.pstride, pp, P.status) * (size_t)REC;
        prep::quant_head<HD>(P.kvk + roff, k0, k1, lane);
        prep::quant_head<HD>(P.kvv + roff, v0, v1, lane);
    }
}

// RoPE tables of a launch's rows: [theta 1e7 | theta 1e4], HD/2 entries each (bruce.cu:1641-1654).  The
// expressions are the reference's, so the device math library gives the reference's values.
struct TableParams {
    float* cs;
    float* sn;
    const int* pos;
    int rows, n_rows;
};

template <int HD>
__global__ void k_rope_tables(const TableParams P) {
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x;
    if (m >= P.n_rows) return;
    const int p = P.pos[m / P.rows] + m % P.rows;
    const int i = threadIdx.x;                    // HD/2 threads
    float* c = P.cs + (size_t)m * HD;
    float* s = P.sn + (size_t)m * HD;
    const float th = (float)p * powf(10000000.0f, -2.0f * (float)i / (float)HD);
    c[i] = cosf(th); s[i] = sinf(th);
    const float th2 = (float)p * powf(10000.0f, -2.0f * (float)i / (float)HD);
    c[HD / 2 + i] = cosf(th2); s[HD / 2 + i] = sinf(th2);
}

}  // namespace battn
