// Quantise-on-append: fp32 K/V rows -> q8_0 records in the scale-first, head-major cache.
// Replaces the store half of k_qkv_prep / k_qkv_prep_rows / k_qkv_prep_fast / k_qkv_prep_fast_ms
// (engine/src/bruce.cu:690-710, 1713-1725, 1789-1812, 1888-1918).  HBM-bound byte work: one warp
// per (sequence, row, kv head, K|V) record, 16-byte loads, 4-byte packed stores.
#pragma once
#include "common.cuh"

namespace battn {

struct AppendParams {
    const float* k;
    const float* v;
    uint8_t* kvk;
    uint8_t* kvv;
    const int* pos;
    const int* kslot;   // null: single sequence, caches point at the slot base
    const int* act;     // null: every sequence active
    int n_seq, rows, Hkv;
    int pstride;        // slot_ctx or 2*W
    int ring_mask;      // 2*W-1 for a sliding-window layer, -1 (all ones) otherwise
    int n_slots;
    int* status;
    Paging pg;          // table != nullptr: paged cache (pstride = positions a table row can hold)
};

// One warp quantises one (kv head, position) row of HD fp32 values into a scale-first q8_0 record at `dst` (global or
// shared memory): per 32 values d = amax / 127, id = d ? 1 / d : 0, q = lrintf(x * id), scale = fp16(d), no clamp
// (bruce.cu:698-710).  The one quantiser of the library: the append kernel and the decode kernel that appends its own
// row both call it, so their bytes are the same by construction.
template <int HD>
__device__ __forceinline__ void quantise_record(const float* __restrict__ src, uint8_t* dst, int lane) {
    constexpr int NBLK = HD / 32;
#pragma unroll
    for (int it = 0; it < HD / 128; ++it) {
        const float4 x = *reinterpret_cast<const float4*>(src + it * 128 + lane * 4);
        float amax = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
        // 8 lanes x 4 values = one 32-value block
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        const float d = __fdiv_rn(amax, 127.f);                       // IEEE divide (bruce.cu:704)
        const float id = d != 0.f ? __fdiv_rn(1.f, d) : 0.f;          // (bruce.cu:705)
        // lrintf(x * id): one fp32 multiply, round half to even, no clamp (bruce.cu:709)
        const uint32_t q0 = (uint32_t)(uint8_t)(int8_t)__float2int_rn(__fmul_rn(x.x, id));
        const uint32_t q1 = (uint32_t)(uint8_t)(int8_t)__float2int_rn(__fmul_rn(x.y, id));
        const uint32_t q2 = (uint32_t)(uint8_t)(int8_t)__float2int_rn(__fmul_rn(x.z, id));
        const uint32_t q3 = (uint32_t)(uint8_t)(int8_t)__float2int_rn(__fmul_rn(x.w, id));
        *reinterpret_cast<uint32_t*>(dst + 2 * NBLK + it * 128 + lane * 4) = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
        if ((lane & 7) == 0)
            reinterpret_cast<__half*>(dst)[it * 4 + (lane >> 3)] = __float2half_rn(d);   // (bruce.cu:708)
    }
}

template <int HD>
__global__ void __launch_bounds__(256) k_kv_append(const AppendParams P) {
    constexpr int NBLK = HD / 32;
    constexpr int REC = HD + 2 * NBLK;
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long total = (long long)P.n_seq * P.rows * P.Hkv * 2;
    if (wid >= total) return;
    const int which = (int)(wid & 1);                 // 0 = K, 1 = V
    long long t = wid >> 1;
    const int kvh = (int)(t % P.Hkv); t /= P.Hkv;
    const int r = (int)(t % P.rows);
    const int i = (int)(t / P.rows);

    if (P.act && !P.act[i]) return;                   // idle rows never write KV (bruce.cu:1869)
    const int slot = P.kslot ? P.kslot[i] : 0;
    const int p = P.pos[i] + r;
    const bool bad = p < 0 || (P.ring_mask < 0 && p >= P.pstride) || slot < 0 ||
                     (P.kslot && slot >= P.n_slots);
    if (bad) {
        if (lane == 0) atomicOr(P.status, BATTN_DEV_BAD_POSITION);
        return;
    }
    const int pp = p & P.ring_mask;                   // ring slot (bruce.cu:691); identity when -1
    const float* src = (which ? P.v : P.k) + (((size_t)i * P.rows + r) * P.Hkv + kvh) * HD;
    uint8_t* dst = (which ? P.kvv : P.kvk) + kv_rec_index(P.pg, slot, kvh, P.Hkv, P.pstride, pp, P.status) * (size_t)REC;

    quantise_record<HD>(src, dst, lane);
}

// Prefix sharing between slots: the first n_pos cached positions of slot `src` copied into slot `dst` of the same
// layer buffer, K and V, every kv head (a request whose prompt starts like another slot's cache skips that part of
// its prompt).  Records are position-contiguous per kv head, so this is n_kv contiguous runs per tensor, moved
// with 16-byte loads.  Full-attention layers copy [0, n_pos); a sliding-window layer copies the ring slots of
// the last min(n_pos, 2W) positions (p & (2W - 1) is the same slot in both partitions).
struct CopyParams {
    uint8_t* kvk;
    uint8_t* kvv;
    int src, dst, n_pos, Hkv, rec, pstride, ring;      // ring = 2W on a sliding-window layer, else 0
};

__global__ void __launch_bounds__(256) k_kv_copy_prefix(const CopyParams P) {
    pdl_wait();
    pdl_trigger();
    const int first = P.ring ? max(0, P.n_pos - P.ring) : 0;                   // first position to copy
    const size_t run = (size_t)(P.n_pos - first) * P.rec;                      // bytes per kv head when contiguous
    const int kvh = blockIdx.y;
    uint8_t* base = blockIdx.z ? P.kvv : P.kvk;
    const size_t so = ((size_t)P.src * P.Hkv + kvh) * P.pstride * (size_t)P.rec;
    const size_t dof = ((size_t)P.dst * P.Hkv + kvh) * P.pstride * (size_t)P.rec;
    if (!P.ring) {
        // [0, n_pos) is one run: 16-byte chunks (the partition base is 16-byte aligned), then the odd tail bytes
        const size_t n16 = run >> 4;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
            reinterpret_cast<uint4*>(base + dof)[i] = reinterpret_cast<const uint4*>(base + so)[i];
        if (blockIdx.x == 0 && threadIdx.x < (int)(run & 15)) base[dof + (n16 << 4) + threadIdx.x] = base[so + (n16 << 4) + threadIdx.x];
    } else {
        // ring slots of positions [first, n_pos): 8-byte words (a record is a multiple of 8 bytes)
        const int w8 = P.rec >> 3;
        const size_t total = (size_t)(P.n_pos - first) * w8;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const int p = first + (int)(i / w8), wi = (int)(i % w8);
            const size_t off = (size_t)(p & (P.ring - 1)) * P.rec + (size_t)wi * 8;
            *reinterpret_cast<uint2*>(base + dof + off) = *reinterpret_cast<const uint2*>(base + so + off);
        }
    }
}

}  // namespace battn
