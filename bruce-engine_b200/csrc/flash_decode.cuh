// Flash-decoding over the q8_0 scale-first KV cache: decode (1 row), speculative verify (2..8 rows
// sharing one KV sweep) and multi-slot decode (one row per independent sequence), one kernel.
//
// Behaviour replaced: k_attn_m1_w, k_attn_mv_w<R>, k_attn_tc_rs_opt<4,3> for <= 8 rows, and the
// multi-slot grid of launch_attn_ms (engine/src/bruce.cu:3385-3599, 3643-3803, 2750-3131,
// 4158-4177).  The contract (key ranges, masks, split records) is that of the exact kernels
// k_attn / k_attn_m (:713-785, 2087-2143).
//
// Design (sm_100a):
//   * Work = (sequence, kv head, 64-key tile).  The flattened tile list is cut into equal contiguous
//     shares, one per CTA (positions are device-resident, so every CTA derives the same cut from
//     pos[] itself); a CTA therefore streams a contiguous byte range of one or more (sequence, head)
//     items.  Each (CTA, item) piece yields one split record; records land at slot (cta + item), which
//     is unique because pieces form a monotone staircase in (cta, item).
//   * A producer warp streams raw K and V tiles (64 records = 8704 B each for head_dim 128) with
//     cp.async.bulk into a ring of shared-memory stages guarded by mbarriers: large contiguous HBM
//     reads with no register staging.  The cache is head-major with positions contiguous, so a tile
//     is one contiguous run; tiles are 64-aligned in position, so they never wrap the SWA ring.
//   * Four consumer warps each own 16 of the 64 keys.  S^T = K Q^T with keys on the MMA M side and
//     the (row, head) pairs on the N side, so no MMA row is wasted on a 1-row decode; int8 -> fp16 is
//     the exact byte-permute conversion and the per-32-block scales are applied to the fp32
//     accumulators after the MMA.  O^T = V^T P^T with the V scale folded into the fp16 V operand.
//     Everything accumulates in fp32.
//   * The key owned by MMA row kappa of a warp is 4*pi(kappa)+warp (pi swaps neighbours in odd groups
//     of four), which makes every shared-memory read of the 136-byte-stride records conflict-free.
#pragma once
#include "common.cuh"
#include "kv_append.cuh"
#include "qkv_prep.cuh"
#include "work_cut.h"

namespace battn {
namespace fd {

constexpr int NW = 4;                     // consumer warps
constexpr int TILE = 64;                  // keys per stage
constexpr int NTHREADS = (NW + 1) * 32;   // + one producer warp
// pipeline depth: three stages of 2 x 8.7 KB at head_dim 128; two stages of 2 x 17.4 KB at head_dim 256, so that
// three CTAs (twelve consumer warps) still fit one SM -- with three stages only two CTAs fit and the conversion
// work of the wider head leaves the kernel issue-bound (3.1 instead of 4 TB/s at 64K)
template <int HD, int NT>
__host__ __device__ constexpr int stages_of() { return HD == 256 ? 2 : 3; }

struct Params {
    const void* q;
    const uint8_t* kvk;
    const uint8_t* kvv;
    const int* pos;
    const int* kslot;
    const int* act;
    int* hdr;        // workspace header: {tiles_per_cta, total_tiles, cum[n_seq + 1]}
    float* part;     // workspace records, slot stride RG * (HD + 4) floats
    int n_seq, rows, Hq, Hkv, G, RG;
    int W, pstride, ring_mask, slot_ctx, n_slots, is_swa, q_f16;
    float scale_log2;   // softmax scale * log2(e): scores are kept in log2 units
    int* status;
    // sequence split across devices: the step counter the merge epilogue reads is advanced here, one kernel
    // earlier, so that every block of the epilogue sees the same value (null when there is no exchange)
    int* epoch_ptr;
    int epoch_advance;
    Paging pg;       // table != nullptr: paged cache of a full-causal layer (pages hold whole tiles)
    // Early KV streaming.  The kernel is launched with programmatic stream serialisation, so its CTAs may start while
    // the previous kernel of the stream (normally the append of this step's rows) is still running.  With early != 0
    // the positions are read and the bulk copies of every tile that lies entirely below the step's first row are
    // issued BEFORE griddepcontrol.wait -- those cache rows were written by earlier steps, and everything older than
    // the immediate predecessor has completed by the time this grid starts -- so the first stages are in shared
    // memory when the predecessor finishes.  Q, the tile that holds the step's own rows, and every write (header,
    // records, epoch) come after the wait.  The host sets early only when the predecessor wrote no other cache rows.
    int early;
    // Decode that appends its own row (rows == 1): k_new / v_new are the step's fp32 K and V rows
    // [n_seq][n_kv][head_dim].  The CTA whose share holds the tile of position pos[i] quantises the row of its kv head
    // into that tile in shared memory (the bulk copy brought the slot's old bytes) and into the cache, with the append
    // kernel's own quantiser, before the tile is used: no separate append launch in front of the attention call.
    int cph;              // > 0: one sequence, cph CTAs per kv head (see the cut in k_flash_decode); 0: linear cut
    // AP == 2, the decode call that runs the whole QKV prologue itself: raw q [n_seq][Hq][HD], sqk [Hq][HD], the rows'
    // RoPE tables cs / sn [n_seq][HD] (table_off selects the theta), and k_new / v_new are the RAW k and v rows
    const float* q_raw;
    const float* sqk;
    const float* cs;
    const float* sn;
    int table_off;
    const float* k_new;
    const float* v_new;
    uint8_t* kvk_w;  // the caches again, writable
    uint8_t* kvv_w;
};

template <int HD>
struct Cfg {
    static constexpr int NBLK = HD / 32;
    static constexpr int REC = HD + 2 * NBLK;
    static constexpr int KSTEP = HD == 128 ? 4 : 2;     // key stride between consecutive MMA rows
    static constexpr int TILE_BYTES = TILE * REC;
    static constexpr int QSTR = HD + 32;                 // halves per staged Q row (64 B of padding)
};

// shared-memory bytes of one CTA
template <int HD, int NT>
__host__ __device__ constexpr size_t smem_bytes(int RG, int n_seq) {
    return (size_t)stages_of<HD, NT>() * 2 * Cfg<HD>::TILE_BYTES + (size_t)NT * 8 * Cfg<HD>::QSTR * 2 +
           (size_t)NW * RG * (HD + 2) * 4 + 2 * stages_of<HD, NT>() * 8 + (size_t)(n_seq + 2) * 4 + 16;
}

__device__ __forceinline__ int perm16(int kappa) { return kappa ^ ((kappa >> 2) & 1); }

// AP: 1 = the decode call that appends its own (prepared) row, 2 = the one that also runs the QKV prologue of its row
// (separate instances, so that the plain kernel carries none of it)
template <int HD, int NT, int AP = 0>
__global__ void __launch_bounds__(NTHREADS, (NT == 1 ? 3 : (NT == 2 ? 2 : 1)))
k_flash_decode(const Params P) {
    using C = Cfg<HD>;
    constexpr int NBLK = C::NBLK, REC = C::REC, KSTEP = C::KSTEP, TILE_BYTES = C::TILE_BYTES, QSTR = C::QSTR;
    constexpr int STAGES = stages_of<HD, NT>();
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_abort;
    const int RG = P.RG;
    uint8_t* stages = smem;
    __half* qs = reinterpret_cast<__half*>(smem + STAGES * 2 * TILE_BYTES);
    float* mbuf = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(qs) + NT * 8 * QSTR * 2);
    uint64_t* full = reinterpret_cast<uint64_t*>(mbuf + (size_t)NW * RG * (HD + 2));
    uint64_t* empty = full + STAGES;
    int* cum = reinterpret_cast<int*>(empty + STAGES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- every CTA derives the same work cut from the device-resident positions -------------------
    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], NW); }
        mbar_fence_init();
    }
    const bool early = P.early != 0;
    if (!early) {
        pdl_wait();      // nothing above reads or writes global memory
        pdl_trigger();
    }
    if (P.n_seq == 1) {
        // one sequence (decode / verify of a single stream): no prefix sum, one barrier
        if (tid == 0) {
            const SeqRange sr = seq_range(P.pos, P.kslot, P.act, 0, P.rows, P.is_swa, P.W, P.slot_ctx, P.n_slots, P.status);
            cum[0] = 0;
            cum[1] = sr.active ? ((sr.hi + TILE - 1) / TILE - sr.lo / TILE) : 0;
        }
        __syncthreads();
    } else {
        for (int i = tid; i < P.n_seq; i += NTHREADS) {
            const SeqRange sr = seq_range(P.pos, P.kslot, P.act, i, P.rows, P.is_swa, P.W, P.slot_ctx, P.n_slots, P.status);
            cum[i + 1] = sr.active ? ((sr.hi + TILE - 1) / TILE - sr.lo / TILE) : 0;
        }
        if (tid == 0) cum[0] = 0;
        __syncthreads();
        if (warp == 0) {
            int carry = 0;
            for (int base = 0; base < P.n_seq; base += 32) {
                const int idx = base + lane;
                int v = idx < P.n_seq ? cum[idx + 1] : 0;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, v, o);
                    if (lane >= o) v += t;
                }
                v += carry;
                if (idx < P.n_seq) cum[idx + 1] = v;
                carry = __shfl_sync(0xffffffffu, v, 31);
            }
        }
        __syncthreads();
    }
    const int total = P.Hkv * cum[P.n_seq];
    const Share share = cut_share(cum, P.n_seq, P.Hkv, P.cph, (int)blockIdx.x, (int)gridDim.x);
    const int per = share.per;
    if (blockIdx.x == 0) {
        // the header and the step counter are read by the previous call's merge: written after the wait
        if (early) { pdl_wait(); pdl_trigger(); }
        if (P.epoch_ptr && tid == 0) *P.epoch_ptr += P.epoch_advance;
        if (tid == 0) { P.hdr[0] = per; P.hdr[1] = total; }
        for (int i = tid; i <= P.n_seq; i += NTHREADS) P.hdr[2 + i] = cum[i];
    }
    const int g0 = share.g0, g1 = share.g1;
    if (g0 >= g1) return;                           // uniform for the whole CTA

    if (warp == NW) {
        // =========================== producer: one thread issues the bulk copies ===================
        if (lane == 0) {
            int cnt = 0;
            bool waited = !early || blockIdx.x == 0;
            for (int g = g0; g < g1;) {
                const Piece pc = locate(g, g1, cum, P.n_seq, P.Hkv);
                const SeqRange sr = seq_range(P.pos, P.kslot, P.act, pc.i, P.rows, P.is_swa, P.W, P.slot_ctx,
                                              P.n_slots, P.status);
                const size_t hb = ((size_t)sr.slot * P.Hkv + pc.kvh) * P.pstride * (size_t)REC;
                const int tile0 = sr.lo / TILE + pc.tl;
                // paged cache: the table entry of the next tile is fetched one tile ahead, so the look-up never sits
                // between a freed stage and its refill
                const int* trow = P.pg.table ? P.pg.table + (size_t)sr.slot * P.pg.max_pages : nullptr;
                int page_nx = trow ? trow[(tile0 * TILE) >> P.pg.shift] : 0;
                for (int t = 0; t < pc.n; ++t, ++cnt) {
                    const int s = cnt % STAGES, use = cnt / STAGES;
                    const int page = page_nx;
                    if (trow && t + 1 < pc.n) page_nx = trow[((tile0 + t + 1) * TILE) >> P.pg.shift];
                    // early streaming stops at the tile that holds the row BEFORE this step's own rows (the decode
                    // kernel of a preceding appending call, which writes that row, may still be running: its merge
                    // releases this launch before it waits), and before the first stage that needs the consumers
                    // (they do not start before the predecessor has finished)
                    if (!waited && ((tile0 + t + 1) * TILE >= sr.p0 || use > 0)) {
                        pdl_wait();
                        pdl_trigger();
                        waited = true;
                    }
                    if (use > 0 && !*(volatile int*)&s_abort) {
                        if (!mbar_wait_bounded(&empty[s], (use - 1) & 1)) {
                            atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
                            *(volatile int*)&s_abort = 1;
                        }
                    }
                    if (*(volatile int*)&s_abort) continue;     // stop issuing; consumers skip their waits
                    const int sp = ((tile0 + t) * TILE) & P.ring_mask;
                    const int nk = trow ? TILE : min(TILE, P.pstride - sp);
                    const uint32_t bytes = (uint32_t)nk * REC;
                    const size_t src = trow ? kv_rec_index_page(P.pg, page, pc.kvh, P.Hkv, sp, P.status) * (size_t)REC
                                            : hb + (size_t)sp * REC;
                    uint8_t* dstk = stages + (size_t)s * 2 * TILE_BYTES;
                    mbar_expect_tx(&full[s], 2 * bytes);
                    bulk_g2s(dstk, P.kvk + src, bytes, &full[s]);
                    bulk_g2s(dstk + TILE_BYTES, P.kvv + src, bytes, &full[s]);
                }
                g += pc.n;
            }
            if (!waited) { pdl_wait(); pdl_trigger(); }
        }
    } else {
        // =========================== consumers ======================================================
        if (early && blockIdx.x != 0) { pdl_wait(); pdl_trigger(); }      // Q and the records come after the predecessor
        const int gid = lane >> 2, t4 = lane & 3;
        const int ctid = tid;                                     // 0..127
        // local key (within the 64-key tile) of MMA row kappa for this warp
        auto kloc = [&](int kappa) {
            return (warp / KSTEP) * 16 * KSTEP + KSTEP * perm16(kappa) + (warp % KSTEP);
        };
        const int kl0 = kloc(gid), kl1 = kloc(gid + 8);            // rows of the S^T accumulator
        const int klA = kloc(2 * t4), klB = kloc(2 * t4 + 1);      // contraction rows of the P.V MMA
        const int klC = kloc(2 * t4 + 8), klD = kloc(2 * t4 + 9);

        int cnt = 0;
        for (int g = g0; g < g1;) {
            const Piece pc = locate(g, g1, cum, P.n_seq, P.Hkv);
            const SeqRange sr = seq_range(P.pos, P.kslot, P.act, pc.i, P.rows, P.is_swa, P.W, P.slot_ctx,
                                          P.n_slots, P.status);
            const int item = pc.i * P.Hkv + pc.kvh;

            named_bar_sync(1, NW * 32);            // previous piece finished with qs / mbuf
            // ---- stage Q of this item as fp16 [pair][HD]; pair = row * G + head-in-group ----------
            if constexpr (AP == 2) {
                // the prologue of this item's query heads, one warp per head, with the prologue kernel's arithmetic
                // (qkv_prep.cuh); the fp16 rounding is the one battn_qkv_prep (fp16 q) or the staging below (fp32 q) applies
                constexpr int VEC = HD / 64, H2 = HD / 2;
                float c[VEC], s_[VEC];
                prep::tables<HD>(P.cs + (size_t)pc.i * HD + P.table_off, P.sn + (size_t)pc.i * HD + P.table_off, lane, c, s_);
                for (int n = warp; n < NT * 8; n += NW) {
                    __half* row = qs + n * QSTR;
                    if (n < RG) {
                        const int hq = pc.kvh * P.G + n;             // rows == 1: pair n is head n of the group
                        float lo[VEC], hi[VEC];
                        prep::q_head<HD>(P.q_raw + ((size_t)pc.i * P.Hq + hq) * HD, P.sqk + (size_t)hq * HD, c, s_, lane, lo, hi);
#pragma unroll
                        for (int j = 0; j < VEC; j += 2) {
                            *reinterpret_cast<__half2*>(row + VEC * lane + j) = __floats2half2_rn(lo[j], lo[j + 1]);
                            *reinterpret_cast<__half2*>(row + H2 + VEC * lane + j) = __floats2half2_rn(hi[j], hi[j + 1]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < VEC; j += 2) {
                            *reinterpret_cast<__half2*>(row + VEC * lane + j) = __floats2half2_rn(0.f, 0.f);
                            *reinterpret_cast<__half2*>(row + H2 + VEC * lane + j) = __floats2half2_rn(0.f, 0.f);
                        }
                    }
                }
            } else
            for (int idx = ctid; idx < NT * 8 * (HD / 8); idx += NW * 32) {
                const int n = idx / (HD / 8), ch = idx - n * (HD / 8);
                uint4 val = make_uint4(0u, 0u, 0u, 0u);
                if (n < RG) {
                    const int r = n / P.G, h = n - r * P.G;
                    const size_t qi = (((size_t)pc.i * P.rows + r) * P.Hq + pc.kvh * P.G + h) * HD + ch * 8;
                    if (P.q_f16) {
                        val = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(P.q) + qi);
                    } else {
                        const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.q) + qi);
                        const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.q) + qi + 4);
                        val = make_uint4(pack_h2(a.x, a.y), pack_h2(a.z, a.w), pack_h2(b.x, b.y), pack_h2(b.z, b.w));
                    }
                }
                *reinterpret_cast<uint4*>(qs + n * QSTR + ch * 8) = val;
            }
            named_bar_sync(1, NW * 32);

            // per-column visibility limits: column (nt, e) is pair n = nt*8 + 2*t4 + e, row r = n / G
            int lim[NT][2], low[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int r = min((nt * 8 + 2 * t4 + e) / P.G, P.rows - 1);
                    lim[nt][e] = sr.p0 + r;                                       // bruce.cu:2056
                    low[nt][e] = P.is_swa ? max(0, sr.p0 + r + 1 - P.W) : 0;      // bruce.cu:3688
                }
            const int full_lo = P.is_swa ? max(0, sr.p0 + P.rows - P.W) : 0;      // window start of the last row

            float m[NT][2], l[NT][2], O[NBLK][2][NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                m[nt][0] = m[nt][1] = NEG_BIG;
                l[nt][0] = l[nt][1] = 0.f;
#pragma unroll
                for (int b = 0; b < NBLK; ++b)
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int c = 0; c < 4; ++c) O[b][u][nt][c] = 0.f;
            }

            const int tile0 = sr.lo / TILE + pc.tl;
            for (int t = 0; t < pc.n; ++t, ++cnt) {
                const int s = cnt % STAGES, use = cnt / STAGES;
                if (!*(volatile int*)&s_abort) {
                    if (!mbar_wait_bounded(&full[s], use & 1)) {
                        atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
                        *(volatile int*)&s_abort = 1;
                    }
                }
                const uint8_t* Kt = stages + (size_t)s * 2 * TILE_BYTES;
                const uint8_t* Vt = Kt + TILE_BYTES;
                const int t0 = (tile0 + t) * TILE;
                if (AP && sr.p0 >= t0 && sr.p0 < t0 + TILE) {
                    // the tile of the call's own row: warp 0 writes the K record, warp 1 the V record
                    if (warp < 2) {
                        const float* src = (warp ? P.v_new : P.k_new) + ((size_t)pc.i * P.Hkv + pc.kvh) * HD;
                        uint8_t* tile = stages + (size_t)s * 2 * TILE_BYTES + (warp ? TILE_BYTES : 0);
                        const size_t ri = kv_rec_index(P.pg, sr.slot, pc.kvh, P.Hkv, P.pstride, sr.p0 & P.ring_mask, P.status);
                        uint8_t* rec_t = tile + (sr.p0 - t0) * REC;
                        uint8_t* rec_c = (warp ? P.kvv_w : P.kvk_w) + ri * (size_t)REC;
                        if constexpr (AP == 2) {
                            // raw rows: k is scaled and rotated first, v is quantised as it is (qkv_prep.cuh)
                            constexpr int VEC = HD / 64, H2 = HD / 2;
                            float x0[VEC], x1[VEC];
                            if (warp == 0) {
                                float c[VEC], s_[VEC];
                                prep::tables<HD>(P.cs + (size_t)pc.i * HD + P.table_off, P.sn + (size_t)pc.i * HD + P.table_off,
                                                 lane, c, s_);
                                prep::k_head<HD>(src, c, s_, lane, x0, x1);
                            } else {
                                prep::load<VEC>(src + VEC * lane, x0);
                                prep::load<VEC>(src + H2 + VEC * lane, x1);
                            }
                            prep::quant_head<HD>(rec_t, x0, x1, lane);
                            prep::quant_head<HD>(rec_c, x0, x1, lane);
                        } else {
                            quantise_record<HD>(src, rec_t, lane);
                            quantise_record<HD>(src, rec_c, lane);
                        }
                        // the stage is refilled by a bulk copy later: order these generic-proxy writes before it
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    }
                    named_bar_sync(1, NW * 32);
                }
                // tiles every row sees completely take the mask-free path (bruce.cu:2927-2928)
                const bool masked = !(t0 >= full_lo && t0 + TILE - 1 <= sr.p0);

                // ---------------- S^T = K Q^T : 16 keys x (8*NT) pairs --------------------------------
                float sv[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) sv[nt][0] = sv[nt][1] = sv[nt][2] = sv[nt][3] = 0.f;
                {
                    const uint8_t* k0 = Kt + kl0 * REC;
                    const uint8_t* k1 = Kt + kl1 * REC;
                    float d0[NBLK], d1[NBLK];
                    if constexpr (NBLK == 4) {
                        const uint2 a = *reinterpret_cast<const uint2*>(k0);
                        const uint2 b = *reinterpret_cast<const uint2*>(k1);
                        const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&a.x));
                        const float2 a1 = __half22float2(*reinterpret_cast<const __half2*>(&a.y));
                        const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(&b.x));
                        const float2 b1 = __half22float2(*reinterpret_cast<const __half2*>(&b.y));
                        d0[0] = a0.x; d0[1] = a0.y; d0[2] = a1.x; d0[3] = a1.y;
                        d1[0] = b0.x; d1[1] = b0.y; d1[2] = b1.x; d1[3] = b1.y;
                    } else {
#pragma unroll
                        for (int b = 0; b < NBLK; ++b) {
                            d0[b] = __half2float(reinterpret_cast<const __half*>(k0)[b]);
                            d1[b] = __half2float(reinterpret_cast<const __half*>(k1)[b]);
                        }
                    }
#pragma unroll
                    for (int b = 0; b < NBLK; ++b) {
                        const uint2 w0 = *reinterpret_cast<const uint2*>(k0 + 2 * NBLK + b * 32 + t4 * 8);
                        const uint2 w1 = *reinterpret_cast<const uint2*>(k1 + 2 * NBLK + b * 32 + t4 * 8);
                        const uint32_t x0 = w0.x ^ 0x80808080u, x1 = w1.x ^ 0x80808080u;
                        const uint32_t y0 = w0.y ^ 0x80808080u, y1 = w1.y ^ 0x80808080u;
                        uint32_t a[2][4];
                        a[0][0] = sub1152(widen_lo(x0)); a[0][1] = sub1152(widen_lo(x1));
                        a[0][2] = sub1152(widen_hi(x0)); a[0][3] = sub1152(widen_hi(x1));
                        a[1][0] = sub1152(widen_lo(y0)); a[1][1] = sub1152(widen_lo(y1));
                        a[1][2] = sub1152(widen_hi(y0)); a[1][3] = sub1152(widen_hi(y1));
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const uint4 qv = *reinterpret_cast<const uint4*>(qs + (nt * 8 + gid) * QSTR + b * 32 + t4 * 8);
                            float acc[4] = {0.f, 0.f, 0.f, 0.f};
                            mma16816(acc, a[0], qv.x, qv.y);
                            mma16816(acc, a[1], qv.z, qv.w);
                            sv[nt][0] = fmaf(d0[b], acc[0], sv[nt][0]);
                            sv[nt][1] = fmaf(d0[b], acc[1], sv[nt][1]);
                            sv[nt][2] = fmaf(d1[b], acc[2], sv[nt][2]);
                            sv[nt][3] = fmaf(d1[b], acc[3], sv[nt][3]);
                        }
                    }
                }

                // ---------------- online softmax over this warp's 16 keys ------------------------------
                uint32_t pb0[NT], pb1[NT];
                bool any_rescale = false;
                float alpha[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float pe[4];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        float v0 = sv[nt][e] * P.scale_log2, v1 = sv[nt][2 + e] * P.scale_log2;
                        if (masked) {
                            const int key0 = t0 + kl0, key1 = t0 + kl1;
                            if (key0 > lim[nt][e] || key0 < low[nt][e]) v0 = NEG_BIG;
                            if (key1 > lim[nt][e] || key1 < low[nt][e]) v1 = NEG_BIG;
                        }
                        float mx = fmaxf(v0, v1);
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                        const float mn = fmaxf(m[nt][e], mx);
                        const float al = fast_exp2(m[nt][e] - mn);
                        float p0 = fast_exp2(v0 - mn), p1 = fast_exp2(v1 - mn);
                        if (masked) {
                            if (v0 < -1e29f) p0 = 0.f;
                            if (v1 < -1e29f) p1 = 0.f;
                        }
                        any_rescale |= (mn != m[nt][e]);
                        alpha[nt][e] = al;
                        m[nt][e] = mn;
                        pe[e] = p0; pe[2 + e] = p1;
                    }
                    const uint32_t h01 = pack_h2(pe[0], pe[1]), h23 = pack_h2(pe[2], pe[3]);
                    // the denominator sums the fp16-rounded weights the MMA will use, so that
                    // out = sum(p v) / sum(p) stays a convex combination of the V rows
                    const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
                    const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
                    l[nt][0] = fmaf(l[nt][0], alpha[nt][0], f01.x + f23.x);
                    l[nt][1] = fmaf(l[nt][1], alpha[nt][1], f01.y + f23.y);
                    pb0[nt] = movmatrix_trans(h01);     // keys kappa = 2t4, 2t4+1
                    pb1[nt] = movmatrix_trans(h23);     // keys kappa = 2t4+8, 2t4+9
                }
                if (__any_sync(0xffffffffu, any_rescale)) {
#pragma unroll
                    for (int b = 0; b < NBLK; ++b)
#pragma unroll
                        for (int u = 0; u < 2; ++u)
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                O[b][u][nt][0] *= alpha[nt][0]; O[b][u][nt][1] *= alpha[nt][1];
                                O[b][u][nt][2] *= alpha[nt][0]; O[b][u][nt][3] *= alpha[nt][1];
                            }
                }

                // ---------------- O^T += V^T P^T ---------------------------------------------------------
                {
                    const uint8_t* vA = Vt + klA * REC;
                    const uint8_t* vB = Vt + klB * REC;
                    const uint8_t* vC = Vt + klC * REC;
                    const uint8_t* vD = Vt + klD * REC;
                    // V scales as half2 pairs (key A, key B) and (key C, key D) per block
                    uint32_t sAB[NBLK], sCD[NBLK];
                    {
                        uint32_t wa[NBLK / 2], wb[NBLK / 2], wc[NBLK / 2], wd[NBLK / 2];
#pragma unroll
                        for (int j = 0; j < NBLK / 2; ++j) {
                            wa[j] = reinterpret_cast<const uint32_t*>(vA)[j];
                            wb[j] = reinterpret_cast<const uint32_t*>(vB)[j];
                            wc[j] = reinterpret_cast<const uint32_t*>(vC)[j];
                            wd[j] = reinterpret_cast<const uint32_t*>(vD)[j];
                        }
                        if (masked) {
                            // keys outside [lo, hi) were never written for this sequence: their bytes
                            // are arbitrary, so their V scale is forced to zero (their P is zero too)
                            const bool okA = t0 + klA >= sr.lo && t0 + klA < sr.hi;
                            const bool okB = t0 + klB >= sr.lo && t0 + klB < sr.hi;
                            const bool okC = t0 + klC >= sr.lo && t0 + klC < sr.hi;
                            const bool okD = t0 + klD >= sr.lo && t0 + klD < sr.hi;
#pragma unroll
                            for (int j = 0; j < NBLK / 2; ++j) {
                                if (!okA) wa[j] = 0u;
                                if (!okB) wb[j] = 0u;
                                if (!okC) wc[j] = 0u;
                                if (!okD) wd[j] = 0u;
                            }
                        }
#pragma unroll
                        for (int j = 0; j < NBLK / 2; ++j) {
                            sAB[2 * j] = __byte_perm(wa[j], wb[j], 0x5410);
                            sAB[2 * j + 1] = __byte_perm(wa[j], wb[j], 0x7632);
                            sCD[2 * j] = __byte_perm(wc[j], wd[j], 0x5410);
                            sCD[2 * j + 1] = __byte_perm(wc[j], wd[j], 0x7632);
                        }
                    }
#pragma unroll
                    for (int b = 0; b < NBLK; ++b) {
                        const int off = 2 * NBLK + b * 32 + gid * 4;
                        const uint32_t xa = *reinterpret_cast<const uint32_t*>(vA + off) ^ 0x80808080u;
                        const uint32_t xb = *reinterpret_cast<const uint32_t*>(vB + off) ^ 0x80808080u;
                        const uint32_t xc = *reinterpret_cast<const uint32_t*>(vC + off) ^ 0x80808080u;
                        const uint32_t xd = *reinterpret_cast<const uint32_t*>(vD + off) ^ 0x80808080u;
                        // [A.b0 B.b0 A.b1 B.b1] and [A.b2 B.b2 A.b3 B.b3]: key pairs side by side per dim
                        const uint32_t ab[2] = {__byte_perm(xa, xb, 0x5140), __byte_perm(xa, xb, 0x7362)};
                        const uint32_t cd[2] = {__byte_perm(xc, xd, 0x5140), __byte_perm(xc, xd, 0x7362)};
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            uint32_t a[4];
                            a[0] = hmul2_u32(sub1152(widen_lo(ab[u])), sAB[b]);   // dim 4gid+2u,   keys A,B
                            a[1] = hmul2_u32(sub1152(widen_hi(ab[u])), sAB[b]);   // dim 4gid+2u+1, keys A,B
                            a[2] = hmul2_u32(sub1152(widen_lo(cd[u])), sCD[b]);   // dim 4gid+2u,   keys C,D
                            a[3] = hmul2_u32(sub1152(widen_hi(cd[u])), sCD[b]);   // dim 4gid+2u+1, keys C,D
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) mma16816(O[b][u][nt], a, pb0[nt], pb1[nt]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }

            // ---------------- piece end: merge the four warps' states, write one split record ----------
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float v = l[nt][e];
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    v += __shfl_xor_sync(0xffffffffu, v, 8);
                    v += __shfl_xor_sync(0xffffffffu, v, 16);
                    l[nt][e] = v;
                }
            float* mb = mbuf + (size_t)warp * RG * (HD + 2);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int n = nt * 8 + 2 * t4 + e;
                    if (n < RG) {
                        float* row = mb + (size_t)n * (HD + 2);
#pragma unroll
                        for (int b = 0; b < NBLK; ++b)
#pragma unroll
                            for (int u = 0; u < 2; ++u) {
                                row[b * 32 + gid * 4 + 2 * u] = O[b][u][nt][e];
                                row[b * 32 + gid * 4 + 2 * u + 1] = O[b][u][nt][2 + e];
                            }
                        if (gid == 0) { row[HD] = m[nt][e]; row[HD + 1] = l[nt][e]; }
                    }
                }
            named_bar_sync(1, NW * 32);
            // records in the workspace are padded to HD + 4 floats (16-byte aligned for the merge kernel)
            float* dst = P.part + (size_t)(blockIdx.x + item) * RG * (HD + 4);
            for (int idx = ctid; idx < RG * HD; idx += NW * 32) {
                const int n = idx / HD, d = idx - n * HD;
                float mw[NW], M = NEG_BIG;
#pragma unroll
                for (int w = 0; w < NW; ++w) {
                    mw[w] = mbuf[((size_t)w * RG + n) * (HD + 2) + HD];
                    M = fmaxf(M, mw[w]);
                }
                float acc = 0.f, L = 0.f;
#pragma unroll
                for (int w = 0; w < NW; ++w) {
                    const float f = fast_exp2(mw[w] - M);
                    acc = fmaf(mbuf[((size_t)w * RG + n) * (HD + 2) + d], f, acc);
                    L = fmaf(mbuf[((size_t)w * RG + n) * (HD + 2) + HD + 1], f, L);
                }
                dst[(size_t)n * (HD + 4) + d] = acc;
                if (d == 0) { dst[(size_t)n * (HD + 4) + HD] = M; dst[(size_t)n * (HD + 4) + HD + 1] = L; }
            }
            g += pc.n;
        }
    }
    __syncthreads();   // keep the CTA (and its shared memory) alive until every role is done
}

}  // namespace fd
}  // namespace battn
