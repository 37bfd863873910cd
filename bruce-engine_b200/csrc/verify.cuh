// Wide speculative-verify attention: 5..8 query rows (17..32 (row, head) pairs per kv head) sharing one
// sweep over the q8_0 cache.
//
// Behaviour replaced: k_attn_tc_rs_opt<4,3,false,true> for 5..8 verify rows and its dispatch
// (engine/src/bruce.cu:3994-4019); contract as k_attn_m<M> (:2087-2143): rows at p0..p0+rows-1, keys before
// p0 visible to every row, in-chunk causal mask key <= p0 + r, optional per-row window.
//
// Why a second kernel: with 32 pairs per kv head the flash-decode kernel (each warp: 16 keys x all pairs)
// needs 128 accumulator registers per thread, runs one CTA per SM and is instruction-bound at a quarter
// of HBM rate.  Here the four consumer warps first convert their quarter of a 64-key tile to fp16 in
// shared memory (K as exact integers, V with its scale folded in), then each warp owns ONE group of 8
// pairs over all 64 keys: A operands come from the shared fp16 tile with ldmatrix (V transposed by
// ldmatrix.trans), accumulators are 32 registers, the row maximum is taken once per tile, and no merge
// across warps is needed.  Work cut, TMA bulk-copy producer, split records and the merge kernel are the
// flash-decode kernel's.
#pragma once
#include "common.cuh"
#include "flash_decode.cuh"

namespace battn {
namespace vw {

constexpr int NW = 4;
constexpr int TILE = fd::TILE;            // 64 keys
constexpr int NTHREADS = (NW + 1) * 32;
constexpr int STAGES = 2;

template <int HD>
struct Cfg {
    static constexpr int NBLK = HD / 32;
    static constexpr int REC = HD + 2 * NBLK;
    static constexpr int TILE_BYTES = TILE * REC;
    static constexpr int HSTR = HD + 8;                    // halves per fp16 row (16 B of padding: ldmatrix conflict-free)
    static constexpr int H_BYTES = TILE * HSTR * 2;        // one fp16 tile (K or V)
};

template <int HD>
__host__ __device__ constexpr size_t smem_bytes(int n_seq) {
    return (size_t)STAGES * 2 * Cfg<HD>::TILE_BYTES + 2 * (size_t)Cfg<HD>::H_BYTES + 2 * STAGES * 8 +
           (size_t)(n_seq + 2) * 4 + 16;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}

template <int HD>
__global__ void __launch_bounds__(NTHREADS, HD == 128 ? 3 : 1) k_verify_wide(const fd::Params P) {
    using C = Cfg<HD>;
    constexpr int NBLK = C::NBLK, REC = C::REC, TILE_BYTES = C::TILE_BYTES, HSTR = C::HSTR;
    constexpr int RS = HD + 4;                               // floats per split record in the workspace
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_abort;
    uint8_t* stages = smem;
    __half* Kh = reinterpret_cast<__half*>(smem + STAGES * 2 * TILE_BYTES);
    __half* Vh = Kh + TILE * HSTR;
    uint64_t* full = reinterpret_cast<uint64_t*>(Vh + TILE * HSTR);
    uint64_t* empty = full + STAGES;
    int* cum = reinterpret_cast<int*>(empty + STAGES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int RG = P.RG;

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], NW); }
        mbar_fence_init();
    }
    pdl_wait();
    pdl_trigger();
    if (P.epoch_ptr && blockIdx.x == 0 && tid == 0) *P.epoch_ptr += P.epoch_advance;
    // ---- the flash-decode work cut: every CTA derives the same tile shares from the positions -------
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
    const int total = P.Hkv * cum[P.n_seq];
    const fd::Share share = fd::cut_share(cum, P.n_seq, P.Hkv, P.cph, (int)blockIdx.x, (int)gridDim.x);
    const int per = share.per;
    if (blockIdx.x == 0) {
        if (tid == 0) { P.hdr[0] = per; P.hdr[1] = total; }
        for (int i = tid; i <= P.n_seq; i += NTHREADS) P.hdr[2 + i] = cum[i];
    }
    const int g0 = share.g0, g1 = share.g1;
    if (g0 >= g1) return;

    if (warp == NW) {
        // =========================== producer ==========================================================
        if (lane == 0) {
            int cnt = 0;
            for (int g = g0; g < g1;) {
                const fd::Piece pc = fd::locate(g, g1, cum, P.n_seq, P.Hkv);
                const SeqRange sr = seq_range(P.pos, P.kslot, P.act, pc.i, P.rows, P.is_swa, P.W, P.slot_ctx,
                                              P.n_slots, P.status);
                const size_t hb = ((size_t)sr.slot * P.Hkv + pc.kvh) * P.pstride * (size_t)REC;
                const int tile0 = sr.lo / TILE + pc.tl;
                // paged cache: the table entry of the next tile is fetched one tile ahead of its use
                const int* trow = P.pg.table ? P.pg.table + (size_t)sr.slot * P.pg.max_pages : nullptr;
                int page_nx = trow ? trow[(tile0 * TILE) >> P.pg.shift] : 0;
                for (int t = 0; t < pc.n; ++t, ++cnt) {
                    const int s = cnt % STAGES, use = cnt / STAGES;
                    const int page = page_nx;
                    if (trow && t + 1 < pc.n) page_nx = trow[((tile0 + t + 1) * TILE) >> P.pg.shift];
                    if (use > 0 && !*(volatile int*)&s_abort) {
                        if (!mbar_wait_bounded(&empty[s], (use - 1) & 1)) {
                            atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
                            *(volatile int*)&s_abort = 1;
                        }
                    }
                    if (*(volatile int*)&s_abort) continue;
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
        }
    } else {
        // =========================== consumers =========================================================
        const int gid = lane >> 2, t4 = lane & 3;
        const int pair0 = warp * 8;                              // this warp's 8 (row, head) pairs
        // ldmatrix lane addressing: matrix index l/8, row-in-matrix l%8
        const int lm_row = (lane & 7) + 8 * ((lane >> 3) & 1);   // K: rows 0-15 of the m tile, matrices 0/1 (2/3 same rows)
        const int lm_col = 8 * (lane >> 4);                      // K: k offset 0 or 8
        const int lv_key = (lane & 7) + 8 * (lane >> 4);         // V^T: key row of the 8x8 block, matrices 2/3 are keys +8
        const int lv_dim = 8 * ((lane >> 3) & 1);                // V^T: matrices 1/3 are dims +8

        int cnt = 0;
        for (int g = g0; g < g1;) {
            const fd::Piece pc = fd::locate(g, g1, cum, P.n_seq, P.Hkv);
            const SeqRange sr = seq_range(P.pos, P.kslot, P.act, pc.i, P.rows, P.is_swa, P.W, P.slot_ctx,
                                          P.n_slots, P.status);
            const int item = pc.i * P.Hkv + pc.kvh;

            // ---- Q^T B fragments of this warp's pairs, all k-steps: q[pair gid][16 ks + 2 t4 (+8)] ------
            uint32_t qb[HD / 16][2];
            {
                const int n = pair0 + gid;
                const bool live = n < RG;
                const int r = live ? n / P.G : 0, h = live ? n - r * P.G : 0;
                const size_t qi = (((size_t)pc.i * P.rows + r) * P.Hq + pc.kvh * P.G + h) * HD;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    if (!live) { qb[ks][0] = qb[ks][1] = 0u; continue; }
                    if (P.q_f16) {
                        const __half* qp = reinterpret_cast<const __half*>(P.q) + qi + ks * 16 + 2 * t4;
                        qb[ks][0] = *reinterpret_cast<const uint32_t*>(qp);
                        qb[ks][1] = *reinterpret_cast<const uint32_t*>(qp + 8);
                    } else {
                        const float* qp = reinterpret_cast<const float*>(P.q) + qi + ks * 16 + 2 * t4;
                        const float2 a = *reinterpret_cast<const float2*>(qp), b = *reinterpret_cast<const float2*>(qp + 8);
                        qb[ks][0] = pack_h2(a.x, a.y);
                        qb[ks][1] = pack_h2(b.x, b.y);
                    }
                }
            }
            // visibility limits of this thread's two columns (pairs pair0 + 2 t4 + e)
            int lim[2], low[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int r = min((pair0 + 2 * t4 + e) / P.G, P.rows - 1);
                lim[e] = sr.p0 + r;                                            // bruce.cu:2056
                low[e] = P.is_swa ? max(0, sr.p0 + r + 1 - P.W) : 0;           // bruce.cu:3688
            }
            const int full_lo = P.is_swa ? max(0, sr.p0 + P.rows - P.W) : 0;

            float m[2] = {NEG_BIG, NEG_BIG}, l[2] = {0.f, 0.f};
            float O[HD / 16][4];                                               // O^T: 16-dim tiles x (2 dims x 2 pairs)
#pragma unroll
            for (int dt = 0; dt < HD / 16; ++dt) O[dt][0] = O[dt][1] = O[dt][2] = O[dt][3] = 0.f;

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
                const bool masked = !(t0 >= full_lo && t0 + TILE - 1 <= sr.p0);

                named_bar_sync(1, NW * 32);          // every warp is done with the previous fp16 tile
                // ---------------- convert this warp's 16 keys: 8-byte chunks, 16 per key -----------------
#pragma unroll
                for (int it = 0; it < (16 * HD / 8) / 32; ++it) {
                    const int idx = it * 32 + lane;
                    const int key = warp * 16 + idx / (HD / 8), ch = idx % (HD / 8);
                    const uint8_t* kr = Kt + key * REC;
                    const uint8_t* vr = Vt + key * REC;
                    const uint2 kw = *reinterpret_cast<const uint2*>(kr + 2 * NBLK + ch * 8);
                    const uint2 vw = *reinterpret_cast<const uint2*>(vr + 2 * NBLK + ch * 8);
                    __half dv = reinterpret_cast<const __half*>(vr)[ch >> 2];
                    if (masked && (t0 + key < sr.lo || t0 + key >= sr.hi)) dv = __float2half_rn(0.f);   // never-written slot
                    const __half2 d2 = __half2half2(dv);
                    const uint32_t du = *reinterpret_cast<const uint32_t*>(&d2);
                    const uint32_t kx = kw.x ^ 0x80808080u, ky = kw.y ^ 0x80808080u;
                    const uint32_t vx = vw.x ^ 0x80808080u, vy = vw.y ^ 0x80808080u;
                    const uint4 ko = make_uint4(sub1152(widen_lo(kx)), sub1152(widen_hi(kx)), sub1152(widen_lo(ky)),
                                                sub1152(widen_hi(ky)));
                    const uint4 vo = make_uint4(hmul2_u32(sub1152(widen_lo(vx)), du), hmul2_u32(sub1152(widen_hi(vx)), du),
                                                hmul2_u32(sub1152(widen_lo(vy)), du), hmul2_u32(sub1152(widen_hi(vy)), du));
                    *reinterpret_cast<uint4*>(Kh + key * HSTR + ch * 8) = ko;
                    *reinterpret_cast<uint4*>(Vh + key * HSTR + ch * 8) = vo;
                }
                named_bar_sync(1, NW * 32);          // the whole fp16 tile is in place

                // ---------------- S^T = K Q^T for 64 keys x 8 pairs; K scales applied per 32-dim block -----
                float sv[4][4];
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) {
                    sv[mt][0] = sv[mt][1] = sv[mt][2] = sv[mt][3] = 0.f;
                    const uint8_t* k0 = Kt + (mt * 16 + gid) * REC;          // scales of this thread's two keys
                    const uint8_t* k1 = k0 + 8 * REC;
#pragma unroll
                    for (int b = 0; b < NBLK; ++b) {
                        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int kk = 0; kk < 2; ++kk) {
                            const int ks = 2 * b + kk;
                            uint32_t a[4];
                            ldmatrix_x4(a, Kh + (mt * 16 + lm_row) * HSTR + ks * 16 + lm_col);
                            mma16816(acc, a, qb[ks][0], qb[ks][1]);
                        }
                        const float d0 = __half2float(reinterpret_cast<const __half*>(k0)[b]);
                        const float d1 = __half2float(reinterpret_cast<const __half*>(k1)[b]);
                        sv[mt][0] = fmaf(d0, acc[0], sv[mt][0]); sv[mt][1] = fmaf(d0, acc[1], sv[mt][1]);
                        sv[mt][2] = fmaf(d1, acc[2], sv[mt][2]); sv[mt][3] = fmaf(d1, acc[3], sv[mt][3]);
                    }
                }
                // raw tile no longer needed by this warp (the scales above were the last read)
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);

                // ---------------- online softmax, one maximum per column per tile ------------------------------
                float mx[2] = {NEG_BIG, NEG_BIG};
#pragma unroll
                for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        float v0 = sv[mt][e] * P.scale_log2, v1 = sv[mt][2 + e] * P.scale_log2;
                        if (masked) {
                            const int key0 = t0 + mt * 16 + gid, key1 = key0 + 8;
                            if (key0 > lim[e] || key0 < low[e]) v0 = NEG_BIG;
                            if (key1 > lim[e] || key1 < low[e]) v1 = NEG_BIG;
                        }
                        sv[mt][e] = v0; sv[mt][2 + e] = v1;
                        mx[e] = fmaxf(mx[e], fmaxf(v0, v1));
                    }
                float alpha[2];
                bool resc = false;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 4));
                    mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 8));
                    mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 16));
                    const float mn = fmaxf(m[e], mx[e]);
                    alpha[e] = fast_exp2(m[e] - mn);
                    resc |= (mn != m[e]);
                    m[e] = mn;
                }
                uint32_t pb[4][2];                                         // P^T B fragments, one k-step per m tile
                float lsum[2] = {0.f, 0.f};
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) {
                    float pe[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float v = sv[mt][c];
                        pe[c] = (masked && v < -1e29f) ? 0.f : fast_exp2(v - m[c & 1]);
                    }
                    const uint32_t h01 = pack_h2(pe[0], pe[1]), h23 = pack_h2(pe[2], pe[3]);
                    // the denominator sums the fp16-rounded weights the MMA will use
                    const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
                    const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
                    lsum[0] += f01.x + f23.x; lsum[1] += f01.y + f23.y;
                    pb[mt][0] = movmatrix_trans(h01);                       // keys 2t4, 2t4+1 of the m tile
                    pb[mt][1] = movmatrix_trans(h23);                       // keys 2t4+8, 2t4+9
                }
                l[0] = fmaf(l[0], alpha[0], lsum[0]);
                l[1] = fmaf(l[1], alpha[1], lsum[1]);
                if (__any_sync(0xffffffffu, resc)) {
#pragma unroll
                    for (int dt = 0; dt < HD / 16; ++dt) {
                        O[dt][0] *= alpha[0]; O[dt][1] *= alpha[1]; O[dt][2] *= alpha[0]; O[dt][3] *= alpha[1];
                    }
                }
                // ---------------- O^T += V^T P^T : 16-dim tiles x four 16-key steps ----------------------------
#pragma unroll
                for (int dt = 0; dt < HD / 16; ++dt)
#pragma unroll
                    for (int mt = 0; mt < 4; ++mt) {
                        uint32_t a[4];
                        ldmatrix_x4_trans(a, Vh + (mt * 16 + lv_key) * HSTR + dt * 16 + lv_dim);
                        mma16816(O[dt], a, pb[mt][0], pb[mt][1]);
                    }
            }

            // ---------------- piece end: this warp's pairs go straight into the split record -----------------
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v = l[e];
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                l[e] = v;
            }
            float* dst = P.part + (size_t)(blockIdx.x + item) * RG * RS;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int n = pair0 + 2 * t4 + e;
                if (n < RG) {
                    float* row = dst + (size_t)n * RS;
#pragma unroll
                    for (int dt = 0; dt < HD / 16; ++dt) {
                        row[dt * 16 + gid] = O[dt][e];
                        row[dt * 16 + gid + 8] = O[dt][2 + e];
                    }
                    if (gid == 0) { row[HD] = m[e]; row[HD + 1] = l[e]; }
                }
            }
            g += pc.n;
        }
    }
    __syncthreads();
}

}  // namespace vw
}  // namespace battn
