// Prompt-chunk attention for head_dim 128 on the 5th-generation tensor cores: causal + sliding-window
// flash attention of a chunk of query rows against the growing q8_0 cache (the chunk's own keys were
// appended first).
//
// Behaviour replaced: k_attn_tc_rs_opt<NW,...> for rows > 8 and its dispatch
// (engine/src/bruce.cu:2750-3131, 4021-4078); masks as bruce.cu:2799-2805, 3012-3029.
//
// One CTA per (128-row M tile, kv head); the keys stream through in tiles of 64.  Twenty warps, each
// warpgroup resized with setmaxnreg for its role:
//   warps 0-3   softmax group A (even key tiles), one thread per accumulator row
//   warps 4-7   softmax group B (odd key tiles), one thread per accumulator row
//   warps 8-11  K dequant: raw q8_0 records -> fp16 K operand [key][dim], scale folded in
//   warps 12-15 V dequant: raw q8_0 records -> fp16 V^T operand [dim][key], scale folded in
//   warp 16     issues the S MMAs, warp 19 the P.V MMAs;  warps 17/18 stream raw K / V tiles with bulk copies
// Data flow per key tile j (every ring below is three deep and indexed j mod 3):
//   loader -> raw K/V tile (shared memory) -> dequant -> fp16 operand (128-byte-swizzled shared memory)
//   K operand         two fp16 parts per value: hi = fp16(d*x) and lo = d*x - hi (exact: the product of an int8
//                     and an fp16 scale has 19 significant bits, fp16 keeps 11, the rest fits the second part),
//                     so S carries no rounding of K -- a single folded operand alone moves single (row, head)
//                     outputs by up to 7e-4 relative, most of the 1e-3 budget
//   S_j = Q K_hi^T + Q K_lo^T   Q lives in tensor memory (the A operand), S_j in one of three 64-column buffers
//   softmax           the owning group reads S_j once into registers, takes the row maximum, and writes
//                     P_j = 2^(S_j*c - ref) as fp16 pairs over the first half of the same buffer
//   O += P_j [V_j | 1]  P_j is the tensor-memory A operand; sixteen rows of ones appended to the V^T
//                     operand make the same MMA accumulate sum(P) in fp32 next to O, from exactly the
//                     fp16-rounded P it multiplies with V
// The S issuer runs up to three tiles ahead of O, so when a softmax group finishes tile j, S_{j+2} is ready;
// the two groups run half a tile apart, which lets one group's exponentials (the special-function pipe)
// overlap the other group's loads, maxima and stores.
// The row reference `ref` (a lazily updated running maximum, bruce.cu:3034-3060 in spirit) is shared by
// the two threads that own a row in alternate tiles: decisions are taken strictly in tile order (a small
// sequence word per 32-row quarter), and O is rescaled in tensor memory only when a row maximum grows by
// more than 2^8 over the reference; the final normalisation uses the same reference, so the result does
// not depend on how rarely it moves.
// Row n of the K operand / column n of S holds key kappa(n), a fixed permutation inside each 64-key span
// chosen so that every shared-memory access of the dequant warps is bank-conflict free.
// Every wait is bounded; a wait that runs out sets the device status word, the remaining waits are
// skipped, tensor memory is released and the kernel returns.
#pragma once
#include "prefill.cuh"

namespace battn {
namespace pf128 {

using namespace pf;

#ifndef BATTN_PF_NB
#define BATTN_PF_NB 3
#endif
#ifndef BATTN_PF_KLO
#define BATTN_PF_KLO 1
#endif
constexpr int HD = 128, BN = 64, NB = BATTN_PF_NB;     // NB: depth of every ring (raw tiles, operands, S/P)
constexpr bool KLO = BATTN_PF_KLO != 0;
constexpr int NBLK = HD / 32, REC = HD + 2 * NBLK;
constexpr int NTHREADS = 640;
constexpr int W_KDQ = 8, W_VDQ = 12, W_MMA = 16, W_LDK = 17, W_LDV = 18, W_PV = 19;
constexpr int REGS_LAUNCH = 96, REGS_SOFT = 144, REGS_DEQ = 72, REGS_CTL = 40;
static_assert(2 * REGS_SOFT + 2 * REGS_DEQ + REGS_CTL <= 5 * REGS_LAUNCH, "register budget per scheduler");

constexpr int VROWS = HD + 16;                         // V^T operand rows: head_dim + the block of ones
constexpr int K_BYTES = BN * HD * 2;                   // two 64-dim sub-tiles of [64 keys][128 B]
constexpr int V_BYTES = VROWS * 128;                   // [144 rows][64 keys] fp16
constexpr int RAW_BYTES = BN * REC;
constexpr int OFF_K = 0;                                // K operand, high part: fp16(d * x)
constexpr int OFF_KLO = OFF_K + NB * K_BYTES;           // K operand, low part: fp16(d * x - high part), exact
constexpr int OFF_V = OFF_KLO + (KLO ? NB * K_BYTES : 0);
constexpr int OFF_RAWK = OFF_V + NB * V_BYTES;
constexpr int OFF_RAWV = OFF_RAWK + NB * RAW_BYTES;
constexpr int OFF_BAR = OFF_RAWV + NB * RAW_BYTES;
enum { B_KRAW_FULL = 0, B_KRAW_FREE = 4, B_VRAW_FULL = 8, B_VRAW_FREE = 12, B_KF = 16, B_S = 20, B_P = 24, B_PV = 28,
       N_BARS = 32 };
constexpr int OFF_MISC = OFF_BAR + N_BARS * 8;          // [0] tmem base, [1] abort flag, [4..7] decision sequence
constexpr int OFF_MREF = OFF_MISC + 32;                 // [128] row references
constexpr int TOTAL = OFF_MREF + 128 * 4 + 1024;        // + slack to align the base to 1024
static_assert(TOTAL <= 226 * 1024, "shared memory budget");
static_assert(K_BYTES % 1024 == 0 && V_BYTES % 1024 == 0 && RAW_BYTES % 16 == 0, "operand alignment");

constexpr int T_O = 0;                                  // tensor-memory columns
constexpr int T_L = HD;                                 // 16 columns, each = sum of P
constexpr int T_S = HD + 32;                            // NB S/P buffers of BN columns
constexpr int T_Q = T_S + NB * BN;                      // HD/2 columns of fp16 pairs
static_assert(T_Q + HD / 2 <= TMEM_COLS, "tensor memory budget");

__global__ void __maxnreg__(REGS_LAUNCH) k_prefill_hd128(const Params P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);      // 1024-byte aligned
    uint8_t* Ksm = smem + OFF_K;
    uint8_t* Klo = smem + OFF_KLO;
    uint8_t* Vsm = smem + OFF_V;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem + OFF_MISC);
    volatile float* mref = reinterpret_cast<volatile float*>(smem + OFF_MREF);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = P.G, MR = 128 / G;                        // query positions per M tile
    const int n_mt = (P.rows + MR - 1) / MR;
    const int mt = n_mt - 1 - (int)blockIdx.x;              // longest key ranges first (bruce.cu:2770)
    const int kvh = blockIdx.y;
    const int p0 = P.pos[0];
    if (p0 < 0 || (!P.is_swa && p0 + P.rows > P.slot_ctx)) {
        if (tid == 0) atomicOr(P.status, BATTN_DEV_BAD_POSITION);
        return;
    }
    const int rbase = mt * MR;
    const int rows_eff = min(MR, P.rows - rbase);
    const int p_first = p0 + rbase, p_last = p_first + rows_eff - 1;
    const int lo_cta = P.is_swa ? max(0, p_first + 1 - P.W) : 0;       // bruce.cu:2801
    const int hi_cta = p_last + 1;
    const int full_lo = P.is_swa ? max(0, p_last + 1 - P.W) : 0;
    // key split: gridDim.z CTAs share this (M tile, kv head), each takes a contiguous share of the key tiles
    const int tile_lo = lo_cta / BN;
    const int n_all = (hi_cta + BN - 1) / BN - tile_lo;
    const int per_split = (n_all + P.nsplit - 1) / P.nsplit;
    const int tile_first = tile_lo + (int)blockIdx.z * per_split;
    const int n_tiles = max(0, min(per_split, n_all - (int)blockIdx.z * per_split));
    if (n_tiles == 0) {
        // more splits than key tiles (shallow context): an empty record, so the merge ignores this share
        if (tid < 128 && tid / G < rows_eff) {
            float* rec = P.recs + ((((size_t)blockIdx.z * P.rows) + rbase + tid / G) * P.Hq + kvh * G + tid % G) * (size_t)(HD + 2);
            for (int i = 0; i < HD; ++i) rec[i] = 0.f;
            rec[HD] = NEG_BIG; rec[HD + 1] = 0.f;
        }
        return;
    }

    // ---- set-up: barriers, tensor memory, the rows of ones, Q -----------------------------------------
    if (tid == 0) {
        for (int b = 0; b < NB; ++b) {
            mbar_init(&bars[B_KRAW_FULL + b], 1); mbar_init(&bars[B_VRAW_FULL + b], 1);
            mbar_init(&bars[B_KRAW_FREE + b], 4); mbar_init(&bars[B_VRAW_FREE + b], 4);
            mbar_init(&bars[B_KF + b], 4);
            mbar_init(&bars[B_S + b], 1); mbar_init(&bars[B_PV + b], 1);
            mbar_init(&bars[B_P + b], 8);                      // 4 softmax warps (P written) + 4 V dequant warps (operand ready)
        }
        misc[1] = 0;
        misc[4] = misc[5] = misc[6] = misc[7] = 0;
        mbar_fence_init();
    }
    if (tid < 128) mref[tid] = NEG_BIG;
    if (warp == W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(&misc[0]))), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // rows HD .. HD+15 of every V^T operand buffer: ones (the denominator columns of the P.V MMA)
    for (int idx = tid; idx < NB * 16 * 8; idx += NTHREADS) {
        const int b = idx / (16 * 8), rem = idx - b * (16 * 8);
        reinterpret_cast<uint4*>(Vsm + b * V_BYTES + HD * 128)[rem] =
            make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];
    // Q into tensor memory: lane = row m = (position m / G, head m % G) (the reference's pair packing,
    // bruce.cu:2288-2296), 32-bit column c = dims (2c, 2c+1); two threads per row
    if (tid < 256) {
        const int m = tid & 127, half = tid >> 7;
        const int r = m / G, h = m - r * G;
        uint32_t qv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) qv[i] = 0u;
        if (r < rows_eff) {
            const size_t qi = (((size_t)(rbase + r)) * P.Hq + kvh * G + h) * HD + half * 64;
            if (P.q_f16) {
                const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(P.q) + qi);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 w = src[i];
                    qv[4 * i] = w.x; qv[4 * i + 1] = w.y; qv[4 * i + 2] = w.z; qv[4 * i + 3] = w.w;
                }
            } else {
                const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.q) + qi);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float4 w = src[i];
                    qv[2 * i] = pack_h2(w.x, w.y); qv[2 * i + 1] = pack_h2(w.z, w.w);
                }
            }
        }
        tmem_st32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + T_Q + half * 32, qv);
        tmem_st_wait();
    }
    // Q only concerns its writers (the eight softmax warps) and its reader (the S issuer): the loaders, the dequant
    // warps and the P.V issuer go straight to work, so the first raw tiles and their conversion overlap the Q load
    if (warp < 8 || warp == W_MMA) {
        tc_fence_before();
        named_bar_sync(3, 9 * 32);
        tc_fence_after();
    }

    // bounded wait that degrades to "do not wait" once any wait has run out
    auto wait = [&](int b, uint32_t parity, uint32_t sleep_ns) {
        if (mbar_try_wait(&bars[b], parity)) return;               // the common case costs one poll
        if (misc[1]) return;
        if (!mbar_wait_backoff(&bars[b], parity, sleep_ns)) {
            atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
            misc[1] = 1;
        }
    };
    // ring slot and phase parity of tile j
    auto slot = [](int j) { return j % NB; };
    auto phase = [](int j) { return (uint32_t)((j / NB) & 1); };

    const size_t hb = (size_t)kvh * P.pstride * (size_t)REC;

    if (warp >= W_MMA) {
        regs_shrink<REGS_CTL>();                                   // the whole last warpgroup
        if (warp == W_MMA && lane == 0) {
            // ======================= S = Q K^T for every tile ===========================================
            // Runs ahead of the P.V issuer as far as the rings allow: S of tile j refills the buffer whose P
            // the P.V MMA of tile j-NB has consumed.
            const uint32_t idS = umma_idesc(128, BN);
            const uint64_t kd0 = umma_desc(smem_u32(Ksm)), kl0 = umma_desc(smem_u32(Klo));
            for (int j = 0; j < n_tiles; ++j) {
                wait(B_KF + slot(j), phase(j), 20);
                if (j >= NB) wait(B_PV + slot(j), phase(j - NB), 20);
                tc_fence_after();
                const uint32_t d = tmem + T_S + slot(j) * BN;
                const uint64_t kd = kd0 + (uint64_t)(slot(j) * (K_BYTES >> 4));
                const uint64_t kl = kl0 + (uint64_t)(slot(j) * (K_BYTES >> 4));
                // S = Q K_hi^T + Q K_lo^T: the two fp16 parts add up to the exact product d * x of every cached
                // value, so the scores carry no rounding of the K operand
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    umma_f16_ts(d, tmem + T_Q + 8 * ks, kd + (uint64_t)((ks >> 2) * ((BN * 128) >> 4) + 2 * (ks & 3)), idS, ks > 0);
#pragma unroll
                for (int ks = 0; KLO && ks < HD / 16; ++ks)
                    umma_f16_ts(d, tmem + T_Q + 8 * ks, kl + (uint64_t)((ks >> 2) * ((BN * 128) >> 4) + 2 * (ks & 3)), idS, 1u);
                umma_commit(&bars[B_S + slot(j)]);
            }
        } else if (warp == W_PV && lane == 0) {
            // ======================= O += P [V | 1] for every tile ======================================
            const uint32_t idO = umma_idesc(128, VROWS);
            const uint64_t vd0 = umma_desc(smem_u32(Vsm));
            for (int j = 0; j < n_tiles; ++j) {
                wait(B_P + slot(j), phase(j), 20);                         // P written and the V operand ready
                tc_fence_after();
                const uint32_t tP = tmem + T_S + slot(j) * BN;                // P overwrote the S tile
                const uint64_t vd = vd0 + (uint64_t)(slot(j) * (V_BYTES >> 4));
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)
                    umma_f16_ts(tmem + T_O, tP + 8 * ks, vd + (uint64_t)(2 * ks), idO, (j > 0 || ks > 0) ? 1u : 0u);
                umma_commit(&bars[B_PV + slot(j)]);
            }
        } else if ((warp == W_LDK || warp == W_LDV) && lane == 0) {
            // ======================= loaders: raw K (or V) tiles into their ring with bulk copies =======
            const bool isv = warp == W_LDV;
            const uint8_t* src = isv ? P.kvv : P.kvk;
            uint8_t* ring = smem + (isv ? OFF_RAWV : OFF_RAWK);
            const int full = isv ? B_VRAW_FULL : B_KRAW_FULL, free_ = isv ? B_VRAW_FREE : B_KRAW_FREE;
            for (int j = 0; j < n_tiles; ++j) {
                if (j >= NB) wait(free_ + slot(j), phase(j - NB), 200);         // the dequant group left it (no hurry: the ring is three deep)
                const int sp = ((tile_first + j) * BN) & P.ring_mask;
                const int nk = P.pg.table ? BN : min(BN, P.pstride - sp);
                const uint32_t bytes = (uint32_t)nk * REC;
                // (a paged look-up here is hidden by the ring: the loader runs three tiles ahead of the dequant warps)
                const size_t off = P.pg.table ? kv_rec_index(P.pg, P.slot, kvh, P.Hkv, P.pstride, sp, P.status) * (size_t)REC
                                              : hb + (size_t)sp * REC;
                mbar_expect_tx(&bars[full + slot(j)], bytes);
                bulk_g2s(ring + slot(j) * RAW_BYTES, src + off, bytes, &bars[full + slot(j)]);
            }
        }
    } else if (warp >= W_VDQ) {
        // ======================= V dequant warps: V^T operand, [dim][key] ================================
        regs_shrink<REGS_DEQ>();
        const int t = tid - W_VDQ * 32, wq = t >> 5;
        constexpr int NWG = HD / 16;                            // groups of four dim-words
        constexpr int UPT = (HD / 4) * (BN / 8) / 128;          // micro-tiles (4 dims x 8 keys) per thread
        const int cc = lane & 7, wl = lane >> 3;                // key chunk (8 keys), fixed per thread
        int vkey[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) vkey[jj] = kappa(8 * cc + jj);

        for (int j = 0; j < n_tiles; ++j) {
            const int t0 = (tile_first + j) * BN;
            const uint8_t* Vraw = smem + OFF_RAWV + slot(j) * RAW_BYTES;
            wait(B_VRAW_FULL + slot(j), phase(j), 50);
            // the P.V MMA that last read this V buffer (tile j - NB) must be complete
            if (j >= NB) wait(B_PV + slot(j), phase(j - NB), 50);
            uint8_t* Vdst = Vsm + slot(j) * V_BYTES;
            // keys outside [lo, hi) were never written for this chunk's rows: their bytes are arbitrary,
            // so their scale is forced to zero (their P is zero as well)
            bool kok[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) kok[jj] = (t0 + vkey[jj] >= lo_cta) && (t0 + vkey[jj] < hi_cta);
            uint32_t sp[4];
#pragma unroll
            for (int it = 0; it < UPT; ++it) {
                const int u = UPT * wq + it;
                const int w = 4 * (u % NWG) + wl;                       // dim word: dims 4w .. 4w+3
                if ((it & 1) == 0) {                                    // two consecutive micro-tiles share a block
                    const int vblk = (u % NWG) >> 1;
#pragma unroll
                    for (int pr = 0; pr < 4; ++pr) {
                        const uint32_t sa = kok[2 * pr] ? reinterpret_cast<const uint16_t*>(Vraw + vkey[2 * pr] * REC)[vblk] : 0u;
                        const uint32_t sb = kok[2 * pr + 1] ? reinterpret_cast<const uint16_t*>(Vraw + vkey[2 * pr + 1] * REC)[vblk] : 0u;
                        sp[pr] = sa | (sb << 16);
                    }
                }
                uint32_t x[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj)
                    x[jj] = *reinterpret_cast<const uint32_t*>(Vraw + vkey[jj] * REC + 2 * NBLK + 4 * w) ^ 0x80808080u;
                uint32_t chunk[4][4];
#pragma unroll
                for (int pr = 0; pr < 4; ++pr) {
                    const uint32_t lo = __byte_perm(x[2 * pr], x[2 * pr + 1], 0x5140);
                    const uint32_t hi = __byte_perm(x[2 * pr], x[2 * pr + 1], 0x7362);
                    chunk[0][pr] = hmul2_u32(sub1152(widen_lo(lo)), sp[pr]);
                    chunk[1][pr] = hmul2_u32(sub1152(widen_hi(lo)), sp[pr]);
                    chunk[2][pr] = hmul2_u32(sub1152(widen_lo(hi)), sp[pr]);
                    chunk[3][pr] = hmul2_u32(sub1152(widen_hi(hi)), sp[pr]);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int d = 4 * w + i;
                    *reinterpret_cast<uint4*>(Vdst + sw128(d, cc)) = make_uint4(chunk[i][0], chunk[i][1], chunk[i][2], chunk[i][3]);
                }
            }
            proxy_fence();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&bars[B_P + slot(j)]); mbar_arrive(&bars[B_VRAW_FREE + slot(j)]); }
        }
    } else if (warp >= W_KDQ) {
        // ======================= K dequant warps: K operand, [key][dim] ==================================
        regs_shrink<REGS_DEQ>();
        const int t = tid - W_KDQ * 32;
        const int krow = t & (BN - 1);                          // each thread converts one 64-dim half of one row
        const int sub = t / BN;                                 // which 64-dim sub-tile
        const int kkey = kappa(krow);
        for (int j = 0; j < n_tiles; ++j) {
            const uint8_t* src = smem + OFF_RAWK + slot(j) * RAW_BYTES + kkey * REC;
            wait(B_KRAW_FULL + slot(j), phase(j), 50);
            // the S MMA that last read this K buffer (tile j - NB) must be complete
            if (j >= NB) wait(B_S + slot(j), phase(j - NB), 50);
            uint8_t* Kdst = Ksm + slot(j) * K_BYTES + sub * (BN * 128);
            uint8_t* Ldst = Klo + slot(j) * K_BYTES + sub * (BN * 128);
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                const __half sc = reinterpret_cast<const __half*>(src)[2 * sub + blk];
                const __half2 s2 = __half2half2(sc);
                const uint32_t su = *reinterpret_cast<const uint32_t*>(&s2);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int ch = 4 * blk + c;                 // 16-byte chunk inside the sub-tile row
                    const uint2 w = *reinterpret_cast<const uint2*>(src + 2 * NBLK + (8 * sub + ch) * 8);
                    const uint32_t x = w.x ^ 0x80808080u, y = w.y ^ 0x80808080u;
                    const uint32_t i0 = sub1152(widen_lo(x)), i1 = sub1152(widen_hi(x));
                    const uint32_t i2 = sub1152(widen_lo(y)), i3 = sub1152(widen_hi(y));
                    uint4 o, r;
                    o.x = hmul2_u32(i0, su); r.x = hfma2_residual(i0, su, o.x);
                    o.y = hmul2_u32(i1, su); r.y = hfma2_residual(i1, su, o.y);
                    o.z = hmul2_u32(i2, su); r.z = hfma2_residual(i2, su, o.z);
                    o.w = hmul2_u32(i3, su); r.w = hfma2_residual(i3, su, o.w);
                    *reinterpret_cast<uint4*>(Kdst + sw128(krow, ch)) = o;
                    if (KLO) *reinterpret_cast<uint4*>(Ldst + sw128(krow, ch)) = r;
                }
            }
            proxy_fence();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&bars[B_KF + slot(j)]); mbar_arrive(&bars[B_KRAW_FREE + slot(j)]); }
        }
    } else {
        // ======================= softmax warps: one thread per accumulator row, groups alternate tiles ====
        regs_grow<REGS_SOFT>();
        const int m = tid & 127;                               // row = TMEM lane
        const int grp = tid >> 7;                              // 0: even tiles, 1: odd tiles
        const int qtr = warp & 3;
        const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
        const int r = m / G, h = m - r * G;
        const bool row_ok = r < rows_eff;
        const int prow = p_first + r;
        const int row_lo = P.is_swa ? max(0, prow + 1 - P.W) : 0;     // bruce.cu:3014
        const float c2 = P.scale_log2;
        const float thr = RESCALE_THRESHOLD / c2;              // threshold in raw-score units
        const uint64_t c2p = pack_f2(c2, c2);

        for (int j = grp; j < n_tiles; j += 2) {
            const int t0 = (tile_first + j) * BN;
            const uint32_t tS = tmem + lane_base + T_S + slot(j) * BN;
            // tiles every row of the CTA sees completely skip the mask code (bruce.cu:2927-2928)
            // (rows past the end of a ragged M tile hold zero queries: whatever they compute is finite and never stored)
            const bool masked = !(t0 >= full_lo && t0 + BN - 1 <= p_first);
            wait(B_S + slot(j), phase(j), 50);
            tc_fence_after();
            uint32_t v[2][32];
            tmem_ld32_nowait(tS, v[0]);
            tmem_ld32_nowait(tS + 32, v[1]);
            tmem_ld_wait();
            if (masked) {
                // Tiles that some row of the CTA sees only partly (the causal diagonal, the window edge, a
                // ragged last chunk): hidden columns are replaced by "minus infinity" (bruce.cu:3021-3028),
                // after which the common code below needs no mask.  The visibility bits are built by a rolled
                // loop to keep this rarely executed path small.
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t bits = 0u;
#pragma unroll 1
                    for (int i = 0; i < 32; ++i) {
                        const int key = t0 + kappa(c * 32 + i);
                        const bool ok = row_ok && key <= prow && key >= row_lo;
                        bits |= (ok ? 1u : 0u) << i;
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (!((bits >> i) & 1u)) v[c][i] = __float_as_uint(NEG_BIG);
                }
            }
            float mx;
            {
                float m0 = __uint_as_float(v[0][0]), m1 = __uint_as_float(v[0][1]);
                float m2 = __uint_as_float(v[0][2]), m3 = __uint_as_float(v[0][3]);
#pragma unroll
                for (int i = 4; i + 8 <= 32; i += 8) {
                    m0 = fmax3(m0, __uint_as_float(v[0][i]), __uint_as_float(v[0][i + 1]));
                    m1 = fmax3(m1, __uint_as_float(v[0][i + 2]), __uint_as_float(v[0][i + 3]));
                    m2 = fmax3(m2, __uint_as_float(v[0][i + 4]), __uint_as_float(v[0][i + 5]));
                    m3 = fmax3(m3, __uint_as_float(v[0][i + 6]), __uint_as_float(v[0][i + 7]));
                }
                m0 = fmax3(m0, __uint_as_float(v[0][28]), __uint_as_float(v[0][29]));
                m1 = fmax3(m1, __uint_as_float(v[0][30]), __uint_as_float(v[0][31]));
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    m0 = fmax3(m0, __uint_as_float(v[1][i]), __uint_as_float(v[1][i + 1]));
                    m1 = fmax3(m1, __uint_as_float(v[1][i + 2]), __uint_as_float(v[1][i + 3]));
                    m2 = fmax3(m2, __uint_as_float(v[1][i + 4]), __uint_as_float(v[1][i + 5]));
                    m3 = fmax3(m3, __uint_as_float(v[1][i + 6]), __uint_as_float(v[1][i + 7]));
                }
                mx = fmax3(fmaxf(m0, m1), m2, m3);
            }
            // The row reference is decided in tile order: wait until the other group has published its decision
            // for tile j-1 (normally long done: that group started half a tile earlier).
            if (j > 0 && !misc[1]) {
                uint32_t spins = 0;
                while (misc[4 + qtr] < (uint32_t)j) {
                    if (++spins > (1u << 24)) {
                        atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
                        misc[1] = 1;
                        break;
                    }
                }
                __threadfence_block();
            }
            float m_ref = mref[m];
            const float m_new = fmaxf(m_ref, mx);
            const bool need = m_new > m_ref + thr;
            if (__any_sync(0xffffffffu, need)) {
                if (j > 0) {
                    wait(B_PV + slot(j - 1), phase(j - 1), 50);         // O must be complete before it is rescaled
                    tc_fence_after();
                    const float alpha = need ? fast_exp2((m_ref - m_new) * c2) : 1.f;
#pragma unroll 1
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t o[32];
                        const uint32_t ta = tmem + lane_base + T_O + c * 32;
                        tmem_ld32(ta, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(ta, o);
                    }
                    const uint32_t tl = tmem + lane_base + T_L;
                    tmem_st1(tl, __float_as_uint(__uint_as_float(tmem_ld1(tl)) * alpha));
                    tmem_st_wait();
                    tc_fence_before();
                }
                if (need) { m_ref = m_new; mref[m] = m_new; }
            }
            __syncwarp();
            if (lane == 0) {
                __threadfence_block();
                misc[4 + qtr] = (uint32_t)(j + 1);
            }
            // p = 2^(s*c2 - m_ref*c2); a row that has seen no key yet keeps the offset at zero, so its hidden
            // columns ("minus infinity") still come out as exactly zero
            const float nb = m_ref > 0.5f * NEG_BIG ? -m_ref * c2 : 0.f;
            const uint64_t nbp = pack_f2(nb, nb);
            // P (fp16 pairs) overwrites the first half of the S columns, which this thread has already read
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float e0, e1;
                    ffma2(e0, e1, __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]), c2p, nbp);
                    pk[c * 16 + (i >> 1)] = pack_h2(fast_exp2(e0), fast_exp2(e1));
                }
            }
            tmem_st32(tS, pk);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[B_P + slot(j)]);
        }
        // ---- epilogue: O / sum(P) -> global; each of the two threads of a row writes half of it ----------
        // A parity wait on phase k of a barrier is only meaningful once phase k-1 is known to be complete (before
        // that it is satisfied at once).  The group that did not own the last tile therefore first waits for the
        // P.V product of its OWN last tile -- whose predecessor in that ring slot completed before this group was
        // handed the tile's scores -- and only then for the last tile's.
        {
            const int own_last = n_tiles - 1 - ((n_tiles - 1 - grp) & 1);
            if (own_last >= 0 && own_last != n_tiles - 1) wait(B_PV + slot(own_last), phase(own_last), 50);
        }
        wait(B_PV + slot(n_tiles - 1), phase(n_tiles - 1), 50);
        tc_fence_after();
        const float l = __uint_as_float(tmem_ld1(tmem + lane_base + T_L));
        const float il = l > 0.f ? 1.f / l : 0.f;
        const size_t oi = (((size_t)(rbase + r)) * P.Hq + kvh * G + h) * HD + grp * (HD / 2);
        // with key splits: a split record (unnormalised o, m in log2 units, l) instead of the output row
        float* rec = P.recs ? P.recs + ((((size_t)blockIdx.z * P.rows) + rbase + r) * P.Hq + kvh * G + h) * (size_t)(HD + 2)
                                  : nullptr;
        if (rec && row_ok && grp == 0) {
            const float mr = mref[m];
            rec[HD] = mr > 0.5f * NEG_BIG ? mr * c2 : NEG_BIG;
            rec[HD + 1] = l;
        }
#pragma unroll 1
        for (int c = 0; c < HD / 64; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem + lane_base + T_O + grp * (HD / 2) + c * 32, o);
            if (row_ok) {
                if (rec) {
                    float2* dst = reinterpret_cast<float2*>(rec + grp * (HD / 2) + c * 32);     // records are 8-byte aligned
#pragma unroll
                    for (int q2 = 0; q2 < 16; ++q2)
                        dst[q2] = make_float2(__uint_as_float(o[2 * q2]), __uint_as_float(o[2 * q2 + 1]));
                } else if (P.out_f16) {
                    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(P.out) + oi + c * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            w[e] = pack_h2(__uint_as_float(o[q4 * 8 + 2 * e]) * il, __uint_as_float(o[q4 * 8 + 2 * e + 1]) * il);
                        dst[q4] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                } else {
                    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(P.out) + oi + c * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4)
                        dst[q4] = make_float4(__uint_as_float(o[4 * q4]) * il, __uint_as_float(o[4 * q4 + 1]) * il,
                                              __uint_as_float(o[4 * q4 + 2]) * il, __uint_as_float(o[4 * q4 + 3]) * il);
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == W_MMA) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace pf128
}  // namespace battn
