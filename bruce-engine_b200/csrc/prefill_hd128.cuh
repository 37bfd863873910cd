// Prompt-chunk attention for head_dim 128 on the 5th-generation tensor cores: causal + sliding-window
// flash attention of a chunk of query rows against the growing q8_0 cache (the chunk's own keys were
// appended first).
//
// Behaviour replaced: k_attn_tc_rs_opt<NW,...> for rows > 8 and its dispatch
// (engine/src/bruce.cu:2750-3131, 4021-4078); masks as bruce.cu:2799-2805, 3012-3029.
//
// One CTA per (128-row M tile, kv head); the keys stream through in tiles of 64.  Chunks of more than one M tile
// run as clusters of two CTAs (template parameter PAIR): 256 rows per pair with tcgen05.mma.cta_group::2, issued
// by the first CTA of the cluster.  Every CTA keeps its own 128 rows of Q, S, P and O in its tensor memory, but
// the B operands are split between the two: a CTA converts and holds only 32 of a tile's 64 keys of the K operand
// and 64 of the 128 head dimensions (plus a block of ones) of the V^T operand, so the int8 -> fp16 conversion per
// attended row is halved; "my share is ready" is a plain remote mbarrier arrive on the issuing CTA's barrier (a
// cluster-scope release there stalled every dequant warp on a memory barrier and cost 20 %), completion comes back
// through tcgen05.commit with a two-CTA multicast.  In that mode the S products are issued for two key tiles at a
// time (N = 128): a 64-column product runs at about half the tensor rate.
// Twenty warps, each warpgroup resized with setmaxnreg for its role:
//   warps 0-7   softmax: two threads per accumulator row, warps 0-3 own the first 32 columns of every key tile,
//               warps 4-7 the other 32
//   warps 8-11  K dequant: raw q8_0 records -> fp16 K operand [key][dim], scale folded in
//   warps 12-15 V dequant: raw q8_0 records -> fp16 V^T operand [dim][key], scale folded in
//   warp 16     issues the S MMAs, warp 19 the P.V MMAs;  warps 17/18 stream raw K / V tiles with bulk copies
// Data flow per key tile j (every ring below is three deep -- four in a pair -- and indexed j mod the depth):
//   loader -> raw K/V tile (shared memory) -> dequant -> fp16 operand (128-byte-swizzled shared memory)
//   K operand         two fp16 parts per value: hi = fp16(d*x) and lo = d*x - hi (exact: the product of an int8
//                     and an fp16 scale has 19 significant bits, fp16 keeps 11, the rest fits the second part),
//                     so S carries no rounding of K -- a single folded operand alone moves single (row, head)
//                     outputs by up to 7e-4 relative, most of the 1e-3 budget
//   S_j = Q K_hi^T + Q K_lo^T   Q lives in tensor memory (the A operand), S_j in a 64-column buffer of the ring
//   softmax           each of a row's two threads reads its 32 scores once into registers; the row maximum is
//                     exchanged through shared memory (one 64-thread named barrier per tile); both write
//                     P_j = 2^(S_j*c - ref) as fp16 pairs over the first 32 columns of the same buffer
//   O += P_j [V_j | 1]  P_j is the tensor-memory A operand; sixteen rows of ones appended to the V^T
//                     operand make the same MMA accumulate sum(P) in fp32 next to O, from exactly the
//                     fp16-rounded P it multiplies with V
// The S issuer runs ahead of O as far as the ring of S/P buffers allows; a buffer is free again when the P.V
// product that read its P has completed, and that turn-around (S product -> softmax -> P.V product) is what
// bounds the kernel.
// The row reference `ref` (a lazily updated running maximum, bruce.cu:3034-3060 in spirit) is kept in a register
// by both threads of a row -- they see the same maxima and take the same decisions -- and O is rescaled in tensor
// memory only when a row maximum grows by more than 2^8 over the reference; the final normalisation uses the same
// reference, so the result does not depend on how rarely it moves.
// Row n of the K operand / column n of S holds key kappa(n), a fixed permutation inside each 64-key span
// chosen so that every shared-memory access of the dequant warps is bank-conflict free.
// Every wait is bounded; a wait that runs out sets the device status word, the remaining waits are
// skipped, tensor memory is released and the kernel returns.
#pragma once
#include "prefill.cuh"

namespace battn {
namespace pf128 {

using namespace pf;

constexpr int HD = 128, BN = 64;
constexpr int NBLK = HD / 32, REC = HD + 2 * NBLK;
constexpr int NTHREADS = 640;
constexpr int W_KDQ = 8, W_VDQ = 12, W_MMA = 16, W_LDK = 17, W_LDV = 18, W_PV = 19;
constexpr int REGS_LAUNCH = 96, REGS_SOFT = 144, REGS_DEQ = 72, REGS_CTL = 40;
static_assert(2 * REGS_SOFT + 2 * REGS_DEQ + REGS_CTL <= 5 * REGS_LAUNCH, "register budget per scheduler");

constexpr int RAW_BYTES = BN * REC;
enum { B_KRAW_FULL = 0, B_KRAW_FREE = 4, B_VRAW_FULL = 8, B_VRAW_FREE = 12, B_KF = 16, B_S = 20, B_P = 24, B_PV = 28,
       B_Q = 32, N_BARS = 33 };

// Shared- and tensor-memory layout.  PAIR = false: one CTA per 128-row M tile.  PAIR = true: two CTAs of a cluster
// work on 256 rows with tcgen05.mma.cta_group::2 -- every CTA keeps its own 128 rows of Q, S, P and O, but the B
// operands are split between them: each CTA converts and holds only 32 of a tile's 64 keys of the K operand and
// 64 of the 128 head dimensions (plus its own block of ones) of the V^T operand, so the conversion work per
// attended row is halved.
template <bool PAIR>
struct Lay {
    // depth of every ring (raw tiles, operands, S/P); PAIR: four, because the S products are issued for two tiles at
    // a time (N = 128: a 64-column S product runs at about half the tensor rate, measured) and the two tiles'
    // K operands and S buffers are neighbours in their rings
    static constexpr int NB = PAIR ? 4 : 3;
    static constexpr bool S2 = PAIR;
    static constexpr int KROWS = PAIR ? BN / 2 : BN;        // K operand rows (keys) this CTA holds per tile
    static constexpr int K_SUB = KROWS * 128;                // one 64-dim sub-tile [KROWS][128 B]
    static constexpr int K_BYTES = 2 * K_SUB;
    static constexpr int VDIMS = PAIR ? HD / 2 : HD;         // head dimensions of the V^T operand this CTA holds
    static constexpr int VROWS = VDIMS + 16;                 // + the block of ones
    static constexpr int V_BYTES = VROWS * 128;              // [VROWS][64 keys] fp16
    static constexpr int N_PV = PAIR ? 2 * VROWS : VROWS;    // N of the P.V product: 160 or 144
    static constexpr int OFF_K = 0;                          // K operand, high part: fp16(d * x)
    static constexpr int OFF_KLO = OFF_K + NB * K_BYTES;     // K operand, low part: fp16(d * x - high part), exact
    static constexpr int OFF_V = OFF_KLO + NB * K_BYTES;
    static constexpr int OFF_RAWK = OFF_V + NB * V_BYTES;
    static constexpr int OFF_RAWV = OFF_RAWK + NB * RAW_BYTES;
    static constexpr int OFF_BAR = OFF_RAWV + NB * RAW_BYTES;
    static constexpr int OFF_MISC = OFF_BAR + N_BARS * 8 + 8;   // [0] tmem base, [1] abort flag
    static constexpr int OFF_MREF = OFF_MISC + 32;           // [tile parity][column half][128 rows] row maxima
    static constexpr int TOTAL = OFF_MREF + 2 * 2 * 128 * 4 + 1024;  // + slack to align the base to 1024
    static_assert(TOTAL <= 226 * 1024, "shared memory budget");
    static_assert(K_SUB % 1024 == 0 && V_BYTES % 1024 == 0 && RAW_BYTES % 16 == 0, "operand alignment");
    // tensor-memory columns.  PAIR: the P.V product has N = 160 = [dims 0-63 | ones | dims 64-127 | ones], so the
    // two halves of O sit at columns 0 and 80 and the denominator at column 64.
    static constexpr int T_O = 0;
    static constexpr int T_OHI = PAIR ? VROWS : HD / 2;      // column of dims 64..127
    static constexpr int T_L = PAIR ? HD / 2 : HD;           // 16 columns, each = sum of P
    static constexpr int T_S = HD + 32;                      // NB S/P buffers of BN columns
    static constexpr int T_Q = T_S + NB * BN;                // HD/2 columns of fp16 pairs
    static_assert(N_PV <= T_S && T_Q + HD / 2 <= TMEM_COLS, "tensor memory budget");
    __device__ static constexpr int ocol(int c) { return c < 2 ? c * 32 : T_OHI + (c - 2) * 32; }   // 32-column chunk c of O
    // byte offset of sub-tile `sub` of the K operand in ring slot `sl`.  S2: slots 2p and 2p+1 interleave, so that
    // the rows of both tiles are consecutive 8-row groups of one operand with N = 128.
    __device__ static constexpr int koff(int sl, int sub) {
        return S2 ? (sl >> 1) * (2 * K_BYTES) + sub * (2 * K_SUB) + (sl & 1) * K_SUB : sl * K_BYTES + sub * K_SUB;
    }
    // S2, cta_group::2: columns of the pair's 128-column S product are [tile 2p keys 0-31 | tile 2p+1 keys 0-31 |
    // tile 2p keys 32-63 | tile 2p+1 keys 32-63] (each CTA supplies its rows of both tiles); a last tile without a
    // partner is an ordinary 64-column product in the first half.  First 32-column chunk of the tile in slot sl, and
    // distance to its second chunk:
    __device__ static constexpr int scol(int sl) { return S2 ? (sl >> 1) * (2 * BN) + (sl & 1) * 32 : sl * BN; }
    __device__ static constexpr int schunk(bool paired) { return S2 && paired ? 64 : 32; }
};
constexpr int TOTAL = Lay<false>::TOTAL, TOTAL_PAIR = Lay<true>::TOTAL;

// ---- cluster helpers (PAIR) -------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t cta) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(bar)), "r"(cta));
#ifdef BATTN_PF_ARRIVE_CLUSTER_RELEASE
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(ra) : "memory");
#else
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(ra) : "memory");
#endif
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// the two-CTA forms of the MMA (A in tensor memory) and of its completion signal, which arrives on the barrier at
// the same offset in both CTAs of the pair
__device__ __forceinline__ void umma2_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void umma2_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}

template <bool PAIR>
__global__ void __maxnreg__(REGS_LAUNCH) k_prefill_hd128(const Params P) {
    using L = Lay<PAIR>;
    constexpr int NB = L::NB;
    constexpr int OFF_K = L::OFF_K, OFF_KLO = L::OFF_KLO, OFF_V = L::OFF_V, OFF_RAWK = L::OFF_RAWK, OFF_RAWV = L::OFF_RAWV;
    constexpr int OFF_BAR = L::OFF_BAR, OFF_MISC = L::OFF_MISC, OFF_MREF = L::OFF_MREF;
    constexpr int K_SUB = L::K_SUB, V_BYTES = L::V_BYTES, VDIMS = L::VDIMS;
    constexpr int T_O = L::T_O, T_L = L::T_L, T_S = L::T_S, T_Q = L::T_Q;
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
    // PAIR: CTA 0 of a cluster (the one that issues the MMAs) takes the later M tile of its pair, CTA 1 the one
    // before it; with an odd number of M tiles the last pair's second CTA has no rows of its own (mt = -1) and
    // only contributes its halves of the operands.
    const int crank = PAIR ? (int)cluster_rank() : 0;
    const bool leader = crank == 0;
    const int mt_pair = n_mt - 1 - (PAIR ? (int)blockIdx.x & ~1 : (int)blockIdx.x);    // longest key ranges first (bruce.cu:2770)
    const int mt = mt_pair - crank;
    const int kvh = blockIdx.y;
    const bool early = P.early != 0;
    if (!early) { pdl_wait(); pdl_trigger(); }
    const int p0 = P.pos[0];
    if (p0 < 0 || (!P.is_swa && p0 + P.rows > P.slot_ctx)) {
        if (tid == 0) atomicOr(P.status, BATTN_DEV_BAD_POSITION);
        return;
    }
    const int rbase = max(mt, 0) * MR;
    const int rows_eff = mt < 0 ? 0 : min(MR, P.rows - rbase);
    const int p_first = p0 + rbase, p_last = p_first + rows_eff - 1;
    const int full_lo = P.is_swa ? max(0, p_last + 1 - P.W) : 0;
    // key range of the CTA, or of the pair (both CTAs walk the same tiles)
    const int rbase_lo = PAIR ? max(mt_pair - 1, 0) * MR : rbase;
    const int lo_cta = P.is_swa ? max(0, p0 + rbase_lo + 1 - P.W) : 0;       // bruce.cu:2801
    const int hi_cta = p0 + min(P.rows, (mt_pair + 1) * MR);
    // key split: gridDim.z CTAs share this (M tile, kv head), each takes a contiguous share of the key tiles
    const int tile_lo = lo_cta / BN;
    const int n_all = (hi_cta + BN - 1) / BN - tile_lo;
    const int per_split = (n_all + P.nsplit - 1) / P.nsplit;
    const int tile_first = tile_lo + (int)blockIdx.z * per_split;
    const int n_tiles = max(0, min(per_split, n_all - (int)blockIdx.z * per_split));
    if (n_tiles == 0) {
        // more splits than key tiles (shallow context): an empty record, so the merge ignores this share
        if (early) pdl_wait();
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
            mbar_init(&bars[B_S + b], 1); mbar_init(&bars[B_PV + b], 1);
            // K operand ready: 4 dequant warps; P written and V operand ready: 8 softmax + 4 dequant warps --
            // PAIR: of both CTAs, counted on the issuing CTA's barriers
            mbar_init(&bars[B_KF + b], PAIR ? 8 : 4);
            mbar_init(&bars[B_P + b], PAIR ? 24 : 12);
        }
        mbar_init(&bars[B_Q], 1);
        misc[1] = 0;
        mbar_fence_init();
    }
    if (warp == W_MMA) {
        if (PAIR) {
            // the same warp of both CTAs of the pair allocates the same columns in both tensor memories
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(const_cast<uint32_t*>(&misc[0]))), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(const_cast<uint32_t*>(&misc[0]))), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    // the last sixteen rows of every V^T operand buffer: ones (the denominator columns of the P.V MMA)
    for (int idx = tid; idx < NB * 16 * 8; idx += NTHREADS) {
        const int b = idx / (16 * 8), rem = idx - b * (16 * 8);
        reinterpret_cast<uint4*>(Vsm + b * V_BYTES + VDIMS * 128)[rem] =
            make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();          // both CTAs' barriers are initialised before either arrives on the other's
    tc_fence_after();
    const uint32_t tmem = misc[0];
    // Q into tensor memory: lane = row m = (position m / G, head m % G) (the reference's pair packing,
    // bruce.cu:2288-2296), 32-bit column c = dims (2c, 2c+1); two threads per row
    if (tid < 256) {
        if (early) { pdl_wait(); pdl_trigger(); }              // Q is the predecessor's output; so is everything these warps write
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
        // PAIR: the issuing CTA's S MMA reads Q from both tensor memories
        if (PAIR && !leader && warp == W_MMA && lane == 0) mbar_arrive_remote(&bars[B_Q], 0);
    }

    // bounded wait that degrades to "do not wait" once any wait has run out
    auto wait = [&](int b, uint32_t parity, uint32_t sleep_ns) {
        if (mbar_try_wait(&bars[b], parity)) return;               // the common case costs one poll
        if (misc[1]) return;
#ifdef BATTN_PF_SLEEP_DIV
        sleep_ns = sleep_ns / BATTN_PF_SLEEP_DIV;
#endif
        if (!mbar_wait_backoff(&bars[b], parity, sleep_ns)) {
            atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
            misc[1] = 1;
        }
    };
    // the same for a barrier the other CTA of the pair arrives on (acquire at cluster scope)
    auto wait_pair = [&](int b, uint32_t parity, uint32_t sleep_ns) {
#ifndef BATTN_PF_WAIT_CLUSTER_ACQUIRE
        wait(b, parity, sleep_ns);
        return;
#endif
        if (!PAIR) { wait(b, parity, sleep_ns); return; }
        if (misc[1]) return;
        for (uint32_t i = 0; i < (1u << 22); ++i) {
            if (mbar_try_wait_cluster(&bars[b], parity)) return;
            __nanosleep(sleep_ns);
        }
        atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
        misc[1] = 1;
    };
    // "this CTA's share of tile j is ready": on the own barrier, or on the issuing CTA's
    auto arrive_issuer = [&](int b) {
        if (PAIR) mbar_arrive_remote(&bars[b], 0); else mbar_arrive(&bars[b]);
    };
    // ring slot and phase parity of tile j
    auto slot = [](int j) { return j % NB; };
    auto phase = [](int j) { return (uint32_t)((j / NB) & 1); };

    const size_t hb = (size_t)kvh * P.pstride * (size_t)REC;

    if (warp >= W_MMA) {
        regs_shrink<REGS_CTL>();                                   // the whole last warpgroup
        if (warp == W_MMA && lane == 0 && leader) {
            // ======================= S = Q K^T for every tile ===========================================
            // Runs ahead of the P.V issuer as far as the rings allow: S of tile j refills the buffer whose P
            // the P.V MMA of tile j-NB has consumed.
            const uint32_t idS = umma_idesc(PAIR ? 256 : 128, BN);
            const uint64_t kd0 = umma_desc(smem_u32(Ksm)), kl0 = umma_desc(smem_u32(Klo));
            if (PAIR) wait_pair(B_Q, 0, 20);                               // the other CTA's Q is in its tensor memory
            const int step = L::S2 ? 2 : 1;
            for (int j = 0; j < n_tiles; j += step) {
                const bool two = L::S2 && j + 1 < n_tiles;                 // tiles j and j+1 in one product
                const int jl = two ? j + 1 : j;
                wait_pair(B_KF + slot(j), phase(j), 20);
                if (two) wait_pair(B_KF + slot(jl), phase(jl), 20);
                // the S buffers are free once the P.V products that read them are complete (products complete in
                // order).  S2: always both buffers of the ring pair -- a last tile without a partner is a 64-column
                // product that spills over the partner buffer's first chunk.
                const int jw = L::S2 ? j + 1 : j;
                if (jw >= NB) wait(B_PV + slot(jw), phase(jw - NB), 20);
                tc_fence_after();
                const uint32_t d = tmem + T_S + L::scol(slot(j));
                const uint32_t id = two ? umma_idesc(256, 2 * BN) : idS;
                const uint32_t sub_step = (uint32_t)((L::S2 ? 2 * K_SUB : K_SUB) >> 4);
                const uint64_t kd = kd0 + (uint64_t)(L::koff(slot(j), 0) >> 4);
                const uint64_t kl = kl0 + (uint64_t)(L::koff(slot(j), 0) >> 4);
                // S = Q K_hi^T + Q K_lo^T: the two fp16 parts add up to the exact product d * x of every cached
                // value, so the scores carry no rounding of the K operand
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint64_t off = (uint64_t)((ks >> 2) * sub_step + 2 * (ks & 3));
                    if (PAIR) umma2_f16_ts(d, tmem + T_Q + 8 * ks, kd + off, id, ks > 0);
                    else      umma_f16_ts(d, tmem + T_Q + 8 * ks, kd + off, id, ks > 0);
                }
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint64_t off = (uint64_t)((ks >> 2) * sub_step + 2 * (ks & 3));
                    if (PAIR) umma2_f16_ts(d, tmem + T_Q + 8 * ks, kl + off, id, 1u);
                    else      umma_f16_ts(d, tmem + T_Q + 8 * ks, kl + off, id, 1u);
                }
                if (PAIR) {
                    umma2_commit(&bars[B_S + slot(j)]);
                    if (two) umma2_commit(&bars[B_S + slot(jl)]);
                } else {
                    umma_commit(&bars[B_S + slot(j)]);
                }
            }
        } else if (warp == W_PV && lane == 0 && leader) {
            // ======================= O += P [V | 1] for every tile ======================================
            const uint32_t idO = umma_idesc(PAIR ? 256 : 128, L::N_PV);
            const uint64_t vd0 = umma_desc(smem_u32(Vsm));
            for (int j = 0; j < n_tiles; ++j) {
                wait_pair(B_P + slot(j), phase(j), 20);                    // P written and the V operand ready
                tc_fence_after();
                const uint32_t tP = tmem + T_S + L::scol(slot(j));            // P overwrote the first chunk of the S tile
                const uint64_t vd = vd0 + (uint64_t)(slot(j) * (V_BYTES >> 4));
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    if (PAIR) umma2_f16_ts(tmem + T_O, tP + 8 * ks, vd + (uint64_t)(2 * ks), idO, (j > 0 || ks > 0) ? 1u : 0u);
                    else      umma_f16_ts(tmem + T_O, tP + 8 * ks, vd + (uint64_t)(2 * ks), idO, (j > 0 || ks > 0) ? 1u : 0u);
                }
                if (PAIR) umma2_commit(&bars[B_PV + slot(j)]); else umma_commit(&bars[B_PV + slot(j)]);
            }
        } else if ((warp == W_LDK || warp == W_LDV) && lane == 0) {
            // ======================= loaders: raw K (or V) tiles into their ring with bulk copies =======
            const bool isv = warp == W_LDV;
            const uint8_t* src = isv ? P.kvv : P.kvk;
            uint8_t* ring = smem + (isv ? OFF_RAWV : OFF_RAWK);
            const int full = isv ? B_VRAW_FULL : B_KRAW_FULL, free_ = isv ? B_VRAW_FREE : B_KRAW_FREE;
            bool waited = !early;
            for (int j = 0; j < n_tiles; ++j) {
                // early streaming stops at the first tile that holds a row of this chunk
                if (!waited && (tile_first + j + 1) * BN > p0) { pdl_wait(); pdl_trigger(); waited = true; }
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
        constexpr int NWG = VDIMS / 16;                         // groups of four dim-words this CTA converts
        constexpr int UPT = (VDIMS / 4) * (BN / 8) / 128;       // micro-tiles (4 dims x 8 keys) per thread: 2, PAIR: 1
        const int wfirst = PAIR ? crank * (VDIMS / 4) : 0;      // first dim word of this CTA's half of the head
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
                const int wloc = 4 * (u % NWG) + wl;                    // dim word inside this CTA's operand
                const int w = wfirst + wloc;                            // dim word of the head: dims 4w .. 4w+3
                if (UPT == 1 || (it & 1) == 0) {                        // two consecutive micro-tiles share a block
                    const int vblk = w >> 3;
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
                    const int d = 4 * wloc + i;                         // operand row
                    *reinterpret_cast<uint4*>(Vdst + sw128(d, cc)) = make_uint4(chunk[i][0], chunk[i][1], chunk[i][2], chunk[i][3]);
                }
            }
            proxy_fence();
            __syncwarp();
            if (lane == 0) { arrive_issuer(B_P + slot(j)); mbar_arrive(&bars[B_VRAW_FREE + slot(j)]); }
        }
    } else if (warp >= W_KDQ) {
        // ======================= K dequant warps: K operand, [key][dim] ==================================
        regs_shrink<REGS_DEQ>();
        const int t = tid - W_KDQ * 32;
        // a thread converts NBT 32-dim blocks of one operand row: a 64-dim half of one of 64 rows, or (PAIR) one
        // block of one of this CTA's 32 rows
        constexpr int KROWS = L::KROWS, NBT = PAIR ? 1 : 2;
        const int krow = t & (KROWS - 1);
        const int part = t / KROWS;                             // 0..1, PAIR: 0..3
        const int sub = PAIR ? part >> 1 : part;                // which 64-dim sub-tile
        const int blk0 = PAIR ? part & 1 : 0;                   // first block inside the sub-tile
        const int kkey = kappa(crank * KROWS + krow);           // S column = operand row of the pair's tile
        for (int j = 0; j < n_tiles; ++j) {
            const uint8_t* src = smem + OFF_RAWK + slot(j) * RAW_BYTES + kkey * REC;
            wait(B_KRAW_FULL + slot(j), phase(j), 50);
            // the S MMA that last read this K buffer (tile j - NB) must be complete
            if (j >= NB) wait(B_S + slot(j), phase(j - NB), 50);
            uint8_t* Kdst = Ksm + L::koff(slot(j), sub);
            uint8_t* Ldst = Klo + L::koff(slot(j), sub);
#pragma unroll
            for (int bb = 0; bb < NBT; ++bb) {
                const int blk = blk0 + bb;
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
                    *reinterpret_cast<uint4*>(Ldst + sw128(krow, ch)) = r;
                }
            }
            proxy_fence();
            __syncwarp();
            if (lane == 0) { arrive_issuer(B_KF + slot(j)); mbar_arrive(&bars[B_KRAW_FREE + slot(j)]); }
        }
    } else {
        // ======================= softmax warps: one thread per accumulator row, groups alternate tiles ====
        regs_grow<REGS_SOFT>();
        const int m = tid & 127;                               // row = TMEM lane
        const int grp = tid >> 7;                              // which 32 of a tile's 64 columns this thread owns
        const int qtr = warp & 3;
        const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
        const int r = m / G, h = m - r * G;
        const bool row_ok = r < rows_eff;
        const int prow = p_first + r;
        const int row_lo = P.is_swa ? max(0, prow + 1 - P.W) : 0;     // bruce.cu:3014
        const float c2 = P.scale_log2;
        const float thr = RESCALE_THRESHOLD / c2;              // threshold in raw-score units
        const uint64_t c2p = pack_f2(c2, c2);
        // the two threads of a row keep the row reference in a register each: they see the same maxima and take
        // the same decisions
        float m_ref = NEG_BIG;

        for (int j = 0; j < n_tiles; ++j) {
            const int t0 = (tile_first + j) * BN;
            const int ch2 = L::schunk((j ^ 1) < n_tiles);          // the tile's second 32 columns (see Lay::scol)
            const uint32_t tS = tmem + lane_base + T_S + L::scol(slot(j));
            // tiles every row of the CTA sees completely skip the mask code (bruce.cu:2927-2928)
            // (rows past the end of a ragged M tile hold zero queries: whatever they compute is finite and never stored)
            const bool masked = !(t0 >= full_lo && t0 + BN - 1 <= p_first);
            wait(B_S + slot(j), phase(j), 50);
            tc_fence_after();
            uint32_t v[32];
            tmem_ld32(tS + (grp ? ch2 : 0), v);
            if (masked) {
                // Tiles that some row of the CTA sees only partly (the causal diagonal, the window edge, a
                // ragged last chunk): hidden columns are replaced by "minus infinity" (bruce.cu:3021-3028),
                // after which the common code below needs no mask.  The visibility bits are built by a rolled
                // loop to keep this rarely executed path small.
                uint32_t bits = 0u;
#pragma unroll 1
                for (int i = 0; i < 32; ++i) {
                    const int key = t0 + kappa(grp * 32 + i);
                    const bool ok = row_ok && key <= prow && key >= row_lo;
                    bits |= (ok ? 1u : 0u) << i;
                }
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (!((bits >> i) & 1u)) v[i] = __float_as_uint(NEG_BIG);
            }
            float mx;
            {
                float m0 = __uint_as_float(v[0]), m1 = __uint_as_float(v[1]);
                float m2 = __uint_as_float(v[2]), m3 = __uint_as_float(v[3]);
#pragma unroll
                for (int i = 4; i + 8 <= 32; i += 8) {
                    m0 = fmax3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                    m1 = fmax3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                    m2 = fmax3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                    m3 = fmax3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                }
                m0 = fmax3(m0, __uint_as_float(v[28]), __uint_as_float(v[29]));
                m1 = fmax3(m1, __uint_as_float(v[30]), __uint_as_float(v[31]));
                mx = fmax3(fmaxf(m0, m1), m2, m3);
            }
            // the row maximum of the tile: exchange the two halves through shared memory (double-buffered by tile
            // parity; the barrier of the next tile separates a buffer's reads from its next writes)
            {
                volatile float* x = mref + (j & 1) * 256;
                x[grp * 128 + m] = mx;
                named_bar_sync(4 + qtr, 64);
                mx = fmaxf(mx, x[(grp ^ 1) * 128 + m]);
            }
            const float m_new = fmaxf(m_ref, mx);
            const bool need = m_new > m_ref + thr;
            if (__any_sync(0xffffffffu, need)) {
                if (j > 0) {
                    wait(B_PV + slot(j - 1), phase(j - 1), 50);         // O must be complete before it is rescaled
                    tc_fence_after();
                    const float alpha = need ? fast_exp2((m_ref - m_new) * c2) : 1.f;
#pragma unroll 1
                    for (int c = 0; c < HD / 64; ++c) {                 // each thread its half of the row
                        uint32_t o[32];
                        const uint32_t ta = tmem + lane_base + T_O + L::ocol(2 * grp + c);
                        tmem_ld32(ta, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(ta, o);
                    }
                    if (grp == 0) {
                        const uint32_t tl = tmem + lane_base + T_L;
                        tmem_st1(tl, __float_as_uint(__uint_as_float(tmem_ld1(tl)) * alpha));
                    }
                    tmem_st_wait();
                    tc_fence_before();
                }
                if (need) m_ref = m_new;
            }
            // p = 2^(s*c2 - m_ref*c2); a row that has seen no key yet keeps the offset at zero, so its hidden
            // columns ("minus infinity") still come out as exactly zero
            const float nb = m_ref > 0.5f * NEG_BIG ? -m_ref * c2 : 0.f;
            const uint64_t nbp = pack_f2(nb, nb);
            // P (fp16 pairs): the tile's 32 packed columns overwrite its first 32 S columns, this thread's half of
            // them at offset 16 * grp.  The other thread of the row may still be reading those S columns: both have
            // passed the barrier above only after their loads completed.
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float e0, e1;
                ffma2(e0, e1, __uint_as_float(v[i]), __uint_as_float(v[i + 1]), c2p, nbp);
                pk[i >> 1] = pack_h2(fast_exp2(e0), fast_exp2(e1));
            }
            tmem_st16(tS + 16 * grp, pk);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_issuer(B_P + slot(j));
        }
        // ---- epilogue: O / sum(P) -> global; each of the two threads of a row writes half of it ----------
        // (the last tile's predecessor in its ring slot completed before this thread was handed the tile's scores,
        // so the parity wait below cannot be satisfied early)
        wait(B_PV + slot(n_tiles - 1), phase(n_tiles - 1), 50);
        tc_fence_after();
        const float l = __uint_as_float(tmem_ld1(tmem + lane_base + T_L));
        const float il = l > 0.f ? 1.f / l : 0.f;
        const size_t oi = (((size_t)(rbase + r)) * P.Hq + kvh * G + h) * HD + grp * (HD / 2);
        // with key splits: a split record (unnormalised o, m in log2 units, l) instead of the output row
        float* rec = P.recs ? P.recs + ((((size_t)blockIdx.z * P.rows) + rbase + r) * P.Hq + kvh * G + h) * (size_t)(HD + 2)
                                  : nullptr;
        if (rec && row_ok && grp == 0) {
            const float mr = m_ref;
            rec[HD] = mr > 0.5f * NEG_BIG ? mr * c2 : NEG_BIG;
            rec[HD + 1] = l;
        }
#pragma unroll 1
        for (int c = 0; c < HD / 64; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem + lane_base + T_O + L::ocol(2 * grp + c), o);
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
    if (PAIR) cluster_sync_all();          // neither CTA leaves (or frees tensor memory) while the other may still use it
    if (warp == W_MMA) {
        tc_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
        else      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace pf128
}  // namespace battn
