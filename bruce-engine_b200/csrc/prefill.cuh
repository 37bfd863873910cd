// Prompt-chunk attention on the 5th-generation tensor cores: causal + sliding-window flash attention of
// a chunk of query rows against the growing q8_0 cache (the chunk's own keys were appended first).
//
// Behaviour replaced: k_attn_tc_rs_opt<NW,...> for rows > 8 and its dispatch
// (engine/src/bruce.cu:2750-3131, 4021-4078); masks as bruce.cu:2799-2805, 3012-3029.
//
// This file holds the kernel for head_dim 256 (the reference's own geometry) and the helpers shared with the
// head_dim 128 kernel (prefill_hd128.cuh).
//
// Design (sm_100a), one CTA per (128-row M tile, kv head, key split), 20 warps, each warpgroup resized with
// setmaxnreg for its role (8 softmax, 4 K-dequant, 4 V-dequant, S issuer, loader, P.V issuer, 1 idle):
//   * M tile = 128/G consecutive query positions x the G query heads of one kv head (row m = position
//     m / G, head m % G, the reference's pair packing, bruce.cu:2288-2296): every dequantised K/V tile
//     serves all G heads, and the causal diagonal of a tile spans only 128/G positions.
//   * A loader thread streams raw K and V tiles (64 records each, one contiguous run per tile because the
//     cache is head-major) with cp.async.bulk into a two-stage ring.
//   * Two groups of four dequant warps (K and V in parallel) turn raw q8_0 records into fp16 operands in
//     128-byte-swizzled K-major shared memory: K as [key][dim] in two fp16 parts, hi = fp16(d*x) and
//     lo = d*x - hi (exact), so that S carries no rounding of the K operand (a single folded operand alone moves
//     single (row, head) outputs by up to 7e-4 relative); V transposed to [dim][key] with byte-permute
//     interleaves, scale folded in, double-buffered.  The K buffers hold one 128-dim half of the tile each and
//     are refilled half by half as the S MMAs release them.
//   * S = Q K^T (M 128, N 64, K head_dim) and O += P V (M 128, N head_dim, K 64) run as tcgen05.mma with
//     fp32 accumulators in tensor memory, issued by two threads (one per product) so that neither waits on
//     the other's barriers.  Q is the tensor-memory A operand of the first product, P of the second; the
//     512 tensor-memory columns are O (256) + two S/P buffers (64 each) + Q (128).
//   * Eight softmax warps: TMEM lane = accumulator row, two threads per row (one per half of the S
//     columns): one tcgen05.ld, 3-input max, an exchange of the row maximum through shared memory, packed
//     fma + ex2, and P written back as fp16 pairs over the S columns just read.  With no tensor-memory
//     column left for it, the softmax denominator is summed by these threads (fp32, next to P).  O is
//     rescaled in TMEM only when a row maximum grows by more than 2^8 (the reference value is kept otherwise
//     and the final normalisation uses the same reference, so the result is unchanged).
//   * Key splits: when the (M tile, kv head) grid leaves SMs idle (64 CTAs for a 512-row chunk), gridDim.z
//     CTAs share one M tile, each taking a contiguous share of the key tiles and leaving split records
//     (unnormalised o, m, l) for the merge kernel.
//   * Row n of the K operand / column n of S holds key kappa(n), a fixed permutation inside each 64-key
//     span chosen so that every shared-memory access of the dequant warps is bank-conflict free.
//   * Every mbarrier wait is bounded; a wait that runs out sets the device status word, the remaining
//     waits are skipped, tensor memory is released and the kernel returns.
#pragma once
#include "common.cuh"

namespace battn {
namespace pf {

constexpr int NSOFT = 256, NDEQ = 128;              // NDEQ threads dequantise K, another NDEQ dequantise V
constexpr int NTHREADS = NSOFT + 2 * NDEQ + 128;    // warps 0-7 softmax, 8-11 K dequant, 12-15 V dequant, 16 MMA issue, 17 loader, 18-19 idle
// Registers per thread: the kernel launches with REGS_LAUNCH everywhere (five warps share each quarter of the
// register file); every warpgroup then resizes itself for its role with setmaxnreg, so the softmax warps can
// hold a whole S row segment in registers.  Per quarter: 2*REGS_SOFT + 2*REGS_DEQ + REGS_CTL <= 5*REGS_LAUNCH.
constexpr int REGS_LAUNCH = 96, REGS_SOFT = 144, REGS_DEQ = 72, REGS_CTL = 40;
static_assert(2 * REGS_SOFT + 2 * REGS_DEQ + REGS_CTL <= 5 * REGS_LAUNCH, "register budget per scheduler");
constexpr int TMEM_COLS = 512;
constexpr float RESCALE_THRESHOLD = 8.0f;   // log2 units

struct Params {
    const void* q;
    void* out;
    const uint8_t* kvk;
    const uint8_t* kvv;
    const int* pos;
    int rows, Hq, Hkv, G;
    int W, pstride, ring_mask, slot_ctx, is_swa, q_f16, out_f16;
    float scale_log2;
    int* status;
    // key split: gridDim.z CTAs share one (M tile, kv head), each takes a contiguous share of the key tiles and
    // writes split records [split][row][head][HD+2] = (unnormalised o, m in log2 units, l) for the merge kernel;
    // recs != null with nsplit == 1 leaves the single record per row in place of the output (for the fused
    // merge + gate-norm epilogue)
    int nsplit;
    float* recs;
    Paging pg;       // table != nullptr: paged cache of a full-causal layer; `slot` is the table row of the sequence
    int slot = 0;
    // Both prompt kernels are launched with programmatic stream serialisation: with early != 0 the position is read and
    // the key tiles that lie entirely below the chunk's first row are streamed and converted before
    // griddepcontrol.wait, i.e. while the append of the chunk's own rows is still running; Q, the tiles holding the
    // chunk's rows and every write come after it (same contract as fd::Params::early)
    int early = 0;
};

template <int HD, int BN>
struct Cfg {
    static constexpr int NBLK = HD / 32;
    static constexpr int REC = HD + 2 * NBLK;
    // Q lives in tensor memory (the TMEM A operand of the S MMA) and the shared memory it would take
    // double-buffers the fp16 K and V operands, so dequantising tile j+1 overlaps the MMAs of tile j.
    // At head_dim 256 that uses every tensor-memory column (O 256 + two S buffers of 64 + Q 128), so the
    // softmax denominator cannot be accumulated by the tensor core there: the softmax threads sum it.
    static constexpr bool Q_TMEM = true;
    static constexpr bool L_MMA = HD == 128;
    static constexpr int KV_BUFS = 2;
    static constexpr int RAW_STAGES = 2;
    static constexpr int Q_BYTES = Q_TMEM ? 0 : 128 * HD * 2;
    // K operand: two buffers, one per 128-dim half of the head, each holding that half of the current tile twice:
    // hi = fp16(d * x) and lo = d * x - hi (exact), 16 KB each.  (Not double-buffered across tiles: the dequant
    // of half h of tile j+1 starts as soon as the S MMAs over half h of tile j have completed.)
    static constexpr int K_PART_BYTES = BN * 128 * 2;          // [BN keys][128 dims] fp16 = two 64-dim sub-tiles
    static constexpr int K_HALF_BYTES = 2 * K_PART_BYTES;      // hi + lo
    static constexpr int K_BYTES = BN * HD * 2;                // KV_BUFS * K_BYTES == 2 * K_HALF_BYTES
    static constexpr int V_BYTES = HD * BN * 2;
    static constexpr int RAW_BYTES = BN * REC;              // one raw K (or V) tile
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + Q_BYTES;
    static constexpr int OFF_V = OFF_K + KV_BUFS * K_BYTES;
    static constexpr int ONES_BYTES = L_MMA ? 16 * BN * 2 : 0;   // 16 operand rows of ones: the denominator MMA
    static constexpr int OFF_ONES = OFF_V + KV_BUFS * V_BYTES;
    static constexpr int OFF_RAW = OFF_ONES + ONES_BYTES;    // [RAW_STAGES buffers][K | V]
    static constexpr int OFF_BAR = OFF_RAW + RAW_STAGES * 2 * RAW_BYTES;
    static constexpr int N_BARS = 18;
    static constexpr int OFF_MISC = OFF_BAR + N_BARS * 8;    // tmem base, abort flag
    static constexpr int OFF_RMAX = OFF_MISC + 16;           // [tile parity][2 halves][128 rows] row maxima
    static constexpr int TOTAL = OFF_RMAX + 2 * 2 * 128 * 4 + 1024;   // + slack to align the base to 1024
    static constexpr int T_O = 0;                            // TMEM columns
    static constexpr int T_L = HD;                           // 16 columns, each = sum of P
    static constexpr int T_S0 = HD + (L_MMA ? 32 : 0);
    static constexpr int T_S1 = T_S0 + BN;
    static constexpr int T_Q = T_S1 + BN;                    // HD/2 columns of fp16 pairs
    static_assert(T_Q + HD / 2 <= TMEM_COLS, "tensor memory budget");
    static_assert(RAW_BYTES % 16 == 0, "bulk copy size");
    static_assert(HD == 256 && BN == 64 && KV_BUFS == 2, "supported tile shape");
    static_assert(TOTAL <= 226 * 1024, "shared memory budget");
};

// barrier indices
// every role-to-role barrier exists twice and alternates with the tile parity, so that no role can complete
// two phases of a barrier before its waiter has observed the first
// (B_KF0 + h and B_KFREE0 + h are indexed by the 128-dim half h of the K operand instead and complete once per tile)
enum { B_RAW_FULL0 = 0, B_RAW_FREE0 = 3, B_KF0 = 6, B_VF0 = 8, B_S0 = 10, B_P0 = 12, B_PV0 = 14, B_KFREE0 = 16 };

// byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a [rows x 64 halves] sub-tile stored
// K-major with the 128-byte swizzle (8-row atoms of 1024 B, chunk index XOR row-in-atom)
__device__ __forceinline__ uint32_t sw128(int row, int chunk) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + (((chunk ^ row) & 7) << 4));
}

// key (offset inside the tile) held by operand row / S column n
__host__ __device__ constexpr int kappa(int n) {
    return (n & ~63) + 16 * ((n & 7) >> 1) + 2 * ((((n >> 3) & 7) + 2 * ((n & 7) >> 1)) & 7) + (n & 1);
}

// shared-memory matrix descriptor: K-major, SWIZZLE_128B, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// instruction descriptor, kind::f16: fp16 A and B (both K-major), fp32 accumulator, M x N
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
// same, with the A operand in tensor memory (fp16 pairs packed in 32-bit columns, lane = row)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
          "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// single-column TMEM access (the denominator column)
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    return r;
}
__device__ __forceinline__ void tmem_st1(uint32_t taddr, uint32_t r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(r) : "memory");
}
// 32 columns without the wait, so several loads can be in flight
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// three-input maximum and two-wide fp32 multiply-add: each halves the instruction count of its softmax pass
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pack_f2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void ffma2(float& o0, float& o1, float x0, float x1, uint64_t mul, uint64_t add) {
    asm("{\n\t.reg .b64 a, r;\n\tmov.b64 a, {%2, %3};\n\tfma.rn.f32x2 r, a, %4, %5;\n\tmov.b64 {%0, %1}, r;\n\t}"
        : "=f"(o0), "=f"(o1)
        : "f"(x0), "f"(x1), "l"(mul), "l"(add));
}
template <int N> __device__ __forceinline__ void regs_grow() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void regs_shrink() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

template <int HD, int BN>
__global__ void __maxnreg__(REGS_LAUNCH) k_prefill(const Params P) {
    using C = Cfg<HD, BN>;
    constexpr int NBLK = C::NBLK, REC = C::REC;
    constexpr int HC = BN / 2;                               // S columns per softmax thread
    constexpr int NCH = HC / 32;                             // ... in TMEM loads of 32 columns
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);      // 1024-byte aligned
    uint8_t* Qsm = smem + C::OFF_Q;
    uint8_t* Ksm = smem + C::OFF_K;
    uint8_t* Vsm = smem + C::OFF_V;
    uint8_t* ONES = smem + C::OFF_ONES;
    uint8_t* RAW = smem + C::OFF_RAW;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC);   // [0] tmem base, [1] abort
    volatile float* rmax = reinterpret_cast<volatile float*>(smem + C::OFF_RMAX);          // [2][2][128]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = P.G, MR = 128 / G;                        // query positions per M tile
    const int n_mt = (P.rows + MR - 1) / MR;
    const int mt = n_mt - 1 - (int)blockIdx.x;              // longest key ranges first (bruce.cu:2770)
    const int kvh = blockIdx.y;
    const bool early = P.early != 0;                        // see Params::early
    if (!early) { pdl_wait(); pdl_trigger(); }
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
    const int tile_lo = lo_cta / BN;
    const int n_all = (hi_cta + BN - 1) / BN - tile_lo;                // key tiles of this M tile
    const int per_split = (n_all + P.nsplit - 1) / P.nsplit;
    const int tile_first = tile_lo + (int)blockIdx.z * per_split;      // this CTA's share
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

    // ---- set-up: barriers, tensor memory, the Q operand, the block of ones ---------------------------
    if (tid == 0) {
        for (int st = 0; st < C::RAW_STAGES; ++st) {
            mbar_init(&bars[B_RAW_FULL0 + st], 1);
            mbar_init(&bars[B_RAW_FREE0 + st], 2 * NDEQ / 32);
        }
        for (int par = 0; par < 2; ++par) {
            mbar_init(&bars[B_KF0 + par], NDEQ / 64); mbar_init(&bars[B_VF0 + par], NDEQ / 32);
            mbar_init(&bars[B_KFREE0 + par], 1);
            mbar_init(&bars[B_S0 + par], 1); mbar_init(&bars[B_PV0 + par], 1);
            mbar_init(&bars[B_P0 + par], NSOFT / 32);
        }
        misc[1] = 0;
        mbar_fence_init();
    }
    if (warp == (NSOFT + 2 * NDEQ) / 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(&misc[0]))), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Q: row m = (position m / G, head m % G), fp16, 64-dim sub-tiles, swizzled (shared-memory variant)
    for (int idx = tid; idx < (C::Q_TMEM ? 0 : 128 * (HD / 8)); idx += NTHREADS) {
        const int m = idx / (HD / 8), ch = idx - m * (HD / 8);
        const int r = m / G, h = m - r * G;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (r < rows_eff) {
            const size_t qi = (((size_t)(rbase + r)) * P.Hq + kvh * G + h) * HD + ch * 8;
            if (P.q_f16) {
                val = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(P.q) + qi);
            } else {
                const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.q) + qi);
                const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.q) + qi + 4);
                val = make_uint4(pack_h2(a.x, a.y), pack_h2(a.z, a.w), pack_h2(b.x, b.y), pack_h2(b.z, b.w));
            }
        }
        *reinterpret_cast<uint4*>(Qsm + (ch >> 3) * (128 * 128) + sw128(m, ch & 7)) = val;
    }
    for (int idx = tid; idx < C::ONES_BYTES / 16; idx += NTHREADS)
        reinterpret_cast<uint4*>(ONES)[idx] = make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];
    if constexpr (C::Q_TMEM) {
        // Q into tensor memory: lane = row m, 32-bit column c = dims (2c, 2c+1); two threads per row
        if (tid < NSOFT) {
            if (early) { pdl_wait(); pdl_trigger(); }             // Q is the predecessor's output; so is everything these warps write
            const int m = tid & 127, half = tid >> 7;
            const int r = m / G, h = m - r * G;
#pragma unroll 1
            for (int cq = 0; cq < HD / 128; ++cq) {               // 64 dims = 32 columns per store
                uint32_t qv[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) qv[i] = 0u;
                if (r < rows_eff) {
                    const size_t qi = (((size_t)(rbase + r)) * P.Hq + kvh * G + h) * HD + half * (HD / 2) + cq * 64;
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
                tmem_st32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + C::T_Q + half * (HD / 4) + cq * 32, qv);
            }
            tmem_st_wait();
        }
        // Q only concerns its writers (the softmax warps) and its reader (the S issuer): the loader, the dequant
        // warps and the P.V issuer go straight to work, so the first raw tiles and their conversion overlap the Q load
        if (warp < NSOFT / 32 || warp == (NSOFT + 2 * NDEQ) / 32) {
            tc_fence_before();
            named_bar_sync(6, NSOFT + 32);
            tc_fence_after();
        }
    }

    // bounded wait that degrades to "do not wait" once any wait has run out
    auto wait = [&](int b, uint32_t parity) {
        if (mbar_try_wait(&bars[b], parity)) return;               // the common case costs one poll
        if (misc[1]) return;
        if (!mbar_wait_backoff(&bars[b], parity)) {
            atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
            misc[1] = 1;
        }
    };

    const size_t hb = (size_t)kvh * P.pstride * (size_t)REC;

    if (warp >= (NSOFT + 2 * NDEQ) / 32) regs_shrink<REGS_CTL>();          // the whole last warpgroup
    if (warp == (NSOFT + 2 * NDEQ) / 32) {
        // ======================= S = Q K^T for every tile ==============================================
        // A thread of its own: one thread that polls three barriers and issues every MMA of a tile is itself
        // the critical path.  S of tile j+1 refills the buffer whose P the P.V MMA of tile j-1 consumed.
        if (lane == 0) {
            const uint32_t idS = umma_idesc(128, BN);
            const uint32_t ka = smem_u32(Ksm);
            for (int j = 0; j < n_tiles; ++j) {
                if (j >= 2) wait(B_PV0 + (j & 1), ((j - 2) >> 1) & 1);
                const uint32_t d = tmem + ((j & 1) ? C::T_S1 : C::T_S0);
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    wait(B_KF0 + hf, j & 1);
                    tc_fence_after();
                    // S += Q_half K_hi^T + Q_half K_lo^T: the two fp16 parts add up to the exact product d * x of
                    // every cached value, so the scores carry no rounding of the K operand
#pragma unroll
                    for (int part = 0; part < 2; ++part)
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {
                            const uint64_t b = umma_desc(ka + hf * C::K_HALF_BYTES + part * C::K_PART_BYTES + (ks >> 2) * (BN * 128)) + 2 * (ks & 3);
                            umma_f16_ts(d, tmem + C::T_Q + 8 * (8 * hf + ks), b, idS, (hf | part | ks) != 0);
                        }
                    umma_commit(&bars[B_KFREE0 + hf]);          // the dequant warps may refill this half
                }
                umma_commit(&bars[B_S0 + (j & 1)]);
            }
        }
    } else if (warp == (NSOFT + 2 * NDEQ) / 32 + 2) {
        // ======================= O += P V (and the denominator block) for every tile ====================
        if (lane == 0) {
            const uint32_t idO = umma_idesc(128, HD), idL = umma_idesc(128, 16);
            const uint32_t va = smem_u32(Vsm), oa = smem_u32(ONES);
            for (int j = 0; j < n_tiles; ++j) {
                wait(B_P0 + (j & 1), (j >> 1) & 1);
                wait(B_VF0 + (j & 1), (j >> 1) & 1);
                tc_fence_after();
                const uint32_t vb = va + (j % C::KV_BUFS) * C::V_BYTES;
                const uint32_t tP = tmem + ((j & 1) ? C::T_S1 : C::T_S0);     // P overwrote the S tile
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    const uint32_t acc = (j > 0 || ks > 0) ? 1u : 0u;
                    // keys of column half hf sit in 32-bit columns [hf*BN/2, hf*BN/2 + BN/4): 8 per k-step
                    const uint32_t a = tP + (ks / (BN / 32)) * (BN / 2) + 8 * (ks % (BN / 32));
                    const uint64_t b = umma_desc(vb + (ks >> 2) * (HD * 128)) + 2 * (ks & 3);
                    const uint64_t o = umma_desc(oa + (ks >> 2) * (16 * 128)) + 2 * (ks & 3);
                    umma_f16_ts(tmem + C::T_O, a, b, idO, acc);
                    if constexpr (C::L_MMA) umma_f16_ts(tmem + C::T_L, a, o, idL, acc);   // every column = sum of P
                }
                umma_commit(&bars[B_PV0 + (j & 1)]);
            }
        }
    } else if (warp == (NSOFT + 2 * NDEQ) / 32 + 1) {
        // ======================= loader: streams raw K and V tiles into the ring with bulk copies ========
        if (lane == 0) {
            bool waited = !early;
            for (int j = 0; j < n_tiles; ++j) {
                const int b = j % C::RAW_STAGES;
                // early streaming stops at the first tile that holds a row of this chunk
                if (!waited && (tile_first + j + 1) * BN > p0) { pdl_wait(); pdl_trigger(); waited = true; }
                if (j >= C::RAW_STAGES) wait(B_RAW_FREE0 + b, (j / C::RAW_STAGES - 1) & 1);   // both dequant groups left it
                const int sp = ((tile_first + j) * BN) & P.ring_mask;
                const int nk = P.pg.table ? BN : min(BN, P.pstride - sp);
                const uint32_t bytes = (uint32_t)nk * REC;
                // (a paged look-up here is hidden by the ring: the loader runs RAW_STAGES tiles ahead of the dequant warps)
                const size_t off = P.pg.table ? kv_rec_index(P.pg, P.slot, kvh, P.Hkv, P.pstride, sp, P.status) * (size_t)REC
                                              : hb + (size_t)sp * REC;
                uint8_t* dst = RAW + b * 2 * C::RAW_BYTES;
                mbar_expect_tx(&bars[B_RAW_FULL0 + b], 2 * bytes);
                bulk_g2s(dst, P.kvk + off, bytes, &bars[B_RAW_FULL0 + b]);
                bulk_g2s(dst + C::RAW_BYTES, P.kvv + off, bytes, &bars[B_RAW_FULL0 + b]);
            }
        }
    } else if (warp > (NSOFT + 2 * NDEQ) / 32 + 2) {
        // idle warp that completes the last warpgroup
    } else if (warp >= (NSOFT + NDEQ) / 32) {
        // ======================= V dequant warps: V^T operand, [dim][key] ============================
        regs_shrink<REGS_DEQ>();
        const int t = tid - NSOFT - NDEQ, wq = t >> 5;
        constexpr int NWG = HD / 16;                            // groups of four dim-words
        constexpr int UPT = (HD / 4) * (BN / 8) / NDEQ;         // micro-tiles (4 dims x 8 keys) per thread
        const int ccl = lane & 7, wl = lane >> 3;
        const int cc = 8 * ((UPT * wq) / NWG) + ccl;            // key chunk (8 keys), fixed per thread
        int vkey[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) vkey[jj] = kappa(8 * cc + jj);

        for (int j = 0; j < n_tiles; ++j) {
            const int b = j % C::RAW_STAGES;
            const int t0 = (tile_first + j) * BN;
            const uint8_t* Vraw = RAW + b * 2 * C::RAW_BYTES + C::RAW_BYTES;
            wait(B_RAW_FULL0 + b, (j / C::RAW_STAGES) & 1);
            // the P.V MMA that last read this V buffer (tile j - KV_BUFS) must be complete
            if (j >= C::KV_BUFS) wait(B_PV0 + ((j - C::KV_BUFS) & 1), ((j - C::KV_BUFS) >> 1) & 1);
            uint8_t* Vdst = Vsm + (j % C::KV_BUFS) * C::V_BYTES;
            {
                // keys outside [lo, hi) were never written for this chunk's rows: their bytes are arbitrary,
                // so their scale is forced to zero (their P is zero as well)
                bool kok[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) kok[jj] = (t0 + vkey[jj] >= lo_cta) && (t0 + vkey[jj] < hi_cta);
                uint32_t sp[4];
#pragma unroll 1
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
                        *reinterpret_cast<uint4*>(Vdst + (cc >> 3) * (HD * 128) + sw128(d, cc & 7)) =
                            make_uint4(chunk[i][0], chunk[i][1], chunk[i][2], chunk[i][3]);
                    }
                }
            }
            proxy_fence();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&bars[B_VF0 + (j & 1)]); mbar_arrive(&bars[B_RAW_FREE0 + b]); }
        }
    } else if (warp >= NSOFT / 32) {
        // ======================= K dequant warps: K operand, [key][dim] ==============================
        regs_shrink<REGS_DEQ>();
        const int t = tid - NSOFT;
        const int krow = t & (BN - 1);                          // each thread converts one 128-dim half of one row
        const int hf = t / BN;                                  // which half: warps 0-1 -> dims 0..127, warps 2-3 -> 128..255
        const int kkey = kappa(krow);
        for (int j = 0; j < n_tiles; ++j) {
            const int b = j % C::RAW_STAGES;
            const uint8_t* Kraw = RAW + b * 2 * C::RAW_BYTES;
            wait(B_RAW_FULL0 + b, (j / C::RAW_STAGES) & 1);
            // the S MMAs over this half of tile j - 1 must be complete before the buffer is refilled
            if (j >= 1) wait(B_KFREE0 + hf, (j - 1) & 1);
            uint8_t* Kdst = Ksm + hf * C::K_HALF_BYTES;
            {
                const uint8_t* src = Kraw + kkey * REC;
#pragma unroll 2
                for (int c = 0; c < 16; ++c) {
                    const int ch = 16 * hf + c;                 // 16-byte chunk of the fp16 row (8 dims)
                    const __half sc = reinterpret_cast<const __half*>(src)[ch >> 2];
                    const __half2 s2 = __half2half2(sc);
                    const uint32_t su = *reinterpret_cast<const uint32_t*>(&s2);
                    const uint2 w = *reinterpret_cast<const uint2*>(src + 2 * NBLK + ch * 8);
                    const uint32_t x = w.x ^ 0x80808080u, y = w.y ^ 0x80808080u;
                    const uint32_t i0 = sub1152(widen_lo(x)), i1 = sub1152(widen_hi(x));
                    const uint32_t i2 = sub1152(widen_lo(y)), i3 = sub1152(widen_hi(y));
                    uint4 o, r;
                    o.x = hmul2_u32(i0, su); r.x = hfma2_residual(i0, su, o.x);
                    o.y = hmul2_u32(i1, su); r.y = hfma2_residual(i1, su, o.y);
                    o.z = hmul2_u32(i2, su); r.z = hfma2_residual(i2, su, o.z);
                    o.w = hmul2_u32(i3, su); r.w = hfma2_residual(i3, su, o.w);
                    const uint32_t off = (c >> 3) * (BN * 128) + sw128(krow, c & 7);
                    *reinterpret_cast<uint4*>(Kdst + off) = o;
                    *reinterpret_cast<uint4*>(Kdst + C::K_PART_BYTES + off) = r;
                }
            }
            proxy_fence();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&bars[B_KF0 + hf]); mbar_arrive(&bars[B_RAW_FREE0 + b]); }
        }
    } else {
        // ======================= softmax warps: two threads per accumulator row ========================
        regs_grow<REGS_SOFT>();
        const int m = tid & 127;                               // row = TMEM lane
        const int half = tid >> 7;                             // which half of the S columns / O columns
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const int r = m / G, h = m - r * G;
        const bool row_ok = r < rows_eff;
        const int prow = p_first + r;
        const int row_lo = P.is_swa ? max(0, prow + 1 - P.W) : 0;     // bruce.cu:3014
        const float c2 = P.scale_log2;
        const float thr = RESCALE_THRESHOLD / c2;              // threshold in raw-score units
        float m_ref = NEG_BIG;                                 // reference maximum, raw-score units
        float l_part = 0.f;                                    // this thread's share of sum(P) when the tensor core cannot keep it

        for (int j = 0; j < n_tiles; ++j) {
            const int t0 = (tile_first + j) * BN;
            const uint32_t tS = tmem + lane_base + ((j & 1) ? C::T_S1 : C::T_S0) + half * HC;
            // tiles every row of the CTA sees completely skip the mask code (bruce.cu:2927-2928)
            // (rows past the end of a ragged M tile hold zero queries: whatever they compute is finite and never stored)
            const bool masked = !(t0 >= full_lo && t0 + BN - 1 <= p_first);
            wait(B_S0 + (j & 1), (j >> 1) & 1);
            tc_fence_after();
            // One read of this thread's S columns; they stay in registers for both the maximum and the
            // exponentials.
            uint32_t v[NCH][32];
#pragma unroll
            for (int c = 0; c < NCH; ++c) tmem_ld32_nowait(tS + c * 32, v[c]);
            tmem_ld_wait();
            if (masked) {
                // Tiles that some row of the CTA sees only partly (the causal diagonal, the window edge, a
                // ragged last chunk): hidden columns are replaced by "minus infinity" (bruce.cu:3021-3028),
                // after which the common code below needs no mask.  The visibility bits are built by a rolled
                // loop to keep this rarely executed path small.
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    uint32_t bits = 0u;
#pragma unroll 1
                    for (int i = 0; i < 32; ++i) {
                        const int key = t0 + kappa(half * HC + c * 32 + i);
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
                for (int c = 0; c < NCH; ++c) {
#pragma unroll
                    for (int i = (c == 0 ? 4 : 0); i + 8 <= 32; i += 8) {
                        m0 = fmax3(m0, __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]));
                        m1 = fmax3(m1, __uint_as_float(v[c][i + 2]), __uint_as_float(v[c][i + 3]));
                        m2 = fmax3(m2, __uint_as_float(v[c][i + 4]), __uint_as_float(v[c][i + 5]));
                        m3 = fmax3(m3, __uint_as_float(v[c][i + 6]), __uint_as_float(v[c][i + 7]));
                    }
                    if (c == 0) {
                        m0 = fmax3(m0, __uint_as_float(v[0][28]), __uint_as_float(v[0][29]));
                        m1 = fmax3(m1, __uint_as_float(v[0][30]), __uint_as_float(v[0][31]));
                    }
                }
                mx = fmax3(fmaxf(m0, m1), m2, m3);
            }
            // exchange with the thread that holds the other half of this row (same lane, warp +-4); the buffer
            // alternates with the tile parity so that a fast thread's next write cannot overtake a slow
            // partner's read
            rmax[(j & 1) * 256 + half * 128 + m] = mx;
            named_bar_sync(2 + (warp & 3), 64);
            mx = fmaxf(mx, rmax[(j & 1) * 256 + (half ^ 1) * 128 + m]);
            float m_new = fmaxf(m_ref, mx);
            const bool need = m_new > m_ref + thr;
            if (!need) m_new = m_ref;
            const bool warp_need = __any_sync(0xffffffffu, need);
            if (warp_need) {
                if (j > 0) {
                    wait(B_PV0 + ((j - 1) & 1), ((j - 1) >> 1) & 1);        // O must be complete before it is rescaled
                    tc_fence_after();
                    const float alpha = fast_exp2((m_ref - m_new) * c2);  // 1 for rows that keep their reference
#pragma unroll 1
                    for (int c = 0; c < HD / 64; ++c) {
                        uint32_t o[32];
                        const uint32_t ta = tmem + lane_base + C::T_O + half * (HD / 2) + c * 32;
                        tmem_ld32(ta, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(ta, o);
                    }
                    if constexpr (C::L_MMA) {
                        if (half == 0) {
                            const uint32_t tl = tmem + lane_base + C::T_L;
                            tmem_st1(tl, __float_as_uint(__uint_as_float(tmem_ld1(tl)) * alpha));
                        }
                    } else {
                        l_part *= alpha;
                    }
                    tmem_st_wait();
                }
                m_ref = m_new;
            }
            // p = 2^(s*c2 - m_ref*c2); a row that has seen no key yet keeps the offset at zero, so its hidden
            // columns ("minus infinity") still come out as exactly zero
            const float nb = m_ref > 0.5f * NEG_BIG ? -m_ref * c2 : 0.f;
            const uint64_t c2p = pack_f2(c2, c2), nbp = pack_f2(nb, nb);
            // P (fp16 pairs) overwrites S columns this thread owns and has already read: chunk c of S
            // (32 columns) becomes 16 columns of P at the start of the thread's region; nobody else reads
            // or writes them, and the MMA that refills this S buffer is ordered after the P.V MMA
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float e0, e1;
                    ffma2(e0, e1, __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]), c2p, nbp);
                    const uint32_t ph = pack_h2(fast_exp2(e0), fast_exp2(e1));
                    if constexpr (!C::L_MMA) {
                        // the denominator sums the fp16-rounded weights the MMA multiplies with V, so that
                        // out = sum(p v) / sum(p) stays a convex combination of the V rows
                        const float2 pf = __half22float2(*reinterpret_cast<const __half2*>(&ph));
                        l_part += pf.x + pf.y;
                    }
                    pk[i >> 1] = ph;
                }
                tmem_st16(tS + c * 16, pk);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[B_P0 + (j & 1)]);
        }
        // ---- epilogue: O / sum(P) -> global; each thread writes half of its row -----------------------
        wait(B_PV0 + ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1);
        tc_fence_after();
        float l;
        if constexpr (C::L_MMA) {
            l = __uint_as_float(tmem_ld1(tmem + lane_base + C::T_L));
        } else {
            // the two threads of a row add their shares; the exchange buffer of the opposite tile parity is idle
            volatile float* xch = rmax + (n_tiles & 1) * 256;
            xch[half * 128 + m] = l_part;
            named_bar_sync(2 + (warp & 3), 64);
            l = l_part + xch[(half ^ 1) * 128 + m];
        }
        const float il = l > 0.f ? 1.f / l : 0.f;
        const size_t oi = (((size_t)(rbase + r)) * P.Hq + kvh * G + h) * HD + half * (HD / 2);
        float* rec = P.recs ? P.recs + ((((size_t)blockIdx.z * P.rows) + rbase + r) * P.Hq + kvh * G + h) * (size_t)(HD + 2)
                                  : nullptr;
        if (rec && row_ok && half == 0) {
            rec[HD] = m_ref > 0.5f * NEG_BIG ? m_ref * c2 : NEG_BIG;
            rec[HD + 1] = l;
        }
#pragma unroll 1
        for (int c = 0; c < HD / 64; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem + lane_base + C::T_O + half * (HD / 2) + c * 32, o);
            if (row_ok) {
                if (rec) {
                    float2* dst = reinterpret_cast<float2*>(rec + half * (HD / 2) + c * 32);    // records are 8-byte aligned
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
    if (warp == (NSOFT + 2 * NDEQ) / 32) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace pf
}  // namespace battn
