// Wide speculative-verify attention for head_dim 128 on the 5th-generation tensor cores: 17..32 (row, head) pairs
// per kv head (5..8 query rows at 4 heads per kv head) share one sweep over the q8_0 cache.
//
// Behaviour replaced: k_attn_tc_rs_opt<4,3,false,true> for 5..8 verify rows and its dispatch
// (engine/src/bruce.cu:3994-4019); contract as k_attn_m<M> (:2087-2143): rows at p0..p0+rows-1, keys before p0
// visible to every row, in-chunk causal mask key <= p0 + r, optional per-row window (:3686-3689).
//
// Why tensor memory here: with the warp-level MMA the dequantised fp16 tile has to be re-read from shared memory
// by every warp (ldmatrix), and that traffic -- eleven times the KV bytes -- bounds the kernel at a third of HBM
// rate.  tcgen05.mma reads each operand once, straight from shared memory.
//
// Orientation: KEYS on the M side.  Per 128-key tile
//     S^T[128 keys x 32 pairs] = K[128 keys x 128 dims] . Q^T        (A = K operand, B = Q, N = 32)
//     O^T[128 dims x 32 pairs] += V^T[128 dims x 128 keys] . P^T     (A = V^T operand, B = P^T, N = 32)
// so no MMA row is wasted on the 8 query rows, both accumulators are 32 columns of tensor memory, and K enters as
// EXACT integers: S^T is accumulated separately for the four 32-dim blocks of the head (4 x 32 columns), and the
// softmax thread that owns a key applies that key's four q8_0 block scales in fp32 -- the arithmetic of the
// flash-decode kernel (scales after the product), not the folded fp16 operand of the prompt kernels.
//
// One CTA per SM, 24 warps, each warpgroup resized with setmaxnreg for its role (together exactly the register file):
//   warps 0-7    softmax, two groups of four: a thread owns TMEM lane n = key kappa(n) of the tile and half of the
//                pairs (group 0: pairs 0-15, group 1: pairs 16-31): it reads its 4 x 16 partial scores, applies the
//                key's block scales, masks, and writes P^T = 2^(s - ref) (fp16) into the B-operand buffer of the
//                second product.  The references move lazily: only when some score of a tile exceeds its pair's
//                reference by more than 2^8 does the group take the per-pair maximum over the 128 keys (a butterfly
//                of warp shuffles, then a few words through shared memory) and rescale its columns of O^T in tensor
//                memory; the common tile needs no maximum at all.  The denominator is summed per thread, from the
//                fp16-rounded weights, and reduced once per piece.  The two groups never talk to each other.
//   warps 8-11   K dequant: raw q8_0 records -> exact-integer fp16 K operand [key][dim] (+ the scales, as fp32)
//   warps 12-19  V dequant: raw q8_0 records -> fp16 V^T operand [dim][key], scale folded in
//   warp 20      issues the S^T MMAs; warp 23 the O^T MMAs; warps 21 / 22 stream raw K / V tiles (bulk copies)
// Work cut, split records and the merge kernel are the flash-decode kernel's, in units of 128-key tiles.
// Every wait is bounded; a wait that runs out sets the device status word, the remaining waits are skipped, tensor
// memory is released and the kernel returns.
#pragma once
#include "flash_decode.cuh"
#include "prefill.cuh"

namespace battn {
namespace vt {

using namespace pf;


#ifdef BATTN_VT_TRACE
// debugging aid (not compiled into the library): per-role time stamps of CTA 0
__device__ long long* g_vt_trace = nullptr;
__device__ __forceinline__ long long vt_now() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define VT_TRACE(role, tile, ev) do { if (g_vt_trace && blockIdx.x == 0 && (tile) < 32) g_vt_trace[((role) * 32 + (tile)) * 4 + (ev)] = vt_now(); } while (0)
#else
#define VT_TRACE(role, tile, ev) do { } while (0)
#endif

constexpr int HD = 128, BK = 128, NP = 32;             // head_dim, keys per tile, (row, head) pairs (padded)
constexpr int NBLK = HD / 32, REC = HD + 2 * NBLK;
constexpr int NTHREADS = 768;
constexpr int NPH = NP / 2;                            // pairs per softmax group
constexpr int W_KDQ = 8, W_VDQ = 12, W_MMA = 20, W_LDK = 21, W_LDV = 22, W_PV = 23;
constexpr int REGS_LAUNCH = 80, REGS_SOFT = 120, REGS_DEQ = 64, REGS_CTL = 48;
// Each scheduler hosts two softmax warps, one K dequant warp, two V dequant warps and one control warp, and the
// registers they hold after resizing must fit in what the six warps were launched with: a setmaxnreg.inc that asks
// for more than the others released would wait forever.
static_assert(2 * REGS_SOFT + 3 * REGS_DEQ + REGS_CTL <= 6 * REGS_LAUNCH, "register budget per scheduler");
static_assert(NTHREADS * REGS_LAUNCH <= 65536, "register file");

constexpr int NB = 2;                                   // depth of the operand rings and of the S^T buffers
constexpr int V_SUB = HD * 128;                         // [128 dims][64 keys]
constexpr int V_BYTES = 2 * V_SUB;
constexpr int P_SUB = NP * 128;                         // [32 pairs][64 keys]
constexpr int P_BYTES = 2 * P_SUB;
constexpr int Q_SUB = NP * 128;                         // [32 pairs][64 dims]
constexpr int Q_BYTES = 2 * Q_SUB;
constexpr int RAW_BYTES = BK * REC;
constexpr int OFF_V = 0;
constexpr int OFF_P = OFF_V + NB * V_BYTES;             // two P^T buffers, by tile parity: the softmax of tile j+1 does not wait
constexpr int OFF_Q = OFF_P + 2 * P_BYTES;             // for the P.V product of tile j
constexpr int OFF_RAWK = OFF_Q + Q_BYTES;
constexpr int OFF_RAWV = OFF_RAWK + NB * RAW_BYTES;
constexpr int OFF_KSC = OFF_RAWV + NB * RAW_BYTES;      // [NB][128 keys][4] block scales * softmax scale * log2 e
// per softmax group: [2 parities][4 warps][16] column maxima / sums, [4][16] references, [4][16] alpha, [2][4] flags
constexpr int XCH_GROUP = 2 * 4 * NPH + 4 * NPH + 4 * NPH + 8;
constexpr int OFF_XCH = OFF_KSC + NB * BK * 16;
constexpr int OFF_BAR = OFF_XCH + 2 * XCH_GROUP * 4;
enum { B_KRAW_FULL = 0, B_KRAW_FREE = 2, B_VRAW_FULL = 4, B_VRAW_FREE = 6, B_KF = 8, B_VF = 10, B_S = 12, B_SR = 14,
       B_PV = 16, B_PF = 18, B_Q = 20, N_BARS = 21 };
constexpr int OFF_MISC = OFF_BAR + N_BARS * 8;          // [0] tmem base, [1] abort flag
constexpr int OFF_CUM = OFF_MISC + 16;                  // cum[n_seq + 1]
// tensor-memory columns: O^T (32), NB x 4 x 32 of S^T, then the K operand itself: NB tiles of [128 keys = lanes][128
// dims as 64 columns of fp16 pairs].  The S^T product takes its A operand from there: an MMA whose 4 KB A operand comes
// from shared memory occupied the issue path for 110-150 cycles per instruction (measured), eight of them per tile.
constexpr int T_O = 0, T_S = 32, T_K = T_S + NB * 4 * NP, K_COLS = HD / 2;
static_assert(T_K + NB * K_COLS <= 512, "tensor memory budget");
static_assert(V_SUB % 1024 == 0 && P_SUB % 1024 == 0 && RAW_BYTES % 16 == 0 && OFF_Q % 1024 == 0 &&
              OFF_P % 1024 == 0, "operand alignment");

__host__ __device__ constexpr size_t smem_bytes(int n_seq) { return (size_t)OFF_CUM + (size_t)(n_seq + 2) * 4 + 1024; }

// Column maxima / sums across the 32 lanes of a warp: every lane holds v[0..31] (one value per pair); afterwards
// lane p holds the reduction of v[p] over all lanes.  Five exchange stages, 31 shuffles.
template <bool IS_MAX>
__device__ __forceinline__ float warp_columns(float (&v)[32], int lane) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < off; ++i) {
            const float send = up ? v[i] : v[i + off];
            const float keep = up ? v[i + off] : v[i];
            const float recv = __shfl_xor_sync(0xffffffffu, send, off);
            v[i] = IS_MAX ? fmaxf(keep, recv) : keep + recv;
        }
    }
    return v[0];
}

// The same for 16 values per lane: afterwards lanes 2c and 2c + 1 both hold the reduction of v[c] over all lanes.
template <bool IS_MAX>
__device__ __forceinline__ float warp_columns16(float (&v)[16], int lane) {
#pragma unroll
    for (int off = 16; off >= 2; off >>= 1) {
        const int half = off / 2;
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float send = up ? v[i] : v[i + half];
            const float keep = up ? v[i + half] : v[i];
            const float recv = __shfl_xor_sync(0xffffffffu, send, off);
            v[i] = IS_MAX ? fmaxf(keep, recv) : keep + recv;
        }
    }
    const float o = __shfl_xor_sync(0xffffffffu, v[0], 1);
    return IS_MAX ? fmaxf(v[0], o) : v[0] + o;
}

__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// value of one of 16 registers chosen by a run-time index (a chain of selects: registers cannot be indexed)
__device__ __forceinline__ float pick16(const float (&v)[16], int idx) {
    float r = v[0];
#pragma unroll
    for (int i = 1; i < 16; ++i) r = idx == i ? v[i] : r;
    return r;
}

__global__ void __maxnreg__(REGS_LAUNCH) k_verify_tc(const fd::Params P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);      // 1024-byte aligned
    uint8_t* Vsm = smem + OFF_V;
    uint8_t* Psm = smem + OFF_P;
    uint8_t* Qsm = smem + OFF_Q;
    float* ksc = reinterpret_cast<float*>(smem + OFF_KSC);
    float* xch = reinterpret_cast<float*>(smem + OFF_XCH);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem + OFF_MISC);
    int* cum = reinterpret_cast<int*>(smem + OFF_CUM);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int RG = P.RG;
    constexpr int RS = HD + 4;                               // floats per split record in the workspace

    if (tid == 0) {
        for (int b = 0; b < NB; ++b) {
            mbar_init(&bars[B_KRAW_FULL + b], 1); mbar_init(&bars[B_VRAW_FULL + b], 1);
            mbar_init(&bars[B_KRAW_FREE + b], 4); mbar_init(&bars[B_VRAW_FREE + b], 8);
            mbar_init(&bars[B_KF + b], 4); mbar_init(&bars[B_VF + b], 8);
            mbar_init(&bars[B_S + b], 1); mbar_init(&bars[B_PV + b], 1);
            mbar_init(&bars[B_SR + b], 8);
        }
        mbar_init(&bars[B_PF], 8); mbar_init(&bars[B_PF + 1], 8);
        mbar_init(&bars[B_Q], 8);
        misc[1] = 0;
        mbar_fence_init();
    }
    if (warp == W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(&misc[0]))), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_wait();          // nothing above reads or writes global memory
    pdl_trigger();
    if (P.epoch_ptr && blockIdx.x == 0 && tid == 0) *P.epoch_ptr += P.epoch_advance;
    // ---- the flash-decode work cut in 128-key tiles: every CTA derives the same shares from the positions --------
    for (int i = tid; i < P.n_seq; i += NTHREADS) {
        const SeqRange sr = seq_range(P.pos, P.kslot, P.act, i, P.rows, P.is_swa, P.W, P.slot_ctx, P.n_slots, P.status);
        cum[i + 1] = sr.active ? ((sr.hi + BK - 1) / BK - sr.lo / BK) : 0;
    }
    if (tid == 0) cum[0] = 0;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
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
    const uint32_t tmem = misc[0];
    const int total = P.Hkv * cum[P.n_seq];
    const fd::Share share = fd::cut_share(cum, P.n_seq, P.Hkv, P.cph, (int)blockIdx.x, (int)gridDim.x);
    const int per = share.per;
    if (blockIdx.x == 0) {
        if (tid == 0) { P.hdr[0] = per; P.hdr[1] = total; }
        for (int i = tid; i <= P.n_seq; i += NTHREADS) P.hdr[2 + i] = cum[i];
    }
    const int g0 = share.g0, g1 = share.g1;                                          // empty share: g0 == g1

    // bounded wait that degrades to "do not wait" once any wait has run out
    auto wait = [&](int b, uint32_t parity, uint32_t sleep_ns) {
        if (mbar_try_wait(&bars[b], parity)) return;               // the common case costs one poll
        if (misc[1]) return;
        if (!mbar_wait_backoff(&bars[b], parity, sleep_ns)) {
            atomicOr(P.status, BATTN_DEV_WAIT_TIMEOUT);
            misc[1] = 1;
        }
    };
    auto slot = [](int c) { return c & (NB - 1); };
    auto phase = [](int c) { return (uint32_t)((c / NB) & 1); };

    if (warp >= W_MMA) {
        regs_shrink<REGS_CTL>();
        if (warp == W_MMA && lane == 0) {
            // ======================= S^T = K Q^T, one accumulator per 32-dim block =========================
            const uint32_t idS = umma_idesc(128, NP);
            const uint64_t qd0 = umma_desc(smem_u32(Qsm));
            int cnt = 0, piece = 0;
            for (int g = g0; g < g1; ++piece) {
                const fd::Piece pc = fd::locate(g, g1, cum, P.n_seq, P.Hkv);
                wait(B_Q, piece & 1, 20);                                  // this piece's Q operand is in place
                for (int t = 0; t < pc.n; ++t, ++cnt) {
                    wait(B_KF + slot(cnt), phase(cnt), 20);
                    if (cnt >= NB) wait(B_SR + slot(cnt), phase(cnt - NB), 20);    // softmax has read the old S^T
                    tc_fence_after();
                    VT_TRACE(0, cnt, 0);
                    const uint32_t ka = tmem + T_K + slot(cnt) * K_COLS;           // K tile: lane = key, 8 columns per 16 dims
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks) {
                        const uint64_t qoff = (uint64_t)((ks >> 2) * (Q_SUB >> 4) + 2 * (ks & 3));
                        umma_f16_ts(tmem + T_S + slot(cnt) * 4 * NP + (ks >> 1) * NP, ka + 8 * ks, qd0 + qoff, idS, ks & 1);
                    }
                    umma_commit(&bars[B_S + slot(cnt)]);
                    VT_TRACE(0, cnt, 1);
                }
                g += pc.n;
            }
        } else if (warp == W_PV && lane == 0) {
            // ======================= O^T += V^T P^T ========================================================
            const uint32_t idO = umma_idesc(128, NP);
            const uint64_t vd0 = umma_desc(smem_u32(Vsm)), pd0 = umma_desc(smem_u32(Psm));
            int cnt = 0;
            for (int g = g0; g < g1;) {
                const fd::Piece pc = fd::locate(g, g1, cum, P.n_seq, P.Hkv);
                for (int t = 0; t < pc.n; ++t, ++cnt) {
                    wait(B_PF + (cnt & 1), (cnt >> 1) & 1, 20);
                    wait(B_VF + slot(cnt), phase(cnt), 20);
                    tc_fence_after();
                    const uint64_t vd = vd0 + (uint64_t)(slot(cnt) * (V_BYTES >> 4));
                    const uint64_t pd = pd0 + (uint64_t)((cnt & 1) * (P_BYTES >> 4));
                    VT_TRACE(1, cnt, 0);
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks)
                        umma_f16(tmem + T_O, vd + (uint64_t)((ks >> 2) * (V_SUB >> 4) + 2 * (ks & 3)),
                                 pd + (uint64_t)((ks >> 2) * (P_SUB >> 4) + 2 * (ks & 3)), idO, (t > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(&bars[B_PV + slot(cnt)]);
                    VT_TRACE(1, cnt, 1);
                }
                g += pc.n;
            }
        } else if ((warp == W_LDK || warp == W_LDV) && lane == 0) {
            // ======================= loaders: raw K (or V) tiles with bulk copies ===========================
            const bool isv = warp == W_LDV;
            uint8_t* ring = smem + (isv ? OFF_RAWV : OFF_RAWK);
            const int full = isv ? B_VRAW_FULL : B_KRAW_FULL, free_ = isv ? B_VRAW_FREE : B_KRAW_FREE;
            int cnt = 0;
            for (int g = g0; g < g1;) {
                const fd::Piece pc = fd::locate(g, g1, cum, P.n_seq, P.Hkv);
                const SeqRange sr = seq_range(P.pos, P.kslot, P.act, pc.i, P.rows, P.is_swa, P.W, P.slot_ctx, P.n_slots,
                                              P.status);
                const size_t hb = ((size_t)sr.slot * P.Hkv + pc.kvh) * P.pstride * (size_t)REC;
                const uint8_t* src = isv ? P.kvv : P.kvk;
                const int tile0 = sr.lo / BK + pc.tl;
                // paged cache: the table entry of the next tile is fetched one tile ahead of its use
                const int* trow = P.pg.table ? P.pg.table + (size_t)sr.slot * P.pg.max_pages : nullptr;
                int page_nx = trow ? trow[(tile0 * BK) >> P.pg.shift] : 0;
                for (int t = 0; t < pc.n; ++t, ++cnt) {
                    const int page = page_nx;
                    if (trow && t + 1 < pc.n) page_nx = trow[((tile0 + t + 1) * BK) >> P.pg.shift];
                    if (cnt >= NB) wait(free_ + slot(cnt), phase(cnt - NB), 100);
                    if (misc[1]) continue;
                    VT_TRACE(isv ? 3 : 2, cnt, 0);
                    const int sp = ((tile0 + t) * BK) & P.ring_mask;
                    const int nk = trow ? BK : min(BK, P.pstride - sp);
                    const uint32_t bytes = (uint32_t)nk * REC;
                    const size_t off = trow ? kv_rec_index_page(P.pg, page, pc.kvh, P.Hkv, sp, P.status) * (size_t)REC
                                            : hb + (size_t)sp * REC;
                    mbar_expect_tx(&bars[full + slot(cnt)], bytes);
                    bulk_g2s(ring + slot(cnt) * RAW_BYTES, src + off, bytes, &bars[full + slot(cnt)]);
                }
                g += pc.n;
            }
        }
    } else if (warp >= W_VDQ) {
        // ======================= V dequant warps: V^T operand, [dim][key], scale folded in ======================
        regs_shrink<REGS_DEQ>();
        const int t = tid - W_VDQ * 32;                         // 0..255
        const int kh = t >> 7, wq = (t >> 5) & 3;               // key half (64 keys), warp within the half
        constexpr int NWG = HD / 16;                            // groups of four dim-words
        constexpr int UPT = 2;                                  // micro-tiles (4 dims x 8 keys) per thread
        const int cc = lane & 7, wl = lane >> 3;                // key chunk (8 keys) inside the half, fixed per thread
        int vkey[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) vkey[jj] = 64 * kh + kappa(8 * cc + jj);
        int cnt = 0;
        for (int g = g0; g < g1;) {
            const fd::Piece pc = fd::locate(g, g1, cum, P.n_seq, P.Hkv);
            const SeqRange sr = seq_range(P.pos, P.kslot, P.act, pc.i, P.rows, P.is_swa, P.W, P.slot_ctx, P.n_slots, P.status);
            const int tile0 = sr.lo / BK + pc.tl;
            for (int tt = 0; tt < pc.n; ++tt, ++cnt) {
                const int t0 = (tile0 + tt) * BK;
                const uint8_t* Vraw = smem + OFF_RAWV + slot(cnt) * RAW_BYTES;
                wait(B_VRAW_FULL + slot(cnt), phase(cnt), 50);
                if (t == 0) VT_TRACE(4, cnt, 0);
                if (cnt >= NB) wait(B_PV + slot(cnt), phase(cnt - NB), 50);       // the product that read this buffer is done
                if (t == 0) VT_TRACE(4, cnt, 1);
                uint8_t* Vdst = Vsm + slot(cnt) * V_BYTES + kh * V_SUB;
                // keys outside [lo, hi) were never written for this sequence: their bytes are arbitrary, so
                // their scale is forced to zero (their P is zero as well)
                bool kok[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) kok[jj] = (t0 + vkey[jj] >= sr.lo) && (t0 + vkey[jj] < sr.hi);
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
                    for (int i = 0; i < 4; ++i)
                        *reinterpret_cast<uint4*>(Vdst + sw128(4 * w + i, cc)) =
                            make_uint4(chunk[i][0], chunk[i][1], chunk[i][2], chunk[i][3]);
                }
                proxy_fence();
                __syncwarp();
                if (lane == 0) { mbar_arrive(&bars[B_VF + slot(cnt)]); mbar_arrive(&bars[B_VRAW_FREE + slot(cnt)]); }
                if (t == 0) VT_TRACE(4, cnt, 2);
            }
            g += pc.n;
        }
    } else if (warp >= W_KDQ) {
        // ======================= K dequant warps: exact-integer K operand [key][dim] + fp32 scales ================
        regs_shrink<REGS_DEQ>();
        const int krow = tid - W_KDQ * 32;                      // operand row = TMEM lane of S^T, 0..127
        const int kkey = kappa(krow);                           // the key it holds
        int cnt = 0;
        for (int g = g0; g < g1;) {
            const fd::Piece pc = fd::locate(g, g1, cum, P.n_seq, P.Hkv);
            for (int tt = 0; tt < pc.n; ++tt, ++cnt) {
                const uint8_t* src = smem + OFF_RAWK + slot(cnt) * RAW_BYTES + kkey * REC;
                wait(B_KRAW_FULL + slot(cnt), phase(cnt), 50);
                if (krow == 0) VT_TRACE(5, cnt, 0);
                // the S^T product that read this K buffer (tile cnt - NB) is complete once the softmax warps have
                // signalled that they read its result
                if (cnt >= NB) wait(B_SR + slot(cnt), phase(cnt - NB), 50);
                const uint32_t kt = tmem + ((uint32_t)((warp & 3) * 32) << 16) + T_K + slot(cnt) * K_COLS;
                if (krow == 0) VT_TRACE(5, cnt, 1);
                {
                    const uint2 sc = *reinterpret_cast<const uint2*>(src);
                    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sc.x));
                    const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sc.y));
                    *reinterpret_cast<float4*>(ksc + (slot(cnt) * BK + krow) * 4) =
                        make_float4(s01.x * P.scale_log2, s01.y * P.scale_log2, s23.x * P.scale_log2, s23.y * P.scale_log2);
                }
                // the key's 128 exact integers as 64 columns of fp16 pairs in this thread's tensor-memory lane, 16 at a time
#pragma unroll 1
                for (int g4 = 0; g4 < HD / 32; ++g4) {
                    uint32_t col[16];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint2 w = *reinterpret_cast<const uint2*>(src + 2 * NBLK + (4 * g4 + c) * 8);
                        const uint32_t x = w.x ^ 0x80808080u, y = w.y ^ 0x80808080u;
                        col[4 * c] = sub1152(widen_lo(x)); col[4 * c + 1] = sub1152(widen_hi(x));
                        col[4 * c + 2] = sub1152(widen_lo(y)); col[4 * c + 3] = sub1152(widen_hi(y));
                    }
                    tmem_st16(kt + 16 * g4, col);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { mbar_arrive(&bars[B_KF + slot(cnt)]); mbar_arrive(&bars[B_KRAW_FREE + slot(cnt)]); }
                if (krow == 0) VT_TRACE(5, cnt, 2);
            }
            g += pc.n;
        }
    } else {
        // ======================= softmax warps: a thread owns one key of every tile and half of the pairs ==========
        regs_grow<REGS_SOFT>();
        const int gp = warp >> 2, wq = warp & 3;               // pair group, TMEM lane quarter
        const int n = wq * 32 + lane;                          // TMEM lane = operand row, 0..127
        const int pbase = gp * NPH;                            // first pair of this group
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const int kkey = kappa(n);
        const int bar_a = 1 + 2 * gp, bar_b = 2 + 2 * gp;      // this group's named barriers
        float* gx = xch + gp * XCH_GROUP;
        // [2][4][16] per-warp column maxima / sums, double-buffered by tile parity: a warp that runs ahead writes the
        // other half, and cannot reach this half again before the whole group has passed the next tile's barrier
        float* colx2 = gx;
        float* refx = gx + 8 * NPH + wq * NPH;                 // this warp's row: new references (log2 units)
        float* alphx = gx + 12 * NPH + wq * NPH;               // this warp's row: rescale factors
        float* flagx = gx + 16 * NPH;                          // [2][4] "some score outgrew its reference", per tile parity
        const int mycol = lane >> 1;                           // the pair (within the group) this lane decides for
        int cnt = 0, piece = 0;
        for (int g = g0; g < g1; ++piece) {
            const fd::Piece pc = fd::locate(g, g1, cum, P.n_seq, P.Hkv);
            const SeqRange sr = seq_range(P.pos, P.kslot, P.act, pc.i, P.rows, P.is_swa, P.W, P.slot_ctx, P.n_slots, P.status);
            const int item = pc.i * P.Hkv + pc.kvh;
            // ---- this item's Q as the B operand [pair][dim]: a thread writes 16 bytes of two pairs ----------------
            // (the previous piece's last S^T product has completed: these threads consumed its result)
            {
                const int idx = gp * 128 + n;                  // 0..255
                const int pr0 = idx >> 4, ch2 = idx & 15;      // pairs pr0 and pr0 + 16, chunk of 8 dims
#pragma unroll
                for (int k2 = 0; k2 < 2; ++k2) {
                    const int pr = pr0 + 16 * k2;
                    uint4 val = make_uint4(0u, 0u, 0u, 0u);
                    if (pr < RG) {
                        const int r = pr / P.G, h = pr - r * P.G;
                        const size_t qi = (((size_t)pc.i * P.rows + r) * P.Hq + pc.kvh * P.G + h) * HD + ch2 * 8;
                        if (P.q_f16) {
                            val = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(P.q) + qi);
                        } else {
                            const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.q) + qi);
                            const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.q) + qi + 4);
                            val = make_uint4(pack_h2(a.x, a.y), pack_h2(a.z, a.w), pack_h2(b.x, b.y), pack_h2(b.z, b.w));
                        }
                    }
                    *reinterpret_cast<uint4*>(Qsm + (ch2 >> 3) * Q_SUB + sw128(pr, ch2 & 7)) = val;
                }
                proxy_fence();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[B_Q]);
            }
            const int full_lo = P.is_swa ? max(0, sr.p0 + P.rows - P.W) : 0;      // window start of the last row
            // References (log2 units), one per pair, held by EVERY thread of the group.  A reference moves only when
            // some score of a tile exceeds it by more than 2^8 (then to that tile's maximum): weights stay below 2^8,
            // well inside fp16, and on the common tile each thread only checks its own differences.
            float ref[NPH];
            float lsum[NPH];                                   // this thread's key: sum of its weights per pair
#pragma unroll
            for (int i = 0; i < NPH; ++i) { ref[i] = NEG_BIG; lsum[i] = 0.f; }
            // shared-memory addresses of this thread's key column inside the P^T rows, per row-in-atom (128-byte swizzle)
            uint32_t pcol[8];
            {
                const int kc = (n & 63) >> 3, kb = (n & 7) * 2;
#pragma unroll
                for (int r8 = 0; r8 < 8; ++r8)
                    pcol[r8] = smem_u32(Psm) + (n >> 6) * P_SUB + (pbase >> 3) * 1024 + (((kc ^ r8) & 7) << 4) + kb;
            }

            const int tile0 = sr.lo / BK + pc.tl;
            for (int t = 0; t < pc.n; ++t, ++cnt) {
                const int t0 = (tile0 + t) * BK;
                const bool masked = !(t0 >= full_lo && t0 + BK - 1 <= sr.p0);
                wait(B_S + slot(cnt), phase(cnt), 30);
                tc_fence_after();
                if (tid == 0) VT_TRACE(6, cnt, 0);
                // ---- scores of this key against the group's 16 pairs: four block partials, scaled in fp32 -----------
                float v[NPH];
                {
                    const float4 sc = *reinterpret_cast<const float4*>(ksc + (slot(cnt) * BK + n) * 4);
                    const uint32_t tS = tmem + lane_base + T_S + slot(cnt) * 4 * NP + pbase;
                    uint32_t a[NPH], b[NPH], c[NPH], d[NPH];
                    tmem_ld16_nowait(tS, a);
                    tmem_ld16_nowait(tS + NP, b);
                    tmem_ld16_nowait(tS + 2 * NP, c);
                    tmem_ld16_nowait(tS + 3 * NP, d);
                    tmem_ld_wait();
                    // two pairs per instruction (fma.rn.f32x2): the same products and sums, in the same order
                    const uint64_t sx = pack_f2(sc.x, sc.x), sy = pack_f2(sc.y, sc.y), sz = pack_f2(sc.z, sc.z), sw = pack_f2(sc.w, sc.w);
#pragma unroll
                    for (int i = 0; i < NPH; i += 2) {
                        uint64_t t;
                        asm("{\n\t.reg .b64 x;\n\tmov.b64 x, {%1, %2};\n\tmul.rn.f32x2 %0, x, %3;\n\t}" : "=l"(t) : "r"(a[i]), "r"(a[i + 1]), "l"(sx));
                        asm("{\n\t.reg .b64 x;\n\tmov.b64 x, {%1, %2};\n\tfma.rn.f32x2 %0, x, %3, %0;\n\t}" : "+l"(t) : "r"(b[i]), "r"(b[i + 1]), "l"(sy));
                        asm("{\n\t.reg .b64 x;\n\tmov.b64 x, {%1, %2};\n\tfma.rn.f32x2 %0, x, %3, %0;\n\t}" : "+l"(t) : "r"(c[i]), "r"(c[i + 1]), "l"(sz));
                        asm("{\n\t.reg .b64 x;\n\tmov.b64 x, {%1, %2};\n\tfma.rn.f32x2 %0, x, %3, %0;\n\t}" : "+l"(t) : "r"(d[i]), "r"(d[i + 1]), "l"(sw));
                        asm("mov.b64 {%0, %1}, %2;" : "=f"(v[i]), "=f"(v[i + 1]) : "l"(t));
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[B_SR + slot(cnt)]);           // S^T buffer (and its K operand) released
                if (tid == 0) VT_TRACE(6, cnt, 1);
                if (__builtin_expect(masked, 0)) {
                    // hidden keys score minus infinity (a true one: it stays hidden against every reference)
                    const int key = t0 + kkey;
#pragma unroll
                    for (int i = 0; i < NPH; ++i) {                    // (i / G folds to a shift per pair for G = 4)
                        const int r = min((pbase + i) / P.G, P.rows - 1);
                        const int lim = sr.p0 + r;                                         // bruce.cu:2056
                        const int low = P.is_swa ? max(0, sr.p0 + r + 1 - P.W) : 0;        // bruce.cu:3688
                        if (key > lim || key < low) v[i] = -INFINITY;
                    }
                }
                // ---- does any score of the tile outgrow its reference?  (own differences, then a vote) --------------
                float dv[NPH];                                     // score minus reference: the exponent of the weight
#pragma unroll
                for (int i = 0; i < NPH; ++i) dv[i] = v[i] - ref[i];
                float dmax = fmax3(dv[0], dv[1], dv[2]);
#pragma unroll
                for (int i = 3; i + 1 < NPH; i += 2) dmax = fmax3(dmax, dv[i], dv[i + 1]);
                dmax = fmaxf(dmax, dv[NPH - 1]);
                const bool over = __any_sync(0xffffffffu, dmax > RESCALE_THRESHOLD);
                if (lane == 0) flagx[(cnt & 1) * 4 + wq] = over ? 1.f : 0.f;
                named_bar_sync(bar_a, 128);
                const float4 fl = *reinterpret_cast<const float4*>(flagx + (cnt & 1) * 4);
                if (__builtin_expect(fl.x + fl.y + fl.z + fl.w > 0.f, 0)) {
                    // ---- rare: per-pair maximum over the 128 keys, new references, O^T and the sums rescaled -----------
                    float* colx = colx2 + (cnt & 1) * 4 * NPH;
                    float w[NPH];
#pragma unroll
                    for (int i = 0; i < NPH; ++i) w[i] = v[i];
                    const float cmax = warp_columns16<true>(w, lane);
                    colx[wq * NPH + mycol] = cmax;
                    named_bar_sync(bar_b, 128);
                    // lanes 2c and 2c + 1 decide for pair c; every warp computes the same from the same words
                    const float tmax = fmaxf(fmaxf(colx[mycol], colx[NPH + mycol]), fmaxf(colx[2 * NPH + mycol], colx[3 * NPH + mycol]));
                    const float myref = pick16(ref, mycol);
                    const bool need = tmax > myref + RESCALE_THRESHOLD;
                    const float newref = need ? tmax : myref;
                    // this warp's rows of the exchange area: new references and rescale factors 2^(old - new)
                    refx[mycol] = newref;
                    alphx[mycol] = need ? fast_exp2(myref - newref) : 1.f;         // 0 for a first reference
                    __syncwarp();
                    if (t > 0) {
                        wait(B_PV + slot(cnt - 1), phase(cnt - 1), 30);          // O^T complete before it is rescaled
                        tc_fence_after();
                    }
                    float al[NPH];
#pragma unroll
                    for (int i = 0; i < NPH; i += 4) {
                        const float4 a4 = *reinterpret_cast<const float4*>(alphx + i);
                        const float4 r4 = *reinterpret_cast<const float4*>(refx + i);
                        al[i] = a4.x; al[i + 1] = a4.y; al[i + 2] = a4.z; al[i + 3] = a4.w;
                        ref[i] = r4.x; ref[i + 1] = r4.y; ref[i + 2] = r4.z; ref[i + 3] = r4.w;
                    }
#pragma unroll
                    for (int i = 0; i < NPH; ++i) lsum[i] *= al[i];
                    if (t > 0) {
                        uint32_t o[NPH];
                        tmem_ld16_nowait(tmem + lane_base + T_O + pbase, o);       // lane = dim (this warp's quarter), column = pair
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < NPH; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * al[i]);
                        tmem_st16(tmem + lane_base + T_O + pbase, o);
                        tmem_st_wait();
                        tc_fence_before();
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < NPH; ++i) dv[i] = v[i] - ref[i];           // against the new references
                }
                // ---- P^T = 2^(s - ref), fp16, into the B operand [pair][key]; the sums take the rounded weights ----
                // the product that read this P buffer (two tiles ago) must be complete
                if (cnt >= 2) wait(B_PV + slot(cnt - 2), phase(cnt - 2), 30);
                const uint32_t poff = (uint32_t)((cnt & 1) * P_BYTES);
                if (tid == 0) VT_TRACE(6, cnt, 2);
#pragma unroll
                for (int i = 0; i < NPH; i += 2) {
                    const uint32_t ph = pack_h2(fast_exp2(dv[i]), fast_exp2(dv[i + 1]));
                    // the two fp16 weights back as fp32 without the conversion unit: the half's bits moved into an fp32
                    // word, times 2^112 (exact for every non-negative half, subnormals included)
                    lsum[i] = fmaf(__uint_as_float((ph << 13) & 0x0FFFE000u), 5.192296858534828e33f, lsum[i]);
                    lsum[i + 1] = fmaf(__uint_as_float((ph >> 3) & 0x0FFFE000u), 5.192296858534828e33f, lsum[i + 1]);
                    asm volatile("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\t"
                                 "st.shared.b16 [%0], lo;\n\tst.shared.b16 [%1], hi;\n\t}"
                                 ::"r"(pcol[i & 7] + poff + (uint32_t)((i >> 3) * 1024 + (i & 7) * 128)),
                                   "r"(pcol[(i + 1) & 7] + poff + (uint32_t)(((i + 1) >> 3) * 1024 + ((i + 1) & 7) * 128)), "r"(ph)
                                 : "memory");
                }
                proxy_fence();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[B_PF + (cnt & 1)]);
                if (tid == 0) VT_TRACE(6, cnt, 3);
            }

            // ---- piece end: O^T, the references and the sums become this item's split record -----------------------
            if (pc.n > 0) {
                wait(B_PV + slot(cnt - 1), phase(cnt - 1), 30);
                tc_fence_after();
            }
            const float myref = pick16(ref, mycol);
            const float csum = warp_columns16<false>(lsum, lane);
            named_bar_sync(bar_a, 128);                              // the last tile's words have been read
            float* colx = colx2;
            colx[wq * NPH + mycol] = csum;
            named_bar_sync(bar_b, 128);
            float* dst = P.part + (size_t)(blockIdx.x + item) * RG * RS;
            if (wq == 0 && (lane & 1) == 0 && pbase + mycol < RG) {
                const float L = colx[mycol] + colx[NPH + mycol] + colx[2 * NPH + mycol] + colx[3 * NPH + mycol];
                *reinterpret_cast<float2*>(dst + (size_t)(pbase + mycol) * RS + HD) = make_float2(myref, L);
            }
            {
                uint32_t o[NPH];
                tmem_ld16_nowait(tmem + lane_base + T_O + pbase, o);     // lane = dim n, column = pair
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < NPH; ++i)
                    if (pbase + i < RG) dst[(size_t)(pbase + i) * RS + n] = __uint_as_float(o[i]);
            }
            tc_fence_before();
            named_bar_sync(bar_a, 128);                              // sums read before the next piece reuses the words
            g += pc.n;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace vt
}  // namespace battn
