// Shared declarations of the attention library: geometry, the handle, PTX helpers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/battn.h"

namespace battn {

constexpr int MAX_SEQ        = 1024;  // sequences per call (the reference stops at 8, bruce.cu:93-94)
constexpr int MAX_VERIFY     = 8;     // rows sharing one KV sweep (bruce.cu:94)
constexpr int MAX_PREFILL    = 512;   // rows per prompt chunk (MBUF, bruce.cu:1058)
constexpr int MAX_SPLITS     = 128;   // PART_MAX_SPLITS (bruce.cu:1059)
constexpr float NEG_BIG      = -1e30f;  // "minus infinity" of the reference (bruce.cu:737)
constexpr float LOG2E        = 1.4426950408889634f;
constexpr float LN2          = 0.6931471805599453f;

struct Geom {
    int Hq, Hkv, HD, G;      // query heads, KV heads, head dim, heads per KV head
    int W, ring;             // window and ring slots (2*W)
    int slot_ctx, n_slots;
    int rec, nblk;           // record bytes, 32-value blocks per record
    int q_f16, out_f16;
    float scale;
};

}  // namespace battn

struct battn_handle {
    battn::Geom g;
    int device;
    int num_sms;
    int* d_status;           // device status word (bits BATTN_DEV_*)
    int last_cuda_error;
    long long launches;
    cudaEvent_t* prof_ev;    // 2 * prof_cap events while profiling, else null
    int prof_cap, prof_n;
    void* noalloc_ws;        // device address of the library's built-in scratch array on this device
    int vw_ctas_per_sm;      // resident CTAs per SM of the wide verify kernel
    int fd_ctas_per_sm[3];   // resident CTAs per SM of the flash-decode kernel, per NT in {1,2}
    int fd_smem[3];
    // Early KV streaming of the decode kernels (see fd::Params::early): allowed for a call when the last launch on
    // this handle wrote no cache rows other than the call's own (kvw_kind 0: none, 1: rows_per_seq rows at kvw_pos of
    // n_seq sequences, 2: anything else, 3: the appending decode call wrote one row per sequence into kvw_cache -- its
    // merge releases the next launch before that decode kernel has finished; the flash-decode kernel never streams
    // the tile of the row before its own early, the other kernels stream early only from a different cache).
    int early_stream;
    int kvw_kind, kvw_nseq, kvw_rows;
    const int* kvw_pos;
    const void* kvw_cache;
};

// Receive area of one device in a sequence split (see XchgView in exact.cuh) and its mappings of the peers' areas.
struct battn_xchg {
    battn_handle* h;
    int world, rank, max_items;
    size_t rec_bytes, bytes;          // the receive area: records whose words carry their step number
    void* area[8];                    // area[d]: device d's receive area as mapped into this process
    bool ipc_opened[8];
    unsigned wait_polls;
};

namespace battn {

// ---- small device helpers ---------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// [x.b0, 0x64, x.b1, 0x64] / [x.b2, 0x64, x.b3, 0x64]: two bytes widened to fp16 1024+u
__device__ __forceinline__ uint32_t widen_lo(uint32_t x) { return __byte_perm(x, 0x64646464u, 0x4140); }
__device__ __forceinline__ uint32_t widen_hi(uint32_t x) { return __byte_perm(x, 0x64646464u, 0x4342); }

// half2 (1024 + (b ^ 0x80)) - 1152 == exact int8 value b, the integer step of the reference's
// dequant_i8x4_to_h2 (bruce.cu:2225-2237)
__device__ __forceinline__ uint32_t sub1152(uint32_t h2) {
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h2), __float2half2_rn(1152.0f));
    return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// a * b - p with one rounding, p = the fp16-rounded product a * b: the exact rounding error of that product
// (an 8-bit integer times an 11-bit scale has 19 significant bits; the residual fits fp16 exactly)
__device__ __forceinline__ uint32_t hfma2_residual(uint32_t a, uint32_t b, uint32_t p) {
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b),
                              __hneg2(*reinterpret_cast<const __half2*>(&p)));
    return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 8x8 b16 transpose across the warp: thread (gid, t4) holds M[gid][2t4..2t4+1] and receives
// M[2t4][gid], M[2t4+1][gid]
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}

// ---- mbarrier + bulk copy (TMA, untiled) -------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls and reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Bounded wait with back-off: idle roles sleep between polls instead of flooding the issue slots and the
// shared-memory pipe that the working warps need.
__device__ __forceinline__ bool mbar_wait_backoff(uint64_t* bar, uint32_t parity, uint32_t sleep_ns = 100,
                                                  uint32_t limit = (1u << 22)) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < limit; ++i) {
        __nanosleep(sleep_ns);
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
// global -> shared bulk copy; dst, src 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialisation attribute may start
// while its predecessor in the stream is still draining.  pdl_wait() blocks until the predecessor has
// completed and its writes are visible (a no-op for an ordinary launch); everything before it must not
// touch global memory.  pdl_trigger() lets the successor begin its own launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- paged cache ------------------------------------------------------------------------------------
// A full-causal layer's cache can be a pool of pages instead of one contiguous partition per slot (the reference
// carves contiguous ctx/N partitions, bruce.cu:5471-5503): a page holds 2^shift consecutive positions of every kv
// head, laid out [kv head][position][record], so a 64- or 128-key tile of one head is still one contiguous run.
// Row `slot` of the device-resident table maps logical page (pos >> shift) to a physical page.  Sequences that
// share a prefix point at the same physical pages.  table == nullptr: the contiguous partitions.
struct Paging {
    const int* table = nullptr;
    int max_pages = 0, shift = 0, n_pages = 0;
};
// index, in records, of position `sp` (already reduced modulo the ring on a window layer) of (slot, kv head)
__device__ __forceinline__ size_t kv_rec_index_page(const Paging& pg, int page, int kvh, int Hkv, int sp, int* status) {
    if ((unsigned)page >= (unsigned)pg.n_pages) {          // a table entry outside the pool: flag it, stay in bounds
        atomicOr(status, BATTN_DEV_BAD_POSITION);
        page = 0;
    }
    return ((((size_t)page * Hkv + kvh) << pg.shift) | (size_t)(sp & ((1 << pg.shift) - 1)));
}
__device__ __forceinline__ size_t kv_rec_index(const Paging& pg, int slot, int kvh, int Hkv, int pstride, int sp,
                                               int* status) {
    if (!pg.table) return ((size_t)slot * Hkv + kvh) * pstride + sp;
    return kv_rec_index_page(pg, pg.table[(size_t)slot * pg.max_pages + (sp >> pg.shift)], kvh, Hkv, sp, status);
}

// ---- per-sequence key range ---------------------------------------------------------------------
// Sequence i with `rows` query rows at p0 .. p0+rows-1: union of the rows' visible keys is
// [lo, hi), lo = is_swa ? max(0, p0 + 1 - W) : 0, hi = p0 + rows  (bruce.cu:724-727, 3670-3675).
struct SeqRange {
    int p0, lo, hi, slot;
    bool active;
};

__device__ __forceinline__ SeqRange seq_range(const int* __restrict__ pos, const int* __restrict__ kslot,
                                              const int* __restrict__ act, int i, int rows, int is_swa, int W,
                                              int slot_ctx, int n_slots, int* status) {
    SeqRange s;
    s.active = act ? (act[i] != 0) : true;
    s.slot = kslot ? kslot[i] : 0;
    s.p0 = pos[i];
    s.lo = is_swa ? max(0, s.p0 + 1 - W) : 0;
    s.hi = s.p0 + rows;
    if (s.active) {
        const bool bad = s.p0 < 0 || (!is_swa && s.hi > slot_ctx) || s.slot < 0 || (kslot && s.slot >= n_slots);
        if (bad) {
            atomicOr(status, BATTN_DEV_BAD_POSITION);
            s.active = false;
        }
    }
    if (!s.active) { s.lo = 0; s.hi = 0; }
    return s;
}

}  // namespace battn
