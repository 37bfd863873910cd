// C ABI of the attention library (see include/battn.h): argument checks, launch geometry, dispatch.
// No allocation, synchronisation or host read of device state happens inside the per-step entry
// points, so they can be recorded into CUDA graphs like the reference's launches
// (engine/src/bruce.cu:7877-7900, 8046-8055).
#include <algorithm>
#include <cstring>
#include <new>

#include "common.cuh"
#include "exact.cuh"
#include "flash_decode.cuh"
#include "gate_norm.cuh"
#include "kv_append.cuh"
#include "qkv_prep.cuh"
#include "prefill.cuh"
#include "prefill_hd128.cuh"
#include "verify.cuh"
#include "verify_tc.cuh"

using namespace battn;

#ifndef BATTN_PF_PAIR
#define BATTN_PF_PAIR 1
#endif

namespace {

// The wait self-test: thread 0 waits on an mbarrier that has one pending arrival nobody will make.
__global__ void k_wait_selftest(int* status, uint32_t limit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        if (!mbar_wait_bounded(&bar, 0, limit)) atomicOr(status, BATTN_DEV_WAIT_TIMEOUT);
    }
}

constexpr size_t SMEM_MAX = 226 * 1024;     // dynamic shared memory per CTA: the 227 KB opt-in limit of sm_100
                                            // minus room for the kernels' static shared variables
int g_init_cuda_error = 0;                  // cudaError_t of the last failing battn_init
constexpr int FD_MAX_CTAS_PER_SM = 4;

// Built-in split-K scratch of battn_decode_noalloc: part of the library image, one copy per device that
// loads it.  In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
__device__ __align__(256) unsigned char g_noalloc_scratch[BATTN_NOALLOC_SCRATCH_BYTES];

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline int cuda_fail(battn_handle* h, cudaError_t e) {
    h->last_cuda_error = (int)e;
    return BATTN_ERR_CUDA;
}

inline int nt_index(int RG) { return RG <= 8 ? 0 : (RG <= 16 ? 1 : 2); }

template <int HD, int NT>
cudaError_t fd_prepare(battn_handle* h, int idx) {
    auto kern = fd::k_flash_decode<HD, NT>;
    cudaError_t e = cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
    if (e != cudaSuccess) return e;
    int nb = 0;
    const size_t sm = fd::smem_bytes<HD, NT>(NT * 8, 1);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, (const void*)kern, fd::NTHREADS, sm);
    if (e != cudaSuccess) return e;
    h->fd_ctas_per_sm[idx] = nb < 1 ? 1 : (nb > FD_MAX_CTAS_PER_SM ? FD_MAX_CTAS_PER_SM : nb);
    h->fd_smem[idx] = (int)sm;
    return cudaSuccess;
}

template <int HD>
cudaError_t vw_prepare(battn_handle* h) {
    auto kern = vw::k_verify_wide<HD>;
    cudaError_t e = cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
    if (e != cudaSuccess) return e;
    int nb = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, (const void*)kern, vw::NTHREADS, vw::smem_bytes<HD>(1));
    if (e != cudaSuccess) return e;
    h->vw_ctas_per_sm = nb < 1 ? 1 : (nb > FD_MAX_CTAS_PER_SM ? FD_MAX_CTAS_PER_SM : nb);
    return cudaSuccess;
}

template <int HD>
cudaError_t fd_prepare_all(battn_handle* h) {
    cudaError_t e;
    if ((e = vw_prepare<HD>(h)) != cudaSuccess) return e;
    if (HD == 128) {
        e = cudaFuncSetAttribute((const void*)vt::k_verify_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (e != cudaSuccess) return e;
    }
    if (HD == 128) {
        e = cudaFuncSetAttribute((const void*)pf128::k_prefill_hd128<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf128::TOTAL);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute((const void*)pf128::k_prefill_hd128<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf128::TOTAL_PAIR);
    }
    else           e = cudaFuncSetAttribute((const void*)pf::k_prefill<256, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf::Cfg<256, 64>::TOTAL);
    if (e != cudaSuccess) return e;
    if ((e = fd_prepare<HD, 1>(h, 0)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute((const void*)fd::k_flash_decode<HD, 1, 1>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute((const void*)fd::k_flash_decode<HD, 1, 2>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX)) != cudaSuccess) return e;
    if ((e = fd_prepare<HD, 2>(h, 1)) != cudaSuccess) return e;
    return cudaSuccess;
}

// workspace of the flash-decode path: header + one record slot per (CTA + item)
struct FdWs {
    size_t hdr_bytes, rec_bytes, total;
    int max_ctas;
};
inline FdWs fd_workspace(const battn_handle* h, int n_seq, int rows) {
    const Geom& g = h->g;
    FdWs w;
    w.max_ctas = h->num_sms * FD_MAX_CTAS_PER_SM;
    w.hdr_bytes = align_up((size_t)(n_seq + 3) * sizeof(int), 256);
    w.rec_bytes = (size_t)(w.max_ctas + (size_t)n_seq * g.Hkv) * rows * g.G * (g.HD + 4) * sizeof(float);
    w.total = w.hdr_bytes + w.rec_bytes;
    return w;
}

inline int exact_default_splits(int rows) { return rows > 64 ? 2 : (rows > 8 ? 8 : 32); }

// Key splits of the prompt kernel: its grid is (M tiles) x (kv heads), which leaves SMs idle for short chunks and
// for few kv heads (64 CTAs for a 512-row chunk in the 16/4/256 geometry); each (M tile, kv head) is then shared by several CTAs that take
// contiguous shares of the key tiles and leave split records for the merge kernel.  Positions are device-resident,
// so the choice depends on the chunk shape only.
inline int prefill_splits(const battn_handle* h, int rows, int is_swa) {
    const Geom& g = h->g;
    const int ctas = ((rows + 128 / g.G - 1) / (128 / g.G)) * g.Hkv;
    int s = h->num_sms / ctas;
    // a share should keep at least 16 key tiles of 64, or the merge costs more than the split saves; a
    // sliding-window layer never has more than window/64 + 1 tiles per M tile
    if (is_swa && s > g.W / (64 * 16)) s = g.W / (64 * 16);
    return s < 1 ? 1 : (s > 8 ? 8 : s);
}

inline size_t exact_workspace(const battn_handle* h, int n_seq, int rows, int nsplit) {
    const Geom& g = h->g;
    return (size_t)n_seq * rows * g.Hq * nsplit * (g.HD + 2) * sizeof(float);
}

// split records of a prompt chunk of `rows` rows (full-attention layers take at least as many splits as
// sliding-window layers)
inline size_t prefill_workspace(const battn_handle* h, int rows) {
    return exact_workspace(h, 1, rows, prefill_splits(h, rows, 0));
}

int check_seq_args(const battn_handle* h, const void* a, const void* b, const void* c, const void* d,
                   const int* pos, const int* kslot, int n_seq, int rows, int max_rows) {
    if (!h || !a || !b || !c || !d || !pos) return BATTN_ERR_ARG;
    // every data pointer is read or written with 16-byte accesses (float4 / uint4 loads, bulk copies)
    if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d) & 15) != 0) return BATTN_ERR_ARG;
    if (n_seq < 1 || rows < 1) return BATTN_ERR_ARG;
    if (!kslot && n_seq != 1) return BATTN_ERR_ARG;
    if (n_seq > MAX_SEQ || rows > max_rows) return BATTN_ERR_CAPACITY;
    return BATTN_OK;
}

// Launch with the programmatic-stream-serialisation attribute: the kernel may begin launching while the
// previous kernel of the stream drains; it calls pdl_wait() before it touches global memory.
template <typename Params>
cudaError_t launch_pdl(void (*kernel)(const Params), dim3 grid, dim3 block, size_t smem, cudaStream_t st, const Params& p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

// event pair around the main kernel of a call while profiling is on
struct ProfScope {
    battn_handle* h; cudaStream_t st; int idx;
    ProfScope(battn_handle* h_, cudaStream_t st_) : h(h_), st(st_), idx(-1) {
        if (h->prof_ev && h->prof_n < h->prof_cap) { idx = h->prof_n++; cudaEventRecord(h->prof_ev[2 * idx], st); }
    }
    ~ProfScope() { if (idx >= 0) cudaEventRecord(h->prof_ev[2 * idx + 1], st); }
};

// a caller's paged cache, validated: the device-side view plus what replaces the contiguous geometry
struct PagedView {
    Paging pg;
    int n_tables, capacity;          // table rows; positions one row can hold
};
int paged_view(const battn_pages* pages, PagedView& v) {
    if (!pages || !pages->pool_k || !pages->pool_v || !pages->table) return BATTN_ERR_ARG;
    if ((((uintptr_t)pages->pool_k | (uintptr_t)pages->pool_v) & 15) || ((uintptr_t)pages->table & 3)) return BATTN_ERR_ARG;
    const int L = pages->page_len;
    if (L < 128 || L > 65536 || (L & (L - 1))) return BATTN_ERR_ARG;        // whole 128-key tiles per page
    if (pages->n_pages < 1 || pages->n_tables < 1 || pages->max_pages < 1) return BATTN_ERR_ARG;
    if ((long long)pages->max_pages * L > 0x7fffffffLL) return BATTN_ERR_CAPACITY;
    int shift = 0;
    while ((1 << shift) < L) ++shift;
    v.pg.table = pages->table; v.pg.max_pages = pages->max_pages; v.pg.shift = shift; v.pg.n_pages = pages->n_pages;
    v.n_tables = pages->n_tables; v.capacity = pages->max_pages * L;
    return BATTN_OK;
}
// overrides the contiguous-partition fields of a kernel's parameters with the paged view
template <typename P_>
void apply_paging(P_& P, const PagedView* pv) {
    if (!pv) return;
    P.pg = pv->pg; P.pstride = pv->capacity; P.ring_mask = -1; P.slot_ctx = pv->capacity;
}

int launch_exact(battn_handle* h, void* out, float* rec_out, const void* q, const uint8_t* kvk, const uint8_t* kvv,
                 const int* pos, const int* kslot, const int* act, void* ws, int n_seq, int rows, int nsplit,
                 int is_swa, cudaStream_t st, const PagedView* pv = nullptr) {
    const Geom& g = h->g;
    ExactParams P;
    P.q = q; P.kvk = kvk; P.kvv = kvv; P.pos = pos; P.kslot = kslot; P.act = act;
    P.part = reinterpret_cast<float*>(ws);
    P.n_seq = n_seq; P.rows = rows; P.Hq = g.Hq; P.Hkv = g.Hkv; P.G = g.G;
    P.W = g.W; P.pstride = is_swa ? g.ring : g.slot_ctx; P.ring_mask = is_swa ? g.ring - 1 : -1;
    P.slot_ctx = g.slot_ctx; P.n_slots = g.n_slots; P.is_swa = is_swa; P.q_f16 = g.q_f16;
    P.scale = g.scale; P.status = h->d_status;
    apply_paging(P, pv);
    if (pv) P.n_slots = pv->n_tables;
    h->kvw_kind = 0;
    const dim3 grid(n_seq * g.Hkv, nsplit, rows), block(32 * g.G);
    {
        ProfScope prof(h, st);
        if (g.HD == 128) k_attn_exact<128><<<grid, block, 0, st>>>(P);
        else             k_attn_exact<256><<<grid, block, 0, st>>>(P);
    }
    MergeParams M{};
    M.mode = MERGE_REGULAR; M.part = P.part; M.out = out; M.rec_out = rec_out;
    M.n_rows = n_seq * rows; M.rows = rows; M.Hq = g.Hq; M.Hkv = g.Hkv; M.G = g.G;
    M.count = nsplit; M.log2_domain = 0; M.out_f16 = g.out_f16;
    M.pos = pos; M.kslot = kslot; M.act = act; M.is_swa = is_swa; M.W = g.W; M.slot_ctx = P.slot_ctx;
    M.n_slots = P.n_slots; M.status = h->d_status; M.hdr = nullptr;
    if (g.HD == 128) k_merge<128><<<n_seq * rows * g.Hq, MERGE_THREADS, 0, st>>>(M);
    else             k_merge<256><<<n_seq * rows * g.Hq, MERGE_THREADS, 0, st>>>(M);
    h->launches += 2;
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

// inputs of the QKV prologue for the decode call that runs it itself
struct PrologueIn {
    const float* q_raw;
    const float* sqk;
    const float* cs;
    const float* sn;
    int table_off;
};

template <int HD, int NT>
cudaError_t launch_fd_kernel(const fd::Params& P, int grid, size_t smem, cudaStream_t st) {
    if constexpr (NT == 1) {
        if (P.q_raw) return launch_pdl(fd::k_flash_decode<HD, 1, 2>, dim3(grid), dim3(fd::NTHREADS), smem, st, P);
        if (P.k_new) return launch_pdl(fd::k_flash_decode<HD, 1, 1>, dim3(grid), dim3(fd::NTHREADS), smem, st, P);
    }
    return launch_pdl(fd::k_flash_decode<HD, NT>, dim3(grid), dim3(fd::NTHREADS), smem, st, P);
}

// decode / verify / multi-slot decode through the flash-decode kernel and the balanced merge
int launch_flash(battn_handle* h, void* out, float* rec_out, const void* q, const uint8_t* kvk, const uint8_t* kvv,
                 const int* pos, const int* kslot, const int* act, void* ws, int n_seq, int rows, int is_swa,
                 cudaStream_t st, const XchgView* xv = nullptr, int* epoch_ptr = nullptr, int epoch_advance = 0,
                 const PagedView* pv = nullptr, const float* k_new = nullptr, const float* v_new = nullptr,
                 const PrologueIn* pro = nullptr) {
    const Geom& g = h->g;
    const int RG = rows * g.G;
    if (RG > 32) return BATTN_ERR_CAPACITY;
    const int idx = nt_index(RG);
    const FdWs w = fd_workspace(h, n_seq, rows);
    fd::Params P;
    P.q = q; P.kvk = kvk; P.kvv = kvv; P.pos = pos; P.kslot = kslot; P.act = act;
    P.hdr = reinterpret_cast<int*>(ws);
    P.part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + w.hdr_bytes);
    P.n_seq = n_seq; P.rows = rows; P.Hq = g.Hq; P.Hkv = g.Hkv; P.G = g.G; P.RG = RG;
    P.W = g.W; P.pstride = is_swa ? g.ring : g.slot_ctx; P.ring_mask = is_swa ? g.ring - 1 : -1;
    P.slot_ctx = g.slot_ctx; P.n_slots = g.n_slots; P.is_swa = is_swa; P.q_f16 = g.q_f16;
    P.scale_log2 = g.scale * LOG2E; P.status = h->d_status;
    P.epoch_ptr = epoch_ptr; P.epoch_advance = epoch_advance;
    P.cph = 0;
    P.q_raw = pro ? pro->q_raw : nullptr; P.sqk = pro ? pro->sqk : nullptr; P.cs = pro ? pro->cs : nullptr;
    P.sn = pro ? pro->sn : nullptr; P.table_off = pro ? pro->table_off : 0;
    P.k_new = k_new; P.v_new = v_new; P.kvk_w = const_cast<uint8_t*>(kvk); P.kvv_w = const_cast<uint8_t*>(kvv);
    apply_paging(P, pv);
    if (pv) P.n_slots = pv->n_tables;
    // early KV streaming: only when the last launch on this handle wrote no cache rows but this call's own
    P.early = h->early_stream && (h->kvw_kind == 0 || (h->kvw_kind == 1 && h->kvw_pos == pos && h->kvw_nseq == n_seq &&
                                                       h->kvw_rows == rows) ||
                                  (h->kvw_kind == 3 && (RG <= 16 || h->kvw_cache != (const void*)kvk)));
    h->kvw_kind = k_new ? 3 : 0;
    h->kvw_cache = kvk;

    cudaError_t e;
    int fd_grid = 0;                                   // grid of the flash-decode kernel, when that one runs
    if (RG > 16 && g.HD == 128 && g.W >= 64 && vt::smem_bytes(n_seq) <= SMEM_MAX) {
        // 5..8 rows at head_dim 128: the tensor-memory verify kernel, one CTA per SM (128-key tiles must not wrap the
        // ring, hence the window bound; very large batches exceed its shared memory and take the kernel below)
        if (n_seq == 1 && h->num_sms >= g.Hkv) P.cph = h->num_sms / g.Hkv;
        ProfScope prof(h, st);
        e = launch_pdl(vt::k_verify_tc, dim3(h->num_sms), dim3(vt::NTHREADS), vt::smem_bytes(n_seq), st, P);
    } else if (RG > 16) {
        // 5..8 rows: the wide verify kernel (each warp owns 8 pairs over all keys of a tile)
        const size_t smem = g.HD == 128 ? vw::smem_bytes<128>(n_seq) : vw::smem_bytes<256>(n_seq);
        if (smem > SMEM_MAX) return BATTN_ERR_CAPACITY;
        int per_sm = (int)(SMEM_MAX / (smem + 1024));
        if (per_sm > h->vw_ctas_per_sm) per_sm = h->vw_ctas_per_sm;
        if (per_sm < 1) per_sm = 1;
        const int grid = h->num_sms * per_sm;
        if (n_seq == 1 && grid >= g.Hkv) P.cph = grid / g.Hkv;
        ProfScope prof(h, st);
        e = g.HD == 128 ? launch_pdl(vw::k_verify_wide<128>, dim3(grid), dim3(vw::NTHREADS), smem, st, P)
                        : launch_pdl(vw::k_verify_wide<256>, dim3(grid), dim3(vw::NTHREADS), smem, st, P);
    } else {
        size_t smem;
        if (g.HD == 128) smem = idx == 0 ? fd::smem_bytes<128, 1>(RG, n_seq) : fd::smem_bytes<128, 2>(RG, n_seq);
        else             smem = idx == 0 ? fd::smem_bytes<256, 1>(RG, n_seq) : fd::smem_bytes<256, 2>(RG, n_seq);
        if (smem > SMEM_MAX) return BATTN_ERR_CAPACITY;
        int per_sm = (int)(SMEM_MAX / (smem + 1024));
        if (per_sm > h->fd_ctas_per_sm[idx]) per_sm = h->fd_ctas_per_sm[idx];
        if (per_sm < 1) per_sm = 1;
        const int grid = h->num_sms * per_sm;
        fd_grid = grid;
        if (n_seq == 1 && grid >= g.Hkv) P.cph = grid / g.Hkv;     // one sequence: no share crosses a kv head
        ProfScope prof(h, st);
        if (g.HD == 128) e = idx == 0 ? launch_fd_kernel<128, 1>(P, grid, smem, st) : launch_fd_kernel<128, 2>(P, grid, smem, st);
        else             e = idx == 0 ? launch_fd_kernel<256, 1>(P, grid, smem, st) : launch_fd_kernel<256, 2>(P, grid, smem, st);
    }
    if (e != cudaSuccess) return cuda_fail(h, e);
    MergeParams M{};
    M.mode = 0; M.part = P.part; M.out = out; M.rec_out = rec_out;
    M.n_rows = n_seq * rows; M.rows = rows; M.Hq = g.Hq; M.Hkv = g.Hkv; M.G = g.G;
    M.count = 0; M.log2_domain = 1; M.out_f16 = g.out_f16; M.hdr = P.hdr; M.status = h->d_status;
    M.cph = P.cph;
    if (P.early && fd_grid > 0 && n_seq == 1) {
        // the merge recomputes the cut from the positions while it waits for the decode kernel
        M.pre_grid = fd_grid; M.pre_tile = fd::TILE;
        M.pos = pos; M.kslot = kslot; M.act = act; M.is_swa = is_swa; M.W = g.W; M.slot_ctx = P.slot_ctx; M.n_slots = P.n_slots;
    }
    if (xv) M.xchg = *xv;
    if (g.HD == 128) e = launch_pdl(k_merge_balanced<128>, dim3(n_seq * rows * g.Hq), dim3(MERGE_B_THREADS), 0, st, M);
    else             e = launch_pdl(k_merge_balanced<256>, dim3(n_seq * rows * g.Hq), dim3(MERGE_B_THREADS), 0, st, M);
    h->launches += 2;
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

// prompt chunk on the tcgen05 kernel: one CTA per (128-row M tile, kv head), normalised output
int launch_prefill(battn_handle* h, void* out, const void* q, const uint8_t* kvk, const uint8_t* kvv, const int* pos,
                   void* ws, int rows, int is_swa, cudaStream_t st, const GateNormParams* gn = nullptr,
                   const PagedView* pv = nullptr, int table_row = 0) {
    const Geom& g = h->g;
    if (128 % g.G) return BATTN_ERR_ARG;
    pf::Params P;
    P.q = q; P.out = out; P.kvk = kvk; P.kvv = kvv; P.pos = pos;
    P.rows = rows; P.Hq = g.Hq; P.Hkv = g.Hkv; P.G = g.G;
    P.W = g.W; P.pstride = is_swa ? g.ring : g.slot_ctx; P.ring_mask = is_swa ? g.ring - 1 : -1;
    P.slot_ctx = g.slot_ctx; P.is_swa = is_swa; P.q_f16 = g.q_f16; P.out_f16 = g.out_f16;
    P.scale_log2 = g.scale * LOG2E; P.status = h->d_status;
    apply_paging(P, pv);
    if (pv) P.slot = table_row;
    // early KV streaming: only behind the append / prologue of exactly this chunk, or no cache write
    P.early = h->early_stream &&
              (h->kvw_kind == 0 || (h->kvw_kind == 1 && h->kvw_pos == pos && h->kvw_nseq == 1 && h->kvw_rows == rows) ||
               (h->kvw_kind == 3 && h->kvw_cache != (const void*)kvk));
    h->kvw_kind = 0;
    const int MR = 128 / g.G;
    P.nsplit = prefill_splits(h, rows, is_swa);
    P.recs = (P.nsplit > 1 || gn) ? reinterpret_cast<float*>(ws) : nullptr;
    const dim3 grid((rows + MR - 1) / MR, g.Hkv, P.nsplit);
    {
        ProfScope prof(h, st);
        if (g.HD == 128 && BATTN_PF_PAIR && grid.x >= 2) {
            // two M tiles per cluster of two CTAs (tcgen05.mma.cta_group::2): each CTA converts half of every operand
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((grid.x + 1) & ~1u, grid.y, grid.z); cfg.blockDim = dim3(pf128::NTHREADS);
            cfg.dynamicSmemBytes = pf128::TOTAL_PAIR; cfg.stream = st;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr; cfg.numAttrs = 2;
            cudaLaunchKernelEx(&cfg, pf128::k_prefill_hd128<true>, P);
        } else if (g.HD == 128) {
            launch_pdl(pf128::k_prefill_hd128<false>, grid, dim3(pf128::NTHREADS), pf128::TOTAL, st, P);
        }
        else             launch_pdl(pf::k_prefill<256, 64>, grid, dim3(pf::NTHREADS), pf::Cfg<256, 64>::TOTAL, st, P);
    }
    h->launches += 1;
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && gn) {
        // the fused epilogue: merge of the split records, sigmoid gate, L2 norm and q8 copy, one block per row
        GateNormParams G = *gn;
        G.recs = P.recs; G.nsplit = P.nsplit; G.rows = rows; G.Hq = g.Hq; G.n = g.Hq * g.HD;
        if (g.HD == 128) e = launch_pdl(k_merge_gate_norm<128>, dim3(rows), dim3(256), 0, st, G);
        else             e = launch_pdl(k_merge_gate_norm<256>, dim3(rows), dim3(256), 0, st, G);
        h->launches += 1;
        if (e == cudaSuccess) e = cudaGetLastError();
        return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
    }
    if (e == cudaSuccess && P.nsplit > 1) {
        MergeParams M{};
        M.mode = MERGE_GATHERED; M.part = P.recs; M.out = out; M.rec_out = nullptr;
        M.n_rows = rows; M.rows = 1; M.Hq = g.Hq; M.Hkv = g.Hkv; M.G = g.G;
        M.count = P.nsplit; M.log2_domain = 1; M.out_f16 = g.out_f16; M.status = h->d_status;
        // (head_dim 128: programmatic launch, the merge's blocks are resident and past their launch when the prompt
        // kernel drains -- 2 us less on a short chunk; at head_dim 256, where every 512-row chunk is split and the merge
        // has thousands of blocks, the early launch cost 2 % and the plain launch stays)
        if (g.HD == 128) launch_pdl(k_merge<128>, dim3(rows * g.Hq), dim3(MERGE_THREADS), 0, st, M);
        else             k_merge<256><<<rows * g.Hq, MERGE_THREADS, 0, st>>>(M);
        h->launches += 1;
        e = cudaGetLastError();
    }
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

// device-side view of an exchange for one launch
XchgView xchg_view(const battn_xchg* x, const int* epoch, int push, int wait) {
    XchgView v{};
    for (int d = 0; d < x->world; ++d) v.area[d] = reinterpret_cast<uint8_t*>(x->area[d]);
    v.world = x->world; v.rank = x->rank; v.max_items = x->max_items; v.epoch_ptr = epoch;
    v.wait_polls = x->wait_polls; v.push = push; v.wait = wait;
    return v;
}

// validates a caller's geometry and derives the internal one
int geom_from(const battn_geom* geom, Geom& g) {
    if (!geom) return BATTN_ERR_ARG;
    if (geom->head_dim != 128 && geom->head_dim != 256) return BATTN_ERR_ARG;
    if (geom->n_head < 1 || geom->n_kv < 1 || geom->n_head % geom->n_kv) return BATTN_ERR_ARG;
    const int G = geom->n_head / geom->n_kv;
    if (G > 8) return BATTN_ERR_ARG;
    if (geom->window < 32 || (geom->window & (geom->window - 1))) return BATTN_ERR_ARG;
    if (geom->slot_ctx < 2 || (geom->slot_ctx & 1) || geom->n_slots < 1) return BATTN_ERR_ARG;
    if ((geom->q_dtype != BATTN_F32 && geom->q_dtype != BATTN_F16) ||
        (geom->out_dtype != BATTN_F32 && geom->out_dtype != BATTN_F16)) return BATTN_ERR_ARG;
    g.Hq = geom->n_head; g.Hkv = geom->n_kv; g.HD = geom->head_dim; g.G = G;
    g.W = geom->window; g.ring = 2 * geom->window;
    g.slot_ctx = geom->slot_ctx; g.n_slots = geom->n_slots;
    g.nblk = g.HD / 32; g.rec = g.HD + 2 * g.nblk;
    g.q_f16 = geom->q_dtype == BATTN_F16; g.out_f16 = geom->out_dtype == BATTN_F16;
    g.scale = geom->softmax_scale != 0.f ? geom->softmax_scale : 1.f / sqrtf((float)g.HD);
    return BATTN_OK;
}

// scratch bytes that ONE call of exactly this shape writes (its split records and their header)
size_t call_workspace(const battn_handle* h, int n_seq, int rows) {
    if (rows * h->g.G <= 32) return fd_workspace(h, n_seq, rows).total;
    return n_seq == 1 ? prefill_workspace(h, rows) : 0;
}

}  // namespace

extern "C" {

int battn_version(void) { return BATTN_VERSION; }

int battn_init(const battn_geom* geom, int device, battn_handle** out_handle) {
    if (!geom || !out_handle) return BATTN_ERR_ARG;
    *out_handle = nullptr;
    Geom g0;
    const int grc = geom_from(geom, g0);
    if (grc) return grc;

    battn_handle* h = new (std::nothrow) battn_handle();
    if (!h) return BATTN_ERR_ARG;
    Geom& g = h->g;
    g = g0;
    h->device = device; h->last_cuda_error = 0; h->launches = 0; h->d_status = nullptr;
    h->prof_ev = nullptr; h->prof_cap = 0; h->prof_n = 0;
    h->early_stream = 0; h->kvw_kind = 0; h->kvw_nseq = 0; h->kvw_rows = 0; h->kvw_pos = nullptr; h->kvw_cache = nullptr;

    cudaError_t e = cudaSetDevice(device);
    cudaDeviceProp prop;
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device);
    if (e == cudaSuccess && prop.major < 10) e = cudaErrorInvalidDevice;      // sm_100a only
    if (e == cudaSuccess) { h->num_sms = prop.multiProcessorCount; e = cudaMalloc(&h->d_status, 16); }
    if (e == cudaSuccess) e = cudaMemset(h->d_status, 0, 16);
    if (e == cudaSuccess) e = g.HD == 128 ? fd_prepare_all<128>(h) : fd_prepare_all<256>(h);
    // device address of the built-in scratch on THIS device (it is current here)
    h->noalloc_ws = nullptr;
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&h->noalloc_ws, g_noalloc_scratch);
    if (e != cudaSuccess) {
        g_init_cuda_error = (int)e;
        if (h->d_status) cudaFree(h->d_status);
        delete h;
        return BATTN_ERR_CUDA;
    }
    *out_handle = h;
    return BATTN_OK;
}

int battn_destroy(battn_handle* h) {
    if (!h) return BATTN_ERR_ARG;
    cudaSetDevice(h->device);
    if (h->prof_ev) { int n = 0; battn_profile_stop(h, nullptr, 0, &n); }
    if (h->d_status) cudaFree(h->d_status);
    delete h;
    return BATTN_OK;
}

int battn_kv_layer_bytes(const battn_handle* h, int is_swa, size_t* out_bytes) {
    if (!h || !out_bytes) return BATTN_ERR_ARG;
    const Geom& g = h->g;
    *out_bytes = (size_t)g.n_slots * (is_swa ? g.ring : g.slot_ctx) * g.Hkv * g.rec;   // bruce.cu:5476-5481
    return BATTN_OK;
}

int battn_workspace_bytes(const battn_handle* h, int n_seq, int rows_per_seq, size_t* out_bytes) {
    if (!h || !out_bytes || n_seq < 1 || rows_per_seq < 1) return BATTN_ERR_ARG;
    if (n_seq > MAX_SEQ || rows_per_seq > MAX_PREFILL) return BATTN_ERR_CAPACITY;
    // The buffer must serve every call of UP TO rows_per_seq rows (a prompt's last chunk is shorter than the
    // chunk the buffer was sized for), and the split count of a prompt chunk grows as the chunk shrinks, so the
    // need is not monotone in the row count: take the maximum over all shorter calls.
    size_t need = 0;
    for (int r = 1; r <= rows_per_seq; ++r) {
        size_t f = exact_workspace(h, n_seq, r, exact_default_splits(r));
        const size_t w = call_workspace(h, n_seq, r);
        if (w > f) f = w;
        if (f > need) need = f;
    }
    *out_bytes = align_up(need, 256);
    return BATTN_OK;
}

int battn_call_workspace_bytes(const battn_geom* geom, int num_sms, int n_seq, int rows_per_seq, size_t* out_bytes) {
    if (!out_bytes || num_sms < 1 || n_seq < 1 || rows_per_seq < 1) return BATTN_ERR_ARG;
    if (n_seq > MAX_SEQ || rows_per_seq > MAX_PREFILL) return BATTN_ERR_CAPACITY;
    battn_handle tmp{};
    const int rc = geom_from(geom, tmp.g);
    if (rc) return rc;
    tmp.num_sms = num_sms;
    *out_bytes = call_workspace(&tmp, n_seq, rows_per_seq);
    return BATTN_OK;
}

int battn_exact_workspace_bytes(const battn_handle* h, int n_seq, int rows_per_seq, int nsplit, size_t* out_bytes) {
    if (!h || !out_bytes || n_seq < 1 || rows_per_seq < 1 || nsplit < 1 || nsplit > MAX_SPLITS) return BATTN_ERR_ARG;
    *out_bytes = align_up(exact_workspace(h, n_seq, rows_per_seq, nsplit), 256);
    return BATTN_OK;
}

static int kv_append_impl(battn_handle* h, const float* k, const float* v, uint8_t* kvk, uint8_t* kvv, const int* pos,
                          const int* kslot, const int* act, int n_seq, int rows_per_seq, int is_swa, void* stream,
                          const PagedView* pv) {
    const int rc = check_seq_args(h, k, v, kvk, kvv, pos, kslot, n_seq, rows_per_seq, MAX_PREFILL);
    if (rc) return rc;
    const Geom& g = h->g;
    // one call must not wrap the ring onto itself: two rows of the same launch would race for a slot
    // (the reference appends at most 512 rows into a 2048-slot ring, bruce.cu:50-53, 1058)
    if (is_swa && rows_per_seq > g.ring) return BATTN_ERR_CAPACITY;
    AppendParams P;
    P.k = k; P.v = v; P.kvk = kvk; P.kvv = kvv; P.pos = pos; P.kslot = kslot; P.act = act;
    P.n_seq = n_seq; P.rows = rows_per_seq; P.Hkv = g.Hkv;
    P.pstride = is_swa ? g.ring : g.slot_ctx; P.ring_mask = is_swa ? g.ring - 1 : -1;
    P.n_slots = g.n_slots; P.status = h->d_status;
    if (pv) { P.pg = pv->pg; P.pstride = pv->capacity; P.ring_mask = -1; P.n_slots = pv->n_tables; }
    h->kvw_kind = 1; h->kvw_pos = pos; h->kvw_nseq = n_seq; h->kvw_rows = rows_per_seq;
    const long long warps = (long long)n_seq * rows_per_seq * g.Hkv * 2;
    const int blocks = (int)((warps + 7) / 8);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (g.HD == 128) e = launch_pdl(k_kv_append<128>, dim3(blocks), dim3(256), 0, st, P);
    else             e = launch_pdl(k_kv_append<256>, dim3(blocks), dim3(256), 0, st, P);
    h->launches += 1;
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

int battn_kv_append(battn_handle* h, const float* k, const float* v, uint8_t* kvk, uint8_t* kvv, const int* pos,
                    const int* kslot, const int* act, int n_seq, int rows_per_seq, int is_swa, void* stream) {
    return kv_append_impl(h, k, v, kvk, kvv, pos, kslot, act, n_seq, rows_per_seq, is_swa, stream, nullptr);
}

int battn_kv_copy_prefix(battn_handle* h, uint8_t* kvk, uint8_t* kvv, int src_slot, int dst_slot, int n_pos, int is_swa,
                         void* stream) {
    if (!h || !kvk || !kvv || ((((uintptr_t)kvk | (uintptr_t)kvv)) & 15)) return BATTN_ERR_ARG;
    const Geom& g = h->g;
    if (src_slot < 0 || dst_slot < 0 || src_slot >= g.n_slots || dst_slot >= g.n_slots || src_slot == dst_slot) return BATTN_ERR_ARG;
    if (n_pos < 0 || (!is_swa && n_pos > g.slot_ctx)) return BATTN_ERR_CAPACITY;
    if (n_pos == 0) return BATTN_OK;
    h->kvw_kind = 2;
    CopyParams P;
    P.kvk = kvk; P.kvv = kvv; P.src = src_slot; P.dst = dst_slot; P.n_pos = n_pos; P.Hkv = g.Hkv; P.rec = g.rec;
    P.pstride = is_swa ? g.ring : g.slot_ctx; P.ring = is_swa ? g.ring : 0;
    const int copied = is_swa && n_pos > g.ring ? g.ring : n_pos;
    const int bx = (int)std::min<size_t>(64, ((size_t)copied * g.rec / 16 + 255) / 256 + 1);
    cudaError_t e = launch_pdl(k_kv_copy_prefix, dim3(bx, g.Hkv, 2), dim3(256), 0, (cudaStream_t)stream, P);
    h->launches += 1;
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

static int qkv_prep_impl(battn_handle* h, void* q_out, const float* q, const float* k, const float* v, const float* sqk,
                         const float* cs, const float* sn, int theta_sel, uint8_t* kvk, uint8_t* kvv, const int* pos,
                         const int* kslot, const int* act, int n_seq, int rows_per_seq, int is_swa, void* stream,
                         const PagedView* pv) {
    const int rc = check_seq_args(h, k, v, kvk, kvv, pos, kslot, n_seq, rows_per_seq, MAX_PREFILL);
    if (rc) return rc;
    if (!q_out || !q || !sqk || !cs || !sn || (theta_sel != 1 && theta_sel != 2)) return BATTN_ERR_ARG;
    if ((((uintptr_t)q_out | (uintptr_t)q | (uintptr_t)sqk | (uintptr_t)cs | (uintptr_t)sn) & 15) != 0) return BATTN_ERR_ARG;   // k, v, kvk, kvv: check_seq_args
    const Geom& g = h->g;
    if (is_swa && rows_per_seq > g.ring) return BATTN_ERR_CAPACITY;        // as battn_kv_append
    PrepParams P;
    P.q = q; P.q_out = q_out; P.k = k; P.v = v; P.sqk = sqk; P.cs = cs; P.sn = sn; P.kvk = kvk; P.kvv = kvv;
    P.pos = pos; P.kslot = kslot; P.act = act; P.n_seq = n_seq; P.rows = rows_per_seq; P.Hq = g.Hq; P.Hkv = g.Hkv;
    P.table_off = theta_sel == 2 ? g.HD / 2 : 0; P.q_out_f16 = g.q_f16;
    P.pstride = is_swa ? g.ring : g.slot_ctx; P.ring_mask = is_swa ? g.ring - 1 : -1;
    P.n_slots = g.n_slots; P.status = h->d_status;
    if (pv) { P.pg = pv->pg; P.pstride = pv->capacity; P.ring_mask = -1; P.n_slots = pv->n_tables; }
    h->kvw_kind = 1; h->kvw_pos = pos; h->kvw_nseq = n_seq; h->kvw_rows = rows_per_seq;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    const dim3 grid(n_seq * rows_per_seq, (g.Hq + g.Hkv + 7) / 8);
    if (g.HD == 128) e = launch_pdl(k_qkv_prep<128>, grid, dim3(256), 0, st, P);
    else             e = launch_pdl(k_qkv_prep<256>, grid, dim3(256), 0, st, P);
    h->launches += 1;
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

int battn_qkv_prep(battn_handle* h, void* q_out, const float* q, const float* k, const float* v, const float* sqk,
                   const float* cs, const float* sn, int theta_sel, uint8_t* kvk, uint8_t* kvv, const int* pos,
                   const int* kslot, const int* act, int n_seq, int rows_per_seq, int is_swa, void* stream) {
    return qkv_prep_impl(h, q_out, q, k, v, sqk, cs, sn, theta_sel, kvk, kvv, pos, kslot, act, n_seq, rows_per_seq, is_swa,
                         stream, nullptr);
}

int battn_rope_tables(battn_handle* h, float* cs, float* sn, const int* pos, int n_seq, int rows_per_seq, void* stream) {
    if (!h || !cs || !sn || !pos || n_seq < 1 || rows_per_seq < 1 || rows_per_seq > MAX_PREFILL) return BATTN_ERR_ARG;
    const Geom& g = h->g;
    TableParams P;
    P.cs = cs; P.sn = sn; P.pos = pos; P.rows = rows_per_seq; P.n_rows = n_seq * rows_per_seq;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (g.HD == 128) e = launch_pdl(k_rope_tables<128>, dim3(P.n_rows), dim3(64), 0, st, P);
    else             e = launch_pdl(k_rope_tables<256>, dim3(P.n_rows), dim3(128), 0, st, P);
    h->launches += 1;
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

int battn_decode(battn_handle* h, void* out, const void* q, const uint8_t* kvk, const uint8_t* kvv, const int* pos,
                 const int* kslot, const int* act, void* ws, int n_seq, int is_swa, void* stream) {
    const int rc = check_seq_args(h, out, q, kvk, kvv, pos, kslot, n_seq, 1, 1);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15)) return BATTN_ERR_ARG;
    return launch_flash(h, out, nullptr, q, kvk, kvv, pos, kslot, act, ws, n_seq, 1, is_swa, (cudaStream_t)stream);
}

int battn_decode_append(battn_handle* h, void* out, const void* q, const float* k, const float* v, uint8_t* kvk,
                        uint8_t* kvv, const int* pos, const int* kslot, const int* act, void* ws, int n_seq, int is_swa,
                        void* stream) {
    const int rc = check_seq_args(h, out, q, kvk, kvv, pos, kslot, n_seq, 1, 1);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15) || !k || !v || ((((uintptr_t)k | (uintptr_t)v)) & 15)) return BATTN_ERR_ARG;
    return launch_flash(h, out, nullptr, q, kvk, kvv, pos, kslot, act, ws, n_seq, 1, is_swa, (cudaStream_t)stream, nullptr,
                        nullptr, 0, nullptr, k, v);
}

int battn_qkv_decode(battn_handle* h, void* out, const float* q, const float* k, const float* v, const float* sqk,
                     const float* cs, const float* sn, int theta_sel, uint8_t* kvk, uint8_t* kvv, const int* pos,
                     const int* kslot, const int* act, void* ws, int n_seq, int is_swa, void* stream) {
    const int rc = check_seq_args(h, out, q, kvk, kvv, pos, kslot, n_seq, 1, 1);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15) || !k || !v || !sqk || !cs || !sn || (theta_sel != 1 && theta_sel != 2)) return BATTN_ERR_ARG;
    if ((((uintptr_t)k | (uintptr_t)v | (uintptr_t)sqk | (uintptr_t)cs | (uintptr_t)sn) & 15) != 0) return BATTN_ERR_ARG;
    PrologueIn pro{q, sqk, cs, sn, theta_sel == 2 ? h->g.HD / 2 : 0};
    return launch_flash(h, out, nullptr, q, kvk, kvv, pos, kslot, act, ws, n_seq, 1, is_swa, (cudaStream_t)stream, nullptr,
                        nullptr, 0, nullptr, k, v, &pro);
}

int battn_decode_noalloc(battn_handle* h, void* out, const void* q, const uint8_t* kvk, const uint8_t* kvv,
                         const int* pos, const int* kslot, const int* act, int n_seq, int is_swa, void* stream) {
    const int rc = check_seq_args(h, out, q, kvk, kvv, pos, kslot, n_seq, 1, 1);
    if (rc) return rc;
    if (!h->noalloc_ws) return BATTN_ERR_ARG;
    // the built-in array is all the scratch there is: larger requests are refused, never truncated
    if (fd_workspace(h, n_seq, 1).total > (size_t)BATTN_NOALLOC_SCRATCH_BYTES) return BATTN_ERR_CAPACITY;
    return launch_flash(h, out, nullptr, q, kvk, kvv, pos, kslot, act, h->noalloc_ws, n_seq, 1, is_swa,
                        (cudaStream_t)stream);
}

int battn_verify(battn_handle* h, void* out, const void* q, const uint8_t* kvk, const uint8_t* kvv, const int* pos,
                 const int* kslot, const int* act, void* ws, int rows, int batch, int is_swa, void* stream) {
    const int rc = check_seq_args(h, out, q, kvk, kvv, pos, kslot, batch, rows, MAX_VERIFY);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15)) return BATTN_ERR_ARG;
    return launch_flash(h, out, nullptr, q, kvk, kvv, pos, kslot, act, ws, batch, rows, is_swa, (cudaStream_t)stream);
}

int battn_partials(battn_handle* h, float* rec, const void* q, const uint8_t* kvk, const uint8_t* kvv,
                   const int* pos, const int* kslot, const int* act, void* ws, int rows, int batch, int is_swa,
                   void* stream) {
    const int rc = check_seq_args(h, rec, q, kvk, kvv, pos, kslot, batch, rows, MAX_VERIFY);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15)) return BATTN_ERR_ARG;
    return launch_flash(h, nullptr, rec, q, kvk, kvv, pos, kslot, act, ws, batch, rows, is_swa, (cudaStream_t)stream);
}

int battn_prefill(battn_handle* h, void* out, const void* q, const uint8_t* kvk, const uint8_t* kvv, const int* pos,
                  void* ws, int rows, int is_swa, void* stream) {
    const int rc = check_seq_args(h, out, q, kvk, kvv, pos, nullptr, 1, rows, MAX_PREFILL);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15)) return BATTN_ERR_ARG;
    // the ring must hold the whole chunk plus the oldest row's window (bruce.cu:50-53)
    if (is_swa && rows > h->g.W) return BATTN_ERR_CAPACITY;
    if (h->g.W < 64) return BATTN_ERR_ARG;               // key tiles of 64 / 128 must not wrap the ring
    if (rows * h->g.G <= 32)
        return launch_flash(h, out, nullptr, q, kvk, kvv, pos, nullptr, nullptr, ws, 1, rows, is_swa, (cudaStream_t)stream);
    return launch_prefill(h, out, q, kvk, kvv, pos, ws, rows, is_swa, (cudaStream_t)stream);
}

int battn_gate_norm(battn_handle* h, float* dst, const void* aout, const float* gate, const float* sgate, int8_t* xq,
                    float* xd, int* xsum, int rows, void* stream) {
    if (!h || !aout || !gate || !sgate || !xq || !xd || !xsum || rows < 1) return BATTN_ERR_ARG;
    if ((((uintptr_t)dst | (uintptr_t)aout | (uintptr_t)gate | (uintptr_t)sgate | (uintptr_t)xq) & 15) != 0) return BATTN_ERR_ARG;
    const Geom& g = h->g;
    const int n = g.Hq * g.HD;
    if (n % 1024 || n > 4096) return BATTN_ERR_ARG;
    GateNormParams G{};
    G.dst = dst; G.aout = aout; G.aout_f16 = g.out_f16; G.gate = gate; G.sgate = sgate; G.xq = xq; G.xd = xd; G.xsum = xsum;
    G.n = n;
    cudaError_t e = launch_pdl(k_gate_norm, dim3(rows), dim3(256), 0, (cudaStream_t)stream, G);
    h->launches += 1;
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

int battn_prefill_gate_norm(battn_handle* h, float* dst, const void* q, const uint8_t* kvk, const uint8_t* kvv,
                            const int* pos, void* ws, const float* gate, const float* sgate, int8_t* xq, float* xd,
                            int* xsum, int rows, int is_swa, void* stream) {
    const int rc = check_seq_args(h, q, q, kvk, kvv, pos, nullptr, 1, rows, MAX_PREFILL);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15) || !gate || !sgate || !xq || !xd || !xsum) return BATTN_ERR_ARG;
    if ((((uintptr_t)dst | (uintptr_t)gate | (uintptr_t)sgate | (uintptr_t)xq) & 15) != 0) return BATTN_ERR_ARG;
    const Geom& g = h->g;
    const int n = g.Hq * g.HD;
    if (n % 1024 || n > 4096 || g.Hq > 32) return BATTN_ERR_ARG;
    if (rows * g.G <= 32) return BATTN_ERR_ARG;              // short calls: battn_decode / battn_verify, then battn_gate_norm
    if (is_swa && rows > g.W) return BATTN_ERR_CAPACITY;
    if (g.W < 64) return BATTN_ERR_ARG;
    GateNormParams G{};
    G.dst = dst; G.gate = gate; G.sgate = sgate; G.xq = xq; G.xd = xd; G.xsum = xsum;
    return launch_prefill(h, nullptr, q, kvk, kvv, pos, ws, rows, is_swa, (cudaStream_t)stream, &G);
}

int battn_attend_exact(battn_handle* h, void* out, const void* q, const uint8_t* kvk, const uint8_t* kvv,
                       const int* pos, const int* kslot, const int* act, void* ws, int n_seq, int rows_per_seq,
                       int nsplit, int is_swa, void* stream) {
    const int rc = check_seq_args(h, out, q, kvk, kvv, pos, kslot, n_seq, rows_per_seq, MAX_PREFILL);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15) || nsplit < 1 || nsplit > MAX_SPLITS) return BATTN_ERR_ARG;
    return launch_exact(h, out, nullptr, q, kvk, kvv, pos, kslot, act, ws, n_seq, rows_per_seq, nsplit, is_swa,
                        (cudaStream_t)stream);
}

// ---- paged cache (full-causal layers) -----------------------------------------------------------------------
int battn_pages_pool_bytes(const battn_handle* h, int n_pages, int page_len, size_t* out_bytes) {
    if (!h || !out_bytes || n_pages < 1 || page_len < 128 || (page_len & (page_len - 1))) return BATTN_ERR_ARG;
    *out_bytes = (size_t)n_pages * h->g.Hkv * (size_t)page_len * h->g.rec;
    return BATTN_OK;
}

int battn_pages_copy(battn_handle* h, const battn_pages* pages, int from_page, int to_page, void* stream) {
    PagedView pv;
    const int rc = paged_view(pages, pv);
    if (rc) return rc;
    if (!h || from_page < 0 || to_page < 0 || from_page >= pages->n_pages || to_page >= pages->n_pages) return BATTN_ERR_ARG;
    if (from_page == to_page) return BATTN_OK;
    h->kvw_kind = 2;
    const size_t page_bytes = (size_t)h->g.Hkv * pages->page_len * h->g.rec;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(pages->pool_k + to_page * page_bytes, pages->pool_k + from_page * page_bytes, page_bytes,
                                    cudaMemcpyDeviceToDevice, st);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(pages->pool_v + to_page * page_bytes, pages->pool_v + from_page * page_bytes, page_bytes,
                            cudaMemcpyDeviceToDevice, st);
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

int battn_kv_append_paged(battn_handle* h, const battn_pages* pages, const float* k, const float* v, const int* pos,
                          const int* ktab, const int* act, int n_seq, int rows_per_seq, void* stream) {
    PagedView pv;
    const int rc = paged_view(pages, pv);
    if (rc) return rc;
    return kv_append_impl(h, k, v, pages->pool_k, pages->pool_v, pos, ktab, act, n_seq, rows_per_seq, 0, stream, &pv);
}

int battn_qkv_prep_paged(battn_handle* h, void* q_out, const float* q, const float* k, const float* v, const float* sqk,
                         const float* cs, const float* sn, int theta_sel, const battn_pages* pages, const int* pos,
                         const int* ktab, const int* act, int n_seq, int rows_per_seq, void* stream) {
    PagedView pv;
    const int rc = paged_view(pages, pv);
    if (rc) return rc;
    return qkv_prep_impl(h, q_out, q, k, v, sqk, cs, sn, theta_sel, pages->pool_k, pages->pool_v, pos, ktab, act, n_seq,
                         rows_per_seq, 0, stream, &pv);
}

int battn_decode_paged(battn_handle* h, void* out, const void* q, const battn_pages* pages, const int* pos,
                       const int* ktab, const int* act, void* ws, int n_seq, void* stream) {
    PagedView pv;
    int rc = paged_view(pages, pv);
    if (rc) return rc;
    rc = check_seq_args(h, out, q, pages->pool_k, pages->pool_v, pos, ktab, n_seq, 1, 1);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15)) return BATTN_ERR_ARG;
    return launch_flash(h, out, nullptr, q, pages->pool_k, pages->pool_v, pos, ktab, act, ws, n_seq, 1, 0,
                        (cudaStream_t)stream, nullptr, nullptr, 0, &pv);
}

int battn_decode_append_paged(battn_handle* h, void* out, const void* q, const float* k, const float* v,
                              const battn_pages* pages, const int* pos, const int* ktab, const int* act, void* ws,
                              int n_seq, void* stream) {
    PagedView pv;
    int rc = paged_view(pages, pv);
    if (rc) return rc;
    rc = check_seq_args(h, out, q, pages->pool_k, pages->pool_v, pos, ktab, n_seq, 1, 1);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15) || !k || !v || ((((uintptr_t)k | (uintptr_t)v)) & 15)) return BATTN_ERR_ARG;
    return launch_flash(h, out, nullptr, q, pages->pool_k, pages->pool_v, pos, ktab, act, ws, n_seq, 1, 0,
                        (cudaStream_t)stream, nullptr, nullptr, 0, &pv, k, v);
}

int battn_qkv_decode_paged(battn_handle* h, void* out, const float* q, const float* k, const float* v, const float* sqk,
                           const float* cs, const float* sn, int theta_sel, const battn_pages* pages, const int* pos,
                           const int* ktab, const int* act, void* ws, int n_seq, void* stream) {
    PagedView pv;
    int rc = paged_view(pages, pv);
    if (rc) return rc;
    rc = check_seq_args(h, out, q, pages->pool_k, pages->pool_v, pos, ktab, n_seq, 1, 1);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15) || !k || !v || !sqk || !cs || !sn || (theta_sel != 1 && theta_sel != 2)) return BATTN_ERR_ARG;
    if ((((uintptr_t)k | (uintptr_t)v | (uintptr_t)sqk | (uintptr_t)cs | (uintptr_t)sn) & 15) != 0) return BATTN_ERR_ARG;
    PrologueIn pro{q, sqk, cs, sn, theta_sel == 2 ? h->g.HD / 2 : 0};
    return launch_flash(h, out, nullptr, q, pages->pool_k, pages->pool_v, pos, ktab, act, ws, n_seq, 1, 0,
                        (cudaStream_t)stream, nullptr, nullptr, 0, &pv, k, v, &pro);
}

int battn_verify_paged(battn_handle* h, void* out, const void* q, const battn_pages* pages, const int* pos,
                       const int* ktab, const int* act, void* ws, int rows, int batch, void* stream) {
    PagedView pv;
    int rc = paged_view(pages, pv);
    if (rc) return rc;
    rc = check_seq_args(h, out, q, pages->pool_k, pages->pool_v, pos, ktab, batch, rows, MAX_VERIFY);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15)) return BATTN_ERR_ARG;
    return launch_flash(h, out, nullptr, q, pages->pool_k, pages->pool_v, pos, ktab, act, ws, batch, rows, 0,
                        (cudaStream_t)stream, nullptr, nullptr, 0, &pv);
}

int battn_prefill_paged(battn_handle* h, void* out, const void* q, const battn_pages* pages, int table_row,
                        const int* pos, void* ws, int rows, void* stream) {
    PagedView pv;
    int rc = paged_view(pages, pv);
    if (rc) return rc;
    rc = check_seq_args(h, out, q, pages->pool_k, pages->pool_v, pos, nullptr, 1, rows, MAX_PREFILL);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15) || table_row < 0 || table_row >= pages->n_tables) return BATTN_ERR_ARG;
    if (rows * h->g.G <= 32) return BATTN_ERR_ARG;       // short calls: battn_decode_paged / battn_verify_paged
    return launch_prefill(h, out, q, pages->pool_k, pages->pool_v, pos, ws, rows, 0, (cudaStream_t)stream, nullptr, &pv,
                          table_row);
}

int battn_attend_exact_paged(battn_handle* h, void* out, const void* q, const battn_pages* pages, const int* pos,
                             const int* ktab, const int* act, void* ws, int n_seq, int rows_per_seq, int nsplit,
                             void* stream) {
    PagedView pv;
    int rc = paged_view(pages, pv);
    if (rc) return rc;
    rc = check_seq_args(h, out, q, pages->pool_k, pages->pool_v, pos, ktab, n_seq, rows_per_seq, MAX_PREFILL);
    if (rc) return rc;
    if (!ws || ((uintptr_t)ws & 15) || nsplit < 1 || nsplit > MAX_SPLITS) return BATTN_ERR_ARG;
    return launch_exact(h, out, nullptr, q, pages->pool_k, pages->pool_v, pos, ktab, act, ws, n_seq, rows_per_seq, nsplit,
                        0, (cudaStream_t)stream, &pv);
}

int battn_xchg_create(battn_handle* h, int rank, int world, int max_rows, battn_xchg** out_x, void* ipc_handle_out) {
    if (!h || !out_x || world < 1 || world > XCHG_MAX_WORLD || rank < 0 || rank >= world) return BATTN_ERR_ARG;
    if (max_rows < 1 || max_rows > MAX_VERIFY) return BATTN_ERR_ARG;
    *out_x = nullptr;
    battn_xchg* x = new (std::nothrow) battn_xchg();
    if (!x) return BATTN_ERR_ARG;
    const Geom& g = h->g;
    x->h = h; x->world = world; x->rank = rank; x->max_items = max_rows * g.Hq;
    // [2 parities][world][items] records of HD + 2 words, every word paired with its step number (exact.cuh)
    x->rec_bytes = align_up((size_t)2 * world * x->max_items * (g.HD + 2) * 8, 256);
    x->bytes = x->rec_bytes;
    x->wait_polls = 1u << 17;                          // about 20 ms
    for (int d = 0; d < 8; ++d) { x->area[d] = nullptr; x->ipc_opened[d] = false; }
    cudaError_t e = cudaSetDevice(h->device);
    if (e == cudaSuccess) e = cudaMalloc(&x->area[rank], x->bytes);
    if (e == cudaSuccess) e = cudaMemset(x->area[rank], 0, x->bytes);      // step numbers start below every epoch >= 1
    if (e == cudaSuccess && ipc_handle_out) {
        cudaIpcMemHandle_t ih;
        e = cudaIpcGetMemHandle(&ih, x->area[rank]);
        if (e == cudaSuccess) memcpy(ipc_handle_out, &ih, sizeof(ih));
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (x->area[rank]) cudaFree(x->area[rank]);
        delete x;
        return cuda_fail(h, e);
    }
    *out_x = x;
    return BATTN_OK;
}

int battn_xchg_connect(battn_xchg* x, const void* all_ipc_handles) {
    if (!x || (!all_ipc_handles && x->world > 1)) return BATTN_ERR_ARG;
    cudaError_t e = cudaSetDevice(x->h->device);
    for (int d = 0; d < x->world && e == cudaSuccess; ++d) {
        if (d == x->rank || x->area[d]) continue;
        cudaIpcMemHandle_t ih;
        memcpy(&ih, reinterpret_cast<const uint8_t*>(all_ipc_handles) + (size_t)d * BATTN_IPC_HANDLE_BYTES, sizeof(ih));
        e = cudaIpcOpenMemHandle(&x->area[d], ih, cudaIpcMemLazyEnablePeerAccess);
        if (e == cudaSuccess) x->ipc_opened[d] = true;
    }
    return e == cudaSuccess ? BATTN_OK : cuda_fail(x->h, e);
}

int battn_xchg_connect_ptrs(battn_xchg* x, void* const* areas) {
    if (!x || !areas) return BATTN_ERR_ARG;
    for (int d = 0; d < x->world; ++d) {
        if (d == x->rank) continue;
        if (!areas[d] || ((uintptr_t)areas[d] & 255)) return BATTN_ERR_ARG;
        x->area[d] = areas[d];
    }
    return BATTN_OK;
}

int battn_xchg_area(const battn_xchg* x, void** out_ptr, size_t* out_bytes) {
    if (!x || !out_ptr || !out_bytes) return BATTN_ERR_ARG;
    *out_ptr = x->area[x->rank]; *out_bytes = x->bytes;
    return BATTN_OK;
}

int battn_xchg_set_wait_polls(battn_xchg* x, unsigned polls) {
    if (!x || polls < 1) return BATTN_ERR_ARG;
    x->wait_polls = polls;
    return BATTN_OK;
}

int battn_xchg_destroy(battn_xchg* x) {
    if (!x) return BATTN_ERR_ARG;
    cudaSetDevice(x->h->device);
    cudaDeviceSynchronize();
    for (int d = 0; d < x->world; ++d)
        if (x->ipc_opened[d]) cudaIpcCloseMemHandle(x->area[d]);
    if (x->area[x->rank]) cudaFree(x->area[x->rank]);
    delete x;
    return BATTN_OK;
}

int battn_partials_push(battn_handle* h, battn_xchg* x, void* out, const void* q, const uint8_t* kvk,
                        const uint8_t* kvv, const int* pos, const int* kslot, const int* act, void* ws, int rows,
                        int batch, int is_swa, int* epoch, int epoch_advance, void* stream) {
    const int rc = check_seq_args(h, q, q, kvk, kvv, pos, kslot, batch, rows, MAX_VERIFY);
    if (rc) return rc;
    if (!x || x->h != h || !ws || ((uintptr_t)ws & 15) || ((uintptr_t)out & 15) || !epoch || epoch_advance < 0) return BATTN_ERR_ARG;
    if (batch * rows * h->g.Hq > x->max_items) return BATTN_ERR_CAPACITY;
    for (int d = 0; d < x->world; ++d)
        if (!x->area[d]) return BATTN_ERR_ARG;                  // battn_xchg_connect has not run
    const XchgView v = xchg_view(x, epoch, 1, out != nullptr);
    return launch_flash(h, out, nullptr, q, kvk, kvv, pos, kslot, act, ws, batch, rows, is_swa, (cudaStream_t)stream, &v,
                        epoch, epoch_advance);
}

int battn_merge_wait(battn_handle* h, battn_xchg* x, void* out, int n_rows, const int* epoch, void* stream) {
    if (!h || !x || x->h != h || !out || ((uintptr_t)out & 15) || n_rows < 1 || !epoch) return BATTN_ERR_ARG;
    if (n_rows * h->g.Hq > x->max_items) return BATTN_ERR_CAPACITY;
    const Geom& g = h->g;
    MergeParams M{};
    M.out = out; M.out_f16 = g.out_f16; M.Hq = g.Hq; M.status = h->d_status;
    M.xchg = xchg_view(x, epoch, 0, 1);
    cudaError_t e;
    if (g.HD == 128) e = launch_pdl(k_merge_wait<128>, dim3(n_rows * g.Hq), dim3(32), 0, (cudaStream_t)stream, M);
    else             e = launch_pdl(k_merge_wait<256>, dim3(n_rows * g.Hq), dim3(64), 0, (cudaStream_t)stream, M);
    h->launches += 1;
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

int battn_merge(battn_handle* h, void* out, const float* parts, int n_parts, int n_rows, void* stream) {
    if (!h || !out || !parts || n_parts < 1 || n_rows < 1) return BATTN_ERR_ARG;
    if ((((uintptr_t)out | (uintptr_t)parts) & 15) != 0) return BATTN_ERR_ARG;
    if (n_parts > MERGE_MAX_COUNT) return BATTN_ERR_CAPACITY;
    const Geom& g = h->g;
    MergeParams M{};
    M.mode = MERGE_GATHERED; M.part = parts; M.out = out; M.rec_out = nullptr;
    M.n_rows = n_rows; M.rows = 1; M.Hq = g.Hq; M.Hkv = g.Hkv; M.G = g.G;
    M.count = n_parts; M.log2_domain = 0; M.out_f16 = g.out_f16; M.status = h->d_status;
    cudaStream_t st = (cudaStream_t)stream;
    if (g.HD == 128) k_merge<128><<<n_rows * g.Hq, MERGE_THREADS, 0, st>>>(M);
    else             k_merge<256><<<n_rows * g.Hq, MERGE_THREADS, 0, st>>>(M);
    h->launches += 1;
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

int battn_set_early_kv_stream(battn_handle* h, int enable) {
    if (!h) return BATTN_ERR_ARG;
    h->early_stream = enable != 0;
    return BATTN_OK;
}

int battn_device_status(battn_handle* h, int* out_bits, int clear) {
    if (!h || !out_bits) return BATTN_ERR_ARG;
    cudaError_t e = cudaMemcpy(out_bits, h->d_status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && clear) e = cudaMemset(h->d_status, 0, sizeof(int));
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

int battn_selftest_wait_timeout(battn_handle* h, unsigned poll_limit, void* stream) {
    if (!h || poll_limit < 1 || poll_limit > (1u << 22)) return BATTN_ERR_ARG;
    k_wait_selftest<<<1, 32, 0, (cudaStream_t)stream>>>(h->d_status, poll_limit);
    h->launches += 1;
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

int battn_profile_start(battn_handle* h, int max_launches) {
    if (!h || max_launches < 1 || h->prof_ev) return BATTN_ERR_ARG;
    cudaEvent_t* ev = new (std::nothrow) cudaEvent_t[2 * (size_t)max_launches];
    if (!ev) return BATTN_ERR_ARG;
    for (int i = 0; i < 2 * max_launches; ++i) {
        const cudaError_t e = cudaEventCreate(&ev[i]);
        if (e != cudaSuccess) {
            for (int j = 0; j < i; ++j) cudaEventDestroy(ev[j]);
            delete[] ev;
            return cuda_fail(h, e);
        }
    }
    h->prof_ev = ev; h->prof_cap = max_launches; h->prof_n = 0;
    return BATTN_OK;
}

int battn_profile_stop(battn_handle* h, float* ms_out, int cap, int* n_out) {
    if (!h || !h->prof_ev || !n_out) return BATTN_ERR_ARG;
    cudaError_t e = cudaSuccess;
    const int n = h->prof_n;
    if (n > 0) e = cudaEventSynchronize(h->prof_ev[2 * n - 1]);
    for (int i = 0; i < n && i < cap && ms_out && e == cudaSuccess; ++i)
        e = cudaEventElapsedTime(&ms_out[i], h->prof_ev[2 * i], h->prof_ev[2 * i + 1]);
    for (int i = 0; i < 2 * h->prof_cap; ++i) cudaEventDestroy(h->prof_ev[i]);
    delete[] h->prof_ev;
    h->prof_ev = nullptr; h->prof_cap = 0; h->prof_n = 0;
    *n_out = n;
    return e == cudaSuccess ? BATTN_OK : cuda_fail(h, e);
}

int battn_last_cuda_error(const battn_handle* h) { return h ? h->last_cuda_error : g_init_cuda_error; }

long long battn_launch_count(const battn_handle* h) { return h ? h->launches : 0; }

}  // extern "C"
