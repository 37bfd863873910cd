/*
 * battn.h -- C ABI of the B200 (sm_100a) attention hot path for the Bruce inference engine.
 *
 * The reference engine (engine/src/bruce.cu) has no FFI: its attention path is a handful of
 * `static` launches in one translation unit.  This header is the boundary a host engine binds
 * instead of those launches.  Every entry point cites the reference call it replaces.
 *
 * Conventions
 *   - Plain pointers and sizes only.  Every pointer named q/k/v/out/kvk/kvv/pos/kslot/act/ws is a
 *     DEVICE pointer owned by the caller (the reference allocates them once in alloc_buffers,
 *     bruce.cu:5460-5588) and merely borrowed for the duration of the call.
 *   - `stream` is a cudaStream_t passed as void*.  Launches are asynchronous and contain no
 *     allocation, no synchronisation and no host read of device state, so they can be recorded
 *     into a CUDA graph exactly like the reference's launches (bruce.cu:7877-7900, 8046-8055).
 *   - Positions are device-resident ints read inside the kernels (bruce.cu:653, 724, 1054), so a
 *     captured graph replays at new positions.
 *   - Every function returns an int status (BATTN_OK == 0).  Nothing prints, nothing exits
 *     (the reference's CK()/exit(1), bruce.cu:70-71, 3961-3962, becomes a status code).
 *
 * KV cache layout (bruce.cu:56-65, 690-693, 1888-1892, 5473-5503), one K and one V buffer per layer:
 *     [slot s][kv head h][position p'][record]
 *     record  = [HD/32 fp16 scales][HD int8 values]            (136 B for HD 128, 272 B for HD 256)
 *     address = base + ((s * n_kv + h) * pstride + p') * record_bytes
 *     pstride = slot_ctx (full-attention layer) or 2*window (sliding-window layer, a ring)
 *     p'      = p (full) or p & (2*window - 1) (sliding window)
 * Requirements added by this implementation: slot_ctx is even, window is a power of two >= 32, and EVERY
 * data pointer handed to an entry point (q, q_out, k, v, out, rec, parts, kvk, kvv, ws, sqk, cs, sn) is
 * 16-byte aligned: the kernels use 16-byte loads, stores and bulk copies.  A misaligned pointer is
 * rejected on the host with BATTN_ERR_ARG.
 */
#ifndef BATTN_H
#define BATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BATTN_VERSION 4

/* status codes */
enum {
    BATTN_OK            = 0,
    BATTN_ERR_ARG       = 1,   /* null pointer, unsupported geometry, rows out of range          */
    BATTN_ERR_CAPACITY  = 2,   /* more sequences / rows than the call supports                  */
    BATTN_ERR_CUDA      = 3,   /* a CUDA runtime call failed; battn_last_cuda_error() has it    */
    BATTN_ERR_DEVICE    = 4    /* a kernel recorded a fault (bad position, bounded wait ran out) */
};

/* element types of q and out */
enum { BATTN_F32 = 0, BATTN_F16 = 1 };

/* bits of the device status word (battn_device_status) */
enum {
    BATTN_DEV_BAD_POSITION = 1,  /* a row's position fell outside the cache; the row was skipped  */
    BATTN_DEV_WAIT_TIMEOUT = 2   /* a bounded in-kernel wait ran out; results of that launch void */
};

/* Geometry: the reference fixes these with #defines (bruce.cu:43-53); here they are run-time. */
typedef struct battn_geom {
    int   n_head;         /* query heads (reference 16; graded configs 32)                        */
    int   n_kv;           /* KV heads    (reference 4;  graded configs 8); n_head % n_kv == 0     */
    int   head_dim;       /* 128 or 256                                                           */
    int   window;         /* sliding window W (reference 1024; graded 4096); ring holds 2*W       */
    int   slot_ctx;       /* positions per slot in a full-attention layer (g_kv_nctx, :65, :5482) */
    int   n_slots;        /* KV partitions (serving slots, bruce.cu:90-94)                        */
    int   q_dtype;        /* BATTN_F32 (as the reference) or BATTN_F16                            */
    int   out_dtype;      /* BATTN_F32 (as the reference) or BATTN_F16                            */
    float softmax_scale;  /* 0 => 1/sqrt(head_dim) (0.0625 in the reference, bruce.cu:756)        */
} battn_geom;

typedef struct battn_handle battn_handle;

/* One-time set-up: replaces the lazy cudaFuncSetAttribute calls (bruce.cu:3948-3955, 4161-4168)
 * and the g_kv_nctx symbol upload (bruce.cu:5482).  Makes `device` current, allocates one small
 * device status word, sets every kernel attribute.  Call outside stream capture. */
int battn_init(const battn_geom* geom, int device, battn_handle** out_handle);
int battn_destroy(battn_handle* h);

/* Bytes of ONE layer's K (or V) buffer for all slots: the sizes alloc_buffers computes at
 * bruce.cu:5476-5481 (n_slots * pstride * n_kv * record_bytes). */
int battn_kv_layer_bytes(const battn_handle* h, int is_swa, size_t* out_bytes);

/* Bytes of the split-K scratch (`part` in the reference, bruce.cu:1058-1070, 5564) needed for a
 * call with up to n_seq sequences of up to rows_per_seq query rows each: a buffer of this size serves
 * every call with 1..rows_per_seq rows (a prompt's shorter last chunk included). */
int battn_workspace_bytes(const battn_handle* h, int n_seq, int rows_per_seq, size_t* out_bytes);

/* Bytes of scratch that ONE call of exactly (n_seq sequences x rows_per_seq rows) writes on a device with
 * num_sms multiprocessors -- the term battn_workspace_bytes maximises over all row counts up to its
 * argument.  Needs no handle and no device: hosts use it to size `part` before a device is initialised
 * (the reference sizes it from compile-time constants, bruce.cu:1058-1066), tests use it to check that
 * battn_workspace_bytes covers every shorter call.  0 for shapes that use no scratch. */
int battn_call_workspace_bytes(const battn_geom* geom, int num_sms, int n_seq, int rows_per_seq,
                               size_t* out_bytes);

/* Bytes of scratch battn_attend_exact needs for an explicit split count (the reference sizes
 * `part` as rows * nsplit records, bruce.cu:1060-1066). */
int battn_exact_workspace_bytes(const battn_handle* h, int n_seq, int rows_per_seq, int nsplit,
                                size_t* out_bytes);

/* KV append: the quantise-and-store half of k_qkv_prep (bruce.cu:690-710), k_qkv_prep_rows
 * (:1713-1725), k_qkv_prep_fast (:1789-1812) and k_qkv_prep_fast_ms (:1888-1918).
 *   k, v   fp32 [n_seq][rows_per_seq][n_kv][head_dim], already RoPE'd / normalised by the host
 *   kslot == NULL : single-sequence call.  kvk/kvv are that sequence's SLOT base (M.kvk_ptr[b]),
 *                   n_seq must be 1 and row r is stored at position pos[0] + r      (:1732, :7671)
 *   kslot != NULL : multi-slot call.  kvk/kvv are the LAYER base (M.kvk_layer[b]); sequence i
 *                   writes rows pos[i] .. pos[i]+rows_per_seq-1 of partition kslot[i]; sequences
 *                   with act[i] == 0 write nothing                                  (:1835-1869)
 * On a sliding-window layer one call may append at most 2*window rows per sequence (more would
 * alias ring slots inside one launch).
 * Per 32 values: d = amax/127.f, id = d ? 1.f/d : 0, q = lrintf(x*id), scale = fp16(d), no clamp.
 * The bytes written are identical to the reference's. */
int battn_kv_append(battn_handle* h, const float* k, const float* v, uint8_t* kvk, uint8_t* kvv,
                    const int* pos, const int* kslot, const int* act,
                    int n_seq, int rows_per_seq, int is_swa, void* stream);

/* Prefix sharing between slots: copies the cache of the first n_pos positions of partition src_slot into partition
 * dst_slot of the same layer (K and V, every kv head), so that a request whose prompt begins like another slot's
 * cached conversation starts its prompt at n_pos.  The reference reuses a prefix only inside ONE slot
 * (Session::cache_hit, engine/src/session.h:337-346, with the slot chosen by affinity, server.h:376-396); with its
 * contiguous per-slot partitions (bruce.cu:5471-5503) sharing across slots is a copy, and this is that copy.
 * kvk, kvv: the LAYER base pointers.  On a sliding-window layer the ring slots of the last min(n_pos, 2*window)
 * positions are copied.  Bytes are copied verbatim: the destination's records equal the source's. */
int battn_kv_copy_prefix(battn_handle* h, uint8_t* kvk, uint8_t* kvv, int src_slot, int dst_slot, int n_pos, int is_swa,
                         void* stream);

/* QKV prologue fused with the append, one launch: everything k_qkv_prep (bruce.cu:645-710),
 * k_qkv_prep_rows (:1656-1725), k_qkv_prep_fast (:1732-1812) and k_qkv_prep_fast_ms (:1835-1918) do.
 * Per row m = i*rows_per_seq + r (sequence i, row r, position pos[i] + r) and per head:
 *   scale = l2_scale(sum of squares, head_dim)                               (:305-307)
 *   NeoX rotate-half RoPE with the row's cos/sin table                       (:1757-1764)
 *   q additionally times sqk[head][dim]; k is then quantised into kvk, v is quantised RAW into kvv.
 *   q      fp32 [n_seq*rows_per_seq][n_head][head_dim] (read)
 *   q_out  same shape in the geometry's q_dtype: fp32 (may be q itself: the reference works in place) or
 *          fp16 (the operand the attention calls take; must not overlap q)
 *   k, v   fp32 [n_seq*rows_per_seq][n_kv][head_dim], sqk fp32 [n_head][head_dim]
 *   cs, sn fp32 [n_seq*rows_per_seq][head_dim]: per row two tables of head_dim/2 entries, theta_sel 1 uses
 *          the first, 2 the second (the reference's 256-float rows, :1739-1740); battn_rope_tables fills them
 *   kvk, kvv, pos, kslot, act, is_swa: exactly as battn_kv_append; idle sequences (act[i] == 0) still get
 *          their q prepared but write no KV (:1869)
 * Every fp32 step is performed in the order of the reference kernel as compiled by nvcc (fused multiply-adds
 * included): q_out (fp32) and the K/V bytes are bit-identical to the reference's. */
int battn_qkv_prep(battn_handle* h, void* q_out, const float* q, const float* k, const float* v,
                   const float* sqk, const float* cs, const float* sn, int theta_sel,
                   uint8_t* kvk, uint8_t* kvv, const int* pos, const int* kslot, const int* act,
                   int n_seq, int rows_per_seq, int is_swa, void* stream);

/* RoPE tables for the rows of one launch: k_rope_tables (bruce.cu:328-336), k_rope_tables_rows (:1641-1654)
 * and k_rope_tables_rows_ms (:1821-1833).  Row m = i*rows_per_seq + r gets, for position p = pos[i] + r and
 * j < head_dim/2: cs[m][j] = cosf(p * powf(1e7, -2j/head_dim)), cs[m][head_dim/2 + j] the same with base 1e4,
 * sn likewise with sinf.  cs, sn: fp32 [n_seq*rows_per_seq][head_dim]. */
int battn_rope_tables(battn_handle* h, float* cs, float* sn, const int* pos, int n_seq, int rows_per_seq,
                      void* stream);

/* Decode attention, one query row per sequence, normalised output:
 * launch_attn_m(rows = 1) + k_attn_combine_fast (bruce.cu:3942-3963, 928-990, call :7958-7969)
 * when kslot == NULL, launch_attn_ms (bruce.cu:4158-4177, call :7720) when kslot != NULL.
 *   q, out [n_seq][n_head][head_dim] in q_dtype / out_dtype; row i attends keys
 *   [kstart, pos[i]] of its partition, kstart = is_swa ? max(0, pos[i]+1-window) : 0  (:724-729).
 *   Rows with act[i] == 0 produce no output and touch no KV (:3398-3406). */
int battn_decode(battn_handle* h, void* out, const void* q, const uint8_t* kvk, const uint8_t* kvv,
                 const int* pos, const int* kslot, const int* act, void* ws,
                 int n_seq, int is_swa, void* stream);

/* Decode that appends its own row: battn_kv_append (one row per sequence) and battn_decode in ONE launch pair.
 *   k, v   fp32 [n_seq][n_kv][head_dim], already RoPE'd / normalised (as for battn_kv_append)
 * The CTA of the decode kernel that streams the tile of position pos[i] quantises the row of its kv head -- with the
 * append kernel's own quantiser, so the cache bytes are those battn_kv_append writes -- into that tile in shared memory
 * and into the cache, before the tile is used.  Saves the append launch and the kernel boundary between it and the
 * attention kernel (about 2.7 us per call).  For hosts that keep their own prologue kernel; hosts that use
 * battn_qkv_prep (prologue and append fused) call battn_decode after it as before.
 * With early KV streaming on: the merge of this call releases its successor before the decode kernel that wrote
 * the row has finished, so a decode call never streams the tile of the row before its own early, and a verify or
 * prompt call that follows streams early only from a different cache (kvk pointer, or pool). */
int battn_decode_append(battn_handle* h, void* out, const void* q, const float* k, const float* v, uint8_t* kvk,
                        uint8_t* kvv, const int* pos, const int* kslot, const int* act, void* ws, int n_seq, int is_swa,
                        void* stream);

/* Decode that runs the QKV prologue of its row itself: battn_qkv_prep (one row per sequence) and battn_decode in ONE
 * launch pair.  q, k, v, sqk, cs, sn, theta_sel: the RAW inputs, exactly as for battn_qkv_prep.  Every CTA of the decode
 * kernel prepares the query heads it needs (L2 scale, RoPE, sqk; rounded to fp16 as the attention kernels take them), the
 * CTA that streams the tile of position pos[i] prepares and quantises the K row and quantises the V row of its kv head:
 * the same device functions as the prologue kernel, so cache bytes and output bits are those of battn_qkv_prep followed
 * by battn_decode.  The prepared q is not written anywhere.  Same rule for early KV streaming as battn_decode_append. */
int battn_qkv_decode(battn_handle* h, void* out, const float* q, const float* k, const float* v, const float* sqk,
                     const float* cs, const float* sn, int theta_sel, uint8_t* kvk, uint8_t* kvv, const int* pos,
                     const int* kslot, const int* act, void* ws, int n_seq, int is_swa, void* stream);

/* Decode attention for callers that cannot hand the library a scratch buffer.  (This entry point has
 * no counterpart in the reference, whose host always owns a `part` allocation.)
 *
 * Some hosts cannot call cudaMalloc once they are running: an inference server that gave every byte of
 * HBM to its KV pool at start-up has nothing left to allocate from, and a latency-critical decode loop
 * cannot afford the implicit device-wide synchronisation an allocation may cause.  For them this variant
 * of battn_decode takes no `ws`: its split-K scratch is a fixed array of BATTN_NOALLOC_SCRATCH_BYTES that
 * lives inside the library image, so every GPU that loads the library holds that much memory until the
 * process exits.  The call itself allocates nothing, on the host or on the device.
 *
 *   - Same arguments, results and status codes as battn_decode, minus `ws`.
 *   - battn_init() resolves the array's device address once for the handle's device (with that device
 *     current), so there is no first-call set-up cost here; call battn_init outside stream capture.
 *   - A call whose scratch need exceeds the array (about 175 sequences at 8 KV heads / head_dim 128,
 *     about 100 at 4 KV heads / head_dim 256) is rejected with BATTN_ERR_CAPACITY before anything is
 *     launched.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  The kernels
 *     overwrite every word they later read, so nothing needs clearing between calls, but two calls that
 *     overlap on the GPU (different streams, or different handles on the same device) race on it:
 *     issue them on one stream or serialise them yourself. */
#define BATTN_NOALLOC_SCRATCH_BYTES (4u << 20)
int battn_decode_noalloc(battn_handle* h, void* out, const void* q, const uint8_t* kvk,
                         const uint8_t* kvv, const int* pos, const int* kslot, const int* act,
                         int n_seq, int is_swa, void* stream);

/* Speculative-verify attention: `rows` (1..8) query rows at positions pos[i] .. pos[i]+rows-1 that
 * share one sweep over sequence i's KV and are causal among themselves:
 * launch_attn_m(rows 2..8) + k_attn_combine_rows (bruce.cu:3965-4019, 1999-2016; exact form
 * k_attn_m<M> :2087-2143).  Row r sees keys [lo_r, pos[i]+r], lo_r = is_swa ?
 * max(0, pos[i]+r-window+1) : 0 (:3686-3689, :2056).  `batch` sequences are processed in one call
 * (kslot/act as in battn_decode; kslot == NULL requires batch == 1).
 *   q, out [batch][rows][n_head][head_dim]. */
int battn_verify(battn_handle* h, void* out, const void* q, const uint8_t* kvk, const uint8_t* kvv,
                 const int* pos, const int* kslot, const int* act, void* ws,
                 int rows, int batch, int is_swa, void* stream);

/* Prompt-chunk attention: `rows` (1..512) query rows at pos[0] .. pos[0]+rows-1 against the cache
 * AFTER the chunk's own K/V were appended: launch_attn_m(rows > 8) + the merge
 * (bruce.cu:4021-4078, 2750-3131, call :7729-7732).  Causal plus optional window.
 *   q, out [rows][n_head][head_dim].  kvk/kvv are the slot base.
 *   ws: scratch of battn_workspace_bytes(1, rows) bytes.  When the chunk's (M tile, kv head) grid would leave
 *   SMs idle, several CTAs share an M tile over disjoint key ranges and leave split records there, which a merge
 *   launch turns into `out` (the reference's own prompt kernel does the same with its `ns` splits, :7696-7706). */
int battn_prefill(battn_handle* h, void* out, const void* q, const uint8_t* kvk, const uint8_t* kvv,
                  const int* pos, void* ws, int rows, int is_swa, void* stream);

/* The step after attention: sigmoid gate, L2 norm over the token's whole attention vector and the q8 activation copy
 * for the output projection -- k_gate_norm_vec4 (bruce.cu:1526-1568; calls :7746-7755, :7975).  Per token row m with
 * n = n_head * head_dim (a multiple of 1024, at most 4096):
 *     t = aout / (1 + __expf(-(gate * sgate))),  k = l2_scale(sum t^2, n) (:305-307),  v = t * k
 *     per 32 values: d = amax * (1/127), q = clamp(rint(v / d), -127, 127)   (the ACTIVATION quantiser, :1405-1428)
 *   aout  [rows][n] in out_dtype        gate [rows][n] fp32        sgate [n] fp32
 *   dst   [rows][n] fp32 or NULL        xq [rows][n] int8          xd [rows][n/32] fp32      xsum [rows][n/32] int32
 * Sums are formed in the reference kernel's order: for fp32 aout the outputs are bit-identical to k_gate_norm_vec4's. */
int battn_gate_norm(battn_handle* h, float* dst, const void* aout, const float* gate, const float* sgate, int8_t* xq,
                    float* xd, int* xsum, int rows, void* stream);

/* Prompt-chunk attention fused with that step: battn_prefill whose result never goes to memory as an attention
 * output -- the chunk's split records are merged, gated, normalised and quantised by one block per token row, as
 * the reference's k_combine_gate_norm_rows_opt does with its own records (bruce.cu:1577-1639, call :7743).
 * Arguments as battn_prefill (without `out`) and battn_gate_norm (without `aout`); rows * (n_head / n_kv) > 32
 * (shorter calls: battn_decode / battn_verify followed by battn_gate_norm). */
int battn_prefill_gate_norm(battn_handle* h, float* dst, const void* q, const uint8_t* kvk, const uint8_t* kvv,
                            const int* pos, void* ws, const float* gate, const float* sgate, int8_t* xq, float* xd,
                            int* xsum, int rows, int is_swa, void* stream);

/* The exact fp32 path: per-key online softmax in fp32 with no tensor cores, the same arithmetic as
 * k_attn / k_attn_rows / k_attn_m (bruce.cu:713-785, 1921-1997, 2087-2143) followed by
 * k_attn_combine_rows (:1999-2016).  Any rows_per_seq >= 1.  `nsplit` (1..128) is the reference's
 * split count (key range rule :724-729).  Same argument meaning as battn_verify. */
int battn_attend_exact(battn_handle* h, void* out, const void* q, const uint8_t* kvk,
                       const uint8_t* kvv, const int* pos, const int* kslot, const int* act,
                       void* ws, int n_seq, int rows_per_seq, int nsplit, int is_swa, void* stream);

/* Partial records for a sequence split across devices: like battn_verify, but instead of the
 * normalised output each (sequence, row, head) yields the reference's split record
 * (bruce.cu:781-783, 1058-1070): head_dim fp32 unnormalised o, then m (max score, natural-log
 * units), then l (sum of exp(score - m)).
 *   rec fp32 [batch][rows][n_head][head_dim + 2].  An empty key range gives (0, -1e30, 0). */
int battn_partials(battn_handle* h, float* rec, const void* q, const uint8_t* kvk,
                   const uint8_t* kvv, const int* pos, const int* kslot, const int* act, void* ws,
                   int rows, int batch, int is_swa, void* stream);

/* Early KV streaming (off by default; battn_set_early_kv_stream(h, 1) turns it on for the handle).  The decode and
 * 2..4-row verify kernels and the prompt kernels are launched so that they may start while the previous kernel of the stream is still
 * running; with this option they read pos / kslot / act and begin to stream the cache tiles that lie entirely below
 * the call's first position before that kernel has finished, while Q, the tile holding the call's own rows and every
 * write wait for it (about 0.8 us less per call).  The host promises that the kernel which precedes the call in the
 * stream writes neither pos / kslot / act (nor the page table of a paged call) nor cache rows other than the call's own (pos[i] .. pos[i]+rows-1) --
 * the reference's step order: positions uploaded by a copy at the start of the step (bruce.cu:8043, 8259),
 * k_qkv_prep* right before the attention launch (:7667-7732).  Copies and graph launches order fully and are always
 * safe predecessors.  The library additionally checks what it can see: a call streams early only if the last launch
 * on this handle was not a cache write, or was the append / prologue of exactly these rows (same pos pointer,
 * sequence and row counts). */
int battn_set_early_kv_stream(battn_handle* h, int enable);

/* Log-sum-exp merge of n_parts records per (row, head): k_attn_combine (bruce.cu:992-1007).
 *   parts fp32 [n_parts][n_rows][n_head][head_dim + 2]; out [n_rows][n_head][head_dim] out_dtype.
 *   out = sum_s o_s e^(m_s-M) / sum_s l_s e^(m_s-M), M = max_s m_s; empty records contribute 0. */
int battn_merge(battn_handle* h, void* out, const float* parts, int n_parts, int n_rows,
                void* stream);

/* ---- Paged cache of a full-causal layer -----------------------------------------------------------------------
 * The reference gives every slot one contiguous partition of ctx/N positions (alloc_buffers, bruce.cu:5471-5503),
 * so a short conversation reserves as much memory as the longest one may use, and two slots whose prompts share a
 * prefix each hold their own copy (prefix reuse is per slot, engine/src/session.h:337-346).  With a paged cache
 * the layer is a pool of pages; a page holds page_len consecutive positions of every kv head,
 *     page p, kv head h, position-in-page j  ->  pool + ((p * n_kv + h) * page_len + j) * record bytes,
 * records exactly as in the contiguous layout, so a key tile of one head is still one contiguous run and every
 * kernel streams it the same way.  `table` (device memory, int32 [n_tables][max_pages]) maps logical page
 * pos / page_len of a sequence to a physical page; it is read by the kernels, so a host may edit it between
 * launches without re-capturing graphs.  Sequences that share a prefix point at the same physical pages (the
 * host un-shares the page a sequence is about to append into).  `ktab[i]` is the table row of sequence i, in
 * place of the partition number `kslot[i]` of the contiguous calls; ktab == NULL means one sequence using row 0.
 * A table entry outside [0, n_pages) sets BATTN_DEV_BAD_POSITION (the access is redirected to page 0, in bounds).
 * Sliding-window layers keep their 2*window ring per slot (a bounded allocation already) and use the contiguous
 * calls.  Results equal those of the contiguous calls on the same records, bit for bit. */
typedef struct battn_pages {
    uint8_t* pool_k;     /* n_pages pages of n_kv * page_len records (battn_pages_pool_bytes), 16-byte aligned */
    uint8_t* pool_v;
    const int* table;    /* device, [n_tables][max_pages] */
    int n_pages, n_tables, max_pages;
    int page_len;        /* positions per page: a power of two, 128 .. 65536 */
} battn_pages;
int battn_pages_pool_bytes(const battn_handle* h, int n_pages, int page_len, size_t* out_bytes);
/* Copy on write: the K and V records of physical page from_page copied into to_page (two device-to-device copies on
 * `stream`), for a sequence that is about to append into a page it shares with another one. */
int battn_pages_copy(battn_handle* h, const battn_pages* pages, int from_page, int to_page, void* stream);
/* as battn_kv_append / battn_decode (battn_decode_append, battn_qkv_decode) / battn_verify / battn_prefill (more than
 * 32 / group rows; one sequence, table row `table_row`) / battn_attend_exact, is_swa = 0 */
int battn_kv_append_paged(battn_handle* h, const battn_pages* pages, const float* k, const float* v, const int* pos,
                          const int* ktab, const int* act, int n_seq, int rows_per_seq, void* stream);
/* as battn_qkv_prep (the whole prologue fused with the append), storing into the pages */
int battn_qkv_prep_paged(battn_handle* h, void* q_out, const float* q, const float* k, const float* v, const float* sqk,
                         const float* cs, const float* sn, int theta_sel, const battn_pages* pages, const int* pos,
                         const int* ktab, const int* act, int n_seq, int rows_per_seq, void* stream);
int battn_decode_paged(battn_handle* h, void* out, const void* q, const battn_pages* pages, const int* pos,
                       const int* ktab, const int* act, void* ws, int n_seq, void* stream);
int battn_decode_append_paged(battn_handle* h, void* out, const void* q, const float* k, const float* v,
                              const battn_pages* pages, const int* pos, const int* ktab, const int* act, void* ws,
                              int n_seq, void* stream);
int battn_qkv_decode_paged(battn_handle* h, void* out, const float* q, const float* k, const float* v, const float* sqk,
                           const float* cs, const float* sn, int theta_sel, const battn_pages* pages, const int* pos,
                           const int* ktab, const int* act, void* ws, int n_seq, void* stream);
int battn_verify_paged(battn_handle* h, void* out, const void* q, const battn_pages* pages, const int* pos,
                       const int* ktab, const int* act, void* ws, int rows, int batch, void* stream);
int battn_prefill_paged(battn_handle* h, void* out, const void* q, const battn_pages* pages, int table_row,
                        const int* pos, void* ws, int rows, void* stream);
int battn_attend_exact_paged(battn_handle* h, void* out, const void* q, const battn_pages* pages, const int* pos,
                             const int* ktab, const int* act, void* ws, int n_seq, int rows_per_seq, int nsplit,
                             void* stream);

/* ---- One sequence split by position range across several devices (no counterpart in the reference, which is
 * single-GPU; built on its split record and merge, bruce.cu:781-783, 992-1007) ------------------------------------
 * Device r of `world` holds positions [r*N/world, (r+1)*N/world) of the sequence in its own cache, with LOCAL
 * positions.  A decode step runs the ordinary split-K decode on every shard; the epilogue of that kernel stores the
 * shard's merged record (o, m, l) of every (row, head) straight into a receive area on EVERY device of the group
 * (plain 16-byte stores through peer-mapped pointers over NVLink, every payload word paired with the step number:
 * no fence and no separate flag), and then waits -- bounded -- until the words of the other devices' records carry
 * the step's number locally and merges them.
 * No collective library call, no host round trip: one decode + one merge launch per step per device.
 *
 * battn_xchg_create allocates this device's receive area (cudaMalloc; call outside stream capture) and returns a
 * BATTN_IPC_HANDLE_BYTES-byte handle the host passes to the other processes by whatever transport it has;
 * battn_xchg_connect maps the peers' areas from their handles (`all_ipc_handles`: world handles in rank order;
 * the own entry is ignored).  A host that drives several devices from ONE process exchanges raw pointers
 * instead (battn_xchg_area / battn_xchg_connect_ptrs, after enabling peer access itself).
 *
 * battn_partials_push: arguments as battn_partials, minus `rec`.  `epoch` points to this device's step counter in
 * DEVICE memory (4 bytes the host allocates and zeroes once, together with the exchange object: the counter never goes
 * back while the object lives, stale records are told from fresh ones by it); the call adds `epoch_advance` to it on
 * the device before use -- 1 in the normal case, so that a captured graph replays at successive steps; 1 + k after this
 * device sat out k steps of the group -- and the resulting step number must be the same on every device.  With
 * out != NULL the same launch also performs the wait-and-merge and writes the normalised output
 * [batch*rows][n_head][head_dim]; with out == NULL it only pushes and battn_merge_wait finishes the step later.
 * A device whose shard holds no visible key passes act = {0}: it pushes the empty record.
 * If a peer's record does not arrive within the wait bound (battn_xchg_set_wait_polls, polls of ~100 ns, default
 * 2^17), the launch sets BATTN_DEV_WAIT_TIMEOUT in the device status word, leaves `out` untouched and returns
 * normally; the next step can proceed. */
#define BATTN_IPC_HANDLE_BYTES 64
typedef struct battn_xchg battn_xchg;
int battn_xchg_create(battn_handle* h, int rank, int world, int max_rows, battn_xchg** out_x, void* ipc_handle_out);
int battn_xchg_connect(battn_xchg* x, const void* all_ipc_handles);
int battn_xchg_area(const battn_xchg* x, void** out_ptr, size_t* out_bytes);
int battn_xchg_connect_ptrs(battn_xchg* x, void* const* areas);
int battn_xchg_set_wait_polls(battn_xchg* x, unsigned polls);
int battn_xchg_destroy(battn_xchg* x);
int battn_partials_push(battn_handle* h, battn_xchg* x, void* out, const void* q, const uint8_t* kvk,
                        const uint8_t* kvv, const int* pos, const int* kslot, const int* act, void* ws, int rows,
                        int batch, int is_swa, int* epoch, int epoch_advance, void* stream);
int battn_merge_wait(battn_handle* h, battn_xchg* x, void* out, int n_rows, const int* epoch, void* stream);

/* Device status word (bits BATTN_DEV_*), read with a blocking copy; clears it when `clear` != 0.
 * Not for use inside stream capture. */
int battn_device_status(battn_handle* h, int* out_bits, int clear);

/* Self-test of the bounded waits: launches one tiny kernel in which a thread waits, with the same
 * bounded mbarrier wait the attention kernels use, on a barrier nothing ever arrives on; after
 * poll_limit polls (1 .. 1<<22) the wait gives up, the kernel sets BATTN_DEV_WAIT_TIMEOUT in the device
 * status word and returns normally.  Shows that a wait that runs out is reported through
 * battn_device_status and leaves the context usable.  (The reference has no bounded waits: its kernels
 * use __syncthreads only, and a stuck launch is a hung process.) */
int battn_selftest_wait_timeout(battn_handle* h, unsigned poll_limit, void* stream);

/* Per-kernel timing, the counterpart of the reference's --probe CUDA-event phase timing
 * (bruce.cu:8334-8397).  Between battn_profile_start and battn_profile_stop every attention call
 * brackets its MAIN kernel (flash-decode / prefill; not the merge) with a pair of CUDA events on the
 * caller's stream, up to max_launches pairs.  battn_profile_stop synchronises on the last event and
 * returns the elapsed milliseconds of each bracketed launch in call order.  Not capturable. */
int battn_profile_start(battn_handle* h, int max_launches);
int battn_profile_stop(battn_handle* h, float* ms_out, int cap, int* n_out);

/* cudaError_t of the last failing runtime call on this handle (0 if none); with h == NULL, of the
 * last failing battn_init. */
int battn_last_cuda_error(const battn_handle* h);

/* Number of kernels this library has launched through `h` since init (for launch accounting). */
long long battn_launch_count(const battn_handle* h);

int battn_version(void);

#ifdef __cplusplus
}
#endif
#endif /* BATTN_H */
