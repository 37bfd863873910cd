/*
 * battn_bruce_shim.h -- drop-in shim for the reference engine's attention call sites.
 *
 * The reference (engine/src/bruce.cu) launches its attention kernels through a handful of `static`
 * functions.  Including this header after `#include "battn.h"` gives the host code functions with the
 * reference's own names, argument order and meaning, implemented by the C ABI, so the call sites at
 * bruce.cu:7665-7761 (batched) and :7936-7980 (single row) change by a rename at most.
 *
 * What differs from the reference, by design:
 *   - two forms of the append: `qkv_prep_rows` / `qkv_prep_ms` do everything k_qkv_prep* does in one launch
 *     (L2 norm, NeoX RoPE, sqk scale, quantised store; bruce.cu:657-710, 1742-1812), bit-identical to the
 *     reference; `kv_append_*` is only the quantise-and-store half (:690-710) for hosts whose k and v
 *     arrive already RoPE'd and normalised.
 *   - launch_attn_m / launch_attn_ms write the NORMALISED output and ignore `ns`: the host then takes its
 *     existing ns == 1 branch (k_gate_norm_vec4 on `out`, bruce.cu:7745-7751) and never launches
 *     k_attn_combine* / k_combine_gate_norm_rows_opt.
 *   - a non-zero status is reported through battn_shim_fail() (default: print and exit(1), the
 *     reference's CK() behaviour, bruce.cu:70-71); hosts that want to recover install their own.
 */
#ifndef BATTN_BRUCE_SHIM_H
#define BATTN_BRUCE_SHIM_H

#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>

#include "battn.h"

static battn_handle* g_battn = nullptr;   /* set once by battn_shim_init() from alloc_buffers() */
static int g_battn_group = 1;             /* query heads per KV head */

static inline void battn_shim_fail(const char* what, int rc) {
    std::fprintf(stderr, "battn: %s failed with status %d (cudaError %d)\n", what, rc,
                 battn_last_cuda_error(g_battn));
    std::exit(1);
}
#define BATTN_CK(call) do { int rc_ = (call); if (rc_) battn_shim_fail(#call, rc_); } while (0)

/* alloc_buffers() (bruce.cu:5460-5507): geometry from the engine's #defines / model fields.
 * Replaces the g_kv_nctx upload (:5482) and the lazy cudaFuncSetAttribute calls (:3948-3955). */
static inline void battn_shim_init(int n_head, int n_kv, int hd, int swa, int slot_ctx, int n_slots) {
    battn_geom g = {n_head, n_kv, hd, swa, slot_ctx, n_slots, BATTN_F32, BATTN_F32, 0.f};
    BATTN_CK(battn_init(&g, 0, &g_battn));
    g_battn_group = n_head / n_kv;
    /* The engine's step order is the one early KV streaming asks for: positions reach the device by copies
     * (bruce.cu:8043, 8259) or by k_advance at the END of a step (:8051), and the kernel in front of every
     * attention launch is the prologue that writes that step's rows (:7667-7732). */
    BATTN_CK(battn_set_early_kv_stream(g_battn, 1));
}
/* size of M.part (bruce.cu:5564): rows = MBUF for the prompt path */
static inline size_t battn_shim_part_bytes(int max_slots, int max_rows) {
    size_t a = 0, b = 0;
    BATTN_CK(battn_workspace_bytes(g_battn, max_slots, 8, &a));
    BATTN_CK(battn_workspace_bytes(g_battn, 1, max_rows, &b));
    return a > b ? a : b;
}

/* store half of k_qkv_prep / k_qkv_prep_fast (bruce.cu:644, 1732; calls :7671, :7941):
 * rows of ONE sequence at *pos .. *pos+rows-1, kvk/kvv = slot base (M.kvk_ptr[b]) */
static inline void kv_append_rows(const float* k, const float* v, uint8_t* kvk, uint8_t* kvv, const int* pos,
                                  int rows, int is_swa, cudaStream_t st) {
    BATTN_CK(battn_kv_append(g_battn, k, v, kvk, kvv, pos, nullptr, nullptr, 1, rows, is_swa, st));
}
/* store half of k_qkv_prep_fast_ms (bruce.cu:1835; call :7667): one row per slot, layer base pointers */
static inline void kv_append_ms(const float* k, const float* v, uint8_t* kvk_layer, uint8_t* kvv_layer,
                                const int* pos, const int* kslot, const int* act, int rows, int is_swa,
                                cudaStream_t st) {
    BATTN_CK(battn_kv_append(g_battn, k, v, kvk_layer, kvv_layer, pos, kslot, act, rows, 1, is_swa, st));
}

/* k_qkv_prep / k_qkv_prep_rows / k_qkv_prep_fast as launched at bruce.cu:7671-7675, :7941: the whole prologue
 * (L2 scale, RoPE, sqk) and the append for rows of ONE sequence; q is prepared in place like the reference's */
static inline void qkv_prep_rows(float* q, const float* k, const float* v, const float* sqk, uint8_t* kvk,
                                 uint8_t* kvv, const int* pos, int rows, int is_swa, int theta_sel,
                                 const float* cs, const float* sn, cudaStream_t st) {
    BATTN_CK(battn_qkv_prep(g_battn, q, q, k, v, sqk, cs, sn, theta_sel, kvk, kvv, pos, nullptr, nullptr, 1, rows,
                            is_swa, st));
}
/* k_qkv_prep_fast_ms as launched at bruce.cu:7667: one row per slot, layer base pointers */
static inline void qkv_prep_ms(float* q, const float* k, const float* v, const float* sqk, uint8_t* kvk_layer,
                               uint8_t* kvv_layer, const int* pos, const int* kslot, const int* act, int rows,
                               int is_swa, int theta_sel, const float* cs, const float* sn, cudaStream_t st) {
    BATTN_CK(battn_qkv_prep(g_battn, q, q, k, v, sqk, cs, sn, theta_sel, kvk_layer, kvv_layer, pos, kslot, act, rows,
                            1, is_swa, st));
}
/* k_rope_tables_rows (bruce.cu:7625) and k_rope_tables_rows_ms (:7623) */
static inline void rope_tables_rows(float* cs, float* sn, const int* pos, int rows, cudaStream_t st) {
    BATTN_CK(battn_rope_tables(g_battn, cs, sn, pos, 1, rows, st));
}
static inline void rope_tables_rows_ms(float* cs, float* sn, const int* row_pos, int rows, cudaStream_t st) {
    BATTN_CK(battn_rope_tables(g_battn, cs, sn, row_pos, rows, 1, st));
}

/* launch_attn_m (bruce.cu:3942; calls :7729, :7732, :7958) with the merge folded in */
static inline void launch_attn_m(float* out, const float* q, const uint8_t* kvk, const uint8_t* kvv,
                                 const int* pos, float* part, int rows, int /*ns*/, int is_swa, cudaStream_t st) {
    /* battn_verify shares one KV sweep among at most 32 (row, head) pairs per KV head; geometries with more
     * than 4 query heads per KV head reach that limit before 8 rows and take the prompt-chunk path instead */
    const int group = g_battn_group;
    if (rows == 1)                             BATTN_CK(battn_decode(g_battn, out, q, kvk, kvv, pos, nullptr, nullptr, part, 1, is_swa, st));
    else if (rows <= 8 && rows * group <= 32)  BATTN_CK(battn_verify(g_battn, out, q, kvk, kvv, pos, nullptr, nullptr, part, rows, 1, is_swa, st));
    else                                       BATTN_CK(battn_prefill(g_battn, out, q, kvk, kvv, pos, part, rows, is_swa, st));
}

/* The decode step's pair of launches -- k_qkv_prep_fast then launch_attn_m with rows == 1 (bruce.cu:7671-7675, :7729)
 * or k_qkv_prep_fast_ms then launch_attn_ms (:7667, :7720) -- as ONE call: the decode kernel prepares q, prepares and
 * appends the K/V row and attends.  Same cache bytes and outputs; q is left as it was (the prepared q is not stored). */
static inline void qkv_prep_attn_m1(float* out, const float* q, const float* k, const float* v, const float* sqk,
                                    uint8_t* kvk, uint8_t* kvv, const int* pos, float* part, int is_swa, int theta_sel,
                                    const float* cs, const float* sn, cudaStream_t st) {
    BATTN_CK(battn_qkv_decode(g_battn, out, q, k, v, sqk, cs, sn, theta_sel, kvk, kvv, pos, nullptr, nullptr, part, 1,
                              is_swa, st));
}
static inline void qkv_prep_attn_ms(float* out, const float* q, const float* k, const float* v, const float* sqk,
                                    uint8_t* kvk_layer, uint8_t* kvv_layer, const int* pos, const int* kslot,
                                    const int* act, float* part, int rows, int is_swa, int theta_sel, const float* cs,
                                    const float* sn, cudaStream_t st) {
    BATTN_CK(battn_qkv_decode(g_battn, out, q, k, v, sqk, cs, sn, theta_sel, kvk_layer, kvv_layer, pos, kslot, act, part,
                              rows, is_swa, st));
}

/* launch_attn_ms (bruce.cu:4158; call :7720) with the merge folded in */
static inline void launch_attn_ms(float* out, const float* q, const uint8_t* kvk, const uint8_t* kvv,
                                  const int* pos, const int* kslot, const int* act, float* part, int rows,
                                  int /*ns*/, int is_swa, cudaStream_t st) {
    BATTN_CK(battn_decode(g_battn, out, q, kvk, kvv, pos, kslot, act, part, rows, is_swa, st));
}

/* k_gate_norm_vec4 as launched at bruce.cu:7746-7755 and :7975 (the host's ns == 1 branch, which this library's
 * normalised outputs always take): sigmoid gate, L2 norm, q8 copy of `rows` attention rows; dst may be null */
static inline void gate_norm_rows(float* dst, const float* aout, const float* gate, const float* sgate, int8_t* xq,
                                  float* xd, int* xsum, int rows, cudaStream_t st) {
    BATTN_CK(battn_gate_norm(g_battn, dst, aout, gate, sgate, xq, xd, xsum, rows, st));
}
/* launch_attn_m(rows > 8) followed by k_combine_gate_norm_rows_opt<16> (bruce.cu:7729-7743) in one call: the
 * prompt chunk's attention output never goes to memory */
static inline void attn_gate_norm_rows(const float* q, const uint8_t* kvk, const uint8_t* kvv, const int* pos, float* part,
                                       const float* gate, const float* sgate, int8_t* xq, float* xd, int* xsum, int rows,
                                       int is_swa, cudaStream_t st) {
    BATTN_CK(battn_prefill_gate_norm(g_battn, nullptr, q, kvk, kvv, pos, part, gate, sgate, xq, xd, xsum, rows, is_swa, st));
}

/* --prefill-tc 0 / BRUCE_ATTN_M1PATH=0: the exact fp32 path, k_attn_rows + k_attn_combine_rows
 * (bruce.cu:7735, 7753) */
static inline void launch_attn_exact(float* out, const float* q, const uint8_t* kvk, const uint8_t* kvv,
                                     const int* pos, float* part, int rows, int ns, int is_swa, cudaStream_t st) {
    BATTN_CK(battn_attend_exact(g_battn, out, q, kvk, kvv, pos, nullptr, nullptr, part, 1, rows, ns, is_swa, st));
}

#endif /* BATTN_BRUCE_SHIM_H */
