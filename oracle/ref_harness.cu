// Harness around the reference engine's OWN attention kernels (test infrastructure only).
//
// Built by oracle/ref_build.py, and only where the reference tree is present: the reference's
// translation unit (engine/src/bruce.cu) is included unmodified from a temporary copy (its main() is
// renamed away), and a few extern "C" entry points launch its static kernels on caller-provided device
// buffers.  Nothing of the reference is copied into this repository; the resulting library lives in
// oracle/_ref/ and is used by tests to pin this repository's kernels and oracle against the reference's
// kernels in the reference's native geometry (16 q-heads / 4 KV heads / head_dim 256 / window 1024).
#define main bruce_reference_main
#include "bruce.cu"
#undef main

extern "C" {

// {N_HEAD, N_KV, HD, SWA, SWA_SLOTS, KV_KVH_BYTES, PART_MAX_SPLITS}
void ref_geometry(int* out) {
    out[0] = N_HEAD; out[1] = N_KV; out[2] = HD; out[3] = SWA; out[4] = SWA_SLOTS; out[5] = KV_KVH_BYTES;
    out[6] = PART_MAX_SPLITS;
}

static int ref_sync_status() {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return (int)e;
}

static void ref_set_nctx(int nctx) { cudaMemcpyToSymbol(g_kv_nctx, &nctx, sizeof(nctx)); }

// The reference's append kernel for a chunk of rows of one sequence, k_qkv_prep_fast (bruce.cu:1732):
// L2-norm + RoPE + sqk scale on q (in place) and k, then q8_0 quantise k and RAW v into the cache.
// cs / sn: [rows][256] RoPE tables, sqk: [N_HEAD][HD]; all device pointers.
int ref_kv_append(float* q, const float* k, const float* v, const float* sqk, uint8_t* kvk, uint8_t* kvv,
                  const int* d_pos, int rows, int is_swa, int nctx, const float* cs, const float* sn) {
    ref_set_nctx(nctx);
    k_qkv_prep_fast<<<rows, 256>>>(q, k, v, sqk, kvk, kvv, d_pos, is_swa, 1, cs, sn);
    return ref_sync_status();
}

// The reference's multi-slot append, k_qkv_prep_fast_ms (bruce.cu:1835): one row per slot, per-row position,
// partition and "writes KV" flag; kvk/kvv are layer bases.
int ref_kv_append_ms(float* q, const float* k, const float* v, const float* sqk, uint8_t* kvk, uint8_t* kvv,
                     const int* d_pos, const int* d_slot, const int* d_act, int rows, int is_swa, int theta_sel,
                     int nctx, const float* cs, const float* sn) {
    ref_set_nctx(nctx);
    k_qkv_prep_fast_ms<<<rows, 256>>>(q, k, v, sqk, kvk, kvv, d_pos, d_slot, d_act, is_swa, theta_sel, cs, sn);
    return ref_sync_status();
}

// The same single-sequence kernel as ref_kv_append with the table selector exposed.
int ref_kv_append_theta(float* q, const float* k, const float* v, const float* sqk, uint8_t* kvk, uint8_t* kvv,
                        const int* d_pos, int rows, int is_swa, int theta_sel, int nctx, const float* cs,
                        const float* sn) {
    ref_set_nctx(nctx);
    k_qkv_prep_fast<<<rows, 256>>>(q, k, v, sqk, kvk, kvv, d_pos, is_swa, theta_sel, cs, sn);
    return ref_sync_status();
}

// The reference's RoPE table kernels: rows of one sequence (bruce.cu:1641) / one row per slot (:1821).
int ref_rope_tables(float* cs, float* sn, const int* d_pos, int rows, int per_row_pos) {
    if (per_row_pos) k_rope_tables_rows_ms<<<rows, 128>>>(cs, sn, d_pos, rows);
    else             k_rope_tables_rows<<<rows, 128>>>(cs, sn, d_pos, rows);
    return ref_sync_status();
}

// The reference's exact fp32 attention: k_attn_rows (bruce.cu:1921) + k_attn_combine_rows (:1999).
// part must hold rows * N_KV * ns * 4 * (HD + 2) floats.
int ref_attn_exact(float* out, const float* q, const uint8_t* kvk, const uint8_t* kvv, const int* d_pos,
                   float* part, int rows, int ns, int is_swa, int nctx) {
    ref_set_nctx(nctx);
    k_attn_rows<<<dim3(N_KV, ns, rows), 128>>>(out, q, kvk, kvv, d_pos, is_swa, part);
    if (ns > 1) k_attn_combine_rows<<<dim3(N_HEAD, rows), 32>>>(out, part, ns);
    return ref_sync_status();
}

// The reference's gate-norm step after attention, k_gate_norm_vec4 (bruce.cu:1526): sigmoid gate, L2 norm over the
// token's N_HEAD*HD values, q8 activation copy.  dst may be null.
int ref_gate_norm(float* dst, const float* aout, const float* gate, const float* sg, int8_t* xq, float* xd, int* xs,
                  int rows) {
    k_gate_norm_vec4<<<rows, 256>>>(dst, aout, gate, sg, N_HEAD * HD, xq, xd, xs);
    return ref_sync_status();
}

// The reference's shipping dispatch, launch_attn_m (bruce.cu:3942) + k_attn_combine_rows: tensor-core
// kernels with fp16 accumulation.  Returns the elapsed milliseconds of `reps` back-to-back calls in *ms.
int ref_attn_shipping(float* out, const float* q, const uint8_t* kvk, const uint8_t* kvv, const int* d_pos,
                      float* part, int rows, int ns, int is_swa, int nctx, int reps, float* ms) {
    ref_set_nctx(nctx);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    launch_attn_m(out, q, kvk, kvv, d_pos, part, rows, ns, is_swa, 0);          // sets lazy attributes
    if (ns > 1) k_attn_combine_rows<<<dim3(N_HEAD, rows), 32>>>(out, part, ns);
    cudaDeviceSynchronize();
    cudaEventRecord(e0);
    for (int i = 0; i < reps; ++i) {
        launch_attn_m(out, q, kvk, kvv, d_pos, part, rows, ns, is_swa, 0);
        if (ns > 1) k_attn_combine_rows<<<dim3(N_HEAD, rows), 32>>>(out, part, ns);
    }
    cudaEventRecord(e1);
    const int rc = ref_sync_status();
    if (ms) cudaEventElapsedTime(ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    return rc;
}

}  // extern "C"
