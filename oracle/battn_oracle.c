/*
 * battn_oracle.c -- CPU restatement of the reference engine's attention arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA library is compared against
 * (and the timed CPU baseline of the benchmark).  It is never linked into, loaded by, or called
 * from the product library; the product has no CPU path.
 *
 * PARITY STATUS: the reference ships no golden vectors, known-answer tests or fixtures for this path, and
 * its kernels cannot execute without a GPU, so the pins were made here: (a) golden vectors produced by the
 * reference's own kernels (k_rope_tables_rows, k_qkv_prep_fast, k_qkv_prep_fast_ms) on a B200 through the
 * harness in ref_harness.cu, committed as tests/golden/qkv_prep_ref.npz with the script that made them --
 * oracle_qkv_prep and the quantiser reproduce them bit for bit; (b) hand-derived known-answer cases, an
 * independent numpy restatement and fixtures generated from this file for the attention functions, whose
 * agreement with the reference's exact kernels (2e-5) is checked on a GPU box by
 * tests/test_gpu_reference_kernels.py.
 *
 * Each function cites the reference lines (engine/src/bruce.cu) it follows.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct oracle_geom {
    int   n_head, n_kv, head_dim, window, slot_ctx, n_slots;
    float softmax_scale; /* 0 => 1/sqrt(head_dim) */
} oracle_geom;

/* ---- fp16 <-> fp32, IEEE round-to-nearest-even (what __float2half / __half2float do) ---- */
uint16_t oracle_f32_to_f16(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) return (uint16_t)(sign | (absx > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);      /* rounds to inf (>= 65520) */
    if (absx < 0x33000001u) return (uint16_t)sign;                    /* <= 2^-25 rounds to zero  */
    int e = (int)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7fffffu) | 0x800000u;                    /* 24-bit significand       */
    int shift;                                                        /* bits dropped             */
    uint32_t hexp;
    if (e < -14) { shift = 13 + (-14 - e); hexp = 0; }                /* subnormal half           */
    else         { shift = 13;             hexp = (uint32_t)(e + 15); }
    uint32_t kept = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u))) kept++;
    uint32_t h;
    if (hexp == 0) h = kept;                     /* a carry out of the subnormal lands in exp=1 */
    else           h = ((hexp - 1) << 10) + kept; /* kept carries the implicit bit              */
    return (uint16_t)(sign | h);
}

float oracle_f16_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu, x;
    if (e == 0) {
        if (m == 0) x = sign;
        else { int s = 0; while (!(m & 0x400u)) { m <<= 1; s++; }
               x = sign | ((uint32_t)(113 - s) << 23) | ((m & 0x3ffu) << 13); }
    } else if (e == 31) x = sign | 0x7f800000u | (m << 13);
    else x = sign | ((e + 112u) << 23) | (m << 13);
    float f; memcpy(&f, &x, 4); return f;
}

/* ---- layout (bruce.cu:56-65, 690-693, 1888-1892, 5473-5503) ---- */
static int rec_bytes(const oracle_geom* g) { return g->head_dim + 2 * (g->head_dim / 32); }
static int pstride_of(const oracle_geom* g, int is_swa) { return is_swa ? 2 * g->window : g->slot_ctx; }

size_t oracle_kv_layer_bytes(const oracle_geom* g, int is_swa) {
    return (size_t)g->n_slots * pstride_of(g, is_swa) * g->n_kv * rec_bytes(g);
}

static size_t rec_offset(const oracle_geom* g, int is_swa, int slot, int kvh, int p) {
    const int ps = pstride_of(g, is_swa);
    const int pp = is_swa ? (p & (2 * g->window - 1)) : p;      /* ring slot, bruce.cu:691, 740 */
    return (((size_t)slot * g->n_kv + kvh) * ps + pp) * (size_t)rec_bytes(g);
}

/* ---- the KV quantiser, one 32-value block (bruce.cu:698-710, 1896-1915) ----
 * d = amax / 127.f (IEEE divide); id = d ? 1.f/d : 0; q = lrintf(x*id) (half-even, no clamp);
 * stored scale = __float2half(d). */
void oracle_quant_block32(const float* x, uint16_t* scale, int8_t* q) {
    float amax = 0.f;
    for (int i = 0; i < 32; ++i) { const float a = fabsf(x[i]); if (a > amax) amax = a; }
    const volatile float d = amax / 127.f;
    const volatile float id = d != 0.f ? 1.f / d : 0.f;
    *scale = oracle_f32_to_f16(d);
    for (int i = 0; i < 32; ++i) {
        const volatile float t = x[i] * id;          /* a lone fp32 multiply, never contracted */
        q[i] = (int8_t)lrintf(t);
    }
}

void oracle_quant_record(const oracle_geom* g, const float* x, uint8_t* rec) {
    const int nblk = g->head_dim / 32;
    for (int b = 0; b < nblk; ++b) {
        uint16_t s;
        oracle_quant_block32(x + b * 32, &s, (int8_t*)(rec + 2 * nblk + b * 32));
        memcpy(rec + 2 * b, &s, 2);                  /* scales grouped first, bruce.cu:57-61, 708 */
    }
}

/* dequantise one record into HD floats: half2float(scale) * (float)int8, exact in fp32
 * (bruce.cu:742-749) */
static void dequant_record(const oracle_geom* g, const uint8_t* rec, float* out) {
    const int nblk = g->head_dim / 32;
    for (int b = 0; b < nblk; ++b) {
        uint16_t s; memcpy(&s, rec + 2 * b, 2);
        const float d = oracle_f16_to_f32(s);
        const int8_t* q = (const int8_t*)(rec + 2 * nblk + b * 32);
        for (int i = 0; i < 32; ++i) out[b * 32 + i] = d * (float)q[i];
    }
}

/* ---- KV append (bruce.cu:690-710 single row, :1789-1812 rows of one sequence,
 *      :1868-1892 multi-slot with per-row pos / kslot / act) ----
 * kslot == NULL: one sequence, kvk/kvv = slot base, row r at pos[0] + r.
 * kslot != NULL: kvk/kvv = layer base, sequence i at partition kslot[i], rows pos[i] + r. */
int oracle_kv_append(const oracle_geom* g, const float* k, const float* v, uint8_t* kvk,
                     uint8_t* kvv, const int* pos, const int* kslot, const int* act,
                     int n_seq, int rows, int is_swa) {
    const int HD = g->head_dim;
    if (!kslot && n_seq != 1) return 1;
    for (int i = 0; i < n_seq; ++i) {
        if (act && !act[i]) continue;                              /* idle rows never write KV */
        const int slot = kslot ? kslot[i] : 0;
        for (int r = 0; r < rows; ++r) {
            const int p = pos[i] + r;
            if (p < 0 || (!is_swa && p >= g->slot_ctx)) return 2;
            for (int h = 0; h < g->n_kv; ++h) {
                const size_t src = (((size_t)i * rows + r) * g->n_kv + h) * HD;
                const size_t off = rec_offset(g, is_swa, slot, h, p);
                oracle_quant_record(g, k + src, kvk + off);
                oracle_quant_record(g, v + src, kvv + off);
            }
        }
    }
    return 0;
}

/* ---- QKV prologue + append (k_qkv_prep_fast, bruce.cu:1732-1812; multi-slot k_qkv_prep_fast_ms,
 *      :1835-1918): per head an L2 scale (l2_scale, :305-307), NeoX rotate-half RoPE with per-row
 *      cos/sin tables, the per-head sqk scale on q; k gets scale + RoPE and is quantised, v is quantised raw.
 * The fp32 operation order below is the one nvcc generates for the reference source (fused
 * multiply-adds included); it reproduces the reference kernel's q output and K/V records bit for bit
 * (tests/golden/qkv_prep_ref.npz holds outputs of the reference kernel itself).
 *   lane l of the warp that owns a head holds VEC = HD/64 consecutive values of each half:
 *     e[0..VEC) = x[VEC*l ..], f[0..VEC) = x[HD/2 + VEC*l ..]
 *     partial(e) = fma(e[VEC-1], e[VEC-1], ... fma(e[2], e[2], fma(e[0], e[0], rn(e[1]*e[1]))))
 *     ss_lane = partial(e) + partial(f);  ss = shfl_down tree over 32 lanes (16, 8, 4, 2, 1), lane 0
 *   norm = (1 / sqrt(ss/HD + 1e-6f/HD)) * (1 / sqrt(HD))                         (each step rounded)
 *   lo = fma(x0, c, -rn(x1*s)),  hi = fma(x0, s, rn(x1*c));  then * norm, then (q only) * sqk
 * Tables: row m = i*rows + r uses cs/sn + m*HD + (theta_sel == 2 ? HD/2 : 0), HD/2 entries. */
static float prep_sumsq(const float* x, int HD) {
    const int VEC = HD / 64;
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        float part[2];
        for (int half = 0; half < 2; ++half) {
            const float* e = x + half * (HD / 2) + VEC * l;
            float t = fmaf(e[0], e[0], e[1] * e[1]);
            for (int j = 2; j < VEC; ++j) t = fmaf(e[j], e[j], t);
            part[half] = t;
        }
        lane[l] = part[0] + part[1];
    }
    for (int o = 16; o > 0; o >>= 1)
        for (int l = 0; l + o < 32; ++l) lane[l] = lane[l] + lane[l + o];   /* lanes >= 32-o keep their value */
    return lane[0];
}

static float prep_l2_scale(float ss, int n) {
    const float a = ss / (float)n + 1e-6f / (float)n;
    return (1.0f / sqrtf(a)) * (1.0f / sqrtf((float)n));
}

static void prep_rotate(const float* x, const float* c, const float* s, float norm, const float* extra,
                        float* out, int HD) {
    const int H2 = HD / 2;
    for (int i = 0; i < H2; ++i) {
        const float x0 = x[i], x1 = x[i + H2];
        float lo = fmaf(x0, c[i], -(x1 * s[i]));
        float hi = fmaf(x0, s[i], x1 * c[i]);
        lo = lo * norm; hi = hi * norm;
        if (extra) { lo = lo * extra[i]; hi = hi * extra[i + H2]; }
        out[i] = lo; out[i + H2] = hi;
    }
}

int oracle_qkv_prep(const oracle_geom* g, float* q, const float* k, const float* v, const float* sqk,
                    const float* cs, const float* sn, int theta_sel, uint8_t* kvk, uint8_t* kvv,
                    const int* pos, const int* kslot, const int* act, int n_seq, int rows, int is_swa) {
    const int HD = g->head_dim;
    if (!kslot && n_seq != 1) return 1;
    float* tmp = (float*)malloc(sizeof(float) * (size_t)HD);
    if (!tmp) return 3;
    for (int i = 0; i < n_seq; ++i) {
        const int slot = kslot ? kslot[i] : 0;
        for (int r = 0; r < rows; ++r) {
            const size_t m = (size_t)i * rows + r;
            const float* c = cs + m * HD + (theta_sel == 2 ? HD / 2 : 0);
            const float* s = sn + m * HD + (theta_sel == 2 ? HD / 2 : 0);
            for (int h = 0; h < g->n_head; ++h) {
                float* qh = q + (m * g->n_head + h) * HD;
                const float norm = prep_l2_scale(prep_sumsq(qh, HD), HD);
                prep_rotate(qh, c, s, norm, sqk + (size_t)h * HD, tmp, HD);
                memcpy(qh, tmp, sizeof(float) * (size_t)HD);
            }
            if (act && !act[i]) continue;                      /* idle rows normalise q but never write KV (:1869) */
            const int p = pos[i] + r;
            if (p < 0 || (!is_swa && p >= g->slot_ctx)) { free(tmp); return 2; }
            for (int h = 0; h < g->n_kv; ++h) {
                const size_t src = (m * g->n_kv + h) * HD;
                const size_t off = rec_offset(g, is_swa, slot, h, p);
                const float norm = prep_l2_scale(prep_sumsq(k + src, HD), HD);
                prep_rotate(k + src, c, s, norm, NULL, tmp, HD);
                oracle_quant_record(g, tmp, kvk + off);
                oracle_quant_record(g, v + src, kvv + off);
            }
        }
    }
    free(tmp);
    return 0;
}

/* ---- attention ----
 * One function serves decode (rows = 1), speculative verify (rows 2..8) and prompt chunks
 * (rows up to 512), single-sequence or multi-slot.  Row r of sequence i sits at position
 * p = pos[i] + r and sees keys [lo, p], lo = is_swa ? max(0, p + 1 - W) : 0
 * (bruce.cu:724-727 decode; :2056, :2119-2123 in-chunk causal mask; :3686-3689, :3012-3029 the
 * windowed rows).  Scores are (q . dequant(k)) * scale (:742-756); softmax; out = sum p v / sum p.
 * Accumulation is in double so that the oracle itself adds no rounding noise; the per-key
 * online-softmax order of k_attn (:737-776) is mirrored by oracle_attend_f32 below.
 *
 * key_lo / key_hi additionally clip the key range to [key_lo, key_hi) (used to restate a
 * sequence split; pass 0 and INT32_MAX for the whole range).
 *
 * out  != NULL : normalised output  [n_seq][rows][n_head][HD] fp32
 * recs != NULL : split records      [n_seq][rows][n_head][HD+2] (o, m, l)   (bruce.cu:781-783)
 */
int oracle_attend(const oracle_geom* g, float* out, float* recs, const float* q,
                  const uint8_t* kvk, const uint8_t* kvv, const int* pos, const int* kslot,
                  const int* act, int n_seq, int rows, int is_swa, int key_lo, int key_hi,
                  int nthreads) {
    const int HD = g->head_dim, G = g->n_head / g->n_kv;
    const double scale = g->softmax_scale != 0.f ? (double)g->softmax_scale : 1.0 / sqrt((double)HD);
    if (!kslot && n_seq != 1) return 1;
    const int njobs = n_seq * g->n_kv;
#ifdef _OPENMP
    if (nthreads > 0) omp_set_num_threads(nthreads);
#else
    (void)nthreads;
#endif
    int err = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int job = 0; job < njobs; ++job) {
        const int i = job / g->n_kv, kvh = job % g->n_kv;
        if (act && !act[i]) continue;                    /* idle rows produce no output (:3402) */
        const int slot = kslot ? kslot[i] : 0;
        const int p0 = pos[i];
        if (p0 < 0 || (!is_swa && p0 + rows > g->slot_ctx)) { err = 2; continue; }
        const int RG = rows * G;
        double* m = (double*)malloc(sizeof(double) * RG);
        double* l = (double*)malloc(sizeof(double) * RG);
        double* o = (double*)calloc((size_t)RG * HD, sizeof(double));
        float* kf = (float*)malloc(sizeof(float) * HD);
        float* vf = (float*)malloc(sizeof(float) * HD);
        for (int a = 0; a < RG; ++a) { m[a] = -1e30; l[a] = 0.0; }
        int lo_all = is_swa ? p0 + 1 - g->window : 0;
        if (lo_all < 0) lo_all = 0;
        if (lo_all < key_lo) lo_all = key_lo;
        int hi_all = p0 + rows;
        if (hi_all > key_hi) hi_all = key_hi;
        for (int key = lo_all; key < hi_all; ++key) {
            const size_t off = rec_offset(g, is_swa, slot, kvh, key);
            dequant_record(g, kvk + off, kf);
            dequant_record(g, kvv + off, vf);
            for (int r = 0; r < rows; ++r) {
                const int p = p0 + r;
                int lo = is_swa ? p + 1 - g->window : 0;
                if (lo < 0) lo = 0;
                if (key > p || key < lo) continue;
                for (int h = 0; h < G; ++h) {
                    const int a = r * G + h;
                    const float* qv = q + (((size_t)i * rows + r) * g->n_head + kvh * G + h) * HD;
                    double dot = 0.0;
                    for (int d = 0; d < HD; ++d) dot += (double)qv[d] * (double)kf[d];
                    dot *= scale;
                    double* oa = o + (size_t)a * HD;
                    if (dot > m[a]) {
                        const double c = exp(m[a] - dot);
                        l[a] = l[a] * c + 1.0;
                        for (int d = 0; d < HD; ++d) oa[d] = oa[d] * c + (double)vf[d];
                        m[a] = dot;
                    } else {
                        const double pw = exp(dot - m[a]);
                        l[a] += pw;
                        for (int d = 0; d < HD; ++d) oa[d] += pw * (double)vf[d];
                    }
                }
            }
        }
        for (int r = 0; r < rows; ++r)
            for (int h = 0; h < G; ++h) {
                const int a = r * G + h;
                const size_t row = ((size_t)i * rows + r) * g->n_head + kvh * G + h;
                if (out) {
                    const double il = l[a] > 0.0 ? 1.0 / l[a] : 0.0;      /* bruce.cu:778 */
                    for (int d = 0; d < HD; ++d) out[row * HD + d] = (float)(o[(size_t)a * HD + d] * il);
                }
                if (recs) {
                    float* rc = recs + row * (HD + 2);
                    for (int d = 0; d < HD; ++d) rc[d] = (float)o[(size_t)a * HD + d];
                    rc[HD] = (float)m[a]; rc[HD + 1] = (float)l[a];
                }
            }
        free(m); free(l); free(o); free(kf); free(vf);
    }
    return err;
}

/* fp32 mirror of the reference's exact path: per-key online softmax with `nsplit` key splits and
 * the serial merge, float arithmetic throughout (k_attn bruce.cu:713-785, k_attn_rows :1921-1997,
 * k_attn_combine :992-1007; split rule :724-729; empty split = (0, -1e30, 0)).  Differs from the
 * GPU only in the association of the 32-lane dot-product reduction. */
int oracle_attend_f32(const oracle_geom* g, float* out, const float* q, const uint8_t* kvk,
                      const uint8_t* kvv, const int* pos, const int* kslot, const int* act,
                      int n_seq, int rows, int is_swa, int nsplit) {
    const int HD = g->head_dim, G = g->n_head / g->n_kv;
    const float scale = g->softmax_scale != 0.f ? g->softmax_scale : 1.f / sqrtf((float)HD);
    if (!kslot && n_seq != 1) return 1;
    if (nsplit < 1) nsplit = 1;
    float* kf = (float*)malloc(sizeof(float) * HD);
    float* vf = (float*)malloc(sizeof(float) * HD);
    float* part = (float*)malloc(sizeof(float) * (size_t)nsplit * (HD + 2));
    for (int i = 0; i < n_seq; ++i) {
        if (act && !act[i]) continue;
        const int slot = kslot ? kslot[i] : 0;
        for (int r = 0; r < rows; ++r) {
            const int p = pos[i] + r, kend = p + 1;
            int kstart = is_swa ? kend - g->window : 0;
            if (kstart < 0) kstart = 0;
            const int nkeys = kend - kstart, per = (nkeys + nsplit - 1) / nsplit;
            for (int hq = 0; hq < g->n_head; ++hq) {
                const int kvh = hq / G;
                const float* qv = q + (((size_t)i * rows + r) * g->n_head + hq) * HD;
                for (int s = 0; s < nsplit; ++s) {
                    const int a0 = kstart + s * per;
                    int a1 = a0 + per; if (a1 > kend) a1 = kend;
                    float m = -1e30f, l = 0.f;
                    float* o = part + (size_t)s * (HD + 2);
                    for (int d = 0; d < HD; ++d) o[d] = 0.f;
                    for (int key = a0; key < a1; ++key) {
                        const size_t off = rec_offset(g, is_swa, slot, kvh, key);
                        dequant_record(g, kvk + off, kf);
                        dequant_record(g, kvv + off, vf);
                        float dot = 0.f;
                        for (int d = 0; d < HD; ++d) dot = fmaf(qv[d], kf[d], dot);
                        dot *= scale;
                        const float mnew = fmaxf(m, dot);
                        const float pw = expf(dot - mnew), corr = expf(m - mnew);
                        l = l * corr + pw; m = mnew;
                        for (int d = 0; d < HD; ++d) o[d] = fmaf(o[d], corr, pw * vf[d]);
                    }
                    o[HD] = m; o[HD + 1] = l;
                }
                float M = -1e30f;
                for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part[(size_t)s * (HD + 2) + HD]);
                float L = 0.f;
                float* orow = out + (((size_t)i * rows + r) * g->n_head + hq) * HD;
                for (int d = 0; d < HD; ++d) orow[d] = 0.f;
                for (int s = 0; s < nsplit; ++s) {
                    const float* b = part + (size_t)s * (HD + 2);
                    const float w = expf(b[HD] - M);
                    L += b[HD + 1] * w;
                    for (int d = 0; d < HD; ++d) orow[d] = fmaf(b[d], w, orow[d]);
                }
                const float il = L > 0.f ? 1.f / L : 0.f;
                for (int d = 0; d < HD; ++d) orow[d] *= il;
            }
        }
    }
    free(kf); free(vf); free(part);
    return 0;
}

/* Log-sum-exp merge of split records (k_attn_combine, bruce.cu:992-1007):
 * parts [n_parts][n_items][HD+2], out [n_items][HD].  Accumulates in double. */
void oracle_merge(float* out, const float* parts, int n_parts, int n_items, int HD) {
    for (int it = 0; it < n_items; ++it) {
        double M = -1e30;
        for (int s = 0; s < n_parts; ++s) {
            const double m = parts[((size_t)s * n_items + it) * (HD + 2) + HD];
            if (m > M) M = m;
        }
        double L = 0.0;
        for (int d = 0; d < HD; ++d) out[(size_t)it * HD + d] = 0.f;
        double* acc = (double*)calloc(HD, sizeof(double));
        for (int s = 0; s < n_parts; ++s) {
            const float* b = parts + ((size_t)s * n_items + it) * (HD + 2);
            const double w = exp((double)b[HD] - M);
            L += (double)b[HD + 1] * w;
            for (int d = 0; d < HD; ++d) acc[d] += (double)b[d] * w;
        }
        const double il = L > 0.0 ? 1.0 / L : 0.0;
        for (int d = 0; d < HD; ++d) out[(size_t)it * HD + d] = (float)(acc[d] * il);
        free(acc);
    }
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---- the step after attention: sigmoid gate, L2 norm, q8 activation copy ----
 * k_gate_norm_vec4 (bruce.cu:1526-1568) with its helpers l2_scale (:305-307), block_red_n<8> (:1252-1265),
 * warp_sum (:263-267) and q8_group_vec4 (:1405-1428).  Per token row m, n = n_head * head_dim values:
 *     t = a / (1 + exp(-(gate * sgate)));  k = l2_scale(sum t^2, n);  v = t * k -> dst
 *     per 32 values: d = amax * (1/127), id = d > 0 ? 1/d : 0, q = clamp(rint(v * id), -127, 127)
 * The partial sums are formed in the kernel's order: thread i (of 256) owns the float4 i + 256 b, adds
 * (x^2 + y^2) + (z^2 + w^2) per float4 with the products contracted the way nvcc contracts them, then the
 * shuffle-down trees.  One thing cannot be restated on a CPU: the kernel's exponential is the GPU's approximate
 * ex2 unit (__expf), this one is expf; values agree to a few ulp, so quantised bytes may differ by one step where a
 * value sits on a rounding boundary (the tests bound both).
 * aout fp32 [rows][n]; dst may be NULL. */
static float gn_tree_down(float* v, int count) {
    /* v += shfl_down(v, o) for o = 16 .. 1 over `count` lanes (lanes beyond read their own value: unused results) */
    float t[32];
    for (int i = 0; i < 32; ++i) t[i] = i < count ? v[i] : 0.f;
    for (int o = 16; o > 0; o >>= 1) {
        float nx[32];
        for (int i = 0; i < 32; ++i) nx[i] = t[i] + (i + o < 32 ? t[i + o] : t[i]);
        for (int i = 0; i < 32; ++i) t[i] = nx[i];
    }
    return t[0];
}

int oracle_gate_norm(int n, int rows, const float* aout, const float* gate, const float* sgate, float* dst,
                     int8_t* xq, float* xd, int* xsum) {
    if (n % 1024 || n > 4096) return 1;
    const int nb = n / 1024;
    float* t = (float*)malloc(sizeof(float) * (size_t)n);
    for (int m = 0; m < rows; ++m) {
        const float* a = aout + (size_t)m * n;
        const float* g = gate + (size_t)m * n;
        for (int i = 0; i < n; ++i) {
            const float gx = g[i] * sgate[i];
            t[i] = a[i] / (1.f + expf(-gx));
        }
        float wsum[8];
        for (int w = 0; w < 8; ++w) {
            float lane_ss[32];
            for (int l = 0; l < 32; ++l) {
                const int tid = w * 32 + l;
                float ss = 0.f;
                for (int b = 0; b < nb; ++b) {
                    const float* e = t + 4 * (tid + 256 * b);
                    const float p = fmaf(e[0], e[0], e[1] * e[1]);
                    const float q = fmaf(e[2], e[2], e[3] * e[3]);
                    ss += p + q;
                }
                lane_ss[l] = ss;
            }
            wsum[w] = gn_tree_down(lane_ss, 32);
        }
        const float ss = gn_tree_down(wsum, 8);
        const float k = (1.0f / sqrtf(ss / (float)n + 1e-6f / (float)n)) * (1.0f / sqrtf((float)n));
        for (int grp = 0; grp < n / 32; ++grp) {
            float v[32], amax = 0.f;
            for (int i = 0; i < 32; ++i) {
                v[i] = t[grp * 32 + i] * k;
                if (dst) dst[(size_t)m * n + grp * 32 + i] = v[i];
                amax = fmaxf(amax, fabsf(v[i]));
            }
            const float d = amax * (1.f / 127.f);
            const float id = d > 0.f ? 1.f / d : 0.f;
            int s = 0;
            for (int i = 0; i < 32; ++i) {
                int q = (int)nearbyintf(v[i] * id);
                q = q > 127 ? 127 : (q < -127 ? -127 : q);
                xq[(size_t)m * n + grp * 32 + i] = (int8_t)q;
                s += q;
            }
            xd[(size_t)m * (n / 32) + grp] = d;
            xsum[(size_t)m * (n / 32) + grp] = s;
        }
    }
    free(t);
    return 0;
}
