// The step right after attention: sigmoid gate, L2 norm over the token's whole attention vector, and the q8
// activation copy the following projection consumes.
//
// Behaviour replaced: k_gate_norm_vec4 (engine/src/bruce.cu:1526-1568, calls :7746-7755, :7975) and, fused with
// the merge of split records, k_combine_gate_norm_rows_opt (:1577-1639, call :7743).  Per token row m, with
// n = n_head * head_dim elements:
//     t_i = a_i / (1 + __expf(-(gate_i * sgate_i)))                      (:1543-1546)
//     k   = l2_scale(sum t_i^2, n)                                       (:305-307, :1554-1555)
//     v_i = t_i * k                                                      -> dst (fp32, optional)
//     per 32 elements: d = amax * (1/127), id = d > 0 ? 1/d : 0, q = clamp(rint(v * id), -127, 127),
//                      xq = q (int8), xd = d, xsum = sum q               (q8_group_vec4, :1405-1428)
// (the activation quantiser: NOT the KV formula -- it multiplies by 1/127 and clamps.)
//
// k_gate_norm keeps the reference's thread-to-element map (thread i owns the float4 i + 256 b, b = 0..3) and its
// reduction trees, so that sums are formed in the reference's order and the outputs are bit-identical to
// k_gate_norm_vec4's for the same inputs.  k_merge_gate_norm computes a_i from this library's split records in
// registers (the attention output of a split prompt chunk then never goes to memory, the point of the reference's
// fused kernel) and continues with the same code.
#pragma once
#include "common.cuh"

namespace battn {

struct GateNormParams {
    float* dst;              // [rows][n] fp32 normalised, gated output, or null
    const void* aout;        // [rows][n] attention output (fp32 or fp16), k_gate_norm only
    int aout_f16;
    const float* gate;       // [rows][n]
    const float* sgate;      // [n]
    int8_t* xq;              // [rows][n]
    float* xd;               // [rows][n / 32]
    int* xsum;               // [rows][n / 32]
    int n;                   // n_head * head_dim, a multiple of 1024, at most 4096
    // k_merge_gate_norm only: split records [split][row][head][HD + 2] = (unnormalised o, m in log2 units, l)
    const float* recs;
    int nsplit, rows, Hq;
};

constexpr float GN_EPS_L2 = 1e-6f;                      // EPS_L2, bruce.cu:73

__device__ __forceinline__ float gn_l2_scale(float ss, int n) {                       // bruce.cu:305-307
    return (1.0f / sqrtf(ss / (float)n + GN_EPS_L2 / (float)n)) * (1.0f / sqrtf((float)n));
}
__device__ __forceinline__ float gn_warp_sum(float v) {                               // bruce.cu:263-267
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}
// block_red_n<8> (bruce.cu:1252-1265): warp sums, then warp 0 sums the eight partials
__device__ __forceinline__ float gn_block_sum8(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    v = gn_warp_sum(v);
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = (lane < 8) ? red[lane] : 0.f;
        t = gn_warp_sum(t);
        if (lane == 0) red[0] = t;
    }
    __syncthreads();
    return red[0];
}
// q8_group_vec4 (bruce.cu:1405-1428): eight lanes own one group of 32 values
__device__ __forceinline__ void gn_q8_group(int8_t* __restrict__ xq, float* __restrict__ xd, int* __restrict__ xsum, int g,
                                            float4 v, int sub8) {
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const float d = amax * (1.f / 127.f);
    const float id = d > 0.f ? 1.f / d : 0.f;
    const int q0 = max(-127, min(127, __float2int_rn(v.x * id)));
    const int q1 = max(-127, min(127, __float2int_rn(v.y * id)));
    const int q2 = max(-127, min(127, __float2int_rn(v.z * id)));
    const int q3 = max(-127, min(127, __float2int_rn(v.w * id)));
    const uint32_t pack = ((uint32_t)(uint8_t)q0) | (((uint32_t)(uint8_t)q1) << 8) | (((uint32_t)(uint8_t)q2) << 16) |
                          (((uint32_t)(uint8_t)q3) << 24);
    *reinterpret_cast<uint32_t*>(xq + g * 32 + sub8 * 4) = pack;
    int s = (q0 + q1) + (q2 + q3);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if (sub8 == 0) { xd[g] = d; xsum[g] = s; }
}

// gate, sum of squares, norm, q8 on the four float4 a thread owns (a[b] = attention values of float4 tid + 256 b)
__device__ __forceinline__ void gn_finish(const GateNormParams& P, int m, const float4 (&a)[4], int nb, float* red) {
    const int tid = threadIdx.x, qwarp = tid >> 3, sub8 = tid & 7;
    const int n = P.n;
    const float4* gr4 = reinterpret_cast<const float4*>(P.gate + (size_t)m * n);
    const float4* sg4 = reinterpret_cast<const float4*>(P.sgate);
    float4 r[4];
    float ss = 0.f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        if (b >= nb) break;
        const int idx4 = (qwarp + b * 32) * 8 + sub8;
        const float4 av = a[b], gv = gr4[idx4], sv = sg4[idx4];
        float4 t;
        float gx = gv.x * sv.x; t.x = av.x / (1.f + __expf(-gx));
        float gy = gv.y * sv.y; t.y = av.y / (1.f + __expf(-gy));
        float gz = gv.z * sv.z; t.z = av.z / (1.f + __expf(-gz));
        float gw = gv.w * sv.w; t.w = av.w / (1.f + __expf(-gw));
        r[b] = t;
        ss += (t.x * t.x + t.y * t.y) + (t.z * t.z + t.w * t.w);
    }
    ss = gn_block_sum8(ss, red);
    const float k = gn_l2_scale(ss, n);
    float* dr = P.dst ? P.dst + (size_t)m * n : nullptr;
    int8_t* xqr = P.xq + (size_t)m * n;
    float* xdr = P.xd + (size_t)m * (n >> 5);
    int* xsr = P.xsum + (size_t)m * (n >> 5);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        if (b >= nb) break;
        const int g_ = qwarp + b * 32;
        const float4 v = make_float4(r[b].x * k, r[b].y * k, r[b].z * k, r[b].w * k);
        if (dr) reinterpret_cast<float4*>(dr)[g_ * 8 + sub8] = v;
        gn_q8_group(xqr, xdr, xsr, g_, v, sub8);
    }
}

__global__ void __launch_bounds__(256, 2) k_gate_norm(const GateNormParams P) {
    __shared__ float red[8];
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x, tid = threadIdx.x;
    const int nb = P.n >> 10;                               // float4 per thread: n / (4 * 256)
    float4 a[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        a[b] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b >= nb) continue;
        const size_t idx4 = (size_t)m * (P.n >> 2) + tid + 256 * b;
        if (P.aout_f16) {
            const uint2 w = reinterpret_cast<const uint2*>(P.aout)[idx4];
            const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
            const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
            a[b] = make_float4(lo.x, lo.y, hi.x, hi.y);
        } else {
            a[b] = reinterpret_cast<const float4*>(P.aout)[idx4];
        }
    }
    gn_finish(P, m, a, nb, red);
}

// One block per token row.  First the merge weights of every head (m in log2 units; empty splits weigh zero), one
// warp per head in turn; then every thread merges its own four float4 of the attention vector from the split
// records and hands them to the gate / norm / q8 code above.
template <int HD>
__global__ void __launch_bounds__(256, 2) k_merge_gate_norm(const GateNormParams P) {
    __shared__ float red[8];
    __shared__ float s_w[32][8];                            // [head][split] weight 2^(m_s - M) / L
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const size_t rstride = (size_t)P.rows * P.Hq * (HD + 2);                        // floats between splits
    const float* rowrec = P.recs + (size_t)m * P.Hq * (HD + 2);
    for (int head = w; head < P.Hq; head += 8) {
        float mval = NEG_BIG, lval = 0.f;
        if (lane < P.nsplit) {
            const float2 ml = *reinterpret_cast<const float2*>(rowrec + (size_t)lane * rstride + (size_t)head * (HD + 2) + HD);
            mval = ml.x; lval = ml.y;
        }
        float M = mval;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));      // nsplit <= 8
        const float wg = lane < P.nsplit ? fast_exp2(mval - M) : 0.f;
        float L = lval * wg;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
        if (lane < 8) s_w[head][lane] = L > 0.f ? wg / L : 0.f;
    }
    __syncthreads();
    const int nb = P.n >> 10;
    float4 a[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        a[b] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b >= nb) continue;
        const int e = 4 * (tid + 256 * b);                  // first element of this float4
        const int head = e / HD, dim = e - head * HD;
        const float* base = rowrec + (size_t)head * (HD + 2) + dim;
        for (int s = 0; s < P.nsplit; ++s) {
            const float2 lo = *reinterpret_cast<const float2*>(base + (size_t)s * rstride);     // records are 8-byte aligned
            const float2 hi = *reinterpret_cast<const float2*>(base + (size_t)s * rstride + 2);
            const float ws = s_w[head][s];
            a[b].x = fmaf(lo.x, ws, a[b].x); a[b].y = fmaf(lo.y, ws, a[b].y);
            a[b].z = fmaf(hi.x, ws, a[b].z); a[b].w = fmaf(hi.y, ws, a[b].w);
        }
    }
    gn_finish(P, m, a, nb, red);
}

}  // namespace battn
