// Query pre-rotation for the whole-step form of the decode attention, sm_100a.
//
// The reference rotates the query inside every attention CTA, q_rot[d] = sum_k R[d][k] * q[k]
// (engine/kernels.cu:1676-1680).  Here all query heads of all layers of a step are rotated by ONE small launch on the
// tensor cores (mma.sync m16n8k16, fp16 in, fp32 accumulate) and stored as fp16, already multiplied by
// log2(e) / sqrt(128), in the order the attention kernel's score product consumes them; the attention kernel then
// fetches a sequence's block with one bulk copy instead of rotating at the start of every segment.
#pragma once

#include "tq_common.cuh"

namespace tq {

constexpr int QROT_WARPS = 8;  // warp w owns the output coordinate blocks w and w + 8 (8 coordinates each)

struct QRotParams {
    const __half* q;         // head vector v of the launch lies at q + (v / H) * q_dim + (v % H) * 128
    const __half* rotation;  // R row-major [128][128]
    __half* q_rot;           // [n_vec][128]
    long long n_vec;         // query head vectors: layers * G * H
    int H, q_dim;
    // Producer form (PRODUCER = true): q holds the projection's raw output; the per-head RMS norm with weights and the
    // rotary embedding of the reference's qk_norm_batch_kernel + rope_batch_kernel (engine/kernels.cu:880-962) are
    // applied on the way in, with the reference's arithmetic and its two roundings to fp16, so that what is rotated
    // is bit for bit what the reference would have stored in its q buffer.
    const __half* norm_w;    // [layers][128] RMS-norm weights of the query heads
    const __half* rope_cos;  // [positions][rope_dim / 2]
    const __half* rope_sin;
    const int* positions;    // [G] device
    int G;                   // sequences per layer: vector v belongs to layer v / (G * H), sequence (v / H) % G
    int rope_dim;            // 64 or 128
    float eps;
    int biased;              // weights are stored minus one (the reference's `biased` flag)
};

// RMS norm + rotary embedding of one head vector spread over the four lanes of a row: lane t4 holds, for m = 0 .. 3,
// the coordinates 32 m + 8 t4 + j (j = 0 .. 7) in a[m].  Sum of squares in the order of the reference's block
// reduction (shuffle-down tree over 32 lanes, then (p0 + p2) + (p1 + p3)); all four lanes get the result.
__device__ __forceinline__ void qk_norm_rope_row(uint4 (&a)[4], const __half* w_row, const __half* cos_row, const __half* sin_row,
                                                 int rope_dim, float eps, int biased, int t4) {
    float val[4][8];
    float part[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const __half2* h2 = reinterpret_cast<const __half2*>(&a[m]);
        float s8[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h2[e]);
            val[m][2 * e] = f.x;
            val[m][2 * e + 1] = f.y;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) s8[j] = mul_ftz(val[m][j], val[m][j]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s8[j] = add_ftz(s8[j], __shfl_xor_sync(0xffffffffu, s8[j], 2));  // lanes i, i + 16
#pragma unroll
        for (int j = 0; j < 8; ++j) s8[j] = add_ftz(s8[j], __shfl_xor_sync(0xffffffffu, s8[j], 1));  // lanes i, i + 8
#pragma unroll
        for (int j = 0; j < 4; ++j) s8[j] = add_ftz(s8[j], s8[j + 4]);
        s8[0] = add_ftz(s8[0], s8[2]);
        s8[1] = add_ftz(s8[1], s8[3]);
        part[m] = add_ftz(s8[0], s8[1]);
    }
    const float ss = add_ftz(add_ftz(part[0], part[2]), add_ftz(part[1], part[3]));
    const float rms = rsqrt_approx_ftz(fma_ftz(ss, 1.0f / HEAD_DIM, eps));  // ss / 128 is exact
    __half hv[4][8];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const uint4 wu = __ldg(reinterpret_cast<const uint4*>(w_row + 32 * m) + t4);
        const __half2* w2 = reinterpret_cast<const __half2*>(&wu);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float2 wf = __half22float2(w2[e]);
            if (biased) { wf.x = add_ftz(wf.x, 1.0f); wf.y = add_ftz(wf.y, 1.0f); }
            hv[m][2 * e] = __float2half_rn(mul_ftz(mul_ftz(val[m][2 * e], rms), wf.x));
            hv[m][2 * e + 1] = __float2half_rn(mul_ftz(mul_ftz(val[m][2 * e + 1], rms), wf.y));
        }
    }
    // rotary pairs (d, d + rope_dim / 2): chunk m with chunk m + rope_dim / 64, both in this lane
    const int hr32 = rope_dim >> 6;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        if (m < hr32) {
            const uint4 cu = __ldg(reinterpret_cast<const uint4*>(cos_row + 32 * m) + t4);
            const uint4 su = __ldg(reinterpret_cast<const uint4*>(sin_row + 32 * m) + t4);
            const __half* ch = reinterpret_cast<const __half*>(&cu);
            const __half* sh = reinterpret_cast<const __half*>(&su);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float c = __half2float(ch[j]), sv = __half2float(sh[j]);
                const float x0 = __half2float(hv[m][j]);
                const float x1 = hr32 == 2 ? __half2float(hv[m + 2][j]) : __half2float(hv[m + 1][j]);
                const __half lo = __float2half_rn(fma_ftz(x0, c, -mul_ftz(x1, sv)));
                const __half hi = __float2half_rn(fma_ftz(x0, sv, mul_ftz(x1, c)));
                hv[m][j] = lo;
                if (hr32 == 2) hv[m + 2][j] = hi; else hv[m + 1][j] = hi;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        __half2 o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = __halves2half2(hv[m][2 * e], hv[m][2 * e + 1]);
        a[m] = *reinterpret_cast<const uint4*>(o);
    }
}

template <bool PRODUCER>
__global__ void __launch_bounds__(QROT_WARPS * 32) rotate_queries_kernel(const QRotParams p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gl = lane >> 2, t4 = lane & 3;
    // B fragments of this warp's two column blocks, kept in registers for the whole launch: 16 contiguous bytes per
    // lane and load; the contraction index is permuted the same way on both operands (step (m, e) of lane t4 covers
    // k = 32 m + 8 t4 + 4 e .. + 3).
    uint4 bq[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint4* rr = reinterpret_cast<const uint4*>(p.rotation + (size_t)(8 * (warp + i * QROT_WARPS) + gl) * HEAD_DIM) + t4;
#pragma unroll
        for (int m = 0; m < 4; ++m) bq[i][m] = __ldg(rr + 4 * m);
    }
    const float sc = 0.12751743074602467f;  // log2(e) / sqrt(128)
    for (long long v0 = (long long)blockIdx.x * 16; v0 < p.n_vec; v0 += (long long)gridDim.x * 16) {
        // rows gl and gl + 8 of this group of 16 head vectors
        uint4 a_lo[4], a_hi[4];
        const long long va = v0 + gl, vb = v0 + gl + 8;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            a_lo[m] = a_hi[m] = make_uint4(0u, 0u, 0u, 0u);
            if (va < p.n_vec)
                a_lo[m] = __ldg(reinterpret_cast<const uint4*>(p.q + (size_t)(va / p.H) * p.q_dim + (size_t)(va % p.H) * HEAD_DIM + 32 * m) + t4);
            if (vb < p.n_vec)
                a_hi[m] = __ldg(reinterpret_cast<const uint4*>(p.q + (size_t)(vb / p.H) * p.q_dim + (size_t)(vb % p.H) * HEAD_DIM + 32 * m) + t4);
        }
        if constexpr (PRODUCER) {
            // (rows past the end carry zeros: their norm is eps, their results are never stored; every lane takes part
            // in the shuffles)
            const long long ra = va < p.n_vec ? va : 0, rb = vb < p.n_vec ? vb : 0;
            const long long lga = ra / p.H, lgb = rb / p.H;
            const int half_rope = p.rope_dim / 2;
            const size_t pa = (size_t)p.positions[(int)(lga % p.G)] * half_rope, pb = (size_t)p.positions[(int)(lgb % p.G)] * half_rope;
            qk_norm_rope_row(a_lo, p.norm_w + (size_t)(lga / p.G) * HEAD_DIM, p.rope_cos + pa, p.rope_sin + pa, p.rope_dim, p.eps, p.biased, t4);
            qk_norm_rope_row(a_hi, p.norm_w + (size_t)(lgb / p.G) * HEAD_DIM, p.rope_cos + pb, p.rope_sin + pb, p.rope_dim, p.eps, p.biased, t4);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int nb = warp + i * QROT_WARPS;
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                mma16816(c, a_lo[m].x, a_hi[m].x, a_lo[m].y, a_hi[m].y, bq[i][m].x, bq[i][m].y);
                mma16816(c, a_lo[m].z, a_hi[m].z, a_lo[m].w, a_hi[m].w, bq[i][m].z, bq[i][m].w);
            }
            const int d = 8 * nb + 2 * t4;
            if (va < p.n_vec) *reinterpret_cast<__half2*>(p.q_rot + (size_t)va * HEAD_DIM + d) = __floats2half2_rn(c[0] * sc, c[1] * sc);
            if (vb < p.n_vec) *reinterpret_cast<__half2*>(p.q_rot + (size_t)vb * HEAD_DIM + d) = __floats2half2_rn(c[2] * sc, c[3] * sc);
        }
    }
}

}  // namespace tq
