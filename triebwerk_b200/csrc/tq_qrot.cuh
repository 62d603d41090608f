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
};

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
