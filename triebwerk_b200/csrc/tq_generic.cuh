// Decode attention over the packed cache for head layouts outside the streaming kernel's (tq_attention.cuh serves
// 4 or 8 KV heads with at most 8 query heads each and at most 32 query heads).  The reference kernels take any
// layout (engine/kernels.cu:1641-1660, grid (G, num_heads)); this kernel keeps that generality -- one CTA per
// (sequence, query head), any num_heads that is a multiple of num_kv_heads -- with the same mathematics evaluated as
// an online softmax, so it needs no score scratch either.  It is the slow path: every cache byte is read once per
// query head, as in the reference.
#pragma once

#include "tq_common.cuh"

namespace tq {

struct GenericAttnParams {
    const uint8_t* ck;
    const uint8_t* cv;
    const __half* kn;
    const __half* vn;
    const __half* q;          // [G][q_dim], not rotated
    const __half* rotation;   // R row-major
    __half* out;              // [G][q_dim]
    const int* positions;     // device [G] or null
    const long long* row_base;
    int pos_value, max_seq_len;
    int G, H, Hkv, q_dim, bits;
};

constexpr int GENERIC_WARPS = 4;

// FP16 = true: the kv_bits = 0 twin (rows of fp16 values, ck/cv viewed as __half [rows][Hkv * 128], no norms, no rotation).
template <bool FP16>
__global__ void __launch_bounds__(GENERIC_WARPS * 32) generic_decode_attention_kernel(const GenericAttnParams p) {
    __shared__ float q_s[HEAD_DIM];                     // the query, then its rotation
    __shared__ float qr_s[HEAD_DIM];
    __shared__ float acc_s[GENERIC_WARPS][HEAD_DIM];
    __shared__ float ml_s[GENERIC_WARPS][2];
    const int g = blockIdx.x, head = blockIdx.y;
    const int d = threadIdx.x, lane = d & 31, warp = d >> 5;
    const int kvh = head / (p.H / p.Hkv);
    const int pos = p.positions ? p.positions[g] : p.pos_value;
    const int L = (pos < 0 ? 0 : pos) + 1;
    const long long row0 = p.row_base ? p.row_base[g] : (long long)g * p.max_seq_len;
    const int vpb = p.bits == 2 ? 4 : 2, bph = FP16 ? HEAD_DIM * 2 : HEAD_DIM / vpb, kvp = p.Hkv * bph;  // bytes per head / per row

    // q_rot[d] = sum_k R[d][k] * q[k] (k ascending, as the reference), scaled by log2(e) / sqrt(128)
    q_s[d] = __half2float(p.q[(size_t)g * p.q_dim + (size_t)head * HEAD_DIM + d]);
    __syncthreads();
    if (FP16) {
        qr_s[d] = q_s[d] * 0.12751743074602467f;
    } else {
        float r = 0.0f;
        const __half* rrow = p.rotation + (size_t)d * HEAD_DIM;
        for (int k = 0; k < HEAD_DIM; ++k) r = fmaf(__half2float(rrow[k]), q_s[k], r);
        qr_s[d] = r * 0.12751743074602467f;
    }
    __syncthreads();

    // lane owns the coordinates 4 * lane .. 4 * lane + 3: two code bytes at 4-bit, one at 2-bit
    const float4 ql = *reinterpret_cast<const float4*>(&qr_s[4 * lane]);
    auto centroids4 = [&](const uint8_t* base) -> float4 {  // the lane's four values of one head row
        if (FP16) {
            const uint2 u = *reinterpret_cast<const uint2*>(base + 8 * lane);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
            return make_float4(a.x, a.y, b.x, b.y);
        }
        if (p.bits == 4) {
            const unsigned short w = *reinterpret_cast<const unsigned short*>(base + 2 * lane);
            return make_float4(kCent4[w & 15], kCent4[(w >> 4) & 15], kCent4[(w >> 8) & 15], kCent4[(w >> 12) & 15]);
        }
        const uint8_t b = base[lane];
        return make_float4(kCent2[b & 3], kCent2[(b >> 2) & 3], kCent2[(b >> 4) & 3], kCent2[(b >> 6) & 3]);
    };
    float m = -1e30f, l = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int t = warp; t < L; t += GENERIC_WARPS) {
        const size_t row = (size_t)(row0 + t);
        const float4 kc = centroids4(p.ck + row * kvp + (size_t)kvh * bph);
        float dot = ql.x * kc.x + ql.y * kc.y + ql.z * kc.z + ql.w * kc.w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float s = FP16 ? dot : dot * __half2float(p.kn[row * p.Hkv + kvh]);
        const float mn = fmaxf(m, s);
        const float corr = ex2_approx(m - mn), w = ex2_approx(s - mn);
        const float wv = FP16 ? w : w * __half2float(p.vn[row * p.Hkv + kvh]);
        const float4 vc = centroids4(p.cv + row * kvp + (size_t)kvh * bph);
        acc.x = acc.x * corr + wv * vc.x; acc.y = acc.y * corr + wv * vc.y;
        acc.z = acc.z * corr + wv * vc.z; acc.w = acc.w * corr + wv * vc.w;
        l = l * corr + w;
        m = mn;
    }
    *reinterpret_cast<float4*>(&acc_s[warp][4 * lane]) = acc;
    if (lane == 0) {
        ml_s[warp][0] = m;
        ml_s[warp][1] = l;
    }
    __syncthreads();
    // merge the warps' partial results; thread d owns rotated coordinate d
    float M = -1e30f;
#pragma unroll
    for (int w = 0; w < GENERIC_WARPS; ++w) M = fmaxf(M, ml_s[w][0]);
    float Z = 0.0f, a = 0.0f;
#pragma unroll
    for (int w = 0; w < GENERIC_WARPS; ++w) {
        const float e = ex2_approx(ml_s[w][0] - M);
        Z += ml_s[w][1] * e;
        a += acc_s[w][d] * e;
    }
    __syncthreads();
    q_s[d] = a / (Z + 1e-8f);
    __syncthreads();
    // out[d] = sum_k R[k][d] * acc[k]
    float o = FP16 ? q_s[d] : 0.0f;
    for (int k = 0; !FP16 && k < HEAD_DIM; ++k) o = fmaf(__half2float(p.rotation[(size_t)k * HEAD_DIM + d]), q_s[k], o);
    p.out[(size_t)g * p.q_dim + (size_t)head * HEAD_DIM + d] = __float2half_rn(o);
}

}  // namespace tq
