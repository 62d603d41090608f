// kv_bits = 0 twin: fp16 KV-cache write and GQA decode attention, sm_100a.
//
// Replaces kv_cache_write_batch_kernel, gqa_attention_batch_kernel and gqa_attention_decode_kernel
// (reference engine/kernels.cu:964-1066, 244-345).  Same mathematics: score = (q . K[p]) / sqrt(128), softmax
// over positions 0..pos with denominator + 1e-8, out = sum w[p] V[p].  The evaluation is split-K with an
// online softmax: a CTA owns (sequence, KV head, 512-token chunk), serves every query head of the KV head
// from one pass over the rows (the reference reads them once per query head), keeps scores in registers
// and leaves (acc, m, l) per query head in the workspace; the last CTA of a sequence-head to arrive (one
// atomicAdd ticket, no spinning) merges the chunks and writes fp16.
//
// A cache row of one head is 256 B, four times the packed 4-bit row, so the instruction budget per byte
// is four times larger than on the quantised path and plain fp32 FMAs with 8-lane shuffle reductions
// keep up with HBM: 8 lanes share a token (16 coordinates each), a warp covers 4 tokens per step, and the rows
// reach the lanes through a per-warp ring of asynchronous 16-byte copies that runs three steps ahead.
#pragma once

#include "tq_common.cuh"

namespace tq {

constexpr int FP16_CHUNK = 512;    // tokens per CTA
constexpr int FP16_WARPS = 4;
constexpr int FP16_STAGES = 4;   // ring slots per warp (2 KB each)
constexpr int FP16_RING_BYTES = FP16_WARPS * FP16_STAGES * 4 * 32 * 16;
constexpr int FP16_MAX_GRP = 8;

struct Fp16AttnParams {
    const __half* q;          // [G][q_dim]
    const __half* ck;         // [rows][kv_dim]
    const __half* cv;
    __half* out;              // [G][q_dim]
    const int* positions;
    const long long* row_base;
    int* tickets;             // [G][Hkv]
    float* partials;          // [G][Hkv][nchunk_max][grp][PART_STRIDE]
    int* status;
    int pos_value;
    int max_seq_len;
    int nchunk_max;
    int G, H, Hkv, q_dim, kv_dim;  // Hkv counts VIRTUAL KV heads: real heads << KV_SHIFT (2^KV_SHIFT CTAs share the
                                   // rows of one real KV head, each serving GRP of its query heads)
};

__global__ void fp16_cache_write_kernel(__half* ck, __half* cv, const __half* k, const __half* v, const int* positions,
                                        const long long* row_base, int max_seq_len, int capacity_rows, int G,
                                        int kv_dim, int* status, const int* seq_capacity = nullptr) {
    const int g = blockIdx.x;
    if (g >= G) return;
    const int pos = positions[g];
    if (seq_capacity) capacity_rows = seq_capacity[g];  // ragged slots: every sequence has its own limit
    if (pos < 0 || (capacity_rows > 0 && pos >= capacity_rows)) {
        if (threadIdx.x == 0 && status) atomicMax(status, ST_BAD_POSITION);
        return;
    }
    const long long row = (row_base ? row_base[g] : (long long)g * max_seq_len) + pos;
    // 16-byte vectors: kv_dim is a multiple of 128
    const uint4* ks = reinterpret_cast<const uint4*>(k + (size_t)g * kv_dim);
    const uint4* vs = reinterpret_cast<const uint4*>(v + (size_t)g * kv_dim);
    uint4* kd = reinterpret_cast<uint4*>(ck + (size_t)row * kv_dim);
    uint4* vd = reinterpret_cast<uint4*>(cv + (size_t)row * kv_dim);
    for (int i = threadIdx.x; i < kv_dim / 8; i += blockDim.x) {
        kd[i] = ks[i];
        vd[i] = vs[i];
    }
}

template <int GRP, int KV_SHIFT>
__global__ void __launch_bounds__(FP16_WARPS * 32)
fp16_decode_attention_kernel(const Fp16AttnParams p) {
    const int kvh = blockIdx.x, chunk = blockIdx.y, g = blockIdx.z;
    const int pos = p.positions ? p.positions[g] : p.pos_value;
    const int L = (pos < 0 ? 0 : pos) + 1;
    const int c0 = chunk * FP16_CHUNK;
    if (c0 >= L) return;
    const int c1 = min(L, c0 + FP16_CHUNK);
    const int nparts = (L + FP16_CHUNK - 1) / FP16_CHUNK;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane & 7;   // which 16 coordinates of the row: 8*sub .. 8*sub+7 and 64+8*sub .. 64+8*sub+7 (a copy
                                // instruction of 8 lanes then covers 128 contiguous bytes)
    const int tg = lane >> 3;   // which of the 4 tokens of a step
    const long long row0 = p.row_base ? p.row_base[g] : (long long)g * p.max_seq_len;

    // queries of this KV head, 16 coordinates per lane, scaled by log2(e)/sqrt(128)
    float qf[GRP][16];
#pragma unroll
    for (int h = 0; h < GRP; ++h) {
        const __half* src = p.q + (size_t)g * p.q_dim + (size_t)(kvh * GRP + h) * HEAD_DIM + 8 * sub;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint4 u = __ldg(reinterpret_cast<const uint4*>(src + 64 * i));
            const __half2* h2 = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __half22float2(h2[j]);
                qf[h][8 * i + 2 * j] = f.x * 0.12751743074602467f;
                qf[h][8 * i + 2 * j + 1] = f.y * 0.12751743074602467f;
            }
        }
    }
    float m_run[GRP], l_run[GRP], acc[GRP][16];
#pragma unroll
    for (int h = 0; h < GRP; ++h) {
        m_run[h] = -1e30f;
        l_run[h] = 0.0f;
#pragma unroll
        for (int c = 0; c < 16; ++c) acc[h][c] = 0.0f;
    }

    // tokens of this warp: c0 + warp*4 + tg, stepping by 4*FP16_WARPS
    const int step = 4 * FP16_WARPS;
    // Rows travel through a per-warp ring in shared memory filled by 16-byte asynchronous copies, FP16_STAGES - 1 steps
    // (2 KB each) ahead of the arithmetic.  Every lane reads back exactly the 64 bytes it asked for itself, so waiting
    // for its own copy groups is all the synchronisation the ring needs.
    __shared__ __align__(16) unsigned char sm_ring[FP16_RING_BYTES];
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(sm_ring) + (uint32_t)warp * (FP16_STAGES * 4 * 32 * 16) + (uint32_t)lane * 16u;
    const int t_first = c0 + warp * 4;
    const int nsteps = t_first < c1 ? (c1 - t_first + step - 1) / step : 0;
    auto issue = [&](int i) {
        const int tok = t_first + i * step + tg;
        if (i < nsteps && tok < c1) {
            const size_t off = (size_t)(row0 + tok) * p.kv_dim + (size_t)(kvh >> KV_SHIFT) * HEAD_DIM + 8 * sub;
            const uint32_t dst = ring + (uint32_t)(i % FP16_STAGES) * (4 * 32 * 16);
            const __half* kp = p.ck + off;
            const __half* vp = p.cv + off;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(kp) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 512u), "l"(kp + 64) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 1024u), "l"(vp) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 1536u), "l"(vp + 64) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per step, empty or not: the count stays uniform
    };
#pragma unroll
    for (int i = 0; i < FP16_STAGES - 1; ++i) issue(i);
    for (int i = 0; i < nsteps; ++i) {
        const int tok = t_first + i * step + tg;
        const bool valid = tok < c1;
        issue(i + FP16_STAGES - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(FP16_STAGES - 1) : "memory");
        uint4 k0 = make_uint4(0, 0, 0, 0), k1 = k0, v0 = k0, v1 = k0;
        if (valid) {
            const uint32_t src = ring + (uint32_t)(i % FP16_STAGES) * (4 * 32 * 16);
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(k0.x), "=r"(k0.y), "=r"(k0.z), "=r"(k0.w) : "r"(src) : "memory");
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(k1.x), "=r"(k1.y), "=r"(k1.z), "=r"(k1.w) : "r"(src + 512u) : "memory");
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v0.x), "=r"(v0.y), "=r"(v0.z), "=r"(v0.w) : "r"(src + 1024u) : "memory");
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v1.x), "=r"(v1.y), "=r"(v1.z), "=r"(v1.w) : "r"(src + 1536u) : "memory");
        }
        float kf[16], vf[16];
        {
            const __half2* a = reinterpret_cast<const __half2*>(&k0);
            const __half2* b = reinterpret_cast<const __half2*>(&k1);
            const __half2* c = reinterpret_cast<const __half2*>(&v0);
            const __half2* d = reinterpret_cast<const __half2*>(&v1);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f;
                f = __half22float2(a[j]); kf[2 * j] = f.x; kf[2 * j + 1] = f.y;
                f = __half22float2(b[j]); kf[8 + 2 * j] = f.x; kf[8 + 2 * j + 1] = f.y;
                f = __half22float2(c[j]); vf[2 * j] = f.x; vf[2 * j + 1] = f.y;
                f = __half22float2(d[j]); vf[8 + 2 * j] = f.x; vf[8 + 2 * j + 1] = f.y;
            }
        }
        float s[GRP];
#pragma unroll
        for (int h = 0; h < GRP; ++h) {
            float d = 0.0f;
#pragma unroll
            for (int c = 0; c < 16; ++c) d = fmaf(qf[h][c], kf[c], d);
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            d += __shfl_xor_sync(0xffffffffu, d, 2);
            d += __shfl_xor_sync(0xffffffffu, d, 4);
            s[h] = valid ? d : -1e30f;
        }
        bool grew = false;
#pragma unroll
        for (int h = 0; h < GRP; ++h) grew |= (s[h] > m_run[h]);
        if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
            for (int h = 0; h < GRP; ++h) {
                const float mn = fmaxf(m_run[h], s[h]);
                const float corr = ex2_approx(m_run[h] - mn);
                m_run[h] = mn;
                l_run[h] *= corr;
#pragma unroll
                for (int c = 0; c < 16; ++c) acc[h][c] *= corr;
            }
        }
#pragma unroll
        for (int h = 0; h < GRP; ++h) {
            const float pw = valid ? ex2_approx(s[h] - m_run[h]) : 0.0f;
            l_run[h] += pw;
#pragma unroll
            for (int c = 0; c < 16; ++c) acc[h][c] = fmaf(pw, vf[c], acc[h][c]);
        }
    }

    // ---- combine the 4 token groups of the warp, then the warps ----
    // the ring is idle from here on (every copy group has been waited for): the per-warp results reuse its space
    static_assert(sizeof(float) * FP16_WARPS * GRP * HEAD_DIM <= FP16_RING_BYTES, "results must fit the ring");
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    float (*sm_acc)[GRP][HEAD_DIM] = reinterpret_cast<float (*)[GRP][HEAD_DIM]>(sm_ring);
    __shared__ float sm_m[FP16_WARPS][GRP], sm_l[FP16_WARPS][GRP];
    __shared__ int sm_last;
#pragma unroll
    for (int h = 0; h < GRP; ++h) {
        float m = m_run[h];
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
        const float w = ex2_approx(m_run[h] - m);
        float l = l_run[h] * w;
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            float a = acc[h][c] * w;
            a += __shfl_xor_sync(0xffffffffu, a, 8);
            a += __shfl_xor_sync(0xffffffffu, a, 16);
            if (tg == 0) sm_acc[warp][h][(c < 8 ? 0 : 56) + 8 * sub + c] = a;
        }
        if (lane == 0) {
            sm_m[warp][h] = m;
            sm_l[warp][h] = l;
        }
    }
    __syncthreads();
    float* part = p.partials + ((((size_t)g * p.Hkv + kvh) * p.nchunk_max + chunk) * GRP) * PART_STRIDE;
    for (int idx = tid; idx < GRP * HEAD_DIM; idx += blockDim.x) {
        const int h = idx >> 7, dcoord = idx & 127;
        float M = -1e30f;
#pragma unroll
        for (int w = 0; w < FP16_WARPS; ++w) M = fmaxf(M, sm_m[w][h]);
        float a = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < FP16_WARPS; ++w) {
            const float wt = ex2_approx(sm_m[w][h] - M);
            a += sm_acc[w][h][dcoord] * wt;
            l += sm_l[w][h] * wt;
        }
        if (nparts == 1) {
            p.out[(size_t)g * p.q_dim + (size_t)(kvh * GRP + h) * HEAD_DIM + dcoord] = __float2half_rn(a / (l + 1e-8f));
        } else {
            part[(size_t)h * PART_STRIDE + dcoord] = a;
            if (dcoord == 0) {
                part[(size_t)h * PART_STRIDE + HEAD_DIM] = M;
                part[(size_t)h * PART_STRIDE + HEAD_DIM + 1] = l;
            }
        }
    }
    if (nparts == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(p.tickets + g * p.Hkv + kvh, 1);
        sm_last = (old == nparts - 1);
        if (sm_last) p.tickets[g * p.Hkv + kvh] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!sm_last) return;
    __threadfence();
    const float* base = p.partials + (((size_t)g * p.Hkv + kvh) * p.nchunk_max) * GRP * PART_STRIDE;
    for (int idx = tid; idx < GRP * HEAD_DIM; idx += blockDim.x) {
        const int h = idx >> 7, dcoord = idx & 127;
        float M = -1e30f;
        for (int c = 0; c < nparts; ++c) M = fmaxf(M, __ldcg(base + ((size_t)c * GRP + h) * PART_STRIDE + HEAD_DIM));
        float a = 0.0f, l = 0.0f;
        for (int c = 0; c < nparts; ++c) {
            const float* src = base + ((size_t)c * GRP + h) * PART_STRIDE;
            const float wt = ex2_approx(__ldcg(src + HEAD_DIM) - M);
            a += __ldcg(src + dcoord) * wt;
            l += __ldcg(src + HEAD_DIM + 1) * wt;
        }
        p.out[(size_t)g * p.q_dim + (size_t)(kvh * GRP + h) * HEAD_DIM + dcoord] = __float2half_rn(a / (l + 1e-8f));
    }
}

}  // namespace tq
