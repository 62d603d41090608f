// kv_bits = 0 twin on the tensor cores: GQA decode attention over an fp16 cache for 4 or 8 query heads per KV head
// (and fewer), sm_100a.
//
// Replaces gqa_attention_batch_kernel / gqa_attention_decode_kernel (reference engine/kernels.cu:981-1066, 244-345).
// Same mathematics and the same split-K decomposition as fp16_decode_attention_kernel (tq_fp16.cuh): a CTA owns
// (sequence, KV head, 512-token chunk), its four warps leave (acc, m, l) per query head, the last CTA of a sequence
// and KV head to arrive merges the chunks.  What differs is the arithmetic: with four or eight query heads per KV head
// the fp32-FMA form needs 4-8 FMAs per cache byte and is bound by them (half or a quarter of the copy bandwidth); here
// the fp16 rows ARE tensor-core operands:
//   * scores   S^T = K (16 token rows x 16 coordinates) . Q^T (16 coordinates x 8 query heads), 8 steps per 16 tokens,
//     K fragments straight from shared memory by ldmatrix, Q fragments resident in registers (unscaled fp16: exact);
//   * values   out^T (16 coordinates x 8 heads) += V^T (16 coordinates x 16 tokens) . P^T (16 tokens x 8 heads), V^T
//     fragments by ldmatrix.trans from the row-major tile, P^T from the score layout by movmatrix.
// Rows reach shared memory by TMA tensor-map copies (no multicast) of 16 rows x 256 B per array with the 128-byte
// swizzle, into a ring that is PRIVATE to a warp (three stages of 8 KB): the warp that fills a stage is the one that
// reads it, so one mbarrier per stage and no hand-over between warps.  Every wait is bounded.
#pragma once

#include "tq_attention.cuh"  // movmatrix_trans
#include "tq_fp16.cuh"

namespace tq {

constexpr int FP16TC_WARPS = 4;
constexpr int FP16TC_STAGES = 3;
constexpr int FP16TC_BLOCK = 16;                                // tokens per step of a warp
constexpr uint32_t FP16TC_ARRAY_BYTES = FP16TC_BLOCK * 256u;    // one array's rows of a step: [2 blocks][16 rows][128 B]
constexpr uint32_t FP16TC_STAGE_BYTES = 2u * FP16TC_ARRAY_BYTES;
constexpr size_t FP16TC_SMEM = (size_t)FP16TC_WARPS * FP16TC_STAGES * FP16TC_STAGE_BYTES + 1024 + 256;  // + alignment + barriers

// GRP = query heads per KV head (1, 2, 4 or 8).  tmK / tmV: the fp16 arrays viewed as bytes, dimensions (128 B, rows,
// 128-byte blocks of a row), box (128 B, 16 rows, 2 blocks = one head's 256 B).
template <int GRP>
__global__ void __launch_bounds__(FP16TC_WARPS * 32)
fp16_tc_decode_attention_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                                const Fp16AttnParams p) {
    extern __shared__ __align__(1024) uint8_t tc16_smem[];
    const int kvh = blockIdx.x, chunk = blockIdx.y, g = blockIdx.z;
    const int pos = p.positions ? p.positions[g] : p.pos_value;
    const int L = (pos < 0 ? 0 : pos) + 1;
    const int c0 = chunk * FP16_CHUNK;
    if (c0 >= L) return;
    const int c1 = min(L, c0 + FP16_CHUNK);
    const int nparts = (L + FP16_CHUNK - 1) / FP16_CHUNK;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gl = lane >> 2, t4 = lane & 3;
    const long long row0 = p.row_base ? p.row_base[g] : (long long)g * p.max_seq_len;

    const uint32_t base = (smem_u32(tc16_smem) + 1023u) & ~1023u;
    const uint32_t ring = base + (uint32_t)warp * (FP16TC_STAGES * FP16TC_STAGE_BYTES);
    const uint32_t bars = base + (uint32_t)FP16TC_WARPS * (FP16TC_STAGES * FP16TC_STAGE_BYTES) + (uint32_t)warp * (FP16TC_STAGES * 8u);
    if (lane == 0) {
        for (int s = 0; s < FP16TC_STAGES; ++s) mbar_init(bars + 8u * s, 1);
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    __syncwarp();

    // Q^T fragments of this KV head's query heads: lane (gl, t4) holds head gl, coordinates 16 j + 2 t4 (+1) and + 8
    uint32_t qb[8][2];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        qb[j][0] = qb[j][1] = 0u;
        if (gl < GRP) {
            const __half* src = p.q + (size_t)g * p.q_dim + (size_t)(kvh * GRP + gl) * HEAD_DIM + 16 * j + 2 * t4;
            qb[j][0] = __ldg(reinterpret_cast<const unsigned int*>(src));
            qb[j][1] = __ldg(reinterpret_cast<const unsigned int*>(src + 8));
        }
    }

    // this warp's token blocks: c0 + 16 * (warp + 4 * i)
    const int t_first = c0 + warp * FP16TC_BLOCK;
    constexpr int step = FP16TC_BLOCK * FP16TC_WARPS;
    const int nsteps = t_first < c1 ? (c1 - t_first + step - 1) / step : 0;
    auto issue = [&](int i) {  // lane 0 only
        const int tok = t_first + i * step;
        const uint32_t dst = ring + (uint32_t)(i % FP16TC_STAGES) * FP16TC_STAGE_BYTES;
        const uint32_t bar = bars + 8u * (uint32_t)(i % FP16TC_STAGES);
        mbar_arrive_expect_tx(bar, FP16TC_STAGE_BYTES);  // a box always delivers its full size (rows past the array end: zeros)
        tma_load_3d(dst, &tmK, bar, 0, (int)(row0 + tok), 2 * kvh);
        tma_load_3d(dst + FP16TC_ARRAY_BYTES, &tmV, bar, 0, (int)(row0 + tok), 2 * kvh);
    };
    if (lane == 0)
        for (int i = 0; i < FP16TC_STAGES && i < nsteps; ++i) issue(i);

    float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.0f, 0.0f};  // columns = heads 2 t4, 2 t4 + 1
    float acc[8][4];
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.0f;
    bool dead = false;
    // ldmatrix row addresses: matrix mi = lane >> 3, row within it lane & 7.  Element (row r, 16-byte chunk c of the 256-byte
    // head row) lies at block (c >> 3) * 2048 + r * 128 + ((c & 7) ^ (r & 7)) * 16.
    const int mi = lane >> 3, mr = lane & 7;
    const int k_row = (mi & 1) * 8 + mr, k_cadd = mi >> 1;   // K: matrices (rows 0-7, c), (rows 8-15, c), (rows 0-7, c+1), (rows 8-15, c+1)
    const int v_row = (mi >> 1) * 8 + mr, v_cadd = mi & 1;   // V^T: (tokens 0-7, c), (tokens 0-7, c+1), (tokens 8-15, c), (tokens 8-15, c+1)

    for (int i = 0; i < nsteps; ++i) {
        const int tok0 = t_first + i * step;
        const int s = i % FP16TC_STAGES;
        const uint32_t bar = bars + 8u * (uint32_t)s, parity = (uint32_t)(i / FP16TC_STAGES) & 1u;
        if (!dead) {
            uint32_t ok = 0;
            for (uint32_t it = 0; it < (1u << 14) && !ok; ++it) ok = mbar_try_wait_hint(bar, parity, 20000u);
            if (!ok) {
                dead = true;
                if (lane == 0 && p.status) atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
            }
            dead = __any_sync(0xffffffffu, dead);
        }
        if (dead) break;
        const uint32_t kt = ring + (uint32_t)s * FP16TC_STAGE_BYTES, vt = kt + FP16TC_ARRAY_BYTES;
        const int valid = min(FP16TC_BLOCK, c1 - tok0);  // rows of the block that are attended to
        if (valid < FP16TC_BLOCK) {
            // the rows past the position may hold anything (even NaN): zero the V rows so that 0 * x stays 0
            for (int idx = lane; idx < (FP16TC_BLOCK - valid) * 16; idx += 32) {
                const int r = valid + (idx >> 4), c = idx & 15;
                const uint32_t a = vt + (uint32_t)(c >> 3) * 2048u + (uint32_t)r * 128u + (uint32_t)(((c & 7) ^ (r & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(a), "r"(0u) : "memory");
            }
            __syncwarp();
        }
        // ---- scores: two accumulator chains over the eight 16-coordinate steps ----
        float ce[4] = {0.f, 0.f, 0.f, 0.f}, co[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t a[4];
            const int c = 2 * j + k_cadd;
            ldmatrix_x4(a, kt + (uint32_t)(c >> 3) * 2048u + (uint32_t)k_row * 128u + (uint32_t)(((c & 7) ^ (k_row & 7)) << 4));
            if (j & 1) mma16816(co, a[0], a[1], a[2], a[3], qb[j][0], qb[j][1]);
            else mma16816(ce, a[0], a[1], a[2], a[3], qb[j][0], qb[j][1]);
        }
        // sv[half][e]: token tok0 + gl + 8 * half, head 2 t4 + e; log2(e) / sqrt(128) folded in here (the queries stay exact)
        float sv[2][2];
        const float sc = 0.12751743074602467f;
        sv[0][0] = (ce[0] + co[0]) * sc; sv[0][1] = (ce[1] + co[1]) * sc;
        sv[1][0] = (ce[2] + co[2]) * sc; sv[1][1] = (ce[3] + co[3]) * sc;
        if (gl >= valid) sv[0][0] = sv[0][1] = -1e30f;
        if (gl + 8 >= valid) sv[1][0] = sv[1][1] = -1e30f;
        float mx0 = fmaxf(sv[0][0], sv[1][0]), mx1 = fmaxf(sv[0][1], sv[1][1]);
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
        }
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        if (__any_sync(0xffffffffu, mn0 > m_run[0] || mn1 > m_run[1])) {
            const float f0 = ex2_approx(m_run[0] - mn0), f1 = ex2_approx(m_run[1] - mn1);
            l_run[0] *= f0;
            l_run[1] *= f1;
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                acc[b][0] *= f0; acc[b][2] *= f0;
                acc[b][1] *= f1; acc[b][3] *= f1;
            }
            m_run[0] = mn0;
            m_run[1] = mn1;
        }
        float pv[2][2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            pv[h][0] = ex2_approx(sv[h][0] - m_run[0]);
            pv[h][1] = ex2_approx(sv[h][1] - m_run[1]);
        }
        if (gl >= valid) pv[0][0] = pv[0][1] = 0.0f;
        if (gl + 8 >= valid) pv[1][0] = pv[1][1] = 0.0f;
        l_run[0] += pv[0][0] + pv[1][0];
        l_run[1] += pv[0][1] + pv[1][1];
        // P^T as the B operand: lane (gl, t4) receives head gl of the tokens 2 t4, 2 t4 + 1 (and + 8)
        const uint32_t pb0 = movmatrix_trans(pack_half2(pv[0][0], pv[0][1]));
        const uint32_t pb1 = movmatrix_trans(pack_half2(pv[1][0], pv[1][1]));
        // ---- values: eight blocks of 16 coordinates ----
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            uint32_t a[4];
            const int c = 2 * b + v_cadd;
            ldmatrix_x4_trans(a, vt + (uint32_t)(c >> 3) * 2048u + (uint32_t)v_row * 128u + (uint32_t)(((c & 7) ^ (v_row & 7)) << 4));
            mma16816(acc[b], a[0], a[1], a[2], a[3], pb0, pb1);
        }
        // the stage is free again (its reads fed the mma instructions above): this warp's block FP16TC_STAGES further on
        __syncwarp();
        if (lane == 0 && i + FP16TC_STAGES < nsteps) {
            fence_proxy_async_smem();
            issue(i + FP16TC_STAGES);
        }
    }
    if (dead) {  // give copies still in flight a bounded chance to land before the shared memory goes away
        for (int s = 0; s < FP16TC_STAGES; ++s) {
            mbar_wait_bounded(bars + 8u * s, 0u, 1u << 14);
            mbar_wait_bounded(bars + 8u * s, 1u, 1u << 14);
        }
    }

    // ---- combine the lanes' token rows, then the warps (the rings are idle: their space takes the per-warp results) ----
    float ls0 = l_run[0], ls1 = l_run[1];
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        ls0 += __shfl_xor_sync(0xffffffffu, ls0, o);
        ls1 += __shfl_xor_sync(0xffffffffu, ls1, o);
    }
    __syncthreads();
    static_assert(sizeof(float) * FP16TC_WARPS * 8 * HEAD_DIM <= (size_t)FP16TC_WARPS * FP16TC_STAGES * FP16TC_STAGE_BYTES, "results must fit the rings");
    float (*sm_acc)[8][HEAD_DIM] = reinterpret_cast<float (*)[8][HEAD_DIM]>(tc16_smem + (base - smem_u32(tc16_smem)));
    __shared__ float sm_m[FP16TC_WARPS][8], sm_l[FP16TC_WARPS][8];
    __shared__ int sm_last;
#pragma unroll
    for (int b = 0; b < 8; ++b) {  // acc[b]: coordinates 16 b + gl (and + 8), heads 2 t4, 2 t4 + 1
        sm_acc[warp][2 * t4][16 * b + gl] = acc[b][0];
        sm_acc[warp][2 * t4 + 1][16 * b + gl] = acc[b][1];
        sm_acc[warp][2 * t4][16 * b + gl + 8] = acc[b][2];
        sm_acc[warp][2 * t4 + 1][16 * b + gl + 8] = acc[b][3];
    }
    if (gl == 0) {
        sm_m[warp][2 * t4] = m_run[0];
        sm_m[warp][2 * t4 + 1] = m_run[1];
        sm_l[warp][2 * t4] = ls0;
        sm_l[warp][2 * t4 + 1] = ls1;
    }
    __syncthreads();
    float* part = p.partials + ((((size_t)g * p.Hkv + kvh) * p.nchunk_max + chunk) * GRP) * PART_STRIDE;
    for (int idx = tid; idx < GRP * HEAD_DIM; idx += blockDim.x) {
        const int h = idx >> 7, dcoord = idx & 127;
        float M = -1e30f;
#pragma unroll
        for (int w = 0; w < FP16TC_WARPS; ++w) M = fmaxf(M, sm_m[w][h]);
        float a = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < FP16TC_WARPS; ++w) {
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
    const float* pbase = p.partials + (((size_t)g * p.Hkv + kvh) * p.nchunk_max) * GRP * PART_STRIDE;
    for (int idx = tid; idx < GRP * HEAD_DIM; idx += blockDim.x) {
        const int h = idx >> 7, dcoord = idx & 127;
        float M = -1e30f;
        for (int c = 0; c < nparts; ++c) M = fmaxf(M, __ldcg(pbase + ((size_t)c * GRP + h) * PART_STRIDE + HEAD_DIM));
        float a = 0.0f, l = 0.0f;
        for (int c = 0; c < nparts; ++c) {
            const float* src = pbase + ((size_t)c * GRP + h) * PART_STRIDE;
            const float wt = ex2_approx(__ldcg(src + HEAD_DIM) - M);
            a += __ldcg(src + dcoord) * wt;
            l += __ldcg(src + HEAD_DIM + 1) * wt;
        }
        p.out[(size_t)g * p.q_dim + (size_t)(kvh * GRP + h) * HEAD_DIM + dcoord] = __float2half_rn(a / (l + 1e-8f));
    }
}

}  // namespace tq
