// GQA decode attention over the TurboQuant packed cache, sm_100a.
//
// Replaces turbo_gqa_attention_batch_kernel / turbo_gqa_attention_kernel (reference
// engine/kernels.cu:1641-1870).  Same mathematics -- score = (q_rot . centroids[codesK]) * k_norm / sqrt(128),
// softmax over positions 0..pos with denominator + 1e-8, V accumulated in rotated space as
// sum w * v_norm * centroids[codesV], one multiplication by R^T per head -- evaluated as a split-K
// online-softmax (flash-decoding) so that no score ever goes to global memory.
//
// Decomposition
//   * The (sequence, 32-token tile) pairs of the whole batch form one flat list (lengths come from the
//     device-side positions, so the launch geometry never depends on them and the launch can be captured in
//     a CUDA graph).  CTA i of W takes the contiguous slice [i*N/W, (i+1)*N/W) of that list: every SM gets
//     the same number of bytes whatever the mix of sequence lengths.
//   * Inside a CTA warp w owns KV head w and all of its query heads (2 for Qwen3-0.6B, 4 for Qwen3-8B): every
//     cache byte is fetched from HBM once, not once per query head as in the reference.
//   * Each warp runs its own TMA pipeline: lane 0 issues cp.async.bulk.tensor.2d (no multicast) for a
//     [32 tokens][64 B] K box and V box of its head into a 4-deep ring of shared-memory stages, completion on
//     one mbarrier per stage.  Warps never wait for one another inside a sequence.
//   * Codes are turned into fp16 centroids one BYTE at a time (2 codes for 4-bit, 4 for 2-bit) through a
//     shared-memory table with one private column per lane (bank-conflict free); the table sits at shared
//     address 0x10000 so that a single PRMT builds the lookup address from the packed word.
//   * The dot products run on the tensor cores with warp-level mma.sync.m16n8k16 (fp16 in, fp32 accumulate):
//     scores as Q(16 x 16) * K^T(16 x 8 tokens) with the query split into an fp16 high part (rows 0-7) and
//     low part (rows 8-15) so that no query precision is lost, and the value sum in transposed form
//     V^T(16 coords x 16 tokens) * P^T(16 tokens x 8 heads).  Scalar fp32 FMAs cannot keep up with HBM3e on
//     this path: 512 FMAs per 132-byte row would need more than the SMs can issue.
//   * A CTA that finishes its part of a sequence writes (acc[128], m, l) per query head to the workspace and
//     takes a ticket; the last arrival merges all parts, divides, multiplies by R^T and writes fp16.  Nobody
//     spins on anybody: the ticket is a single atomicAdd.
#pragma once

#include "tq_common.cuh"

namespace tq {

constexpr int ATTN_STAGES = 4;
constexpr uint32_t LUT_ABS = 0x10000u;        // absolute shared address of the byte -> centroid table
constexpr uint32_t LUT_BYTES = 0x10000u;      // 256 entries x 256 B
constexpr uint32_t REGION_B_ABS = 0x20000u;   // stages 1.. live above the table
constexpr int ATTN_MAX_HEADS = 32;            // merge buffer is 128 x 32 floats
constexpr size_t ATTN_DYN_SMEM = 226 * 1024;  // requested dynamic shared memory

struct AttnParams {
    const __half* kn;
    const __half* vn;
    const float* q_rot;       // [G][H][128], pre-scaled by log2(e)/sqrt(128)
    const __half* rotation;   // [128][128]
    __half* out;              // [G][q_dim]
    const int* positions;     // device [G] or null
    const long long* row_base;
    const int* tile_start;    // [G+1]
    int* tickets;             // [G]
    float* partials;          // [W+G][H][PART_STRIDE]
    int* status;
    int pos_value;
    int max_seq_len;
    int G, H, Hkv, q_dim;
};

template <int BITS>
struct AttnGeom {
    static constexpr int BPH = (BITS == 4) ? 64 : 32;         // code bytes per head per token
    static constexpr int TILE_BYTES = TILE_TOKENS * BPH;      // one K (or V) box
    static constexpr int WARP_STAGE_BYTES = 2 * TILE_BYTES;   // K box + V box
};

// Region A (below the table): barriers, norm stash, merge buffer, stage 0.
struct RegionA {
    static constexpr uint32_t BAR_OFF = 0;                                   // up to 16 warps x 4 stages x 8 B
    static constexpr uint32_t NORM_OFF = 512;                                // 16 warps x 2 x 32 floats = 4 KB
    static constexpr uint32_t CTRL_OFF = NORM_OFF + 16 * 2 * 32 * 4;         // flags
    static constexpr uint32_t MERGE_OFF = CTRL_OFF + 256;                    // 128 x 32 floats = 16 KB
    static constexpr uint32_t STAGE0_OFF = MERGE_OFF + HEAD_DIM * ATTN_MAX_HEADS * 4;  // 21248 -> align 1024
};

template <int BITS>
__global__ void __launch_bounds__(256, 1)
decode_attention_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const AttnParams p) {
    using Geo = AttnGeom<BITS>;
    extern __shared__ __align__(1024) uint8_t dyn_smem[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;           // = KV head
    const int gl = lane >> 2;            // mma "group id": token (K side), coordinate row (V side), head (S layout)
    const int t4 = lane & 3;             // mma "thread in group"
    const int grp = p.H / p.Hkv;         // query heads per KV head (<= 8)
    const int nthreads = blockDim.x;

    // ---- shared memory map (absolute shared addresses) ----
    const uint32_t dyn_base = smem_u32(dyn_smem);
    const uint32_t a_base = (dyn_base + 1023u) & ~1023u;
    const uint32_t stage0 = (a_base + RegionA::STAGE0_OFF + 1023u) & ~1023u;
    const uint32_t set_bytes = (uint32_t)p.Hkv * Geo::WARP_STAGE_BYTES;
    {
        bool ok = (stage0 + set_bytes <= LUT_ABS) &&
                  (REGION_B_ABS + (ATTN_STAGES - 1) * set_bytes <= dyn_base + (uint32_t)ATTN_DYN_SMEM);
        if (!ok) {
            if (tid == 0) atomicMax(p.status, ST_SMEM_LAYOUT);
            return;
        }
    }
    const uint32_t bar0 = a_base + RegionA::BAR_OFF + (uint32_t)warp * ATTN_STAGES * 8u;
    const uint32_t norm_s = a_base + RegionA::NORM_OFF + (uint32_t)warp * 256u;  // kn[32] floats, vn[32] floats
    const uint32_t ctrl_s = a_base + RegionA::CTRL_OFF;
    const uint32_t merge_s = a_base + RegionA::MERGE_OFF;
    auto stage_addr = [&](int s) -> uint32_t {
        return (s == 0 ? stage0 : REGION_B_ABS + (uint32_t)(s - 1) * set_bytes) + (uint32_t)warp * Geo::WARP_STAGE_BYTES;
    };

    // ---- work slice ----
    const int W = gridDim.x;
    const int G = p.G;
    const long long N = p.tile_start[G];
    const long long lo = (long long)blockIdx.x * N / W;
    const long long hi = (long long)(blockIdx.x + 1) * N / W;
    if (lo >= hi) return;  // uniform for the CTA

    // ---- byte -> centroid table, one column per lane ----
    if (BITS == 4) {
        for (int idx = tid; idx < 256 * 32; idx += nthreads) {
            int v = idx >> 5, l = idx & 31;
            uint32_t val = pack_half2(kCent4[v & 15], kCent4[v >> 4]);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(LUT_ABS + (uint32_t)v * 256u + (uint32_t)l * 4u), "r"(val) : "memory");
        }
    } else {
        for (int idx = tid; idx < 256 * 32; idx += nthreads) {
            int v = idx >> 5, l = idx & 31;
            uint32_t lo2 = pack_half2(kCent2[v & 3], kCent2[(v >> 2) & 3]);
            uint32_t hi2 = pack_half2(kCent2[(v >> 4) & 3], kCent2[(v >> 6) & 3]);
            asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(LUT_ABS + (uint32_t)v * 256u + (uint32_t)l * 8u),
                         "r"(lo2), "r"(hi2) : "memory");
        }
    }
    if (lane == 0) {
        for (int s = 0; s < ATTN_STAGES; ++s) mbar_init(bar0 + 8u * s, 1);
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    __syncthreads();

    // first sequence of the slice: largest g with tile_start[g] <= lo
    int g;
    {
        int a = 0, b = G;  // invariant: tile_start[a] <= lo < tile_start[b]
        while (b - a > 1) {
            int mid = (a + b) >> 1;
            if ((long long)p.tile_start[mid] <= lo) a = mid; else b = mid;
        }
        g = a;
    }

    // ---- producer cursor (warp-uniform) ----
    long long ptile = lo;
    int pg = g;
    long long pg_end = p.tile_start[pg + 1];
    int issued = 0, consumed = 0;
    bool dead = false;  // a bounded wait gave up: keep the control flow, stop touching the pipeline
    const int xcoord = warp * Geo::BPH;

    auto issue_one = [&]() {
        while (ptile >= pg_end) {
            ++pg;
            pg_end = p.tile_start[pg + 1];
        }
        const long long local = ptile - p.tile_start[pg];
        const long long row = (p.row_base ? p.row_base[pg] : (long long)pg * p.max_seq_len) + local * TILE_TOKENS;
        const int s = issued % ATTN_STAGES;
        if (lane == 0) {
            const uint32_t bar = bar0 + 8u * s;
            const uint32_t dst = stage_addr(s);
            mbar_arrive_expect_tx(bar, Geo::WARP_STAGE_BYTES);
            tma_load_2d(dst, &tmK, bar, xcoord, (int)row);
            tma_load_2d(dst + Geo::TILE_BYTES, &tmV, bar, xcoord, (int)row);
        }
        ++issued;
        ++ptile;
    };
    for (int s = 0; s < ATTN_STAGES; ++s)
        if (ptile < hi) issue_one();

    const uint32_t lutlane = LUT_ABS | ((uint32_t)lane << (BITS == 4 ? 2 : 3));

    long long tile = lo;
    while (tile < hi) {
        // ================= one segment: tiles [tile, seg_end) of sequence g =================
        const long long ts_g = p.tile_start[g];
        const long long ts_g1 = p.tile_start[g + 1];
        const long long seg_end = hi < ts_g1 ? hi : ts_g1;
        const int pos = p.positions ? p.positions[g] : p.pos_value;
        const int L = (pos < 0 ? 0 : pos) + 1;
        const long long row0 = p.row_base ? p.row_base[g] : (long long)g * p.max_seq_len;

        // query fragments: lane (gl, t4) holds coordinates 32*t4 .. 32*t4+31 of head warp*grp + gl
        uint32_t qa[8][4];
        {
            float qv[32];
            if (gl < grp) {
                const float4* src =
                    reinterpret_cast<const float4*>(p.q_rot + ((size_t)g * p.H + (size_t)warp * grp + gl) * HEAD_DIM + 32 * t4);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float4 f = __ldg(src + i);
                    qv[4 * i] = f.x; qv[4 * i + 1] = f.y; qv[4 * i + 2] = f.z; qv[4 * i + 3] = f.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) qv[i] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                __half2 h01 = __floats2half2_rn(qv[4 * j], qv[4 * j + 1]);
                __half2 h23 = __floats2half2_rn(qv[4 * j + 2], qv[4 * j + 3]);
                float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
                qa[j][0] = *reinterpret_cast<uint32_t*>(&h01);
                qa[j][2] = *reinterpret_cast<uint32_t*>(&h23);
                qa[j][1] = pack_half2(qv[4 * j] - f01.x, qv[4 * j + 1] - f01.y);
                qa[j][3] = pack_half2(qv[4 * j + 2] - f23.x, qv[4 * j + 3] - f23.y);
            }
        }

        float m_run = -1e30f, l_run = 0.0f;
        float acc[8][4];
#pragma unroll
        for (int b = 0; b < 8; ++b) { acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.0f; }

        // norm prefetch ring: lane <-> token of the tile
        auto load_norms = [&](long long tl, float& kf, float& vf) {
            kf = 0.0f; vf = 0.0f;
            if (tl < seg_end) {
                const long long tok = (tl - ts_g) * TILE_TOKENS + lane;
                if (tok < L) {
                    const size_t off = (size_t)(row0 + tok) * p.Hkv + warp;
                    kf = __half2float(p.kn[off]);
                    vf = __half2float(p.vn[off]);
                }
            }
        };
        float kn0, vn0, kn1, vn1;
        load_norms(tile, kn0, vn0);
        load_norms(tile + 1, kn1, vn1);

        for (; tile < seg_end; ++tile) {
            const int t0 = (int)(tile - ts_g) * TILE_TOKENS;
            // stash this tile's norms, fetch the ones two tiles ahead
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(norm_s + 4u * lane), "f"(kn0) : "memory");
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(norm_s + 128u + 4u * lane), "f"(vn0) : "memory");
            kn0 = kn1; vn0 = vn1;
            load_norms(tile + 2, kn1, vn1);
            __syncwarp();

            const int s = consumed % ATTN_STAGES;
            if (!dead) {
                if (!mbar_wait_bounded(bar0 + 8u * s, (uint32_t)(consumed / ATTN_STAGES) & 1u)) {
                    dead = true;
                    if (lane == 0) atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
                }
            }
            dead = __any_sync(0xffffffffu, dead);
            if (!dead) {
                const uint32_t kt = stage_addr(s);
                const uint32_t vt = kt + Geo::TILE_BYTES;

                // ---------------- scores: 4 blocks of 8 tokens ----------------
                float sv[8];
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
                    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (BITS == 4) {
                        const uint4 kw = lds128(kt + (uint32_t)(8 * blk + gl) * 64u + (uint32_t)t4 * 16u);
                        const uint32_t w[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t word = w[j >> 1];
                            const uint32_t b0 = lds32(prmt(word, lutlane, (j & 1) ? 0x7624u : 0x7604u));
                            const uint32_t b1 = lds32(prmt(word, lutlane, (j & 1) ? 0x7634u : 0x7614u));
                            mma16816(c, qa[j][0], qa[j][1], qa[j][2], qa[j][3], b0, b1);
                        }
                    } else {
                        const uint2 kw = lds64(kt + (uint32_t)(8 * blk + gl) * 32u + (uint32_t)t4 * 8u);
                        const uint32_t w[2] = {kw.x, kw.y};
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t word = w[j >> 2];
                            const uint2 bb = lds64(prmt(word, lutlane, 0x7604u | ((uint32_t)(j & 3) << 4)));
                            mma16816(c, qa[j][0], qa[j][1], qa[j][2], qa[j][3], bb.x, bb.y);
                        }
                    }
                    float2 kn2;
                    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(kn2.x), "=f"(kn2.y)
                                 : "r"(norm_s + 4u * (uint32_t)(8 * blk + 2 * t4)));
                    sv[2 * blk] = (c[0] + c[2]) * kn2.x;
                    sv[2 * blk + 1] = (c[1] + c[3]) * kn2.y;
                }

                // ---------------- online softmax (rows = heads gl < grp) ----------------
                float tmax = -1e30f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int tok = t0 + 8 * (i >> 1) + 2 * t4 + (i & 1);
                    if (tok >= L) sv[i] = -1e30f;
                    tmax = fmaxf(tmax, sv[i]);
                }
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
                const float m_new = fmaxf(m_run, tmax);
                const bool grew = (gl < grp) && (m_new > m_run);
                if (__any_sync(0xffffffffu, grew)) {
                    const float corr = ex2_approx(m_run - m_new);  // 1 when unchanged, 0 at the first tile
                    l_run *= corr;
                    // accumulators of head (2*t4 + e) live in lanes with this t4; its corr lives in lanes gl' = 2*t4 + e
                    const float c0 = __shfl_sync(0xffffffffu, corr, (2 * t4) * 4);
                    const float c1 = __shfl_sync(0xffffffffu, corr, ((2 * t4 + 1) & 7) * 4);
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        acc[b][0] *= c0; acc[b][2] *= c0;
                        acc[b][1] *= c1; acc[b][3] *= c1;
                    }
                    m_run = m_new;
                }
                float pv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int tok = t0 + 8 * (i >> 1) + 2 * t4 + (i & 1);
                    const float e = ex2_approx(sv[i] - m_run);
                    pv[i] = (tok < L && gl < grp) ? e : 0.0f;
                    l_run += pv[i];
                }

                // ---------------- values: 2 blocks of 16 tokens ----------------
#pragma unroll
                for (int gam = 0; gam < 2; ++gam) {
                    float2 va, vb;
                    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(va.x), "=f"(va.y)
                                 : "r"(norm_s + 128u + 4u * (uint32_t)(16 * gam + 2 * t4)));
                    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(vb.x), "=f"(vb.y)
                                 : "r"(norm_s + 128u + 4u * (uint32_t)(16 * gam + 8 + 2 * t4)));
                    const uint32_t pb0 = pack_half2(pv[4 * gam] * va.x, pv[4 * gam + 1] * va.y);
                    const uint32_t pb1 = pack_half2(pv[4 * gam + 2] * vb.x, pv[4 * gam + 3] * vb.y);
                    const uint32_t rowA = (uint32_t)(16 * gam + 2 * t4);
                    if (BITS == 4) {
                        const uint2 xa = lds64(vt + (rowA + 0) * 64u + (uint32_t)gl * 8u);
                        const uint2 xb = lds64(vt + (rowA + 1) * 64u + (uint32_t)gl * 8u);
                        const uint2 xc = lds64(vt + (rowA + 8) * 64u + (uint32_t)gl * 8u);
                        const uint2 xd = lds64(vt + (rowA + 9) * 64u + (uint32_t)gl * 8u);
#pragma unroll
                        for (int b = 0; b < 8; ++b) {
                            const uint32_t sel = 0x7604u | ((uint32_t)(b & 3) << 4);
                            const uint32_t la = lds32(prmt(b < 4 ? xa.x : xa.y, lutlane, sel));
                            const uint32_t lb = lds32(prmt(b < 4 ? xb.x : xb.y, lutlane, sel));
                            const uint32_t lc = lds32(prmt(b < 4 ? xc.x : xc.y, lutlane, sel));
                            const uint32_t ld = lds32(prmt(b < 4 ? xd.x : xd.y, lutlane, sel));
                            mma16816(acc[b], prmt(la, lb, 0x5410u), prmt(la, lb, 0x7632u), prmt(lc, ld, 0x5410u),
                                     prmt(lc, ld, 0x7632u), pb0, pb1);
                        }
                    } else {
                        const uint32_t xa = lds32(vt + (rowA + 0) * 32u + (uint32_t)gl * 4u);
                        const uint32_t xb = lds32(vt + (rowA + 1) * 32u + (uint32_t)gl * 4u);
                        const uint32_t xc = lds32(vt + (rowA + 8) * 32u + (uint32_t)gl * 4u);
                        const uint32_t xd = lds32(vt + (rowA + 9) * 32u + (uint32_t)gl * 4u);
#pragma unroll
                        for (int bb = 0; bb < 4; ++bb) {
                            const uint32_t sel = 0x7604u | ((uint32_t)bb << 4);
                            const uint2 la = lds64(prmt(xa, lutlane, sel));
                            const uint2 lb = lds64(prmt(xb, lutlane, sel));
                            const uint2 lc = lds64(prmt(xc, lutlane, sel));
                            const uint2 ld = lds64(prmt(xd, lutlane, sel));
                            mma16816(acc[2 * bb], prmt(la.x, lb.x, 0x5410u), prmt(la.x, lb.x, 0x7632u),
                                     prmt(lc.x, ld.x, 0x5410u), prmt(lc.x, ld.x, 0x7632u), pb0, pb1);
                            mma16816(acc[2 * bb + 1], prmt(la.y, lb.y, 0x5410u), prmt(la.y, lb.y, 0x7632u),
                                     prmt(lc.y, ld.y, 0x5410u), prmt(lc.y, ld.y, 0x7632u), pb0, pb1);
                        }
                    }
                }
            }
            __syncwarp();
            ++consumed;
            if (!dead && ptile < hi) issue_one();
        }

        // ================= end of segment: publish the partial, maybe merge =================
        const int slot = blockIdx.x + g;
        {
            float lsum = l_run;
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
            if (gl < grp && t4 == 0) {
                float* dst = p.partials + ((size_t)slot * p.H + (size_t)warp * grp + gl) * PART_STRIDE;
                dst[HEAD_DIM] = m_run;
                dst[HEAD_DIM + 1] = lsum;
            }
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int hq = 2 * t4 + e;
                if (hq < grp) {
                    float* dst = p.partials + ((size_t)slot * p.H + (size_t)warp * grp + hq) * PART_STRIDE + 16 * gl;
#pragma unroll
                    for (int b2 = 0; b2 < 4; ++b2) {
                        float4 o;
                        o.x = acc[2 * b2][e]; o.y = acc[2 * b2][2 + e];
                        o.z = acc[2 * b2 + 1][e]; o.w = acc[2 * b2 + 1][2 + e];
                        *reinterpret_cast<float4*>(dst + 4 * b2) = o;
                    }
                }
            }
        }
        __threadfence();
        __syncthreads();
        // number of CTAs that hold a part of sequence g
        const int first_w = (int)(((ts_g + 1) * W - 1) / N);
        const int last_w = (int)((ts_g1 * W - 1) / N);
        if (tid == 0) {
            const int parts = last_w - first_w + 1;
            const int old = atomicAdd(p.tickets + g, 1);
            const uint32_t flag = (old == parts - 1) ? 1u : 0u;
            if (flag) p.tickets[g] = 0;  // everybody has arrived: leave the ticket ready for the next launch
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(ctrl_s), "r"(flag) : "memory");
        }
        __syncthreads();
        uint32_t is_last;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(is_last) : "r"(ctrl_s) : "memory");
        if (is_last) {
            __threadfence();
            const int H = p.H;
            const int Hp = (H + 7) & ~7;
            // phase A: combine the parts, normalise -> merge[k][head]
            for (int idx = tid; idx < H * HEAD_DIM; idx += nthreads) {
                const int hq = idx >> 7, k = idx & 127;
                float M = -1e30f;
                for (int wk = first_w; wk <= last_w; ++wk)
                    M = fmaxf(M, __ldcg(p.partials + ((size_t)(wk + g) * H + hq) * PART_STRIDE + HEAD_DIM));
                float Z = 0.0f, a = 0.0f;
                for (int wk = first_w; wk <= last_w; ++wk) {
                    const float* src = p.partials + ((size_t)(wk + g) * H + hq) * PART_STRIDE;
                    const float wgt = ex2_approx(__ldcg(src + HEAD_DIM) - M);
                    Z += __ldcg(src + HEAD_DIM + 1) * wgt;
                    a += __ldcg(src + k) * wgt;
                }
                const float val = a / (Z + 1e-8f);
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(merge_s + 4u * (uint32_t)(k * Hp + hq)), "f"(val) : "memory");
            }
            __syncthreads();
            // phase B: out[head][d] = sum_k R[k][d] * merge[k][head]
            const int d = tid & 127;
            const int part = tid >> 7, nparts = nthreads >> 7;
            for (int h0 = part * 8; h0 < H; h0 += nparts * 8) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = 0.0f;
#pragma unroll 4
                for (int k = 0; k < HEAD_DIM; ++k) {
                    const float r = __half2float(__ldg(p.rotation + k * HEAD_DIM + d));
                    const uint4 u0 = lds128(merge_s + 4u * (uint32_t)(k * Hp + h0));
                    const uint4 u1 = lds128(merge_s + 4u * (uint32_t)(k * Hp + h0 + 4));
                    o[0] = fmaf(r, __uint_as_float(u0.x), o[0]); o[1] = fmaf(r, __uint_as_float(u0.y), o[1]);
                    o[2] = fmaf(r, __uint_as_float(u0.z), o[2]); o[3] = fmaf(r, __uint_as_float(u0.w), o[3]);
                    o[4] = fmaf(r, __uint_as_float(u1.x), o[4]); o[5] = fmaf(r, __uint_as_float(u1.y), o[5]);
                    o[6] = fmaf(r, __uint_as_float(u1.z), o[6]); o[7] = fmaf(r, __uint_as_float(u1.w), o[7]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (h0 + i < H) p.out[(size_t)g * p.q_dim + (size_t)(h0 + i) * HEAD_DIM + d] = __float2half_rn(o[i]);
            }
            __syncthreads();
        }
        ++g;
    }

    // A warp that gave up on a wait may still have copies in flight: give them a bounded chance to land
    // before the CTA (and its shared memory) goes away.
    if (dead) {
        for (int n = consumed; n < issued; ++n)
            mbar_wait_bounded(bar0 + 8u * (n % ATTN_STAGES), (uint32_t)(n / ATTN_STAGES) & 1u, 1u << 16);
    }
}

}  // namespace tq
