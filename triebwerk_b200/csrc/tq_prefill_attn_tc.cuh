// Causal prefill attention on the 5th-generation tensor cores (tcgen05 + tensor memory), sm_100a.
//
// The same job as prefill_attention_kernel (tq_prefill_attn.cuh; reference engine/kernels.cu:1874-1960 and :1071-1158):
// query token t of a prompt attends to cache rows 0 .. t.  Here the products run as tcgen05.mma with the operands read
// from shared memory by the tensor core itself and the accumulators in tensor memory, so no warp spends its
// shared-memory bandwidth on ldmatrix:
//   * one CTA = 128 score rows (128 / GRP query tokens x the GRP query heads of one KV head) = the M dimension, 256 threads;
//   * warps 0-3 ("row threads": thread r owns score row r = TMEM lane r) do the softmax and keep the output row in
//     registers; warps 4-7 dequantise the cache tiles: K as [64 tokens][128 coordinates] (the B operand of S = Q . K^T) and
//     V TRANSPOSED as [128 coordinates][64 tokens] (the B operand of O += P . V), both fp16 in the canonical K-major
//     128-byte-swizzled layout, double buffered and handed over through mbarriers;
//   * per 64-row tile: S (128 x 64, fp32) -> tensor memory -> registers; K norm, causal limit, online softmax; P (times the
//     V norm, fp16) -> shared memory as an A operand; P . V -> tensor memory -> added to the output row in registers;
//   * packed forms: the query rotation (Q . R^T) at the start and the way back (O . R, with O split into fp16 high and low
//     parts) at the end are tcgen05 products as well.
// Every wait on a barrier is bounded; a wait that runs out raises the status word and the kernel runs to its end.
#pragma once

#include "tq_prefill_attn.cuh"
#include "tq_prefill_tc.cuh"

namespace tq {

constexpr int PTC_THREADS = 256;
constexpr int PTC_KT = 64;  // cache rows per tile

struct PtcSmem {
    static constexpr uint32_t Q = 0;            // A operand [2 regions][128 rows][128 B]; at the end: high parts of the results
    static constexpr uint32_t K = 32768;        // 2 buffers x [2 regions][64 rows][128 B]; at the start: R; at the end: low parts
    static constexpr uint32_t V = 65536;        // 2 buffers x [128 coordinate rows][128 B = 64 tokens]; at the end: R^T
    static constexpr uint32_t P = 98304;        // A operand [128 rows][128 B = 64 tokens]
    static constexpr uint32_t NORM = 114688;    // [2 buffers][K, V][64] halves
    static constexpr uint32_t CTRL = NORM + 512;  // mbarriers: mma, ready[2], free[2]; tensor-memory base
    static constexpr uint32_t LUT = CTRL + 128;   // 4-bit: [256][32 lanes] half2
    static constexpr uint32_t BYTES = LUT + 32768;
};
constexpr size_t PTC_DYN_SMEM = PtcSmem::BYTES + 1024;  // + alignment slack

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// fp16 x fp16 -> fp32, both operands K-major, M = 128
constexpr uint32_t PTC_IDESC_N64 = (1u << 4) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t PTC_IDESC_N128 = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

// byte offset of the 16-byte chunk `ch` (8 halves; 0 .. 15 for a 128-element row) of row `row` in an operand tile whose
// 64-element regions lie `region_bytes` apart
__device__ __forceinline__ uint32_t ptc_chunk(uint32_t region_bytes, int row, int ch) {
    return (uint32_t)(ch >> 3) * region_bytes + (uint32_t)row * 128u + (uint32_t)(((ch & 7) ^ (row & 7)) << 4);
}

template <int BITS>
__global__ void __launch_bounds__(PTC_THREADS, 1) prefill_attention_tc_kernel(const PrefillAttnParams p) {
    static_assert(BITS == 4 || BITS == 0, "forms built on tcgen05: the 4-bit cache and the fp16 cache");
    extern __shared__ __align__(1024) uint8_t ptc_smem[];
    const uint32_t sb = (smem_u32(ptc_smem) + 1023u) & ~1023u;
    uint8_t* gb = ptc_smem + (sb - smem_u32(ptc_smem));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool is_row = tid < 128;
    const int gs = p.grp_shift, GRP = 1 << gs, QT = PFA_ROWS >> gs;
    const int qb = (int)gridDim.y - 1 - (int)blockIdx.y;  // the longest causal prefixes of all heads and prompts first
    const int seq = (int)blockIdx.x / p.Hkv;
    const int kvh = (int)blockIdx.x - seq * p.Hkv;
    const int q0 = qb * QT;
    const int q_last = min(q0 + QT, p.T) - 1;
    const int n_tiles = q_last / PTC_KT + 1;
    constexpr int ROW_BYTES = BITS == 4 ? 64 : 256;  // bytes of one head in a cache row
    const size_t row_stride = (size_t)p.Hkv * ROW_BYTES;
    const long long seq_row0 = p.row_base ? p.row_base[seq] : (long long)seq * p.seq_rows;
    const __half* const q_seq = p.q + (size_t)seq * (size_t)p.T * (size_t)p.q_tok_stride;
    __half* const out_seq = p.out + (size_t)seq * (size_t)p.T * (size_t)p.q_dim;
    const uint8_t* const ck_seq = p.ck + (size_t)seq_row0 * row_stride + (size_t)kvh * ROW_BYTES;
    const uint8_t* const cv_seq = p.cv + (size_t)seq_row0 * row_stride + (size_t)kvh * ROW_BYTES;
    const __half* const kn_seq = BITS != 0 ? p.kn + (size_t)seq_row0 * p.Hkv + kvh : nullptr;
    const __half* const vn_seq = BITS != 0 ? p.vn + (size_t)seq_row0 * p.Hkv + kvh : nullptr;

    const uint32_t bar_mma = sb + PtcSmem::CTRL;
    const uint32_t bar_ready0 = sb + PtcSmem::CTRL + 8u, bar_free0 = sb + PtcSmem::CTRL + 24u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gb + PtcSmem::CTRL + 64);
    bool dead = false;
    auto give_up = [&]() {
        dead = true;
        if (p.status) atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
    };

    // ---- once: tensor memory, barriers, table, this block's queries, R ----
    if (warp == 0) {
        tmem_alloc(sb + PtcSmem::CTRL + 64u, 512u);  // [0, 128): rotation products; [128, 192): S; [256, 384): P . V of a tile
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(bar_mma, 1);
        mbar_init(bar_ready0, 128);
        mbar_init(bar_ready0 + 8u, 128);
        mbar_init(bar_free0, 128);
        mbar_init(bar_free0 + 8u, 128);
        fence_mbar_init();
    }
    if (BITS == 4) {
        for (int i = tid; i < 256 * 32; i += PTC_THREADS) {
            const int e = i >> 5;
            reinterpret_cast<uint32_t*>(gb + PtcSmem::LUT)[i] = pack_half2(kCent4[e & 15], kCent4[e >> 4]);
        }
    }
    const uint32_t lut = sb + PtcSmem::LUT + 4u * (uint32_t)lane;
    const int my_tok = q0 + (tid >> gs), my_head = kvh * GRP + (tid & (GRP - 1));  // row threads: the score row's query
    if (is_row) {
        const uint4* src = reinterpret_cast<const uint4*>(q_seq + (size_t)my_tok * p.q_tok_stride + (size_t)my_head * HEAD_DIM);
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) {
            const uint4 u = my_tok < p.T ? __ldg(src + ch) : make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(gb + PtcSmem::Q + ptc_chunk(16384u, tid, ch)) = u;
        }
    }
    if (BITS != 0) {  // R [d][k] as a B operand (rows = output coordinate d) over the K buffers
        for (int i = tid; i < 128 * 16; i += PTC_THREADS) {
            const int row = i >> 4, ch = i & 15;
            *reinterpret_cast<uint4*>(gb + PtcSmem::K + ptc_chunk(16384u, row, ch)) =
                __ldg(reinterpret_cast<const uint4*>(p.rotation + (size_t)row * HEAD_DIM) + ch);
        }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t my_lanes = tmem + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's quarter of the tensor-memory lanes
    uint32_t mph = 0;  // phase of bar_mma (row threads)

    auto wait_mma = [&]() {
        if (!dead && !mbar_wait_bounded(bar_mma, mph, 1u << 22)) give_up();
        mph ^= 1u;
        tc_fence_after();
    };

    if (BITS != 0) {
        // ---- q_rot = Q . R^T (reference engine/kernels.cu:1896-1903), scaled by log2(e) / sqrt(128), back into the Q tile ----
        if (tid == 0) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t koff = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                umma_f16(tmem, umma_desc_sw128(sb + PtcSmem::Q + koff), umma_desc_sw128(sb + PtcSmem::K + koff), PTC_IDESC_N128, ks != 0);
            }
            umma_commit(bar_mma);
        }
        if (is_row) {
            wait_mma();
#pragma unroll 1
            for (int c4 = 0; c4 < 4; ++c4) {
                uint32_t r[32];
                tmem_ld32(my_lanes + 32u * c4, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 u;
                    const float sc = 0.12751743074602467f;
                    u.x = pack_half2(__uint_as_float(r[8 * i]) * sc, __uint_as_float(r[8 * i + 1]) * sc);
                    u.y = pack_half2(__uint_as_float(r[8 * i + 2]) * sc, __uint_as_float(r[8 * i + 3]) * sc);
                    u.z = pack_half2(__uint_as_float(r[8 * i + 4]) * sc, __uint_as_float(r[8 * i + 5]) * sc);
                    u.w = pack_half2(__uint_as_float(r[8 * i + 6]) * sc, __uint_as_float(r[8 * i + 7]) * sc);
                    *reinterpret_cast<uint4*>(gb + PtcSmem::Q + ptc_chunk(16384u, tid, 4 * c4 + i)) = u;
                }
            }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        __syncthreads();  // the rotated queries are in place and R has been consumed: the K buffers may take tiles
        tc_fence_after();
    }

    float o[128];
    float m_run = -1e30f, l_run = 0.0f;
#pragma unroll
    for (int i = 0; i < 128; ++i) o[i] = 0.0f;

    if (!is_row) {
        // ================= producers: tile j into buffer j & 1 =================
        const int pt = tid - 128;
        const int ktr = pt & 63, kc = pt >> 6;  // K: token row of the tile, half of its 128 coordinates
        const int vcp = pt & 63, vth = pt >> 6;  // V: coordinate pair (2 vcp, 2 vcp + 1), half of the tile's 64 tokens
        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            if (j >= 2 && !dead && !mbar_wait_bounded(bar_free0 + 8u * b, (uint32_t)(((j >> 1) - 1) & 1), 1u << 22)) give_up();
            const int row0 = j * PTC_KT;
            uint8_t* kt = gb + PtcSmem::K + (uint32_t)b * 16384u;
            uint8_t* vt = gb + PtcSmem::V + (uint32_t)b * 16384u;
            {   // K tile: row ktr, chunks 8 kc .. 8 kc + 7
                const int row = min(row0 + ktr, p.rows - 1);
                const bool blank = BITS == 0 && row0 + ktr >= p.T;  // fp16 rows past the prompt may hold anything
                if (BITS == 4) {
                    const uint4* src = reinterpret_cast<const uint4*>(ck_seq + (size_t)row * row_stride + 32 * kc);
                    const uint4 w0 = __ldg(src), w1 = __ldg(src + 1);
                    const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        uint4 u;
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.x) : "r"(lut + ((w[i] & 0xffu) << 7)));
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.y) : "r"(lut + (((w[i] >> 8) & 0xffu) << 7)));
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.z) : "r"(lut + (((w[i] >> 16) & 0xffu) << 7)));
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.w) : "r"(lut + ((w[i] >> 24) << 7)));
                        *reinterpret_cast<uint4*>(kt + ptc_chunk(8192u, ktr, 8 * kc + i)) = u;
                    }
                } else {
                    const uint4* src = reinterpret_cast<const uint4*>(ck_seq + (size_t)row * row_stride + 128 * kc);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint4 u = blank ? make_uint4(0u, 0u, 0u, 0u) : __ldg(src + i);
                        *reinterpret_cast<uint4*>(kt + ptc_chunk(8192u, ktr, 8 * kc + i)) = u;
                    }
                }
            }
            {   // V tile, transposed: coordinates 2 vcp and 2 vcp + 1 of the tokens 32 vth .. 32 vth + 31
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint32_t x[8];  // (coordinate 2 vcp, coordinate 2 vcp + 1) of 8 consecutive tokens
#pragma unroll
                    for (int u8 = 0; u8 < 8; ++u8) {
                        const int t = 32 * vth + 8 * g + u8;
                        const int row = min(row0 + t, p.rows - 1);
                        if (BITS == 4) {
                            const uint32_t code = __ldg(cv_seq + (size_t)row * row_stride + vcp);
                            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x[u8]) : "r"(lut + (code << 7)));
                        } else {
                            x[u8] = row0 + t >= p.T ? 0u : __ldg(reinterpret_cast<const uint32_t*>(cv_seq + (size_t)row * row_stride) + vcp);
                        }
                    }
                    uint4 lo, hi;  // row 2 vcp: the low halves; row 2 vcp + 1: the high halves
                    lo.x = prmt(x[0], x[1], 0x5410u); lo.y = prmt(x[2], x[3], 0x5410u);
                    lo.z = prmt(x[4], x[5], 0x5410u); lo.w = prmt(x[6], x[7], 0x5410u);
                    hi.x = prmt(x[0], x[1], 0x7632u); hi.y = prmt(x[2], x[3], 0x7632u);
                    hi.z = prmt(x[4], x[5], 0x7632u); hi.w = prmt(x[6], x[7], 0x7632u);
                    const int ch = 4 * vth + g;  // 8 tokens = one 16-byte chunk of the 64-token row
                    *reinterpret_cast<uint4*>(vt + ptc_chunk(0u, 2 * vcp, ch)) = lo;
                    *reinterpret_cast<uint4*>(vt + ptc_chunk(0u, 2 * vcp + 1, ch)) = hi;
                }
            }
            if (BITS != 0) {
                const int row = min(row0 + (pt & 63), p.rows - 1);
                reinterpret_cast<__half*>(gb + PtcSmem::NORM)[b * 128 + pt] = (pt < 64 ? kn_seq : vn_seq)[(size_t)row * p.Hkv];
            }
            fence_proxy_async_smem();  // generic-proxy writes of the operands before the tensor core reads them
            mbar_arrive(bar_ready0 + 8u * b);
        }
    } else {
        // ================= row threads =================
        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            if (!dead && !mbar_wait_bounded(bar_ready0 + 8u * b, (uint32_t)((j >> 1) & 1), 1u << 22)) give_up();
            tc_fence_after();
            if (tid == 0 && !dead) {  // S = Q . K^T: 128 x 64, 8 steps of 16 coordinates
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t ka = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                    const uint32_t kb = (uint32_t)(ks >> 2) * 8192u + (uint32_t)(ks & 3) * 32u;
                    umma_f16(tmem + 128u, umma_desc_sw128(sb + PtcSmem::Q + ka),
                             umma_desc_sw128(sb + PtcSmem::K + (uint32_t)b * 16384u + kb), PTC_IDESC_N64, ks != 0);
                }
                umma_commit(bar_mma);
            }
            wait_mma();
            uint32_t sr[64];
            tmem_ld32(my_lanes + 128u, reinterpret_cast<uint32_t(&)[32]>(sr[0]));
            tmem_ld32(my_lanes + 160u, reinterpret_cast<uint32_t(&)[32]>(sr[32]));
            tmem_ld_wait();
            // ---- K norm, causal limit, online softmax; P (times the V norm) as fp16 into the A operand tile ----
            const bool diagonal = j * PTC_KT + PTC_KT - 1 > q0;
            const uint4* nrm = reinterpret_cast<const uint4*>(gb + PtcSmem::NORM + (uint32_t)b * 256u);
            float mx = -1e30f;
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                float kn8[8];
                if (BITS != 0) {
                    const uint4 u = nrm[c8];  // (every thread reads the same words: a broadcast)
                    const __half2* h2 = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(h2[e]);
                        kn8[2 * e] = f.x;
                        kn8[2 * e + 1] = f.y;
                    }
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int c = 8 * c8 + e;
                    float s = __uint_as_float(sr[c]) * (BITS != 0 ? kn8[e] : p.score_scale);
                    if (diagonal && j * PTC_KT + c > my_tok) s = -1e30f;
                    sr[c] = __float_as_uint(s);
                    mx = fmaxf(mx, s);
                }
            }
            const float mn = fmaxf(m_run, mx);
            const float corr = ex2_approx(m_run - mn);
            m_run = mn;
            float lsum = 0.0f;
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                float vn8[8];
                if (BITS != 0) {
                    const uint4 u = nrm[8 + c8];
                    const __half2* h2 = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(h2[e]);
                        vn8[2 * e] = f.x;
                        vn8[2 * e + 1] = f.y;
                    }
                }
                float pv[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float s = __uint_as_float(sr[8 * c8 + e]);
                    const float pe = s <= -1e30f ? 0.0f : ex2_approx(s - mn);
                    lsum += pe;
                    // (rows past the prompt can hold anything, a norm that is not a number included: select, do not multiply)
                    pv[e] = pe == 0.0f ? 0.0f : (BITS != 0 ? pe * vn8[e] : pe);
                }
                uint4 u;
                u.x = pack_half2(pv[0], pv[1]); u.y = pack_half2(pv[2], pv[3]);
                u.z = pack_half2(pv[4], pv[5]); u.w = pack_half2(pv[6], pv[7]);
                *reinterpret_cast<uint4*>(gb + PtcSmem::P + ptc_chunk(0u, tid, c8)) = u;
            }
            l_run = l_run * corr + lsum;
            fence_proxy_async_smem();
            tc_fence_before();
            named_barrier(2, 128);  // every row's P is written; every row has taken its S out of tensor memory
            if (tid == 0 && !dead) {  // O_tile = P . V: 128 x 128, 4 steps of 16 tokens
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma_f16(tmem + 256u, umma_desc_sw128(sb + PtcSmem::P + 32u * ks),
                             umma_desc_sw128(sb + PtcSmem::V + (uint32_t)b * 16384u + 32u * ks), PTC_IDESC_N128, ks != 0);
                umma_commit(bar_mma);
            }
#pragma unroll
            for (int i = 0; i < 128; ++i) o[i] *= corr;  // (while the product runs)
            wait_mma();
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                uint32_t r[32];
                tmem_ld32(my_lanes + 256u + 32u * c4, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[32 * c4 + i] += __uint_as_float(r[i]);
            }
            tc_fence_before();
            mbar_arrive(bar_free0 + 8u * b);  // the products that read buffer b (and the P tile) have completed
        }
    }

    // ================= results =================
    const float inv = 1.0f / (l_run + 1e-8f);
    __half* const dst = out_seq + (size_t)my_tok * p.q_dim + (size_t)my_head * HEAD_DIM;
    if (BITS == 0) {
        if (is_row && my_tok < p.T) {
#pragma unroll
            for (int ch = 0; ch < 16; ++ch) {
                uint4 u;
                u.x = pack_half2(o[8 * ch] * inv, o[8 * ch + 1] * inv); u.y = pack_half2(o[8 * ch + 2] * inv, o[8 * ch + 3] * inv);
                u.z = pack_half2(o[8 * ch + 4] * inv, o[8 * ch + 5] * inv); u.w = pack_half2(o[8 * ch + 6] * inv, o[8 * ch + 7] * inv);
                *reinterpret_cast<uint4*>(dst + 8 * ch) = u;
            }
        }
    } else {
        // out[d] = sum_k R[k][d] * acc[k] (reference engine/kernels.cu:1957): the normalised rows, split into fp16 high and low
        // parts, times R^T [d][k] (the B operand's rows are the output coordinates)
        __syncthreads();  // every product of the tile loop has completed (each row thread waited for the last one)
        if (is_row) {
#pragma unroll
            for (int ch = 0; ch < 16; ++ch) {
                uint4 uh, ul;
                uint32_t* ph = &uh.x;
                uint32_t* pl = &ul.x;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float x0 = o[8 * ch + 2 * e] * inv, x1 = o[8 * ch + 2 * e + 1] * inv;
                    const __half2 h = __floats2half2_rn(x0, x1);
                    const float2 f = __half22float2(h);
                    ph[e] = *reinterpret_cast<const uint32_t*>(&h);
                    pl[e] = pack_half2(x0 - f.x, x1 - f.y);
                }
                *reinterpret_cast<uint4*>(gb + PtcSmem::Q + ptc_chunk(16384u, tid, ch)) = uh;
                *reinterpret_cast<uint4*>(gb + PtcSmem::K + ptc_chunk(16384u, tid, ch)) = ul;
            }
        }
        for (int i = tid; i < 128 * 16; i += PTC_THREADS) {
            const int row = i >> 4, ch = i & 15;
            *reinterpret_cast<uint4*>(gb + PtcSmem::V + ptc_chunk(16384u, row, ch)) =
                __ldg(reinterpret_cast<const uint4*>(p.rotation_t + (size_t)row * HEAD_DIM) + ch);
        }
        fence_proxy_async_smem();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        if (tid == 0 && !dead) {
#pragma unroll
            for (int part = 0; part < 2; ++part) {
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t koff = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                    umma_f16(tmem, umma_desc_sw128(sb + (part ? PtcSmem::K : PtcSmem::Q) + koff), umma_desc_sw128(sb + PtcSmem::V + koff),
                             PTC_IDESC_N128, (part | ks) != 0);
                }
            }
            umma_commit(bar_mma);
        }
        if (is_row) {
            wait_mma();
#pragma unroll 1
            for (int c4 = 0; c4 < 4; ++c4) {
                uint32_t r[32];
                tmem_ld32(my_lanes + 32u * c4, r);
                tmem_ld_wait();
                if (my_tok < p.T) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 u;
                        u.x = pack_half2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]));
                        u.y = pack_half2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                        u.z = pack_half2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                        u.w = pack_half2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                        *reinterpret_cast<uint4*>(dst + 32 * c4 + 8 * i) = u;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512u);
}

}  // namespace tq
