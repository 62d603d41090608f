// Causal prefill attention over the cache of ONE sequence with the query tokens in the M dimension, sm_100a.
//
// Replaces turbo_gqa_prefill_attention_kernel (reference engine/kernels.cu:1874-1960, packed cache) and
// gqa_prefill_attention_kernel (engine/kernels.cu:1071-1158, fp16 cache): query token t attends to cache rows 0 .. t.
// The reference runs one CTA per (head, query token), reads every cache row once per query token and keeps a
// [T][heads][T] score array in global memory.  Here one CTA owns 128 score rows = (128 / GRP) consecutive query tokens x
// the GRP query heads of ONE KV head and walks the cache in tiles of 64 rows:
//   * a tile's codes are dequantised ONCE per CTA into an fp16 tile in shared memory (byte -> centroid pair through a
//     table with a private column per lane; the fp16 cache is copied as it is), 128-byte-chunk swizzled;
//   * S = Q . K^T on the tensor cores (mma.sync m16n8k16): each warp holds 16 query rows as A fragments for the whole
//     launch, the B fragments come from the K tile by ldmatrix; the K norm multiplies the score column, the causal limit
//     masks it, the softmax runs online in registers (base 2, the scale folded into the queries);
//   * O += P . V with P taken from the score accumulators as the A operand (times the V norm) and the V tile through
//     ldmatrix.trans; O stays in registers (16 rows x 128 coordinates per warp);
//   * the next tile is fetched into registers before the arithmetic of the current one and dequantised into the other
//     half of the double buffer after it: one barrier per tile.
// Packed form: each warp first rotates its 16 query rows (one tensor-core product against R in the still idle tile
// buffers, scaled by log2(e) / sqrt(128)), and at the end normalises its 16 result rows and multiplies them by R^T with
// one more product (fp16 high + low parts against R copied into the buffers again).  fp16 form: the result is
// normalised and stored.  One launch, no O(T^2) scratch, no workspace.
#pragma once

#include "tq_common.cuh"

namespace tq {

constexpr int PFA_THREADS = 256;   // 8 warps x 16 score rows
constexpr int PFA_ROWS = 128;      // score rows per CTA
constexpr int PFA_KT = 64;         // cache rows per tile

struct PfaSmem {
    static constexpr uint32_t K = 0;             // [2][64 rows][256 B]
    static constexpr uint32_t V = 32768;         // [2][64 rows][256 B]
    static constexpr uint32_t NORMS = 65536;     // [2 buffers][K, V][64] halves
    static constexpr uint32_t LUT = 66048;       // 4-bit: [256][32 lanes] half2; 2-bit: [16][32 lanes] half2
    static constexpr uint32_t BYTES = LUT + 32768;
};

struct PrefillAttnParams {
    const __half* q;          // queries [T][q_dim] as the model makes them
    long long q_tok_stride;   // halves between the queries of consecutive tokens
    const uint8_t* ck;        // packed codes [rows][kvp], or fp16 rows [rows][Hkv * 128]
    const uint8_t* cv;
    const __half* kn;         // [rows][Hkv] (packed forms)
    const __half* vn;
    const __half* rotation;   // packed forms: R row-major [128][128] (the way back out of the rotated space)
    const __half* rotation_t; // tcgen05 form, packed: R^T row-major [128][128] (null: the mma.sync form is used)
    int* status;              // optional device status word (a bounded wait that gave up raises it)
    __half* out;              // [T][q_dim]
    int q_dim;
    int T;                    // query tokens = cache rows in use
    int rows;                 // cache rows that exist (loads are clamped to them)
    int H, Hkv, grp_shift;    // GRP = 1 << grp_shift query heads per KV head
    // Several prompts of the same length in one launch (grid.x = Hkv * n_seq): prompt i reads its queries and writes its
    // results T * q_tok_stride halves behind prompt i - 1's, and its cache rows start at row_base[i] (or i * seq_rows).
    int n_seq;
    long long seq_rows;
    const long long* row_base;
    float score_scale;        // fp16 form: log2(e) / sqrt(128); packed forms: 1 (the rotated queries carry it)
};

template <int BITS>
__global__ void __launch_bounds__(PFA_THREADS, 1) prefill_attention_kernel(const PrefillAttnParams p) {
    extern __shared__ __align__(1024) uint8_t pfa_smem[];
    const uint32_t sb = smem_u32(pfa_smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gl = lane >> 2, t4 = lane & 3;
    const int gs = p.grp_shift, GRP = 1 << gs, QT = PFA_ROWS >> gs;
    const int qb = (int)gridDim.y - 1 - (int)blockIdx.y;  // the blocks with the longest prefixes start first, of all heads
    const int seq = (int)blockIdx.x / p.Hkv;               // and prompts
    const int kvh = (int)blockIdx.x - seq * p.Hkv;
    const int q0 = qb * QT;
    const int q_last = min(q0 + QT, p.T) - 1;
    const int n_tiles = q_last / PFA_KT + 1;
    constexpr int ROW_BYTES = BITS == 4 ? 64 : BITS == 2 ? 32 : 256;  // bytes of one head in a cache row
    const size_t row_stride = (size_t)p.Hkv * ROW_BYTES;
    const long long seq_row0 = p.row_base ? p.row_base[seq] : (long long)seq * p.seq_rows;
    const __half* const q_seq = p.q + (size_t)seq * (size_t)p.T * (size_t)p.q_tok_stride;
    __half* const out_seq = p.out + (size_t)seq * (size_t)p.T * (size_t)p.q_dim;
    const uint8_t* const ck_seq = p.ck + (size_t)seq_row0 * row_stride;
    const uint8_t* const cv_seq = p.cv + (size_t)seq_row0 * row_stride;
    const __half* const kn_seq = BITS != 0 ? p.kn + (size_t)seq_row0 * p.Hkv : nullptr;
    const __half* const vn_seq = BITS != 0 ? p.vn + (size_t)seq_row0 * p.Hkv : nullptr;

    // ---- byte (4-bit) or nibble (2-bit) -> two fp16 centroids, one column per lane: no bank conflicts ----
    if (BITS == 4) {
        for (int i = tid; i < 256 * 32; i += PFA_THREADS) {
            const int e = i >> 5;
            reinterpret_cast<uint32_t*>(pfa_smem + PfaSmem::LUT)[i] = pack_half2(kCent4[e & 15], kCent4[e >> 4]);
        }
    } else if (BITS == 2) {
        for (int i = tid; i < 16 * 32; i += PFA_THREADS) {
            const int e = i >> 5;
            reinterpret_cast<uint32_t*>(pfa_smem + PfaSmem::LUT)[i] = pack_half2(kCent2[e & 3], kCent2[e >> 2]);
        }
    }
    const uint32_t lut = sb + PfaSmem::LUT + 4u * (uint32_t)lane;

    // ---- this warp's 16 query rows as A fragments: rows gl and gl + 8, 8 steps of 16 coordinates ----
    uint32_t qa[8][4];
    {
        const int r_lo = 16 * warp + gl, r_hi = r_lo + 8;
        const int tok_lo = q0 + (r_lo >> gs), tok_hi = q0 + (r_hi >> gs);
        const __half* ql = q_seq + (size_t)tok_lo * p.q_tok_stride + (size_t)(kvh * GRP + (r_lo & (GRP - 1))) * HEAD_DIM + 2 * t4;
        const __half* qh = q_seq + (size_t)tok_hi * p.q_tok_stride + (size_t)(kvh * GRP + (r_hi & (GRP - 1))) * HEAD_DIM + 2 * t4;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qa[ks][0] = tok_lo < p.T ? __ldg(reinterpret_cast<const uint32_t*>(ql + 16 * ks)) : 0u;
            qa[ks][1] = tok_hi < p.T ? __ldg(reinterpret_cast<const uint32_t*>(qh + 16 * ks)) : 0u;
            qa[ks][2] = tok_lo < p.T ? __ldg(reinterpret_cast<const uint32_t*>(ql + 16 * ks + 8)) : 0u;
            qa[ks][3] = tok_hi < p.T ? __ldg(reinterpret_cast<const uint32_t*>(qh + 16 * ks + 8)) : 0u;
        }
    }
    const int tq_lo = q0 + ((16 * warp + gl) >> gs), tq_hi = q0 + ((16 * warp + gl + 8) >> gs);

    // ---- tile fetch and dequantisation: thread (row tr of the tile, c) owns the 16-byte chunks c, c + 4, c + 8, c + 12
    //      of the row's 256 fp16 bytes; the two rows of a quarter warp lie 4 apart, so their swizzled chunks never share
    //      a bank group ----
    const int tr = 8 * warp + ((lane >> 2) & 1) * 4 + (lane >> 3), c = lane & 3;
    using Raw = typename std::conditional<BITS == 0, uint4, typename std::conditional<BITS == 4, uint32_t, unsigned short>::type>::type;
    Raw rawk[4], rawv[4];
    __half nrm_next = __float2half(1.0f);
    auto fetch = [&](int j) {
        int row = j * PFA_KT + tr;
        row = min(row, p.rows - 1);
        const uint8_t* kp = ck_seq + (size_t)row * row_stride + (size_t)kvh * ROW_BYTES;
        const uint8_t* vp = cv_seq + (size_t)row * row_stride + (size_t)kvh * ROW_BYTES;
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // chunk c + 4 i: 16 fp16 bytes = 8 coordinates = 4 (4-bit) / 2 (2-bit) code bytes
            const int ch = c + 4 * i;
            rawk[i] = __ldg(reinterpret_cast<const Raw*>(kp + ch * (int)sizeof(Raw)));
            rawv[i] = __ldg(reinterpret_cast<const Raw*>(vp + ch * (int)sizeof(Raw)));
        }
        if (BITS != 0 && tid < 2 * PFA_KT) {
            const int r = min(j * PFA_KT + (tid & (PFA_KT - 1)), p.rows - 1);
            nrm_next = (tid < PFA_KT ? kn_seq : vn_seq)[(size_t)r * p.Hkv + kvh];
        }
    };
    auto dequant = [&](Raw w) -> uint4 {
        if constexpr (BITS == 0) {
            return w;
        } else if constexpr (BITS == 4) {
            uint4 o;
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(o.x) : "r"(lut + ((w & 0xffu) << 7)));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(o.y) : "r"(lut + (((w >> 8) & 0xffu) << 7)));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(o.z) : "r"(lut + (((w >> 16) & 0xffu) << 7)));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(o.w) : "r"(lut + ((w >> 24) << 7)));
            return o;
        } else {
            const uint32_t u = w;
            uint4 o;
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(o.x) : "r"(lut + ((u & 0xfu) << 7)));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(o.y) : "r"(lut + (((u >> 4) & 0xfu) << 7)));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(o.z) : "r"(lut + (((u >> 8) & 0xfu) << 7)));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(o.w) : "r"(lut + ((u >> 12) << 7)));
            return o;
        }
    };
    auto stage = [&](int b, int j) {  // the fetched tile j into buffer b
        // fp16 rows past the prompt may hold anything (a masked weight of 0 times a value that is not a number would
        // still poison the sums): they enter as zeros.  Packed rows dequantise to finite centroids whatever they hold.
        const bool blank = BITS == 0 && j * PFA_KT + tr >= p.T;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t off = (uint32_t)b * 16384u + (uint32_t)tr * 256u + (uint32_t)(((c + 4 * i) ^ (tr & 7)) << 4);
            uint4 kq = dequant(rawk[i]), vq = dequant(rawv[i]);
            if (blank) kq = vq = make_uint4(0u, 0u, 0u, 0u);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(sb + PfaSmem::K + off), "r"(kq.x), "r"(kq.y), "r"(kq.z), "r"(kq.w) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(sb + PfaSmem::V + off), "r"(vq.x), "r"(vq.y), "r"(vq.z), "r"(vq.w) : "memory");
        }
        if (BITS != 0 && tid < 2 * PFA_KT)
            reinterpret_cast<__half*>(pfa_smem + PfaSmem::NORMS)[b * 2 * PFA_KT + tid] = nrm_next;
    };

    float o[16][4];
#pragma unroll
    for (int nb = 0; nb < 16; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;
    float m_lo = -1e30f, m_hi = -1e30f, l_lo = 0.0f, l_hi = 0.0f;

    if (BITS != 0) {
        // ---- packed forms: the queries arrive as the model makes them; q_rot[d] = sum_k R[d][k] q[k] (reference
        //      engine/kernels.cu:1896-1903) is one tensor-core product per warp against R [d][k] in the (still idle) tile
        //      buffers, read like a K tile; the results, times log2(e) / sqrt(128), are the A fragments of the score product ----
        for (int i = tid; i < 128 * 16; i += PFA_THREADS) {
            const int row = i >> 4, ch = i & 15;
            const uint4 u = __ldg(reinterpret_cast<const uint4*>(p.rotation + (size_t)row * HEAD_DIM) + ch);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(sb + PfaSmem::K + (uint32_t)row * 256u + (uint32_t)((ch ^ (row & 7)) << 4)),
                         "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
        }
        __syncthreads();
        const int mi0 = lane >> 3, mr0 = lane & 7;
        uint32_t qr[8][4];
#pragma unroll
        for (int np = 0; np < 8; ++np) {  // output coordinates 16 np .. 16 np + 15
            float c0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, c1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const int row = 16 * np + (mi0 >> 1) * 8 + mr0, ch = 2 * ks + (mi0 & 1);
                uint32_t r[4];
                ldmatrix_x4(r, sb + PfaSmem::K + (uint32_t)row * 256u + (uint32_t)((ch ^ (row & 7)) << 4));
                mma16816(c0, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r[0], r[1]);
                mma16816(c1, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r[2], r[3]);
            }
            const float sc = 0.12751743074602467f;  // log2(e) / sqrt(128)
            qr[np][0] = pack_half2(c0[0] * sc, c0[1] * sc);   // row gl, coordinates 16 np + 2 t4, + 1
            qr[np][1] = pack_half2(c0[2] * sc, c0[3] * sc);   // row gl + 8
            qr[np][2] = pack_half2(c1[0] * sc, c1[1] * sc);   // row gl, coordinates 16 np + 8 + 2 t4, + 1
            qr[np][3] = pack_half2(c1[2] * sc, c1[3] * sc);
        }
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qa[ks][0] = qr[ks][0]; qa[ks][1] = qr[ks][1]; qa[ks][2] = qr[ks][2]; qa[ks][3] = qr[ks][3];
        }
    }
    __syncthreads();  // the table is complete; R has been read by every warp
    fetch(0);
    stage(0, 0);
    if (n_tiles > 1) fetch(1);
    __syncthreads();

    // ldmatrix lane roles: matrix mi = lane / 8, row lane % 8 of it
    const int mi = lane >> 3, mrow = lane & 7;
    const int k_tok = (mi >> 1) * 8 + mrow, k_chunk = mi & 1;   // K: matrices (tokens 0-7 | 8-15) x (chunk 0 | 1)
    const int v_tok = (mi & 1) * 8 + mrow, v_chunk = mi >> 1;   // V: matrices (tokens 0-7 | 8-15) x (chunk 0 | 1), transposed

    for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        const uint32_t kt = sb + PfaSmem::K + (uint32_t)b * 16384u, vt = sb + PfaSmem::V + (uint32_t)b * 16384u;
        // ---- S = Q . K^T: 8 blocks of 8 cache rows ----
        float s[8][4];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                const int tok = 16 * np + k_tok, ch = 2 * ks + k_chunk;
                uint32_t r[4];
                ldmatrix_x4(r, kt + (uint32_t)tok * 256u + (uint32_t)((ch ^ (tok & 7)) << 4));
                mma16816(s[2 * np], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r[0], r[1]);
                mma16816(s[2 * np + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r[2], r[3]);
            }
        }
        // ---- norms, causal limit, online softmax (columns 8 nb + 2 t4, + 1 of the tile; rows gl and gl + 8) ----
        const bool diagonal = j * PFA_KT + PFA_KT - 1 > q0;
        const uint32_t nk = sb + PfaSmem::NORMS + (uint32_t)b * 4u * PFA_KT + 4u * (uint32_t)t4;
        float mx_lo = -1e30f, mx_hi = -1e30f;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            float2 kn2 = make_float2(p.score_scale, p.score_scale);
            if (BITS != 0) {
                uint32_t w;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(nk + 16u * nb));
                kn2 = __half22float2(*reinterpret_cast<const __half2*>(&w));
                kn2.x *= p.score_scale;
                kn2.y *= p.score_scale;
            }
            s[nb][0] *= kn2.x; s[nb][1] *= kn2.y; s[nb][2] *= kn2.x; s[nb][3] *= kn2.y;
            if (diagonal) {
                const int tk = j * PFA_KT + 8 * nb + 2 * t4;
                if (tk > tq_lo) s[nb][0] = -1e30f;
                if (tk + 1 > tq_lo) s[nb][1] = -1e30f;
                if (tk > tq_hi) s[nb][2] = -1e30f;
                if (tk + 1 > tq_hi) s[nb][3] = -1e30f;
            }
            mx_lo = fmaxf(mx_lo, fmaxf(s[nb][0], s[nb][1]));
            mx_hi = fmaxf(mx_hi, fmaxf(s[nb][2], s[nb][3]));
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float cr_lo = ex2_approx(m_lo - mn_lo), cr_hi = ex2_approx(m_hi - mn_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        l_lo *= cr_lo;
        l_hi *= cr_hi;
#pragma unroll
        for (int nb = 0; nb < 16; ++nb) {
            o[nb][0] *= cr_lo; o[nb][1] *= cr_lo; o[nb][2] *= cr_hi; o[nb][3] *= cr_hi;
        }
        uint32_t pa[4][4];  // P (times the V norm) as A fragments: step kk covers the tile's rows 16 kk .. 16 kk + 15
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            // a masked column weighs exactly 0 (its score is -1e30; a row that has seen no live column yet has m = -1e30,
            // but every row's first tile holds cache row 0, which is live)
            const float p0 = s[nb][0] <= -1e30f ? 0.0f : ex2_approx(s[nb][0] - m_lo);
            const float p1 = s[nb][1] <= -1e30f ? 0.0f : ex2_approx(s[nb][1] - m_lo);
            const float p2 = s[nb][2] <= -1e30f ? 0.0f : ex2_approx(s[nb][2] - m_hi);
            const float p3 = s[nb][3] <= -1e30f ? 0.0f : ex2_approx(s[nb][3] - m_hi);
            l_lo += p0 + p1;
            l_hi += p2 + p3;
            float2 vn2 = make_float2(1.0f, 1.0f);
            if (BITS != 0) {
                uint32_t w;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(nk + 2u * PFA_KT + 16u * nb));
                vn2 = __half22float2(*reinterpret_cast<const __half2*>(&w));
            }
            // (rows past the prompt can hold anything, a norm that is not a number included: select, do not multiply)
            pa[nb >> 1][(nb & 1) * 2] = pack_half2(p0 == 0.0f ? 0.0f : p0 * vn2.x, p1 == 0.0f ? 0.0f : p1 * vn2.y);
            pa[nb >> 1][(nb & 1) * 2 + 1] = pack_half2(p2 == 0.0f ? 0.0f : p2 * vn2.x, p3 == 0.0f ? 0.0f : p3 * vn2.y);
        }
        // ---- O += P . V: 4 steps of 16 cache rows x 16 blocks of 8 coordinates ----
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int np = 0; np < 8; ++np) {
                const int tok = 16 * kk + v_tok, ch = 2 * np + v_chunk;
                uint32_t r[4];
                ldmatrix_x4_trans(r, vt + (uint32_t)tok * 256u + (uint32_t)((ch ^ (tok & 7)) << 4));
                mma16816(o[2 * np], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], r[0], r[1]);
                mma16816(o[2 * np + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], r[2], r[3]);
            }
        }
        // ---- the next tile into the other buffer (all warps left it before the previous barrier), the one after it
        //      on its way into registers ----
        if (j + 1 < n_tiles) {
            stage(b ^ 1, j + 1);
            if (j + 2 < n_tiles) fetch(j + 2);
        }
        __syncthreads();
    }

    // ---- row sums over the four lanes of a row ----
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = 1.0f / (l_lo + 1e-8f), inv_hi = 1.0f / (l_hi + 1e-8f);
    const int r_lo = 16 * warp + gl, r_hi = r_lo + 8;
    const int otok_lo = q0 + (r_lo >> gs), otok_hi = q0 + (r_hi >> gs);
    __half* dst_lo = out_seq + (size_t)otok_lo * p.q_dim + (size_t)(kvh * GRP + (r_lo & (GRP - 1))) * HEAD_DIM + 2 * t4;
    __half* dst_hi = out_seq + (size_t)otok_hi * p.q_dim + (size_t)(kvh * GRP + (r_hi & (GRP - 1))) * HEAD_DIM + 2 * t4;
    if (BITS == 0) {
#pragma unroll
        for (int nb = 0; nb < 16; ++nb) {
            if (otok_lo < p.T) *reinterpret_cast<__half2*>(dst_lo + 8 * nb) = __floats2half2_rn(o[nb][0] * inv_lo, o[nb][1] * inv_lo);
            if (otok_hi < p.T) *reinterpret_cast<__half2*>(dst_hi + 8 * nb) = __floats2half2_rn(o[nb][2] * inv_hi, o[nb][3] * inv_hi);
        }
        return;
    }
    // ---- packed forms: back out of the rotated space, out[d] = sum_k R[k][d] * acc[k] (reference engine/kernels.cu:1957),
    //      as one more tensor-core product per warp: the normalised sums, split into fp16 high and low parts, are the A
    //      operand exactly as the weights were in P . V, and R [k][d] (copied into the idle tile buffers, same swizzle)
    //      plays V's part through ldmatrix.trans ----
    uint32_t ah[8][4], al[8][4];  // step ks: coordinates k = 16 ks .. 16 ks + 15 of the rows gl and gl + 8
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const float x0 = o[2 * ks + h2][0] * inv_lo, x1 = o[2 * ks + h2][1] * inv_lo;
            const float y0 = o[2 * ks + h2][2] * inv_hi, y1 = o[2 * ks + h2][3] * inv_hi;
            const __half2 hx = __floats2half2_rn(x0, x1), hy = __floats2half2_rn(y0, y1);
            const float2 fx = __half22float2(hx), fy = __half22float2(hy);
            ah[ks][2 * h2] = *reinterpret_cast<const uint32_t*>(&hx);
            ah[ks][2 * h2 + 1] = *reinterpret_cast<const uint32_t*>(&hy);
            al[ks][2 * h2] = pack_half2(x0 - fx.x, x1 - fx.y);
            al[ks][2 * h2 + 1] = pack_half2(y0 - fy.x, y1 - fy.y);
        }
    }
    // (every warp left the tile buffers at the loop's last barrier) R: 128 rows of 256 bytes over the K buffers
    for (int i = tid; i < 128 * 16; i += PFA_THREADS) {
        const int row = i >> 4, ch = i & 15;
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(p.rotation + (size_t)row * HEAD_DIM) + ch);
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(sb + PfaSmem::K + (uint32_t)row * 256u + (uint32_t)((ch ^ (row & 7)) << 4)),
                     "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
    }
    __syncthreads();
#pragma unroll
    for (int np = 0; np < 8; ++np) {
        float c0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, c1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const int row = 16 * ks + v_tok, ch = 2 * np + v_chunk;
            uint32_t r[4];
            ldmatrix_x4_trans(r, sb + PfaSmem::K + (uint32_t)row * 256u + (uint32_t)((ch ^ (row & 7)) << 4));
            mma16816(c0, ah[ks][0], ah[ks][1], ah[ks][2], ah[ks][3], r[0], r[1]);
            mma16816(c0, al[ks][0], al[ks][1], al[ks][2], al[ks][3], r[0], r[1]);
            mma16816(c1, ah[ks][0], ah[ks][1], ah[ks][2], ah[ks][3], r[2], r[3]);
            mma16816(c1, al[ks][0], al[ks][1], al[ks][2], al[ks][3], r[2], r[3]);
        }
        if (otok_lo < p.T) {
            *reinterpret_cast<__half2*>(dst_lo + 16 * np) = __floats2half2_rn(c0[0], c0[1]);
            *reinterpret_cast<__half2*>(dst_lo + 16 * np + 8) = __floats2half2_rn(c1[0], c1[1]);
        }
        if (otok_hi < p.T) {
            *reinterpret_cast<__half2*>(dst_hi + 16 * np) = __floats2half2_rn(c0[2], c0[3]);
            *reinterpret_cast<__half2*>(dst_hi + 16 * np + 8) = __floats2half2_rn(c1[2], c1[3]);
        }
    }
}

}  // namespace tq
