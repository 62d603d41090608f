// Causal prefill attention on the 5th-generation tensor cores (tcgen05 + tensor memory), sm_100a.
//
// The same job as prefill_attention_kernel (tq_prefill_attn.cuh; reference engine/kernels.cu:1874-1960 and :1071-1158):
// query token t of a prompt attends to cache rows 0 .. t.  Here the products run as tcgen05.mma with the operands read
// from shared memory by the tensor core itself and the accumulators in tensor memory, so no warp spends its
// shared-memory bandwidth on ldmatrix:
//   * one CTA = 128 score rows (128 / GRP query tokens x the GRP query heads of one KV head) = the M dimension, 21 warps;
//   * warps 0-15 do the softmax, four threads per score row (row = TMEM lane; warps w, w + 4, w + 8, w + 12 reach the same
//     lanes and take a quarter of a tile's 64 columns each, their row maxima meet through shared memory); warp 20 issues
//     every product (one thread); warps 16-19 dequantise the cache
//     tiles: K as [64 tokens][128 coordinates] (the B operand of S = Q . K^T) and V TRANSPOSED as [128 coordinates][64
//     tokens] (the B operand of O += P . V; transposed 8 x 8 blocks at a time with ldmatrix.trans + stmatrix), both fp16
//     in the canonical K-major 128-byte-swizzled layout, double buffered and handed over through mbarriers;
//   * per 64-row tile: S (128 x 64, fp32) -> tensor memory -> registers; K norm, causal limit, online softmax; P (times the
//     V norm, fp16) -> shared memory as an A operand; O += P . V accumulates in tensor memory, and a warp rescales its 32
//     output rows in place (tcgen05.ld / .st) only in tiles where one of their maxima grew; S is double buffered in
//     tensor memory and the score product of tile j + 2 follows the value product of tile j on the tensor pipe, so the
//     scores of the next tile are waiting when the softmax threads finish a tile;
//   * packed forms: the query rotation (Q . R^T) at the start and the way back (O . R, with O split into fp16 high and low
//     parts) at the end are tcgen05 products as well.
// Every wait on a barrier is bounded; a wait that runs out raises the status word and the kernel runs to its end.
#pragma once

#include "tq_prefill_attn.cuh"
#include "tq_prefill_tc.cuh"

namespace tq {

constexpr int PTC_SPR = 4;                          // softmax threads per score row
constexpr int PTC_CPT = 64 / PTC_SPR;               // score columns of a tile per softmax thread
constexpr int PTC_OPT = 128 / PTC_SPR;              // output coordinates per softmax thread
constexpr int PTC_SOFT = 128 * PTC_SPR;             // softmax threads
constexpr int PTC_THREADS = PTC_SOFT + 128 + 32;    // + 4 producer warps + 1 warp that issues the products
constexpr int PTC_KT = 64;  // cache rows per tile

constexpr int PTC_STAGES = 3;  // K / V tile buffers
constexpr float PTC_SLACK = 4.0f;  // see the softmax: how far a row maximum may run ahead of the exponentials' reference point

struct PtcSmem {
    static constexpr uint32_t Q = 0;            // A operand [2 regions][128 rows][128 B]; at the end: high parts of the results
    static constexpr uint32_t K = 32768;        // PTC_STAGES x [2 regions][64 rows][128 B]; at the start: R; at the end: low parts
    static constexpr uint32_t V = K + PTC_STAGES * 16384;   // PTC_STAGES x [128 coordinate rows][128 B = 64 tokens]; at the end: R^T
    static constexpr uint32_t P = V + PTC_STAGES * 16384;   // A operand [128 rows][128 B = 64 tokens]
    static constexpr uint32_t VRM = P + 16384;  // V tile as it lies in the cache, [64 tokens][256 B], chunk c of row r at c ^ (r & 7)
    static constexpr uint32_t NORM = VRM + 16384;  // [PTC_STAGES][K, V][64] floats (converted once, by the producers)
    static constexpr uint32_t CTRL = NORM + PTC_STAGES * 512;  // mbarriers and the tensor-memory base
    static constexpr uint32_t XCH = CTRL + 128;   // float[2][PTC_SOFT]: exchange between the threads of a score row (by tile parity)
    static constexpr uint32_t LUT = XCH + 8 * PTC_SOFT;   // 4-bit: [256][32 lanes] half2
    static constexpr uint32_t BYTES = LUT + 32768;
};
constexpr size_t PTC_DYN_SMEM = PtcSmem::BYTES + 1024;  // + alignment slack

// 32 lanes x 32 consecutive 32-bit columns, registers -> tensor memory (the counterpart of tmem_ld32)
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void stmatrix_x4(uint32_t addr, const uint32_t (&r)[4]) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
                 : "memory");
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
    static_assert(BITS == 4 || BITS == 2 || BITS == 0, "kv_bits");
    extern __shared__ __align__(1024) uint8_t ptc_smem[];
    const uint32_t sb = (smem_u32(ptc_smem) + 1023u) & ~1023u;
    uint8_t* gb = ptc_smem + (sb - smem_u32(ptc_smem));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // roles: the first 4 PTC_SPR warps softmax (thread = score row 32 (warp & 3) + lane, column part warp >> 2), then 4 producer
    // warps, then the warp that issues the products
    constexpr int SW = 4 * PTC_SPR;
    const bool is_soft = warp < SW, is_prod = warp >= SW && warp < SW + 4, is_mma = warp == SW + 4;
    const int gs = p.grp_shift, GRP = 1 << gs, QT = PFA_ROWS >> gs;
    const int qb = (int)gridDim.y - 1 - (int)blockIdx.y;  // the longest causal prefixes of all heads and prompts first
    const int seq = (int)blockIdx.x / p.Hkv;
    const int kvh = (int)blockIdx.x - seq * p.Hkv;
    const int q0 = qb * QT;
    const int q_last = min(q0 + QT, p.T) - 1;
    const int n_tiles = q_last / PTC_KT + 1;
    constexpr int ROW_BYTES = BITS == 4 ? 64 : BITS == 2 ? 32 : 256;  // bytes of one head in a cache row
    const size_t row_stride = (size_t)p.Hkv * ROW_BYTES;
    const long long seq_row0 = p.row_base ? p.row_base[seq] : (long long)seq * p.seq_rows;
    const __half* const q_seq = p.q + (size_t)seq * (size_t)p.T * (size_t)p.q_tok_stride;
    __half* const out_seq = p.out + (size_t)seq * (size_t)p.T * (size_t)p.q_dim;
    const uint8_t* const ck_seq = p.ck + (size_t)seq_row0 * row_stride + (size_t)kvh * ROW_BYTES;
    const uint8_t* const cv_seq = p.cv + (size_t)seq_row0 * row_stride + (size_t)kvh * ROW_BYTES;
    const __half* const kn_seq = BITS != 0 ? p.kn + (size_t)seq_row0 * p.Hkv + kvh : nullptr;
    const __half* const vn_seq = BITS != 0 ? p.vn + (size_t)seq_row0 * p.Hkv + kvh : nullptr;

    // mbarriers
    const uint32_t bar_rot = sb + PtcSmem::CTRL;            // the two rotation products (count 1, tcgen05.commit)
    const uint32_t bar_pv = sb + PtcSmem::CTRL + 8u;        // value product of a tile done (count 1, commit)
    const uint32_t bar_sfull0 = sb + PtcSmem::CTRL + 16u;   // [2] score product into S buffer i done (count 1, commit)
    const uint32_t bar_pfull = sb + PtcSmem::CTRL + 32u;    // P of a tile written by all softmax threads
    const uint32_t bar_ready0 = sb + PtcSmem::CTRL + 40u;   // [PTC_STAGES] tile staged by the 128 producers
    const uint32_t bar_free0 = sb + PtcSmem::CTRL + 64u;    // [PTC_STAGES] the products that read the stage are done (commit)
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gb + PtcSmem::CTRL + 96);
    float* xch = reinterpret_cast<float*>(gb + PtcSmem::XCH);  // [256] row maxima / sums exchanged between the two halves of a row
    bool dead = false;
    auto give_up = [&]() {
        dead = true;
        if (p.status) atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
    };
    auto wait_bar = [&](uint32_t bar, uint32_t parity) {
        // (a third of this kernel's instructions were polls: each poll may now sleep up to 2 us inside the instruction)
        if (!dead && !mbar_wait_bounded_hint(bar, parity, 1u << 17, 2000u)) give_up();
    };

    // ---- once: tensor memory, barriers, table, this block's queries, R ----
    if (warp == 0) {
        // columns [0, 128): rotation products; [128, 192) and [192, 256): S of even / odd tiles; [256, 384): the output rows
        tmem_alloc(sb + PtcSmem::CTRL + 96u, 512u);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(bar_rot, 1);
        mbar_init(bar_pv, 1);
        mbar_init(bar_sfull0, 1);
        mbar_init(bar_sfull0 + 8u, 1);
        mbar_init(bar_pfull, PTC_SOFT);
        for (int i = 0; i < PTC_STAGES; ++i) {
            mbar_init(bar_ready0 + 8u * i, 128);
            mbar_init(bar_free0 + 8u * i, 1);
        }
        fence_mbar_init();
    }
    if (BITS == 4) {  // byte -> the two centroids of its nibbles, one column per lane
        for (int i = tid; i < 256 * 32; i += PTC_THREADS) {
            const int e = i >> 5;
            reinterpret_cast<uint32_t*>(gb + PtcSmem::LUT)[i] = pack_half2(kCent4[e & 15], kCent4[e >> 4]);
        }
    } else if (BITS == 2) {  // nibble -> the two centroids of its 2-bit codes
        for (int i = tid; i < 16 * 32; i += PTC_THREADS) {
            const int e = i >> 5;
            reinterpret_cast<uint32_t*>(gb + PtcSmem::LUT)[i] = pack_half2(kCent2[e & 3], kCent2[e >> 2]);
        }
    }
    const uint32_t lut = sb + PtcSmem::LUT + 4u * (uint32_t)lane;
    // softmax threads: score row, column part, the row's query
    const int srow = (warp & 3) * 32 + lane, part = is_soft ? (warp >> 2) : 0;
    const int my_tok = q0 + (srow >> gs), my_head = kvh * GRP + (srow & (GRP - 1));
    if (is_soft) {  // the query row: this thread's share of its 16 chunks
        const uint4* src = reinterpret_cast<const uint4*>(q_seq + (size_t)my_tok * p.q_tok_stride + (size_t)my_head * HEAD_DIM);
#pragma unroll
        for (int c = 0; c < 16 / PTC_SPR; ++c) {
            const int ch = (16 / PTC_SPR) * part + c;
            const uint4 u = my_tok < p.T ? __ldg(src + ch) : make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(gb + PtcSmem::Q + ptc_chunk(16384u, srow, ch)) = u;
        }
    }
    if (BITS != 0) {  // R [d][k] as a B operand (rows = output coordinate d) over the K stages
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
    constexpr uint32_t O_COL = 256u;

    if (BITS != 0) {
        // ---- q_rot = Q . R^T (reference engine/kernels.cu:1896-1903), scaled by log2(e) / sqrt(128), back into the Q tile ----
        if (is_mma && lane == 0) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t koff = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                umma_f16(tmem, umma_desc_sw128(sb + PtcSmem::Q + koff), umma_desc_sw128(sb + PtcSmem::K + koff), PTC_IDESC_N128, ks != 0);
            }
            umma_commit(bar_rot);
        }
        if (is_soft) {
            wait_bar(bar_rot, 0u);
            tc_fence_after();
#pragma unroll 1
            for (int c2 = 0; c2 < PTC_OPT / 32; ++c2) {  // this thread's coordinates
                uint32_t r[32];
                tmem_ld32(my_lanes + (uint32_t)(PTC_OPT * part) + 32u * c2, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 u;
                    const float sc = 0.12751743074602467f;
                    u.x = pack_half2(__uint_as_float(r[8 * i]) * sc, __uint_as_float(r[8 * i + 1]) * sc);
                    u.y = pack_half2(__uint_as_float(r[8 * i + 2]) * sc, __uint_as_float(r[8 * i + 3]) * sc);
                    u.z = pack_half2(__uint_as_float(r[8 * i + 4]) * sc, __uint_as_float(r[8 * i + 5]) * sc);
                    u.w = pack_half2(__uint_as_float(r[8 * i + 6]) * sc, __uint_as_float(r[8 * i + 7]) * sc);
                    *reinterpret_cast<uint4*>(gb + PtcSmem::Q + ptc_chunk(16384u, srow, (PTC_OPT / 8) * part + 4 * c2 + i)) = u;
                }
            }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        __syncthreads();  // the rotated queries are in place and R has been consumed: the K stages may take tiles
        tc_fence_after();
    }

    float m_run = -1e30f, l_run = 0.0f;

    if (is_prod) {
        // ================= producers: tile j into stage j % PTC_STAGES =================
        const int pt = tid - PTC_SOFT, pw = pt >> 5;
        const int ktr = pt & 63, kc = pt >> 6;  // token row of the tile, half of its 128 coordinates
        constexpr int NRAW = BITS == 4 ? 2 : BITS == 2 ? 1 : 8;  // 16-byte loads per thread and array (64 coordinates)
        constexpr int HALF_ROW = BITS == 4 ? 32 : BITS == 2 ? 16 : 128;  // their bytes
        uint4 kraw[NRAW], vraw[NRAW];
        __half nraw = __float2half(1.0f);
        auto fetch = [&](int j) {  // the raw words of tile j into registers
            const int row = min(j * PTC_KT + ktr, p.rows - 1);
            const uint4* ksrc = reinterpret_cast<const uint4*>(ck_seq + (size_t)row * row_stride + HALF_ROW * kc);
            const uint4* vsrc = reinterpret_cast<const uint4*>(cv_seq + (size_t)row * row_stride + HALF_ROW * kc);
#pragma unroll
            for (int i = 0; i < NRAW; ++i) {
                kraw[i] = __ldg(ksrc + i);
                vraw[i] = __ldg(vsrc + i);
            }
            if (BITS != 0) {
                const int nrow = min(j * PTC_KT + (pt & 63), p.rows - 1);
                nraw = (pt < 64 ? kn_seq : vn_seq)[(size_t)nrow * p.Hkv];
            }
        };
        fetch(0);
        int b = 0, use = 0;  // stage of tile j and how often the stage has been used before
        for (int j = 0; j < n_tiles; ++j) {
            if (use > 0) wait_bar(bar_free0 + 8u * b, (uint32_t)((use - 1) & 1));
            const int row0 = j * PTC_KT;
            uint8_t* kt = gb + PtcSmem::K + (uint32_t)b * 16384u;
            const uint32_t vt = sb + PtcSmem::V + (uint32_t)b * 16384u;
            const bool blank = BITS == 0 && row0 + ktr >= p.T;  // fp16 rows past the prompt may hold anything
            // K tile (the B operand as it is) and V tile (row-major for now): row ktr, chunks 8 kc .. 8 kc + 7
            if (BITS == 4) {
                const uint32_t kw[8] = {kraw[0].x, kraw[0].y, kraw[0].z, kraw[0].w, kraw[NRAW > 1 ? 1 : 0].x, kraw[NRAW > 1 ? 1 : 0].y,
                                        kraw[NRAW > 1 ? 1 : 0].z, kraw[NRAW > 1 ? 1 : 0].w};
                const uint32_t vw[8] = {vraw[0].x, vraw[0].y, vraw[0].z, vraw[0].w, vraw[NRAW > 1 ? 1 : 0].x, vraw[NRAW > 1 ? 1 : 0].y,
                                        vraw[NRAW > 1 ? 1 : 0].z, vraw[NRAW > 1 ? 1 : 0].w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    uint4 u, w;
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.x) : "r"(lut + ((kw[i] & 0xffu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.y) : "r"(lut + (((kw[i] >> 8) & 0xffu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.z) : "r"(lut + (((kw[i] >> 16) & 0xffu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.w) : "r"(lut + ((kw[i] >> 24) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w.x) : "r"(lut + ((vw[i] & 0xffu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w.y) : "r"(lut + (((vw[i] >> 8) & 0xffu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w.z) : "r"(lut + (((vw[i] >> 16) & 0xffu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w.w) : "r"(lut + ((vw[i] >> 24) << 7)));
                    *reinterpret_cast<uint4*>(kt + ptc_chunk(8192u, ktr, 8 * kc + i)) = u;
                    *reinterpret_cast<uint4*>(gb + PtcSmem::VRM + (uint32_t)ktr * 256u + (uint32_t)(((8 * kc + i) ^ (ktr & 7)) << 4)) = w;
                }
            } else if (BITS == 2) {
                const uint32_t kw[4] = {kraw[0].x, kraw[0].y, kraw[0].z, kraw[0].w};
                const uint32_t vw[4] = {vraw[0].x, vraw[0].y, vraw[0].z, vraw[0].w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {  // chunk i: 8 coordinates = 2 bytes = 4 nibbles
                    const uint32_t k16 = (kw[i >> 1] >> (16 * (i & 1))) & 0xffffu, v16 = (vw[i >> 1] >> (16 * (i & 1))) & 0xffffu;
                    uint4 u, w;
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.x) : "r"(lut + ((k16 & 0xfu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.y) : "r"(lut + (((k16 >> 4) & 0xfu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.z) : "r"(lut + (((k16 >> 8) & 0xfu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u.w) : "r"(lut + ((k16 >> 12) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w.x) : "r"(lut + ((v16 & 0xfu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w.y) : "r"(lut + (((v16 >> 4) & 0xfu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w.z) : "r"(lut + (((v16 >> 8) & 0xfu) << 7)));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w.w) : "r"(lut + ((v16 >> 12) << 7)));
                    *reinterpret_cast<uint4*>(kt + ptc_chunk(8192u, ktr, 8 * kc + i)) = u;
                    *reinterpret_cast<uint4*>(gb + PtcSmem::VRM + (uint32_t)ktr * 256u + (uint32_t)(((8 * kc + i) ^ (ktr & 7)) << 4)) = w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 u = blank ? make_uint4(0u, 0u, 0u, 0u) : kraw[i < NRAW ? i : 0];
                    const uint4 w = blank ? make_uint4(0u, 0u, 0u, 0u) : vraw[i < NRAW ? i : 0];
                    *reinterpret_cast<uint4*>(kt + ptc_chunk(8192u, ktr, 8 * kc + i)) = u;
                    *reinterpret_cast<uint4*>(gb + PtcSmem::VRM + (uint32_t)ktr * 256u + (uint32_t)(((8 * kc + i) ^ (ktr & 7)) << 4)) = w;
                }
            }
            if (BITS != 0) reinterpret_cast<float*>(gb + PtcSmem::NORM)[b * 128 + pt] = __half2float(nraw);
            if (j + 1 < n_tiles) fetch(j + 1);  // on its way during the transposition and the wait for the next stage
            named_barrier(1, 128);  // the row-major V tile is complete
            // V transposed into the B operand [128 coordinate rows][64 tokens]: 8 x 8 blocks through ldmatrix.trans /
            // stmatrix, four at a time; this warp takes the coordinate blocks 4 pw .. 4 pw + 3
            {
                const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
                for (int it = 0; it < 8; ++it) {  // token block `it` (8 tokens), coordinate blocks 4 pw + mi
                    const int tok = 8 * it + mr, cb = 4 * pw + mi;
                    uint32_t r[4];
                    ldmatrix_x4_trans(r, sb + PtcSmem::VRM + (uint32_t)tok * 256u + (uint32_t)((cb ^ (tok & 7)) << 4));
                    // matrix mi now holds (row = coordinate 8 cb + l / 4, columns = tokens 8 it + 2 (l % 4), + 1)
                    const int crow = 8 * cb + mr;
                    stmatrix_x4(vt + ptc_chunk(0u, crow, it), r);
                }
            }
            fence_proxy_async_smem();  // generic-proxy writes of the operands before the tensor core reads them
            mbar_arrive(bar_ready0 + 8u * b);
            named_barrier(1, 128);  // nobody overwrites the row-major tile while a neighbour still transposes it
            if (++b == PTC_STAGES) {
                b = 0;
                ++use;
            }
        }
    } else if (is_mma) {
        // ================= one thread issues every product =================
        // order on the tensor pipe: S(0), S(1), P.V(0), S(2), P.V(1), S(3), ...: the scores of tile j + 1 are ready when
        // the softmax threads finish tile j
        if (lane == 0) {
            auto issue_scores = [&](int j) {  // S(j) = Q . K^T(j): 128 x 64, 8 steps of 16 coordinates, into S buffer j & 1
                const int st = j % PTC_STAGES, use = j / PTC_STAGES;
                wait_bar(bar_ready0 + 8u * st, (uint32_t)(use & 1));
                tc_fence_after();
                if (dead) return;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t ka = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                    const uint32_t kb = (uint32_t)(ks >> 2) * 8192u + (uint32_t)(ks & 3) * 32u;
                    umma_f16(tmem + 128u + 64u * (uint32_t)(j & 1), umma_desc_sw128(sb + PtcSmem::Q + ka),
                             umma_desc_sw128(sb + PtcSmem::K + (uint32_t)st * 16384u + kb), PTC_IDESC_N64, ks != 0);
                }
                umma_commit(bar_sfull0 + 8u * (uint32_t)(j & 1));
            };
            issue_scores(0);
            if (n_tiles > 1) issue_scores(1);
            for (int j = 0; j < n_tiles; ++j) {
                const int st = j % PTC_STAGES;
                wait_bar(bar_pfull, (uint32_t)(j & 1));  // P(j) is written (and S(j) taken out of tensor memory) by every row
                tc_fence_after();
                if (!dead) {  // O += P . V: 128 x 128, 4 steps of 16 tokens
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        umma_f16(tmem + O_COL, umma_desc_sw128(sb + PtcSmem::P + 32u * ks),
                                 umma_desc_sw128(sb + PtcSmem::V + (uint32_t)st * 16384u + 32u * ks), PTC_IDESC_N128, (j | ks) != 0);
                    umma_commit(bar_pv);
                    umma_commit(bar_free0 + 8u * st);  // the stage has been read by S(j) and P.V(j)
                }
                if (j + 2 < n_tiles) issue_scores(j + 2);
            }
        }
    } else {
        // ================= softmax threads: row srow, columns PTC_CPT part .. + PTC_CPT - 1 of every tile =================
        const int pair_bar = 2 + (warp & 3);  // named barrier of the PTC_SPR warps that share 32 rows
        constexpr int ROW_THREADS = 32 * PTC_SPR;
        for (int j = 0; j < n_tiles; ++j) {
            const int st = j % PTC_STAGES, use = j / PTC_STAGES;
            wait_bar(bar_ready0 + 8u * st, (uint32_t)(use & 1));  // (for the tile's norms; the products wait for it themselves)
            wait_bar(bar_sfull0 + 8u * (uint32_t)(j & 1), (uint32_t)((j >> 1) & 1));
            tc_fence_after();
            uint32_t sr[PTC_CPT];
            if constexpr (PTC_CPT == 32) tmem_ld32(my_lanes + 128u + 64u * (uint32_t)(j & 1) + (uint32_t)(PTC_CPT * part), reinterpret_cast<uint32_t(&)[32]>(sr[0]));
            else tmem_ld16(my_lanes + 128u + 64u * (uint32_t)(j & 1) + (uint32_t)(PTC_CPT * part), reinterpret_cast<uint32_t(&)[16]>(sr[0]));
            tmem_ld_wait();
            // ---- K norm, causal limit, row maximum over both halves ----
            const bool diagonal = j * PTC_KT + PTC_KT - 1 > q0;
            const float4* nrm = reinterpret_cast<const float4*>(gb + PtcSmem::NORM + (uint32_t)st * 512u);
            float mx = -1e30f;
#pragma unroll
            for (int c8 = 0; c8 < PTC_CPT / 8; ++c8) {
                float kn8[8];
                if (BITS != 0) {
                    // (every thread of the warp reads the same words: a broadcast)
                    const float4 n0 = nrm[2 * ((PTC_CPT / 8) * part + c8)], n1 = nrm[2 * ((PTC_CPT / 8) * part + c8) + 1];
                    kn8[0] = n0.x; kn8[1] = n0.y; kn8[2] = n0.z; kn8[3] = n0.w;
                    kn8[4] = n1.x; kn8[5] = n1.y; kn8[6] = n1.z; kn8[7] = n1.w;
                }
#pragma unroll
                for (int e = 0; e < 8; e += 2) {  // (two columns per multiplication: the packed fp32 form)
                    const int c = 8 * c8 + e;
                    const float2 sc2 = BITS != 0 ? make_float2(kn8[e], kn8[e + 1]) : make_float2(p.score_scale, p.score_scale);
                    float2 sv = mul2(make_float2(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])), sc2);
                    if (diagonal) {
                        if (j * PTC_KT + PTC_CPT * part + c > my_tok) sv.x = -1e30f;
                        if (j * PTC_KT + PTC_CPT * part + c + 1 > my_tok) sv.y = -1e30f;
                    }
                    sr[c] = __float_as_uint(sv.x);
                    sr[c + 1] = __float_as_uint(sv.y);
                    mx = fmaxf(mx, fmaxf(sv.x, sv.y));
                }
            }
            xch[(j & 1) * PTC_SOFT + tid] = mx;
            named_barrier(pair_bar, ROW_THREADS);
#pragma unroll
            for (int k = 1; k < PTC_SPR; ++k) mx = fmaxf(mx, xch[(j & 1) * PTC_SOFT + ((tid + 128 * k) & (PTC_SOFT - 1))]);
            // The reference point of the exponentials follows the row maximum only when that has grown by more than
            // PTC_SLACK (in powers of two) since the point was set: weights then stay below 2^PTC_SLACK, and the output rows
            // in tensor memory need rescaling in the first tiles only.  The result does not depend on the point.
            const bool grew = mx > m_run + PTC_SLACK;
            const float mn = grew ? mx : m_run;
            const float corr = ex2_approx(m_run - mn);
            m_run = mn;
            // the value product of the previous tile has read the P tile and updated the output rows
            if (j > 0) {
                wait_bar(bar_pv, (uint32_t)((j - 1) & 1));
                tc_fence_after();
                if (__any_sync(0xffffffffu, grew)) {  // a row's maximum grew: this warp's half of the output rows is rescaled in place
#pragma unroll 1
                    for (int c2 = 0; c2 < PTC_OPT / 32; ++c2) {
                        uint32_t r[32];
                        tmem_ld32(my_lanes + O_COL + (uint32_t)(PTC_OPT * part) + 32u * c2, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
                        tmem_st32(my_lanes + O_COL + (uint32_t)(PTC_OPT * part) + 32u * c2, r);
                    }
                    tmem_st_wait();
                }
            }
            // ---- P (times the V norm) as fp16 into the A operand tile ----
            float lsum = 0.0f;
            float2 lsum2 = make_float2(0.0f, 0.0f);
            const float2 minus_mn = make_float2(-mn, -mn);
#pragma unroll
            for (int c8 = 0; c8 < PTC_CPT / 8; ++c8) {
                float vn8[8];
                if (BITS != 0) {
                    const float4 n0 = nrm[16 + 2 * ((PTC_CPT / 8) * part + c8)], n1 = nrm[16 + 2 * ((PTC_CPT / 8) * part + c8) + 1];
                    vn8[0] = n0.x; vn8[1] = n0.y; vn8[2] = n0.z; vn8[3] = n0.w;
                    vn8[4] = n1.x; vn8[5] = n1.y; vn8[6] = n1.z; vn8[7] = n1.w;
                }
                float pv[8];
                if (diagonal) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float sv = __uint_as_float(sr[8 * c8 + e]);
                        const float pe = sv <= -1e30f ? 0.0f : ex2_approx(sv - mn);
                        lsum += pe;
                        // (rows past the prompt can hold anything, a norm that is not a number included: select, do not multiply)
                        pv[e] = pe == 0.0f ? 0.0f : (BITS != 0 ? pe * vn8[e] : pe);
                    }
                } else {  // every row of the tile lies before every query of the block: nothing is masked
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                        const float2 d = add2(make_float2(__uint_as_float(sr[8 * c8 + e]), __uint_as_float(sr[8 * c8 + e + 1])), minus_mn);
                        const float2 pe = make_float2(ex2_approx(d.x), ex2_approx(d.y));
                        lsum2 = add2(lsum2, pe);
                        const float2 w = BITS != 0 ? mul2(pe, make_float2(vn8[e], vn8[e + 1])) : pe;
                        pv[e] = w.x;
                        pv[e + 1] = w.y;
                    }
                }
                uint4 u;
                u.x = pack_half2(pv[0], pv[1]); u.y = pack_half2(pv[2], pv[3]);
                u.z = pack_half2(pv[4], pv[5]); u.w = pack_half2(pv[6], pv[7]);
                *reinterpret_cast<uint4*>(gb + PtcSmem::P + ptc_chunk(0u, srow, (PTC_CPT / 8) * part + c8)) = u;
            }
            l_run = l_run * corr + (lsum + (lsum2.x + lsum2.y));
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar_pfull);
        }
        wait_bar(bar_pv, (uint32_t)((n_tiles - 1) & 1));  // the last value product
        tc_fence_after();
        // the row's sum over both column halves
        named_barrier(pair_bar, ROW_THREADS);  // (the partners have read the last maxima)
        xch[tid] = l_run;
        named_barrier(pair_bar, ROW_THREADS);
#pragma unroll
        for (int k = 1; k < PTC_SPR; ++k) l_run += xch[(tid + 128 * k) & (PTC_SOFT - 1)];
    }

    // ================= results =================
    const float inv = 1.0f / (l_run + 1e-8f);
    __half* const dst = out_seq + (size_t)my_tok * p.q_dim + (size_t)my_head * HEAD_DIM + PTC_OPT * part;
    if (BITS == 0) {
        if (is_soft) {
#pragma unroll 1
            for (int c2 = 0; c2 < PTC_OPT / 32; ++c2) {
                uint32_t r[32];
                tmem_ld32(my_lanes + O_COL + (uint32_t)(PTC_OPT * part) + 32u * c2, r);
                tmem_ld_wait();
                if (my_tok < p.T) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 u;
                        u.x = pack_half2(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
                        u.y = pack_half2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
                        u.z = pack_half2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
                        u.w = pack_half2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + 32 * c2 + 8 * i) = u;
                    }
                }
            }
        }
    } else {
        // out[d] = sum_k R[k][d] * acc[k] (reference engine/kernels.cu:1957): the normalised rows, split into fp16 high and low
        // parts, times R^T [d][k] (the B operand's rows are the output coordinates)
        __syncthreads();  // every product of the tile loop has completed (the softmax threads waited for the last one)
        if (is_soft) {
#pragma unroll 1
            for (int c2 = 0; c2 < PTC_OPT / 32; ++c2) {
                uint32_t r[32];
                tmem_ld32(my_lanes + O_COL + (uint32_t)(PTC_OPT * part) + 32u * c2, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 uh, ul;
                    uint32_t* ph = &uh.x;
                    uint32_t* pl = &ul.x;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float x0 = __uint_as_float(r[8 * i + 2 * e]) * inv, x1 = __uint_as_float(r[8 * i + 2 * e + 1]) * inv;
                        const __half2 h = __floats2half2_rn(x0, x1);
                        const float2 f = __half22float2(h);
                        ph[e] = *reinterpret_cast<const uint32_t*>(&h);
                        pl[e] = pack_half2(x0 - f.x, x1 - f.y);
                    }
                    *reinterpret_cast<uint4*>(gb + PtcSmem::Q + ptc_chunk(16384u, srow, (PTC_OPT / 8) * part + 4 * c2 + i)) = uh;
                    *reinterpret_cast<uint4*>(gb + PtcSmem::K + ptc_chunk(16384u, srow, (PTC_OPT / 8) * part + 4 * c2 + i)) = ul;
                }
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
        if (is_mma && lane == 0 && !dead) {
#pragma unroll
            for (int part = 0; part < 2; ++part) {
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t koff = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                    umma_f16(tmem, umma_desc_sw128(sb + (part ? PtcSmem::K : PtcSmem::Q) + koff), umma_desc_sw128(sb + PtcSmem::V + koff),
                             PTC_IDESC_N128, (part | ks) != 0);
                }
            }
            umma_commit(bar_rot);
        }
        if (is_soft) {
            wait_bar(bar_rot, 1u);
            tc_fence_after();
#pragma unroll 1
            for (int c2 = 0; c2 < PTC_OPT / 32; ++c2) {
                uint32_t r[32];
                tmem_ld32(my_lanes + (uint32_t)(PTC_OPT * part) + 32u * c2, r);
                tmem_ld_wait();
                if (my_tok < p.T) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 u;
                        u.x = pack_half2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]));
                        u.y = pack_half2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                        u.z = pack_half2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                        u.w = pack_half2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                        *reinterpret_cast<uint4*>(dst + 32 * c2 + 8 * i) = u;
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
