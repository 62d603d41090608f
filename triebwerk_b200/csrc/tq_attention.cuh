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
//     a CUDA graph).  The list is cut into equal contiguous slices, one per WORKER; a CTA holds two workers
//     (16 warps on the SM for latency hiding), each a group of Hkv warps with its own named barrier.  Every SM
//     gets the same number of bytes whatever the mix of sequence lengths.
//   * Inside a worker warp w owns KV head w and all of its query heads (2 for Qwen3-0.6B, 4 for Qwen3-8B):
//     every cache byte is fetched from HBM once, not once per query head as in the reference.
//   * A worker streams its tiles through a ring of shared-memory stages filled by the TMA engine (no multicast):
//     the K codes of 32 token rows arrive as [32 rows][128 B] boxes (two heads' bytes per row, four boxes for eight
//     heads) through a 2-D tensor map with the 128-byte swizzle, likewise V, and the fp16 norms as two small
//     contiguous bulk copies; completion on one mbarrier per stage.  (An optional cp.async.bulk.prefetch.L2 of tiles
//     further ahead exists, TQ_ATTN_L2_AHEAD; it is off by default because it did not pay on B200.)  The last warp of the
//     worker to finish a stage (one shared-memory atomic per warp and tile) re-arms it: nobody waits for a slower
//     warp.  With the swizzle, and with the eight tokens of a score block taken in the order 0,5,2,7,4,1,6,3, every
//     16-, 8- and 4-byte read of packed codes is free of bank conflicts.
//   * Codes are turned into fp16 centroids one BYTE at a time (2 codes for 4-bit, 4 for 2-bit) through a
//     shared-memory table with one private column per lane (bank-conflict free); the table sits at shared
//     address 0x10000 so that a single PRMT builds the lookup address from the packed word.
//   * The dot products run on the tensor cores with warp-level mma.sync.m16n8k16 (fp16 in, fp32 accumulate):
//     scores as Q(16 x 16) * K^T(16 x 8 tokens) with the query split into an fp16 high part (rows 0-7) and
//     low part (rows 8-15) so that no query precision is lost, and the value sum in transposed form
//     V^T(16 coords x 16 tokens) * P^T(16 tokens x 8 heads); the token pairs the V^T fragment needs are
//     formed by interleaving the nibbles of two tokens' words BEFORE the table lookup.  Scalar fp32 FMAs cannot
//     keep up with HBM3e on this path: 512 FMAs per 132-byte row is more than the SMs can issue.
//   * A worker that finishes its part of a sequence writes (acc[128], m, l) per query head to the workspace
//     and takes a ticket; the last arrival merges all parts, and multiplies by R^T on the tensor cores
//     (normalised accumulators split into fp16 high + low parts as the A operand, R^T as B).  Nobody spins on
//     anybody: the ticket is a single atomicAdd.
#pragma once

#include <type_traits>

#include "tq_common.cuh"

namespace tq {

constexpr uint32_t LUT_ABS = 0x10000u;        // absolute shared address of the byte -> centroid table
constexpr uint32_t REGION_B_ABS = 0x20000u;   // more stage blocks live above the table
constexpr int ATTN_MAX_HEADS = 32;
constexpr size_t ATTN_DYN_SMEM = 226 * 1024;  // requested dynamic shared memory
constexpr int ATTN_GROUPS = 2;                // workers per CTA
constexpr int ATTN_MAX_STAGES = 4;            // shared-memory stages per worker (as many as fit, at most this)
constexpr int ATTN_L2_AHEAD = 0;              // tiles prefetched into L2 beyond the ring; 0 = off (measured: no gain on B200)
constexpr int MERGE_ROW = 136;                // halves per row of the merge A-operand (padded: conflict-free)

struct AttnParams {
    const uint8_t* ck;         // packed K codes [rows][kvp]
    const uint8_t* cv;
    const __half* kn;          // norms [rows][Hkv]
    const __half* vn;
    const float* q_rot;        // [G][H][128], pre-scaled by log2(e)/sqrt(128)
    const __half* rotation_t;  // R transposed: rotation_t[d][k] = R[k][d]
    __half* out;               // [G][q_dim]
    float* out_f32;            // optional [G][H][128]: the same results before the rounding to fp16 (error reports), or null
    const int* positions;      // device [G] or null
    const long long* row_base;
    // Shared prefixes (optional, both null otherwise): the first prefix_tiles[g] tiles of sequence g are read from the rows
    // prefix_base[g] + 32 * tile (another sequence's slot, which holds the common prompt once); every later tile j from
    // row_base[g] + 32 * j as usual -- row_base[g] then already has the prefix length subtracted.
    const long long* prefix_base;
    const int* prefix_tiles;
    const int* tile_start;     // [G+1]
    const int* worker_g;       // first sequence of each worker's slice, or null (then it is searched for)
    int* tickets;              // [G]
    float* partials;           // [workers+G][H][PART_STRIDE]
    int* status;
    long long total_rows;      // rows of the cache arrays (copies are clipped to it)
    int pos_value;
    int max_seq_len;
    int G, H, Hkv, q_dim;
    // fused form (one launch per layer and step: append the new token, rotate the queries, attend)
    const __half* new_k;       // [G][kv_dim] this step's keys, values and queries
    const __half* new_v;
    const __half* new_q;       // [G][q_dim]
    const __half* rotation;    // R row-major (B operand of the query rotation); rot_copies copies back to back
    int rot_copies;            // every worker reads copy (worker % rot_copies): 300 workers fetching the same 32 KB at once queue up in L2
    int kv_dim;
    int capacity_rows;         // rows a sequence may use (position check)
    const int* seq_capacity;   // optional [G]: rows sequence g may use (ragged slots), instead of capacity_rows
    int app_weight;            // cost of one append in tiles, for the balance of the work list
    int early;                 // 1: positions and this layer's cache tiles may be read before the previous kernel in the
                               // stream has finished (the caller knows it writes neither): table, slice and first copies
                               // then run under that kernel's tail
    // prefill form: a "sequence" of the launch is a group of qg consecutive query tokens of ONE cache (row base 0); its
    // H = qg * (real heads) rows are ordered (kv head, token in group, head of the kv head); token t attends to rows 0..t
    int qg;                    // 0 or 1: plain decode
    int qg_tokens;             // number of query tokens (the last group may be partial)
    int l2_ahead;              // tiles prefetched into L2 beyond the shared-memory ring
    // whole-step form (MODE 2): ONE launch streams the layers [layer0, layer0 + n_layers) back to back -- every worker
    // walks its slice of the tile list once per layer, its ring of stages never drains in between -- rotates the
    // queries itself and only PUBLISHES its split-K partials, per layer; merge_partials_kernel finishes the step.
    // ck/cv/kn/vn are the arrays of layer0, the tensor maps have the layer as their outermost coordinate.
    int layer0, n_layers;
    long long norm_layer_stride;   // halves between consecutive layers' norm arrays
    long long q_layer_stride;      // halves between consecutive layers' queries (and outputs)
    long long part_layer_stride;   // floats between consecutive layers' partial areas
    int* table_out;                // [G + 4]: the tile table, then {workers taking part, total tiles}, for the merge kernel
    const __half* q_rot16;         // whole-step form: pre-rotated, pre-scaled fp16 queries of layer0, [layers][G][H][128]
                                   // (rotate_queries_kernel); a sequence's block reaches shared memory by one bulk copy
#ifdef TQ_TIMING_SWITCHES
    int debug;                 // timing-experiment builds only: bit 0 = skip the math, bit 1 = skip the loads, ... (results are then wrong)
    unsigned long long* stamps;  // timing-experiment builds only: [8] summed clock deltas of the tile loop's sections
#endif
};

// Switches that leave parts of the kernel out, for timing experiments.  They exist only in builds made with
// -DTQ_TIMING_SWITCHES; in the library they are the constant false and the compiler removes the branches.
#ifdef TQ_TIMING_SWITCHES
#define TQ_DBG(bit) ((p.debug & (bit)) != 0)
#define TQ_DBG_FACTOR (p.debug >> 8)
#define TQ_STAMP(i) do { const long long _t = clock64(); stamp_acc[i] += _t - stamp_last; stamp_last = _t; } while (0)
#else
#define TQ_DBG(bit) false
#define TQ_DBG_FACTOR 0
#define TQ_STAMP(i) do { } while (0)
#endif

template <int BITS>
struct AttnGeom {
    static constexpr int BPH = (BITS == 4) ? 64 : 32;  // code bytes per head per token
};

// Region A (below the table): barriers, control words, merge operands, then stage blocks.
struct RegionA {
    static constexpr uint32_t BAR_OFF = 0;       // per group: full[ATTN_MAX_STAGES] mbarriers (8 B each)
    static constexpr uint32_t CNT_OFF = 128;     // per group: done-counters, one u32 per stage
    static constexpr uint32_t CTRL_OFF = 256;    // one word per group
    static constexpr uint32_t MERGE_OFF = 512;   // per group: hi + lo [16][MERGE_ROW] halves
    static constexpr uint32_t MERGE_GROUP_BYTES = 2 * 16 * MERGE_ROW * 2;  // 8704
    static constexpr uint32_t BLOCKS_OFF = MERGE_OFF + ATTN_GROUPS * MERGE_GROUP_BYTES;
    // fused form only: tile table of the launch, then per group the append's codes, partial sums and destinations
    static constexpr uint32_t FUSED_SCAN_OFF = BLOCKS_OFF;           // 32 ints of scan scratch
    static constexpr uint32_t FUSED_TS_OFF = FUSED_SCAN_OFF + 128;   // tile_start[G + 1], G <= FUSED_MAX_G
    static constexpr uint32_t FUSED_APP_OFF = FUSED_TS_OFF + 4096;
    static constexpr uint32_t FUSED_APP_GROUP_BYTES = 16 * 128 + 16 * 4 * 4 + 128;  // codes [16][128], 1/norm [16], spare
    static constexpr uint32_t FUSED_BLOCKS_OFF = FUSED_APP_OFF + ATTN_GROUPS * FUSED_APP_GROUP_BYTES;
};
constexpr int FUSED_MAX_G = 1023;

__device__ __forceinline__ void group_barrier(int group, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(nthreads) : "memory");
}

__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t atom_add_shared(uint32_t addr, uint32_t v) {
    uint32_t old;
    asm volatile("atom.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
    return old;
}
// Loads whose ordering is carried by data dependence (their address derives from a value produced after the
// barrier wait), so the compiler may schedule them freely among the arithmetic of a tile.
__device__ __forceinline__ uint32_t ldsp32(uint32_t addr) {
    uint32_t r;
    asm("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(addr));
    return r;
}
__device__ __forceinline__ uint2 ldsp64(uint32_t addr) {
    uint2 r;
    asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(addr));
    return r;
}
__device__ __forceinline__ uint4 ldsp128(uint32_t addr) {
    uint4 r;
    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}
// The same loads kept in program order relative to barriers and other volatile accesses (staging buffers that are
// rewritten between uses).
__device__ __forceinline__ uint2 ldsv64(uint32_t addr) {
    uint2 r;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(addr));
    return r;
}
__device__ __forceinline__ uint4 ldsv128(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}
__device__ __forceinline__ float ldsv_h2f(uint32_t addr) {  // one fp16 from shared memory as float, kept in program order
    unsigned short h;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(addr));
    return __half2float(__ushort_as_half(h));
}
// Transpose of an 8 x 8 matrix of 16-bit elements held by the warp, one 32-bit register per lane: lane (r, c) holds
// the elements (row r, columns 2c and 2c + 1) before and after.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ float ldsp_h2f(uint32_t addr) {  // one fp16 from shared memory as float
    unsigned short h;
    asm("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(addr));
    return __half2float(__ushort_as_half(h));
}

// Split-K merge of one sequence: combines the `parts` partials (acc[128], m, l) of every query head, normalises, and
// multiplies by R^T on the tensor cores (normalised accumulators split into fp16 high + low parts as the A operand, R^T
// as B).  Run by NW warps (`head` = warp index among them) that share the named barrier `bar_group` and the staging
// area `merge_s` ([2][16][MERGE_ROW] halves of shared memory).  part0: the first part's rows, [H][PART_STRIDE]; parts
// follow each other H * PART_STRIDE floats apart.  out_row(h) / out_row_f32(h): where head h's 128 outputs go, or null.
template <int NW, typename OutRow, typename OutRowF32>
__device__ __forceinline__ void merge_sequence(const float* part0, int parts, int H, uint32_t merge_s, const __half* rotation_t,
                                               int head, int lane, int bar_group, int nthreads, OutRow out_row,
                                               OutRowF32 out_row_f32, bool rotated_out = false) {
    const int gl = lane >> 2, t4 = lane & 3;
    for (int hb = 0; hb < H; hb += 16) {
        // ---- phase A: heads hb .. hb+15, two heads per warp at a time with all their loads in flight
        //      together: combine the parts, normalise, split into fp16 high + low, store as the A operand
        //      [16][MERGE_ROW]
        for (int hh0 = head; hh0 < 16; hh0 += 2 * NW) {
            float4 a[2];
            a[0] = a[1] = make_float4(0.f, 0.f, 0.f, 0.f);
            const size_t pstride = (size_t)H * PART_STRIDE;
            if (parts <= 8) {
                // common case: one round trip for everything, weights afterwards
                float4 v[2][8];
                float2 ml[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int hq = hb + hh0 + r * NW;
                    const float* base = part0 + (size_t)hq * PART_STRIDE;
                    const bool on = hq < H && hh0 + r * NW < 16;
                    ml[r] = make_float2(-1e30f, 0.0f);
                    if (on && lane < parts) ml[r] = __ldcg(reinterpret_cast<const float2*>(base + lane * pstride + HEAD_DIM));
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        v[r][j] = (on && j < parts) ? __ldcg(reinterpret_cast<const float4*>(base + j * pstride) + lane)
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float M = ml[r].x;
#pragma unroll
                    for (int o = 4; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
                    M = __shfl_sync(0xffffffffu, M, 0);
                    const float e = lane < parts ? ex2_approx(ml[r].x - M) : 0.0f;
                    float Z = ml[r].y * e;
#pragma unroll
                    for (int o = 4; o > 0; o >>= 1) Z += __shfl_xor_sync(0xffffffffu, Z, o);
                    Z = __shfl_sync(0xffffffffu, Z, 0);
                    const float sc = e / (Z + 1e-8f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float wj = __shfl_sync(0xffffffffu, sc, j);
                        a[r].x = fmaf(wj, v[r][j].x, a[r].x); a[r].y = fmaf(wj, v[r][j].y, a[r].y);
                        a[r].z = fmaf(wj, v[r][j].z, a[r].z); a[r].w = fmaf(wj, v[r][j].w, a[r].w);
                    }
                }
            } else {
                // many parts: one round trip for all (max, sum) pairs, then the vectors 16 at a time
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int hq = hb + hh0 + r * NW;
                    if (hq >= H || hh0 + r * NW >= 16) continue;
                    const float* base = part0 + (size_t)hq * PART_STRIDE;
                    float M = -1e30f, Z = 0.0f, m0 = -1e30f;  // m0: the max of part `lane` (parts 0 .. 31)
                    for (int j0 = 0; j0 < parts; j0 += 32) {
                        float2 t = make_float2(-1e30f, 0.0f);
                        if (j0 + lane < parts) t = __ldcg(reinterpret_cast<const float2*>(base + (j0 + lane) * pstride + HEAD_DIM));
                        if (j0 == 0) m0 = t.x;
                        const float Mn = fmaxf(M, t.x);
                        Z = Z * ex2_approx(M - Mn) + t.y * ex2_approx(t.x - Mn);
                        M = Mn;
                    }
                    float Mw = M;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) Mw = fmaxf(Mw, __shfl_xor_sync(0xffffffffu, Mw, o));
                    Z *= ex2_approx(M - Mw);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) Z += __shfl_xor_sync(0xffffffffu, Z, o);
                    const float inv = 1.0f / (Z + 1e-8f);
                    for (int j0 = 0; j0 < parts; j0 += 32) {
                        float mj = m0;
                        if (j0 > 0) mj = j0 + lane < parts ? __ldcg(base + (j0 + lane) * pstride + HEAD_DIM) : -1e30f;
                        const float sc = j0 + lane < parts ? ex2_approx(mj - Mw) * inv : 0.0f;
#pragma unroll 1
                        for (int j1 = j0; j1 < parts && j1 < j0 + 32; j1 += 16) {
                            float4 v[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                v[j] = j1 + j < parts ? __ldcg(reinterpret_cast<const float4*>(base + (j1 + j) * pstride) + lane)
                                                      : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const float wj = __shfl_sync(0xffffffffu, sc, (j1 - j0) + j);
                                a[r].x = fmaf(wj, v[j].x, a[r].x); a[r].y = fmaf(wj, v[j].y, a[r].y);
                                a[r].z = fmaf(wj, v[j].z, a[r].z); a[r].w = fmaf(wj, v[j].w, a[r].w);
                            }
                        }
                    }
                }
            }
            if (rotated_out) {
                // the consumer's weights carry R^T (tq_fold_rotation_into_projection): the normalised sums leave as they are
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int hh = hh0 + r * NW;
                    if (hh >= 16) continue;
                    if (__half* o = out_row(hb + hh)) {
                        const __half2 h01 = __floats2half2_rn(a[r].x, a[r].y), h23 = __floats2half2_rn(a[r].z, a[r].w);
                        *reinterpret_cast<uint2*>(o + 4 * lane) = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
                    }
                    if (float* o = out_row_f32(hb + hh)) *reinterpret_cast<float4*>(o + 4 * lane) = a[r];
                }
                continue;
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int hh = hh0 + r * NW;
                if (hh >= 16) continue;
                __half2 h01 = __floats2half2_rn(a[r].x, a[r].y), h23 = __floats2half2_rn(a[r].z, a[r].w);
                float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
                const uint32_t dst = merge_s + (uint32_t)(hh * MERGE_ROW + 4 * lane) * 2u;
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(dst), "r"(*reinterpret_cast<uint32_t*>(&h01)),
                             "r"(*reinterpret_cast<uint32_t*>(&h23)) : "memory");
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(dst + 16u * MERGE_ROW * 2u),
                             "r"(pack_half2(a[r].x - f01.x, a[r].y - f01.y)), "r"(pack_half2(a[r].z - f23.x, a[r].w - f23.y)) : "memory");
            }
        }
        if (rotated_out) continue;
        // ---- phase B: out[h][d] = sum_k a[h][k] * R[k][d]  ==  A(16 x 128) * B with B[k][n=d] = rotation_t[d][k].
        //      Two column blocks of 8 per warp and pass; their B fragments are fetched before the barrier so that
        //      the round trip overlaps the other warps' phase A.
        for (int nb0 = head; nb0 < 16; nb0 += 2 * NW) {
            uint32_t bfrag[2][8][2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int nb = nb0 + i * NW;
                const __half* rt = rotation_t + (size_t)(8 * (nb < 16 ? nb : 0) + gl) * HEAD_DIM + 2 * t4;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    bfrag[i][j][0] = __ldg(reinterpret_cast<const unsigned int*>(rt + 16 * j));
                    bfrag[i][j][1] = __ldg(reinterpret_cast<const unsigned int*>(rt + 16 * j + 8));
                }
            }
            if (nb0 == head) group_barrier(bar_group, nthreads);  // phase A of every warp is in shared memory
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int nb = nb0 + i * NW;
                if (nb >= 16) continue;
                float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t r0 = merge_s + (uint32_t)(gl * MERGE_ROW + 16 * j + 2 * t4) * 2u;
                    const uint32_t r8 = r0 + 8u * MERGE_ROW * 2u;
                    const uint32_t lo_off = 16u * MERGE_ROW * 2u;
                    mma16816(c, lds32(r0), lds32(r8), lds32(r0 + 16u), lds32(r8 + 16u), bfrag[i][j][0], bfrag[i][j][1]);
                    mma16816(c, lds32(r0 + lo_off), lds32(r8 + lo_off), lds32(r0 + lo_off + 16u), lds32(r8 + lo_off + 16u),
                             bfrag[i][j][0], bfrag[i][j][1]);
                }
                const int d = 8 * nb + 2 * t4;
                if (__half* o = out_row(hb + gl))
                    *reinterpret_cast<__half2*>(o + d) = __floats2half2_rn(c[0], c[1]);
                if (__half* o = out_row(hb + gl + 8))
                    *reinterpret_cast<__half2*>(o + d) = __floats2half2_rn(c[2], c[3]);
                if (float* o = out_row_f32(hb + gl)) *reinterpret_cast<float2*>(o + d) = make_float2(c[0], c[1]);
                if (float* o = out_row_f32(hb + gl + 8)) *reinterpret_cast<float2*>(o + d) = make_float2(c[2], c[3]);
            }
        }
        group_barrier(bar_group, nthreads);  // the A operand may be overwritten (next 16 heads, next segment)
    }
}

// MODE 0: queries pre-rotated and tile table built by append_rotate_kernel; 1: the kernel builds its table, rotates the
// queries, optionally appends the step's token (one launch per layer and step); 2: whole-step form, see AttnParams.
template <int BITS, int HKV, int MODE>
__global__ void __launch_bounds__(ATTN_GROUPS * 32 * HKV, 1)
decode_attention_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const AttnParams p) {
    using Geo = AttnGeom<BITS>;
    constexpr bool FUSED = MODE >= 1;
    constexpr bool PERSIST = MODE == 2;
    extern __shared__ __align__(1024) uint8_t dyn_smem[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    constexpr int Hkv = HKV;  // compile time: row pitches, tile sizes and norm strides fold into immediates
    const int group = warp / Hkv;        // worker within the CTA
    const int head = warp - group * Hkv; // KV head of this warp
    const int gl = lane >> 2;            // mma "group id": token (K side), coordinate row (V side), head (S layout)
    const int t4 = lane & 3;             // mma "thread in group"
    const int grp = p.H / Hkv;           // query heads per KV head (<= 8)
    constexpr int gthreads = 32 * Hkv;   // threads of a worker
    const int gtid = tid - group * gthreads;
    constexpr uint32_t kvp = (uint32_t)Hkv * Geo::BPH;               // code bytes per token row (all heads)
    constexpr uint32_t code_tile = TILE_TOKENS * kvp;                // one K (or V) tile
    constexpr uint32_t norm_tile = TILE_TOKENS * (uint32_t)Hkv * 2u; // one norm tile
    // a stage starts on a 1024-byte boundary: the 128-byte swizzle of the tensor-map copies goes by the shared address
    constexpr uint32_t stage_bytes = (2u * code_tile + 2u * norm_tile + 1023u) & ~1023u;

    // ---- shared memory map (absolute shared addresses) ----
    const uint32_t dyn_base = smem_u32(dyn_smem);
    const uint32_t a_base = (dyn_base + 1023u) & ~1023u;
    const uint32_t blocks_a = (a_base + (FUSED ? RegionA::FUSED_BLOCKS_OFF : RegionA::BLOCKS_OFF) + 1023u) & ~1023u;
    const uint32_t n_a = blocks_a < LUT_ABS ? (LUT_ABS - blocks_a) / stage_bytes : 0u;
    const uint32_t dyn_end = dyn_base + (uint32_t)ATTN_DYN_SMEM;
    const uint32_t n_b = dyn_end > REGION_B_ABS ? (dyn_end - REGION_B_ABS) / stage_bytes : 0u;
    const int s_fit = (int)((n_a + n_b) / ATTN_GROUPS);
    // 4-bit: a power of two (stage index and parity are masks and shifts).  2-bit stages are half the size and three of
    // them fit where two 4-bit ones do: there the index and the parity are carried along instead.
    const int S = s_fit >= 4 ? 4 : ((BITS == 2 && s_fit == 3) ? 3 : 2);
    const int s_log = s_fit >= 4 ? 2 : 1;
    auto stage_addr = [&](int s) -> uint32_t {
        const uint32_t blk = (uint32_t)(group * S + s);
        return blk < n_a ? blocks_a + blk * stage_bytes : REGION_B_ABS + (blk - n_a) * stage_bytes;
    };
    bool layout_ok = !(blocks_a >= LUT_ABS || s_fit < 2 || dyn_end < REGION_B_ABS);
    if (!layout_ok) {
        if (tid == 0) atomicMax(p.status, ST_SMEM_LAYOUT);
        return;
    }
    // two barriers and two done-counters per stage: the K part (codes + norms) and the V part are filled, waited for
    // and handed back separately, so that a stage's K half is on its way again while its V half is still being read
    const uint32_t bar0 = a_base + RegionA::BAR_OFF + (uint32_t)group * (ATTN_MAX_STAGES * 16u);
    const uint32_t cnt0 = a_base + RegionA::CNT_OFF + (uint32_t)group * (ATTN_MAX_STAGES * 8u);
    const uint32_t ctrl_s = a_base + RegionA::CTRL_OFF + (uint32_t)group * 16u;
    const uint32_t merge_s = a_base + RegionA::MERGE_OFF + (uint32_t)group * RegionA::MERGE_GROUP_BYTES;

    // The fused form lets its successor start only once it has itself seen its predecessor finish (see `early`).
    if (!FUSED) pdl_launch_dependents();
    if (TQ_DBG(32)) { pdl_wait(); pdl_launch_dependents(); return; }
    const int G = p.G;

    // ---- byte -> centroid table, one column per lane ----
    if (TQ_DBG(16)) {
    } else if (BITS == 4) {
        for (int idx = tid; idx < 256 * 32; idx += blockDim.x) {
            int v = idx >> 5, l = idx & 31;
            uint32_t val = pack_half2(kCent4[v & 15], kCent4[v >> 4]);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(LUT_ABS + (uint32_t)v * 256u + (uint32_t)l * 4u), "r"(val) : "memory");
        }
    } else {
        for (int idx = tid; idx < 256 * 32; idx += blockDim.x) {
            int v = idx >> 5, l = idx & 31;
            // (c0, c2), (c1, c3): the low and the high nibble each give one value to either word.  For K a byte is four
            // coordinates of one token (the query fragments are packed in the same order); for V a byte is put together
            // from the nibbles of two tokens, and either word is then one coordinate of that token pair.
            uint32_t lo2 = pack_half2(kCent2[v & 3], kCent2[(v >> 4) & 3]);
            uint32_t hi2 = pack_half2(kCent2[(v >> 2) & 3], kCent2[(v >> 6) & 3]);
            asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(LUT_ABS + (uint32_t)v * 256u + (uint32_t)l * 8u),
                         "r"(lo2), "r"(hi2) : "memory");
        }
    }
    if (gtid == 0) {
        for (int s = 0; s < 2 * ATTN_MAX_STAGES; ++s) {
            mbar_init(bar0 + 8u * s, 1);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(cnt0 + 4u * s), "r"(0u) : "memory");
        }
        if (PERSIST) mbar_init(a_base + 320u + 8u * (uint32_t)group, 1);
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    // Everything above touches only shared memory and may overlap the tail of the previous kernel in the stream.
    const bool early = FUSED && p.early != 0;
    if (!early) {
        pdl_wait();
        if (FUSED) pdl_launch_dependents();
    }
    // Tile table.  The fused form builds it here, in shared memory, from the positions (every CTA the same table);
    // the plain form reads the one the append kernel left in the workspace.
    const int* ts;
    if constexpr (FUSED) {
        int* ts_s = reinterpret_cast<int*>(dyn_smem + (a_base - dyn_base) + RegionA::FUSED_TS_OFF);
        int* scan_s = reinterpret_cast<int*>(dyn_smem + (a_base - dyn_base) + RegionA::FUSED_SCAN_OFF);
        int carry = 0;
        for (int base = 0; base < G; base += (int)blockDim.x) {
            const int gq = base + tid;
            int n = 0;
            if (gq < G) {
                int pos = p.positions ? p.positions[gq] : p.pos_value;
                if (pos < 0) pos = 0;
                n = (pos + TILE_TOKENS) / TILE_TOKENS;
            }
            int incl = n;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += v;
            }
            if (lane == 31) scan_s[warp] = incl;
            __syncthreads();
            int before = 0, all = 0;
            for (int w2 = 0; w2 < (int)(blockDim.x >> 5); ++w2) {
                const int v = scan_s[w2];
                before += (w2 < warp) ? v : 0;
                all += v;
            }
            if (gq < G) ts_s[gq] = carry + before + incl - n;
            carry += all;
            __syncthreads();
        }
        if (tid == 0) ts_s[G] = carry;
        ts = ts_s;
        if constexpr (PERSIST) {
            if (blockIdx.x == 0) {  // the merge kernel reads the table from global memory
                __syncthreads();
                for (int i = tid; i <= G; i += (int)blockDim.x) p.table_out[i] = ts_s[i];
            }
        }
    } else {
        ts = p.tile_start;
    }
    __syncthreads();
    const long long N = ts[G];

    // ---- work slice of this worker ----
    // At most min(workers, N) workers take part, so that every participant owns at least one tile: the ticket
    // count of a sequence is then simply (last owner - first owner + 1).  Fewer when the list is short.
    const long long w_all = (long long)gridDim.x * ATTN_GROUPS;
    const int W = attention_workers(w_all, N, G, TQ_DBG_FACTOR ? TQ_DBG_FACTOR : 16);
    const int wid = blockIdx.x * ATTN_GROUPS + group;
    if (PERSIST && blockIdx.x == 0 && tid == 0) {
        p.table_out[G + 1] = W;
        p.table_out[G + 2] = (int)N;
    }
    if (wid >= W) return;  // uniform for the worker; no CTA-wide barrier follows
    // The flat list is cut in UNITS: a tile is one unit, except the last tile of a sequence, which counts 1 + A units
    // for what a sequence costs beside its tiles (A = p.app_weight, in tiles): in the fused form its owner also appends
    // the sequence's new token; in the prefill form sequences are short and their partials and merges weigh as much
    // as their tiles.  Sequence g starts at unit ts[g] + g*A; a tile belongs to the worker its first unit falls to.
    const long long A = (long long)p.app_weight;
    const long long U = N + (long long)G * A;
    long long lo, hi;
    int g;
    if (FUSED || A > 0) {
        auto tiles_before = [&](long long x, int* gfirst) -> long long {  // tiles whose first unit is below unit x
            if (x >= U) { *gfirst = G; return N; }
            int a = 0, b = G;  // invariant: unit start of a <= x < unit start of b
            while (b - a > 1) {
                const int mid = (a + b) >> 1;
                if ((long long)ts[mid] + mid * A <= x) a = mid; else b = mid;
            }
            const long long off = x - ((long long)ts[a] + a * A), n = ts[a + 1] - ts[a];
            *gfirst = off >= n ? a + 1 : a;
            return ts[a] + (off < n ? off : n);
        };
        int g_hi;
        lo = tiles_before((long long)wid * U / W, &g);
        hi = tiles_before((long long)(wid + 1) * U / W, &g_hi);
        if (lo >= hi) return;  // the worker's units all lie inside an append's share: nothing to do
    } else {
        lo = (long long)wid * N / W;
        hi = (long long)(wid + 1) * N / W;
        // first sequence of the slice: largest g with tile_start[g] <= lo
        if (p.worker_g && !TQ_DBG_FACTOR) {
            g = p.worker_g[wid];
        } else {
            int a = 0, b = G;  // invariant: tile_start[a] <= lo < tile_start[b]
            while (b - a > 1) {
                int mid = (a + b) >> 1;
                if ((long long)ts[mid] <= lo) a = mid; else b = mid;
            }
            g = a;
        }
    }

    // ---- load cursor over the flat tile list (warp-uniform, advanced in step by every warp of the worker) ----
    // Tile counts and row numbers fit 32 bits (the host refuses caches of 2^31 rows or more).
    const int lo_i = (int)lo, hi_i = (int)hi;
    int cl_tile = lo_i;                         // next tile to load into shared memory
    int cl_g = g;
    int cl_gend = ts[g + 1];
    // first cache row of tile j of sequence gq (j counted from the sequence's first tile)
    auto tile_row = [&](int gq, int j) -> int {
        if (p.prefix_tiles && j < p.prefix_tiles[gq]) return (int)p.prefix_base[gq] + j * TILE_TOKENS;
        return (int)(p.row_base ? p.row_base[gq] : (long long)gq * p.max_seq_len) + j * TILE_TOKENS;
    };
    const int row_lo = tile_row(g, lo_i - ts[g]);
    int cl_switch = p.prefix_tiles ? ts[g] + p.prefix_tiles[g] : -1;  // flat index of the current sequence's first private tile
    int cl_row = row_lo;
    int cl_layer = 0;                           // whole-step form: layer (relative to layer0) the cursor is in
    const int g_lo = g;
    const int n_layers = PERSIST ? p.n_layers : 1;
    auto cursor_advance = [&]() {
        ++cl_tile;
        cl_row += TILE_TOKENS;
        if (PERSIST && cl_tile == hi_i) {  // the same slice again, one layer on
            ++cl_layer;
            cl_tile = lo_i;
            cl_g = g_lo;
            cl_gend = ts[g_lo + 1];
            cl_row = row_lo;
            if (p.prefix_tiles) cl_switch = ts[g_lo] + p.prefix_tiles[g_lo];
        } else if (cl_tile == cl_gend && cl_tile < hi_i) {
            ++cl_g;
            cl_gend = ts[cl_g + 1];
            cl_row = tile_row(cl_g, 0);
            if (p.prefix_tiles) cl_switch = cl_tile + p.prefix_tiles[cl_g];
        } else if (cl_tile == cl_switch) {  // from the shared prefix into the sequence's own rows
            cl_row = tile_row(cl_g, cl_tile - ts[cl_g]);
        }
    };
    auto cursor_more = [&]() -> bool { return PERSIST ? cl_layer < n_layers : cl_tile < hi_i; };
    // whole-step form: the rotated queries of a segment's sequence arrive by a bulk copy into the (otherwise idle) merge
    // area of the worker, completion on a barrier of their own; the copy for the next segment goes out as soon as every
    // warp has taken its fragments of the current one
    const uint32_t qbar = a_base + 320u + 8u * (uint32_t)group;
    const uint32_t q_block_bytes = (uint32_t)p.H * HEAD_DIM * 2u;
    uint32_t q_par = 0;
    auto issue_queries = [&](int layer, int gq) {
        mbar_arrive_expect_tx(qbar, q_block_bytes);
        bulk_load(merge_s, p.q_rot16 + ((size_t)layer * p.G + (size_t)gq) * (size_t)p.H * HEAD_DIM, q_block_bytes, qbar);
    };
    int consumed = 0;
    int s_idx = 0;          // 2-bit form: stage of the tile being consumed and the parity of its barrier
    uint32_t s_par = 0;
    bool dead = false;  // a bounded wait gave up: keep the control flow, stop touching the pipeline
    const bool loads_on = !TQ_DBG(2);
    const int total_rows_i = (int)p.total_rows;

    // One elected thread issues the two copies of a tile's K part (codes, norms) or V part, clipped to the end of the
    // arrays; rows past a sequence's position only ever reach masked tokens.
    auto issue_part = [&](int row, int s, int part, int layer) {
        int nrows = total_rows_i - row;
        if (nrows > TILE_TOKENS) nrows = TILE_TOKENS;
        if (nrows < 0) nrows = 0;
        const uint32_t nb = (uint32_t)nrows * (uint32_t)Hkv * 2u;
        const uint32_t bar = bar0 + 16u * s + 8u * part;
        const uint32_t dst = stage_addr(s);
        // a tensor-map box always delivers its full size (rows past the end of the array arrive as zeros)
        mbar_arrive_expect_tx(bar, code_tile + nb);
        const size_t noff = (size_t)row * Hkv + (PERSIST ? (size_t)layer * (size_t)p.norm_layer_stride : (size_t)0);
        if (part == 0) {
            if (PERSIST) tma_load_4d(dst, &tmK, bar, 0, row, 0, p.layer0 + layer);
            else tma_load_3d(dst, &tmK, bar, 0, row, 0);
            if (nrows > 0) bulk_load(dst + 2u * code_tile, p.kn + noff, nb, bar);
        } else {
            if (PERSIST) tma_load_4d(dst + code_tile, &tmV, bar, 0, row, 0, p.layer0 + layer);
            else tma_load_3d(dst + code_tile, &tmV, bar, 0, row, 0);
            if (nrows > 0) bulk_load(dst + 2u * code_tile + norm_tile, p.vn + noff, nb, bar);
        }
    };
    auto issue_tile = [&](int row, int s, int layer) {
        issue_part(row, s, 0, layer);
        issue_part(row, s, 1, layer);
    };
    // L2 prefetch of the tile ATTN_L2_AHEAD further on, when it belongs to the same sequence (rows are then contiguous)
    auto prefetch_ahead = [&](int row, int tile_idx, int gend) {
        if (tile_idx + p.l2_ahead < gend && tile_idx + p.l2_ahead < hi_i) {  // own slice only: others fetch theirs
            const int prow = row + p.l2_ahead * TILE_TOKENS;
            int nrows = total_rows_i - prow;
            if (nrows > TILE_TOKENS) nrows = TILE_TOKENS;
            if (nrows > 0) {
                bulk_prefetch_l2(p.ck + (size_t)prow * kvp, (uint32_t)nrows * kvp);
                bulk_prefetch_l2(p.cv + (size_t)prow * kvp, (uint32_t)nrows * kvp);
            }
        }
    };
    auto fill_ring = [&]() {  // prologue: fill the ring (and prefetch a few tiles beyond each)
        for (int s = 0; s < S; ++s) {
            if (cursor_more()) {
                if (gtid == 0 && loads_on) {
                    issue_tile(cl_row, s, cl_layer);
                    prefetch_ahead(cl_row, cl_tile, cl_gend);
                }
                cursor_advance();
            }
        }
    };
    if (PERSIST && gtid == 0 && loads_on) issue_queries(0, g);
    if constexpr (FUSED) {
        // The new token of a sequence is appended by the worker that owns the sequence's last tile (the only tile the
        // row can be in), before that tile is fetched.  The rotation of the sequence's 2 * Hkv head vectors runs on the
        // tensor cores (16 rows x 128 x 128, fp16 hi/lo operands as in the prefill kernel); a coordinate within
        // APPEND_MARGIN of a decision bound is recomputed with the reference's exact fp32 chain, so that the stored
        // bytes are the reference's.  The ring is filled first unless one of its tiles is the tile being written.
        int g_app0 = g;  // first sequence whose last tile starts at or after lo
        while (g_app0 < G && ts[g_app0 + 1] - 1 < lo_i) ++g_app0;
        // (without new keys and values the launch only builds its table, rotates the queries and attends)
        const bool have_app = !PERSIST && p.new_k != nullptr && g_app0 < G && ts[g_app0 + 1] - 1 < hi_i;
        const bool fill_before = !have_app || ts[g_app0 + 1] - 1 >= lo_i + S;
        if (early) {
            // none of the tiles filled here can hold a row the step is about to write
            if (fill_before) fill_ring();
            pdl_wait();
            pdl_launch_dependents();
        } else if (fill_before) {
            fill_ring();
        }
        if (have_app) {
            constexpr float APPEND_MARGIN = 1.6e-5f;  // twice the worst-case rounding of a 128-term fp32 sum with sum|r x| <= 1
            constexpr int NVEC = 2 * Hkv;              // head vectors of one token: K heads, then V heads
            const uint32_t hi_a = merge_s, lo_a = merge_s + 16u * MERGE_ROW * 2u;  // A operands [16][MERGE_ROW] fp16 (idle merge area)
            const uint32_t app_a = a_base + RegionA::FUSED_APP_OFF + (uint32_t)group * RegionA::FUSED_APP_GROUP_BYTES;
            const uint32_t codes_a = app_a, inv_a = app_a + 2048u;  // codes [16][128] u8, 1/norm [16] f32
            const uint32_t qcnt_a = app_a + 2112u, queue_a = app_a + 2128u;  // near-bound coordinates: count, [APPEND_QUEUE] items
            constexpr uint32_t APPEND_QUEUE = 64;
            const __half* rot_w = p.rotation + (size_t)(wid % p.rot_copies) * (HEAD_DIM * HEAD_DIM);
            for (int ga = g_app0; ga < G && ts[ga + 1] - 1 < hi_i; ++ga) {
                const int pos = p.positions ? p.positions[ga] : p.pos_value;
                const int cap = p.seq_capacity ? p.seq_capacity[ga] : p.capacity_rows;
                const bool ok = pos >= 0 && (cap <= 0 || pos < cap);
                const long long row = (p.row_base ? p.row_base[ga] : (long long)ga * p.max_seq_len) + pos;
                // B fragments (R), 16 bytes per lane and load, contraction index permuted as in the query rotation
                uint4 bq[16 / Hkv][4];
#pragma unroll
                for (int nbi = 0; nbi < 16 / Hkv; ++nbi) {
                    const uint4* rr = reinterpret_cast<const uint4*>(rot_w + (size_t)(8 * (head + nbi * Hkv) + gl) * HEAD_DIM) + t4;
#pragma unroll
                    for (int m = 0; m < 4; ++m) bq[nbi][m] = __ldg(rr + 4 * m);
                }
                if (gtid == gthreads - 1) asm volatile("st.shared.u32 [%0], %1;" ::"r"(qcnt_a), "r"(0u) : "memory");
                // ---- thread (vector v, 32-coordinate chunk c): sum of squares in the reference's order, norm, hi/lo ----
                if (gtid < NVEC * 4) {
                    const int v = gtid >> 2, c = gtid & 3;
                    const uint4* src = reinterpret_cast<const uint4*>((v < Hkv ? p.new_k : p.new_v) + (size_t)ga * p.kv_dim +
                                                                      (size_t)(v % Hkv) * HEAD_DIM + 32 * c);
                    uint4 raw[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) raw[i] = __ldg(src + i);
                    float val[32], sq[32];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const __half2* h2 = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __half22float2(h2[e]);
                            val[8 * i + 2 * e] = f.x;
                            val[8 * i + 2 * e + 1] = f.y;
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) sq[i] = mul_ftz(val[i], val[i]);
                    // the warp-shuffle tree of the reference (offsets 16, 8, 4, 2, 1), element l taking lane l's place
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                        for (int l = 0; l < off; ++l) sq[l] = add_ftz(sq[l], sq[l + off]);
                    const float part = sq[0];
                    const int l0 = lane & ~3;
                    const float p0 = __shfl_sync(0xffffffffu, part, l0), p1 = __shfl_sync(0xffffffffu, part, l0 + 1);
                    const float p2 = __shfl_sync(0xffffffffu, part, l0 + 2), p3 = __shfl_sync(0xffffffffu, part, l0 + 3);
                    const float tt = add_ftz(add_ftz(add_ftz(p0, p2), add_ftz(p1, p3)), 1e-12f);
                    const float inv = rsqrt_approx_ftz(tt);
                    if (c == 0) {
                        asm volatile("st.shared.f32 [%0], %1;" ::"r"(inv_a + (uint32_t)v * 4u), "f"(inv) : "memory");
                        if (ok) {
                            __half* cn = const_cast<__half*>(v < Hkv ? p.kn : p.vn);
                            cn[(size_t)row * Hkv + (v % Hkv)] = __float2half_rn(sqrt_approx_ftz(tt));
                        } else if (v == 0) {
                            atomicMax(p.status, ST_BAD_POSITION);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {  // 8 coordinates = 16 bytes at a time
                        uint32_t hw[4], lw[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float x0 = mul_ftz(val[8 * i + 2 * e], inv), x1 = mul_ftz(val[8 * i + 2 * e + 1], inv);
                            const __half2 h = __floats2half2_rn(x0, x1);
                            const float2 hf = __half22float2(h);
                            hw[e] = *reinterpret_cast<const uint32_t*>(&h);
                            lw[e] = pack_half2((x0 - hf.x) * 4096.0f, (x1 - hf.y) * 4096.0f);
                        }
                        const uint32_t o = (uint32_t)(v * MERGE_ROW + 32 * c + 8 * i) * 2u;
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(hi_a + o), "r"(hw[0]), "r"(hw[1]), "r"(hw[2]), "r"(hw[3]) : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(lo_a + o), "r"(lw[0]), "r"(lw[1]), "r"(lw[2]), "r"(lw[3]) : "memory");
                    }
                } else if (NVEC < 16) {
                    // fewer than 16 vectors: rows NVEC .. 15 of both operands are zero (16-byte pieces, 17 per row)
                    for (int i = gtid - NVEC * 4; i < (16 - NVEC) * 17; i += gthreads - NVEC * 4) {
                        const uint32_t o = (uint32_t)((NVEC + i / 17) * MERGE_ROW) * 2u + (uint32_t)(i % 17) * 16u;
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(hi_a + o), "r"(0u) : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(lo_a + o), "r"(0u) : "memory");
                    }
                }
                group_barrier(group, gthreads);
                // ---- rotation on the tensor cores: two accumulators per column block (hi part, scaled lo part) ----
                uint4 ah_lo[4], ah_hi[4], al_lo[4], al_hi[4];  // operand hi / lo, rows gl / gl + 8
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    const uint32_t o0 = (uint32_t)(gl * MERGE_ROW + 32 * m + 8 * t4) * 2u, o8 = o0 + 8u * MERGE_ROW * 2u;
                    ah_lo[m] = ldsv128(hi_a + o0);
                    ah_hi[m] = ldsv128(hi_a + o8);
                    al_lo[m] = ldsv128(lo_a + o0);
                    al_hi[m] = ldsv128(lo_a + o8);
                }
                // the exact chain of the reference for coordinate d of vector v (R row from global, x rebuilt from the input)
                auto exact_code = [&](int v, int d) -> int {
                    const uint4* xs = reinterpret_cast<const uint4*>((v < Hkv ? p.new_k : p.new_v) + (size_t)ga * p.kv_dim +
                                                                     (size_t)(v % Hkv) * HEAD_DIM);
                    const uint4* rs = reinterpret_cast<const uint4*>(rot_w + (size_t)d * HEAD_DIM);
                    float inv;
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(inv) : "r"(inv_a + (uint32_t)v * 4u) : "memory");
                    float acc = 0.0f;
#pragma unroll 2
                    for (int j = 0; j < 16; ++j) {
                        const uint4 xv = __ldg(xs + j), rv = __ldg(rs + j);
                        const __half2* xh = reinterpret_cast<const __half2*>(&xv);
                        const __half2* rh = reinterpret_cast<const __half2*>(&rv);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 xf = __half22float2(xh[e]), rf = __half22float2(rh[e]);
                            acc = fma_ftz(rf.x, mul_ftz(xf.x, inv), acc);
                            acc = fma_ftz(rf.y, mul_ftz(xf.y, inv), acc);
                        }
                    }
                    return quantize_code(acc, BITS);
                };
#pragma unroll
                for (int nbi = 0; nbi < 16 / Hkv; ++nbi) {
                    const int nb = head + nbi * Hkv;
                    float ch[4] = {0.0f, 0.0f, 0.0f, 0.0f}, cl[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        mma16816(ch, ah_lo[m].x, ah_hi[m].x, ah_lo[m].y, ah_hi[m].y, bq[nbi][m].x, bq[nbi][m].y);
                        mma16816(ch, ah_lo[m].z, ah_hi[m].z, ah_lo[m].w, ah_hi[m].w, bq[nbi][m].z, bq[nbi][m].w);
                        mma16816(cl, al_lo[m].x, al_hi[m].x, al_lo[m].y, al_hi[m].y, bq[nbi][m].x, bq[nbi][m].y);
                        mma16816(cl, al_lo[m].z, al_hi[m].z, al_lo[m].w, al_hi[m].w, bq[nbi][m].z, bq[nbi][m].w);
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {  // (row gl, col), (row gl, col + 1), (row gl + 8, col), (row gl + 8, col + 1)
                        const int v = gl + 8 * (e >> 1), d = 8 * nb + 2 * t4 + (e & 1);
                        const float dval = fmaf(cl[e], 1.0f / 4096.0f, ch[e]);
                        int code = quantize_code(dval, BITS);
                        float dist = 3.0e38f;  // distance to the nearest decision bound
                        if (BITS == 4) {
#pragma unroll
                            for (int i = 0; i < 15; ++i) dist = fminf(dist, fabsf(dval - kBnd4[i]));
                        } else {
#pragma unroll
                            for (int i = 0; i < 3; ++i) dist = fminf(dist, fabsf(dval - kBnd2[i]));
                        }
                        if (v < NVEC) {
                            if (dist < APPEND_MARGIN) {  // rare (about 1 coordinate in 700): queued for the exact chain below
                                const uint32_t slot = atom_add_shared(qcnt_a, 1u);
                                if (slot < APPEND_QUEUE)
                                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(queue_a + 4u * slot), "r"((uint32_t)(v << 8 | d)) : "memory");
                                else
                                    code = exact_code(v, d);
                            }
                            asm volatile("st.shared.u8 [%0], %1;" ::"r"(codes_a + (uint32_t)(v * HEAD_DIM + d)), "r"(code) : "memory");
                        }
                    }
                }
                group_barrier(group, gthreads);
                // ---- the exact chain of the reference for the queued coordinates, 8 lanes per item: lane s of a group
                //      prepares terms k = 16 s .. 16 s + 15 (one round trip for everything), then the k-ascending chain
                //      runs through the lanes in order, the running sum handed on by a shuffle ----
                {
                    uint32_t queued;
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(queued) : "r"(qcnt_a) : "memory");
                    queued = queued < APPEND_QUEUE ? queued : APPEND_QUEUE;
                    const int sub = lane & 7;
                    for (uint32_t i0 = (uint32_t)head * 4u; i0 < queued; i0 += (uint32_t)Hkv * 4u) {  // warp-uniform
                        const uint32_t i = i0 + (uint32_t)(lane >> 3);
                        const bool live = i < queued;
                        uint32_t item = 0u;
                        if (live) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(item) : "r"(queue_a + 4u * i) : "memory");
                        const int v = (int)(item >> 8), d = (int)(item & 255u);
                        float xs[16], rr[16];
#pragma unroll
                        for (int e = 0; e < 16; ++e) xs[e] = rr[e] = 0.0f;
                        if (live) {
                            const uint4* xsrc = reinterpret_cast<const uint4*>((v < Hkv ? p.new_k : p.new_v) + (size_t)ga * p.kv_dim +
                                                                               (size_t)(v % Hkv) * HEAD_DIM) + 2 * sub;
                            const uint4* rsrc = reinterpret_cast<const uint4*>(rot_w + (size_t)d * HEAD_DIM) + 2 * sub;
                            float inv;
                            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(inv) : "r"(inv_a + (uint32_t)v * 4u) : "memory");
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const uint4 xv = __ldg(xsrc + j), rv = __ldg(rsrc + j);
                                const __half2* xh = reinterpret_cast<const __half2*>(&xv);
                                const __half2* rh = reinterpret_cast<const __half2*>(&rv);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 xf = __half22float2(xh[e]), rf = __half22float2(rh[e]);
                                    xs[8 * j + 2 * e] = mul_ftz(xf.x, inv);
                                    xs[8 * j + 2 * e + 1] = mul_ftz(xf.y, inv);
                                    rr[8 * j + 2 * e] = rf.x;
                                    rr[8 * j + 2 * e + 1] = rf.y;
                                }
                            }
                        }
                        float acc = 0.0f;
#pragma unroll
                        for (int st = 0; st < 8; ++st) {
                            if (sub == st) {
#pragma unroll
                                for (int e = 0; e < 16; ++e) acc = fma_ftz(rr[e], xs[e], acc);
                            }
                            acc = __shfl_sync(0xffffffffu, acc, (lane & ~7) + st);
                        }
                        if (live && sub == 0)
                            asm volatile("st.shared.u8 [%0], %1;" ::"r"(codes_a + (uint32_t)(v * HEAD_DIM + d)), "r"(quantize_code(acc, BITS)) : "memory");
                    }
                }
                group_barrier(group, gthreads);
                // ---- pack: one 32-bit word (8 four-bit or 16 two-bit codes) per thread; NVEC vectors ----
                {
                    constexpr int words_per_vec = (int)Geo::BPH / 4;
                    for (int wi = gtid; ok && wi < NVEC * words_per_vec; wi += gthreads) {
                        const int vi = wi / words_per_vec, wv = wi - vi * words_per_vec;
                        uint32_t word = 0;
                        if (BITS == 2) {
                            uint4 c4;  // ordered after the barrier: a volatile load, unlike the tile loop's
                            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(c4.x), "=r"(c4.y), "=r"(c4.z), "=r"(c4.w)
                                         : "r"(codes_a + (uint32_t)(vi * HEAD_DIM + 16 * wv)) : "memory");
                            const uint32_t cw[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                            for (int b2 = 0; b2 < 4; ++b2) {
                                const uint32_t x = cw[b2];
                                const uint32_t pk = (x & 3u) | ((x >> 6) & 0xcu) | ((x >> 12) & 0x30u) | ((x >> 18) & 0xc0u);
                                word |= pk << (8 * b2);
                            }
                        } else {
                            uint2 c2;
                            asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(c2.x), "=r"(c2.y)
                                         : "r"(codes_a + (uint32_t)(vi * HEAD_DIM + 8 * wv)) : "memory");
                            const uint32_t cw[2] = {c2.x, c2.y};
#pragma unroll
                            for (int hb2 = 0; hb2 < 2; ++hb2) {
                                const uint32_t x = cw[hb2];
                                const uint32_t pk = (x & 0xfu) | ((x >> 4) & 0xf0u) | ((x >> 8) & 0xf00u) | ((x >> 12) & 0xf000u);
                                word |= pk << (16 * hb2);
                            }
                        }
                        uint8_t* cq = const_cast<uint8_t*>(vi < Hkv ? p.ck : p.cv);
                        *reinterpret_cast<uint32_t*>(cq + (size_t)row * kvp + (size_t)(vi % Hkv) * Geo::BPH + 4 * wv) = word;
                    }
                }
                // the row is read back by tensor-map copies (async proxy) of this worker
                __threadfence();
                fence_proxy_async_all();
                group_barrier(group, gthreads);
            }
            if (gtid == 0) fence_proxy_async_all();
        }
        if (!fill_before) fill_ring();
    } else {
        fill_ring();
    }

    if (TQ_DBG(64)) return;
    const uint32_t lutlane = LUT_ABS | ((uint32_t)lane << (BITS == 4 ? 2 : 3));
    // ---- swizzled addressing.  A box holds [32 rows][128 B]; the 16-byte chunk c of row r sits at chunk c ^ (r & 7).
    // Tokens of an 8-token score block are taken in the order tau(n) = n ^ ((n & 1) << 2), which keeps both the
    // K reads (lane <-> token tau(gl)) and the V reads (lane <-> tokens tau(2*t4), tau(2*t4+1)) conflict free.
    const uint32_t hbyte = (uint32_t)head * Geo::BPH;          // this head's first byte within the token row
    const uint32_t box_off = (hbyte >> 7) * 4096u;              // which box
    const uint32_t hchunk = (hbyte & 127u) >> 4;                // first 16-byte chunk of the head inside the box row
    const uint32_t tauK = (uint32_t)gl ^ (((uint32_t)gl & 1u) << 2);
    const uint32_t tokA = 2u * (uint32_t)t4, tokB = (2u * (uint32_t)t4 + 1u) ^ 4u;   // tau(2*t4), tau(2*t4+1)
    uint32_t k_off, vA_off, vB_off;
    if (BITS == 4) {
        k_off = box_off + tauK * 128u + (((hchunk + (uint32_t)t4) ^ tauK) << 4);
        const uint32_t vch = hchunk + ((uint32_t)gl >> 1), vsub = ((uint32_t)gl & 1u) * 8u;
        vA_off = box_off + tokA * 128u + ((vch ^ tokA) << 4) + vsub;
        vB_off = box_off + tokB * 128u + ((vch ^ tokB) << 4) + vsub;
    } else {
        k_off = box_off + tauK * 128u + (((hchunk + ((uint32_t)t4 >> 1)) ^ tauK) << 4) + ((uint32_t)t4 & 1u) * 8u;
        const uint32_t vch = hchunk + ((uint32_t)gl >> 2), vsub = ((uint32_t)gl & 3u) * 4u;
        vA_off = box_off + tokA * 128u + ((vch ^ tokA) << 4) + vsub;
        vB_off = box_off + tokB * 128u + ((vch ^ tokB) << 4) + vsub;
    }

#ifdef TQ_TIMING_SWITCHES
    long long stamp_acc[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    long long stamp_last = clock64();
#endif
    for (int layer = 0; layer < n_layers; ++layer) {  // (one pass unless this is the whole-step form)
    long long tile = lo;
    g = g_lo;
    while (tile < hi) {
        // ================= one segment: tiles [tile, seg_end) of sequence g =================
        const long long ts_g = ts[g];
        const long long ts_g1 = ts[g + 1];
        const long long seg_end = hi < ts_g1 ? hi : ts_g1;
        const int pos = p.positions ? p.positions[g] : p.pos_value;
        const int L = (pos < 0 ? 0 : pos) + 1;
        // causal limit of this lane's score row (row gl) and of the group's first token; equal to L outside the prefill form
        const int qg = FUSED ? 0 : p.qg;  // the fused form is a decode step: no token groups
        const int grp_real = qg > 1 ? grp / qg : grp;
        // (this lane's score columns are the heads 2*t4 and 2*t4 + 1 of its KV head)
        const int Lcol0 = qg > 1 ? min(L, g * qg + (2 * t4) / grp_real + 1) : L;
        const int Lcol1 = qg > 1 ? min(L, g * qg + (2 * t4 + 1) / grp_real + 1) : L;
        const int Lmin = qg > 1 ? min(L, g * qg + 1) : L;

        TQ_STAMP(8);   // loop tail + publishing of the previous segment + this segment's table / position reads
        // query fragments (B operand of the score product): lane (gl, t4) holds coordinates 32*t4 .. 32*t4+31 of head
        // head*grp + gl as fp16
        uint32_t qb[8][2];
        if constexpr (PERSIST) {
            uint32_t ok = (dead || !loads_on) ? 1u : 0u;
            for (uint32_t it = 0; it < (1u << 14) && !ok; ++it) ok = mbar_try_wait_hint(qbar, q_par, 20000u);
            if (!ok) {
                dead = true;
                if (lane == 0) atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
            }
            dead = __any_sync(0xffffffffu, dead);
            q_par ^= 1u;
            TQ_STAMP(9);   // wait for the query block
            // lane (gl, t4): the 32 coordinates 32*t4 .. of head head*grp + gl, 64 bytes
            uint4 qw[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                qw[i] = make_uint4(0u, 0u, 0u, 0u);
                if (gl < grp && !dead) qw[i] = ldsv128(merge_s + (uint32_t)((head * grp + gl) * HEAD_DIM + 32 * t4 + 8 * i) * 2u);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t w4[4] = {qw[i].x, qw[i].y, qw[i].z, qw[i].w};
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    // step j = 2*i + h2 takes the coordinates 4j .. 4j+3: (4j, 4j+1), (4j+2, 4j+3) -- the 2-bit table
                    // returns the four values of a byte as (0, 2), (1, 3)
                    const uint32_t a = w4[2 * h2], b = w4[2 * h2 + 1];
                    qb[2 * i + h2][0] = BITS == 2 ? prmt(a, b, 0x5410u) : a;
                    qb[2 * i + h2][1] = BITS == 2 ? prmt(a, b, 0x7632u) : b;
                }
            }
            TQ_STAMP(10);  // fragments
            group_barrier(group, gthreads);  // every warp holds its fragments: the area may take the next block
            TQ_STAMP(11);  // barrier of the worker's warps
            if (gtid == 0 && !dead && loads_on) {
                fence_proxy_async_smem();
                if (seg_end < hi) issue_queries(layer, g + 1);
                else if (layer + 1 < n_layers) issue_queries(layer + 1, g_lo);
            }
        } else {
            float qv[32];
            if constexpr (FUSED) {
                // Rotate this sequence's queries here: rot[h][d] = sum_k q[h][k] * R[d][k] on the tensor cores, 16 heads
                // at a time, every warp two (Hkv = 8) or four (Hkv = 4) blocks of 8 coordinates; the result goes through
                // shared memory (the idle merge area) to the lanes that need it, scaled by log2(e) / sqrt(128).
                const uint32_t qs_a = merge_s;  // [16][128] fp32
#pragma unroll
                for (int i = 0; i < 32; ++i) qv[i] = 0.0f;
                for (int hb = 0; hb < p.H; hb += 16) {
                    // 16 query heads (4 KB) into shared memory with one coalesced 16-byte load per thread
                    for (int i = gtid; i < 256; i += gthreads) {
                        const int r = i >> 4;
                        uint4 u = make_uint4(0u, 0u, 0u, 0u);
                        if (hb + r < p.H)
                            u = __ldg(reinterpret_cast<const uint4*>(p.new_q + (PERSIST ? (size_t)layer * (size_t)p.q_layer_stride : (size_t)0) +
                                                                     (size_t)g * p.q_dim + (size_t)(hb + r) * HEAD_DIM) + (i & 15));
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(qs_a + (uint32_t)i * 16u), "r"(u.x), "r"(u.y),
                                     "r"(u.z), "r"(u.w) : "memory");
                    }
                    // B fragments straight from R (16 contiguous bytes per lane and load: whole sectors).  The contraction
                    // index is permuted the same way on both sides: step (m, e) of lane t4 covers k = 32m + 8*t4 + 4e .. +3.
                    uint4 bq[16 / Hkv][4];
#pragma unroll
                    for (int nbi = 0; nbi < 16 / Hkv; ++nbi) {
                        const int nb = head + nbi * Hkv;
                        const uint4* rr = reinterpret_cast<const uint4*>(p.rotation + (size_t)(wid % p.rot_copies) * (HEAD_DIM * HEAD_DIM) +
                                                                         (size_t)(8 * nb + gl) * HEAD_DIM) + t4;
#pragma unroll
                        for (int m = 0; m < 4; ++m) bq[nbi][m] = __ldg(rr + 4 * m);
                    }
                    group_barrier(group, gthreads);
                    uint4 a_lo[4], a_hi[4];  // rows gl and gl + 8
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        a_lo[m] = ldsv128(qs_a + (uint32_t)(gl * HEAD_DIM + 32 * m + 8 * t4) * 2u);
                        a_hi[m] = ldsv128(qs_a + (uint32_t)((gl + 8) * HEAD_DIM + 32 * m + 8 * t4) * 2u);
                    }
                    group_barrier(group, gthreads);  // the staging area turns into the fp32 result area
#pragma unroll
                    for (int nbi = 0; nbi < 16 / Hkv; ++nbi) {
                        const int nb = head + nbi * Hkv;
                        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                        for (int m = 0; m < 4; ++m) {
                            mma16816(c, a_lo[m].x, a_hi[m].x, a_lo[m].y, a_hi[m].y, bq[nbi][m].x, bq[nbi][m].y);
                            mma16816(c, a_lo[m].z, a_hi[m].z, a_lo[m].w, a_hi[m].w, bq[nbi][m].z, bq[nbi][m].w);
                        }
                        const float sc = 0.12751743074602467f;
                        const uint32_t o0 = qs_a + (uint32_t)(gl * HEAD_DIM + 8 * nb + 2 * t4) * 4u;
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(o0), "f"(c[0] * sc), "f"(c[1] * sc) : "memory");
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(o0 + 8u * HEAD_DIM * 4u), "f"(c[2] * sc), "f"(c[3] * sc) : "memory");
                    }
                    group_barrier(group, gthreads);
                    const int myrow = head * grp + gl - hb;
                    if (gl < grp && myrow >= 0 && myrow < 16 && !TQ_DBG(8)) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float4 f;
                            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(f.x), "=f"(f.y), "=f"(f.z), "=f"(f.w)
                                         : "r"(qs_a + (uint32_t)(myrow * HEAD_DIM + 32 * t4 + 4 * i) * 4u) : "memory");
                            qv[4 * i] = f.x; qv[4 * i + 1] = f.y; qv[4 * i + 2] = f.z; qv[4 * i + 3] = f.w;
                        }
                    }
                    group_barrier(group, gthreads);
                }
            } else if (gl < grp && !TQ_DBG(8)) {
                const float4* src =
                    reinterpret_cast<const float4*>(p.q_rot + ((size_t)g * p.H + (size_t)head * grp + gl) * HEAD_DIM + 32 * t4);
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
                // the 2-bit table returns the four values of a byte as (0, 2), (1, 3)
                const float x0 = qv[4 * j], x1 = BITS == 2 ? qv[4 * j + 2] : qv[4 * j + 1];
                const float x2 = BITS == 2 ? qv[4 * j + 1] : qv[4 * j + 2], x3 = qv[4 * j + 3];
                qb[j][0] = pack_half2(x0, x1);
                qb[j][1] = pack_half2(x2, x3);
            }
        }

        // running maximum and (per lane: over its own token rows) sum of the two score columns of this lane
        float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.0f, 0.0f};
        float acc[8][4];
#pragma unroll
        for (int b = 0; b < 8; ++b) { acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.0f; }

        for (; tile < seg_end; ++tile) {
            const int t0 = (int)(tile - ts_g) * TILE_TOKENS;
            const bool full = t0 + TILE_TOKENS <= Lmin;  // warp-uniform: no token of the tile is masked for any row
            const int s = BITS == 2 ? s_idx : (consumed & (S - 1));
            const uint32_t parity = BITS == 2 ? s_par : ((uint32_t)(consumed >> s_log) & 1u);
            // the tile that takes this stage's place (warp-uniform; every warp of the worker advances the cursor in step)
            const int next_row = cl_row, next_tile = cl_tile, next_gend = cl_gend, next_layer = cl_layer;
            const bool more = cursor_more();
            if (more) cursor_advance();
            // Wait for one part (0: K codes and norms, 1: V codes and norms) of the stage.  Returns 0 at run time, as a
            // value PRODUCED by the wait: the part's loads take it into their address and so cannot move above the wait.
            auto wait_part = [&](int part) -> uint32_t {
                uint32_t token = 0;
                if (!dead && loads_on) {
                    const uint32_t bar = bar0 + 16u * s + 8u * part;
                    uint32_t ok = 0;
                    for (uint32_t it = 0; it < (1u << 14) && !ok; ++it) ok = mbar_try_wait_hint(bar, parity, 20000u);
                    if (!ok) {
                        dead = true;
                        if (lane == 0) atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
                    }
                    dead = __any_sync(0xffffffffu, dead);
                    token = ok ^ 1u;
                }
                return token;
            };
            // Hand a part back: everything this warp read from it has been consumed by (ordered) instructions above.  The
            // last warp of the worker to get here re-arms the part with the same part of the tile S ahead; nobody waits.
            auto release_part = [&](int part) {
                __syncwarp();
                if (lane == 0 && more && !dead && loads_on) {
                    __threadfence_block();  // this warp's reads of the part are ordered before the hand-over below
                    const uint32_t cnt = cnt0 + 8u * s + 4u * part;
                    const uint32_t old = atom_add_shared(cnt, 1u);
                    if (old == (uint32_t)Hkv - 1u) {
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(cnt), "r"(0u) : "memory");
                        fence_proxy_async_smem();
                        issue_part(next_row, s, part, next_layer);
                        if (part == 1) prefetch_ahead(next_row, next_tile, next_gend);
                    }
                }
            };
            // The tile body exists twice: for tiles in which every token is attended to (all but the last tile of a
            // sequence) without any masking code, and for the last, partly filled tile with it.
            auto tile_body = [&](auto full_tag) {
                constexpr bool FULLT = decltype(full_tag)::value;
                constexpr uint32_t nstride = (uint32_t)Hkv * 2u;
                TQ_STAMP(0);
                const uint32_t tokK = wait_part(0);
                TQ_STAMP(1);
                if (dead) return;
                const uint32_t kt = stage_addr(s) + tokK;
                const uint32_t kns = kt + 2u * code_tile + (uint32_t)head * 2u;

                // ---------------- scores: S^T = K (16 token rows x 16 coordinates) * Q^T (16 coordinates x 8 heads), two
                // blocks of 16 token rows.  Row r of block rb is token 16*rb + 8*(r >> 3) + tau(r & 7) of the tile; the
                // eight 16-coordinate steps of a row block form one accumulator chain.
                float c[2][4];
                {
                    uint32_t w[4][4];
#pragma unroll
                    for (int blk = 0; blk < 4; ++blk) {
                        if (BITS == 4) {
                            const uint4 kw = ldsp128(kt + (uint32_t)blk * 1024u + k_off);
                            w[blk][0] = kw.x; w[blk][1] = kw.y; w[blk][2] = kw.z; w[blk][3] = kw.w;
                        } else {
                            const uint2 kw = ldsp64(kt + (uint32_t)blk * 1024u + k_off);
                            w[blk][0] = kw.x; w[blk][1] = kw.y; w[blk][2] = w[blk][3] = 0u;
                        }
                    }
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb) c[rb][0] = c[rb][1] = c[rb][2] = c[rb][3] = 0.0f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
#pragma unroll
                        for (int rb = 0; rb < 2; ++rb) {
                            uint32_t a0, a1, a2, a3;  // rows gl / gl + 8, coordinate pairs (4j, 4j+1) / (4j+2, 4j+3) of the lane's 32
                            if (BITS == 4) {
                                const uint32_t sel0 = (j & 1) ? 0x7624u : 0x7604u, sel1 = (j & 1) ? 0x7634u : 0x7614u;
                                const uint32_t wlo = w[2 * rb][j >> 1], whi = w[2 * rb + 1][j >> 1];
                                a0 = ldsp32(prmt(wlo, lutlane, sel0));
                                a1 = ldsp32(prmt(whi, lutlane, sel0));
                                a2 = ldsp32(prmt(wlo, lutlane, sel1));
                                a3 = ldsp32(prmt(whi, lutlane, sel1));
                            } else {
                                const uint32_t sel = 0x7604u | ((uint32_t)(j & 3) << 4);
                                const uint2 lo2 = ldsp64(prmt(w[2 * rb][j >> 2], lutlane, sel));
                                const uint2 hi2 = ldsp64(prmt(w[2 * rb + 1][j >> 2], lutlane, sel));
                                a0 = lo2.x; a1 = hi2.x; a2 = lo2.y; a3 = hi2.y;
                            }
                            mma16816(c[rb], a0, a1, a2, a3, qb[j][0], qb[j][1]);
                        }
                    }
                }
                // K norms of this lane's four token rows (ordered loads: they precede the hand-over of the K part)
                float kn4[4];
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) kn4[blk] = ldsv_h2f(kns + ((uint32_t)(8 * blk) + tauK) * nstride);
                release_part(0);
                TQ_STAMP(2);

                // ---------------- online softmax: sv[blk][e] = score of token row (block blk, tau(gl)) and head 2*t4 + e.
                // Columns of heads >= grp carry zeros and are never read.
                float sv[4][2];
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
                    sv[blk][0] = c[blk >> 1][2 * (blk & 1)] * kn4[blk];
                    sv[blk][1] = c[blk >> 1][2 * (blk & 1) + 1] * kn4[blk];
                }
                if constexpr (!FULLT) {  // rows past the position may hold anything (even NaN norms): force them out
#pragma unroll
                    for (int blk = 0; blk < 4; ++blk) {
                        const int tok = t0 + 8 * blk + (int)tauK;
                        if (tok >= Lcol0) sv[blk][0] = -1e30f;
                        if (tok >= Lcol1) sv[blk][1] = -1e30f;
                    }
                }
                float mx0 = fmaxf(fmaxf(sv[0][0], sv[1][0]), fmaxf(sv[2][0], sv[3][0]));
                float mx1 = fmaxf(fmaxf(sv[0][1], sv[1][1]), fmaxf(sv[2][1], sv[3][1]));
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
                }
                const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
                if (__any_sync(0xffffffffu, mn0 > m_run[0] || mn1 > m_run[1])) {
                    // 1 when unchanged, 0 at the first tile; the accumulators of heads 2*t4, 2*t4 + 1 live in this very lane
                    const float c0 = ex2_approx(m_run[0] - mn0), c1 = ex2_approx(m_run[1] - mn1);
                    l_run[0] *= c0;
                    l_run[1] *= c1;
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        acc[b][0] *= c0; acc[b][2] *= c0;
                        acc[b][1] *= c1; acc[b][3] *= c1;
                    }
                    m_run[0] = mn0;
                    m_run[1] = mn1;
                }
                float pv[4][2];
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
                    pv[blk][0] = ex2_approx(sv[blk][0] - m_run[0]);
                    pv[blk][1] = ex2_approx(sv[blk][1] - m_run[1]);
                }
                if constexpr (!FULLT) {
#pragma unroll
                    for (int blk = 0; blk < 4; ++blk) {
                        const int tok = t0 + 8 * blk + (int)tauK;
                        if (tok >= Lcol0) pv[blk][0] = 0.0f;
                        if (tok >= Lcol1) pv[blk][1] = 0.0f;
                    }
                }
                l_run[0] += (pv[0][0] + pv[1][0]) + (pv[2][0] + pv[3][0]);
                l_run[1] += (pv[0][1] + pv[1][1]) + (pv[2][1] + pv[3][1]);

                // ---------------- values: 2 blocks of 16 tokens ----------------
                TQ_STAMP(3);
                const uint32_t tokV = wait_part(1);
                TQ_STAMP(4);
                if (dead) return;
                const uint32_t vt = stage_addr(s) + code_tile + tokV;
                const uint32_t vns = stage_addr(s) + tokV + 2u * code_tile + norm_tile + (uint32_t)head * 2u;
                // weights times V norms as fp16 pairs (heads 2*t4, 2*t4 + 1) of this lane's token rows, then transposed
                // across the warp into the B operand of the value product: lane (gl, t4) receives head gl of the token
                // rows tau(2*t4), tau(2*t4 + 1) of every 8-row block
                uint32_t pb[4];
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
                    float vn = ldsp_h2f(vns + ((uint32_t)(8 * blk) + tauK) * nstride);
                    if constexpr (!FULLT) {  // 0 * NaN would poison the accumulators
                        if (t0 + 8 * blk + (int)tauK >= L) vn = 0.0f;
                    }
                    pb[blk] = movmatrix_trans(pack_half2(pv[blk][0] * vn, pv[blk][1] * vn));
                }
#pragma unroll
                for (int gam = 0; gam < 2; ++gam) {
                    // token rows of this lane: A, B from score block 2*gam, C, D from block 2*gam+1
                    const uint32_t pb0 = pb[2 * gam], pb1 = pb[2 * gam + 1];
                    if (BITS == 4) {
                        // lane reads bytes 8*gl .. 8*gl+7 (coordinates 16*gl .. 16*gl+15) of token rows A, B, C = A+8, D = B+8
                        const uint32_t vg = vt + (uint32_t)gam * 2048u;
                        const uint2 xa = ldsp64(vg + vA_off);
                        const uint2 xb = ldsp64(vg + vB_off);
                        const uint2 xc = ldsp64(vg + vA_off + 1024u);
                        const uint2 xd = ldsp64(vg + vB_off + 1024u);
                        // Interleave the nibbles of two tokens: byte b of `ev` = (code of token A, code of token B) for the
                        // EVEN coordinate of byte b, `od` for the odd one.  The table then returns the (A, B) pair directly.
                        const uint32_t wa[2] = {xa.x, xa.y}, wb[2] = {xb.x, xb.y}, wc[2] = {xc.x, xc.y}, wd[2] = {xd.x, xd.y};
#pragma unroll
                        for (int w2 = 0; w2 < 2; ++w2) {
                            const uint32_t ev_ab = (wa[w2] & 0x0f0f0f0fu) | ((wb[w2] << 4) & 0xf0f0f0f0u);
                            const uint32_t od_ab = ((wa[w2] >> 4) & 0x0f0f0f0fu) | (wb[w2] & 0xf0f0f0f0u);
                            const uint32_t ev_cd = (wc[w2] & 0x0f0f0f0fu) | ((wd[w2] << 4) & 0xf0f0f0f0u);
                            const uint32_t od_cd = ((wc[w2] >> 4) & 0x0f0f0f0fu) | (wd[w2] & 0xf0f0f0f0u);
#pragma unroll
                            for (int b = 0; b < 4; ++b) {
                                const uint32_t sel = 0x7604u | ((uint32_t)b << 4);
                                const uint32_t a0 = ldsp32(prmt(ev_ab, lutlane, sel));
                                const uint32_t a1 = ldsp32(prmt(od_ab, lutlane, sel));
                                const uint32_t a2 = ldsp32(prmt(ev_cd, lutlane, sel));
                                const uint32_t a3 = ldsp32(prmt(od_cd, lutlane, sel));
                                mma16816(acc[4 * w2 + b], a0, a1, a2, a3, pb0, pb1);
                            }
                        }
                    } else {
                        const uint32_t vg = vt + (uint32_t)gam * 2048u;
                        const uint32_t xa = ldsp32(vg + vA_off);
                        const uint32_t xb = ldsp32(vg + vB_off);
                        const uint32_t xc = ldsp32(vg + vA_off + 1024u);
                        const uint32_t xd = ldsp32(vg + vB_off + 1024u);
                        // As in the 4-bit form: byte b of `ev` = (low nibble of token A, low nibble of token B), `od` the high
                        // nibbles; the table turns it into the (A, B) pairs of two coordinates, which are two rows of the operand.
                        const uint32_t ev_ab = (xa & 0x0f0f0f0fu) | ((xb << 4) & 0xf0f0f0f0u);
                        const uint32_t od_ab = ((xa >> 4) & 0x0f0f0f0fu) | (xb & 0xf0f0f0f0u);
                        const uint32_t ev_cd = (xc & 0x0f0f0f0fu) | ((xd << 4) & 0xf0f0f0f0u);
                        const uint32_t od_cd = ((xc >> 4) & 0x0f0f0f0fu) | (xd & 0xf0f0f0f0u);
#pragma unroll
                        for (int bb = 0; bb < 4; ++bb) {
                            const uint32_t sel = 0x7604u | ((uint32_t)bb << 4);
                            const uint2 eab = ldsp64(prmt(ev_ab, lutlane, sel));
                            const uint2 ecd = ldsp64(prmt(ev_cd, lutlane, sel));
                            const uint2 oab = ldsp64(prmt(od_ab, lutlane, sel));
                            const uint2 ocd = ldsp64(prmt(od_cd, lutlane, sel));
                            mma16816(acc[2 * bb], eab.x, eab.y, ecd.x, ecd.y, pb0, pb1);
                            mma16816(acc[2 * bb + 1], oab.x, oab.y, ocd.x, ocd.y, pb0, pb1);
                        }
                    }
                }
            };
            if (!dead && !TQ_DBG(1)) {
                if (full) tile_body(std::true_type{});
                else tile_body(std::false_type{});
            }
            TQ_STAMP(5);
            if (TQ_DBG(1)) {  // timing experiments: the copies without the arithmetic
                wait_part(0);
                release_part(0);
                wait_part(1);
            }
            release_part(1);
            ++consumed;
            if (BITS == 2) {
                if (++s_idx == S) {
                    s_idx = 0;
                    s_par ^= 1u;
                }
            }
        }

        TQ_STAMP(12);  // (zero-length marker: everything up to here went to the tile stamps)
        // ================= end of segment: publish the partial, maybe merge =================
        const int slot = wid + g;
        float* const part_base = p.partials + (PERSIST ? (size_t)layer * (size_t)p.part_layer_stride : (size_t)0);
        if (!TQ_DBG(8)) {
            float lsum0 = l_run[0], lsum1 = l_run[1];  // per lane over its own token rows: sum over the eight row lanes
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                lsum0 += __shfl_xor_sync(0xffffffffu, lsum0, o);
                lsum1 += __shfl_xor_sync(0xffffffffu, lsum1, o);
            }
            if (gl == 0) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int hq = 2 * t4 + e;
                    if (hq < grp) {
                        float* dst = part_base + ((size_t)slot * p.H + (size_t)head * grp + hq) * PART_STRIDE;
                        dst[HEAD_DIM] = e ? m_run[1] : m_run[0];
                        dst[HEAD_DIM + 1] = e ? lsum1 : lsum0;
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int hq = 2 * t4 + e;
                if (hq < grp) {
                    float* dst = part_base + ((size_t)slot * p.H + (size_t)head * grp + hq) * PART_STRIDE + 16 * gl;
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
        if (TQ_DBG(4)) { ++g; continue; }
        if constexpr (PERSIST) {  // the partials of all layers are merged by merge_partials_kernel
            ++g;
            continue;
        }
        // number of workers that hold a part of sequence g
        // owners of the sequence's first and last tile (of the units those tiles start at)
        const int first_w = (int)(((ts_g + g * A + 1) * W - 1) / U);
        const int last_w = (int)(((ts_g1 + g * A) * W - 1) / U);
        const int parts = last_w - first_w + 1;
        group_barrier(group, gthreads);  // every warp's partial is written (happens-before the fence below)
        uint32_t is_last = 1u;
        if (parts > 1) {
            if (gtid == 0) {
                __threadfence();  // cumulative: orders the whole worker's partials before the ticket
                const int old = atomicAdd(p.tickets + g, 1);
                const uint32_t flag = (old == parts - 1) ? 1u : 0u;
                if (flag) {
                    p.tickets[g] = 0;  // everybody has arrived: leave the ticket ready for the next launch
                }
                asm volatile("st.shared.u32 [%0], %1;" ::"r"(ctrl_s), "r"(flag) : "memory");
            }
            group_barrier(group, gthreads);
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(is_last) : "r"(ctrl_s) : "memory");
        }
        if (is_last) {
            const int H = p.H;
            // where row vh of this sequence's output goes (null: nowhere)
            auto out_row = [&](int vh) -> __half* {
                if (vh >= H) return nullptr;
                if (qg <= 1) return p.out + (size_t)g * p.q_dim + (size_t)vh * HEAD_DIM;
                const int kvh = vh / grp, r = vh - kvh * grp, qi = r / grp_real, hq = r - qi * grp_real;
                const int token = g * qg + qi;
                if (token >= p.qg_tokens) return nullptr;
                return p.out + (size_t)token * p.q_dim + (size_t)(kvh * grp_real + hq) * HEAD_DIM;
            };
            // optional copy of the results before their rounding to fp16 (decode form only)
            auto out_row_f32 = [&](int vh) -> float* {
                if (!p.out_f32 || vh >= H || qg > 1) return nullptr;
                return p.out_f32 + ((size_t)g * H + (size_t)vh) * HEAD_DIM;
            };
            merge_sequence<Hkv>(p.partials + (size_t)(first_w + g) * H * PART_STRIDE, parts, H, merge_s, p.rotation_t, head, lane,
                                group, gthreads, out_row, out_row_f32);
        }
        ++g;
    }
    }

#ifdef TQ_TIMING_SWITCHES
    if (p.stamps && lane == 0) {
        TQ_STAMP(6);
        for (int i = 0; i < 15; ++i) atomicAdd(p.stamps + i, (unsigned long long)stamp_acc[i]);
        atomicAdd(p.stamps + 15, 1ull);
    }
#endif
    // A warp that gave up on a wait may still have copies in flight: give them a bounded chance to land
    // before the CTA (and its shared memory) goes away.
    if (dead) {
        for (int n = consumed; n < consumed + S && n < (int)(hi - lo) * n_layers; ++n) {
            mbar_wait_bounded(bar0 + 16u * (uint32_t)(n % S), (uint32_t)(n / S) & 1u, 1u << 16);
            mbar_wait_bounded(bar0 + 16u * (uint32_t)(n % S) + 8u, (uint32_t)(n / S) & 1u, 1u << 16);
        }
    }
}

// ---- whole-step form: merge of the published partials --------------------------------------------------------------
struct MergeParams {
    const float* partials;       // [layers][workers + G][H][PART_STRIDE]
    const int* table;            // tile table [G + 1], then {workers that took part, total tiles}
    const __half* rotation_t;
    __half* out;                 // [layers][G][q_dim]
    float* out_f32;              // optional [layers][G][H][128]
    long long part_layer_stride; // floats
    long long q_layer_stride;    // halves
    int G, H, q_dim;
    int rotated_out;             // 1: leave the results in rotated space (the consumer's weights carry R^T)
};
constexpr int MERGE_WARPS = 8;

// One CTA per (sequence, layer): the merge that decode_attention_kernel's last-arriving worker does in the one-launch
// forms, here as a launch of its own after the whole-step kernel, spread over the whole GPU.
__global__ void __launch_bounds__(MERGE_WARPS * 32) merge_partials_kernel(const MergeParams p) {
    __shared__ __align__(16) uint8_t merge_buf[RegionA::MERGE_GROUP_BYTES];
    pdl_wait();  // the partials and the table come from the previous kernel in the stream
    const int g = blockIdx.x, layer = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long ts_g = p.table[g], ts_g1 = p.table[g + 1];
    const long long W = p.table[p.G + 1], N = p.table[p.G + 2];
    if (N <= 0 || W <= 0) return;
    // owners of the sequence's first and last tile: worker w holds the tiles [w * N / W, (w + 1) * N / W)
    const int first_w = (int)(((ts_g + 1) * W - 1) / N);
    const int last_w = (int)((ts_g1 * W - 1) / N);
    const int parts = last_w - first_w + 1;
    const int H = p.H;
    auto out_row = [&](int vh) -> __half* {
        if (vh >= H) return nullptr;
        return p.out + (size_t)layer * (size_t)p.q_layer_stride + (size_t)g * p.q_dim + (size_t)vh * HEAD_DIM;
    };
    auto out_row_f32 = [&](int vh) -> float* {
        if (!p.out_f32 || vh >= H) return nullptr;
        return p.out_f32 + (((size_t)layer * p.G + (size_t)g) * H + (size_t)vh) * HEAD_DIM;
    };
    merge_sequence<MERGE_WARPS>(p.partials + (size_t)layer * (size_t)p.part_layer_stride + (size_t)(first_w + g) * H * PART_STRIDE,
                                parts, H, smem_u32(merge_buf), p.rotation_t, warp, lane, 0, MERGE_WARPS * 32, out_row, out_row_f32,
                                p.rotated_out != 0);
}

}  // namespace tq
