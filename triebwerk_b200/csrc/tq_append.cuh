// TurboQuant append (normalise -> rotate -> quantise -> pack) and query pre-rotation, sm_100a.
//
// Replaces turbo_kv_quantize_kernel / turbo_kv_quantize_batch_kernel (reference engine/kernels.cu:1482-1636)
// and phase 1 of the attention kernels (:1676-1680).  Stored bytes must equal the reference's, so the
// arithmetic keeps the reference's order and instructions (it is built with --use_fast_math):
//   * sum of squares: per-warp shfl_down tree (16,8,4,2,1), then (p0+p2)+(p1+p3);
//   * inv = rsqrt.approx.ftz(ss + 1e-12f); xh = v * inv (mul.ftz);
//   * rot[d] = fma.rn.ftz chain over k = 0..127 of float(R[d][k]) * xh[k], starting from 0;
//   * code = number of bounds <= rot (NaN -> 15 for 4-bit, 0 for 2-bit); norm = half(sqrt.approx.ftz(ss + 1e-12f)).
// What changes is the data movement: a CTA stages R once in shared memory as fp32, laid out so that thread d
// (output coordinate d) fetches R[d][k..k+3] with one conflict-free 16-byte load, and streams many head vectors
// through it (the reference re-reads all 32 KB of R, uncoalesced, for every single vector); K, V and the query
// rotation share one launch; NV vectors advance together, step by step, for instruction-level parallelism along
// the 128-long dependent FMA chain; the chain is a short rolled loop (a fully unrolled one is instruction-fetch
// bound, every warp runs it once).
#pragma once

#include "tq_common.cuh"

namespace tq {

constexpr int APPEND_GROUPS = 4;   // 128-thread groups per CTA, sharing one copy of R
constexpr int APPEND_THREADS = 128 * APPEND_GROUPS;
constexpr int APPEND_MAX_NV = 4;   // head vectors a group carries together: 1, 2 or 4 (chosen per launch)

struct AppendParams {
    // destinations (K cache, V cache); either pair may be null
    uint8_t* ck;
    __half* kn;
    uint8_t* cv;
    __half* vn;
    // sources: k_buf/v_buf [n_src][kv_dim], q [n_src][q_dim]; any may be null
    const __half* k_buf;
    const __half* v_buf;
    const __half* q;
    const __half* rotation;      // [128][128] row-major
    const float* rot_prep;       // optional: R as fp32 in the kernel's shared-memory order [k/4][d][k%4] (64 KB)
    const int* positions;        // device; batch mode: [G]; token mode: [T]
    const long long* row_base;   // batch mode, optional [G]
    float* q_rot;                // [G][H][128]
    int* tile_start;             // [G+1], optional (written by block 0 in batch mode)
    int* tickets;                // [G], optional (zeroed by block 0)
    int* worker_g;               // [n_workers], optional: first sequence of each attention worker's slice
    int n_workers;               // attention workers the tile list will be cut into
    int* total_tiles;
    int* status;
    long long token_row0;        // token mode: first row of the sequence the tokens belong to
    int token_mode;              // 0: one token per sequence (row = row(g)+positions[g]); 1: row = row0+positions[t]
    int max_seq_len;
    int capacity_rows;           // rows a sequence may use (position check); <=0 disables the check
    const int* seq_capacity;     // batch mode, optional [G]: rows sequence g may use (ragged slots), instead of capacity_rows
    int n_src;                   // G (batch mode) or T (token mode)
    int H, Hkv, q_dim, kv_dim, bits;
    int pos_value;               // used when positions == nullptr (token mode: token t goes to position pos_value + t)
    int qg;                      // > 1: rotated queries are stored for the prefill form of the attention (groups of qg tokens)
};

// One CTA = APPEND_GROUPS groups of 128 threads around one copy of R in shared memory; thread d of a group owns
// output coordinate d and row d of R, and a group carries NV head vectors at a time.  When the launch also has to
// build the attention kernel's tables, block 0 does only that and the head vectors start at block 1.
template <int NV>
__global__ void __launch_bounds__(APPEND_THREADS) append_rotate_kernel(const AppendParams p) {
    __shared__ __align__(16) float xs[APPEND_GROUPS][NV][HEAD_DIM];
    __shared__ float warp_part[APPEND_GROUPS][NV][4];
    __shared__ __align__(16) uint8_t codes[APPEND_GROUPS][NV][HEAD_DIM];
    __shared__ long long dest_row[APPEND_GROUPS][NV];
    __shared__ int dest_meta[APPEND_GROUPS][NV];
    __shared__ __align__(8) unsigned long long r_bar;
    extern __shared__ __align__(128) float Rs[];

    const int tid = threadIdx.x;
    const int grp = tid >> 7, d = tid & 127;
    const int lane = tid & 31, wid = (tid >> 5) & 3;

    pdl_launch_dependents();
    const bool has_tables = p.tile_start != nullptr && !p.token_mode;
    const bool table_block = blockIdx.x == 0 && has_tables;

    const int nk = p.k_buf ? p.Hkv : 0;
    const int nv = p.v_buf ? p.Hkv : 0;
    const int nq = p.q ? p.H : 0;
    const int per_src = nk + nv + nq;
    const int total = p.n_src * per_src;  // the host refuses launches with 2^31 vectors or more
    const int vblock = (int)blockIdx.x - (has_tables ? 1 : 0);  // index among the blocks that process vectors
    const int vblocks = (int)gridDim.x - (has_tables ? 1 : 0);
    constexpr int PER_ITER = APPEND_GROUPS * NV;
    const bool has_work = !table_block && vblock * PER_ITER < total;

    // R into shared memory as fp32, Rs[k/4][d][k%4]: thread d later reads R[d][4j..4j+3] as one float4, consecutive
    // threads 16 bytes apart.  When the caller holds R in that form already, one bulk copy brings it in while the
    // threads fetch their inputs; otherwise the threads convert the fp16 matrix themselves.  R is never written by a
    // kernel, so this may run while the previous kernel in the stream is still finishing.
    const uint32_t bar = smem_u32(&r_bar);
    const bool r_async = p.rot_prep != nullptr;
    if (has_work) {
        if (r_async) {
            if (tid == 0) {
                mbar_init(bar, 1);
                fence_mbar_init();
                mbar_arrive_expect_tx(bar, (uint32_t)(HEAD_DIM * HEAD_DIM * sizeof(float)));
                bulk_load(smem_u32(Rs), p.rot_prep, (uint32_t)(HEAD_DIM * HEAD_DIM * sizeof(float)), bar);
            }
        } else {
            const uint4* src = reinterpret_cast<const uint4*>(p.rotation + (size_t)d * HEAD_DIM) + 4 * grp;
            uint4 rr[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) rr[i] = __ldg(src + i);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 u = rr[i];
                const __half2* h2 = reinterpret_cast<const __half2*>(&u);
                const float2 f0 = __half22float2(h2[0]), f1 = __half22float2(h2[1]);
                const float2 f2 = __half22float2(h2[2]), f3 = __half22float2(h2[3]);
                const int j = 2 * (4 * grp + i);
                *reinterpret_cast<float4*>(&Rs[(j * HEAD_DIM + d) * 4]) = make_float4(f0.x, f0.y, f1.x, f1.y);
                *reinterpret_cast<float4*>(&Rs[((j + 1) * HEAD_DIM + d) * 4]) = make_float4(f2.x, f2.y, f3.x, f3.y);
            }
        }
    }
    pdl_wait();  // inputs come from earlier kernels; the workspace may still be read by the previous attention

    // Block 0 also prepares the attention kernel's tables: tickets = 0, tile_start = prefix of tiles, and the
    // first sequence of every worker's slice of the flat tile list.
    if (table_block) {
        if (tid >= 128) return;
        __shared__ int scan[128];
        const int G = p.n_src;
        const int per = (G + 127) / 128;
        int local = 0;
        for (int i = 0; i < per; ++i) {
            int g = d * per + i;
            if (g < G) {
                int pos = p.positions ? p.positions[g] : p.pos_value;
                if (pos < 0) pos = 0;
                local += (pos + 1 + TILE_TOKENS - 1) / TILE_TOKENS;
                if (p.tickets) p.tickets[g] = 0;
            }
        }
        // inclusive scan over 128 entries: shuffles inside the warps, then the four warp totals
        int incl = local;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += v;
        }
        if (lane == 31) scan[wid] = incl;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        int before = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) before += (w < wid) ? scan[w] : 0;
        const int N = scan[0] + scan[1] + scan[2] + scan[3];
        int run = before + incl - local;  // exclusive
        const int W = attention_workers(p.n_workers, N, G);
        for (int i = 0; i < per; ++i) {
            int g = d * per + i;
            if (g < G) {
                p.tile_start[g] = run;
                int pos = p.positions ? p.positions[g] : p.pos_value;
                if (pos < 0) pos = 0;
                const int next = run + (pos + 1 + TILE_TOKENS - 1) / TILE_TOKENS;
                if (p.worker_g) {
                    // worker w starts at tile floor(w*N/W); it starts inside sequence g iff ceil(run*W/N) <= w < ceil(next*W/N)
                    const int w0 = (int)(((long long)run * W + N - 1) / N);
                    const int w1 = (int)(((long long)next * W + N - 1) / N);
                    for (int w = w0; w < w1; ++w) p.worker_g[w] = g;
                }
                run = next;
            }
        }
        if (d == 127) {
            p.tile_start[G] = N;
            if (p.total_tiles) *p.total_tiles = N;
        }
        return;
    }
    if (!has_work) return;

    const int vpb = (p.bits == 2) ? 4 : 2;
    const int bph = HEAD_DIM / vpb;
    const int kvp = p.kv_dim / vpb;
    bool r_ready = !r_async;

    for (int base = vblock * PER_ITER; base < total; base += vblocks * PER_ITER) {
        // ---- decode the NV work items of this group without branches, then issue every load at once ----
        const int gbase = base + grp * NV;
        int kind[NV];  // 0 = K, 1 = V, 2 = Q, -1 = none
        int srcid[NV], head[NV];
        const __half* src[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int item = gbase + v;
            const bool live = item < total;
            const int s = live ? item / per_src : 0;
            const int w = live ? item - s * per_src : 0;
            srcid[v] = s;
            const bool is_k = w < nk, is_v = !is_k && w < nk + nv;
            kind[v] = !live ? -1 : (is_k ? 0 : (is_v ? 1 : 2));
            head[v] = is_k ? w : (is_v ? w - nk : w - nk - nv);
            const __half* basep = is_k ? p.k_buf : (is_v ? p.v_buf : p.q);
            const int stride = (is_k || is_v) ? p.kv_dim : p.q_dim;
            src[v] = basep + (size_t)s * stride + (size_t)head[v] * HEAD_DIM + d;
        }
        float val[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) val[v] = kind[v] >= 0 ? __half2float(*src[v]) : 0.0f;
        // thread v of the group also fetches where vector v goes (position and first row of its sequence)
        int my_pos = p.pos_value;  // (token mode without a position array: consecutive positions from pos_value, set below)
        int my_cap = p.capacity_rows;
        long long my_row0 = 0;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            if (d == v && (kind[v] == 0 || kind[v] == 1)) {
                if (p.positions) my_pos = p.positions[srcid[v]];
                else if (p.token_mode) my_pos = p.pos_value + srcid[v];
                if (p.seq_capacity && !p.token_mode) my_cap = p.seq_capacity[srcid[v]];
                my_row0 = p.token_mode ? p.token_row0
                                       : (p.row_base ? p.row_base[srcid[v]] : (long long)srcid[v] * p.max_seq_len);
            }
        }
        // ---- sum of squares (reference order), normalise ----
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            float sq = mul_ftz(val[v], val[v]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sq = add_ftz(sq, __shfl_down_sync(0xffffffffu, sq, off));
            if (lane == 0) warp_part[grp][v][wid] = sq;
        }
        __syncthreads();
        float t[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            float ss = add_ftz(add_ftz(warp_part[grp][v][0], warp_part[grp][v][2]),
                               add_ftz(warp_part[grp][v][1], warp_part[grp][v][3]));
            t[v] = add_ftz(ss, 1e-12f);
            float inv = rsqrt_approx_ftz(t[v]);
            // queries are rotated as they are (no normalisation)
            xs[grp][v][d] = (kind[v] == 2) ? val[v] : mul_ftz(val[v], inv);
        }
        __syncthreads();
        if (!r_ready) {
            if (!mbar_wait_bounded(bar, 0u, 1u << 22) && tid == 0) atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
            r_ready = true;
        }

        // ---- rotation: k-ascending fused chain per output coordinate, the NV chains interleaved step by step ----
        float acc[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v] = 0.0f;
#pragma unroll 4
        for (int j = 0; j < HEAD_DIM / 4; ++j) {
            const float4 r = *reinterpret_cast<const float4*>(&Rs[(j * HEAD_DIM + d) * 4]);
            float4 x[NV];
#pragma unroll
            for (int v = 0; v < NV; ++v) x[v] = *reinterpret_cast<const float4*>(&xs[grp][v][4 * j]);
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[v] = fma_ftz(r.x, x[v].x, acc[v]);
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[v] = fma_ftz(r.y, x[v].y, acc[v]);
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[v] = fma_ftz(r.z, x[v].z, acc[v]);
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[v] = fma_ftz(r.w, x[v].w, acc[v]);
        }

        // ---- quantise; rotated queries go straight out ----
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            codes[grp][v][d] = (uint8_t)quantize_code(acc[v], p.bits);
            // log2(e) / sqrt(128): the attention kernel works with exp2 and folds the softmax scale here
            if (kind[v] == 2) {
                size_t qrow = (size_t)srcid[v] * p.H + head[v];
                if (p.qg > 1) {  // row order (group of tokens, kv head, token in group, head of the kv head)
                    const int grp = p.H / p.Hkv, kvh = head[v] / grp, hq = head[v] - kvh * grp;
                    const int gq = srcid[v] / p.qg, qi = srcid[v] - gq * p.qg;
                    qrow = ((size_t)gq * p.Hkv + kvh) * (size_t)(grp * p.qg) + (size_t)qi * grp + hq;
                }
                p.q_rot[qrow * HEAD_DIM + d] = acc[v] * 0.12751743074602467f;
            }
        }
        // destination row and norm of vector v, by thread v of the group
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            if (d == v) {
                const bool kv = kind[v] == 0 || kind[v] == 1;
                const bool ok = my_pos >= 0 && (my_cap <= 0 || my_pos < my_cap);
                long long row = -1;
                if (kv && ok) {
                    row = my_row0 + my_pos;
                    __half* cn = (kind[v] == 0) ? p.kn : p.vn;
                    cn[(size_t)row * p.Hkv + head[v]] = __float2half_rn(sqrt_approx_ftz(t[v]));
                } else if (kv) {
                    atomicMax(p.status, ST_BAD_POSITION);
                }
                dest_row[grp][v] = row;
                dest_meta[grp][v] = (kind[v] << 8) | head[v];
            }
        }
        __syncthreads();
        // ---- pack: one 32-bit word (8 four-bit or 16 two-bit codes) per thread, NV * bph / 4 words per group ----
        {
            const int words_per_vec = bph / 4;
            for (int wi = d; wi < NV * words_per_vec; wi += 128) {
                const int v = wi / words_per_vec, wv = wi - v * words_per_vec;
                const long long row = dest_row[grp][v];
                if (row >= 0) {
                    const int meta = dest_meta[grp][v];
                    uint32_t word = 0;
                    if (p.bits == 2) {
                        const uint4 c4 = *reinterpret_cast<const uint4*>(&codes[grp][v][16 * wv]);
                        const uint32_t cw[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                        for (int b = 0; b < 4; ++b) {  // 4 code bytes -> one packed byte
                            const uint32_t x = cw[b];
                            const uint32_t pk = (x & 3u) | ((x >> 6) & 0xcu) | ((x >> 12) & 0x30u) | ((x >> 18) & 0xc0u);
                            word |= pk << (8 * b);
                        }
                    } else {
                        const uint2 c2 = *reinterpret_cast<const uint2*>(&codes[grp][v][8 * wv]);
                        const uint32_t cw[2] = {c2.x, c2.y};
#pragma unroll
                        for (int hbyte = 0; hbyte < 2; ++hbyte) {  // 4 code bytes -> two packed bytes
                            const uint32_t x = cw[hbyte];
                            const uint32_t pk = (x & 0xfu) | ((x >> 4) & 0xf0u) | ((x >> 8) & 0xf00u) | ((x >> 12) & 0xf000u);
                            word |= pk << (16 * hbyte);
                        }
                    }
                    uint8_t* cq = ((meta >> 8) == 0) ? p.ck : p.cv;
                    *reinterpret_cast<uint32_t*>(cq + (size_t)row * kvp + (size_t)(meta & 0xff) * bph + 4 * wv) = word;
                }
            }
        }
        __syncthreads();
    }
}

}  // namespace tq
