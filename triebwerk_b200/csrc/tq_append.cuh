// TurboQuant append (normalise -> rotate -> quantise -> pack) and query pre-rotation, sm_100a.
//
// Replaces turbo_kv_quantize_kernel / turbo_kv_quantize_batch_kernel (reference engine/kernels.cu:1482-1636)
// and phase 1 of the attention kernels (:1676-1680).  Stored bytes must equal the reference's, so the
// arithmetic keeps the reference's order and instructions (it is built with --use_fast_math):
//   * sum of squares: per-warp shfl_down tree (16,8,4,2,1), then (p0+p2)+(p1+p3);
//   * inv = rsqrt.approx.ftz(ss + 1e-12f); xh = v * inv (mul.ftz);
//   * rot[d] = fma.rn.ftz chain over k = 0..127 of float(R[d][k]) * xh[k], starting from 0;
//   * code = number of bounds <= rot (NaN -> 15 for 4-bit, 0 for 2-bit); norm = half(sqrt.approx.ftz(ss + 1e-12f)).
// What changes is the data movement: one CTA keeps row d of R in the registers of thread d and streams
// many head vectors through it (the reference re-reads all 32 KB of R for every single vector), K, V and
// the query rotation share one launch, and NV vectors are in flight per thread for instruction-level
// parallelism along the 128-long dependent FMA chain.
#pragma once

#include "tq_common.cuh"

namespace tq {

constexpr int APPEND_NV = 4;  // head vectors processed together by one CTA

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
    int n_src;                   // G (batch mode) or T (token mode)
    int H, Hkv, q_dim, kv_dim, bits;
    int pos_value;               // used when positions == nullptr
};

__device__ __forceinline__ int quantize_code(float v, int bits) {
    if (bits == 4) {
        if (v != v) return 15;
        int c = 0;
#pragma unroll
        for (int i = 0; i < 15; ++i) c += (v >= kBnd4[i]) ? 1 : 0;
        return c;
    }
    return ((v >= kBnd2[0]) ? 1 : 0) + ((v >= kBnd2[1]) ? 1 : 0) + ((v >= kBnd2[2]) ? 1 : 0);
}

// One CTA = 128 threads; thread d owns output coordinate d and row d of R.
__global__ void __launch_bounds__(128) append_rotate_kernel(const AppendParams p) {
    __shared__ __align__(16) float xs[APPEND_NV][HEAD_DIM];
    __shared__ float warp_part[APPEND_NV][4];
    __shared__ uint8_t codes[APPEND_NV][HEAD_DIM];

    const int d = threadIdx.x;
    const int lane = d & 31, wid = d >> 5;

    pdl_launch_dependents();

    // Row d of R into registers as fp32 (exact: fp16 -> fp32).  R is never written by a kernel, so this may run
    // while the previous kernel in the stream is still finishing.
    float r[HEAD_DIM];
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.rotation + (size_t)d * HEAD_DIM);
#pragma unroll
        for (int i = 0; i < HEAD_DIM / 8; ++i) {
            uint4 u = __ldg(src + i);
            const __half2* h2 = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __half22float2(h2[j]);
                r[8 * i + 2 * j] = f.x;
                r[8 * i + 2 * j + 1] = f.y;
            }
        }
    }
    pdl_wait();  // inputs come from earlier kernels; the workspace may still be read by the previous attention

    // Block 0 also prepares the attention kernel's tables: tickets = 0, tile_start = prefix of tiles, and the
    // first sequence of every worker's slice of the flat tile list.
    if (blockIdx.x == 0 && p.tile_start != nullptr && !p.token_mode) {
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
        scan[d] = local;
        __syncthreads();
        // inclusive scan over 128 entries (Hillis-Steele)
        for (int off = 1; off < 128; off <<= 1) {
            int v = (d >= off) ? scan[d - off] : 0;
            __syncthreads();
            scan[d] += v;
            __syncthreads();
        }
        int run = scan[d] - local;  // exclusive
        for (int i = 0; i < per; ++i) {
            int g = d * per + i;
            if (g < G) {
                p.tile_start[g] = run;
                int pos = p.positions ? p.positions[g] : p.pos_value;
                if (pos < 0) pos = 0;
                run += (pos + 1 + TILE_TOKENS - 1) / TILE_TOKENS;
            }
        }
        const int N = scan[127];
        if (d == 127) {
            p.tile_start[G] = N;
            if (p.total_tiles) *p.total_tiles = N;
        }
        __syncthreads();  // tile_start is complete and visible to this block
        if (p.worker_g) {
            const int W = p.n_workers < N ? p.n_workers : N;
            for (int w = d; w < W; w += 128) {
                const long long lo = (long long)w * N / W;
                int a = 0, b = G;  // invariant: tile_start[a] <= lo < tile_start[b]
                while (b - a > 1) {
                    int mid = (a + b) >> 1;
                    if ((long long)p.tile_start[mid] <= lo) a = mid; else b = mid;
                }
                p.worker_g[w] = a;
            }
        }
        __syncthreads();
    }

    const int nk = p.k_buf ? p.Hkv : 0;
    const int nv = p.v_buf ? p.Hkv : 0;
    const int nq = p.q ? p.H : 0;
    const int per_src = nk + nv + nq;
    const long long total = (long long)p.n_src * per_src;
    if ((long long)blockIdx.x * APPEND_NV >= total) return;

    const int vpb = (p.bits == 2) ? 4 : 2;
    const int bph = HEAD_DIM / vpb;
    const int kvp = p.kv_dim / vpb;

    for (long long base = (long long)blockIdx.x * APPEND_NV; base < total; base += (long long)gridDim.x * APPEND_NV) {
        // ---- load, sum of squares, normalise ----
        float val[APPEND_NV];
        int kind[APPEND_NV];  // 0 = K, 1 = V, 2 = Q, -1 = none
        int srcid[APPEND_NV], head[APPEND_NV];
#pragma unroll
        for (int v = 0; v < APPEND_NV; ++v) {
            long long item = base + v;
            kind[v] = -1;
            val[v] = 0.0f;
            srcid[v] = 0;
            head[v] = 0;
            if (item < total) {
                int s = (int)(item / per_src);
                int w = (int)(item - (long long)s * per_src);
                srcid[v] = s;
                if (w < nk) {
                    kind[v] = 0;
                    head[v] = w;
                    val[v] = __half2float(p.k_buf[(size_t)s * p.kv_dim + (size_t)w * HEAD_DIM + d]);
                } else if (w < nk + nv) {
                    kind[v] = 1;
                    head[v] = w - nk;
                    val[v] = __half2float(p.v_buf[(size_t)s * p.kv_dim + (size_t)(w - nk) * HEAD_DIM + d]);
                } else {
                    kind[v] = 2;
                    head[v] = w - nk - nv;
                    val[v] = __half2float(p.q[(size_t)s * p.q_dim + (size_t)(w - nk - nv) * HEAD_DIM + d]);
                }
            }
        }
#pragma unroll
        for (int v = 0; v < APPEND_NV; ++v) {
            float sq = mul_ftz(val[v], val[v]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sq = add_ftz(sq, __shfl_down_sync(0xffffffffu, sq, off));
            if (lane == 0) warp_part[v][wid] = sq;
        }
        __syncthreads();
        float t[APPEND_NV];
#pragma unroll
        for (int v = 0; v < APPEND_NV; ++v) {
            float ss = add_ftz(add_ftz(warp_part[v][0], warp_part[v][2]), add_ftz(warp_part[v][1], warp_part[v][3]));
            t[v] = add_ftz(ss, 1e-12f);
            float inv = rsqrt_approx_ftz(t[v]);
            // queries are rotated as they are (no normalisation)
            xs[v][d] = (kind[v] == 2) ? val[v] : mul_ftz(val[v], inv);
        }
        __syncthreads();

        // ---- rotation: k-ascending fused chain per output coordinate ----
        float acc[APPEND_NV];
#pragma unroll
        for (int v = 0; v < APPEND_NV; ++v) acc[v] = 0.0f;
#pragma unroll
        for (int k = 0; k < HEAD_DIM; k += 4) {
#pragma unroll
            for (int v = 0; v < APPEND_NV; ++v) {
                float4 x = *reinterpret_cast<const float4*>(&xs[v][k]);
                acc[v] = fma_ftz(r[k + 0], x.x, acc[v]);
                acc[v] = fma_ftz(r[k + 1], x.y, acc[v]);
                acc[v] = fma_ftz(r[k + 2], x.z, acc[v]);
                acc[v] = fma_ftz(r[k + 3], x.w, acc[v]);
            }
        }

        // ---- quantise / store ----
#pragma unroll
        for (int v = 0; v < APPEND_NV; ++v) {
            if (kind[v] == 2) {
                // log2(e) / sqrt(128): the attention kernel works with exp2 and folds the softmax scale here
                p.q_rot[((size_t)srcid[v] * p.H + head[v]) * HEAD_DIM + d] = acc[v] * 0.12751743074602467f;
            } else if (kind[v] >= 0) {
                codes[v][d] = (uint8_t)quantize_code(acc[v], p.bits);
            }
        }
        __syncthreads();
#pragma unroll
        for (int v = 0; v < APPEND_NV; ++v) {
            if (kind[v] == 0 || kind[v] == 1) {
                int pos = p.positions ? p.positions[srcid[v]] : p.pos_value;
                bool ok = pos >= 0 && (p.capacity_rows <= 0 || pos < p.capacity_rows);
                if (!ok) {
                    if (d == 0) atomicMax(p.status, ST_BAD_POSITION);
                    continue;
                }
                long long row;
                if (p.token_mode) {
                    row = p.token_row0 + pos;
                } else {
                    row = (p.row_base ? p.row_base[srcid[v]] : (long long)srcid[v] * p.max_seq_len) + pos;
                }
                uint8_t* cq = (kind[v] == 0) ? p.ck : p.cv;
                __half* cn = (kind[v] == 0) ? p.kn : p.vn;
                if (d < bph) {
                    uint8_t packed;
                    if (p.bits == 2) {
                        packed = (uint8_t)(codes[v][4 * d] | (codes[v][4 * d + 1] << 2) | (codes[v][4 * d + 2] << 4) |
                                           (codes[v][4 * d + 3] << 6));
                    } else {
                        packed = (uint8_t)(codes[v][2 * d] | (codes[v][2 * d + 1] << 4));
                    }
                    cq[(size_t)row * kvp + (size_t)head[v] * bph + d] = packed;
                }
                if (d == 0) cn[(size_t)row * p.Hkv + head[v]] = __float2half_rn(sqrt_approx_ftz(t[v]));
            }
        }
        __syncthreads();
    }
}

}  // namespace tq
