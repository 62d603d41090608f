// Host side of the library: tensor-map encoding, launch wrappers with argument checks, the per-device
// workspace used by the reference-compatible launchers, and the KV arena / engine state that the
// reference keeps inside InferenceEngine (engine/engine.cpp:292-409, 893-1022, 1338-1620).
#pragma once

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <random>
#include <tuple>
#include <vector>

#include <cudaTypedefs.h>

#include "../../include/triebwerk_b200.h"
#include "tq_append.cuh"
#include "tq_prefill_tc.cuh"
#include "tq_attention.cuh"
#include "tq_common.cuh"
#include "tq_fp16.cuh"
#include "tq_fp16_tc.cuh"
#include "tq_qrot.cuh"
#include "tq_generic.cuh"
#include "tq_prefill_attn.cuh"
#include "tq_prefill_attn_tc.cuh"

namespace tq {

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? TQ_OK : (int)e; }

#define TQ_CUDA(call)                                  \
    do {                                               \
        cudaError_t _e = (call);                       \
        if (_e != cudaSuccess) return (int)_e;         \
    } while (0)

struct DeviceProps {
    int sm_count = 0;
};

inline DeviceProps& device_props() {
    static std::mutex mu;
    static std::map<int, DeviceProps> props;
    std::lock_guard<std::mutex> lock(mu);
    int dev = 0;
    cudaGetDevice(&dev);
    DeviceProps& d = props[dev];
    if (d.sm_count == 0) {
        cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (d.sm_count <= 0) d.sm_count = 1;
    }
    return d;
}

// ---- TMA descriptors ----------------------------------------------------------------------------------------------
inline PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
    });
    return fn;
}

// Code array viewed as uint8 [rows][kvp]; box = 128 bytes x TILE_TOKENS rows, 128-byte swizzle in shared memory.
inline int make_code_map(CUtensorMap* m, const void* base, long long rows, int kvp) {
    auto fn = encode_fn();
    if (!fn) return TQ_ERR_UNSUPPORTED;
    if (((uintptr_t)base & 15u) != 0 || rows <= 0 || rows >= (1ll << 31) || kvp % 128 != 0) return TQ_ERR_ARG;
    // Three dimensions: 128 bytes of a row, the rows, and the 128-byte column blocks of a row.  One box covers a whole
    // tile (32 rows x all column blocks) and lands in shared memory as [column block][row][128 B]: one copy
    // instruction per tile and array, and the 128-byte swizzle still goes by the row number.
    cuuint64_t dims[3] = {128u, (cuuint64_t)rows, (cuuint64_t)(kvp / 128)};
    cuuint64_t strides[2] = {(cuuint64_t)kvp, 128u};
    cuuint32_t box[3] = {128u, (cuuint32_t)TILE_TOKENS, (cuuint32_t)(kvp / 128)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TQ_OK : TQ_ERR_ARG;
}

// fp16 K or V array [rows][kv_dim] viewed as bytes for fp16_tc_decode_attention_kernel: box = one head's 256 bytes
// (two 128-byte blocks) x 16 rows, 128-byte swizzle.
inline int make_fp16_rows_map(CUtensorMap* m, const void* base, long long rows, int kv_dim) {
    auto fn = encode_fn();
    if (!fn) return TQ_ERR_UNSUPPORTED;
    const long long row_bytes = (long long)kv_dim * 2;
    if (((uintptr_t)base & 15u) != 0 || rows <= 0 || rows >= (1ll << 31) || row_bytes % 256 != 0) return TQ_ERR_ARG;
    cuuint64_t dims[3] = {128u, (cuuint64_t)rows, (cuuint64_t)(row_bytes / 128)};
    cuuint64_t strides[2] = {(cuuint64_t)row_bytes, 128u};
    cuuint32_t box[3] = {128u, (cuuint32_t)FP16TC_BLOCK, 2u};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TQ_OK : TQ_ERR_ARG;
}

// All layers' code arrays (layer_stride bytes apart) as ONE map with the layer as the fourth coordinate; same boxes.
inline int make_code_map_layers(CUtensorMap* m, const void* base, long long rows, int kvp, int layers, size_t layer_stride) {
    auto fn = encode_fn();
    if (!fn) return TQ_ERR_UNSUPPORTED;
    if (((uintptr_t)base & 15u) != 0 || rows <= 0 || rows >= (1ll << 31) || kvp % 128 != 0 || layers <= 0 ||
        (layer_stride & 15u) != 0 || layer_stride < (size_t)rows * kvp)
        return TQ_ERR_ARG;
    cuuint64_t dims[4] = {128u, (cuuint64_t)rows, (cuuint64_t)(kvp / 128), (cuuint64_t)layers};
    cuuint64_t strides[3] = {(cuuint64_t)kvp, 128u, (cuuint64_t)layer_stride};
    cuuint32_t box[4] = {128u, (cuuint32_t)TILE_TOKENS, (cuuint32_t)(kvp / 128), 1u};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TQ_OK : TQ_ERR_ARG;
}

// fp16 K or V input of an append, [tokens][kv_dim] halves, for prefill_append_tc_kernel's TMA form: one box = the 128 head
// vectors of a tile (128 / Hkv tokens x Hkv heads), landing in shared memory as [half of the vector][token][head][128 B]
// with the 128-byte swizzle -- the K-major operand layout of the tensor core, no instruction of the SM involved.
inline int make_append_input_map(CUtensorMap* m, const void* base, long long tokens, int Hkv, int kv_dim) {
    auto fn = encode_fn();
    if (!fn) return TQ_ERR_UNSUPPORTED;
    const long long row_bytes = (long long)kv_dim * 2;
    if (((uintptr_t)base & 15u) != 0 || tokens <= 0 || tokens >= (1ll << 31) || Hkv <= 0 || Hkv > TC_TILE || TC_TILE % Hkv != 0 ||
        row_bytes % 16 != 0 || kv_dim < Hkv * HEAD_DIM)
        return TQ_ERR_ARG;
    cuuint64_t dims[4] = {128u, (cuuint64_t)Hkv, (cuuint64_t)tokens, 2u};
    cuuint64_t strides[3] = {256u, (cuuint64_t)row_bytes, 128u};
    cuuint32_t box[4] = {128u, (cuuint32_t)Hkv, (cuuint32_t)(TC_TILE / Hkv), 2u};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TQ_OK : TQ_ERR_ARG;
}

// ---- workspace ------------------------------------------------------------------------------------------------------
// The carve of tq_common.cuh plus two helper arrays used by the prefill form (positions 0..T-1 and a
// constant row base) and the fp16 twin's ticket/partial area, which aliases the packed path's partials.
struct FullWorkspace {
    Workspace w;
    int* aux_pos;          // [G]
    long long* aux_rows;   // [G]
    __half* rot_t;         // [128][128] transposed rotation (for callers that only hand over R)
    size_t bytes;
};

inline FullWorkspace carve_full(void* base, int G, int H) {
    FullWorkspace f;
    f.w = carve_workspace(base, G, H);
    size_t off = f.w.bytes;
    char* p = (char*)base;
    f.aux_pos = (int*)(p + off);
    off += align_up((size_t)G * sizeof(int), 256);
    f.aux_rows = (long long*)(p + off);
    off += align_up((size_t)G * sizeof(long long), 256);
    f.rot_t = (__half*)(p + off);
    off += (size_t)HEAD_DIM * HEAD_DIM * sizeof(__half);
    f.bytes = off;
    return f;
}

inline size_t fp16_partials_bytes(int G, int H, int max_seq_len) {
    int nchunk = (max_seq_len + FP16_CHUNK - 1) / FP16_CHUNK;
    return (size_t)G * H * nchunk * PART_STRIDE * sizeof(float);
}

// ---- shape checks -------------------------------------------------------------------------------------------------------
// What the entry points accept: any head layout the reference accepts (head_dim 128, num_heads a multiple of num_kv_heads).
inline int check_shape(int G, int H, int Hkv, int head_dim, int q_dim, int kv_dim, int bits, bool packed) {
    if (head_dim != HEAD_DIM) return TQ_ERR_UNSUPPORTED;
    if (G <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0) return TQ_ERR_ARG;
    if (kv_dim != Hkv * head_dim || q_dim < H * head_dim) return TQ_ERR_ARG;
    if (packed && bits != 2 && bits != 4) return TQ_ERR_ARG;
    return TQ_OK;
}

// What the streaming kernels serve; every other layout takes generic_decode_attention_kernel (one CTA per sequence
// and query head, every cache byte read once per query head, as the reference does).
inline bool fast_shape(int H, int Hkv, bool packed) {
    if (packed) return Hkv % 4 == 0 && Hkv <= 8 && H / Hkv <= 8 && H <= ATTN_MAX_HEADS;
    const int grp = H / Hkv;
    return grp == 1 || grp == 2 || grp == 4 || grp == 8;
}

inline int launch_generic_attention(const GenericAttnParams& p, bool fp16, cudaStream_t s) {
    if (p.G <= 0 || p.H <= 0 || p.G > 2147483647 / 1 || p.H > 65535) return TQ_ERR_ARG;
    dim3 grid((unsigned)p.G, (unsigned)p.H);
    if (fp16) generic_decode_attention_kernel<true><<<grid, GENERIC_WARPS * 32, 0, s>>>(p);
    else generic_decode_attention_kernel<false><<<grid, GENERIC_WARPS * 32, 0, s>>>(p);
    return cuda_status(cudaGetLastError());
}

// ---- launches -------------------------------------------------------------------------------------------------------------
// Launch with the programmatic-serialisation attribute: the kernel may start while the previous kernel of the
// stream is still running; the kernels themselves wait (griddepcontrol.wait) before touching dependent data.
template <typename Kernel, typename Params>
inline int launch_kernel(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl, const Params& p) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cuda_status(cudaLaunchKernelEx(&cfg, kernel, p));
}

constexpr size_t APPEND_SMEM = (size_t)HEAD_DIM * HEAD_DIM * sizeof(float);  // R as fp32

// Opt-in to large dynamic shared memory, once per (device, kernel); safe to call from several host threads.
inline int ensure_dynamic_smem(const void* func, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<int, const void*>, bool> done;
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    bool& d = done[std::make_pair(dev, func)];
    if (!d) {
        TQ_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        d = true;
    }
    return TQ_OK;
}

template <int NV>
inline int launch_append_t(const AppendParams& p, dim3 grid, cudaStream_t s, bool pdl) {
    int r = ensure_dynamic_smem((const void*)append_rotate_kernel<NV>, APPEND_SMEM);
    if (r != TQ_OK) return r;
    return launch_kernel(append_rotate_kernel<NV>, grid, dim3(APPEND_THREADS), APPEND_SMEM, s, pdl, p);
}

// Whole prompts (token form, K and/or V, no queries) go to the tensor-core kernel; TQ_PREFILL_TC=0 keeps them on
// the fp32-chain kernel.  Both store the same bytes.
// producer: the form that applies QK-norm and rotary embedding to the K vectors on the way in (PrefillTcParams)
inline int launch_prefill_tc_params(const PrefillTcParams& t, cudaStream_t s, bool producer = false) {
    const long long tokens = (long long)t.n_seq * t.T;
    const long long tiles = ((tokens * t.Hkv + TC_TILE - 1) / TC_TILE) * ((t.k_buf ? 1 : 0) + (t.v_buf ? 1 : 0));
    long long grid = (long long)(producer ? 2 : TC_CTAS_PER_SM) * device_props().sm_count;
    if (grid > tiles) grid = tiles;
    if (grid < 1) return TQ_OK;
    // The vectors reach the operand tile by tensor-map copies where the layout allows it (TQ_PREFILL_TMA=0: through
    // registers, as in the producer form, whose K vectors are computed on the way in).
    static const bool tma_allowed = !(getenv("TQ_PREFILL_TMA") && atoi(getenv("TQ_PREFILL_TMA")) == 0);
    CUtensorMap tmk{}, tmv{};
    bool tma = !producer && tma_allowed;
    if (tma && t.k_buf) tma = make_append_input_map(&tmk, t.k_buf, tokens, t.Hkv, t.kv_dim) == TQ_OK;
    if (tma && t.v_buf) tma = make_append_input_map(&tmv, t.v_buf, tokens, t.Hkv, t.kv_dim) == TQ_OK;
    const void* kernel = producer ? (const void*)prefill_append_tc_kernel<true, false>
                                  : (tma ? (const void*)prefill_append_tc_kernel<false, true> : (const void*)prefill_append_tc_kernel<false, false>);
    int ar = ensure_dynamic_smem(kernel, TC_DYN_SMEM);
    if (ar != TQ_OK) return ar;
    PrefillTcParams ts = t;
#ifdef TQ_TIMING_SWITCHES
    static unsigned long long* d_stamps = nullptr;
    static int stamp_calls = 0;
    if (getenv("TQ_TC_STAMPS")) {
        if (!d_stamps) { cudaMalloc(&d_stamps, 256); cudaMemset(d_stamps, 0, 256); }
        ts.stamps = d_stamps;
    }
#endif
    if (producer) prefill_append_tc_kernel<true, false><<<(unsigned)grid, TC_THREADS, TC_DYN_SMEM, s>>>(tmk, tmv, ts);
    else if (tma) prefill_append_tc_kernel<false, true><<<(unsigned)grid, TC_THREADS, TC_DYN_SMEM, s>>>(tmk, tmv, ts);
    else prefill_append_tc_kernel<false, false><<<(unsigned)grid, TC_THREADS, TC_DYN_SMEM, s>>>(tmk, tmv, ts);
#ifdef TQ_TIMING_SWITCHES
    if (ts.stamps && ++stamp_calls == 40) {
        unsigned long long h[32];
        cudaStreamSynchronize(s);
        cudaMemcpy(h, d_stamps, 256, cudaMemcpyDeviceToHost);
        for (int w = 0; w < 2; ++w) {
            const double n = (double)h[16 * w + 15] * (double)((tiles + grid - 1) / grid);
            fprintf(stderr, "append stamps, warp %d (cycles per tile): top %.0f | loads %.0f | tree %.0f | wait for the chain warp %.0f | operand + barrier B %.0f | "
                            "mma issue + per-vector %.0f | mma wait + barrier C %.0f | epilogue %.0f | barrier D %.0f | loop back %.0f\n",
                    w ? 7 : 0, h[16 * w] / n, h[16 * w + 1] / n, h[16 * w + 2] / n, h[16 * w + 3] / n, h[16 * w + 4] / n, h[16 * w + 5] / n,
                    h[16 * w + 6] / n, h[16 * w + 7] / n, h[16 * w + 8] / n, h[16 * w + 9] / n);
        }
    }
#endif
    return cuda_status(cudaGetLastError());
}

inline int launch_prefill_tc(const AppendParams& p, cudaStream_t s, int n_seq = 1, long long seq_stride_rows = 0,
                             const long long* seq_row_base = nullptr) {
    PrefillTcParams t{};
    t.ck = p.ck; t.kn = p.kn; t.cv = p.cv; t.vn = p.vn;
    t.k_buf = p.k_buf; t.v_buf = p.v_buf; t.rotation = p.rotation; t.positions = p.positions; t.pos_value = p.pos_value; t.status = p.status;
    t.token_row0 = p.token_row0; t.capacity_rows = p.capacity_rows;
    t.seq_stride_rows = seq_stride_rows; t.row_base = seq_row_base; t.n_seq = n_seq;
    t.T = p.n_src; t.Hkv = p.Hkv; t.kv_dim = p.kv_dim; t.bits = p.bits;
    return launch_prefill_tc_params(t, s);
}

inline int launch_append(const AppendParams& p, cudaStream_t s, bool pdl = false) {
    static const bool prefill_tc = !(getenv("TQ_PREFILL_TC") && atoi(getenv("TQ_PREFILL_TC")) == 0);
    // (the tensor-core kernel moves 16 bytes at a time: every array it touches has to be 16-byte aligned)
    const uintptr_t align_or = (uintptr_t)p.k_buf | (uintptr_t)p.v_buf | (uintptr_t)p.ck | (uintptr_t)p.cv | (uintptr_t)p.rotation;
    if (prefill_tc && p.token_mode && !p.q && (p.k_buf || p.v_buf) && (align_or & 15u) == 0 &&
        p.kv_dim == p.Hkv * HEAD_DIM && (long long)p.n_src * p.Hkv >= 4 * TC_TILE && (long long)p.n_src * p.Hkv < (1ll << 31))
        return launch_prefill_tc(p, s);
    const int nk = p.k_buf ? p.Hkv : 0, nv = p.v_buf ? p.Hkv : 0, nq = p.q ? p.H : 0;
    const long long total = (long long)p.n_src * (nk + nv + nq);
    const bool tables = p.tile_start != nullptr && !p.token_mode;
    if (total <= 0 && !tables) return TQ_OK;
    if (total >= (1ll << 31)) return TQ_ERR_CAPACITY;
    // One CTA per SM at most.  As few vectors per group as still fit the whole launch into that one wave: short
    // dependent chains when the batch is small, amortised staging of R when it is large (then the CTAs loop).
    const long long slots = (long long)device_props().sm_count - 1;
    int nvec = 1;
    while (nvec < APPEND_MAX_NV && (total + nvec * APPEND_GROUPS - 1) / (nvec * APPEND_GROUPS) > slots) nvec *= 2;
    long long blocks = (total + nvec * APPEND_GROUPS - 1) / (nvec * APPEND_GROUPS);
    if (blocks > slots) blocks = slots;
    if (blocks < 1) blocks = 1;
    const dim3 grid((unsigned)(blocks + (tables ? 1 : 0)));
    if (nvec == 1) return launch_append_t<1>(p, grid, s, pdl);
    if (nvec == 2) return launch_append_t<2>(p, grid, s, pdl);
    return launch_append_t<4>(p, grid, s, pdl);
}

// Number of attention CTAs: one per SM (each holds ATTN_GROUPS workers), fewer when the cache cannot hold that
// many tiles.
inline int attention_ctas(int G, int max_seq_len) {
    long long tiles = (long long)G * ((max_seq_len + TILE_TOKENS - 1) / TILE_TOKENS);
    long long w = device_props().sm_count;
    if (w * ATTN_GROUPS > MAX_WORKERS) w = MAX_WORKERS / ATTN_GROUPS;
    long long need = (tiles + ATTN_GROUPS - 1) / ATTN_GROUPS;
    if (need < w) w = need;
    return (int)(w < 1 ? 1 : w);
}

template <int BITS, int HKV, int MODE>
inline int launch_attention_t(const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int ctas, cudaStream_t s,
                              bool pdl) {
    int ar = ensure_dynamic_smem((const void*)decode_attention_kernel<BITS, HKV, MODE>, ATTN_DYN_SMEM);
    if (ar != TQ_OK) return ar;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(ATTN_GROUPS * 32 * HKV);
    cfg.dynamicSmemBytes = ATTN_DYN_SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cuda_status(cudaLaunchKernelEx(&cfg, decode_attention_kernel<BITS, HKV, MODE>, tmK, tmV, p));
}

// mode 0: after append_rotate_kernel (rotated queries and tile table in the workspace); 1: one launch per layer and step
// (table, query rotation, optional append and merge in the kernel); 2: whole-step form over AttnParams::n_layers layers.
inline int launch_attention(int bits, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int ctas,
                            cudaStream_t s, bool pdl = false, int mode = 0) {
    if (p.Hkv != 8 && p.Hkv != 4) return TQ_ERR_UNSUPPORTED;
#define TQ_ATTN_DISPATCH(MODE)                                                                                  \
    if (p.Hkv == 8)                                                                                             \
        return bits == 4 ? launch_attention_t<4, 8, MODE>(tmK, tmV, p, ctas, s, pdl)                            \
                         : launch_attention_t<2, 8, MODE>(tmK, tmV, p, ctas, s, pdl);                           \
    return bits == 4 ? launch_attention_t<4, 4, MODE>(tmK, tmV, p, ctas, s, pdl)                                \
                     : launch_attention_t<2, 4, MODE>(tmK, tmV, p, ctas, s, pdl);
    if (mode == 2) { TQ_ATTN_DISPATCH(2) }
    if (mode == 1) { TQ_ATTN_DISPATCH(1) }
    TQ_ATTN_DISPATCH(0)
#undef TQ_ATTN_DISPATCH
}

__global__ void transpose_rotation_kernel(__half* dst, const __half* src, int* tickets = nullptr, int n_tickets = 0) {
    // dst[d][k] = src[k][d]; one block per 32x32 tile would be overkill for 32 KB: a plain strided copy
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < HEAD_DIM * HEAD_DIM; i += gridDim.x * blockDim.x) {
        const int d = i >> 7, k = i & 127;
        dst[i] = src[k * HEAD_DIM + d];
    }
    // optionally also clears the per-sequence tickets for a launch that is not preceded by the append kernel
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_tickets; i += gridDim.x * blockDim.x) tickets[i] = 0;
}

// Tensor-core form of the twin (tq_fp16_tc.cuh): every query head of a KV head from one pass, whatever their number.
template <int GRP>
inline int launch_fp16_tc_t(const CUtensorMap& tmK, const CUtensorMap& tmV, const Fp16AttnParams& p, cudaStream_t s) {
    int ar = ensure_dynamic_smem((const void*)fp16_tc_decode_attention_kernel<GRP>, FP16TC_SMEM);
    if (ar != TQ_OK) return ar;
    dim3 grid(p.Hkv, p.nchunk_max, p.G);
    fp16_tc_decode_attention_kernel<GRP><<<grid, FP16TC_WARPS * 32, FP16TC_SMEM, s>>>(tmK, tmV, p);
    return cuda_status(cudaGetLastError());
}
inline int launch_fp16_tc_attention(const CUtensorMap& tmK, const CUtensorMap& tmV, const Fp16AttnParams& p, cudaStream_t s) {
    switch (p.H / p.Hkv) {
        case 1: return launch_fp16_tc_t<1>(tmK, tmV, p, s);
        case 2: return launch_fp16_tc_t<2>(tmK, tmV, p, s);
        case 4: return launch_fp16_tc_t<4>(tmK, tmV, p, s);
        case 8: return launch_fp16_tc_t<8>(tmK, tmV, p, s);
        default: return TQ_ERR_UNSUPPORTED;
    }
}

// Causal prefill attention with the query tokens in the M dimension (tq_prefill_attn.cuh); bits 0 = fp16 cache.
inline bool prefill_attn_shape(int H, int Hkv) {
    const int grp = Hkv > 0 ? H / Hkv : 0;
    return Hkv > 0 && Hkv <= 65535 && H == grp * Hkv && (grp == 1 || grp == 2 || grp == 4 || grp == 8 || grp == 16);
}
inline int launch_prefill_attention(int bits, PrefillAttnParams p, cudaStream_t s) {
    const int grp = p.H / p.Hkv;
    p.grp_shift = 0;
    while ((1 << p.grp_shift) < grp) ++p.grp_shift;
    const int qt = PFA_ROWS >> p.grp_shift;
    if (p.n_seq <= 0) p.n_seq = 1;
    if ((long long)p.Hkv * p.n_seq > 2147483647ll || (p.T + qt - 1) / qt > 65535) return TQ_ERR_CAPACITY;
    dim3 grid((unsigned)(p.Hkv * p.n_seq), (unsigned)((p.T + qt - 1) / qt));
    if (p.T <= 0) return TQ_OK;
    int ar;
    // tcgen05 form (default; TQ_PREFILL_ATTN_TC=0 selects the mma.sync form); the packed modes need R^T as well
    static const bool tc = !(getenv("TQ_PREFILL_ATTN_TC") && atoi(getenv("TQ_PREFILL_ATTN_TC")) == 0);
    if (tc && ((bits != 0 && p.rotation_t) || bits == 0)) {
        if (bits == 4) {
            if ((ar = ensure_dynamic_smem((const void*)prefill_attention_tc_kernel<4>, PTC_DYN_SMEM)) != TQ_OK) return ar;
            prefill_attention_tc_kernel<4><<<grid, PTC_THREADS, PTC_DYN_SMEM, s>>>(p);
        } else if (bits == 2) {
            if ((ar = ensure_dynamic_smem((const void*)prefill_attention_tc_kernel<2>, PTC_DYN_SMEM)) != TQ_OK) return ar;
            prefill_attention_tc_kernel<2><<<grid, PTC_THREADS, PTC_DYN_SMEM, s>>>(p);
        } else {
            if ((ar = ensure_dynamic_smem((const void*)prefill_attention_tc_kernel<0>, PTC_DYN_SMEM)) != TQ_OK) return ar;
            prefill_attention_tc_kernel<0><<<grid, PTC_THREADS, PTC_DYN_SMEM, s>>>(p);
        }
        return cuda_status(cudaGetLastError());
    }
    switch (bits) {
        case 4:
            if ((ar = ensure_dynamic_smem((const void*)prefill_attention_kernel<4>, PfaSmem::BYTES)) != TQ_OK) return ar;
            prefill_attention_kernel<4><<<grid, PFA_THREADS, PfaSmem::BYTES, s>>>(p);
            break;
        case 2:
            if ((ar = ensure_dynamic_smem((const void*)prefill_attention_kernel<2>, PfaSmem::BYTES)) != TQ_OK) return ar;
            prefill_attention_kernel<2><<<grid, PFA_THREADS, PfaSmem::BYTES, s>>>(p);
            break;
        case 0:
            if ((ar = ensure_dynamic_smem((const void*)prefill_attention_kernel<0>, PfaSmem::BYTES)) != TQ_OK) return ar;
            prefill_attention_kernel<0><<<grid, PFA_THREADS, PfaSmem::BYTES, s>>>(p);
            break;
        default: return TQ_ERR_UNSUPPORTED;
    }
    return cuda_status(cudaGetLastError());
}

inline int launch_fp16_attention(const Fp16AttnParams& p_in, cudaStream_t s) {
    // A CTA serves at most two query heads per pass over the rows (more cost it its occupancy: 47 % of the copy
    // bandwidth with four, 23 % with eight).  With 4 or 8 query heads per KV head, 2 or 4 CTAs share the rows of a KV
    // head as "virtual" KV heads; they are neighbours in the grid, so all but the first read the rows from L2.
    const int grp = p_in.H / p_in.Hkv;
    Fp16AttnParams p = p_in;
    p.Hkv = p_in.Hkv << (grp == 4 ? 1 : (grp == 8 ? 2 : 0));
    dim3 grid(p.Hkv, p.nchunk_max, p.G);  // KV heads fastest: CTAs that run together read the same 2 KB rows (DRAM page locality)
    dim3 block(FP16_WARPS * 32);
    switch (grp) {
        case 1: fp16_decode_attention_kernel<1, 0><<<grid, block, 0, s>>>(p); break;
        case 2: fp16_decode_attention_kernel<2, 0><<<grid, block, 0, s>>>(p); break;
        case 4: fp16_decode_attention_kernel<2, 1><<<grid, block, 0, s>>>(p); break;
        case 8: fp16_decode_attention_kernel<2, 2><<<grid, block, 0, s>>>(p); break;
        default: return TQ_ERR_UNSUPPORTED;
    }
    return cuda_status(cudaGetLastError());
}

__global__ void iota_rows_kernel(int* pos, long long* rows, int n, long long row0) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        pos[i] = i;
        rows[i] = row0;
    }
}

// positions and row bases of the prefill form's token groups: group j ends at token min((j + 1) * qg, T) - 1, row base 0
__global__ void group_rows_kernel(int* pos, long long* rows, int groups, int qg, int T) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < groups) {
        const int last = (j + 1) * qg;
        pos[j] = (last < T ? last : T) - 1;
        rows[j] = 0;
    }
}

// ---- per-device workspace of the compat launchers + descriptor cache ----------------------------------------------------------
// The reference's launchers get every buffer from their caller; the kernels here need scratch of their own (rotated
// queries, tile table, split-K partials), which the reference-compatible launchers keep per device.  All of this state
// is guarded by ONE mutex that a launcher holds from its first look at the state until its kernels are enqueued: the
// compat launchers serialise per process (their host part is a few microseconds).
struct CompatState {
    void* ws = nullptr;
    size_t ws_bytes = 0;
    std::vector<void*> retired;  // outgrown workspaces: kernels already enqueued may still use them, so they stay allocated
    std::map<std::tuple<const void*, long long, int>, CUtensorMap> maps;  // descriptors by (base, rows, row bytes)
};

inline std::recursive_mutex& compat_mutex() {
    static std::recursive_mutex mu;
    return mu;
}

// Call with compat_mutex() held.
inline CompatState& compat_state() {
    static std::map<int, CompatState> st;
    int dev = 0;
    cudaGetDevice(&dev);
    return st[dev];
}

// Call with compat_mutex() held.  The workspace only ever grows, and by at least a factor of two (first allocation:
// 64 MiB or the request), so a serving loop reaches its final size after a few calls; growth allocates a new buffer
// and retires the old one without waiting for the device.
inline int compat_workspace(size_t need, void** out, cudaStream_t s) {
    CompatState& c = compat_state();
    if (c.ws_bytes < need) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(s, &cs);
        if (cs != cudaStreamCaptureStatusNone) return TQ_ERR_WORKSPACE;  // cannot allocate while capturing
        size_t bytes = std::max(need, std::max(c.ws_bytes * 2, (size_t)64 << 20));
        void* fresh = nullptr;
        if (cudaMalloc(&fresh, bytes) != cudaSuccess) {
            cudaGetLastError();
            bytes = need;
            TQ_CUDA(cudaMalloc(&fresh, bytes));
        }
        TQ_CUDA(cudaMemsetAsync(fresh, 0, bytes, s));
        if (c.ws) c.retired.push_back(c.ws);
        c.ws = fresh;
        c.ws_bytes = bytes;
    }
    *out = c.ws;
    return TQ_OK;
}

// Call with compat_mutex() held.  The fp16 twin's descriptors share the cache (key: minus the row bytes).
inline int cached_fp16_map(CUtensorMap* out, const void* base, long long rows, int kv_dim) {
    CompatState& c = compat_state();
    auto key = std::make_tuple(base, rows, -2 * kv_dim);
    auto it = c.maps.find(key);
    if (it == c.maps.end()) {
        CUtensorMap m;
        int r = make_fp16_rows_map(&m, base, rows, kv_dim);
        if (r != TQ_OK) return r;
        if (c.maps.size() > 4096) c.maps.clear();
        it = c.maps.emplace(key, m).first;
    }
    *out = it->second;
    return TQ_OK;
}

// Call with compat_mutex() held.
inline int cached_code_map(CUtensorMap* out, const void* base, long long rows, int kvp) {
    CompatState& c = compat_state();
    auto key = std::make_tuple(base, rows, kvp);
    auto it = c.maps.find(key);
    if (it == c.maps.end()) {
        CUtensorMap m;
        int r = make_code_map(&m, base, rows, kvp);
        if (r != TQ_OK) return r;
        if (c.maps.size() > 4096) c.maps.clear();
        it = c.maps.emplace(key, m).first;
    }
    *out = it->second;
    return TQ_OK;
}

}  // namespace tq

// =====================================================================================================================
// Engine state (opaque to C callers)
// =====================================================================================================================
struct tq_engine {
    tq_model_shape shape{};
    int ctor_max_seq_len = 0;
    int kv_bits = 0;
    int device = 0;

    // arena
    char* arena = nullptr;
    size_t arena_cap = 0;
    bool arena_external = false;
    bool asleep = false;
    // The last thing this engine put on `chain_stream` was a fused decode launch: positions and caches are as that
    // launch saw them, so the next fused launch may read them before it has seen its predecessor finish.
    bool chain_ok = false;
    cudaStream_t chain_stream = nullptr;
    bool fused = !(getenv("TQ_FUSED") && atoi(getenv("TQ_FUSED")) == 0);  // one launch per layer-step (packed modes)

    // current carving
    int G = 0;
    int msl = 0;          // dense slot size, or the largest capacity in ragged mode
    bool ragged = false;
    long long total_rows = 0;
    std::vector<int> capacities;       // rows of every slot (ragged: rounded up to 32; dense: the slot size)
    std::vector<long long> h_row_base; // first row of every slot
    // Shared prefixes: sequence g reads its first prefix_tokens[g] tokens (a multiple of 32) from the slot of
    // prefix_owner[g]; its own slot then starts at token prefix_tokens[g].  0 / -1: nothing shared.
    std::vector<int> prefix_tokens, prefix_owner;
    bool shared_active = false;
    long long* d_prefix_base = nullptr;  // [G] first row of the shared tiles
    int* d_prefix_tiles = nullptr;       // [G] number of shared tiles
    // the slot table the kernels see (null in the dense layout without shared prefixes: row = g * max_seq_len + pos)
    const long long* rb() const { return (ragged || shared_active) ? d_row_base : nullptr; }
    const int* caps() const { return (ragged || shared_active) ? d_capacities : nullptr; }
    long long row0_eff(int g) const { return h_row_base[g] - prefix_tokens[g]; }   // row of token 0 if the slot started there
    int cap_eff(int g) const { return capacities[g] + prefix_tokens[g]; }          // positions the sequence may reach

    struct Layer {
        void* k = nullptr;
        void* v = nullptr;
        void* kn = nullptr;
        void* vn = nullptr;
        CUtensorMap tmK{}, tmV{};  // packed modes: descriptors of the code arrays
    };
    std::vector<Layer> layers;

    // whole-step form: all layers' code arrays as one tensor map each, per-layer split-K partials, the tile table
    CUtensorMap tmK4{}, tmV4{};
    size_t code_layer_stride = 0;      // bytes between consecutive layers' K (and V) code arrays
    size_t norm_layer_stride = 0;      // bytes between consecutive layers' norm arrays
    float* step_partials = nullptr;    // [layers][workers + G][H][PART_STRIDE]
    size_t step_part_stride = 0;       // floats per layer
    int* step_table = nullptr;         // [G + 4]
    void* step_qrot = nullptr;         // [layers][G][H][128] fp16: pre-rotated, pre-scaled queries
    void* step_kpost = nullptr;        // [layers][G][kv_dim] fp16: K after QK-norm and rotary embedding (producer form)
    bool whole_step = !(getenv("TQ_WHOLE_STEP") && atoi(getenv("TQ_WHOLE_STEP")) == 0);
    float* out_f32 = nullptr;          // optional [layers][G][H][128]: results before the fp16 rounding (outside the arena)
    cudaEvent_t ev_attn[2] = {nullptr, nullptr};  // optional: recorded around the attention launch of the whole-step form

    int* d_positions = nullptr;
    int* d_capacities = nullptr;       // [G] positions each sequence may reach (slot rows + shared prefix tokens)
    long long* d_row_base = nullptr;   // [G] first row of every slot, minus the sequence's shared prefix tokens
    void* workspace = nullptr;
    size_t ws_bytes = 0;
    void* stage_q = nullptr;   // [layers][G][q_dim]
    void* stage_k = nullptr;   // [layers][G][kv_dim]
    void* stage_v = nullptr;
    void* stage_out = nullptr; // [layers][G][q_dim]
    // host-buffer steps: copy streams and events that let the copies of one group of layers overlap the kernels of another
    static constexpr int HOST_STEP_CHUNKS = 9;
    cudaStream_t st_in = nullptr, st_out = nullptr;
    cudaEvent_t ev_begin = nullptr, ev_done = nullptr;
    cudaEvent_t ev_in[HOST_STEP_CHUNKS] = {}, ev_out[HOST_STEP_CHUNKS] = {};

    // rotation: host copy kept across sleep, device copies (R and R transposed, 32 KB each) outside the arena
    std::vector<uint16_t> h_rotation;
    void* d_rotation = nullptr;
    void* d_rotation_t = nullptr;
    float* d_rotation_prep = nullptr;  // fp32, in the append kernel's shared-memory order
    void* d_rotation_rep = nullptr;    // R row-major, several copies, for the fused kernel's query rotation

    // sleep that keeps the sequences: every sequence's written rows as a blob in host memory (see tq_engine_export_sequence)
    struct Kept {
        bool valid = false;
        int G = 0, max_seq_len = 0;
        bool ragged = false;
        std::vector<int> capacities, positions;
        std::vector<std::vector<unsigned char>> blobs;
    } kept;

    int q_dim() const { return shape.num_heads * shape.head_dim; }
    int kv_dim() const { return shape.num_kv_heads * shape.head_dim; }
    int vpb() const { return kv_bits == 2 ? 4 : 2; }
    // bytes per cache row (all KV heads) of one of K / V: engine/engine.cpp:292-294 for the packed modes
    size_t code_row_bytes() const { return kv_bits == 0 ? (size_t)kv_dim() * 2 : (size_t)kv_dim() / vpb(); }
};

namespace tq {

// Walks the arena exactly as tq_engine_alloc_batch carves it.  base == nullptr only measures.
struct ArenaPlan {
    size_t bytes = 0;
    long long total_rows = 0;
};

inline size_t bump(size_t& off, size_t bytes) {
    off = (off + 255) & ~(size_t)255;  // 256-byte alignment, as GpuArena::alloc (engine/model.h:264-279)
    size_t at = off;
    off += bytes;
    return at;
}

inline long long plan_rows(int G, int max_seq_len, const int* capacities, std::vector<int>* caps_out,
                           std::vector<long long>* base_out) {
    long long rows = 0;
    if (capacities == nullptr) {
        for (int g = 0; g < G; ++g) {
            if (caps_out) caps_out->push_back(max_seq_len);
            if (base_out) base_out->push_back((long long)g * max_seq_len);
        }
        return (long long)G * max_seq_len;
    }
    for (int g = 0; g < G; ++g) {
        int c = capacities[g] < 1 ? 1 : capacities[g];
        c = (c + TILE_TOKENS - 1) / TILE_TOKENS * TILE_TOKENS;
        if (caps_out) caps_out->push_back(c);
        if (base_out) base_out->push_back(rows);
        rows += c;
    }
    return rows;
}

}  // namespace tq
