// extern "C" surface of libtriebwerk_b200.so (declared in include/triebwerk_b200.h).
// The whole library is this one translation unit; kernels live in the .cuh files it includes.

#include <algorithm>

#include "tq_host.cuh"

using namespace tq;

static thread_local int g_compat_status = TQ_OK;

static inline cudaStream_t cs(tq_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// The engine's own launches overlap each other's tails (programmatic dependent launch); TQ_PDL=0 turns it off.
static inline bool use_pdl() {
    static const bool on = !(getenv("TQ_PDL") && atoi(getenv("TQ_PDL")) == 0);
    return on;
}

extern "C" {

const char* tq_status_string(int status) {
    switch (status) {
        case TQ_OK: return "ok";
        case TQ_ERR_ARG: return "bad argument";
        case TQ_ERR_CAPACITY: return "capacity exceeded";
        case TQ_ERR_WORKSPACE: return "workspace missing or too small";
        case TQ_ERR_UNSUPPORTED: return "unsupported shape";
        case TQ_ERR_STATE: return "engine in the wrong state";
        case TQ_ERR_DEVICE: return "device-side status set";
        case TQ_ERR_NOMEM: return "out of memory";
        default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
    }
}

int tq_version(void) { return 100; }

int tq_last_compat_status(void) { return g_compat_status; }

// ---- rotation ---------------------------------------------------------------------------------------------------------
// Restates engine/engine.cpp:364-392.  An x86-64 build of the reference rounds after every multiply and
// every add (no FMA contraction); the volatile temporaries below keep that whatever flags build this file.
int tq_rotation_generate(uint32_t seed, void* host_out_half) {
    if (!host_out_half) return TQ_ERR_ARG;
    const int d = HEAD_DIM;
    std::mt19937 gen(seed);
    std::normal_distribution<float> dist(0.0f, 1.0f);
    std::vector<float> m((size_t)d * d);
    for (auto& x : m) x = dist(gen);
    for (int i = 0; i < d; ++i) {
        float* ri = &m[(size_t)i * d];
        for (int j = 0; j < i; ++j) {
            const float* rj = &m[(size_t)j * d];
            volatile float dot = 0.0f;  // volatile: keep every rounding step, whatever the host flags
            for (int k = 0; k < d; ++k) {
                volatile float prod = ri[k] * rj[k];
                dot = dot + prod;
            }
            for (int k = 0; k < d; ++k) {
                volatile float prod = dot * rj[k];
                ri[k] = ri[k] - prod;
            }
        }
        volatile float nrm = 0.0f;
        for (int k = 0; k < d; ++k) {
            volatile float prod = ri[k] * ri[k];
            nrm = nrm + prod;
        }
        const float inv = 1.0f / sqrtf(nrm);
        for (int k = 0; k < d; ++k) ri[k] *= inv;
    }
    __half* out = reinterpret_cast<__half*>(host_out_half);
    for (int i = 0; i < d * d; ++i) out[i] = __float2half_rn(m[i]);
    return TQ_OK;
}

size_t tq_workspace_bytes(int G, int num_heads) {
    if (G <= 0 || num_heads <= 0) return 0;
    return carve_full(nullptr, G, num_heads).bytes;
}

int tq_workspace_status(void* workspace, tq_stream_t s) {
    if (!workspace) return TQ_ERR_WORKSPACE;
    int st = 0;
    TQ_CUDA(cudaMemcpyAsync(&st, workspace, sizeof(int), cudaMemcpyDeviceToHost, cs(s)));
    TQ_CUDA(cudaStreamSynchronize(cs(s)));
    if (st != 0) {
        TQ_CUDA(cudaMemsetAsync(workspace, 0, sizeof(int), cs(s)));
        TQ_CUDA(cudaStreamSynchronize(cs(s)));
    }
    return st;
}

// ---- self-test of the bounded waits ---------------------------------------------------------------------------------------
// Every wait on a copy barrier in this library is bounded: after `limit` polls the waiter records
// ST_TMA_WAIT_TIMEOUT in the status word, stops using the pipeline and lets its kernel finish.  This one-warp kernel
// exercises exactly that give-up path without any fault: it arms a barrier for 16 bytes that nobody ever sends, waits
// with a small limit, and reports what mbar_wait_bounded returned.
__global__ void bounded_wait_probe_kernel(int* status, unsigned limit) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        fence_mbar_init();
        mbar_arrive_expect_tx(b, 16u);
    }
    __syncthreads();
    const bool arrived = mbar_wait_bounded(b, 0u, limit);
    if (!arrived && threadIdx.x == 0) atomicMax(status, ST_TMA_WAIT_TIMEOUT);
    __syncthreads();
    if (threadIdx.x == 0) mbar_inval(b);
}

int tq_selftest_bounded_wait(void* status_word, unsigned limit, tq_stream_t s) {
    if (!status_word || limit == 0 || limit > (1u << 20)) return TQ_ERR_ARG;
    bounded_wait_probe_kernel<<<1, 32, 0, cs(s)>>>((int*)status_word, limit);
    int r = cuda_status(cudaGetLastError());
    if (r != TQ_OK) return r;
    return tq_workspace_status(status_word, s);
}

// ---- peer exchange: outputs of sequence-sharded ranks land in every rank's buffer through the copy engines ----------------
// One buffer per rank, made with cudaMalloc here so that its CUDA IPC handle names the whole allocation.  Peers open
// the handle, copy their rows in with plain device-to-device copies (copy engines over NVLink: no SM is taken from the
// attention kernel, which holds all of them) and announce completion by writing a step number into the owner's flag
// words.  Nothing here reads a peer's memory from a kernel; the only kernel-side peer access is the 8-byte flag store.
struct PeerFlagPtrs {
    unsigned long long* p[TQ_PEER_MAX];
};

__global__ void peer_signal_kernel(PeerFlagPtrs flags, int n, int slot, unsigned long long value) {
    const int i = threadIdx.x;
    if (i < n && flags.p[i]) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flags.p[i] + slot), "l"(value) : "memory");
    }
}

__global__ void peer_wait_kernel(const unsigned long long* flags, int n, unsigned long long value, int* status,
                                 unsigned long long limit_ns) {
    const int i = threadIdx.x;
    if (i >= n) return;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flags + i) : "memory");
        if (v >= value) return;
        __nanosleep(200);
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > limit_ns) {  // give up: the host reads the status word, the context stays usable
            if (status) atomicMax(status, ST_PEER_WAIT_TIMEOUT);
            return;
        }
    }
}

int tq_peer_buffer_create(size_t bytes, void** dptr, void* handle64) {
    if (!dptr || !handle64 || bytes == 0) return TQ_ERR_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return TQ_ERR_NOMEM;
    }
    TQ_CUDA(cudaMemset(p, 0, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        cudaFree(p);
        return (int)e;
    }
    memcpy(handle64, &h, 64);
    *dptr = p;
    return TQ_OK;
}

int tq_peer_buffer_open(const void* handle64, void** dptr) {
    if (!handle64 || !dptr) return TQ_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    cudaError_t e = cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    return TQ_OK;
}

int tq_peer_buffer_close(void* dptr) {
    if (!dptr) return TQ_OK;
    TQ_CUDA(cudaIpcCloseMemHandle(dptr));
    return TQ_OK;
}

int tq_peer_buffer_destroy(void* dptr) {
    if (!dptr) return TQ_OK;
    TQ_CUDA(cudaFree(dptr));
    return TQ_OK;
}

int tq_peer_copy(void* dst, const void* src, size_t bytes, tq_stream_t s) {
    if (!dst || !src) return TQ_ERR_ARG;
    if (bytes == 0) return TQ_OK;
    TQ_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, cs(s)));
    return TQ_OK;
}

int tq_peer_signal(void* const* flag_arrays, int n, int slot, unsigned long long value, tq_stream_t s) {
    if (!flag_arrays || n <= 0 || n > TQ_PEER_MAX || slot < 0 || slot >= TQ_PEER_MAX) return TQ_ERR_ARG;
    PeerFlagPtrs f{};
    for (int i = 0; i < n; ++i) f.p[i] = (unsigned long long*)flag_arrays[i];
    peer_signal_kernel<<<1, TQ_PEER_MAX, 0, cs(s)>>>(f, n, slot, value);
    return cuda_status(cudaGetLastError());
}

int tq_peer_wait(const void* flags, int n, unsigned long long value, void* status_word, unsigned limit_ms, tq_stream_t s) {
    if (!flags || n <= 0 || n > TQ_PEER_MAX || limit_ms == 0 || limit_ms > 10000) return TQ_ERR_ARG;
    peer_wait_kernel<<<1, TQ_PEER_MAX, 0, cs(s)>>>((const unsigned long long*)flags, n, value, (int*)status_word,
                                                  (unsigned long long)limit_ms * 1000000ull);
    return cuda_status(cudaGetLastError());
}

// ---- packed path ---------------------------------------------------------------------------------------------------------
static int append_impl(uint8_t* ck_q, void* k_norms, uint8_t* cv_q, void* v_norms, const void* k_buf, const void* v_buf,
                       const void* q, const void* rotation, const int* positions, int pos_value,
                       const long long* row_base, int token_mode, long long token_row0, int max_seq_len, int n_src,
                       int num_heads, int num_kv_heads, int head_dim, int q_dim, int kv_dim, int bits, void* workspace,
                       size_t workspace_bytes, bool build_tiles, cudaStream_t s, bool pdl = false,
                       const float* rot_prep = nullptr, int qg = 0, const int* seq_capacity = nullptr) {
    if (head_dim != HEAD_DIM) return TQ_ERR_UNSUPPORTED;
    if (bits != 2 && bits != 4) return TQ_ERR_ARG;
    if (n_src <= 0 || num_kv_heads <= 0 || kv_dim != num_kv_heads * head_dim || !rotation) return TQ_ERR_ARG;
    if ((k_buf && (!ck_q || !k_norms)) || (v_buf && (!cv_q || !v_norms))) return TQ_ERR_ARG;
    if (q && (num_heads <= 0 || q_dim < num_heads * head_dim)) return TQ_ERR_ARG;
    if (!workspace) return TQ_ERR_WORKSPACE;
    const int Hws = num_heads > 0 ? num_heads : 1;
    FullWorkspace fw = carve_full(workspace, n_src, Hws);
    if (fw.bytes > workspace_bytes) return TQ_ERR_WORKSPACE;
    AppendParams p{};
    p.ck = ck_q; p.kn = (__half*)k_norms; p.cv = cv_q; p.vn = (__half*)v_norms;
    p.k_buf = (const __half*)k_buf; p.v_buf = (const __half*)v_buf; p.q = (const __half*)q;
    p.rotation = (const __half*)rotation;
    p.rot_prep = rot_prep;
    p.positions = positions; p.row_base = row_base;
    p.q_rot = fw.w.q_rot;
    p.tile_start = build_tiles ? fw.w.tile_start : nullptr;
    p.tickets = build_tiles ? fw.w.tickets : nullptr;
    p.worker_g = build_tiles ? fw.w.worker_g : nullptr;
    p.n_workers = attention_ctas(n_src, max_seq_len) * ATTN_GROUPS;
    p.total_tiles = fw.w.total_tiles;
    p.status = fw.w.status;
    p.token_row0 = token_row0; p.token_mode = token_mode;
    p.max_seq_len = max_seq_len; p.capacity_rows = max_seq_len;
    p.n_src = n_src; p.H = num_heads; p.Hkv = num_kv_heads; p.q_dim = q_dim; p.kv_dim = kv_dim; p.bits = bits;
    p.pos_value = pos_value;
    p.qg = qg;
    p.seq_capacity = seq_capacity;
    return launch_append(p, s, pdl);
}

int tq_append_decode(uint8_t* ck_q, void* k_norms, uint8_t* cv_q, void* v_norms, const void* k_buf, const void* v_buf,
                     const void* q, const void* rotation, const int* positions, const long long* row_base,
                     int max_seq_len, int G, int num_heads, int num_kv_heads, int head_dim, int q_dim, int kv_dim,
                     int bits, void* workspace, size_t workspace_bytes, tq_stream_t s) {
    if (!positions) return TQ_ERR_ARG;
    return append_impl(ck_q, k_norms, cv_q, v_norms, k_buf, v_buf, q, rotation, positions, 0, row_base, 0, 0,
                       max_seq_len, G, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, workspace,
                       workspace_bytes, true, cs(s));
}

// Inputs of the fused per-layer launch (append + query rotation + attention in one kernel).
struct FusedInputs {
    const void* q;
    const void* k;
    const void* v;
    const void* rotation;
    int rot_copies;
    int early;
    const int* seq_capacity;  // ragged slots: per-sequence row limits (device), or null
};

static int attention_impl(void* out, const CUtensorMap& tmK, const CUtensorMap& tmV, const void* ck_q, const void* cv_q,
                          const void* k_norms, const void* v_norms,
                          const void* rotation_t, const int* positions, int pos_value, const long long* row_base,
                          long long total_rows, int max_seq_len, int G, int num_heads, int num_kv_heads, int q_dim,
                          int bits, void* workspace, size_t workspace_bytes, cudaStream_t s, bool pdl = false,
                          const FusedInputs* fused = nullptr, int qg = 0, int qg_tokens = 0, float* out_f32 = nullptr,
                          const long long* prefix_base = nullptr, const int* prefix_tiles = nullptr) {
    FullWorkspace fw = carve_full(workspace, G, num_heads);
    if (fw.bytes > workspace_bytes) return TQ_ERR_WORKSPACE;
    // bulk copies need 16-byte aligned sources: rows are 512/256 B (codes) and 2*Hkv B (norms, Hkv % 4 == 0 -> 8|16 B)
    if ((((uintptr_t)ck_q | (uintptr_t)cv_q | (uintptr_t)k_norms | (uintptr_t)v_norms) & 15u) != 0) return TQ_ERR_ARG;
    // norm rows are 2*Hkv bytes: with 4 KV heads (8 B) every slot and the array end must fall on an even row
    if (num_kv_heads % 8 != 0 && ((max_seq_len & 1) || (total_rows & 1))) return TQ_ERR_UNSUPPORTED;
    AttnParams p{};
    p.ck = (const uint8_t*)ck_q; p.cv = (const uint8_t*)cv_q;
    p.kn = (const __half*)k_norms; p.vn = (const __half*)v_norms;
    p.q_rot = fw.w.q_rot; p.rotation_t = (const __half*)rotation_t; p.out = (__half*)out; p.out_f32 = out_f32;
    p.positions = positions; p.row_base = row_base;
    p.prefix_base = prefix_base; p.prefix_tiles = prefix_tiles;
    p.tile_start = fw.w.tile_start; p.worker_g = fw.w.worker_g; p.tickets = fw.w.tickets; p.partials = fw.w.partials;
    p.status = fw.w.status;
    p.total_rows = total_rows;
    p.pos_value = pos_value; p.max_seq_len = max_seq_len;
    p.G = G; p.H = num_heads; p.Hkv = num_kv_heads; p.q_dim = q_dim;
    p.qg = qg; p.qg_tokens = qg_tokens;
    if (qg > 1) {  // groups of query tokens are short sequences: what each costs beside its tiles, in tiles (measured)
        static const int seq_weight = getenv("TQ_PREFILL_SEQ_WEIGHT") ? atoi(getenv("TQ_PREFILL_SEQ_WEIGHT")) : 10;
        p.app_weight = seq_weight < 0 ? 0 : seq_weight;
    }
#ifdef TQ_TIMING_SWITCHES
    static const int debug_mode = getenv("TQ_ATTN_DEBUG") ? atoi(getenv("TQ_ATTN_DEBUG")) : 0;
    p.debug = debug_mode;
#endif
    static const int l2_ahead = getenv("TQ_ATTN_L2_AHEAD") ? atoi(getenv("TQ_ATTN_L2_AHEAD")) : ATTN_L2_AHEAD;
    p.l2_ahead = l2_ahead > 0 ? l2_ahead : (1 << 28);  // 0 switches the prefetch off
    if (fused) {
        p.new_k = (const __half*)fused->k; p.new_v = (const __half*)fused->v; p.new_q = (const __half*)fused->q;
        p.rotation = (const __half*)fused->rotation;
        p.rot_copies = fused->rot_copies;
        p.early = fused->early;
        // what the append of one token costs its worker, in 32-token tiles (measured; TQ_FUSED_WEIGHT overrides)
        static const int app_weight = getenv("TQ_FUSED_WEIGHT") ? atoi(getenv("TQ_FUSED_WEIGHT")) : 7;
        p.app_weight = (!fused->k || app_weight < 0) ? 0 : app_weight;  // nothing to weigh without an append
        p.kv_dim = num_kv_heads * HEAD_DIM; p.capacity_rows = max_seq_len;
        p.seq_capacity = fused->seq_capacity;
    }
    return launch_attention(bits, tmK, tmV, p, attention_ctas(G, max_seq_len), s, pdl, fused != nullptr ? 1 : 0);
}

int tq_decode_attention(void* out, const uint8_t* ck_q, const uint8_t* cv_q, const void* k_norms, const void* v_norms,
                        const void* rotation, const int* positions, int pos_value, const long long* row_base,
                        long long total_rows, int max_seq_len, int G, int num_heads, int num_kv_heads, int head_dim,
                        int q_dim, int kv_dim, int bits, void* workspace, size_t workspace_bytes, tq_stream_t s) {
    int r = check_shape(G, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, true);
    if (r != TQ_OK) return r;
    // (this entry point reads queries that tq_append_decode rotated for the streaming kernel: its head layouts only;
    // the launch_* symbols and the engine serve every layout)
    if (!fast_shape(num_heads, num_kv_heads, true)) return TQ_ERR_UNSUPPORTED;
    if (!out || !ck_q || !cv_q || !k_norms || !v_norms || !rotation) return TQ_ERR_ARG;
    if (!positions && pos_value < 0) return TQ_ERR_ARG;
    if (!workspace) return TQ_ERR_WORKSPACE;
    // this entry point only receives R: transpose it into the workspace for the merge's tensor-core product
    FullWorkspace fw = carve_full(workspace, G, num_heads);
    if (fw.bytes > workspace_bytes) return TQ_ERR_WORKSPACE;
    transpose_rotation_kernel<<<16, 256, 0, cs(s)>>>(fw.rot_t, (const __half*)rotation);
    r = cuda_status(cudaGetLastError());
    if (r != TQ_OK) return r;
    const int kvp = kv_dim / (bits == 2 ? 4 : 2);
    CUtensorMap tmK, tmV;
    {
        std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());  // the descriptor cache is per-device compat state
        r = cached_code_map(&tmK, ck_q, total_rows, kvp);
        if (r != TQ_OK) return r;
        r = cached_code_map(&tmV, cv_q, total_rows, kvp);
        if (r != TQ_OK) return r;
    }
    return attention_impl(out, tmK, tmV, ck_q, cv_q, k_norms, v_norms, fw.rot_t, positions, pos_value, row_base, total_rows,
                          max_seq_len, G, num_heads, num_kv_heads, q_dim, bits, workspace, workspace_bytes, cs(s));
}

__global__ void causal_rows_kernel(int* pos, long long* rows, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        pos[i] = i;   // query token i attends to rows 0 .. i
        rows[i] = 0;  // of the one sequence whose cache starts at row 0
    }
}

// Any head layout: one CTA per (sequence, query head), see tq_generic.cuh.
static int generic_packed_attention(void* out, const void* q, const void* ck_q, const void* cv_q, const void* k_norms,
                                    const void* v_norms, const void* rotation, const int* positions, int pos_value,
                                    const long long* row_base, int max_seq_len, int G, int H, int Hkv, int q_dim, int bits,
                                    cudaStream_t s) {
    if (!out || !q || !ck_q || !cv_q || !k_norms || !v_norms || !rotation) return TQ_ERR_ARG;
    GenericAttnParams p{};
    p.ck = (const uint8_t*)ck_q; p.cv = (const uint8_t*)cv_q; p.kn = (const __half*)k_norms; p.vn = (const __half*)v_norms;
    p.q = (const __half*)q; p.rotation = (const __half*)rotation; p.out = (__half*)out;
    p.positions = positions; p.row_base = row_base; p.pos_value = pos_value; p.max_seq_len = max_seq_len;
    p.G = G; p.H = H; p.Hkv = Hkv; p.q_dim = q_dim; p.bits = bits;
    return launch_generic_attention(p, false, s);
}

// ---- allocation-free decode attention -----------------------------------------------------------------------------------
// Some embedders may not allocate device memory at all once they are running: every byte of the GPU was handed to
// their own pool at start-up (a raw cudaMalloc would fail or fight that pool), or they sit inside a serving loop whose
// latency limits rule out cudaMalloc (it synchronises the whole device).  For them the scratch that the attention kernel needs lives in the library
// image itself: a fixed device array that every GPU loading this library carries until the process exits.
constexpr size_t TQ_STATIC_SCRATCH_BYTES = (size_t)20 << 20;  // 20 MiB: 64 sequences x 32 query heads fit, see the header
static __device__ __align__(256) unsigned char g_static_scratch[TQ_STATIC_SCRATCH_BYTES];

// In host code the name g_static_scratch is only a stand-in for the device array, never a device address.  Its address
// is looked up once per device, with that device current, and handed to the kernels like any other workspace pointer.
static int static_scratch_ptr(void** out) {
    static std::mutex mu;
    static std::map<int, void*> by_device;
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    auto it = by_device.find(dev);
    if (it == by_device.end()) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!ptr) return TQ_ERR_STATE;
        it = by_device.emplace(dev, ptr).first;
    }
    *out = it->second;
    return TQ_OK;
}

int tq_decode_attention_static(void* out, const void* q, const uint8_t* ck_q, const uint8_t* cv_q, const void* k_norms,
                               const void* v_norms, const void* rotation, const int* positions, long long total_rows,
                               int max_seq_len, int G, int num_heads, int num_kv_heads, int head_dim, int q_dim,
                               int kv_dim, int bits, tq_stream_t s) {
    int r = check_shape(G, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, true);
    if (r != TQ_OK) return r;
    if (!fast_shape(num_heads, num_kv_heads, true)) return TQ_ERR_UNSUPPORTED;
    if (!out || !q || !ck_q || !cv_q || !k_norms || !v_norms || !rotation || !positions) return TQ_ERR_ARG;
    // everything that can refuse the call is checked before the first kernel is enqueued
    if ((((uintptr_t)ck_q | (uintptr_t)cv_q | (uintptr_t)k_norms | (uintptr_t)v_norms) & 15u) != 0) return TQ_ERR_ARG;
    if (num_kv_heads % 8 != 0 && ((max_seq_len & 1) || (total_rows & 1))) return TQ_ERR_UNSUPPORTED;
    const size_t need = carve_full(nullptr, G, num_heads).bytes;
    if (need > TQ_STATIC_SCRATCH_BYTES) return TQ_ERR_CAPACITY;  // batch x heads too large for the built-in scratch
    const int kvp = kv_dim / (bits == 2 ? 4 : 2);
    CUtensorMap tmK, tmV;  // encoded on the host stack every call: no cache, nothing allocated
    r = make_code_map(&tmK, ck_q, total_rows, kvp);
    if (r != TQ_OK) return r;
    r = make_code_map(&tmV, cv_q, total_rows, kvp);
    if (r != TQ_OK) return r;
    void* ws = nullptr;
    r = static_scratch_ptr(&ws);  // first call on a device: one symbol lookup
    if (r != TQ_OK) return r;
    // The array keeps whatever the previous call left.  What has to start from zero: the per-sequence tickets, cleared by
    // the rotate kernel below; everything else is written before it is read.  The status word at the start of the array
    // is NOT cleared here: it collects (atomicMax) until tq_static_status reads and clears it.
    FullWorkspace fw = carve_full(ws, G, num_heads);
    transpose_rotation_kernel<<<16, 256, 0, cs(s)>>>(fw.rot_t, (const __half*)rotation);
    r = cuda_status(cudaGetLastError());
    if (r != TQ_OK) return r;
    r = append_impl(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, q, rotation, positions, 0, nullptr, 0, 0,
                    max_seq_len, G, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, ws, need, true, cs(s));
    if (r != TQ_OK) return r;
    return attention_impl(out, tmK, tmV, ck_q, cv_q, k_norms, v_norms, fw.rot_t, positions, -1, nullptr, total_rows,
                          max_seq_len, G, num_heads, num_kv_heads, q_dim, bits, ws, need, cs(s));
}

int tq_static_status(tq_stream_t s) {
    void* ws = nullptr;
    int r = static_scratch_ptr(&ws);
    if (r != TQ_OK) return r;
    return tq_workspace_status(ws, s);  // reads the word, clears it if it was set; synchronises the stream
}

// ---- fp16 twin ---------------------------------------------------------------------------------------------------------
int tq_fp16_append_decode(void* ck, void* cv, const void* k_buf, const void* v_buf, const int* positions,
                          const long long* row_base, int max_seq_len, int G, int kv_dim, tq_stream_t s) {
    if (!ck || !cv || !k_buf || !v_buf || !positions || G <= 0 || kv_dim <= 0 || kv_dim % 8 != 0) return TQ_ERR_ARG;
    fp16_cache_write_kernel<<<G, 128, 0, cs(s)>>>((__half*)ck, (__half*)cv, (const __half*)k_buf, (const __half*)v_buf,
                                                  positions, row_base, max_seq_len, max_seq_len, G, kv_dim, nullptr);
    return cuda_status(cudaGetLastError());
}

int tq_fp16_decode_attention(void* out, const void* q, const void* ck, const void* cv, const int* positions,
                             int pos_value, const long long* row_base, long long total_rows, int max_seq_len, int G,
                             int num_heads, int num_kv_heads, int head_dim, int q_dim, int kv_dim, void* workspace,
                             size_t workspace_bytes, tq_stream_t s) {
    int r = check_shape(G, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, 0, false);
    if (r != TQ_OK) return r;
    if (!out || !q || !ck || !cv) return TQ_ERR_ARG;
    if (!positions && pos_value < 0) return TQ_ERR_ARG;
    if (!fast_shape(num_heads, num_kv_heads, false)) {  // 3, 5, 6, 7 or more than 8 query heads per KV head
        GenericAttnParams gp{};
        gp.ck = (const uint8_t*)ck; gp.cv = (const uint8_t*)cv; gp.q = (const __half*)q; gp.out = (__half*)out;
        gp.positions = positions; gp.row_base = row_base; gp.pos_value = pos_value; gp.max_seq_len = max_seq_len;
        gp.G = G; gp.H = num_heads; gp.Hkv = num_kv_heads; gp.q_dim = q_dim; gp.bits = 0;
        return launch_generic_attention(gp, true, cs(s));
    }
    if (!workspace) return TQ_ERR_WORKSPACE;
    // fp16 layout of the workspace: [0,256) header, tickets int[G*H] (one per sequence and virtual KV head, at most H), partials
    const size_t tick_bytes = align_up((size_t)G * num_heads * sizeof(int), 256);
    const size_t need = 256 + tick_bytes + fp16_partials_bytes(G, num_heads, max_seq_len);
    if (need > workspace_bytes) return TQ_ERR_WORKSPACE;
    char* base = (char*)workspace;
    Fp16AttnParams p{};
    p.q = (const __half*)q; p.ck = (const __half*)ck; p.cv = (const __half*)cv; p.out = (__half*)out;
    p.positions = positions; p.row_base = row_base;
    p.tickets = (int*)(base + 256); p.partials = (float*)(base + 256 + tick_bytes); p.status = (int*)base;
    p.pos_value = pos_value; p.max_seq_len = max_seq_len;
    p.nchunk_max = (max_seq_len + FP16_CHUNK - 1) / FP16_CHUNK;
    p.G = G; p.H = num_heads; p.Hkv = num_kv_heads; p.q_dim = q_dim; p.kv_dim = kv_dim;
    TQ_CUDA(cudaMemsetAsync(p.tickets, 0, (size_t)G * num_heads * sizeof(int), cs(s)));
    // The tensor-core form by default (with four or eight query heads per KV head the fp32-FMA form is bound by its FMAs).
    // TQ_FP16_TC=0 keeps everything on the FMA form, TQ_FP16_TC=1 only one and two heads per KV head.
    static const int tc_mode = getenv("TQ_FP16_TC") ? atoi(getenv("TQ_FP16_TC")) : 2;
    const int grp = num_heads / num_kv_heads;
    if (tc_mode != 0 && (grp >= 4 || tc_mode == 2) && total_rows > 0 && (((uintptr_t)ck | (uintptr_t)cv | (uintptr_t)q) & 15u) == 0 &&
        (kv_dim * 2) % 256 == 0) {
        CUtensorMap tmK, tmV;
        int r2;
        {
            std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());  // the descriptor cache is per-device compat state
            r2 = cached_fp16_map(&tmK, ck, total_rows, kv_dim);
            if (r2 == TQ_OK) r2 = cached_fp16_map(&tmV, cv, total_rows, kv_dim);
        }
        if (r2 == TQ_OK) return launch_fp16_tc_attention(tmK, tmV, p, cs(s));
    }
    return launch_fp16_attention(p, cs(s));
}

static size_t fp16_workspace_bytes(int G, int H, int Hkv, int max_seq_len) {
    return 256 + align_up((size_t)G * H * sizeof(int), 256) + fp16_partials_bytes(G, H, max_seq_len);
}

// ===================================================================================================================
// Reference-compatible launchers
// ===================================================================================================================
void launch_turbo_kv_quantize(uint8_t* cache_q, void* cache_norms, const void* kv_buf, const void* rotation,
                              const int* positions, int max_seq_len, int num_tokens, int num_kv_heads, int head_dim,
                              int kv_dim, int bits, tq_stream_t s) {
    std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());  // per-device compat state, see tq_host.cuh
    void* ws = nullptr;
    const size_t need = carve_full(nullptr, num_tokens > 0 ? num_tokens : 1, 1).bytes;
    int r = compat_workspace(need, &ws, cs(s));
    if (r == TQ_OK)
        r = append_impl(cache_q, cache_norms, nullptr, nullptr, kv_buf, nullptr, nullptr, rotation, positions, 0,
                        nullptr, 1, 0, max_seq_len, num_tokens, 0, num_kv_heads, head_dim, 0, kv_dim,
                        bits == 4 ? 4 : 2, ws, need, false, cs(s));
    g_compat_status = r;
}

void launch_turbo_kv_quantize_batch(uint8_t* cache_q, void* cache_norms, const void* kv_buf, const void* rotation,
                                    const int* positions, int max_seq_len, int G, int num_kv_heads, int head_dim,
                                    int kv_dim, int bits, tq_stream_t s) {
    std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());  // per-device compat state, see tq_host.cuh
    void* ws = nullptr;
    const size_t need = carve_full(nullptr, G > 0 ? G : 1, 1).bytes;
    int r = compat_workspace(need, &ws, cs(s));
    if (r == TQ_OK)
        r = append_impl(cache_q, cache_norms, nullptr, nullptr, kv_buf, nullptr, nullptr, rotation, positions, 0,
                        nullptr, 0, 0, max_seq_len, G, 0, num_kv_heads, head_dim, 0, kv_dim, bits == 4 ? 4 : 2, ws,
                        need, false, cs(s));
    g_compat_status = r;
}

void launch_turbo_gqa_attention_batch(void* out, const void* q, const uint8_t* ck_q, const uint8_t* cv_q,
                                      const void* k_norms, const void* v_norms, const void* rotation, float* as,
                                      const int* pos, int msl, int G, int num_heads, int num_kv_heads, int head_dim,
                                      int q_dim, int kv_dim, int bits, tq_stream_t s) {
    std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());  // per-device compat state, see tq_host.cuh
    (void)as;
    bits = bits == 4 ? 4 : 2;  // the reference treats anything that is not 4 as 2-bit
    int r = check_shape(G, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, true);
    if (r == TQ_OK && !fast_shape(num_heads, num_kv_heads, true)) {
        g_compat_status = pos ? generic_packed_attention(out, q, ck_q, cv_q, k_norms, v_norms, rotation, pos, -1, nullptr, msl, G,
                                                         num_heads, num_kv_heads, q_dim, bits, cs(s))
                              : TQ_ERR_ARG;
        return;
    }
    void* ws = nullptr;
    size_t need = 0;
    if (r == TQ_OK) {
        need = carve_full(nullptr, G, num_heads).bytes;
        r = compat_workspace(need, &ws, cs(s));
    }
    static const bool one_launch = !(getenv("TQ_FUSED") && atoi(getenv("TQ_FUSED")) == 0);
    if (r == TQ_OK && one_launch && G <= FUSED_MAX_G && pos) {
        // one launch: the attention kernel builds its tile table and rotates the queries itself (its fused form without
        // an append); only the transpose of R for the merge precedes it
        if (!q || !out || !ck_q || !cv_q || !k_norms || !v_norms || !rotation) r = TQ_ERR_ARG;
        FullWorkspace fw = carve_full(ws, G, num_heads);
        CUtensorMap tmK, tmV;
        const int kvp = num_kv_heads * (bits == 4 ? 64 : 32);
        if (r == TQ_OK) r = cached_code_map(&tmK, ck_q, (long long)G * msl, kvp);
        if (r == TQ_OK) r = cached_code_map(&tmV, cv_q, (long long)G * msl, kvp);
        if (r == TQ_OK) {
            // (the shared workspace is carved per call: whatever an earlier call left where the tickets now live goes)
            transpose_rotation_kernel<<<16, 256, 0, cs(s)>>>(fw.rot_t, (const __half*)rotation, fw.w.tickets, G);
            r = cuda_status(cudaGetLastError());
        }
        if (r == TQ_OK) {
            FusedInputs in{q, nullptr, nullptr, rotation, 1, 0, nullptr};
            r = attention_impl(out, tmK, tmV, ck_q, cv_q, k_norms, v_norms, fw.rot_t, pos, -1, nullptr, (long long)G * msl, msl, G,
                               num_heads, num_kv_heads, q_dim, bits, ws, need, cs(s), false, &in);
        }
        g_compat_status = r;
        return;
    }
    if (r == TQ_OK)
        r = append_impl(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, q, rotation, pos, 0, nullptr, 0, 0, msl, G,
                        num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, ws, need, true, cs(s));
    if (r == TQ_OK)
        r = tq_decode_attention(out, ck_q, cv_q, k_norms, v_norms, rotation, pos, -1, nullptr, (long long)G * msl, msl,
                                G, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, ws, need, s);
    g_compat_status = r;
}

void launch_turbo_gqa_attention(const void* q, const uint8_t* ck_q, const uint8_t* cv_q, const void* k_norms,
                                const void* v_norms, const void* rotation, void* output, float* as, int pos, int msl,
                                int num_heads, int num_kv_heads, int head_dim, int bits, tq_stream_t s) {
    std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());  // per-device compat state, see tq_host.cuh
    (void)as;
    bits = bits == 4 ? 4 : 2;
    const int q_dim = num_heads * head_dim, kv_dim = num_kv_heads * head_dim;
    int r = check_shape(1, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, true);
    if (r == TQ_OK && (pos < 0 || pos >= msl)) r = TQ_ERR_CAPACITY;
    if (r == TQ_OK && !fast_shape(num_heads, num_kv_heads, true)) {
        g_compat_status = generic_packed_attention(output, q, ck_q, cv_q, k_norms, v_norms, rotation, nullptr, pos, nullptr, msl, 1,
                                                   num_heads, num_kv_heads, q_dim, bits, cs(s));
        return;
    }
    void* ws = nullptr;
    size_t need = 0;
    if (r == TQ_OK) {
        need = carve_full(nullptr, 1, num_heads).bytes;
        r = compat_workspace(need, &ws, cs(s));
    }
    if (r == TQ_OK)
        r = append_impl(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, q, rotation, nullptr, pos, nullptr, 0, 0,
                        msl, 1, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, ws, need, true, cs(s));
    if (r == TQ_OK)
        r = tq_decode_attention(output, ck_q, cv_q, k_norms, v_norms, rotation, nullptr, pos, nullptr, msl, msl, 1,
                                num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, ws, need, s);
    g_compat_status = r;
}

void launch_turbo_gqa_prefill_attention(void* out, const void* q, const uint8_t* ck_q, const uint8_t* cv_q,
                                        const void* k_norms, const void* v_norms, const void* rotation, float* as,
                                        int T, int msl, int num_heads, int num_kv_heads, int head_dim, int q_dim,
                                        int kv_dim, int bits, tq_stream_t s) {
    std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());  // per-device compat state, see tq_host.cuh
    (void)as;
    // Query t attends to rows 0..t of ONE sequence.  The decode kernel serves up to 8 score rows per KV head at the
    // price of one: groups of qg = 8 / (heads per KV head) consecutive query tokens become the "sequences" of the launch,
    // their rows ordered (kv head, token in group, head), each row with its own causal limit.  Every cache tile is then
    // fetched and dequantised once per group instead of once per token.
    bits = bits == 4 ? 4 : 2;
    int r = check_shape(T, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, true);
    if (r == TQ_OK && T > msl) r = TQ_ERR_CAPACITY;
    if (r == TQ_OK && !fast_shape(num_heads, num_kv_heads, true)) {
        // every query token as a "sequence" of its own: position t, row base 0
        void* gws = nullptr;
        const size_t gneed = align_up((size_t)T * sizeof(int), 256) + align_up((size_t)T * sizeof(long long), 256);
        r = compat_workspace(gneed, &gws, cs(s));
        if (r == TQ_OK) {
            int* gpos = (int*)gws;
            long long* grows = (long long*)((char*)gws + align_up((size_t)T * sizeof(int), 256));
            causal_rows_kernel<<<(T + 127) / 128, 128, 0, cs(s)>>>(gpos, grows, T);
            r = cuda_status(cudaGetLastError());
            if (r == TQ_OK)
                r = generic_packed_attention(out, q, ck_q, cv_q, k_norms, v_norms, rotation, gpos, -1, grows, msl, T, num_heads,
                                             num_kv_heads, q_dim, bits, cs(s));
        }
        g_compat_status = r;
        return;
    }
    static const bool dedicated = !(getenv("TQ_PREFILL_ATTN") && atoi(getenv("TQ_PREFILL_ATTN")) == 0);
    if (r == TQ_OK && dedicated && prefill_attn_shape(num_heads, num_kv_heads)) {
        // the kernel with the query tokens in the M dimension: one launch (it rotates its queries, attends, normalises and
        // applies R^T)
        PrefillAttnParams ap{};
        ap.q = (const __half*)q;
        ap.q_tok_stride = q_dim;
        ap.ck = ck_q;
        ap.cv = cv_q;
        ap.kn = (const __half*)k_norms;
        ap.vn = (const __half*)v_norms;
        ap.rotation = (const __half*)rotation;
        {  // the tcgen05 form wants R^T as well: 32 KB of the launchers' workspace, written by a small launch
            void* pws = nullptr;
            r = compat_workspace((size_t)HEAD_DIM * HEAD_DIM * sizeof(__half) + 256, &pws, cs(s));
            if (r == TQ_OK) {
                ap.status = (int*)pws;
                ap.rotation_t = (const __half*)((char*)pws + 256);
                transpose_rotation_kernel<<<16, 256, 0, cs(s)>>>((__half*)((char*)pws + 256), (const __half*)rotation);
                r = cuda_status(cudaGetLastError());
            }
            if (r != TQ_OK) {
                g_compat_status = r;
                return;
            }
        }
        ap.out = (__half*)out;
        ap.q_dim = q_dim;
        ap.T = T;
        ap.rows = msl;
        ap.H = num_heads;
        ap.Hkv = num_kv_heads;
        ap.score_scale = 1.0f;
        r = launch_prefill_attention(bits, ap, cs(s));
        g_compat_status = r;
        return;
    }
    void* ws = nullptr;
    size_t need = 0;
    int qg = 1, groups = T, vheads = num_heads;
    if (r == TQ_OK) {
        const int grp = num_heads / num_kv_heads;
        static const bool grouped = !(getenv("TQ_PREFILL_QG") && atoi(getenv("TQ_PREFILL_QG")) == 0);
        qg = grouped ? 8 / grp : 1;
        if (qg < 1) qg = 1;
        groups = (T + qg - 1) / qg;
        vheads = num_heads * qg;
        need = std::max(carve_full(nullptr, groups, vheads).bytes, carve_full(nullptr, T, num_heads).bytes);
        r = compat_workspace(need, &ws, cs(s));
    }
    if (r == TQ_OK) {
        FullWorkspace fw = carve_full(ws, groups, vheads);
        // rotated queries of all T tokens (positions play no part in that), written in the grouped row order
        r = append_impl(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, q, rotation, nullptr, 0, nullptr, 0, 0, msl, T,
                        num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits, ws, need, false, cs(s), false, nullptr, qg);
        // the tile table of the groups: group j ends at token min((j + 1) * qg, T) - 1; every group starts at row 0
        if (r == TQ_OK) {
            group_rows_kernel<<<(groups + 127) / 128, 128, 0, cs(s)>>>(fw.aux_pos, fw.aux_rows, groups, qg, T);
            r = cuda_status(cudaGetLastError());
        }
        if (r == TQ_OK)
            r = append_impl(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, rotation, fw.aux_pos, 0, fw.aux_rows,
                            0, 0, msl, groups, vheads, num_kv_heads, head_dim, vheads * head_dim, kv_dim, bits, ws, need, true,
                            cs(s));
        if (r == TQ_OK) {
            CUtensorMap tmK, tmV;
            const int kvp = num_kv_heads * (bits == 4 ? 64 : 32);
            r = cached_code_map(&tmK, ck_q, msl, kvp);
            if (r == TQ_OK) r = cached_code_map(&tmV, cv_q, msl, kvp);
            if (r == TQ_OK) {
                transpose_rotation_kernel<<<16, 256, 0, cs(s)>>>(fw.rot_t, (const __half*)rotation);
                r = cuda_status(cudaGetLastError());
            }
            if (r == TQ_OK)
                r = attention_impl(out, tmK, tmV, ck_q, cv_q, k_norms, v_norms, fw.rot_t, fw.aux_pos, -1, fw.aux_rows, msl, msl,
                                   groups, vheads, num_kv_heads, q_dim, bits, ws, need, cs(s), false, nullptr, qg, T);
        }
    }
    g_compat_status = r;
}

void launch_kv_cache_write_batch(void* ck, void* cv, const void* k, const void* v, const int* pos, int msl, int G,
                                 int kv_dim, tq_stream_t s) {
    g_compat_status = tq_fp16_append_decode(ck, cv, k, v, pos, nullptr, msl, G, kv_dim, s);
}

void launch_gqa_attention_batch(void* out, const void* q, const void* ck, const void* cv, float* as, const int* pos,
                                int msl, int G, int num_heads, int num_kv_heads, int head_dim, int q_dim, int kv_dim,
                                tq_stream_t s) {
    std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());  // per-device compat state, see tq_host.cuh
    (void)as;
    void* ws = nullptr;
    int r = check_shape(G, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, 0, false);
    size_t need = 0;
    if (r == TQ_OK) {
        need = fp16_workspace_bytes(G, num_heads, num_kv_heads, msl);
        r = compat_workspace(need, &ws, cs(s));
    }
    if (r == TQ_OK)
        r = tq_fp16_decode_attention(out, q, ck, cv, pos, -1, nullptr, (long long)G * msl, msl, G, num_heads,
                                     num_kv_heads, head_dim, q_dim, kv_dim, ws, need, s);
    g_compat_status = r;
}

void launch_gqa_attention(const void* q, const void* k_cache, const void* v_cache, void* output, float* attn_scratch,
                          int pos, int max_seq_len, int num_heads, int num_kv_heads, int head_dim, tq_stream_t stream) {
    std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());  // per-device compat state, see tq_host.cuh
    (void)attn_scratch;
    const int q_dim = num_heads * head_dim, kv_dim = num_kv_heads * head_dim;
    void* ws = nullptr;
    int r = check_shape(1, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, 0, false);
    if (r == TQ_OK && (pos < 0 || pos >= max_seq_len)) r = TQ_ERR_CAPACITY;
    size_t need = 0;
    if (r == TQ_OK) {
        need = fp16_workspace_bytes(1, num_heads, num_kv_heads, max_seq_len);
        r = compat_workspace(need, &ws, cs(stream));
    }
    if (r == TQ_OK)
        r = tq_fp16_decode_attention(output, q, k_cache, v_cache, nullptr, pos, nullptr, max_seq_len, max_seq_len, 1,
                                     num_heads, num_kv_heads, head_dim, q_dim, kv_dim, ws, need, stream);
    g_compat_status = r;
}

// Causal prefill attention over an fp16 cache (kv_bits = 0), replaces launch_gqa_prefill_attention
// (engine/kernels.cu:1071-1158, 1359-1362): query token t of ONE sequence attends to cache rows 0 .. t.  Served by the
// fp16 decode kernel with every query token as a "sequence" of its own (position t, row base 0): no O(T^2) score scratch.
void launch_gqa_prefill_attention(void* out, const void* q, const void* ck, const void* cv, float* as, int T, int msl,
                                  int num_heads, int num_kv_heads, int head_dim, int q_dim, int kv_dim, tq_stream_t s) {
    std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());  // per-device compat state, see tq_host.cuh
    (void)as;
    int r = check_shape(T, num_heads, num_kv_heads, head_dim, q_dim, kv_dim, 0, false);
    if (r == TQ_OK && T > msl) r = TQ_ERR_CAPACITY;
    static const bool dedicated = !(getenv("TQ_PREFILL_ATTN") && atoi(getenv("TQ_PREFILL_ATTN")) == 0);
    if (r == TQ_OK && dedicated && prefill_attn_shape(num_heads, num_kv_heads) && kv_dim == num_kv_heads * HEAD_DIM) {
        PrefillAttnParams ap{};
        ap.q = (const __half*)q;
        ap.q_tok_stride = q_dim;
        ap.ck = (const uint8_t*)ck;
        ap.cv = (const uint8_t*)cv;
        ap.out = (__half*)out;
        ap.q_dim = q_dim;
        ap.T = T;
        ap.rows = msl;
        ap.H = num_heads;
        ap.Hkv = num_kv_heads;
        ap.score_scale = 0.12751743074602467f;  // log2(e) / sqrt(128)
        g_compat_status = launch_prefill_attention(0, ap, cs(s));
        return;
    }
    void* ws = nullptr;
    size_t attn_bytes = 0, need = 0;
    if (r == TQ_OK) {
        attn_bytes = align_up(fp16_workspace_bytes(T, num_heads, num_kv_heads, msl), 256);
        need = attn_bytes + align_up((size_t)T * sizeof(int), 256) + align_up((size_t)T * sizeof(long long), 256);
        r = compat_workspace(need, &ws, cs(s));
    }
    if (r == TQ_OK) {
        int* pos = (int*)((char*)ws + attn_bytes);
        long long* rows = (long long*)((char*)pos + align_up((size_t)T * sizeof(int), 256));
        causal_rows_kernel<<<(T + 127) / 128, 128, 0, cs(s)>>>(pos, rows, T);
        r = cuda_status(cudaGetLastError());
        if (r == TQ_OK)
            r = tq_fp16_decode_attention(out, q, ck, cv, pos, -1, rows, msl, msl, T, num_heads, num_kv_heads, head_dim, q_dim,
                                         kv_dim, ws, attn_bytes, s);
    }
    g_compat_status = r;
}

// ===================================================================================================================
// Engine / arena
// ===================================================================================================================
int tq_engine_create(const tq_model_shape* shape, int max_seq_len, int kv_bits, tq_engine** out) {
    if (!shape || !out) return TQ_ERR_ARG;
    if (shape->num_layers <= 0 || shape->num_heads <= 0 || shape->num_kv_heads <= 0 ||
        shape->num_heads % shape->num_kv_heads != 0 || max_seq_len <= 0)
        return TQ_ERR_ARG;
    if (shape->head_dim != HEAD_DIM) return TQ_ERR_UNSUPPORTED;
    if (kv_bits != 0 && kv_bits != 2 && kv_bits != 4) {
        fprintf(stderr, "WARNING: kv_bits=%d not supported, using 0 (fp16)\n", kv_bits);
        kv_bits = 0;
    }
    tq_engine* e = new (std::nothrow) tq_engine();
    if (!e) return TQ_ERR_NOMEM;
    e->shape = *shape;
    e->ctor_max_seq_len = max_seq_len;
    e->kv_bits = kv_bits;
    cudaGetDevice(&e->device);
    e->h_rotation.resize((size_t)HEAD_DIM * HEAD_DIM);
    tq_rotation_generate(42, e->h_rotation.data());
    e->layers.resize(shape->num_layers);
    *out = e;
    return TQ_OK;
}

// R and its transpose (for the merge's tensor-core product) to the device; both live outside the arena.
constexpr int ROT_COPIES = 32;

static int engine_upload_rotation(tq_engine* e, cudaStream_t s) {
    const size_t bytes = e->h_rotation.size() * 2;
    if (!e->d_rotation) TQ_CUDA(cudaMalloc(&e->d_rotation, bytes));
    if (!e->d_rotation_t) TQ_CUDA(cudaMalloc(&e->d_rotation_t, bytes));
    std::vector<uint16_t> t(e->h_rotation.size());
    for (int k = 0; k < HEAD_DIM; ++k)
        for (int d = 0; d < HEAD_DIM; ++d) t[(size_t)d * HEAD_DIM + k] = e->h_rotation[(size_t)k * HEAD_DIM + d];
    TQ_CUDA(cudaMemcpyAsync(e->d_rotation, e->h_rotation.data(), bytes, cudaMemcpyHostToDevice, s));
    TQ_CUDA(cudaMemcpyAsync(e->d_rotation_t, t.data(), bytes, cudaMemcpyHostToDevice, s));
    // R as fp32 in the append kernel's shared-memory order [k/4][d][k%4], so that the kernel stages it with one copy
    if (!e->d_rotation_prep) TQ_CUDA(cudaMalloc(&e->d_rotation_prep, (size_t)HEAD_DIM * HEAD_DIM * sizeof(float)));
    std::vector<float> prep((size_t)HEAD_DIM * HEAD_DIM);
    for (int d = 0; d < HEAD_DIM; ++d)
        for (int k = 0; k < HEAD_DIM; ++k) {
            __half_raw raw;
            raw.x = e->h_rotation[(size_t)d * HEAD_DIM + k];
            prep[((size_t)(k / 4) * HEAD_DIM + d) * 4 + (k % 4)] = __half2float(__half(raw));
        }
    TQ_CUDA(cudaMemcpyAsync(e->d_rotation_prep, prep.data(), prep.size() * sizeof(float), cudaMemcpyHostToDevice, s));
    // For the fused kernel: ROT_COPIES copies of R back to back.  Every worker of the kernel reads all of R at the same
    // moment; with one copy those reads queue up on the same L2 lines.
    if (!e->d_rotation_rep) TQ_CUDA(cudaMalloc(&e->d_rotation_rep, bytes * ROT_COPIES));
    for (int c = 0; c < ROT_COPIES; ++c)
        TQ_CUDA(cudaMemcpyAsync((char*)e->d_rotation_rep + bytes * c, e->h_rotation.data(), bytes, cudaMemcpyHostToDevice, s));
    TQ_CUDA(cudaStreamSynchronize(s));  // t and h_rotation are pageable host memory
    return TQ_OK;
}

static void engine_release_arena(tq_engine* e) {
    if (e->arena && !e->arena_external) cudaFree(e->arena);
    e->arena = nullptr;
    e->arena_cap = 0;
    e->arena_external = false;
    e->G = 0;
    e->total_rows = 0;
    e->d_positions = nullptr;
    e->d_capacities = nullptr;
    e->d_row_base = nullptr;
    e->d_prefix_base = nullptr;
    e->d_prefix_tiles = nullptr;
    e->shared_active = false;
    e->step_partials = nullptr;
    e->step_table = nullptr;
    e->step_qrot = nullptr;
    e->step_kpost = nullptr;
    e->workspace = nullptr;
    for (auto& l : e->layers) l = tq_engine::Layer();
}

void tq_engine_destroy(tq_engine* e) {
    if (e && e->ev_attn[0]) {
        cudaEventDestroy(e->ev_attn[0]);
        cudaEventDestroy(e->ev_attn[1]);
        e->ev_attn[0] = e->ev_attn[1] = nullptr;
    }
    if (!e) return;
    engine_release_arena(e);
    if (e->d_rotation) cudaFree(e->d_rotation);
    if (e->d_rotation_t) cudaFree(e->d_rotation_t);
    if (e->d_rotation_prep) cudaFree(e->d_rotation_prep);
    if (e->d_rotation_rep) cudaFree(e->d_rotation_rep);
    if (e->out_f32) cudaFree(e->out_f32);
    if (e->st_in) {
        cudaStreamDestroy(e->st_in);
        cudaStreamDestroy(e->st_out);
        cudaEventDestroy(e->ev_begin);
        cudaEventDestroy(e->ev_done);
        for (int c = 0; c < tq_engine::HOST_STEP_CHUNKS; ++c) {
            cudaEventDestroy(e->ev_in[c]);
            cudaEventDestroy(e->ev_out[c]);
        }
    }
    delete e;
}

int tq_engine_kv_bits(const tq_engine* e) { return e ? e->kv_bits : TQ_ERR_ARG; }

int tq_engine_set_fused(tq_engine* e, int on) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e) return TQ_ERR_ARG;
    const int prev = e->fused ? 1 : 0;
    e->fused = on != 0;
    return prev;
}

// An engine belongs to the device that was current when it was created; every call that launches work checks it.
static bool engine_on_its_device(const tq_engine* e) {
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess && dev == e->device;
}

// One walk of the arena; with base == nullptr it only measures.
static size_t engine_carve(tq_engine* e, char* base, int G, int msl, long long rows, bool ragged, bool assign) {
    size_t off = 0;
    const size_t code_bytes = (size_t)rows * e->code_row_bytes();
    const size_t norm_bytes = (size_t)rows * e->shape.num_kv_heads * 2;
    for (int l = 0; l < e->shape.num_layers; ++l) {
        size_t ok = bump(off, code_bytes);
        size_t ov = bump(off, code_bytes);
        size_t okn = 0, ovn = 0;
        if (e->kv_bits != 0) {
            okn = bump(off, norm_bytes);
            ovn = bump(off, norm_bytes);
        }
        if (assign) {
            tq_engine::Layer& L = e->layers[l];
            L.k = base + ok;
            L.v = base + ov;
            L.kn = e->kv_bits ? base + okn : nullptr;
            L.vn = e->kv_bits ? base + ovn : nullptr;
        }
    }
    size_t opos = bump(off, (size_t)G * sizeof(int));
    size_t ocap = bump(off, (size_t)G * sizeof(int));
    size_t orb = bump(off, (size_t)G * sizeof(long long));
    size_t opb = bump(off, (size_t)G * sizeof(long long));
    size_t opt = bump(off, (size_t)G * sizeof(int));
    // whole-step form (packed modes): per-layer split-K partials and the tile table handed to the merge kernel
    const size_t part_stride = e->kv_bits ? (size_t)(attention_ctas(G, msl) * ATTN_GROUPS + G) * e->shape.num_heads * PART_STRIDE : 0;
    size_t osp = bump(off, part_stride * e->shape.num_layers * sizeof(float));
    size_t ost = bump(off, (size_t)(G + 4) * sizeof(int));
    size_t osq = bump(off, e->kv_bits ? (size_t)e->shape.num_layers * G * e->shape.num_heads * HEAD_DIM * 2 : 0);
    size_t okp = bump(off, e->kv_bits ? (size_t)e->shape.num_layers * G * e->kv_dim() * 2 : 0);
    size_t ws_bytes = e->kv_bits ? carve_full(nullptr, G, e->shape.num_heads).bytes
                                 : fp16_workspace_bytes(G, e->shape.num_heads, e->shape.num_kv_heads, msl);
    size_t ows = bump(off, ws_bytes);
    const size_t qb = (size_t)e->shape.num_layers * G * e->q_dim() * 2;
    const size_t kb = (size_t)e->shape.num_layers * G * e->kv_dim() * 2;
    size_t oq = bump(off, qb), okk = bump(off, kb), ovv = bump(off, kb), oo = bump(off, qb);
    if (assign) {
        e->d_positions = (int*)(base + opos);
        e->d_capacities = (int*)(base + ocap);
        e->d_row_base = (long long*)(base + orb);
        e->d_prefix_base = (long long*)(base + opb);
        e->d_prefix_tiles = (int*)(base + opt);
        e->step_partials = e->kv_bits ? (float*)(base + osp) : nullptr;
        e->step_part_stride = part_stride;
        e->step_table = (int*)(base + ost);
        e->step_qrot = base + osq;
        e->step_kpost = base + okp;
        e->workspace = base + ows;
        e->ws_bytes = ws_bytes;
        e->stage_q = base + oq;
        e->stage_k = base + okk;
        e->stage_v = base + ovv;
        e->stage_out = base + oo;
    }
    return (off + 255) & ~(size_t)255;
}

size_t tq_engine_arena_bytes(const tq_engine* e, int G, int max_seq_len, const int* capacities) {
    if (!e || G <= 0 || max_seq_len <= 0) return 0;
    long long rows = plan_rows(G, max_seq_len, capacities, nullptr, nullptr);
    return engine_carve(const_cast<tq_engine*>(e), nullptr, G, max_seq_len, rows, capacities != nullptr, false);
}

int tq_engine_set_arena(tq_engine* e, void* device_ptr, size_t bytes) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e || !device_ptr || bytes == 0) return TQ_ERR_ARG;
    if (((uintptr_t)device_ptr & 255u) != 0) return TQ_ERR_ARG;
    engine_release_arena(e);  // frees only memory this library allocated
    e->arena = (char*)device_ptr;
    e->arena_cap = bytes;
    e->arena_external = true;
    e->asleep = false;
    return TQ_OK;
}

static int engine_restore_kept(tq_engine* e);

int tq_engine_alloc_batch(tq_engine* e, int G, int max_seq_len, const int* capacities) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e || G <= 0 || max_seq_len <= 0) return TQ_ERR_ARG;
    if (e->asleep) return TQ_ERR_STATE;
    if (!engine_on_its_device(e)) return TQ_ERR_STATE;
    int r = check_shape(G, e->shape.num_heads, e->shape.num_kv_heads, e->shape.head_dim, e->q_dim(), e->kv_dim(),
                        e->kv_bits, e->kv_bits != 0);
    if (r != TQ_OK) return r;
    const bool ragged = capacities != nullptr;
    // Like alloc_batch (engine/engine.cpp:1338-1443) the arena is re-carved for every new batch shape and
    // only re-allocated when it is too small.
    std::vector<int> caps;
    std::vector<long long> bases;
    long long rows = plan_rows(G, max_seq_len, capacities, &caps, &bases);
    if (rows >= (1ll << 31)) return TQ_ERR_CAPACITY;
    int msl = max_seq_len;
    for (int c : caps) msl = c > msl ? c : msl;
    size_t need = engine_carve(e, nullptr, G, msl, rows, ragged, false);
    if (need > e->arena_cap) {
        if (e->arena_external) return TQ_ERR_CAPACITY;  // never free or replace caller-owned memory
        if (e->arena) {
            cudaDeviceSynchronize();
            cudaFree(e->arena);
            e->arena = nullptr;
            e->arena_cap = 0;
        }
        void* p = nullptr;
        cudaError_t ce = cudaMalloc(&p, need);
        if (ce != cudaSuccess) {
            cudaGetLastError();
            return TQ_ERR_NOMEM;
        }
        e->arena = (char*)p;
        e->arena_cap = need;
    }
    if (e->out_f32 && G != e->G) {  // sized for the previous batch
        cudaFree(e->out_f32);
        e->out_f32 = nullptr;
    }
    e->G = G;
    e->msl = msl;
    e->ragged = ragged;
    e->total_rows = rows;
    e->capacities = caps;
    e->h_row_base = bases;
    engine_carve(e, e->arena, G, msl, rows, ragged, true);
    TQ_CUDA(cudaMemset(e->d_positions, 0, (size_t)G * sizeof(int)));
    TQ_CUDA(cudaMemset(e->workspace, 0, e->ws_bytes));
    e->prefix_tokens.assign(G, 0);
    e->prefix_owner.assign(G, -1);
    e->shared_active = false;
    TQ_CUDA(cudaMemcpy(e->d_row_base, bases.data(), (size_t)G * sizeof(long long), cudaMemcpyHostToDevice));
    TQ_CUDA(cudaMemcpy(e->d_capacities, caps.data(), (size_t)G * sizeof(int), cudaMemcpyHostToDevice));
    TQ_CUDA(cudaMemset(e->d_prefix_base, 0, (size_t)G * sizeof(long long)));
    TQ_CUDA(cudaMemset(e->d_prefix_tiles, 0, (size_t)G * sizeof(int)));
    if (!e->d_rotation) {
        int ur = engine_upload_rotation(e, nullptr);
        if (ur != TQ_OK) return ur;
    }
    if (e->kv_bits != 0 && fast_shape(e->shape.num_heads, e->shape.num_kv_heads, true)) {
        // (other head layouts take the generic kernel, which reads the cache with plain loads: no descriptors)
        const int kvp = e->kv_dim() / e->vpb();
        for (auto& L : e->layers) {
            r = make_code_map(&L.tmK, L.k, rows, kvp);
            if (r != TQ_OK) return r;
            r = make_code_map(&L.tmV, L.v, rows, kvp);
            if (r != TQ_OK) return r;
        }
        // every layer is carved alike, so consecutive layers' arrays lie a constant distance apart
        const int NL = e->shape.num_layers;
        e->code_layer_stride = NL > 1 ? (size_t)((char*)e->layers[1].k - (char*)e->layers[0].k) : (size_t)rows * kvp;
        e->norm_layer_stride = NL > 1 ? (size_t)((char*)e->layers[1].kn - (char*)e->layers[0].kn) : (size_t)rows * e->shape.num_kv_heads * 2;
        r = make_code_map_layers(&e->tmK4, e->layers[0].k, rows, kvp, NL, e->code_layer_stride);
        if (r != TQ_OK) return r;
        r = make_code_map_layers(&e->tmV4, e->layers[0].v, rows, kvp, NL, e->code_layer_stride);
        if (r != TQ_OK) return r;
    }
    return e->kept.valid ? engine_restore_kept(e) : TQ_OK;
}

int tq_engine_reset(tq_engine* e, int zero_cache, tq_stream_t s) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e) return TQ_ERR_ARG;
    if (!e->arena || e->G == 0) return TQ_OK;
    TQ_CUDA(cudaMemsetAsync(e->d_positions, 0, (size_t)e->G * sizeof(int), cs(s)));
    if (zero_cache) {
        const size_t code_bytes = (size_t)e->total_rows * e->code_row_bytes();
        const size_t norm_bytes = (size_t)e->total_rows * e->shape.num_kv_heads * 2;
        for (auto& L : e->layers) {
            TQ_CUDA(cudaMemsetAsync(L.k, 0, code_bytes, cs(s)));
            TQ_CUDA(cudaMemsetAsync(L.v, 0, code_bytes, cs(s)));
            if (L.kn) TQ_CUDA(cudaMemsetAsync(L.kn, 0, norm_bytes, cs(s)));
            if (L.vn) TQ_CUDA(cudaMemsetAsync(L.vn, 0, norm_bytes, cs(s)));
        }
    }
    return TQ_OK;
}

int tq_engine_sleep(tq_engine* e) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e) return TQ_ERR_ARG;
    TQ_CUDA(cudaDeviceSynchronize());
    engine_release_arena(e);
    e->kept = tq_engine::Kept();
    e->asleep = true;
    return TQ_OK;
}

int tq_engine_wake(tq_engine* e) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e) return TQ_ERR_ARG;
    e->asleep = false;  // the arena comes back lazily with the next tq_engine_alloc_batch, as in the reference
    if (e->kept.valid && !e->arena) {
        // sequences were kept (tq_engine_sleep_keep) and no caller-owned arena is pending: re-create the batch now
        const tq_engine::Kept& k = e->kept;
        std::vector<int> caps = k.capacities;
        return tq_engine_alloc_batch(e, k.G, k.max_seq_len, k.ragged ? caps.data() : nullptr);
    }
    return TQ_OK;
}

// ---- cache persistence: a sequence's rows as a self-describing blob -----------------------------------------------------------
// Blob = header (8 x int32: magic, version, kv_bits, layers, kv heads, head_dim, tokens, 0), then per layer the rows
// 0 .. tokens-1 of the four arrays in the on-cache byte layout: K codes [tokens][kvp], V codes, K norms [tokens][Hkv]
// fp16, V norms (packed modes) or K rows [tokens][kv_dim] fp16, V rows (kv_bits = 0).  The same bytes the attention
// kernels read, so a blob can go to disk, to another engine or to another slot and back without re-quantising anything.
constexpr int TQ_BLOB_MAGIC = 0x564b5154;  // "TQKV"
constexpr int TQ_BLOB_VERSION = 1;
constexpr size_t TQ_BLOB_HEADER = 8 * sizeof(int);

size_t tq_engine_sequence_blob_bytes(const tq_engine* e, int n_tokens) {
    if (!e || n_tokens < 0) return 0;
    const size_t per_token = 2 * e->code_row_bytes() + (e->kv_bits ? 2 * (size_t)e->shape.num_kv_heads * 2 : 0);
    return TQ_BLOB_HEADER + (size_t)e->shape.num_layers * per_token * (size_t)n_tokens;
}


int tq_engine_export_sequence(tq_engine* e, int seq, int n_tokens, void* host_blob, size_t blob_bytes, tq_stream_t s) {
    if (!e || !host_blob || seq < 0 || n_tokens < 0) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || seq >= e->G || !engine_on_its_device(e)) return TQ_ERR_STATE;
    if (n_tokens > e->cap_eff(seq)) return TQ_ERR_CAPACITY;
    if (blob_bytes < tq_engine_sequence_blob_bytes(e, n_tokens)) return TQ_ERR_CAPACITY;
    int* hdr = (int*)host_blob;
    hdr[0] = TQ_BLOB_MAGIC; hdr[1] = TQ_BLOB_VERSION; hdr[2] = e->kv_bits; hdr[3] = e->shape.num_layers;
    hdr[4] = e->shape.num_kv_heads; hdr[5] = e->shape.head_dim; hdr[6] = n_tokens; hdr[7] = 0;
    char* dst = (char*)host_blob + TQ_BLOB_HEADER;
    const size_t crow = e->code_row_bytes(), nrow = (size_t)e->shape.num_kv_heads * 2;
    // tokens below the shared prefix length come from the owner's slot, the rest from the sequence's own
    const int shared = std::min(n_tokens, e->prefix_tokens[seq]);
    const long long row_shared = shared ? e->h_row_base[e->prefix_owner[seq]] : 0, row_own = e->h_row_base[seq];
    for (const auto& L : e->layers) {
        const void* arrays[4] = {L.k, L.v, L.kn, L.vn};
        const size_t pitch[4] = {crow, crow, nrow, nrow};
        for (int a = 0; a < (e->kv_bits ? 4 : 2); ++a) {
            const size_t b0 = pitch[a] * (size_t)shared, b1 = pitch[a] * (size_t)(n_tokens - shared);
            if (b0) TQ_CUDA(cudaMemcpyAsync(dst, (const char*)arrays[a] + (size_t)row_shared * pitch[a], b0, cudaMemcpyDeviceToHost, cs(s)));
            if (b1) TQ_CUDA(cudaMemcpyAsync(dst + b0, (const char*)arrays[a] + (size_t)row_own * pitch[a], b1, cudaMemcpyDeviceToHost, cs(s)));
            dst += b0 + b1;
        }
    }
    return cuda_status(cudaStreamSynchronize(cs(s)));
}

int tq_engine_import_sequence(tq_engine* e, int seq, const void* host_blob, size_t blob_bytes, tq_stream_t s) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e || !host_blob || seq < 0 || blob_bytes < TQ_BLOB_HEADER) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || seq >= e->G || !engine_on_its_device(e)) return TQ_ERR_STATE;
    const int* hdr = (const int*)host_blob;
    if (hdr[0] != TQ_BLOB_MAGIC || hdr[1] != TQ_BLOB_VERSION) return TQ_ERR_ARG;
    if (hdr[2] != e->kv_bits || hdr[3] != e->shape.num_layers || hdr[4] != e->shape.num_kv_heads || hdr[5] != e->shape.head_dim)
        return TQ_ERR_UNSUPPORTED;  // written by an engine of another shape or cache mode
    const int n_tokens = hdr[6];
    if (n_tokens < 0 || n_tokens > e->capacities[seq]) return TQ_ERR_CAPACITY;
    if (blob_bytes < tq_engine_sequence_blob_bytes(e, n_tokens)) return TQ_ERR_ARG;
    for (int g = 0; g < e->G; ++g)
        if (e->prefix_tokens[g] > 0 && e->prefix_owner[g] == seq) return TQ_ERR_STATE;  // other sequences read this slot's prompt
    if (e->prefix_tokens[seq] > 0) {  // the imported rows are the slot's own from token 0 on: it stops sharing
        e->prefix_tokens[seq] = 0;
        e->prefix_owner[seq] = -1;
        const long long rb0 = e->h_row_base[seq];
        const int cap0 = e->capacities[seq], zero = 0;
        TQ_CUDA(cudaMemcpyAsync(e->d_row_base + seq, &rb0, sizeof(rb0), cudaMemcpyHostToDevice, cs(s)));
        TQ_CUDA(cudaMemcpyAsync(e->d_capacities + seq, &cap0, sizeof(cap0), cudaMemcpyHostToDevice, cs(s)));
        TQ_CUDA(cudaMemcpyAsync(e->d_prefix_tiles + seq, &zero, sizeof(zero), cudaMemcpyHostToDevice, cs(s)));
        TQ_CUDA(cudaStreamSynchronize(cs(s)));  // the sources are locals of this frame
    }
    const char* src = (const char*)host_blob + TQ_BLOB_HEADER;
    const size_t crow = e->code_row_bytes(), nrow = (size_t)e->shape.num_kv_heads * 2;
    const long long row0 = e->h_row_base[seq];
    for (const auto& L : e->layers) {
        void* arrays[4] = {L.k, L.v, L.kn, L.vn};
        const size_t pitch[4] = {crow, crow, nrow, nrow};
        for (int a = 0; a < (e->kv_bits ? 4 : 2); ++a) {
            const size_t bytes = pitch[a] * (size_t)n_tokens;
            if (bytes) TQ_CUDA(cudaMemcpyAsync((char*)arrays[a] + (size_t)row0 * pitch[a], src, bytes, cudaMemcpyHostToDevice, cs(s)));
            src += bytes;
        }
    }
    // the sequence continues where the blob ends: its next token goes to position n_tokens
    TQ_CUDA(cudaMemcpyAsync(e->d_positions + seq, &hdr[6], sizeof(int), cudaMemcpyHostToDevice, cs(s)));
    return cuda_status(cudaStreamSynchronize(cs(s)));
}

// sleep() that keeps the sequences: their written rows (0 .. position-1) go to host memory, the arena is released as
// tq_engine_sleep does; tq_engine_wake (internal arena) or the next tq_engine_alloc_batch of the same batch shape
// (external arena: after tq_engine_set_arena) brings rows and positions back.  Decoding then continues without
// re-running the prompts.
int tq_engine_sleep_keep(tq_engine* e) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || e->G == 0 || !engine_on_its_device(e)) return TQ_ERR_STATE;
    TQ_CUDA(cudaDeviceSynchronize());
    tq_engine::Kept k;
    k.G = e->G; k.ragged = e->ragged; k.capacities = e->capacities;
    k.positions.resize(e->G);
    TQ_CUDA(cudaMemcpy(k.positions.data(), e->d_positions, (size_t)e->G * sizeof(int), cudaMemcpyDeviceToHost));
    k.blobs.resize(e->G);
    for (int g = 0; g < e->G; ++g) {
        const int n = std::max(0, std::min(k.positions[g], e->cap_eff(g)));
        k.blobs[g].resize(tq_engine_sequence_blob_bytes(e, n));
        int r = tq_engine_export_sequence(e, g, n, k.blobs[g].data(), k.blobs[g].size(), nullptr);
        if (r != TQ_OK) return r;
    }
    k.max_seq_len = e->msl;  // (ragged: the largest capacity; the carving comes out the same)
    k.valid = true;
    engine_release_arena(e);
    e->kept = std::move(k);
    e->asleep = true;
    return TQ_OK;
}

// Called at the end of tq_engine_alloc_batch: a batch of the shape that went to sleep gets its sequences back.
static int engine_restore_kept(tq_engine* e) {
    tq_engine::Kept k = std::move(e->kept);
    e->kept = tq_engine::Kept();
    if (!k.valid || k.G != e->G || k.ragged != e->ragged) return TQ_OK;  // another batch: the kept sequences are dropped
    for (int g = 0; g < e->G; ++g) {
        const int n = ((const int*)k.blobs[g].data())[6];
        if (n > e->capacities[g]) return TQ_OK;  // does not fit the new slots (a shared prefix comes back as own rows): dropped
    }
    for (int g = 0; g < e->G; ++g) {
        int r = tq_engine_import_sequence(e, g, k.blobs[g].data(), k.blobs[g].size(), nullptr);
        if (r != TQ_OK) return r;
    }
    // positions as they were (import sets position = tokens, which is the same unless a position was out of range)
    return cuda_status(cudaMemcpy(e->d_positions, k.positions.data(), (size_t)e->G * sizeof(int), cudaMemcpyHostToDevice));
}

int tq_engine_status(tq_engine* e, tq_stream_t s) {
    if (!e) return TQ_ERR_ARG;
    if (!e->arena || !e->workspace) return TQ_OK;
    return tq_workspace_status(e->workspace, s);
}

int* tq_engine_positions(tq_engine* e) { return e ? e->d_positions : nullptr; }

int tq_engine_set_positions(tq_engine* e, const int* host_positions, int G, tq_stream_t s) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e || !host_positions) return TQ_ERR_ARG;
    if (!e->arena || G != e->G) return TQ_ERR_STATE;
    for (int g = 0; g < G; ++g) {
        if (host_positions[g] < 0 || host_positions[g] >= e->cap_eff(g)) return TQ_ERR_CAPACITY;
    }
    TQ_CUDA(cudaMemcpyAsync(e->d_positions, host_positions, (size_t)G * sizeof(int), cudaMemcpyHostToDevice, cs(s)));
    return TQ_OK;
}

__global__ void advance_positions_kernel(int* pos, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) pos[i] += 1;
}

int tq_engine_advance(tq_engine* e, tq_stream_t s) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e || !e->arena || e->G == 0) return TQ_ERR_STATE;
    advance_positions_kernel<<<(e->G + 127) / 128, 128, 0, cs(s)>>>(e->d_positions, e->G);
    return cuda_status(cudaGetLastError());
}

int tq_engine_layer_ptrs(tq_engine* e, int layer, void** k_codes, void** v_codes, void** k_norms, void** v_norms,
                         long long* total_rows) {
    if (!e || layer < 0 || layer >= e->shape.num_layers) return TQ_ERR_ARG;
    if (!e->arena || e->G == 0) return TQ_ERR_STATE;
    const tq_engine::Layer& L = e->layers[layer];
    if (k_codes) *k_codes = L.k;
    if (v_codes) *v_codes = L.v;
    if (k_norms) *k_norms = L.kn;
    if (v_norms) *v_norms = L.vn;
    if (total_rows) *total_rows = e->total_rows;
    return TQ_OK;
}

const long long* tq_engine_row_base(tq_engine* e) { return e ? e->rb() : nullptr; }
const void* tq_engine_rotation(tq_engine* e) { return e ? e->d_rotation : nullptr; }

int tq_engine_set_rotation(tq_engine* e, const void* host_half, tq_stream_t s) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e || !host_half) return TQ_ERR_ARG;
    memcpy(e->h_rotation.data(), host_half, e->h_rotation.size() * 2);
    return engine_upload_rotation(e, cs(s));
}

int tq_engine_output_f32(tq_engine* e, int enable) {
    if (!e) return TQ_ERR_ARG;
    if (!enable) {
        if (e->out_f32) cudaFree(e->out_f32);
        e->out_f32 = nullptr;
        return TQ_OK;
    }
    if (e->kv_bits == 0 || !e->arena || e->G == 0) return TQ_ERR_STATE;
    if (e->out_f32) cudaFree(e->out_f32);
    e->out_f32 = nullptr;
    const size_t bytes = (size_t)e->shape.num_layers * e->G * e->shape.num_heads * HEAD_DIM * sizeof(float);
    if (cudaMalloc(&e->out_f32, bytes) != cudaSuccess) {
        cudaGetLastError();
        return TQ_ERR_NOMEM;
    }
    return cuda_status(cudaMemset(e->out_f32, 0, bytes));
}

int tq_engine_read_output_f32(tq_engine* e, float* host_out, int first_layer, int n_layers, tq_stream_t s) {
    if (!e || !host_out || first_layer < 0 || n_layers <= 0 || first_layer + n_layers > e->shape.num_layers) return TQ_ERR_ARG;
    if (!e->out_f32) return TQ_ERR_STATE;
    const size_t per_layer = (size_t)e->G * e->shape.num_heads * HEAD_DIM;
    TQ_CUDA(cudaMemcpyAsync(host_out, e->out_f32 + per_layer * first_layer, per_layer * n_layers * sizeof(float),
                            cudaMemcpyDeviceToHost, cs(s)));
    return cuda_status(cudaStreamSynchronize(cs(s)));
}

int tq_engine_decode_layer(tq_engine* e, int layer, const void* q, const void* k, const void* v, void* out,
                           tq_stream_t s) {
    if (!e || layer < 0 || layer >= e->shape.num_layers || !q || !k || !v || !out) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || e->G == 0 || !engine_on_its_device(e)) return TQ_ERR_STATE;
    const bool chained = e->chain_ok;  // whatever happens below, the chain of fused launches starts afresh unless it continues
    e->chain_ok = false;
    const tq_engine::Layer& L = e->layers[layer];
    const int H = e->shape.num_heads, Hkv = e->shape.num_kv_heads, D = e->shape.head_dim;
    float* const f32 = e->out_f32 ? e->out_f32 + (size_t)layer * e->G * H * HEAD_DIM : nullptr;
    if (e->kv_bits == 0) {
        fp16_cache_write_kernel<<<e->G, 128, 0, cs(s)>>>((__half*)L.k, (__half*)L.v, (const __half*)k, (const __half*)v,
                                                         e->d_positions, e->rb(), e->msl, e->msl, e->G,
                                                         e->kv_dim(), (int*)e->workspace, e->caps());
        int r = cuda_status(cudaGetLastError());
        if (r != TQ_OK) return r;
        return tq_fp16_decode_attention(out, q, L.k, L.v, e->d_positions, -1, e->rb(), e->total_rows, e->msl, e->G,
                                        H, Hkv, D, e->q_dim(), e->kv_dim(), e->workspace, e->ws_bytes, s);
    }
    if (!fast_shape(H, Hkv, true)) {
        // a head layout outside the streaming kernel's: append with the chain kernel, attend with the generic one
        if (e->shared_active) return TQ_ERR_UNSUPPORTED;
        int r = append_impl((uint8_t*)L.k, L.kn, (uint8_t*)L.v, L.vn, k, v, nullptr, e->d_rotation, e->d_positions, 0, e->rb(), 0, 0,
                            e->msl, e->G, H, Hkv, D, e->q_dim(), e->kv_dim(), e->kv_bits, e->workspace, e->ws_bytes, false, cs(s),
                            false, e->d_rotation_prep, 0, e->caps());
        if (r != TQ_OK) return r;
        return generic_packed_attention(out, q, L.k, L.v, L.kn, L.vn, e->d_rotation, e->d_positions, -1, e->rb(), e->msl, e->G, H,
                                        Hkv, e->q_dim(), e->kv_bits, cs(s));
    }
    // One launch per layer when the batch fits the kernel's shared-memory tile table (tq_engine_set_fused).
    if (e->fused && e->G <= FUSED_MAX_G) {
        static const bool early_on = !(getenv("TQ_FUSED_EARLY") && atoi(getenv("TQ_FUSED_EARLY")) == 0);
        // (a launch that is being captured into a graph is replayed after whatever the caller puts in front of the
        // graph: it never reads early)
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(cs(s), &cap) != cudaSuccess) cap = cudaStreamCaptureStatusActive;
        const int early = (early_on && use_pdl() && chained && e->chain_stream == cs(s) && cap == cudaStreamCaptureStatusNone) ? 1 : 0;
        FusedInputs in{q, k, v, e->d_rotation_rep, ROT_COPIES, early, e->caps()};
        const int r = attention_impl(out, L.tmK, L.tmV, L.k, L.v, L.kn, L.vn, e->d_rotation_t, e->d_positions, -1, e->rb(),
                                     e->total_rows, e->msl, e->G, H, Hkv, e->q_dim(), e->kv_bits, e->workspace, e->ws_bytes,
                                     cs(s), use_pdl(), &in, 0, 0, f32, e->shared_active ? e->d_prefix_base : nullptr,
                                     e->shared_active ? e->d_prefix_tiles : nullptr);
        e->chain_ok = r == TQ_OK;
        e->chain_stream = cs(s);
        return r;
    }
    int r = append_impl((uint8_t*)L.k, L.kn, (uint8_t*)L.v, L.vn, k, v, q, e->d_rotation, e->d_positions, 0,
                        e->rb(), 0, 0, e->msl, e->G, H, Hkv, D, e->q_dim(), e->kv_dim(), e->kv_bits, e->workspace,
                        e->ws_bytes, true, cs(s), use_pdl(), e->d_rotation_prep, 0, e->caps());
    if (r != TQ_OK) return r;
    return attention_impl(out, L.tmK, L.tmV, L.k, L.v, L.kn, L.vn, e->d_rotation_t, e->d_positions, -1, e->rb(), e->total_rows,
                          e->msl, e->G, H, Hkv, e->q_dim(), e->kv_bits, e->workspace, e->ws_bytes, cs(s), use_pdl(), nullptr, 0, 0, f32,
                          e->shared_active ? e->d_prefix_base : nullptr, e->shared_active ? e->d_prefix_tiles : nullptr);
}

int tq_engine_attend_layer(tq_engine* e, int layer, void* out, tq_stream_t s) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e || layer < 0 || layer >= e->shape.num_layers || !out) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || e->G == 0) return TQ_ERR_STATE;
    if (e->kv_bits == 0 || !fast_shape(e->shape.num_heads, e->shape.num_kv_heads, true)) return TQ_ERR_UNSUPPORTED;
    const tq_engine::Layer& L = e->layers[layer];
    // the tile table of the current positions (a launch of the append kernel without vectors), then the attention
    int r = append_impl(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, e->d_rotation, e->d_positions, 0,
                        e->rb(), 0, 0, e->msl, e->G, e->shape.num_heads, e->shape.num_kv_heads, e->shape.head_dim,
                        e->q_dim(), e->kv_dim(), e->kv_bits, e->workspace, e->ws_bytes, true, cs(s), use_pdl());
    if (r != TQ_OK) return r;
    return attention_impl(out, L.tmK, L.tmV, L.k, L.v, L.kn, L.vn, e->d_rotation_t, e->d_positions, -1, e->rb(), e->total_rows,
                          e->msl, e->G, e->shape.num_heads, e->shape.num_kv_heads, e->q_dim(), e->kv_bits, e->workspace,
                          e->ws_bytes, cs(s), use_pdl(), nullptr, 0, 0, nullptr, e->shared_active ? e->d_prefix_base : nullptr,
                          e->shared_active ? e->d_prefix_tiles : nullptr);
}

int tq_engine_attend_step(tq_engine* e, void* out, tq_stream_t s) {
    if (!e || !out) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || e->G == 0) return TQ_ERR_STATE;
    const size_t qb = (size_t)e->G * e->q_dim() * 2;
    for (int l = 0; l < e->shape.num_layers; ++l) {
        int r = tq_engine_attend_layer(e, l, (char*)out + qb * l, s);
        if (r != TQ_OK) return r;
    }
    return TQ_OK;
}

// Whole-step form of the layers [l0, l0 + n): four launches whatever n is.
//   1. the new token of every sequence goes into every layer's cache at once (tensor-core append, decode-step form);
//   1b. all query heads of the n layers are rotated and scaled (tensor cores), stored as fp16;
//   2. ONE attention launch streams the n layers back to back and publishes its split-K partials per layer;
//   3. the merge kernel (one CTA per sequence and layer) combines them and applies the inverse rotation.
// q, k, v, out point at layer l0's [G][dim] blocks of [layers][G][dim] buffers.
static bool engine_whole_step_ok(const tq_engine* e, const void* q, const void* k, const void* v, const void* out) {
    return e->kv_bits != 0 && e->fused && e->whole_step && e->G <= FUSED_MAX_G && e->step_partials &&
           fast_shape(e->shape.num_heads, e->shape.num_kv_heads, true) &&
           ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15u) == 0);
}

static int engine_step_attend(tq_engine* e, int l0, int n, const void* q, void* out, cudaStream_t s, const tq_step_producer* prod);

// launches 1 and 1b of the whole-step form for the layers [l0, l0 + n): the append and the query rotation
static int engine_step_prepare(tq_engine* e, int l0, int n, const void* q, const void* k, const void* v, cudaStream_t s,
                               const tq_step_producer* prod) {
    e->chain_ok = false;
    const tq_engine::Layer& L = e->layers[l0];
    const int H = e->shape.num_heads, Hkv = e->shape.num_kv_heads, G = e->G;
    PrefillTcParams t{};
    t.ck = (uint8_t*)L.k; t.kn = (__half*)L.kn; t.cv = (uint8_t*)L.v; t.vn = (__half*)L.vn;
    t.k_buf = (const __half*)k; t.v_buf = (const __half*)v; t.rotation = (const __half*)e->d_rotation;
    t.positions = e->d_positions; t.status = (int*)e->workspace;
    t.token_row0 = 0; t.seq_stride_rows = e->msl; t.row_base = e->rb();
    t.capacity_rows = e->msl; t.seq_capacity = e->caps();
    t.n_seq = n * G; t.T = 1; t.Hkv = Hkv; t.kv_dim = e->kv_dim(); t.bits = e->kv_bits;
    t.step_G = G; t.code_layer_stride = (long long)e->code_layer_stride; t.norm_layer_stride = (long long)(e->norm_layer_stride / 2);
    if (prod) {  // QK-norm and rotary embedding of the raw K projection on the way into the append
        t.norm_w = (const __half*)prod->k_norm_weight + (size_t)l0 * HEAD_DIM;
        t.rope_cos = (const __half*)prod->rope_cos; t.rope_sin = (const __half*)prod->rope_sin;
        t.rope_dim = prod->rope_dim; t.eps = prod->eps; t.biased = prod->biased;
        t.k_post = (__half*)e->step_kpost + (size_t)l0 * G * e->kv_dim();
    }
    int r = launch_prefill_tc_params(t, s, prod != nullptr);
    if (r != TQ_OK) return r;
    {   // all query heads of the n layers, rotated and scaled, as fp16 (producer form: normed and rope'd first)
        QRotParams qr{};
        qr.q = (const __half*)q; qr.rotation = (const __half*)e->d_rotation;
        qr.q_rot = (__half*)e->step_qrot + (size_t)l0 * G * H * HEAD_DIM;
        qr.n_vec = (long long)n * G * H; qr.H = H; qr.q_dim = e->q_dim();
        long long blocks = (qr.n_vec + 15) / 16;
        const long long cap = 4ll * device_props().sm_count;
        if (blocks > cap) blocks = cap;
        if (prod) {
            qr.norm_w = (const __half*)prod->q_norm_weight + (size_t)l0 * HEAD_DIM;
            qr.rope_cos = (const __half*)prod->rope_cos; qr.rope_sin = (const __half*)prod->rope_sin;
            qr.positions = e->d_positions; qr.G = G; qr.rope_dim = prod->rope_dim; qr.eps = prod->eps; qr.biased = prod->biased;
            rotate_queries_kernel<true><<<(unsigned)blocks, QROT_WARPS * 32, 0, s>>>(qr);
        } else {
            rotate_queries_kernel<false><<<(unsigned)blocks, QROT_WARPS * 32, 0, s>>>(qr);
        }
        r = cuda_status(cudaGetLastError());
        if (r != TQ_OK) return r;
    }
    return TQ_OK;
}

static int engine_step_layers(tq_engine* e, int l0, int n, const void* q, const void* k, const void* v, void* out, cudaStream_t s,
                              const tq_step_producer* prod = nullptr) {
    int r = engine_step_prepare(e, l0, n, q, k, v, s, prod);
    if (r != TQ_OK) return r;
    return engine_step_attend(e, l0, n, q, out, s, prod);
}

// launches 2 and 3 for the layers [l0, l0 + n): the attention over the rotated queries engine_step_prepare left, and the merge
static int engine_step_attend(tq_engine* e, int l0, int n, const void* q, void* out, cudaStream_t s, const tq_step_producer* prod) {
    e->chain_ok = false;
    const tq_engine::Layer& L = e->layers[l0];
    const int H = e->shape.num_heads, Hkv = e->shape.num_kv_heads, G = e->G;
    int r = TQ_OK;
    FullWorkspace fw = carve_full(e->workspace, G, H);
    AttnParams p{};
    p.ck = (const uint8_t*)L.k; p.cv = (const uint8_t*)L.v; p.kn = (const __half*)L.kn; p.vn = (const __half*)L.vn;
    p.q_rot = fw.w.q_rot; p.rotation_t = (const __half*)e->d_rotation_t; p.out = (__half*)out;
    p.positions = e->d_positions; p.row_base = e->rb();
    if (e->shared_active) { p.prefix_base = e->d_prefix_base; p.prefix_tiles = e->d_prefix_tiles; }
    p.tile_start = fw.w.tile_start; p.worker_g = fw.w.worker_g; p.tickets = fw.w.tickets;
    p.partials = e->step_partials + (size_t)l0 * e->step_part_stride;
    p.status = fw.w.status;
    p.total_rows = e->total_rows; p.pos_value = -1; p.max_seq_len = e->msl;
    p.G = G; p.H = H; p.Hkv = Hkv; p.q_dim = e->q_dim();
    p.new_q = (const __half*)q; p.rotation = (const __half*)e->d_rotation_rep; p.rot_copies = ROT_COPIES;
    p.kv_dim = e->kv_dim(); p.capacity_rows = e->msl;
    static const int l2_ahead = getenv("TQ_ATTN_L2_AHEAD") ? atoi(getenv("TQ_ATTN_L2_AHEAD")) : ATTN_L2_AHEAD;
    p.l2_ahead = l2_ahead > 0 ? l2_ahead : (1 << 28);  // 0 switches the prefetch off
    p.layer0 = l0; p.n_layers = n;
    p.norm_layer_stride = (long long)(e->norm_layer_stride / 2);
    p.q_layer_stride = (long long)G * e->q_dim();
    p.part_layer_stride = (long long)e->step_part_stride;
    p.table_out = e->step_table;
    p.q_rot16 = (const __half*)e->step_qrot + (size_t)l0 * G * H * HEAD_DIM;
#ifdef TQ_TIMING_SWITCHES
    p.debug = getenv("TQ_ATTN_DEBUG") ? atoi(getenv("TQ_ATTN_DEBUG")) : 0;
    static unsigned long long* d_stamps = nullptr;
    static int stamp_calls = 0;
    if (getenv("TQ_ATTN_STAMPS")) {
        if (!d_stamps) cudaMalloc(&d_stamps, 128);
        cudaMemsetAsync(d_stamps, 0, 128, s);
        p.stamps = d_stamps;
    }
#endif
    if (e->ev_attn[0]) cudaEventRecord(e->ev_attn[0], s);
    r = launch_attention(e->kv_bits, e->tmK4, e->tmV4, p, attention_ctas(G, e->msl), s, use_pdl() && !e->ev_attn[0], 2);
    if (e->ev_attn[0]) cudaEventRecord(e->ev_attn[1], s);
    if (r != TQ_OK) return r;

    MergeParams m{};
    m.partials = p.partials; m.table = e->step_table; m.rotation_t = (const __half*)e->d_rotation_t;
    m.out = (__half*)out; m.out_f32 = e->out_f32 ? e->out_f32 + (size_t)l0 * G * H * HEAD_DIM : nullptr;
    m.part_layer_stride = p.part_layer_stride; m.q_layer_stride = p.q_layer_stride;
    m.G = G; m.H = H; m.q_dim = e->q_dim();
    m.rotated_out = (prod && prod->rotated_output) ? 1 : 0;
#ifdef TQ_TIMING_SWITCHES
    if (p.stamps && ++stamp_calls == 30) {
        unsigned long long h[16];
        cudaStreamSynchronize(s);
        cudaMemcpy(h, p.stamps, 128, cudaMemcpyDeviceToHost);
        const double w = (double)h[15];
        fprintf(stderr, "stamps per warp (cycles, %d layers): loop-head %.0f | K wait %.0f | K phase %.0f | softmax %.0f | V wait %.0f | V phase %.0f | exit %.0f | "
                        "seg: tail+publish+reads %.0f | q wait %.0f | fragments %.0f | barrier %.0f | after-loop %.0f | warps %.0f\n",
                n, h[0] / w, h[1] / w, h[2] / w, h[3] / w, h[4] / w, h[5] / w, h[6] / w, h[8] / w, h[9] / w, h[10] / w, h[11] / w, h[12] / w, w);
    }
#endif
    return launch_kernel(merge_partials_kernel, dim3(G, n), dim3(MERGE_WARPS * 32), 0, s, use_pdl(), m);
}

int tq_engine_time_attention(tq_engine* e, int enable) {
    if (!e) return TQ_ERR_ARG;
    if (!engine_on_its_device(e)) return TQ_ERR_STATE;
    if (enable && !e->ev_attn[0]) {
        TQ_CUDA(cudaEventCreate(&e->ev_attn[0]));
        TQ_CUDA(cudaEventCreate(&e->ev_attn[1]));
    } else if (!enable && e->ev_attn[0]) {
        cudaEventDestroy(e->ev_attn[0]);
        cudaEventDestroy(e->ev_attn[1]);
        e->ev_attn[0] = e->ev_attn[1] = nullptr;
    }
    return TQ_OK;
}

int tq_engine_last_attention_ms(tq_engine* e, float* ms) {
    if (!e || !ms) return TQ_ERR_ARG;
    if (!e->ev_attn[0]) return TQ_ERR_STATE;
    TQ_CUDA(cudaEventSynchronize(e->ev_attn[1]));
    TQ_CUDA(cudaEventElapsedTime(ms, e->ev_attn[0], e->ev_attn[1]));
    return TQ_OK;
}

int tq_engine_step_prepare(tq_engine* e, const void* q, const void* k, const void* v, tq_stream_t s) {
    if (!e || !q || !k || !v) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || e->G == 0 || !engine_on_its_device(e)) return TQ_ERR_STATE;
    if (!engine_whole_step_ok(e, q, k, v, q)) return TQ_ERR_UNSUPPORTED;
    return engine_step_prepare(e, 0, e->shape.num_layers, q, k, v, cs(s), nullptr);
}

int tq_engine_step_attend_layers(tq_engine* e, int first_layer, int n_layers, void* out_first, tq_stream_t s) {
    if (!e || !out_first || first_layer < 0 || n_layers <= 0 || first_layer + n_layers > e->shape.num_layers) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || e->G == 0 || !engine_on_its_device(e)) return TQ_ERR_STATE;
    if (!engine_whole_step_ok(e, out_first, out_first, out_first, out_first)) return TQ_ERR_UNSUPPORTED;
    return engine_step_attend(e, first_layer, n_layers, nullptr, out_first, cs(s), nullptr);
}

int tq_engine_decode_layers(tq_engine* e, int first_layer, int n_layers, const void* q, const void* k, const void* v, void* out,
                            tq_stream_t s) {
    if (!e || !q || !k || !v || !out || first_layer < 0 || n_layers <= 0 || first_layer + n_layers > e->shape.num_layers)
        return TQ_ERR_ARG;
    if (e->asleep || !e->arena || e->G == 0 || !engine_on_its_device(e)) return TQ_ERR_STATE;
    if (engine_whole_step_ok(e, q, k, v, out)) return engine_step_layers(e, first_layer, n_layers, q, k, v, out, cs(s));
    const size_t qb = (size_t)e->G * e->q_dim() * 2, kb = (size_t)e->G * e->kv_dim() * 2;
    for (int i = 0; i < n_layers; ++i) {
        int r = tq_engine_decode_layer(e, first_layer + i, (const char*)q + qb * i, (const char*)k + kb * i, (const char*)v + kb * i,
                                       (char*)out + qb * i, s);
        if (r != TQ_OK) return r;
    }
    return TQ_OK;
}

int tq_engine_decode_step(tq_engine* e, const void* q, const void* k, const void* v, void* out, tq_stream_t s) {
    if (!e) return TQ_ERR_ARG;
    return tq_engine_decode_layers(e, 0, e->shape.num_layers, q, k, v, out, s);
}

// The decode step with its producer and consumer folded in: q_raw / k_raw are the projections' raw outputs; per-head RMS
// norm and rotary embedding (the reference's launch_qk_norm_batch + launch_rope_batch, engine/engine.cpp:1972-1977) are
// applied inside the query rotation and inside the append; with rotated_output the inverse rotation is left to the
// consumer's weights (tq_fold_rotation_into_projection).
int tq_engine_decode_step_produce(tq_engine* e, const void* q_raw, const void* k_raw, const void* v, void* out,
                                  const tq_step_producer* prod, tq_stream_t s) {
    if (!e || !q_raw || !k_raw || !v || !out || !prod) return TQ_ERR_ARG;
    if (!prod->q_norm_weight || !prod->k_norm_weight || !prod->rope_cos || !prod->rope_sin) return TQ_ERR_ARG;
    if (prod->rope_dim != 64 && prod->rope_dim != 128) return TQ_ERR_UNSUPPORTED;
    if (e->asleep || !e->arena || e->G == 0 || !engine_on_its_device(e)) return TQ_ERR_STATE;
    if (!engine_whole_step_ok(e, q_raw, k_raw, v, out)) return TQ_ERR_UNSUPPORTED;  // packed modes, streaming head layouts
    if ((((uintptr_t)prod->q_norm_weight | (uintptr_t)prod->k_norm_weight | (uintptr_t)prod->rope_cos | (uintptr_t)prod->rope_sin) & 15u) != 0)
        return TQ_ERR_ARG;
    return engine_step_layers(e, 0, e->shape.num_layers, q_raw, k_raw, v, out, cs(s), prod);
}

__global__ void fold_rotation_kernel(__half* w_out, const __half* w_in, const __half* rotation, long long rows, int num_heads) {
    // w_out[r][h*128 + k] = sum_d w_in[r][h*128 + d] * R[k][d]   (W' = W * blockdiag(R^T): then W' * acc = W * (R^T acc))
    __shared__ float row_s[HEAD_DIM];
    const long long r = blockIdx.x;
    const int h = blockIdx.y, k = threadIdx.x;
    const size_t base = ((size_t)r * num_heads + h) * HEAD_DIM;
    row_s[k] = __half2float(w_in[base + k]);
    __syncthreads();
    float acc = 0.0f;
    const __half* rr = rotation + (size_t)k * HEAD_DIM;
    for (int d = 0; d < HEAD_DIM; ++d) acc = fmaf(row_s[d], __half2float(rr[d]), acc);
    w_out[base + k] = __float2half_rn(acc);
}

int tq_fold_rotation_into_projection(void* w_out, const void* w_in, const void* rotation, long long rows, int num_heads,
                                     tq_stream_t s) {
    if (!w_out || !w_in || !rotation || rows <= 0 || num_heads <= 0 || rows > 2147483647ll || num_heads > 65535) return TQ_ERR_ARG;
    fold_rotation_kernel<<<dim3((unsigned)rows, (unsigned)num_heads), HEAD_DIM, 0, cs(s)>>>((__half*)w_out, (const __half*)w_in,
                                                                                         (const __half*)rotation, rows, num_heads);
    return cuda_status(cudaGetLastError());
}

// Prompts of n_seq consecutive sequences (first_seq ..), all T tokens long and all at positions first_pos ..; inputs
// [n_seq][T][kv_dim].  One launch.
static int engine_prefill_impl(tq_engine* e, int layer, int first_seq, int n_seq, const void* k, const void* v, int first_pos,
                               int T, tq_stream_t s) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e || layer < 0 || layer >= e->shape.num_layers || !k || !v || T <= 0 || first_pos < 0 || n_seq <= 0) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || e->G == 0 || !engine_on_its_device(e)) return TQ_ERR_STATE;
    if (first_seq < 0 || first_seq + n_seq > e->G) return TQ_ERR_ARG;
    int cap = e->cap_eff(first_seq);
    for (int i = 0; i < n_seq; ++i) {
        cap = std::min(cap, e->cap_eff(first_seq + i));
        // rows below a shared prefix belong to another sequence's slot: they are written through that sequence only
        if (first_pos < e->prefix_tokens[first_seq + i]) return TQ_ERR_STATE;
    }
    if (first_pos + T > cap) return TQ_ERR_CAPACITY;
    const tq_engine::Layer& L = e->layers[layer];
    if (e->kv_bits == 0) {
        const size_t row_bytes = (size_t)e->kv_dim() * 2;
        for (int i = 0; i < n_seq; ++i) {
            const long long row0 = e->row0_eff(first_seq + i);
            TQ_CUDA(cudaMemcpyAsync((char*)L.k + (size_t)(row0 + first_pos) * row_bytes, (const char*)k + (size_t)i * T * row_bytes,
                                    (size_t)T * row_bytes, cudaMemcpyDeviceToDevice, cs(s)));
            TQ_CUDA(cudaMemcpyAsync((char*)L.v + (size_t)(row0 + first_pos) * row_bytes, (const char*)v + (size_t)i * T * row_bytes,
                                    (size_t)T * row_bytes, cudaMemcpyDeviceToDevice, cs(s)));
        }
        return TQ_OK;
    }
    // token form: token t goes to position first_pos + t (by value: no position array)
    const long long row0 = e->row0_eff(first_seq);
    // the append kernel only needs the header of the workspace here (status word)
    AppendParams p{};
    p.ck = (uint8_t*)L.k; p.kn = (__half*)L.kn; p.cv = (uint8_t*)L.v; p.vn = (__half*)L.vn;
    p.k_buf = (const __half*)k; p.v_buf = (const __half*)v; p.q = nullptr;
    p.rotation = (const __half*)e->d_rotation;
    p.rot_prep = e->d_rotation_prep;
    p.positions = nullptr; p.row_base = nullptr; p.q_rot = nullptr;
    p.tile_start = nullptr; p.tickets = nullptr; p.total_tiles = nullptr;
    p.status = (int*)e->workspace;
    p.token_row0 = row0; p.token_mode = 1;
    p.max_seq_len = e->msl; p.capacity_rows = cap;
    p.n_src = T; p.H = e->shape.num_heads; p.Hkv = e->shape.num_kv_heads; p.q_dim = e->q_dim(); p.kv_dim = e->kv_dim();
    p.bits = e->kv_bits; p.pos_value = first_pos;
    if (n_seq == 1) return launch_append(p, cs(s));
    if ((long long)n_seq * T * p.Hkv >= (1ll << 31)) return TQ_ERR_CAPACITY;
    // several sequences: the tensor-core kernel takes them in one launch (whatever their number of head vectors)
    return launch_prefill_tc(p, cs(s), n_seq, e->msl, e->rb() ? e->rb() + first_seq : nullptr);
}

// A prompt of T tokens shared by the sequences first_seq .. first_seq + n_seq - 1 (rollouts of one prompt: the
// reference prefills sequence 0 and copies its cache to the others, engine/engine.cpp:2173-2214).  Here the first
// P = 32 * floor(T / 32) tokens are quantised and stored ONCE, in the slot of first_seq; the other sequences read those
// tiles from there (AttnParams::prefix_base) and their own slots start at token P.  The remaining T - P tokens (less
// than a tile) go into every sequence's own rows.  Call it once per layer, with the same T, before anything else is
// appended to these sequences.
int tq_engine_prefill_shared(tq_engine* e, int layer, int first_seq, int n_seq, const void* k, const void* v, int T,
                             tq_stream_t s) {
    if (e) e->chain_ok = false;  // not a fused decode launch: the next one reads nothing early
    if (!e || layer < 0 || layer >= e->shape.num_layers || !k || !v || T <= 0 || n_seq <= 0) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || e->G == 0 || !engine_on_its_device(e)) return TQ_ERR_STATE;
    if (first_seq < 0 || first_seq + n_seq > e->G) return TQ_ERR_ARG;
    if (e->kv_bits == 0) return TQ_ERR_UNSUPPORTED;  // the fp16 twin's kernel reads every sequence from its own slot
    if (!fast_shape(e->shape.num_heads, e->shape.num_kv_heads, true)) return TQ_ERR_UNSUPPORTED;
    const int P = T / TILE_TOKENS * TILE_TOKENS;
    if (e->prefix_tokens[first_seq] != 0 || T > e->capacities[first_seq]) return e->prefix_tokens[first_seq] ? TQ_ERR_STATE : TQ_ERR_CAPACITY;
    bool changed = false;
    for (int i = 1; i < n_seq; ++i) {
        const int g = first_seq + i;
        if (e->prefix_tokens[g] == P && (P == 0 || e->prefix_owner[g] == first_seq)) continue;  // set by an earlier layer's call
        if (e->prefix_tokens[g] != 0) return TQ_ERR_STATE;
        if (T - P > e->capacities[g]) return TQ_ERR_CAPACITY;
        if (P > 0) {
            e->prefix_tokens[g] = P;
            e->prefix_owner[g] = first_seq;
            changed = true;
        }
    }
    if (changed) {
        e->shared_active = true;
        std::vector<long long> rb(e->G), pb(e->G);
        std::vector<int> cp(e->G), pt(e->G);
        for (int g = 0; g < e->G; ++g) {
            rb[g] = e->row0_eff(g);
            cp[g] = e->cap_eff(g);
            pb[g] = e->prefix_tokens[g] ? e->h_row_base[e->prefix_owner[g]] : 0;
            pt[g] = e->prefix_tokens[g] / TILE_TOKENS;
        }
        TQ_CUDA(cudaMemcpyAsync(e->d_row_base, rb.data(), rb.size() * sizeof(long long), cudaMemcpyHostToDevice, cs(s)));
        TQ_CUDA(cudaMemcpyAsync(e->d_capacities, cp.data(), cp.size() * sizeof(int), cudaMemcpyHostToDevice, cs(s)));
        TQ_CUDA(cudaMemcpyAsync(e->d_prefix_base, pb.data(), pb.size() * sizeof(long long), cudaMemcpyHostToDevice, cs(s)));
        TQ_CUDA(cudaMemcpyAsync(e->d_prefix_tiles, pt.data(), pt.size() * sizeof(int), cudaMemcpyHostToDevice, cs(s)));
        TQ_CUDA(cudaStreamSynchronize(cs(s)));  // the sources are locals of this frame
    }
    // the whole prompt into the owner's slot (its rows P .. T-1 are its own remainder), the remainder into the others'
    int r = engine_prefill_impl(e, layer, first_seq, 1, k, v, 0, T, s);
    const size_t row_bytes = (size_t)e->kv_dim() * 2;
    for (int i = 1; i < n_seq && r == TQ_OK && T > P; ++i)
        r = engine_prefill_impl(e, layer, first_seq + i, 1, (const char*)k + (size_t)P * row_bytes, (const char*)v + (size_t)P * row_bytes,
                                P, T - P, s);
    return r;
}

int tq_engine_prefill_append(tq_engine* e, int layer, int seq, const void* k, const void* v, int first_pos, int T,
                             tq_stream_t s) {
    return engine_prefill_impl(e, layer, seq, 1, k, v, first_pos, T, s);
}

int tq_engine_prefill_append_batch(tq_engine* e, int layer, int first_seq, int n_seq, const void* k, const void* v,
                                   int first_pos, int T, tq_stream_t s) {
    return engine_prefill_impl(e, layer, first_seq, n_seq, k, v, first_pos, T, s);
}

// One layer of the prefill of n_seq prompts of T tokens each (reference engine/engine.cpp:2110-2146 for one prompt: cache
// write of all T tokens, then causal self-attention): the tokens of sequence first_seq + i go to positions 0 .. T-1 of its
// slot and its query token t attends to rows 0 .. t.  q [n_seq][T][q_stride] and out [n_seq][T][q_stride] share the stride
// (the reference passes Q_PROJ_DIM for both).  All prompts' blocks are one launch, the longest causal prefixes first.
int tq_engine_prefill_layer_batch(tq_engine* e, int layer, int first_seq, int n_seq, const void* q, const void* k, const void* v,
                                  void* out, int T, int q_stride, tq_stream_t s) {
    if (!e || !q || !out) return TQ_ERR_ARG;
    int r = engine_prefill_impl(e, layer, first_seq, n_seq, k, v, 0, T, s);
    if (r != TQ_OK) return r;
    const int H = e->shape.num_heads, Hkv = e->shape.num_kv_heads;
    if (q_stride < H * HEAD_DIM || (q_stride & 7) != 0) return TQ_ERR_ARG;
    int cap = e->cap_eff(first_seq);
    for (int i = 0; i < n_seq; ++i) {
        // a slot that begins behind a shared prefix holds no rows 0 .. P-1
        if (e->prefix_tokens[first_seq + i] > 0) return TQ_ERR_STATE;
        cap = std::min(cap, e->cap_eff(first_seq + i));
    }
    const tq_engine::Layer& L = e->layers[layer];
    const size_t row_bytes = e->code_row_bytes();
    if (!prefill_attn_shape(H, Hkv)) {   // layouts outside the tiled kernel: the compat launchers' generic path, prompt by prompt
        std::lock_guard<std::recursive_mutex> compat_lock(compat_mutex());
        for (int i = 0; i < n_seq && r == TQ_OK; ++i) {
            const long long row0 = e->row0_eff(first_seq + i);
            const char* qi = (const char*)q + (size_t)i * T * q_stride * 2;
            char* oi = (char*)out + (size_t)i * T * q_stride * 2;
            if (e->kv_bits == 0)
                launch_gqa_prefill_attention(oi, qi, (const char*)L.k + (size_t)row0 * row_bytes, (const char*)L.v + (size_t)row0 * row_bytes,
                                             nullptr, T, cap, H, Hkv, HEAD_DIM, q_stride, e->kv_dim(), s);
            else
                launch_turbo_gqa_prefill_attention(oi, qi, (const uint8_t*)L.k + (size_t)row0 * row_bytes, (const uint8_t*)L.v + (size_t)row0 * row_bytes,
                                                   (const __half*)L.kn + (size_t)row0 * Hkv, (const __half*)L.vn + (size_t)row0 * Hkv,
                                                   e->d_rotation, nullptr, T, cap, H, Hkv, HEAD_DIM, q_stride, e->kv_dim(), e->kv_bits, s);
            r = tq_last_compat_status();
        }
        return r;
    }
    PrefillAttnParams ap{};
    ap.q = (const __half*)q;
    ap.q_tok_stride = q_stride;
    ap.out = (__half*)out;
    ap.q_dim = q_stride;
    ap.T = T;
    ap.rows = cap;
    ap.H = H;
    ap.Hkv = Hkv;
    ap.n_seq = n_seq;
    ap.seq_rows = e->msl;
    ap.row_base = e->rb() ? e->rb() + first_seq : nullptr;
    const long long row0 = ap.row_base ? 0 : e->row0_eff(first_seq);   // dense slots: first_seq * max_seq_len
    ap.ck = (const uint8_t*)L.k + (size_t)row0 * row_bytes;
    ap.cv = (const uint8_t*)L.v + (size_t)row0 * row_bytes;
    if (e->kv_bits == 0) {
        ap.score_scale = 0.12751743074602467f;
    } else {
        ap.kn = (const __half*)L.kn + (size_t)row0 * Hkv;
        ap.vn = (const __half*)L.vn + (size_t)row0 * Hkv;
        ap.rotation = (const __half*)e->d_rotation;
        ap.rotation_t = (const __half*)e->d_rotation_t;
        ap.score_scale = 1.0f;
    }
    ap.status = (int*)e->workspace;
    return launch_prefill_attention(e->kv_bits, ap, cs(s));
}

int tq_engine_prefill_layer(tq_engine* e, int layer, int seq, const void* q, const void* k, const void* v, void* out, int T,
                            int q_stride, tq_stream_t s) {
    return tq_engine_prefill_layer_batch(e, layer, seq, 1, q, k, v, out, T, q_stride, s);
}

int tq_engine_decode_step_host(tq_engine* e, const void* q_host, const void* k_host, const void* v_host, void* out_host,
                               tq_stream_t s) {
    if (!e || !q_host || !k_host || !v_host || !out_host) return TQ_ERR_ARG;
    if (e->asleep || !e->arena || e->G == 0) return TQ_ERR_STATE;
    const int NL = e->shape.num_layers;
    const size_t qb = (size_t)e->G * e->q_dim() * 2, kb = (size_t)e->G * e->kv_dim() * 2;
    // The layers go in a few groups: the inputs of group c+1 are copied in (and the outputs of group c-1 copied out)
    // on two copy streams while the kernels of group c run on the caller's stream.
    constexpr int NC = tq_engine::HOST_STEP_CHUNKS;
    if (!e->st_in) {
        TQ_CUDA(cudaStreamCreateWithFlags(&e->st_in, cudaStreamNonBlocking));
        TQ_CUDA(cudaStreamCreateWithFlags(&e->st_out, cudaStreamNonBlocking));
        TQ_CUDA(cudaEventCreateWithFlags(&e->ev_begin, cudaEventDisableTiming));
        TQ_CUDA(cudaEventCreateWithFlags(&e->ev_done, cudaEventDisableTiming));
        for (int c = 0; c < NC; ++c) {
            TQ_CUDA(cudaEventCreateWithFlags(&e->ev_in[c], cudaEventDisableTiming));
            TQ_CUDA(cudaEventCreateWithFlags(&e->ev_out[c], cudaEventDisableTiming));
        }
    }
    // The first and the last group are single layers: the first copy-in and the last copy-out are the only ones
    // nothing can hide.
    // (in the whole-step form every group costs four launches and a pipeline fill, so few groups: TQ_HOST_STEP_GROUPS)
    static const int want = getenv("TQ_HOST_STEP_GROUPS") ? atoi(getenv("TQ_HOST_STEP_GROUPS")) : 0;
    const bool whole_form = engine_whole_step_ok(e, e->stage_q, e->stage_k, e->stage_v, e->stage_out);
    int nc = want > 0 ? want : (whole_form ? 4 : NC);
    if (nc > NC) nc = NC;
    const int chunks = NL < nc ? NL : nc;
    auto first_layer = [&](int c) {
        if (chunks < 4) return (int)((long long)c * NL / chunks);
        if (c <= 0) return 0;
        if (c >= chunks) return NL;
        return 1 + (int)((long long)(c - 1) * (NL - 2) / (chunks - 2));
    };
    TQ_CUDA(cudaEventRecord(e->ev_begin, cs(s)));  // the staging buffers are free once earlier work on s is done
    TQ_CUDA(cudaStreamWaitEvent(e->st_in, e->ev_begin, 0));
    for (int c = 0; c < chunks; ++c) {
        const int l0 = first_layer(c), n = first_layer(c + 1) - l0;
        TQ_CUDA(cudaMemcpyAsync((char*)e->stage_q + qb * l0, (const char*)q_host + qb * l0, qb * n, cudaMemcpyHostToDevice, e->st_in));
        TQ_CUDA(cudaMemcpyAsync((char*)e->stage_k + kb * l0, (const char*)k_host + kb * l0, kb * n, cudaMemcpyHostToDevice, e->st_in));
        TQ_CUDA(cudaMemcpyAsync((char*)e->stage_v + kb * l0, (const char*)v_host + kb * l0, kb * n, cudaMemcpyHostToDevice, e->st_in));
        TQ_CUDA(cudaEventRecord(e->ev_in[c], e->st_in));
    }
    for (int c = 0; c < chunks; ++c) {
        const int l0 = first_layer(c), l1 = first_layer(c + 1);
        TQ_CUDA(cudaStreamWaitEvent(cs(s), e->ev_in[c], 0));
        const bool whole = engine_whole_step_ok(e, e->stage_q, e->stage_k, e->stage_v, e->stage_out) && ((qb | kb) & 15u) == 0;
        for (int l = l0; l < l1; ++l) {
            int r;
            if (whole) {  // the chunk's layers in one whole-step pass
                r = engine_step_layers(e, l0, l1 - l0, (char*)e->stage_q + qb * l0, (char*)e->stage_k + kb * l0,
                                       (char*)e->stage_v + kb * l0, (char*)e->stage_out + qb * l0, cs(s));
                l = l1;
            } else {
                r = tq_engine_decode_layer(e, l, (char*)e->stage_q + qb * l, (char*)e->stage_k + kb * l,
                                           (char*)e->stage_v + kb * l, (char*)e->stage_out + qb * l, s);
            }
            if (r != TQ_OK) {
                cudaStreamSynchronize(e->st_in);
                cudaStreamSynchronize(cs(s));
                return r;
            }
        }
        TQ_CUDA(cudaEventRecord(e->ev_out[c], cs(s)));
        TQ_CUDA(cudaStreamWaitEvent(e->st_out, e->ev_out[c], 0));
        TQ_CUDA(cudaMemcpyAsync((char*)out_host + qb * l0, (char*)e->stage_out + qb * l0, qb * (l1 - l0), cudaMemcpyDeviceToHost,
                                e->st_out));
    }
    TQ_CUDA(cudaEventRecord(e->ev_done, e->st_out));
    TQ_CUDA(cudaStreamWaitEvent(cs(s), e->ev_done, 0));
    TQ_CUDA(cudaStreamSynchronize(cs(s)));
    return TQ_OK;
}

}  // extern "C"
