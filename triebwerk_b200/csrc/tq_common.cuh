// Shared device helpers for the sm_100a TurboQuant kernels: code books, PTX wrappers (mbarrier, TMA,
// mma.sync, prmt), the workspace layout and the status word.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tq {

constexpr int HEAD_DIM = 128;
constexpr int TILE_TOKENS = 32;  // tokens per attention tile (one lane per token when norms are loaded)

// Lloyd-Max code books for N(0, 1/128): the reference's literals (engine/kernels.cu:1426-1445).
__device__ __constant__ float kCent4[16] = {-0.24155f, -0.18293f, -0.14304f, -0.11099f, -0.08330f, -0.05806f,
                                            -0.03432f, -0.01135f, 0.01135f,  0.03432f,  0.05806f,  0.08330f,
                                            0.11099f,  0.14304f,  0.18293f,  0.24155f};
__device__ __constant__ float kBnd4[15] = {-0.21224f, -0.16299f, -0.12701f, -0.09715f, -0.07068f,
                                           -0.04619f, -0.02284f, 0.00000f,  0.02284f,  0.04619f,
                                           0.07068f,  0.09715f,  0.12701f,  0.16299f,  0.21224f};
__device__ __constant__ float kCent2[4] = {-0.13351f, -0.04003f, 0.04003f, 0.13351f};
__device__ __constant__ float kBnd2[3] = {-0.08677f, 0.0f, 0.08677f};

// Device status word values (written with atomicMax; 0 = fine).
enum : int {
    ST_OK = 0,
    ST_TMA_WAIT_TIMEOUT = 1,   // a bounded wait on a TMA mbarrier ran out
    ST_SMEM_LAYOUT = 2,        // dynamic shared memory does not start where the kernel needs it
    ST_BAD_POSITION = 3,       // a position outside [0, capacity)
    ST_PEER_WAIT_TIMEOUT = 4   // a peer's completion flag did not arrive within the time limit
};

// ---- workspace layout ---------------------------------------------------------------------------------------
// [0,256)                       header: int status; int total_tiles; ...
// q_rot      float [G][H][128]  pre-rotated queries, already multiplied by log2(e)/sqrt(128)
// tile_start int   [G+1]        exclusive prefix of ceil(L_g / TILE_TOKENS)
// tickets    int   [G]          arrivals per sequence (zeroed by the append/rotate kernel)
// worker_g   int   [MAX_WORKERS] first sequence of each attention worker's slice
// partials   float [W+G][H][PART_STRIDE]  acc[128], m, l, pad
constexpr int PART_STRIDE = 132;
constexpr int MAX_WORKERS = 1024;  // upper bound on attention CTAs assumed by the workspace size

struct Workspace {
    int* status;
    int* total_tiles;
    float* q_rot;
    int* tile_start;
    int* tickets;
    int* worker_g;     // [MAX_WORKERS] first sequence of every attention worker (written with tile_start)
    float* partials;
    size_t bytes;
};

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__host__ inline Workspace carve_workspace(void* base, int G, int H) {
    Workspace w;
    char* p = (char*)base;
    size_t off = 0;
    w.status = (int*)(p + off);
    w.total_tiles = (int*)(p + off + 4);
    off += 256;
    w.q_rot = (float*)(p + off);
    off += align_up((size_t)G * H * HEAD_DIM * sizeof(float), 256);
    w.tile_start = (int*)(p + off);
    off += align_up((size_t)(G + 1) * sizeof(int), 256);
    w.tickets = (int*)(p + off);
    off += align_up((size_t)G * sizeof(int), 256);
    w.worker_g = (int*)(p + off);
    off += align_up((size_t)MAX_WORKERS * sizeof(int), 256);
    w.partials = (float*)(p + off);
    off += align_up((size_t)(MAX_WORKERS + G) * H * PART_STRIDE * sizeof(float), 256);
    w.bytes = off;
    return w;
}

// ---- small PTX wrappers ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Number of attention workers that take part when the flat list holds N tiles of G sequences and `w_all` workers were
// launched.  Every participant owns at least one tile; and with few tiles more workers per sequence only lengthen the
// split-K merge, whose cost grows with the parts of a sequence (about 0.17 us each, against about 2 us for a tile):
// the sum is smallest near sqrt(12 * N * G) workers; measured on one to four sequences of 1k to 16k tokens, factors
// 12 to 24 are equally good (one sequence of 4096 tokens: 38.6 -> 25 us per layer-step, of 16384: 69 -> 39 us).  The append kernel's table block and the attention kernel call
// this with the same arguments.
__device__ __forceinline__ int attention_workers(long long w_all, long long N, int G, int factor = 16) {
    long long W = w_all < N ? w_all : N;
    const float cap = sqrtf((float)factor * (float)N * (float)(G > 0 ? G : 1));
    if (cap < (float)W) W = (long long)cap;
    return W < 1 ? 1 : (int)W;
}

__device__ __forceinline__ float rsqrt_approx_ftz(float x) {
    float r;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float sqrt_approx_ftz(float x) {
    float r;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float fma_ftz(float a, float b, float c) {
    float r;
    asm("fma.rn.ftz.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float mul_ftz(float a, float b) {
    float r;
    asm("mul.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float add_ftz(float a, float b) {
    float r;
    asm("add.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t r;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(addr));
    return r;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 r;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(addr));
    return r;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// D += A(16x16, row) * B(16x8, col), fp16 inputs, fp32 accumulate.
// Four 8x8 fp16 matrices from shared memory as mma fragments: lane l supplies the address of row l % 8 of matrix l / 8;
// the plain form hands lane l the elements (row l / 4, columns 2 (l % 4), + 1) of each matrix, the transposed form the
// elements (rows 2 (l % 4), + 1, column l / 4).
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- programmatic dependent launch: a kernel launched with the programmatic-serialisation attribute may start
// while its predecessor in the stream is still running; everything that depends on the predecessor's writes (or
// that overwrites something the predecessor still reads) comes after pdl_wait().  No-ops otherwise.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- mbarrier / TMA ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// generic-proxy writes (any state space) before, async-proxy (bulk / tensor copy) reads after
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// The same with a suspend-time hint (nanoseconds): the thread may sleep inside the instruction until the phase
// completes or the time is up, instead of burning issue slots on polls.
__device__ __forceinline__ uint32_t mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok;
}
// Bounded wait: gives up after `limit` polls (each poll may itself block for a hardware-defined short
// time).  Returns false on give-up; the caller records ST_TMA_WAIT_TIMEOUT and stops using the pipeline.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 20)) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// The same with a suspend-time hint per poll (nanoseconds): for waits that are expected to last, fewer polls.
__device__ __forceinline__ bool mbar_wait_bounded_hint(uint32_t bar, uint32_t parity, uint32_t limit, uint32_t hint_ns) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait_hint(bar, parity, hint_ns)) return true;
    }
    return false;
}

// 2-D tiled TMA load global -> shared of this CTA (no multicast), completion on an mbarrier.
// x = innermost coordinate in elements (bytes here; must be a multiple of 16), y = row.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"((unsigned long long)map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Code of a rotated coordinate: the number of decision bounds it has reached (reference engine/kernels.cu:1540-1560).
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

// Contiguous bulk copy global -> shared of this CTA, completion on an mbarrier.  Addresses 16-byte aligned,
// size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// 3-D form of the same load; the coordinates are (x, y, z) from the innermost dimension outwards.
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"((unsigned long long)map), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// 4-D form: (x, y, z, w) from the innermost dimension outwards.
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst_smem), "l"((unsigned long long)map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

}  // namespace tq
