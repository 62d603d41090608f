// Prefill append on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// Replaces turbo_kv_quantize_kernel (reference engine/kernels.cu:1482-1560) for whole prompts: T tokens x Hkv heads x
// {K, V} head vectors are normalised, rotated by R, quantised and packed.  The rotation of many vectors is a GEMM
// (vectors x 128) . R^T, so it runs as tcgen05.mma (M = 128 vectors, N = 128 coordinates, K = 128) with the
// accumulators in tensor memory.  Stored bytes must still equal the reference's, whose rotation is a k-ascending fp32
// FMA chain; the tensor-core sum has another order.  Therefore:
//   * the tensor cores rotate the vector AS IT ARRIVES: inputs and R are fp16, so every product r_k * v_k is exact in
//     fp32 and the accumulator holds sum r_k v_k to fp32 summation error; the epilogue multiplies by 1/norm.  The
//     reference scales first (x_k = v_k / norm, one fp32 rounding each) and sums then; the two differ by the two
//     summation errors plus 2^-24 relative for the scaling -- no split of x into a high and a low operand is needed,
//     and the operand tile is a plain copy of the input;
//   * a coordinate whose value lies within TC_MARGIN of a decision bound is recomputed with the reference's exact
//     chain (R read back from the shared-memory operand tile, x re-read from the input); everywhere else the
//     two sums cannot fall on different sides of a bound.  TC_MARGIN (1.6e-5) is twice the textbook bound on the
//     distance of a 128-term fp32 sum from the exact value when sum|r_k x_k| <= 1 (128 * 2^-24 = 7.6e-6; |x| = 1 and
//     |R row| = 1): once for the chain, once for the tensor-core sum, with 8e-7 left for the scaling roundings
//     (1.2e-7 for |x.R| < 2 and 6e-8 for the x_k).  About 1 coordinate in 700 takes the exact path.
// Sums of squares, rsqrt/sqrt and the norm use the reference's own order and instructions (see tq_append.cuh).
//
// One CTA = eight worker warps + one chain warp (288 threads), one tile of 128 head vectors at a time (16 tokens x 8 heads
// of K or of V), three CTAs per SM (74 KB of shared memory, 128 columns of tensor memory, 72 registers per thread each):
//   1. the tile's 128 vectors reach the operand tile -- the canonical K-major 128-byte-swizzled layout: rows of 128
//      bytes, 16-byte chunk c of row r at chunk c ^ (r & 7) -- by ONE 4-D tensor-map copy [half][token][head][128 B],
//      issued as soon as the previous tile's MMAs have been waited for, so it lands while that tile is quantised
//      (TMA form); where the layout does not allow a tensor map, and in the producer form, thread (vector, 32-coordinate
//      chunk) loads 64 bytes and stores them there;
//   2. one thread issues 8 tcgen05.mma (K-steps of 16) against the resident R tile and commits to an mbarrier (every
//      wait is bounded); meanwhile the workers build the reference's shuffle-tree sums of squares (packed fp32
//      instructions, from shared memory in the TMA form), and one thread per vector settles it: norm out, 1/norm, where
//      its codes go;
//   3. each thread reads 64 of ITS vector's 128 accumulators from tensor memory (tcgen05.ld, 32 lanes x 32 columns per
//      warp and instruction; warps w and w + 4 share a lane quarter), scales by 1/norm, quantises through a 256-bucket
//      uniform grid (bucket -> code, or -> the one bound inside it; 13 instructions per two coordinates), stores the
//      packed codes straight to the cache and queues near-bound coordinates;
//   4. the chain warp, one tile behind (per-tile arrays exist twice; two mbarrier pairs hand them back and forth),
//      runs the exact chain of the queued coordinates, one lane per coordinate, and patches the stored codes with
//      atomics.  None of the workers' barriers waits for it.
#pragma once

#include "tq_common.cuh"

namespace tq {

constexpr int TC_TILE = 128;       // head vectors per tile = MMA M
constexpr int TC_WORKERS = 256;     // eight warps that load, rotate and quantise
constexpr int TC_THREADS = TC_WORKERS + 32;  // ... and one warp for the exact chains of near-bound coordinates
constexpr float TC_MARGIN = 1.6e-5f;
constexpr int TC_BUCKETS = 256;    // entries of the bucket table
constexpr float TC_BUCKETS_PER_UNIT = 46.0f;  // 1 / bucket width
constexpr int TC_LIST_CAP = 96;    // queued near-bound coordinates per tile; the rest is handled by their owners

// Shared memory by ABSOLUTE shared address (the kernel checks that its dynamic shared memory covers the range): the
// bucket table sits on a 4096-byte boundary so that its look-up address is (bits & 0x3fc) plus a constant.
struct TcSmem {
    // Per-tile arrays exist twice (tile parity): the chain warp works on a tile's queue while the workers are already
    // two phases further.
    static constexpr uint32_t DST0 = 0x0800;             // long long[128] byte offset of each vector's codes in the cache (-1: none)
    static constexpr uint32_t INV0 = DST0 + 1024;        // float[128]: sum of squares, then 1/norm per vector; -1: the vector
                                                         // holds an infinity or a NaN; -2: it is all zeros
    static constexpr uint32_t CTRL = INV0 + 512;         // mma mbarrier (8 B), tmem base (4 B), pad, full[2], empty[2] mbarriers,
                                                         // queue counts [2]
    static constexpr uint32_t GRID = 0x1000;             // uint32[TC_BUCKETS] bucket table, see the kernel
    static constexpr uint32_t A_X = 0x2000;              // the vectors: 2 K-regions x [128 rows][128 B]
    static constexpr uint32_t B_R = 0xA000;              // R: rows = output coordinate d, K-major
    static constexpr uint32_t DST1 = 0x12000;
    static constexpr uint32_t INV1 = DST1 + 1024;
    static constexpr uint32_t LIST0 = INV1 + 512;        // uint32[TC_LIST_CAP] x 2: queued (vector << 8 | coordinate)
    static constexpr uint32_t LIST1 = LIST0 + 4 * TC_LIST_CAP;
    static constexpr uint32_t END = LIST1 + 4 * TC_LIST_CAP;
};
static_assert(TcSmem::CTRL + 64 <= TcSmem::GRID, "control words run into the bucket table");
constexpr size_t TC_DYN_SMEM = TcSmem::END;  // enough wherever the dynamic shared memory starts at or below TcSmem::DST0
constexpr int TC_CTAS_PER_SM = 3;
static_assert(TC_CTAS_PER_SM * (TC_DYN_SMEM + 1024) <= 228 * 1024, "three CTAs of the tensor-core append must fit one SM");

struct PrefillTcParams {
    uint8_t* ck;
    __half* kn;
    uint8_t* cv;
    __half* vn;
    const __half* k_buf;       // [T][kv_dim], either may be null
    const __half* v_buf;
    const __half* rotation;    // [128][128] row-major
    const int* positions;      // [T] device, or null: token t goes to position pos_value + t
    int pos_value;
    int* status;
    long long token_row0;      // first cache row of sequence 0 of the call
    long long seq_stride_rows; // rows between consecutive sequences of the call (when row_base is null)
    const long long* row_base; // optional: first cache row per sequence, indexed from the call's first sequence
    int capacity_rows;
    int n_seq;                 // sequences in the call: inputs are [n_seq][T][kv_dim], all at the same positions
    int T, Hkv, kv_dim, bits;
    // Decode-step form (step_G > 0): the call appends ONE new token of each of step_G sequences in n_seq / step_G layers
    // at once.  "Sequence" s of the call is then (layer s / step_G, sequence s % step_G): T = 1, inputs [layers][step_G]
    // [kv_dim], position positions[s % step_G], row base of sequence s % step_G, and the arrays of layer l lie
    // code_layer_stride bytes (norm_layer_stride halves) behind those of the call's first layer.
    int step_G;
    long long code_layer_stride;
    long long norm_layer_stride;
    const int* seq_capacity;   // optional, decode-step form: rows each sequence may use (else capacity_rows for all)
    // Producer form (PRODUCER = true): k_buf holds the K projection's raw output; the per-head RMS norm with weights and
    // the rotary embedding of the reference's qk_norm_batch_kernel + rope_batch_kernel (engine/kernels.cu:880-962) are
    // applied while the vectors are loaded -- the reference's arithmetic, including its two roundings to fp16 -- so the
    // K vectors that get quantised are bit for bit the ones the reference would have stored in its k buffer.  V vectors
    // are taken as they are.
    const __half* norm_w;      // [layers][128] RMS-norm weights of the K heads (layer of the call's first layer first)
    const __half* rope_cos;    // [positions][rope_dim / 2]
    const __half* rope_sin;
    int rope_dim;              // 64 or 128
    float eps;
    int biased;
#ifdef TQ_TIMING_SWITCHES
    unsigned long long* stamps;  // timing-experiment builds only: [2][16] summed clock deltas of a tile's sections (warps 0, 7)
#endif
    __half* k_post;            // [vectors][128] like k_buf: receives the produced K vectors (what the reference's k buffer
                               // holds after its two kernels); the exact chains of near-bound coordinates re-read them
};

#ifdef TQ_TIMING_SWITCHES
#define TC_STAMP(i) do { const long long _t = clock64(); tc_stamp_acc[i] += _t - tc_stamp_last; tc_stamp_last = _t; } while (0)
#else
#define TC_STAMP(i) do { } while (0)
#endif

// ---- tcgen05 wrappers ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem] * B[smem]^T, fp16 operands, fp32 accumulate, issued by ONE thread
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread l of the warp receives lane (row) base+l
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ bool named_barrier_or(int id, int nthreads, bool pred) {  // true if pred holds for any thread
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %3, 0;\n\t"
        "bar.red.or.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(id), "r"(nthreads), "r"((uint32_t)(pred ? 1 : 0))
        : "memory");
    return r != 0u;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Two fp32 operations per instruction (the packed fp32 forms of this architecture), each half rounded exactly like
// the scalar instruction of the same name.
__device__ __forceinline__ float2 mul2_ftz(float2 a, float2 b) {
    unsigned long long d;
    asm("mul.rn.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 add2_ftz(float2 a, float2 b) {
    unsigned long long d;
    asm("add.rn.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fma2_ftz(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {  // (no flush to zero)
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
// Sum of the squares of 32 fp16 values given as 16 float pairs, in the order of the reference's shuffle tree over 32
// lanes (offsets 16, 8, 4, 2, 1 with element l in lane l's place).  The square of an fp16 value is exact in fp32, so
// the first level's a*a + b*b is one fused multiply-add on top of one multiplication: same bits as two products and a sum.
__device__ __forceinline__ float sumsq_tree32(const float2 (&v)[16]) {
    float2 s[8];
#pragma unroll
    for (int l = 0; l < 8; ++l) s[l] = fma2_ftz(v[l + 8], v[l + 8], mul2_ftz(v[l], v[l]));
#pragma unroll
    for (int l = 0; l < 4; ++l) s[l] = add2_ftz(s[l], s[l + 4]);
    s[0] = add2_ftz(s[0], s[2]);
    s[1] = add2_ftz(s[1], s[3]);
    s[0] = add2_ftz(s[0], s[1]);
    return add_ftz(s[0].x, s[0].y);
}
// One entry of the bucket table (see the kernel), addressed by the low mantissa bits of the grid value.
__device__ __forceinline__ uint32_t bucket_entry(uint32_t grid_bits) {
    uint32_t e;
    asm("ld.shared.u32 %0, [%1 + %2];" : "=r"(e) : "r"(grid_bits & (uint32_t)(4 * TC_BUCKETS - 4)), "n"(TcSmem::GRID));
    return e;
}
// Division of n < 2^31 by a divisor fixed for the launch: q = (n * mul) >> shift with mul = ceil(2^shift / d),
// shift = 31 + ceil(log2 d); exact because n * (mul * d - 2^shift) < 2^shift.
__device__ __forceinline__ uint2 fastdiv_make(uint32_t d) {  // (mul, shift)
    const uint32_t l = d > 1u ? 32u - (uint32_t)__clz((int)(d - 1u)) : 0u;
    return make_uint2((uint32_t)((((unsigned long long)1 << (31u + l)) + d - 1u) / d), 31u + l);
}
__device__ __forceinline__ int fastdiv(int n, uint2 ms) { return (int)(((unsigned long long)(uint32_t)n * ms.x) >> ms.y); }
__device__ __forceinline__ uint32_t mad_hi_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.hi.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Shared-memory matrix descriptor of a K-major operand tile with the 128-byte swizzle: rows of 128 bytes, groups of
// 8 rows 1024 bytes apart; `addr` is the shared address of the tile (1024-byte aligned) plus 32 bytes per K-step.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu)      // start address
           | (1ull << 16)                          // leading byte offset (unused with a swizzle)
           | ((uint64_t)(1024u >> 4) << 32)        // stride byte offset: next group of 8 rows
           | (1ull << 46)                          // descriptor version of this architecture
           | (2ull << 61);                         // layout: 128-byte swizzle
}
// fp16 x fp16 -> fp32, both operands K-major, M = 128, N = 128
constexpr uint32_t TC_IDESC = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ uint32_t tc_operand_addr(uint32_t tile, int row, int k) {  // byte address of element (row, k)
    const uint32_t region = (uint32_t)k >> 6, kk = (uint32_t)k & 63u;
    return tile + region * 16384u + (uint32_t)row * 128u + ((((kk >> 3) ^ ((uint32_t)row & 7u))) << 4) + (kk & 7u) * 2u;
}

// TMA_IN: the tile's 128 vectors reach the operand tile by ONE tensor-map copy (issued while the previous tile is being
// quantised) instead of through registers; the sums of squares are then taken from shared memory while the tensor core
// already rotates.  Needs a tensor map over the input (make_append_input_map) and Hkv dividing 128; never with PRODUCER.
template <bool PRODUCER, bool TMA_IN>
__global__ void __launch_bounds__(TC_THREADS, PRODUCER ? 2 : TC_CTAS_PER_SM)  // (the producer form needs more registers)
prefill_append_tc_kernel(const __grid_constant__ CUtensorMap tm_k_in, const __grid_constant__ CUtensorMap tm_v_in, const PrefillTcParams p) {
    static_assert(!(PRODUCER && TMA_IN), "the producer form computes its K vectors: they cannot come by a bulk copy");
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t dyn_base = smem_u32(tc_smem);
    if (dyn_base > TcSmem::DST0 || dyn_base + (uint32_t)TC_DYN_SMEM < TcSmem::END) {  // (uniform over the CTA)
        if (tid == 0) atomicMax(p.status, ST_SMEM_LAYOUT);
        return;
    }
    constexpr uint32_t base = 0u;                 // TcSmem holds absolute shared addresses
    uint8_t* gbase = tc_smem - dyn_base;          // generic address of shared address 0
    const uint32_t bar = base + TcSmem::CTRL;       // the tensor core's commits arrive here
    const uint32_t bar_full = bar + 16u;            // [2]: a tile's queue, per-vector arrays and stored codes are complete
    const uint32_t bar_empty = bar + 32u;           // [2]: the chain warp is done with them
    const uint32_t bar_ld = bar + 56u;              // TMA_IN: the tile's vectors have arrived in the operand tile
    volatile uint32_t* ctrl = reinterpret_cast<volatile uint32_t*>(gbase + TcSmem::CTRL);  // [2] tmem base, [12 + b] queue count
    uint32_t* grid_s = reinterpret_cast<uint32_t*>(gbase + TcSmem::GRID);
    auto dst_buf = [&](int b) { return reinterpret_cast<long long*>(gbase + (b ? TcSmem::DST1 : TcSmem::DST0)); };
    auto inv_buf = [&](int b) { return reinterpret_cast<float*>(gbase + (b ? TcSmem::INV1 : TcSmem::INV0)); };
    auto list_buf = [&](int b) { return reinterpret_cast<uint32_t*>(gbase + (b ? TcSmem::LIST1 : TcSmem::LIST0)); };

    const int bits = p.bits;
    const int nb = bits == 4 ? 15 : 3;
    const int bpv = bits == 4 ? 64 : 32;  // packed bytes per vector
    const int kvp = p.Hkv * bpv;

    // ---- once per CTA: tensor memory, barrier, R operand tile, bucket table ----
    if (warp == 0) {
        tmem_alloc(base + TcSmem::CTRL + 8u, 128u);  // one accumulator of 128 columns (three CTAs share the SM's 512)
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init(bar_full, 1);
        mbar_init(bar_full + 8u, 1);
        mbar_init(bar_empty, 1);
        mbar_init(bar_empty + 8u, 1);
        mbar_init(bar_ld, 1);
        fence_mbar_init();
    }
    for (int c = tid; c < 2048; c += TC_THREADS) {  // R as the B operand: row d, 16-byte chunk j
        const int d = c >> 4, j = c & 15;
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(p.rotation + (size_t)d * HEAD_DIM) + j);
        *reinterpret_cast<uint4*>(gbase + (tc_operand_addr(base + TcSmem::B_R, d, 8 * j) - base)) = u;
    }
    for (int i = tid; i < TC_BUCKETS; i += TC_THREADS) {
        // Bucket table over the rotated coordinate x.  The epilogue forms k = rne(4 x / w) in the low mantissa bits of
        // fma(x, 1 / w, 1.5 * 2^21) and takes bucket k >> 2 (modulo 256): bucket n holds x in [(n - 0.125) w, (n + 0.875) w],
        // |x| < 2.  The width w = 1/46 is the largest handy one below the smallest distance of two bounds (0.0228 at four
        // bits), so no bucket holds two -- and the 32 buckets around zero, where a rotated coordinate (sigma = 0.088) falls
        // with probability 0.9999, sit in 32 different shared-memory banks: the look-ups of a warp rarely collide.  An
        // entry is ONE float: the decision
        // bound that lies inside the bucket (widened by four margins) with its four lowest mantissa bits replaced by the
        // code a value BELOW the bound gets -- the code is then entry_code + (x > bound) -- or, when no bound is near the
        // bucket, 0x7f000000 (1.7e38: every x is below it) carrying the bucket's code.  The replaced bits move the bound
        // by less than 3e-7; the near-bound test uses a margin wider by more than that, and only coordinates outside it
        // keep the code found here.
        const int n = i < TC_BUCKETS / 2 ? i : i - TC_BUCKETS;
        const float lo = ((float)(4 * n) - 0.5f) * (0.25f / TC_BUCKETS_PER_UNIT), hi = lo + (1.0f / TC_BUCKETS_PER_UNIT);
        int code = 0, amb = -1;
        float ambv = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const float bv = bits == 4 ? kBnd4[b] : kBnd2[b];
            if (bv <= lo) ++code;
            if (bv >= lo - 4.0f * TC_MARGIN && bv <= hi + 4.0f * TC_MARGIN) {
                if (amb >= 0) atomicMax(p.status, ST_SMEM_LAYOUT);  // (two bounds in one bucket: the table cannot say which)
                amb = b;
                ambv = bv;
            }
        }
        grid_s[i] = amb >= 0 ? ((__float_as_uint(ambv) & ~15u) | (uint32_t)amb) : (0x7f000000u | (uint32_t)code);
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctrl[2];

    const int vec_per_seq = p.T * p.Hkv;
    const int vec_per_kind = p.n_seq * vec_per_seq;
    const int tiles_per_kind = (vec_per_kind + TC_TILE - 1) / TC_TILE;
    const int n_kinds = (p.k_buf ? 1 : 0) + (p.v_buf ? 1 : 0);
    const int total_tiles = tiles_per_kind * n_kinds;
    uint32_t phase = 0;
    bool dead = false;
    // Vector -> (token, head) and token -> (sequence, position) without a division per vector: one division per tile for
    // its first vector, then a multiplication by a reciprocal (exact for the small offsets inside a tile) and, for
    // prompts longer than a tile, one conditional step into the next sequence.
    const bool fast_head = p.Hkv <= 256;
    const uint32_t hkv_magic = ((1u << 20) + (uint32_t)p.Hkv - 1u) / (uint32_t)p.Hkv;
    const bool fast_tok = p.T > TC_TILE + 1;
    const uint2 div_hkv = fastdiv_make((uint32_t)p.Hkv), div_T = fastdiv_make((uint32_t)p.T),
                div_G = fastdiv_make((uint32_t)(p.step_G > 0 ? p.step_G : 1));

    const int ev = (warp & 3) * 32 + lane;    // this thread's vector in the epilogue
    const int cc0 = (warp >> 2) * 2;          // its first block of 32 coordinates (warps 0-7)

    // The reference's k-ascending fp32 chain for coordinate d of one vector (x: its 128 fp16 inputs in global memory),
    // by one thread; R comes from the operand tile in shared memory.
    auto exact_code = [&](const __half* x, float inv, int d) -> int {
        const uint4* src = reinterpret_cast<const uint4*>(x);
        float acc = 0.0f;
#pragma unroll 1
        for (int j0 = 0; j0 < 16; j0 += 8) {  // eight 16-byte loads in flight at a time
            uint4 xall[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) xall[j] = src[j0 + j];  // (plain loads: a produced K vector was written by this CTA)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint4 xv = xall[j];
                const uint4 rv = *reinterpret_cast<const uint4*>(gbase + tc_operand_addr(TcSmem::B_R, d, 8 * (j0 + j)));
                const __half2* xh = reinterpret_cast<const __half2*>(&xv);
                const __half2* rh = reinterpret_cast<const __half2*>(&rv);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 xf = __half22float2(xh[e]), rf = __half22float2(rh[e]);
                    acc = fma_ftz(rf.x, mul_ftz(xf.x, inv), acc);
                    acc = fma_ftz(rf.y, mul_ftz(xf.y, inv), acc);
                }
            }
        }
        return quantize_code(acc, bits);
    };
    auto patch = [&](uint8_t* codes, int d, int code) {  // one code of a vector in the cache (the tile's stores came before)
        uint32_t* w = reinterpret_cast<uint32_t*>(codes) + (bits == 4 ? d >> 3 : d >> 4);
        const int sh = bits == 4 ? 4 * (d & 7) : 2 * (d & 15);
        const uint32_t m = (bits == 4 ? 0xfu : 0x3u) << sh;
        atomicAnd(w, ~m);
        atomicOr(w, (uint32_t)code << sh);
    };
    auto vector_input = [&](int kind, int vid) -> const __half* {  // the 128 inputs of vector vid of a kind, as rotated
        const int tok = fastdiv(vid, div_hkv), head = vid - tok * p.Hkv;
        const __half* buf = kind == 0 ? (PRODUCER ? p.k_post : p.k_buf) : p.v_buf;
        return buf + (size_t)tok * p.kv_dim + (size_t)head * HEAD_DIM;
    };

    // ---- the chain warp: step 4 of every tile, one tile behind the workers.  A coordinate within TC_MARGIN of a bound
    //      (about 23 of a tile's 16384) is queued by the epilogue; here one lane per item runs the exact chain and patches
    //      the stored code.  None of the workers' barriers waits for it. ----
    if (warp == TC_WORKERS / 32) {
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            const int b = (int)(it & 1u);
            const int kind = (p.k_buf && tile < tiles_per_kind) ? 0 : 1;
            const int vec0 = (tile - (kind == 0 || !p.k_buf ? 0 : tiles_per_kind)) * TC_TILE;
            uint8_t* cq = kind == 0 ? p.ck : p.cv;
            if (!mbar_wait_bounded_hint(bar_full + 8u * (uint32_t)b, (it >> 1) & 1u, 1u << 18, 4000u)) {
                if (lane == 0) atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
                return;
            }
            const uint32_t queued = min(ctrl[12 + b], (uint32_t)TC_LIST_CAP);
            const uint32_t* list_s = list_buf(b);
            const float* inv_s = inv_buf(b);
            const long long* dst_s = dst_buf(b);
            for (uint32_t i = (uint32_t)lane; i < queued; i += 32u) {
                const uint32_t item = list_s[i];
                const int v = (int)(item >> 8), d = (int)(item & 255u);
                const long long dst = dst_s[v];
                if (dst >= 0) patch(cq + dst, d, exact_code(vector_input(kind, vec0 + v), inv_s[v], d));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8u * (uint32_t)b);
        }
        return;
    }

#ifdef TQ_TIMING_SWITCHES
    long long tc_stamp_acc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0}, tc_stamp_last = clock64();
#endif
    uint32_t it = 0;  // tiles this CTA has started: parity of the per-tile arrays, phase of their barriers
    uint32_t ld_phase = 0;
    // TMA form: where this lane's 32-coordinate chunk of row 8 * warp + (lane & 7) starts in the operand tile (see 2b)
    const uint32_t tree_addr = tc_operand_addr(TcSmem::A_X, 8 * warp + (lane & 7), 32 * (lane >> 3));
    auto issue_load = [&](int tile_n) {  // one thread: the 128 vectors of a tile -> operand tile, [half][token][head][128 B]
        const int kind_n = (p.k_buf && tile_n < tiles_per_kind) ? 0 : 1;
        const int vec0_n = (tile_n - (kind_n == 0 || !p.k_buf ? 0 : tiles_per_kind)) * TC_TILE;
        mbar_arrive_expect_tx(bar_ld, 2u * 16384u);  // (rows past the end of the input arrive as zeros and count)
        tma_load_4d(TcSmem::A_X, kind_n == 0 ? &tm_k_in : &tm_v_in, bar_ld, 0, 0, fastdiv(vec0_n, div_hkv), 0);
    };
    if constexpr (TMA_IN) {
        if (tid == 0 && (int)blockIdx.x < total_tiles) issue_load((int)blockIdx.x);
    }

    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
        TC_STAMP(9);
        const int b = (int)(it & 1u);
        long long* const dst_s = dst_buf(b);
        float* const inv_s = inv_buf(b);
        uint32_t* const list_s = list_buf(b);
        const int kind = (p.k_buf && tile < tiles_per_kind) ? 0 : 1;
        const int vec0 = (tile - (kind == 0 || !p.k_buf ? 0 : tiles_per_kind)) * TC_TILE;
        const __half* src_buf = kind == 0 ? p.k_buf : p.v_buf;
        uint8_t* cq = kind == 0 ? p.ck : p.cv;
        __half* cn = kind == 0 ? p.kn : p.vn;
        const int tok0 = fastdiv(vec0, div_hkv), head0 = vec0 - tok0 * p.Hkv;
        const int seq0 = fastdiv(tok0, div_T), t0 = tok0 - seq0 * p.T;
        auto split_vec = [&](int v, int& tok, int& head) {  // vector vec0 + v of the tile
            if (fast_head) {
                const uint32_t x = (uint32_t)(head0 + v), dq = (x * hkv_magic) >> 20;
                tok = tok0 + (int)dq;
                head = (int)(x - dq * (uint32_t)p.Hkv);
            } else {
                tok = fastdiv(vec0 + v, div_hkv);
                head = (vec0 + v) - tok * p.Hkv;
            }
        };
        auto split_tok = [&](int tok, int& seq, int& t) {
            if (fast_tok) {
                const int tt = t0 + (tok - tok0);
                const bool wrap = tt >= p.T;
                seq = seq0 + (wrap ? 1 : 0);
                t = tt - (wrap ? p.T : 0);
            } else {
                seq = fastdiv(tok, div_T);
                t = tok - seq * p.T;
            }
        };

        TC_STAMP(0);
        // ---- 1. load, sum of squares in the reference's order ----
        constexpr int PASSES = 4 * TC_TILE / TC_WORKERS, VPP = TC_WORKERS / 4;  // passes per tile, vectors per pass
        uint4 raw_all[PASSES][4];
        float tt_all[PASSES];
        if constexpr (!TMA_IN) {
#pragma unroll
        for (int pass = 0; pass < PASSES; ++pass) {  // every load of the tile goes out before the arithmetic starts
            const int vid = vec0 + pass * VPP + (tid >> 2);
            const bool live = vid < vec_per_kind;
            int tok = 0, head = 0;  // tok = sequence * T + t
            if (live) split_vec(pass * VPP + (tid >> 2), tok, head);
            const uint4* src = reinterpret_cast<const uint4*>(src_buf + (size_t)tok * p.kv_dim + (size_t)head * HEAD_DIM + 32 * (tid & 3));
#pragma unroll
            for (int i = 0; i < 4; ++i) raw_all[pass][i] = live ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
        }
        }
        // One thread per vector settles it (norm out, 1/norm, where its codes go): thread v < 128, or, in the TMA form, the
        // lane that ends up holding the vector's sum of squares.  Its position and row base are loads of their own: issued
        // here, needed only once the operands are with the tensor core.
        const int settle_v = TMA_IN ? (lane < 16 ? 64 * (lane >> 3) + 8 * warp + (lane & 7) : -1) : (tid < TC_TILE ? tid : -1);
        long long my_row_base = 0;
        int my_pos = -1, my_head_layer = 0;  // position in the sequence (-1: the vector is not stored), head | layer << 16
        if (settle_v >= 0 && vec0 + settle_v < vec_per_kind) {
            int tok, head, seq, t, layer = 0;
            split_vec(settle_v, tok, head);
            split_tok(tok, seq, t);
            int sq = seq, cap = p.capacity_rows;
            if (p.step_G > 0) {
                layer = fastdiv(seq, div_G);
                sq = seq - layer * p.step_G;
                if (p.seq_capacity) cap = p.seq_capacity[sq];
            }
            const int pos = p.step_G > 0 ? p.positions[sq] : (p.positions ? p.positions[t] : p.pos_value + t);
            my_row_base = p.row_base ? p.row_base[sq] : p.token_row0 + (long long)sq * p.seq_stride_rows;
            my_head_layer = head | (layer << 16);
            if (pos >= 0 && (cap <= 0 || pos < cap)) my_pos = pos;
            else atomicMax(p.status, ST_BAD_POSITION);
        }
        if constexpr (!TMA_IN) {
        {   // the CTA's next tile (same kind or the other one) on its way into L2 while this one is worked on
            const int ntile = tile + (int)gridDim.x;
            if (ntile < total_tiles) {
                const int nkind = (p.k_buf && ntile < tiles_per_kind) ? 0 : 1;
                const int nvid = (ntile - (nkind == 0 || !p.k_buf ? 0 : tiles_per_kind)) * TC_TILE + (tid >> 1);
                if (nvid < vec_per_kind) {  // one 128-byte line per thread
                    const int ntok = fastdiv(nvid, div_hkv), nhead = nvid - ntok * p.Hkv;
                    const __half* a = (nkind == 0 ? p.k_buf : p.v_buf) + (size_t)ntok * p.kv_dim + (size_t)nhead * HEAD_DIM + 64 * (tid & 1);
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
                }
            }
        }
        TC_STAMP(1);
#pragma unroll
        for (int pass = 0; pass < PASSES; ++pass) {
            const int v = pass * VPP + (tid >> 2), c = tid & 3;  // vector within the tile, 32-coordinate chunk
            const int vid = vec0 + v;
            const bool live = vid < vec_per_kind;
            int tok = 0, head = 0, seq = 0, t = 0;
            if (PRODUCER && live) {  // (where the vector goes is worked out once per vector, below)
                split_vec(v, tok, head);
                split_tok(tok, seq, t);
            }
            uint4 (&raw)[4] = raw_all[pass];  // becomes the operand: the input as it is, or the produced K vector
            float2 v2[16];                    // the chunk's 32 values as pairs (2j, 2j + 1)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __half2* h2 = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) v2[4 * i + e] = __half22float2(h2[e]);
            }
            const int l0 = lane & ~3;
            if constexpr (PRODUCER) {
                if (kind == 0) {  // K vectors only; every thread of the warp walks the shuffles
                    // RMS norm: sum of squares by the reference's block tree, x * rms * w rounded to fp16
                    const float qpart = sumsq_tree32(v2);
                    const float q0 = __shfl_sync(0xffffffffu, qpart, l0), q1 = __shfl_sync(0xffffffffu, qpart, l0 + 1);
                    const float q2 = __shfl_sync(0xffffffffu, qpart, l0 + 2), q3 = __shfl_sync(0xffffffffu, qpart, l0 + 3);
                    const float rms = rsqrt_approx_ftz(fma_ftz(add_ftz(add_ftz(q0, q2), add_ftz(q1, q3)), 1.0f / HEAD_DIM, p.eps));
                    int layer = 0, sq_i = seq, ppos;
                    if (p.step_G > 0) {
                        layer = fastdiv(seq, div_G);
                        sq_i = seq - layer * p.step_G;
                        ppos = live ? p.positions[sq_i] : 0;
                    } else {
                        ppos = live ? (p.positions ? p.positions[t] : p.pos_value + t) : 0;
                    }
                    if (ppos < 0) ppos = 0;
                    const uint4* wsrc = reinterpret_cast<const uint4*>(p.norm_w + (size_t)layer * HEAD_DIM + 32 * c);
                    uint32_t nh[16];  // the normalised chunk as fp16 pairs
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 wu = __ldg(wsrc + i);
                        const __half2* w2 = reinterpret_cast<const __half2*>(&wu);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float2 wf = __half22float2(w2[e]);
                            if (p.biased) { wf.x = add_ftz(wf.x, 1.0f); wf.y = add_ftz(wf.y, 1.0f); }
                            const __half2 h = __floats2half2_rn(mul_ftz(mul_ftz(v2[4 * i + e].x, rms), wf.x),
                                                                mul_ftz(mul_ftz(v2[4 * i + e].y, rms), wf.y));
                            nh[4 * i + e] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                    }
                    // rotary pairs (d, d + rope_dim / 2): this thread's chunk c with the chunk of thread c ^ (rope_dim / 64)
                    const int hr32 = p.rope_dim >> 6, half_rope = p.rope_dim >> 1;
                    const bool roped = c < 2 * hr32, low = c < hr32;
                    const int cd = 32 * (low ? c : c - hr32);  // first rotary index of the pair's low chunk
                    const uint4* csrc = reinterpret_cast<const uint4*>(p.rope_cos + (size_t)ppos * half_rope + (roped ? cd : 0));
                    const uint4* ssrc = reinterpret_cast<const uint4*>(p.rope_sin + (size_t)ppos * half_rope + (roped ? cd : 0));
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 cu = __ldg(csrc + i), su = __ldg(ssrc + i);
                        const __half2* c2 = reinterpret_cast<const __half2*>(&cu);
                        const __half2* s2 = reinterpret_cast<const __half2*>(&su);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t mine = nh[4 * i + e];
                            const uint32_t other = __shfl_xor_sync(0xffffffffu, mine, hr32);  // (lanes of one vector differ in c only)
                            const float2 xo = __half22float2(*reinterpret_cast<const __half2*>(&mine));
                            const float2 xp = __half22float2(*reinterpret_cast<const __half2*>(&other));
                            const float2 cf = __half22float2(c2[e]), sf = __half22float2(s2[e]);
                            float2 r = xo;
                            if (roped) {
                                if (low) {  // x0 = mine, x1 = partner: x0 * c - x1 * s
                                    r.x = __half2float(__float2half_rn(fma_ftz(xo.x, cf.x, -mul_ftz(xp.x, sf.x))));
                                    r.y = __half2float(__float2half_rn(fma_ftz(xo.y, cf.y, -mul_ftz(xp.y, sf.y))));
                                } else {    // x0 = partner, x1 = mine: x0 * s + x1 * c
                                    r.x = __half2float(__float2half_rn(fma_ftz(xp.x, sf.x, mul_ftz(xo.x, cf.x))));
                                    r.y = __half2float(__float2half_rn(fma_ftz(xp.y, sf.y, mul_ftz(xo.y, cf.y))));
                                }
                            }
                            v2[4 * i + e] = r;
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {  // (the values are fp16 numbers already: the conversion is exact)
                        __half2 o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) o[e] = __floats2half2_rn(v2[4 * i + e].x, v2[4 * i + e].y);
                        raw[i] = *reinterpret_cast<const uint4*>(o);
                    }
                    if (live) {
                        uint4* dstp = reinterpret_cast<uint4*>(p.k_post + (size_t)tok * p.kv_dim + (size_t)head * HEAD_DIM + 32 * c);
#pragma unroll
                        for (int i = 0; i < 4; ++i) dstp[i] = raw[i];
                    }
                }
            }
            // the warp-shuffle tree of the reference (offsets 16, 8, 4, 2, 1) within the chunk, then across the four chunks
            const float part = sumsq_tree32(v2);
            const float p0 = __shfl_sync(0xffffffffu, part, l0), p1 = __shfl_sync(0xffffffffu, part, l0 + 1);
            const float p2 = __shfl_sync(0xffffffffu, part, l0 + 2), p3 = __shfl_sync(0xffffffffu, part, l0 + 3);
            tt_all[pass] = add_ftz(add_ftz(add_ftz(p0, p2), add_ftz(p1, p3)), 1e-12f);
        }
        }
        TC_STAMP(2);
        // The operand tile is free (its MMAs were waited for, and the epilogue reads tensor memory only); the per-vector
        // arrays and the queue of this parity are free once the chain warp is through with the tile before the last.
        if (!dead && !mbar_wait_bounded(bar_empty + 8u * (uint32_t)b, ((it >> 1) & 1u) ^ 1u, 1u << 24)) {
            dead = true;
            atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
        }
        TC_STAMP(3);
        if (tid == 0) ctrl[12 + b] = 0;
        if constexpr (!TMA_IN) {
#pragma unroll
        for (int pass = 0; pass < PASSES; ++pass) {  // the vectors as they are become the A operand
            const int v = pass * VPP + (tid >> 2), c = tid & 3;
            if (c == 0) inv_s[v] = tt_all[pass];  // turned into 1/norm below
#pragma unroll
            for (int i = 0; i < 4; ++i) {  // 16-byte chunks: coordinates 32c + 8i .. + 7
                const uint32_t a = tc_operand_addr(base + TcSmem::A_X, v, 32 * c + 8 * i);
                const uint4 r = raw_all[pass][i];
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w) : "memory");
            }
        }
        fence_proxy_async_smem();  // generic-proxy writes of the operands before the tensor core reads them
        named_barrier(1, TC_WORKERS);
        } else {
            if (!dead) {
                if (mbar_wait_bounded_hint(bar_ld, ld_phase, 1u << 18, 2000u)) {
                    ld_phase ^= 1u;
                } else {
                    dead = true;
                    atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
                }
            }
        }
        TC_STAMP(4);

        // ---- 2. the rotation: 8 K-steps into one accumulator ----
        if (tid == 0 && !dead) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t koff = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                umma_f16(tmem, umma_desc_sw128(base + TcSmem::A_X + koff), umma_desc_sw128(base + TcSmem::B_R + koff), TC_IDESC, ks != 0);
            }
            umma_commit(bar);
        }
        // ---- 2b. while the tensor core works ----
        float my_tt = 0.0f;
        if constexpr (TMA_IN) {
            // Sums of squares from the operand tile.  Pass q: lane (r, c) of warp w takes chunk c (32 coordinates) of vector
            // 64 q + 8 w + r; the eight lanes of a quarter-warp read eight different rows, whose 128-byte swizzle puts their
            // 16-byte pieces on different banks.  The four chunk sums meet by shuffles, in the reference's order.
            // (piece i of the chunk sits at tree_addr ^ (i << 4): the swizzle only exchanges pieces within the chunk's 64 bytes;
            // pass 1's rows lie 64 rows = 8192 bytes further, with the same swizzle)
            const int r = lane & 7, c = lane >> 3;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                float2 v2[16];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 u = *reinterpret_cast<const uint4*>(gbase + ((tree_addr ^ (uint32_t)(i << 4)) + (uint32_t)(q * 8192)));
                    const __half2* h2 = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                    for (int e = 0; e < 4; ++e) v2[4 * i + e] = __half22float2(h2[e]);
                }
                const float part = sumsq_tree32(v2);
                const float p0 = __shfl_sync(0xffffffffu, part, r), p1 = __shfl_sync(0xffffffffu, part, r + 8);
                const float p2 = __shfl_sync(0xffffffffu, part, r + 16), p3 = __shfl_sync(0xffffffffu, part, r + 24);
                const float tt = add_ftz(add_ftz(add_ftz(p0, p2), add_ftz(p1, p3)), 1e-12f);
                if (c == q) my_tt = tt;
            }
        } else {
            if (settle_v >= 0) my_tt = inv_s[settle_v];
        }
        if (settle_v >= 0) {  // settle the vector: norm out, 1/norm, where its codes go
            const bool abnormal = !(my_tt < 3.0e38f);  // an infinity or a NaN among the inputs: every coordinate is a NaN
            long long my_dst = -1;  // byte offset of the vector's codes in the cache
            if (my_pos >= 0) {
                const long long row = my_row_base + my_pos;
                const int head = my_head_layer & 65535, layer = my_head_layer >> 16;
                my_dst = (long long)layer * p.code_layer_stride + row * kvp + (long long)head * bpv;
                cn[(long long)layer * p.norm_layer_stride + row * p.Hkv + head] = __float2half_rn(sqrt_approx_ftz(my_tt));
            }
            dst_s[settle_v] = my_dst;
            // (an all-zero vector -- padding, say -- has every coordinate ON the bound 0: 128 exact chains, all with the result
            //  +0; it gets its constant codes directly instead.  The sum of squares of any other fp16 vector is at least 3.6e-15.)
            inv_s[settle_v] = abnormal ? -1.0f : (my_tt == 1e-12f ? -2.0f : rsqrt_approx_ftz(my_tt));
        }
        TC_STAMP(5);
        if (!dead && !mbar_wait_bounded_hint(bar, phase, 1u << 18, 2000u)) {
            dead = true;
            atomicMax(p.status, ST_TMA_WAIT_TIMEOUT);
        }
        dead = named_barrier_or(1, TC_WORKERS, dead);
        phase ^= 1u;
        tc_fence_after();
        if constexpr (TMA_IN) {  // the operand tile has been read by the tensor core and by every thread: the next tile's vectors
            if (tid == 0 && !dead && tile + (int)gridDim.x < total_tiles) issue_load(tile + (int)gridDim.x);
        }
        TC_STAMP(6);

        // ---- 3. accumulators -> codes.  A warp reaches the 32 TMEM lanes (vectors) of its rank modulo 4; warps w and
        //         w + 4 share those vectors and take 64 of the 128 coordinates (two blocks of 32 columns) each ----
        uint32_t own0 = 0u, own1 = 0u;  // near-bound coordinates (of this thread's two blocks) that did not fit the shared queue
        long long ev_dst_keep = -1;
        if (!dead) {
            const float inv = inv_s[ev];
            const long long ev_dst = dst_s[ev];
            ev_dst_keep = ev_dst;
            const bool abn = inv < 0.0f;
            const float2 inv2 = make_float2(inv, inv), inv256 = make_float2(inv * TC_BUCKETS_PER_UNIT, inv * TC_BUCKETS_PER_UNIT);
            const float2 magic2 = make_float2(3145728.0f, 3145728.0f), minus1 = make_float2(-1.0f, -1.0f);
            constexpr float kNear = TC_MARGIN + 1.0e-6f;
            const float2 minus_m2 = make_float2(-kNear * kNear, -kNear * kNear);
#pragma unroll 1
            for (int cc = cc0; cc < cc0 + 2; ++cc) {
                uint32_t acc_r[32];
                const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)cc * 32u;
                tmem_ld32(taddr, acc_r);
                tmem_ld_wait();
                uint32_t words[4] = {0u, 0u, 0u, 0u};
                uint32_t near_rev = 0u;  // bit 31 - i: coordinate i is near a bound (queued after the loop)
                // Two coordinates at a time, ascending; codes and near-bound flags are shifted in by funnel shifts, which
                // keep only the bits that count: the entry's four (two) low bits plus one if the value lies above the
                // entry's bound (the sign of bound - value, added as the high word of twice its bits).
                auto two = [&](int i, uint32_t& word, int width) {
                    const float2 a = make_float2(__uint_as_float(acc_r[i]), __uint_as_float(acc_r[i + 1]));
                    const float2 dval = mul2(a, inv2);
                    const float2 kf = fma2(a, inv256, magic2);  // k = rne(4 * 46 x) in the low bits
                    const uint32_t e0 = bucket_entry(__float_as_uint(kf.x)), e1 = bucket_entry(__float_as_uint(kf.y));
                    const float2 dd = fma2(dval, minus1, make_float2(__uint_as_float(e0), __uint_as_float(e1)));  // bound - value
                    const float2 nn = fma2(dd, dd, minus_m2);  // negative where |bound - value| < margin
                    word = __funnelshift_r(word, mad_hi_u32(__float_as_uint(dd.x), 2u, e0), width);
                    word = __funnelshift_r(word, mad_hi_u32(__float_as_uint(dd.y), 2u, e1), width);
                    near_rev = __funnelshift_l(__float_as_uint(nn.x), near_rev, 1);
                    near_rev = __funnelshift_l(__float_as_uint(nn.y), near_rev, 1);
                };
                if (bits == 4) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int k = 0; k < 8; k += 2) two(8 * j + k, words[j], 4);
                } else {
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int k = 0; k < 16; k += 2) two(16 * j + k, words[j], 2);
                }
                uint32_t near_mask = __brev(near_rev);
                if (abn) {  // what the reference's comparisons make of a NaN: the top code at 4 bits, code 0 at 2 bits;
                            // of an all-zero vector: the code of +0 everywhere
                    const uint32_t zero_codes = (uint32_t)quantize_code(0.0f, bits) * (bits == 4 ? 0x11111111u : 0x55555555u);
                    words[0] = words[1] = words[2] = words[3] = inv == -2.0f ? zero_codes : (bits == 4 ? 0xffffffffu : 0u);
                    near_mask = 0u;
                }
                if (ev_dst < 0) near_mask = 0u;  // (a vector past the end of the input is all zeros: every coordinate ON a bound)
                while (near_mask) {
                    const int i = __ffs(near_mask) - 1;
                    near_mask &= near_mask - 1;
                    const uint32_t slot = atomicAdd(const_cast<uint32_t*>(&ctrl[12 + b]), 1u);
                    if (slot < (uint32_t)TC_LIST_CAP) list_s[slot] = ((uint32_t)ev << 8) | (uint32_t)(32 * cc + i);
                    else if (cc == cc0) own0 |= 1u << i;
                    else own1 |= 1u << i;
                }
                // 32 coordinates' codes go straight to the cache (16 or 8 bytes; the other chunks of the same 32-byte sector
                // follow from this thread's next block and from the warp that shares the vector)
                if (ev_dst >= 0) {
                    if (bits == 4) *reinterpret_cast<uint4*>(cq + ev_dst + 16 * cc) = make_uint4(words[0], words[1], words[2], words[3]);
                    else *reinterpret_cast<uint2*>(cq + ev_dst + 8 * cc) = make_uint2(words[0], words[1]);
                }
            }
        }
        TC_STAMP(7);
        tc_fence_before();  // the tensor-memory reads are done before the next tile's mma overwrites the accumulators
        named_barrier(1, TC_WORKERS);  // ... and the queue, the per-vector arrays and the stores above are complete:
        if (tid == 0) mbar_arrive(bar_full + 8u * (uint32_t)b);  // over to the chain warp
        TC_STAMP(8);
        // near-bound coordinates that did not fit the queue (none, ordinarily): their owners run the chains themselves
        if (!dead && (own0 | own1) != 0u && ev_dst_keep >= 0) {
            const __half* x = vector_input(kind, vec0 + ev);
            const float inv = inv_s[ev];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                uint32_t m = k ? own1 : own0;
                while (m) {
                    const int i = __ffs(m) - 1;
                    m &= m - 1;
                    patch(cq + ev_dst_keep, 32 * (cc0 + k) + i, exact_code(x, inv, 32 * (cc0 + k) + i));
                }
            }
        }
    }
#ifdef TQ_TIMING_SWITCHES
    if (p.stamps && lane == 0 && (warp == 0 || warp == 7)) {
        for (int i = 0; i < 10; ++i) atomicAdd(p.stamps + (warp ? 16 : 0) + i, (unsigned long long)tc_stamp_acc[i]);
        atomicAdd(p.stamps + (warp ? 16 : 0) + 15, 1ull);
    }
#endif

    if constexpr (TMA_IN) {
        // Given up on a wait: a copy into the operand tile may still be on its way; it must have landed (or never have
        // been issued: then this runs out) before the CTA's shared memory is handed to another CTA.
        if (dead && tid == 0) (void)mbar_wait_bounded(bar_ld, ld_phase, 1u << 16);
    }
    tc_fence_before();
    named_barrier(1, TC_WORKERS);
    if (warp == 0) tmem_dealloc(tmem, 128u);
}

}  // namespace tq
