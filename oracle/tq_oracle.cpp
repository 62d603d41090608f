// CPU oracle for the TurboQuant KV-cache hot path of BY571/triebwerk.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, on the host and in IEEE fp32, the arithmetic of the
// reference's CUDA kernels so that the GPU library can be checked against it.  Nothing in the product
// path (triebwerk_b200/) may call, link or import it; only tests/, __graft_entry__.smoke() and the
// cpu_baseline / --impl reference legs of bench.py do.
//
// Parity status: the reference's own tests hold no golden vector for this path (no test constructs an
// engine with kv_bits != 0), so the pin is the output of the reference's own kernels (engine/kernels.cu
// compiled unmodified for sm_100a, see oracle/Makefile) run on a B200 on seeded inputs and committed as
// tests/golden/*.npz together with the script that made them.
//
// What each function follows (paths inside the reference project):
//   tables            engine/kernels.cu:1426-1445
//   tqo_quantize      engine/kernels.cu:1448-1473   (code = number of bounds <= value)
//   tqo_centroid      engine/kernels.cu:1476-1478
//   append            engine/kernels.cu:1482-1560 (token form) and :1563-1636 (batched form)
//   attention         engine/kernels.cu:1641-1776 (batched) and :1779-1870 (single sequence)
//   prefill attention engine/kernels.cu:1874-1960
//   fp16 twin         engine/kernels.cu:964-977 (write), :981-1066 (batched attention), :244-345 (single)
//   rotation          engine/engine.cpp:364-392
//
// The reference is built with --use_fast_math (engine/CMakeLists.txt:13), i.e. FMA contraction, flushed
// denormals, rsqrt.approx / sqrt.approx / ex2.approx and approximate division.  This restatement keeps
// the reference's operation ORDER (reduction trees, k-ascending FMA chains, p-ascending V sums) with
// explicit fmaf, and uses correctly rounded sqrt / exp / division where the GPU uses approximations; the
// places where that can change a stored byte (a rotated coordinate that lands within a few ulp of a
// quantiser bound, an fp16 norm on a rounding tie) are what tests classify and count.
//
// Build: g++ -O3 -march=x86-64-v3 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <random>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---- fp16 <-> fp32, bit exact, no hardware dependence -------------------------------------------------
inline float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: renormalise
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// round-to-nearest-even, as cvt.rn.f16.f32 / __float2half
inline uint16_t f2h(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u | ((ax >> 13) & 0x3ffu) : 0u));
    }
    if (ax >= 0x477ff000u) {  // rounds to >= 65520 -> inf
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax < 0x33000001u) {  // < 2^-25 (or exactly 2^-25, a tie to even = 0)
        return (uint16_t)sign;
    }
    int e = (int)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u;
    if (e < -14) {  // subnormal result
        int shift = 13 + (-14 - e);
        uint32_t q = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) ++q;
        return (uint16_t)(sign | q);
    }
    uint32_t q = ((uint32_t)(e + 15) << 10) | ((man >> 13) & 0x3ffu);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) ++q;  // carry may bump the exponent: still right
    return (uint16_t)(sign | q);
}

// ---- code books: engine/kernels.cu:1426-1445 (literals, not recomputed) ---------------------------------
const float CENT2[4] = {-0.13351f, -0.04003f, 0.04003f, 0.13351f};
const float BND2[3] = {-0.08677f, 0.0f, 0.08677f};
const float CENT4[16] = {-0.24155f, -0.18293f, -0.14304f, -0.11099f, -0.08330f, -0.05806f, -0.03432f, -0.01135f,
                         0.01135f,  0.03432f,  0.05806f,  0.08330f,  0.11099f,  0.14304f,  0.18293f,  0.24155f};
const float BND4[15] = {-0.21224f, -0.16299f, -0.12701f, -0.09715f, -0.07068f, -0.04619f, -0.02284f, 0.00000f,
                        0.02284f,  0.04619f,  0.07068f,  0.09715f,  0.12701f,  0.16299f,  0.21224f};

// engine/kernels.cu:1448-1473.  The 4-bit form there is a tree of `val < bound` tests; for every non-NaN
// value that equals the count of bounds <= value.  NaN fails every `<` and walks to the last leaf (15);
// the 2-bit form sums `val >= bound`, which is 0 for NaN.  Both are kept.
inline int quantize(float v, int bits) {
    if (bits == 4) {
        if (v != v) return 15;
        int c = 0;
        for (int i = 0; i < 15; ++i) c += (v >= BND4[i]);
        return c;
    }
    return (v >= BND2[0]) + (v >= BND2[1]) + (v >= BND2[2]);
}
inline float centroid(int idx, int bits) { return bits == 4 ? CENT4[idx] : CENT2[idx]; }

// Distance, in fp32 ulps of the value, from v to the nearest quantiser bound.
inline float ulps_to_bound(float v, int bits) {
    const float* b = bits == 4 ? BND4 : BND2;
    int n = bits == 4 ? 15 : 3;
    float best = INFINITY;
    for (int i = 0; i < n; ++i) best = std::fmin(best, std::fabs(v - b[i]));
    float a = std::fmax(std::fabs(v), 1.17549435e-38f);
    int e;
    std::frexp(a, &e);
    float ulp = std::ldexp(1.0f, e - 24);
    return best / ulp;
}

// The block-wide sum used by every kernel on this path (engine/kernels.cu:1507-1520, 1590-1602,
// 1736-1748): per warp a __shfl_down tree with offsets 16,8,4,2,1 (lane 0 keeps the result), then the
// four warp partials are summed by the same tree in warp 0 with lanes >= 4 holding 0, which reduces to
// (p0+p2)+(p1+p3).  a[] has 128 entries and is clobbered.
inline float block_sum128(float* a) {
    float p[4];
    for (int w = 0; w < 4; ++w) {
        float* x = a + 32 * w;
        for (int off = 16; off > 0; off >>= 1)
            for (int i = 0; i < off; ++i) x[i] = x[i] + x[i + off];
        p[w] = x[0];
    }
    return (p[0] + p[2]) + (p[1] + p[3]);
}

struct Geometry {
    int vpb, bph, kvp;
};
inline Geometry geometry(int bits, int head_dim, int kv_dim) {
    Geometry g;
    g.vpb = (bits == 2) ? 4 : 2;  // engine/kernels.cu:1496 -- anything that is not 2 is treated as 4-bit here,
    g.bph = head_dim / g.vpb;     // while quantize() treats anything that is not 4 as 2-bit (:1449, :1471)
    g.kvp = kv_dim / g.vpb;
    return g;
}

// One head vector: engine/kernels.cu:1503-1559.  x = 128 fp16 values, R = 128x128 fp16 row-major.
// Writes bph code bytes and one fp16 norm; optionally the 128 rotated fp32 coordinates.
void append_one(const uint16_t* x, const uint16_t* R, int bits, int head_dim, uint8_t* dst_codes,
                uint16_t* dst_norm, float* rot_out) {
    float v[128], sq[128], xh[128];
    uint8_t code[128];
    for (int d = 0; d < head_dim; ++d) {
        v[d] = h2f(x[d]);
        sq[d] = v[d] * v[d];
    }
    for (int d = head_dim; d < 128; ++d) sq[d] = 0.0f;
    float ss = block_sum128(sq);
    float t = ss + 1e-12f;
    float inv = (float)(1.0 / std::sqrt((double)t));  // reference: rsqrtf -> rsqrt.approx.ftz
    for (int d = 0; d < head_dim; ++d) xh[d] = v[d] * inv;
    for (int d = 0; d < head_dim; ++d) {
        const uint16_t* row = R + (size_t)d * head_dim;
        float r = 0.0f;
        for (int k = 0; k < head_dim; ++k) r = std::fmaf(h2f(row[k]), xh[k], r);
        if (rot_out) rot_out[d] = r;
        code[d] = (uint8_t)quantize(r, bits);
    }
    int vpb = (bits == 2) ? 4 : 2;
    int bph = head_dim / vpb;
    for (int b = 0; b < bph; ++b) {
        uint8_t packed;
        if (bits == 2) {
            packed = (uint8_t)(code[4 * b] | (code[4 * b + 1] << 2) | (code[4 * b + 2] << 4) | (code[4 * b + 3] << 6));
        } else {
            packed = (uint8_t)(code[2 * b] | (code[2 * b + 1] << 4));
        }
        dst_codes[b] = packed;
    }
    *dst_norm = f2h(std::sqrt(t));  // reference: sqrtf -> sqrt.approx.ftz, then __float2half
}

// One (sequence, query head): engine/kernels.cu:1662-1775.  `row0` is the first cache row of the
// sequence (g*max_seq_len in the batched kernel, 0 in the single-sequence one); `last` is the last
// position attended to (positions[g]; the prefill kernel passes the query's own index).
void attend_one(const uint16_t* q, const uint8_t* ck, const uint8_t* cv, const uint16_t* kn, const uint16_t* vn,
                const uint16_t* R, size_t row0, int last, int kv_head, int num_kv_heads, int head_dim, int kv_dim,
                int bits, uint16_t* out_h, float* out_f) {
    Geometry geo = geometry(bits, head_dim, kv_dim);
    const int D = head_dim;
    const float scale = (float)(1.0 / std::sqrt((double)D));  // reference: rsqrtf((float)head_dim)
    float qraw[128], qrot[128];
    for (int d = 0; d < D; ++d) qraw[d] = h2f(q[d]);
    for (int d = 0; d < D; ++d) {  // phase 1, :1676-1680
        float r = 0.0f;
        const uint16_t* row = R + (size_t)d * D;
        for (int k = 0; k < D; ++k) r = std::fmaf(h2f(row[k]), qraw[k], r);
        qrot[d] = r;
    }
    const int L = last + 1;
    std::vector<float> s((size_t)L);
    float tmax[128];
    for (int d = 0; d < 128; ++d) tmax[d] = -1e30f;
    for (int p = 0; p < L; ++p) {  // phase 2, :1688-1710 (thread d owns p = d, d+128, ...)
        size_t row = row0 + (size_t)p;
        float knorm = h2f(kn[row * num_kv_heads + kv_head]);
        const uint8_t* kb = ck + row * geo.kvp + (size_t)kv_head * geo.bph;
        float dot = 0.0f;
        if (bits == 4) {
            for (int b = 0; b < geo.bph; ++b) {
                uint8_t pk = kb[b];
                dot = std::fmaf(qrot[2 * b + 0], CENT4[pk & 0xF], dot);
                dot = std::fmaf(qrot[2 * b + 1], CENT4[(pk >> 4) & 0xF], dot);
            }
        } else {
            for (int b = 0; b < geo.bph; ++b) {
                uint8_t pk = kb[b];
                dot = std::fmaf(qrot[4 * b + 0], CENT2[(pk)&3], dot);
                dot = std::fmaf(qrot[4 * b + 1], CENT2[(pk >> 2) & 3], dot);
                dot = std::fmaf(qrot[4 * b + 2], CENT2[(pk >> 4) & 3], dot);
                dot = std::fmaf(qrot[4 * b + 3], CENT2[(pk >> 6) & 3], dot);
            }
        }
        dot *= knorm * scale;
        s[p] = dot;
        tmax[p & 127] = std::fmax(tmax[p & 127], dot);
    }
    float m = -1e30f;
    for (int d = 0; d < 128; ++d) m = std::fmax(m, tmax[d]);  // max is order independent
    float part[128];
    for (int d = 0; d < 128; ++d) part[d] = 0.0f;
    for (int p = 0; p < L; ++p) {  // :1730-1734, thread-strided partial sums, p ascending per thread
        float e = std::exp(s[p] - m);  // reference: expf -> ex2.approx path
        s[p] = e;
        part[p & 127] += e;
    }
    float Z = block_sum128(part);
    float inv_sum = 1.0f / (Z + 1e-8f);
    for (int p = 0; p < L; ++p) s[p] *= inv_sum;
    float acc[128];
    for (int c = 0; c < D; ++c) acc[c] = 0.0f;
    for (int p = 0; p < L; ++p) {  // phase 3, :1759-1766, p ascending
        size_t row = row0 + (size_t)p;
        float w = s[p] * h2f(vn[row * num_kv_heads + kv_head]);
        const uint8_t* vb = cv + row * geo.kvp + (size_t)kv_head * geo.bph;
        if (bits == 4) {
            for (int b = 0; b < geo.bph; ++b) {
                uint8_t pk = vb[b];
                acc[2 * b + 0] = std::fmaf(w, CENT4[pk & 0xF], acc[2 * b + 0]);
                acc[2 * b + 1] = std::fmaf(w, CENT4[(pk >> 4) & 0xF], acc[2 * b + 1]);
            }
        } else {
            for (int b = 0; b < geo.bph; ++b) {
                uint8_t pk = vb[b];
                for (int j = 0; j < 4; ++j)
                    acc[4 * b + j] = std::fmaf(w, CENT2[(pk >> (2 * j)) & 3], acc[4 * b + j]);
            }
        }
    }
    for (int d = 0; d < D; ++d) {  // phase 4, :1768-1775: out = R^T acc
        float o = 0.0f;
        for (int k = 0; k < D; ++k) o = std::fmaf(h2f(R[(size_t)k * D + d]), acc[k], o);
        if (out_f) out_f[d] = o;
        if (out_h) out_h[d] = f2h(o);
    }
}

// fp16 twin, one (sequence, query head): engine/kernels.cu:995-1065 and :266-344.
void attend_one_fp16(const uint16_t* q, const uint16_t* ck, const uint16_t* cv, size_t row0, int last, int kv_head,
                     int head_dim, int kv_dim, uint16_t* out_h, float* out_f) {
    const int D = head_dim;
    const float scale = (float)(1.0 / std::sqrt((double)D));
    const int L = last + 1;
    float qf[128];
    for (int d = 0; d < D; ++d) qf[d] = h2f(q[d]);
    std::vector<float> s((size_t)L);
    float m = -1e30f;
    for (int p = 0; p < L; ++p) {
        const uint16_t* kp = ck + (row0 + (size_t)p) * kv_dim + (size_t)kv_head * D;
        float dot = 0.0f;
        for (int d = 0; d < D; ++d) dot = std::fmaf(qf[d], h2f(kp[d]), dot);
        dot *= scale;
        s[p] = dot;
        m = std::fmax(m, dot);
    }
    float part[128];
    for (int d = 0; d < 128; ++d) part[d] = 0.0f;
    for (int p = 0; p < L; ++p) {
        float e = std::exp(s[p] - m);
        s[p] = e;
        part[p & 127] += e;
    }
    float Z = block_sum128(part);
    float inv_sum = 1.0f / (Z + 1e-8f);
    for (int p = 0; p < L; ++p) s[p] *= inv_sum;
    float acc[128];
    for (int d = 0; d < D; ++d) acc[d] = 0.0f;
    for (int p = 0; p < L; ++p) {
        const uint16_t* vp = cv + (row0 + (size_t)p) * kv_dim + (size_t)kv_head * D;
        for (int d = 0; d < D; ++d) acc[d] = std::fmaf(s[p], h2f(vp[d]), acc[d]);
    }
    for (int d = 0; d < D; ++d) {
        if (out_f) out_f[d] = acc[d];
        if (out_h) out_h[d] = f2h(acc[d]);
    }
}

}  // namespace

extern "C" {

int tqo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void tqo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

uint16_t tqo_float_to_half(float f) { return f2h(f); }
float tqo_half_to_float(uint16_t h) { return h2f(h); }
int tqo_quantize(float v, int bits) { return quantize(v, bits); }
float tqo_centroid(int idx, int bits) { return centroid(idx, bits); }
float tqo_ulps_to_bound(float v, int bits) { return ulps_to_bound(v, bits); }

// copies the tables out: cent[16] / bounds[15] (4-bit) or cent[4] / bounds[3] (2-bit)
void tqo_tables(int bits, float* cent, float* bounds) {
    if (bits == 4) {
        std::memcpy(cent, CENT4, sizeof(CENT4));
        std::memcpy(bounds, BND4, sizeof(BND4));
    } else {
        std::memcpy(cent, CENT2, sizeof(CENT2));
        std::memcpy(bounds, BND2, sizeof(BND2));
    }
}

// engine/engine.cpp:364-392: mt19937(seed) -> N(0,1) 128x128 row-major -> row-wise modified Gram-Schmidt
// in fp32 (projections subtracted one earlier row at a time) -> 1/sqrtf normalisation -> fp16 (RNE).
// The reference seeds with 42.  Built with -ffp-contract=off this reproduces the bytes an x86-64 build of
// the reference makes; a build that contracts a*b+c into FMA makes different low bits, so callers must
// pass the SAME R bytes to every implementation they compare.
void tqo_rotation_generate(uint32_t seed, int d, uint16_t* out_half, float* out_f32) {
    std::mt19937 gen(seed);
    std::normal_distribution<float> dist(0.0f, 1.0f);
    std::vector<float> mat((size_t)d * d);
    for (int i = 0; i < d * d; ++i) mat[i] = dist(gen);
    for (int i = 0; i < d; ++i) {
        for (int j = 0; j < i; ++j) {
            float dot = 0;
            for (int k = 0; k < d; ++k) dot += mat[i * d + k] * mat[j * d + k];
            for (int k = 0; k < d; ++k) mat[i * d + k] -= dot * mat[j * d + k];
        }
        float norm = 0;
        for (int k = 0; k < d; ++k) norm += mat[i * d + k] * mat[i * d + k];
        norm = 1.0f / std::sqrt(norm);
        for (int k = 0; k < d; ++k) mat[i * d + k] *= norm;
    }
    for (int i = 0; i < d * d; ++i) {
        if (out_half) out_half[i] = f2h(mat[i]);
        if (out_f32) out_f32[i] = mat[i];
    }
}

// Batched decode append, engine/kernels.cu:1563-1636: one new token per sequence g, written at row
// g*max_seq_len + positions[g].  kv_buf is [G][kv_dim] fp16.  rot_out (optional) is [G][Hkv][head_dim].
void tqo_append_batch(uint8_t* cache_q, uint16_t* cache_norms, const uint16_t* kv_buf, const uint16_t* R,
                      const int* positions, int max_seq_len, int G, int num_kv_heads, int head_dim, int kv_dim,
                      int bits, float* rot_out) {
    Geometry geo = geometry(bits, head_dim, kv_dim);
#pragma omp parallel for collapse(2) schedule(static)
    for (int g = 0; g < G; ++g) {
        for (int h = 0; h < num_kv_heads; ++h) {
            size_t row = (size_t)g * max_seq_len + (size_t)positions[g];
            append_one(kv_buf + (size_t)g * kv_dim + (size_t)h * head_dim, R, bits, head_dim,
                       cache_q + row * geo.kvp + (size_t)h * geo.bph, cache_norms + row * num_kv_heads + h,
                       rot_out ? rot_out + ((size_t)g * num_kv_heads + h) * head_dim : nullptr);
        }
    }
}

// Token-form append (prefill / single sequence), engine/kernels.cu:1482-1560: token t of kv_buf
// [num_tokens][kv_dim] goes to row positions[t] of a single-sequence cache.
void tqo_append_tokens(uint8_t* cache_q, uint16_t* cache_norms, const uint16_t* kv_buf, const uint16_t* R,
                       const int* positions, int max_seq_len, int num_tokens, int num_kv_heads, int head_dim,
                       int kv_dim, int bits, float* rot_out) {
    (void)max_seq_len;
    Geometry geo = geometry(bits, head_dim, kv_dim);
#pragma omp parallel for collapse(2) schedule(static)
    for (int t = 0; t < num_tokens; ++t) {
        for (int h = 0; h < num_kv_heads; ++h) {
            size_t row = (size_t)positions[t];
            append_one(kv_buf + (size_t)t * kv_dim + (size_t)h * head_dim, R, bits, head_dim,
                       cache_q + row * geo.kvp + (size_t)h * geo.bph, cache_norms + row * num_kv_heads + h,
                       rot_out ? rot_out + ((size_t)t * num_kv_heads + h) * head_dim : nullptr);
        }
    }
}

// Batched decode attention, engine/kernels.cu:1641-1776.  q/out are [G][q_dim] fp16 (head h at h*head_dim).
// out_f32 (optional, [G][num_heads][head_dim]) receives the values before the final fp16 rounding.
void tqo_attention_batch(uint16_t* out, float* out_f32, const uint16_t* q, const uint8_t* ck, const uint8_t* cv,
                         const uint16_t* kn, const uint16_t* vn, const uint16_t* R, const int* positions,
                         int max_seq_len, int G, int num_heads, int num_kv_heads, int head_dim, int q_dim,
                         int kv_dim, int bits) {
    int groups = num_heads / num_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int g = 0; g < G; ++g) {
        for (int h = 0; h < num_heads; ++h) {
            attend_one(q + (size_t)g * q_dim + (size_t)h * head_dim, ck, cv, kn, vn, R, (size_t)g * max_seq_len,
                       positions[g], h / groups, num_kv_heads, head_dim, kv_dim, bits,
                       out ? out + (size_t)g * q_dim + (size_t)h * head_dim : nullptr,
                       out_f32 ? out_f32 + ((size_t)g * num_heads + h) * head_dim : nullptr);
        }
    }
}

// Single-sequence decode attention, engine/kernels.cu:1779-1870 (pos by value, q/out are [num_heads*head_dim]).
void tqo_attention_single(uint16_t* out, float* out_f32, const uint16_t* q, const uint8_t* ck, const uint8_t* cv,
                          const uint16_t* kn, const uint16_t* vn, const uint16_t* R, int pos, int max_seq_len,
                          int num_heads, int num_kv_heads, int head_dim, int bits) {
    (void)max_seq_len;
    int groups = num_heads / num_kv_heads;
    int kv_dim = num_kv_heads * head_dim;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < num_heads; ++h) {
        attend_one(q + (size_t)h * head_dim, ck, cv, kn, vn, R, 0, pos, h / groups, num_kv_heads, head_dim, kv_dim,
                   bits, out ? out + (size_t)h * head_dim : nullptr,
                   out_f32 ? out_f32 + (size_t)h * head_dim : nullptr);
    }
}

// Causal prefill attention over a single-sequence packed cache, engine/kernels.cu:1874-1960: query tq
// (row tq of q [T][q_dim]) attends to positions 0..tq.
void tqo_prefill_attention(uint16_t* out, float* out_f32, const uint16_t* q, const uint8_t* ck, const uint8_t* cv,
                           const uint16_t* kn, const uint16_t* vn, const uint16_t* R, int T, int max_seq_len,
                           int num_heads, int num_kv_heads, int head_dim, int q_dim, int kv_dim, int bits) {
    (void)max_seq_len;
    int groups = num_heads / num_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int tq = 0; tq < T; ++tq) {
        for (int h = 0; h < num_heads; ++h) {
            attend_one(q + (size_t)tq * q_dim + (size_t)h * head_dim, ck, cv, kn, vn, R, 0, tq, h / groups,
                       num_kv_heads, head_dim, kv_dim, bits,
                       out ? out + (size_t)tq * q_dim + (size_t)h * head_dim : nullptr,
                       out_f32 ? out_f32 + ((size_t)tq * num_heads + h) * head_dim : nullptr);
        }
    }
}

// kv_bits = 0 cache write, engine/kernels.cu:964-977.
// The producer of the step's q and k (engine/engine.cpp:1972-1977): per-head RMS norm with a weight vector
// (qk_norm_batch_kernel, engine/kernels.cu:880-923) and rotary embedding (rope_batch_kernel, :926-962), both in place
// on fp16 [G][dim] buffers, each rounding its results to fp16.  Arithmetic as the reference's build evaluates it:
// one head per 128-thread block, sum of squares by the block tree above, `s / head_dim + eps` (the division by 128
// is exact), rsqrtf (IEEE here, rsqrt.approx there: results may differ in the last fp16 bit), (x * rms) * w;
// rotary pairs (d, d + rope_dim/2) with x0*c - x1*s evaluated as fma(x0, c, -(x1*s)) and x0*s + x1*c as
// fma(x0, s, x1*c) (how the reference's -fmad=true build contracts the two expressions).
static void qk_norm_one(uint16_t* data, const uint16_t* w, int head_dim, float eps, int biased) {
    float sq[128], v[128];
    for (int d = 0; d < 128; ++d) {
        v[d] = d < head_dim ? h2f(data[d]) : 0.0f;
        sq[d] = v[d] * v[d];
    }
    const float ss = block_sum128(sq);
    const float rms = (float)(1.0 / std::sqrt((double)(ss / (float)head_dim + eps)));
    for (int d = 0; d < head_dim; ++d) {
        float wv = h2f(w[d]);
        if (biased) wv += 1.0f;
        data[d] = f2h((v[d] * rms) * wv);
    }
}
static void rope_one(uint16_t* x, const uint16_t* cos_row, const uint16_t* sin_row, int half_rope) {
    for (int d = 0; d < half_rope; ++d) {
        const float c = h2f(cos_row[d]), sv = h2f(sin_row[d]);
        const float x0 = h2f(x[d]), x1 = h2f(x[d + half_rope]);
        x[d] = f2h(std::fmaf(x0, c, -(x1 * sv)));
        x[d + half_rope] = f2h(std::fmaf(x0, sv, x1 * c));
    }
}
void tqo_qk_norm_rope_batch(uint16_t* q, uint16_t* k, const uint16_t* q_w, const uint16_t* k_w, const uint16_t* cos_table,
                            const uint16_t* sin_table, const int* positions, int G, int num_heads, int num_kv_heads,
                            int head_dim, int q_dim, int kv_dim, int rope_dim, float eps, int biased) {
    const int half_rope = rope_dim / 2;
#pragma omp parallel for schedule(static)
    for (int g = 0; g < G; ++g) {
        const int pos = positions[g];
        for (int h = 0; h < num_heads; ++h) {
            uint16_t* x = q + (size_t)g * q_dim + (size_t)h * head_dim;
            qk_norm_one(x, q_w, head_dim, eps, biased);
            rope_one(x, cos_table + (size_t)pos * half_rope, sin_table + (size_t)pos * half_rope, half_rope);
        }
        for (int h = 0; h < num_kv_heads; ++h) {
            uint16_t* x = k + (size_t)g * kv_dim + (size_t)h * head_dim;
            qk_norm_one(x, k_w, head_dim, eps, biased);
            rope_one(x, cos_table + (size_t)pos * half_rope, sin_table + (size_t)pos * half_rope, half_rope);
        }
    }
}

void tqo_fp16_write_batch(uint16_t* cache_k, uint16_t* cache_v, const uint16_t* k, const uint16_t* v,
                          const int* positions, int max_seq_len, int G, int kv_dim) {
    for (int g = 0; g < G; ++g) {
        size_t dst = ((size_t)g * max_seq_len + (size_t)positions[g]) * kv_dim;
        std::memcpy(cache_k + dst, k + (size_t)g * kv_dim, (size_t)kv_dim * 2);
        std::memcpy(cache_v + dst, v + (size_t)g * kv_dim, (size_t)kv_dim * 2);
    }
}

// kv_bits = 0 batched decode attention, engine/kernels.cu:981-1066.
void tqo_fp16_attention_batch(uint16_t* out, float* out_f32, const uint16_t* q, const uint16_t* ck,
                              const uint16_t* cv, const int* positions, int max_seq_len, int G, int num_heads,
                              int num_kv_heads, int head_dim, int q_dim, int kv_dim) {
    int groups = num_heads / num_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int g = 0; g < G; ++g) {
        for (int h = 0; h < num_heads; ++h) {
            attend_one_fp16(q + (size_t)g * q_dim + (size_t)h * head_dim, ck, cv, (size_t)g * max_seq_len,
                            positions[g], h / groups, head_dim, kv_dim,
                            out ? out + (size_t)g * q_dim + (size_t)h * head_dim : nullptr,
                            out_f32 ? out_f32 + ((size_t)g * num_heads + h) * head_dim : nullptr);
        }
    }
}

// kv_bits = 0 single-sequence decode attention, engine/kernels.cu:244-345 (1/sqrtf scale there; same value).
void tqo_fp16_attention_single(uint16_t* out, float* out_f32, const uint16_t* q, const uint16_t* ck,
                               const uint16_t* cv, int pos, int max_seq_len, int num_heads, int num_kv_heads,
                               int head_dim) {
    (void)max_seq_len;
    int groups = num_heads / num_kv_heads;
    int kv_dim = num_kv_heads * head_dim;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < num_heads; ++h) {
        attend_one_fp16(q + (size_t)h * head_dim, ck, cv, 0, pos, h / groups, head_dim, kv_dim,
                        out ? out + (size_t)h * head_dim : nullptr,
                        out_f32 ? out_f32 + (size_t)h * head_dim : nullptr);
    }
}

}  // extern "C"
