/* triebwerk_b200 -- C ABI of the B200 (sm_100a) TurboQuant KV-cache hot path.
 *
 * Two layers, both plain C (pointers and sizes only; no torch, no C++ types):
 *
 *  1. The reference's own launcher symbols (BY571/triebwerk, engine/kernels.cu, all inside its
 *     extern "C" block) with identical parameter lists, so that the reference's engine.cpp links against
 *     this library instead of its own kernels for this path.  Every pointer is a DEVICE pointer owned by
 *     the caller; calls are asynchronous on the given stream and return nothing, like the reference's.
 *
 *  2. The native tq_* entry points: the same operations with explicit workspaces, fused launches and an
 *     int status (0 = ok, <0 = argument/capacity error, >0 = CUDA error code), plus the KV arena
 *     (sizing, slot table, reset, sleep/wake, external memory) that the reference keeps inside
 *     InferenceEngine (engine/engine.cpp:1338-1560, 1609-1620, 893-1022).
 *
 * Where a declaration below replaces a reference interface, the comment cites it as file:line inside the
 * reference project.  `half` data crosses as void* / uint16 bits; the cache byte layout is the reference's
 * (engine/kernels.cu:1618-1635): codes [row][kv_dim/vpb] uint8, norms [row][num_kv_heads] fp16, row =
 * g*max_seq_len + position.  head_dim must be 128.  kv_bits is 0 (fp16 cache), 2 or 4.
 */
#ifndef TRIEBWERK_B200_H_
#define TRIEBWERK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* An opaque CUDA stream handle (cudaStream_t).  NULL is the legacy default stream, as in the reference's
 * single-sequence path. */
typedef struct CUstream_st* tq_stream_t;

/* ---- status codes of the tq_* entry points ------------------------------------------------------------------ */
enum {
    TQ_OK = 0,
    TQ_ERR_ARG = -1,         /* null pointer, bad kv_bits, head_dim != 128, heads not divisible ... */
    TQ_ERR_CAPACITY = -2,    /* position / sequence count beyond what was reserved */
    TQ_ERR_WORKSPACE = -3,   /* workspace missing or too small */
    TQ_ERR_UNSUPPORTED = -4, /* shape outside what the kernels are built for */
    TQ_ERR_STATE = -5,       /* engine asleep, arena not set ... */
    TQ_ERR_DEVICE = -6,      /* a kernel reported a device-side status (bounded wait ran out) */
    TQ_ERR_NOMEM = -7
};

const char* tq_status_string(int status);
/* Library version as major*10000 + minor*100 + patch. */
int tq_version(void);

/* ===================================================================================================================
 * 1. Reference-compatible launchers.
 *
 * Differences a caller can observe: `as` / `attn_scratch` (the reference's fp32 score buffer,
 * engine/engine.cpp:1371,1467) is accepted and ignored -- scores never leave the SM; a small per-device
 * workspace (pre-rotated queries, split-K partials) is allocated inside the library the first time a
 * launcher needs it and when a later call needs a larger one, so the first call of a given size must come
 * before any stream capture (the reference warms up before it captures, engine/engine.cpp:2369-2387).
 * Errors cannot be returned through these signatures; they are kept for tq_last_compat_status().
 * =================================================================================================================== */

/* engine/kernels.cu:1963-1973 (kernel :1482-1560).  Token-form append into a single-sequence cache:
 * token t of kv_buf [num_tokens][kv_dim] goes to row positions[t]. */
void launch_turbo_kv_quantize(uint8_t* cache_q, void* cache_norms, const void* kv_buf, const void* rotation,
                              const int* positions, int max_seq_len, int num_tokens, int num_kv_heads,
                              int head_dim, int kv_dim, int bits, tq_stream_t s);

/* engine/kernels.cu:1975-1984 (kernel :1563-1636).  One new token per sequence g at row
 * g*max_seq_len + positions[g]; kv_buf is [G][kv_dim]. */
void launch_turbo_kv_quantize_batch(uint8_t* cache_q, void* cache_norms, const void* kv_buf,
                                    const void* rotation, const int* positions, int max_seq_len, int G,
                                    int num_kv_heads, int head_dim, int kv_dim, int bits, tq_stream_t s);

/* engine/kernels.cu:1986-1999 (kernel :1641-1776).  Batched GQA decode attention over the packed cache,
 * positions 0..positions[g] inclusive; q and out are [G][q_dim]. */
void launch_turbo_gqa_attention_batch(void* out, const void* q, const uint8_t* ck_q, const uint8_t* cv_q,
                                      const void* k_norms, const void* v_norms, const void* rotation,
                                      float* as, const int* pos, int msl, int G, int num_heads,
                                      int num_kv_heads, int head_dim, int q_dim, int kv_dim, int bits,
                                      tq_stream_t s);

/* engine/kernels.cu:2001-2013 (kernel :1779-1870).  Single-sequence form, `pos` by value. */
void launch_turbo_gqa_attention(const void* q, const uint8_t* ck_q, const uint8_t* cv_q, const void* k_norms,
                                const void* v_norms, const void* rotation, void* output, float* as, int pos,
                                int msl, int num_heads, int num_kv_heads, int head_dim, int bits,
                                tq_stream_t s);

/* engine/kernels.cu:2015-2028 (kernel :1874-1960).  Causal prefill attention over a single-sequence
 * packed cache: query row tq of q [T][q_dim] attends to positions 0..tq.  Served by a kernel that holds 128 / (heads
 * per KV head) query tokens in the M dimension of the tensor-core products and dequantises every 64-row cache tile once
 * per block, in one launch and without any workspace (the query rotation and the way back through R^T are tensor-core
 * products inside it); `as` (the reference's [T][heads][T] score scratch) is accepted and ignored. */
void launch_turbo_gqa_prefill_attention(void* out, const void* q, const uint8_t* ck_q, const uint8_t* cv_q,
                                        const void* k_norms, const void* v_norms, const void* rotation,
                                        float* as, int T, int msl, int num_heads, int num_kv_heads,
                                        int head_dim, int q_dim, int kv_dim, int bits, tq_stream_t s);

/* engine/kernels.cu:1351-1353 (kernel :964-977).  kv_bits = 0 cache write. */
void launch_kv_cache_write_batch(void* ck, void* cv, const void* k, const void* v, const int* pos, int msl,
                                 int G, int kv_dim, tq_stream_t s);

/* engine/kernels.cu:1354-1357 (kernel :981-1066).  kv_bits = 0 batched decode attention. */
void launch_gqa_attention_batch(void* out, const void* q, const void* ck, const void* cv, float* as,
                                const int* pos, int msl, int G, int num_heads, int num_kv_heads, int head_dim,
                                int q_dim, int kv_dim, tq_stream_t s);

/* engine/kernels.cu:737-752 (kernel :244-345).  kv_bits = 0 single-sequence decode attention. */
void launch_gqa_attention(const void* q, const void* k_cache, const void* v_cache, void* output,
                          float* attn_scratch, int pos, int max_seq_len, int num_heads, int num_kv_heads,
                          int head_dim, tq_stream_t stream);
/* engine/kernels.cu:1071-1158, 1359-1362: causal prefill attention over the fp16 cache of ONE sequence; query token t
 * ([T][q_dim]) attends to rows 0 .. t.  `as` (the reference's [T][heads][T] score scratch) is accepted and ignored. */
void launch_gqa_prefill_attention(void* out, const void* q, const void* ck, const void* cv, float* as, int T, int msl,
                                  int num_heads, int num_kv_heads, int head_dim, int q_dim, int kv_dim, tq_stream_t s);

/* Status of the most recent compat launcher call on this host thread (TQ_OK or an error above). */
int tq_last_compat_status(void);

/* ===================================================================================================================
 * 2. Native entry points.
 * =================================================================================================================== */

/* Rotation matrix of the reference (engine/engine.cpp:364-392): mt19937(seed) normal fill, row-wise
 * modified Gram-Schmidt in fp32, fp16 rounding.  host_out receives 128*128 fp16 values (32 KB, HOST
 * memory).  The reference uses seed 42. */
int tq_rotation_generate(uint32_t seed, void* host_out_half);

/* Bytes of device workspace tq_decode_attention / tq_append_decode need for G sequences and num_heads
 * query heads on the current device (pre-rotated queries, tile table, split-K partials, tickets). */
size_t tq_workspace_bytes(int G, int num_heads);

/* Fused decode-step append (replaces the two launch_turbo_kv_quantize_batch calls of
 * engine/engine.cpp:1985-1990 and phase 1 of the attention kernel, engine/kernels.cu:1676-1680): for every
 * sequence g, quantise k_buf[g] into the K cache and v_buf[g] into the V cache at row
 * row(g) + positions[g], and rotate q[g] into the workspace for tq_decode_attention.  Any of
 * {k_buf, v_buf, q} may be NULL to skip that part.  kv_bits must be 2 or 4 here.
 * row(g) = g*max_seq_len, or row_base[g] when row_base (device, int64[G]) is not NULL. */
int tq_append_decode(uint8_t* ck_q, void* k_norms, uint8_t* cv_q, void* v_norms, const void* k_buf,
                     const void* v_buf, const void* q, const void* rotation, const int* positions,
                     const long long* row_base, int max_seq_len, int G, int num_heads, int num_kv_heads,
                     int head_dim, int q_dim, int kv_dim, int bits, void* workspace, size_t workspace_bytes,
                     tq_stream_t s);

/* Split-K GQA decode attention over the packed cache (replaces launch_turbo_gqa_attention_batch,
 * engine/kernels.cu:1986-1999).  Reads the queries that tq_append_decode rotated into `workspace` on the
 * same stream.  total_rows is the number of rows of the cache arrays (G*max_seq_len for the dense layout).
 * positions may be NULL when pos_value >= 0 gives one position for every sequence. */
int tq_decode_attention(void* out, const uint8_t* ck_q, const uint8_t* cv_q, const void* k_norms,
                        const void* v_norms, const void* rotation, const int* positions, int pos_value,
                        const long long* row_base, long long total_rows, int max_seq_len, int G, int num_heads,
                        int num_kv_heads, int head_dim, int q_dim, int kv_dim, int bits, void* workspace,
                        size_t workspace_bytes, tq_stream_t s);

/* No counterpart in the reference.  Decode attention over the packed cache for callers that cannot allocate device
 * memory once they are running: processes whose memory pool already owns the whole GPU (a raw cudaMalloc would fail or
 * fight that pool) and serving loops that forbid cudaMalloc because it synchronises the device.  Same result as
 * launch_turbo_gqa_attention_batch (it takes the un-rotated queries q [G][q_dim]), but the kernel's scratch (rotated
 * queries, tile table, tickets, split-K partials, transposed rotation) lives in a fixed 20 MiB device array inside the
 * library image, present on every GPU that loads the library until the process exits.  The call makes no cudaMalloc /
 * cudaFree and uses no allocator of any framework.
 *   Limit: tq_workspace_bytes(G, num_heads) must not exceed 20 MiB -- that covers 64 sequences x 32 query heads or
 *   256 x 16; larger requests return TQ_ERR_CAPACITY and launch nothing.  Arguments are checked before anything is
 *   enqueued: a refused call leaves the stream untouched.
 *   The first call on a device looks the array's address up (cudaGetSymbolAddress), once.  All calls share the one
 *   array and it keeps the previous call's contents (the call itself clears what
 *   must start at zero): two calls that overlap on the GPU -- different streams, or work replayed concurrently --
 *   race on it and must be serialised by the caller.
 *   Device-side trouble (a bounded wait that gave up = 1, a shared-memory layout refused = 2) is collected in a status
 *   word inside the array; tq_static_status reads and clears it (0 = fine) and synchronises the stream. */
int tq_decode_attention_static(void* out, const void* q, const uint8_t* ck_q, const uint8_t* cv_q,
                               const void* k_norms, const void* v_norms, const void* rotation,
                               const int* positions, long long total_rows, int max_seq_len, int G, int num_heads,
                               int num_kv_heads, int head_dim, int q_dim, int kv_dim, int bits, tq_stream_t s);
int tq_static_status(tq_stream_t s);

/* kv_bits = 0 twins with the same slot addressing (replace launch_kv_cache_write_batch and
 * launch_gqa_attention_batch, engine/kernels.cu:1351-1357). */
int tq_fp16_append_decode(void* ck, void* cv, const void* k_buf, const void* v_buf, const int* positions,
                          const long long* row_base, int max_seq_len, int G, int kv_dim, tq_stream_t s);
int tq_fp16_decode_attention(void* out, const void* q, const void* ck, const void* cv, const int* positions,
                             int pos_value, const long long* row_base, long long total_rows, int max_seq_len,
                             int G, int num_heads, int num_kv_heads, int head_dim, int q_dim, int kv_dim,
                             void* workspace, size_t workspace_bytes, tq_stream_t s);

/* Reads (and clears) the device status word kept in `workspace`: 0, or a code saying which bounded wait
 * gave up.  Synchronises the stream. */
int tq_workspace_status(void* workspace, tq_stream_t s);

/* Self-test of the bounded waits (no counterpart in the reference, whose kernels have no asynchronous copies): runs a
 * one-warp kernel that arms a copy barrier for bytes nobody sends and waits for them with at most `limit` polls
 * (1 .. 2^20).  The wait gives up, the kernel records status 1 in the int at `status_word` (device memory, zero
 * before the call) and exits normally; the call returns that word (1 expected) after clearing it.  Nothing traps or
 * spins without bound. */
int tq_selftest_bounded_wait(void* status_word, unsigned limit, tq_stream_t s);

/* ---- KV arena / engine state ----------------------------------------------------------------------------------------
 * The part of InferenceEngine that owns the cache: constructor arguments (engine/engine.cpp:300-317),
 * KV_DIM_PACKED (:292-294), alloc_batch sizing and carving (:1338-1560), set_arena (:1609-1620), reset
 * (:893-916), sleep / wake (:922-1022) and the per-layer call sites (:1979-2006).  One handle per device. */
typedef struct tq_engine tq_engine;

typedef struct tq_model_shape {
    int num_layers;   /* attention layers that own a KV cache */
    int num_heads;    /* query heads */
    int num_kv_heads; /* KV heads */
    int head_dim;     /* must be 128 */
} tq_model_shape;

/* Like Engine(max_seq_len, kv_bits): an unsupported kv_bits falls back to 0 with a warning on stderr
 * (engine/engine.cpp:310-313).  Allocates nothing on the device yet. */
int tq_engine_create(const tq_model_shape* shape, int max_seq_len, int kv_bits, tq_engine** out);
void tq_engine_destroy(tq_engine* e);
int tq_engine_kv_bits(const tq_engine* e);

/* Packed modes: choose between ONE launch per layer and step (on = 1, the default: the attention kernel also appends
 * the new token and rotates the queries) and the two-launch form (on = 0: append kernel, then attention kernel).
 * Both store identical bytes.  Returns the previous setting, or a negative status.  The environment variable
 * TQ_FUSED=0 makes the two-launch form the default of new engines.  No counterpart in the reference. */
int tq_engine_set_fused(tq_engine* e, int on);

/* Bytes of arena needed for G sequences.  capacities == NULL: dense slots of max_seq_len rows each (the
 * reference's layout, row(g) = g*max_seq_len).  Otherwise sequence g gets capacities[g] rows (rounded up
 * to 32) and row(g) is the running sum. */
size_t tq_engine_arena_bytes(const tq_engine* e, int G, int max_seq_len, const int* capacities);

/* Use caller-owned device memory as the arena (Engine.set_arena, engine/engine.cpp:1609-1620).  The
 * library never frees it. */
int tq_engine_set_arena(tq_engine* e, void* device_ptr, size_t bytes);

/* Reserve and carve the arena for a batch (alloc_batch, engine/engine.cpp:1338-1560).  Reuses the current
 * carving when it is large enough; grows an internally owned arena; fails with TQ_ERR_CAPACITY when an
 * external arena is too small.  Positions are set to 0. */
int tq_engine_alloc_batch(tq_engine* e, int G, int max_seq_len, const int* capacities);

/* Forget all sequences: positions = 0 (engine reset()).  With zero_cache != 0 also clears the cache
 * bytes as the reference does (engine/engine.cpp:2262-2283); attention never reads rows past a position,
 * so this is only needed by callers that inspect the raw cache. */
int tq_engine_reset(tq_engine* e, int zero_cache, tq_stream_t s);

/* Release (sleep) and re-create (wake) the internally owned arena; contents are not kept, as in the
 * reference (engine/engine.cpp:922-1022).  An external arena is detached by sleep and must be set again. */
int tq_engine_sleep(tq_engine* e);
int tq_engine_wake(tq_engine* e);

/* Cache persistence (the reference's sleep()/wake(), engine/engine.cpp:922-1022, drop the KV cache and the caller
 * has to prefill again; these calls keep it).
 * A sequence's written rows travel as a self-describing blob in the ON-CACHE byte layout: 8 int32 of header ("TQKV",
 * version, kv_bits, layers, kv heads, head_dim, tokens, 0), then per layer K codes [tokens][kvp], V codes, K norms
 * [tokens][kv heads] fp16, V norms (kv_bits = 0: K rows [tokens][kv_dim] fp16, V rows).  A blob can go to disk, to
 * another engine of the same shape or to another slot and back; nothing is re-quantised.
 *   tq_engine_sequence_blob_bytes: size of a blob of n_tokens rows.
 *   tq_engine_export_sequence: rows 0 .. n_tokens-1 of sequence `seq` into host memory; synchronises the stream.
 *   tq_engine_import_sequence: the blob's rows into slot `seq` (TQ_ERR_UNSUPPORTED for a blob of another shape or
 *     cache mode, TQ_ERR_CAPACITY if it does not fit the slot); the slot's position becomes the blob's token count,
 *     i.e. the next token is appended right behind the imported rows.
 *   tq_engine_sleep_keep: like tq_engine_sleep, but every sequence's rows 0 .. position-1 and the positions are kept in
 *     host memory; tq_engine_wake (library-owned arena) or the next tq_engine_alloc_batch of the same batch shape
 *     (caller-owned arena: after tq_engine_set_arena) puts them back, and decoding continues without a new prefill. */
size_t tq_engine_sequence_blob_bytes(const tq_engine* e, int n_tokens);
int tq_engine_export_sequence(tq_engine* e, int seq, int n_tokens, void* host_blob, size_t blob_bytes, tq_stream_t s);
int tq_engine_import_sequence(tq_engine* e, int seq, const void* host_blob, size_t blob_bytes, tq_stream_t s);
int tq_engine_sleep_keep(tq_engine* e);

/* Reads and clears the engine's device status word (0 = fine; 1 = a bounded wait on a TMA barrier gave up;
 * 2 = shared-memory layout refused; 3 = a position outside its slot).  Synchronises the stream. */
int tq_engine_status(tq_engine* e, tq_stream_t s);

/* Positions of the G sequences (device int32[G], advanced by the caller or by tq_engine_advance). */
int* tq_engine_positions(tq_engine* e);
int tq_engine_set_positions(tq_engine* e, const int* host_positions, int G, tq_stream_t s);
int tq_engine_advance(tq_engine* e, tq_stream_t s); /* positions[g] += 1 on the device */

/* Raw device pointers of one layer's cache (for tests and for callers that keep using the compat
 * launchers).  kv_bits != 0: k_codes/v_codes uint8, k_norms/v_norms fp16.  kv_bits == 0: k_codes/v_codes
 * are the fp16 K/V arrays and the norm pointers are NULL. */
int tq_engine_layer_ptrs(tq_engine* e, int layer, void** k_codes, void** v_codes, void** k_norms,
                         void** v_norms, long long* total_rows);
const long long* tq_engine_row_base(tq_engine* e); /* device int64[G], NULL for the dense layout */
const void* tq_engine_rotation(tq_engine* e);      /* device fp16 [128][128] */
int tq_engine_set_rotation(tq_engine* e, const void* host_half, tq_stream_t s);

/* One layer of a decode step on device buffers (steps 4-5 of forward_layer_batch,
 * engine/engine.cpp:1979-2006): append k/v at the current positions, then attend.  q/out [G][q_dim], k/v
 * [G][kv_dim], all fp16 on the device. */
int tq_engine_decode_layer(tq_engine* e, int layer, const void* q, const void* k, const void* v, void* out,
                           tq_stream_t s);

/* The attention over the current positions alone, on whatever rotated queries the engine's workspace holds (those
 * of the last two-launch tq_engine_decode_layer, zeros before; packed modes only).  Used to time the attention
 * kernel by itself. */
int tq_engine_attend_layer(tq_engine* e, int layer, void* out, tq_stream_t s);

/* tq_engine_attend_layer for every layer in turn: out [layers][G][q_dim] on the device. */
int tq_engine_attend_step(tq_engine* e, void* out, tq_stream_t s);

/* Every layer of a decode step on DEVICE buffers: q/out [layers][G][q_dim], k/v [layers][G][kv_dim]; the layers'
 * append + attention of forward_layer_batch (engine/engine.cpp:1979-2006) for callers that hold all layers' q/k/v
 * at once.  Packed modes run it as four launches whatever the number of layers (one append of every layer's new
 * token, one rotation of all queries, one attention launch that streams the layers back to back, one merge); set TQ_WHOLE_STEP=0 in the
 * environment to get one launch per layer instead. */
int tq_engine_decode_step(tq_engine* e, const void* q, const void* k, const void* v, void* out, tq_stream_t s);

/* The step's producer and consumer folded into it.  In the reference the projections' outputs pass through two more
 * kernels before the cache write -- per-head RMS norm with weights (launch_qk_norm_batch) and rotary embedding
 * (launch_rope_batch), engine/engine.cpp:1972-1977, kernels engine/kernels.cu:880-962 -- and the attention result
 * through R^T before o_proj (engine/engine.cpp:2015).  tq_engine_decode_step_produce takes the RAW projections q_raw
 * [layers][G][q_dim] and k_raw [layers][G][kv_dim]: norm and rotary embedding run inside the query rotation and inside
 * the append, with the reference's arithmetic and its roundings to fp16, so cache bytes and results are those of the
 * separate kernels followed by tq_engine_decode_step.  With rotated_output != 0 the results stay in rotated space
 * (out = normalised weighted V sums, no R^T): the consumer multiplies by weights that carry R^T, built once by
 * tq_fold_rotation_into_projection (w [rows][num_heads * 128] fp16, row-major: w_out[:, head block] =
 * w_in[:, head block] * R^T).  Packed modes with the streaming kernels' head layouts; rope_dim 64 or 128; all arrays
 * on the device, 16-byte aligned.  No counterpart in the reference (it runs the separate kernels). */
typedef struct tq_step_producer {
    const void* q_norm_weight; /* fp16 [layers][128] */
    const void* k_norm_weight; /* fp16 [layers][128] */
    const void* rope_cos;      /* fp16 [positions][rope_dim / 2] */
    const void* rope_sin;
    int rope_dim;
    float eps;
    int biased;                /* weights stored minus one (the reference's `biased` flag) */
    int rotated_output;
} tq_step_producer;
int tq_engine_decode_step_produce(tq_engine* e, const void* q_raw, const void* k_raw, const void* v, void* out,
                                  const tq_step_producer* prod, tq_stream_t s);
int tq_fold_rotation_into_projection(void* w_out, const void* w_in, const void* rotation, long long rows, int num_heads,
                                     tq_stream_t s);

/* The same for the layers first_layer .. first_layer + n_layers - 1 only; q, k, v, out point at the block of
 * first_layer ([n_layers][G][dim]).  Lets a caller exchange or copy out one group of layers while the next is computed. */
int tq_engine_decode_layers(tq_engine* e, int first_layer, int n_layers, const void* q, const void* k, const void* v,
                            void* out, tq_stream_t s);

/* tq_engine_decode_step in two phases, for callers that hand the results on group of layers by group of layers (an
 * exchange between GPUs, a copy to the host) while the rest is still being computed: tq_engine_step_prepare appends
 * the new token of every layer and rotates all queries (two launches); tq_engine_step_attend_layers then runs the
 * attention and the merge of the layers first_layer .. (two launches per call); out_first is the [G][q_dim] block of
 * first_layer inside a [layers][G][q_dim] buffer.  Packed modes with the whole-step form (otherwise
 * TQ_ERR_UNSUPPORTED: use tq_engine_decode_layers). */
int tq_engine_step_prepare(tq_engine* e, const void* q, const void* k, const void* v, tq_stream_t s);
int tq_engine_step_attend_layers(tq_engine* e, int first_layer, int n_layers, void* out_first, tq_stream_t s);

/* Error reporting aid, packed modes: with enable != 0 the engine also keeps every attention result as fp32, i.e. before
 * its final rounding to fp16 ([layers][G][num_heads][128], allocated outside the arena; call after
 * tq_engine_alloc_batch, and again after the batch shape changes); enable == 0 frees the buffer.
 * tq_engine_read_output_f32 copies n_layers layers of it to host memory and synchronises the stream.  No counterpart
 * in the reference (its kernels round to fp16 in registers, engine/kernels.cu:1772-1775). */
int tq_engine_output_f32(tq_engine* e, int enable);
int tq_engine_read_output_f32(tq_engine* e, float* host_out, int first_layer, int n_layers, tq_stream_t s);

/* Measurement aid: with enable != 0 the whole-step calls (tq_engine_decode_step / _decode_layers) record a CUDA event on
 * their stream directly before and after the attention launch (which is then launched without the programmatic overlap
 * with its predecessor); tq_engine_last_attention_ms waits for the second event of the most recent call and returns the
 * time between the two: the launch duration of decode_attention_kernel alone.  No counterpart in the reference. */
int tq_engine_time_attention(tq_engine* e, int enable);
int tq_engine_last_attention_ms(tq_engine* e, float* ms);

/* Token-form append of T tokens of sequence `seq` (prefill, engine/engine.cpp:2121-2130): k/v
 * [T][kv_dim] fp16 on the device, written at positions first_pos .. first_pos+T-1. */
int tq_engine_prefill_append(tq_engine* e, int layer, int seq, const void* k, const void* v, int first_pos,
                             int T, tq_stream_t s);

/* The same for n_seq consecutive sequences (first_seq, first_seq + 1, ...) in ONE launch: k, v are
 * [n_seq][T][kv_dim], every sequence receives its T tokens at positions first_pos .. first_pos + T - 1.  The reference
 * prefills one sequence and copies its cache to the others (engine/engine.cpp:2173-2214); this entry point is for
 * batches of different prompts of equal (padded) length.  No counterpart in the reference. */
int tq_engine_prefill_append_batch(tq_engine* e, int layer, int first_seq, int n_seq, const void* k, const void* v,
                                   int first_pos, int T, tq_stream_t s);

/* One layer of a prompt's prefill (engine/engine.cpp:2110-2146: the cache write of all T tokens, then the causal
 * self-attention): k/v [T][kv_dim] of sequence `seq` go to positions 0 .. T-1 of its slot, and query token t of
 * q [T][q_stride] attends to rows 0 .. t; out [T][q_stride] (the reference passes one stride, Q_PROJ_DIM, for both).
 * Packed modes and kv_bits = 0; sequences behind a shared prefix are refused (TQ_ERR_STATE). */
int tq_engine_prefill_layer(tq_engine* e, int layer, int seq, const void* q, const void* k, const void* v, void* out, int T,
                            int q_stride, tq_stream_t s);
/* The same for the n_seq prompts of T tokens of the sequences first_seq .. : q and out [n_seq][T][q_stride], k/v
 * [n_seq][T][kv_dim]; one append launch and one attention launch for all of them. */
int tq_engine_prefill_layer_batch(tq_engine* e, int layer, int first_seq, int n_seq, const void* q, const void* k, const void* v,
                                  void* out, int T, int q_stride, tq_stream_t s);

/* A prompt of T tokens shared by the n_seq sequences first_seq .. (rollouts of one prompt; the reference prefills
 * sequence 0 and copies its cache to the other sequences, engine/engine.cpp:2173-2214, 2296).  The first
 * P = 32 * floor(T / 32) tokens are quantised and stored once, in the slot of first_seq; the other sequences read
 * those tiles from there and their own slots begin at token P (so they may be given smaller capacities); the last
 * T - P tokens go into every sequence's own rows.  k, v: [T][kv_dim] fp16 on the device.  Call once per layer with the
 * same T, before anything else is appended to these sequences; packed modes only.  Decode steps, positions and
 * tq_engine_export_sequence work as for unshared sequences; tq_engine_import_sequence into a sharing slot makes it an
 * ordinary slot again. */
int tq_engine_prefill_shared(tq_engine* e, int layer, int first_seq, int n_seq, const void* k, const void* v, int T,
                             tq_stream_t s);

/* A whole decode step from HOST buffers: q_host [layers][G][q_dim], k_host/v_host [layers][G][kv_dim],
 * out_host [layers][G][q_dim], fp16, ideally pinned.  Copies the inputs in, runs every layer, copies the
 * outputs back and waits.  This is the end-to-end call bench.py times. */
int tq_engine_decode_step_host(tq_engine* e, const void* q_host, const void* k_host, const void* v_host,
                               void* out_host, tq_stream_t s);

/* ===================================================================================================================
 * Peer exchange for sequence-sharded ranks (one process per GPU).  No counterpart in the reference, which runs on one
 * GPU.  Every rank owns one buffer (made here with cudaMalloc so that a CUDA IPC handle names it); its peers open the
 * handle, copy their attention outputs into their slice with plain device-to-device copies (copy engines over NVLink:
 * no SM is taken from the attention kernel) and then write a step number into the owner's flag words; the owner waits,
 * with a time limit, for all of them.  Layout of a buffer is the caller's; the first TQ_PEER_MAX 8-byte words are the
 * flags by convention of triebwerk_b200.sharded.PeerCopyGatherer.
 * =================================================================================================================== */
#define TQ_PEER_MAX 32
/* cudaMalloc + zero fill + IPC handle (64 bytes, to be sent to the peers by any host channel). */
int tq_peer_buffer_create(size_t bytes, void** dptr, void* handle64);
/* Map a peer's buffer into this process (peer access is enabled on first use); close it again. */
int tq_peer_buffer_open(const void* handle64, void** dptr);
int tq_peer_buffer_close(void* dptr);
int tq_peer_buffer_destroy(void* dptr);
/* One asynchronous device-to-device copy on `s` (dst may be a peer's buffer). */
int tq_peer_copy(void* dst, const void* src, size_t bytes, tq_stream_t s);
/* After everything enqueued on `s` so far: flag_arrays[i][slot] = value for the n peers (release, system scope). */
int tq_peer_signal(void* const* flag_arrays, int n, int slot, unsigned long long value, tq_stream_t s);
/* Enqueue a wait on `s` until flags[0 .. n) have all reached `value`; after limit_ms (1 .. 10000) the kernel gives up,
 * raises status 4 in the int at status_word (device memory, may be null) and returns: the context stays usable. */
int tq_peer_wait(const void* flags, int n, unsigned long long value, void* status_word, unsigned limit_ms, tq_stream_t s);

#ifdef __cplusplus
}
#endif
#endif /* TRIEBWERK_B200_H_ */
