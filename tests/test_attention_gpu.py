"""GPU parity of the GQA decode attention over the packed cache, through the C ABI launchers, against the CPU
oracle on oracle-built caches (so that only the attention is under test) and against the committed outputs of
the reference's own kernels.  Tolerance: max-abs 2e-3 and relative 1e-2 in fp16 (tests/helpers.py)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import tqo
from tests import helpers as hp

pytestmark = pytest.mark.gpu
gu = pytest.importorskip("tests.gpu_util")

EDGE_LENGTHS = [1, 2, 31, 32, 33, 127, 128, 129, 511, 512, 513, 1000]


def _scales(kv_dim):
    return np.exp(np.random.default_rng(1).normal(0, 0.5, kv_dim)).astype(np.float32)


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("H", [16, 32])
def test_ragged_batch_edge_lengths(bits, H):
    rng = np.random.default_rng(10 + bits + H)
    R, _ = tqo.rotation()
    Hkv, D, msl = 8, 128, 1024
    lengths = EDGE_LENGTHS
    G = len(lengths)
    ck, kn, cv, vn = hp.build_cache_oracle(rng, G, lengths, msl, Hkv, D, bits, R, _scales(Hkv * D))
    q = rng.standard_normal((G, H * D), dtype=np.float32).astype(np.float16)
    pos = np.array(lengths, np.int32) - 1
    ref, _ = tqo.attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    got = gu.gpu_attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    worst, rel = hp.assert_attention_close(got, ref, H, D, f"tq{bits} H={H}")
    print(f"tq{bits} H={H}: max-abs {worst:.2e}, rel {rel:.2e}")


@pytest.mark.parametrize("bits", [4, 2])
def test_rows_past_the_position_are_ignored(bits):
    """Rows after positions[g] hold other data (here: random bytes and NaN norms): they must not leak in."""
    rng = np.random.default_rng(20)
    R, _ = tqo.rotation()
    G, H, Hkv, D, msl = 3, 16, 8, 128, 96
    lengths = [5, 40, 70]
    ck, kn, cv, vn = hp.build_cache_oracle(rng, G, lengths, msl, Hkv, D, bits, R)
    q = rng.standard_normal((G, H * D), dtype=np.float32).astype(np.float16)
    pos = np.array(lengths, np.int32) - 1
    ref, _ = tqo.attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    for g, n in enumerate(lengths):
        sl = slice(g * msl + n, (g + 1) * msl)
        ck[sl] = rng.integers(0, 256, ck[sl].shape, dtype=np.uint8)
        cv[sl] = rng.integers(0, 256, cv[sl].shape, dtype=np.uint8)
        kn[sl] = np.float16(np.nan)
        vn[sl] = np.float16(np.inf)
    got = gu.gpu_attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    hp.assert_attention_close(got, ref, H, D, f"tq{bits} garbage tail")


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("copies", [1, 3])
def test_long_context_split_over_many_ctas(bits, copies):
    # 8 (24) sequences x 4096 tokens: every sequence is cut across ~37 (~12) workers and merged by the last one to
    # arrive; the merge has one path for up to 8 parts, one for more, and reloads its weights every 32 parts
    rng = np.random.default_rng(30)
    R, _ = tqo.rotation()
    H, Hkv, D, msl = 16, 8, 128, 4096
    lengths = [4096, 4096, 4095, 4065, 3000, 4096, 17, 4096] * copies
    G = len(lengths)
    ck, kn, cv, vn = hp.build_cache_oracle(rng, G, lengths, msl, Hkv, D, bits, R, _scales(Hkv * D))
    q = rng.standard_normal((G, H * D), dtype=np.float32).astype(np.float16)
    pos = np.array(lengths, np.int32) - 1
    ref, _ = tqo.attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    got = gu.gpu_attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    worst, rel = hp.assert_attention_close(got, ref, H, D, f"tq{bits} long")
    print(f"tq{bits} long: max-abs {worst:.2e}, rel {rel:.2e}")
    # run it again: tickets and workspace must be reusable as they are
    got2 = gu.gpu_attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    assert (got2.view(np.uint16) == got.view(np.uint16)).all()


def test_peaked_and_flat_softmax():
    """One key aligned with the query (weight ~1 on one position) and an all-equal cache (uniform weights)."""
    rng = np.random.default_rng(40)
    R, _ = tqo.rotation()
    G, H, Hkv, D, msl, bits = 2, 16, 8, 128, 256, 4
    kv_dim = Hkv * D
    L = 200
    k = rng.standard_normal((L, kv_dim), dtype=np.float32)
    v = rng.standard_normal((L, kv_dim), dtype=np.float32)
    q = rng.standard_normal((G, H * D), dtype=np.float32)
    k[77] = np.tile(q[0].reshape(H, D)[::2], 1).reshape(-1) * 8.0  # KV head h aligned with query head 2h, large norm
    ck, kn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    cv, vn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    posl = np.arange(L, dtype=np.int32)
    tqo.append_tokens(ck, kn, k.astype(np.float16), R, posl, msl, Hkv, D, bits)
    tqo.append_tokens(cv, vn, v.astype(np.float16), R, posl, msl, Hkv, D, bits)
    same_k = np.tile(k[:1], (L, 1)).astype(np.float16)
    tqo.append_tokens(ck[msl:], kn[msl:], same_k, R, posl, msl, Hkv, D, bits)
    tqo.append_tokens(cv[msl:], vn[msl:], v.astype(np.float16), R, posl, msl, Hkv, D, bits)
    q16 = q.astype(np.float16)
    pos = np.array([L - 1, L - 1], np.int32)
    ref, _ = tqo.attention_batch(q16, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    got = gu.gpu_attention_batch(q16, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    hp.assert_attention_close(got, ref, H, D, "peaked/flat")


def test_identical_sequences_and_permutation():
    rng = np.random.default_rng(50)
    R, _ = tqo.rotation()
    H, Hkv, D, msl, bits, L = 16, 8, 128, 320, 4, 300
    ck1, kn1, cv1, vn1 = hp.build_cache_oracle(rng, 1, [L], msl, Hkv, D, bits, R)
    G = 4
    ck, cv = np.tile(ck1, (G, 1)), np.tile(cv1, (G, 1))
    kn, vn = np.tile(kn1, (G, 1)), np.tile(vn1, (G, 1))
    q = np.tile(rng.standard_normal((1, H * D), dtype=np.float32).astype(np.float16), (G, 1))
    pos = np.full(G, L - 1, np.int32)
    out = gu.gpu_attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    assert (out.view(np.uint16) == out[0].view(np.uint16)).all(), "identical sequences gave different outputs"
    # permuting sequences permutes outputs (different lengths, different slices of the CTA partition)
    lengths = [300, 10, 150, 299]
    ck, kn, cv, vn = hp.build_cache_oracle(rng, G, lengths, msl, Hkv, D, bits, R)
    q = rng.standard_normal((G, H * D), dtype=np.float32).astype(np.float16)
    pos = np.array(lengths, np.int32) - 1
    a = gu.gpu_attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    perm = np.array([2, 0, 3, 1])
    rows = np.concatenate([np.arange(g * msl, (g + 1) * msl) for g in perm])
    b = gu.gpu_attention_batch(q[perm], ck[rows], cv[rows], kn[rows], vn[rows], R, pos[perm], msl, H, Hkv, D, bits)
    hp.assert_attention_close(b, a[perm], H, D, "permutation")


@pytest.mark.parametrize("bits", [4, 2])
def test_single_sequence_and_prefill_forms(bits):
    rng = np.random.default_rng(60)
    R, _ = tqo.rotation()
    H, Hkv, D, msl, L = 16, 8, 128, 192, 150
    ck, kn, cv, vn = hp.build_cache_oracle(rng, 1, [L], msl, Hkv, D, bits, R)
    q = rng.standard_normal(H * D, dtype=np.float32).astype(np.float16)
    for pos in (0, 31, 32, L - 1):
        ref, _ = tqo.attention_single(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
        got = gu.gpu_attention_single(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
        hp.assert_attention_close(got[None], ref[None], H, D, f"single pos={pos}")
    T = 70
    qp = rng.standard_normal((T, H * D), dtype=np.float32).astype(np.float16)
    ref, _ = tqo.prefill_attention(qp, ck, cv, kn, vn, R, msl, H, Hkv, D, bits)
    got = gu.gpu_prefill_attention(qp, ck, cv, kn, vn, R, msl, H, Hkv, D, bits)
    hp.assert_attention_close(got, ref, H, D, "prefill")


@pytest.mark.parametrize("bits", [4, 2])
def test_attention_on_reference_cache_bytes_vs_reference_outputs(bits):
    g = hp.load_golden(f"ref_kernels_tq{bits}.npz")
    if g is None:
        pytest.skip("fixture not generated yet")
    H, Hkv, D, msl = int(g["H"]), int(g["Hkv"]), int(g["D"]), int(g["msl"])
    R = hp.h(g["R"])
    got = gu.gpu_attention_batch(hp.h(g["q"]), g["ck"], g["cv"], hp.h(g["kn"]), hp.h(g["vn"]), R, g["final_pos"], msl, H,
                                 Hkv, D, bits)
    hp.assert_attention_close(got, hp.h(g["out"]), H, D, "vs reference kernels (batched)")
    sl = slice(2 * msl, 3 * msl)
    got1 = gu.gpu_attention_single(hp.h(g["q"])[2], g["ck"][sl], g["cv"][sl], hp.h(g["kn"])[sl], hp.h(g["vn"])[sl], R,
                                   int(g["final_pos"][2]), msl, H, Hkv, D, bits)
    hp.assert_attention_close(got1[None], hp.h(g["out_single"])[None], H, D, "vs reference kernels (single)")
    gotp = gu.gpu_prefill_attention(hp.h(g["q_prefill"]), g["ck"][sl], g["cv"][sl], hp.h(g["kn"])[sl],
                                    hp.h(g["vn"])[sl], R, msl, H, Hkv, D, bits)
    hp.assert_attention_close(gotp, hp.h(g["out_prefill"]), H, D, "vs reference kernels (prefill)")


def test_attention_equals_reference_kernels_live():
    if not os.path.exists(gu.REF_SO):
        pytest.skip("reference kernel library not present in this snapshot")
    ref = C.CDLL(gu.REF_SO)
    ref.launch_turbo_gqa_attention_batch.restype = None
    rng = np.random.default_rng(70)
    R, _ = tqo.rotation()
    G, H, Hkv, D, msl, bits = 4, 16, 8, 128, 640, 4
    lengths = [101, 300, 612, 612]  # the reference configuration's context range
    ck, kn, cv, vn = hp.build_cache_oracle(rng, G, lengths, msl, Hkv, D, bits, R, _scales(Hkv * D))
    q = rng.standard_normal((G, H * D), dtype=np.float32).astype(np.float16)
    pos = np.array(lengths, np.int32) - 1
    d = [gu.dev(x) for x in (q, ck, cv, kn, vn, R, pos)]
    out = torch.zeros(G, H * D, dtype=torch.float16, device="cuda")
    scratch = torch.zeros(G * H * msl, dtype=torch.float32, device="cuda")
    vp = lambda t: C.c_void_p(t.data_ptr())
    i = C.c_int
    ref.launch_turbo_gqa_attention_batch(vp(out), vp(d[0]), vp(d[1]), vp(d[2]), vp(d[3]), vp(d[4]), vp(d[5]), vp(scratch),
                                         vp(d[6]), i(msl), i(G), i(H), i(Hkv), i(D), i(H * D), i(Hkv * D), i(bits),
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
    want = gu.host(out)
    got = gu.gpu_attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    worst, rel = hp.assert_attention_close(got, want, H, D, "vs live reference kernels")
    print(f"vs live reference kernels: max-abs {worst:.2e}, rel {rel:.2e}")


def test_three_kv_heads_are_served_and_bad_shapes_refused():
    """3 KV heads is outside the streaming kernel's layouts: the launcher serves it through the generic kernel, as the
    reference would.  What no kernel can serve (heads not divisible, head_dim other than 128) is still refused."""
    import triebwerk_b200 as tq
    from triebwerk_b200 import ops
    R, _ = tqo.rotation()
    rng = np.random.default_rng(80)
    H, Hkv, D, msl, bits = 6, 3, 128, 32, 4
    ck, kn, cv, vn = hp.build_cache_oracle(rng, 1, [4], msl, Hkv, D, bits, R)
    q = rng.standard_normal((1, H * D), dtype=np.float32).astype(np.float16)
    got = gu.gpu_attention_batch(q, ck, cv, kn, vn, R, [3], msl, H, Hkv, D, bits)
    ref, _ = tqo.attention_batch(q, ck, cv, kn, vn, R, np.array([3], np.int32), msl, H, Hkv, D, bits)
    hp.assert_attention_close(got, ref, H, D, "3 KV heads")
    with pytest.raises(tq.TqError) as e:  # 7 query heads over 3 KV heads
        gu.gpu_attention_batch(np.zeros((1, 7 * D), np.float16), ck, cv, kn, vn, R, [3], msl, 7, Hkv, D, bits)
    assert e.value.status == -1
    with pytest.raises(tq.TqError) as e:  # the native entry point on pre-rotated queries: streaming layouts only
        ws = ops.new_workspace(1, H)
        out = torch.zeros(1, H * D, dtype=torch.float16, device="cuda")
        ops.decode_attention(out, gu.dev(ck), gu.dev(cv), gu.dev(kn), gu.dev(vn), gu.dev(R), gu.dev(np.array([3], np.int32)), msl,
                             H, Hkv, bits, ws)
    assert e.value.status == -4


@pytest.mark.parametrize("bits,H,Hkv", [(4, 40, 8), (2, 8, 2), (4, 64, 8), (4, 6, 2), (0, 12, 4), (0, 40, 8)])
def test_head_layouts_outside_the_streaming_kernel(bits, H, Hkv):
    """The reference kernels take any number of heads (grid (G, num_heads)); so do the launchers here: layouts the
    streaming kernels are not built for (more than 32 query heads, 2 KV heads, 3 or 5 query heads per KV head ...) go
    through the generic kernel.  Batched, single-sequence and prefill forms against the oracle."""
    import triebwerk_b200 as tq
    from triebwerk_b200 import ops
    rng = np.random.default_rng(300 + bits + H)
    R, _ = tqo.rotation()
    D, msl = 128, 320
    lengths = [1, 33, 300, 129]
    G = len(lengths)
    q = rng.standard_normal((G, H * D), dtype=np.float32).astype(np.float16)
    pos = np.array(lengths, np.int32) - 1
    if bits == 0:
        ck = rng.standard_normal((G * msl, Hkv * D), dtype=np.float32).astype(np.float16)
        cv = rng.standard_normal((G * msl, Hkv * D), dtype=np.float32).astype(np.float16)
        ref, _ = tqo.fp16_attention_batch(q, ck, cv, pos, msl, H, Hkv, D)
        out = torch.zeros(G, H * D, dtype=torch.float16, device="cuda")
        ops.launch_gqa_attention_batch(out, gu.dev(q), gu.dev(ck), gu.dev(cv), None, gu.dev(pos), msl, G, H, Hkv, D, H * D, Hkv * D)
        hp.assert_attention_close(gu.host(out), ref, H, D, f"generic fp16 H={H} Hkv={Hkv}")
        return
    ck, kn, cv, vn = hp.build_cache_oracle(rng, G, lengths, msl, Hkv, D, bits, R)
    ref, _ = tqo.attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    got = gu.gpu_attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    w, r = hp.assert_attention_close(got, ref, H, D, f"generic batched tq{bits} H={H} Hkv={Hkv}")
    print(f"generic kernel tq{bits} H={H} Hkv={Hkv}: max-abs {w:.2e}, rel {r:.2e}")
    g = 2
    sl = slice(g * msl, (g + 1) * msl)
    got1 = gu.gpu_attention_single(q[g], ck[sl], cv[sl], kn[sl], vn[sl], R, pos[g], msl, H, Hkv, D, bits)
    hp.assert_attention_close(got1[None], ref[g][None], H, D, "generic single-sequence")
    T = 40
    qt = rng.standard_normal((T, H * D), dtype=np.float32).astype(np.float16)
    refp, _ = tqo.prefill_attention(qt, ck[sl], cv[sl], kn[sl], vn[sl], R, msl, H, Hkv, D, bits)
    gotp = gu.gpu_prefill_attention(qt, ck[sl], cv[sl], kn[sl], vn[sl], R, msl, H, Hkv, D, bits)
    hp.assert_attention_close(gotp, refp, H, D, "generic prefill")
    # the engine serves the layout too: append (chain kernel) + generic attention, bytes as the oracle's
    eng = tq.Engine(msl, bits, num_layers=1, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(G, msl)
    ks = [rng.standard_normal((n, Hkv * D), dtype=np.float32).astype(np.float16) for n in lengths]
    vs = [rng.standard_normal((n, Hkv * D), dtype=np.float32).astype(np.float16) for n in lengths]
    for gi, n in enumerate(lengths):
        if n > 1:
            eng.prefill_append(0, gi, gu.dev(ks[gi][:-1]), gu.dev(vs[gi][:-1]), 0)
    eng.set_positions([n - 1 for n in lengths])
    oute = gu.host(eng.decode_layer(0, gu.dev(q), gu.dev(np.stack([k[-1] for k in ks])), gu.dev(np.stack([v[-1] for v in vs]))))
    assert eng.status() == 0
    # (against the oracle run on the engine's OWN cache bytes: a coordinate that sits on a quantiser bound may
    # legitimately fall to the other side than in the oracle's append, see tests/test_append_gpu.py)
    gk, gv, gkn, gvn = (gu.host(t) for t in eng.layer_cache(0))
    n_diff = 0
    for gi, n in enumerate(lengths):
        sl = slice(gi * msl, gi * msl + n)
        r1, _ = tqo.attention_single(q[gi], gk[sl], gv[sl], gkn[sl], gvn[sl], R, n - 1, n, H, Hkv, D, bits)
        hp.assert_attention_close(oute[gi][None], r1[None], H, D, f"generic engine seq {gi}")
        cq, cn = tqo.alloc_cache(1, n, Hkv, D, bits)
        tqo.append_tokens(cq, cn, ks[gi], R, np.arange(n, dtype=np.int32), n, Hkv, D, bits)
        n_diff += int((hp.unpack_codes(cq, bits) != hp.unpack_codes(gk[sl], bits)).sum())
    assert n_diff <= 4, f"{n_diff} K coordinates differ from the oracle's append"


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("H,Hkv", [(16, 8), (32, 8), (8, 8), (32, 4)])
def test_prefill_attention_with_query_tiles_at_ragged_sizes(bits, H, Hkv):
    """launch_turbo_gqa_prefill_attention through the kernel that holds the query tokens in the M dimension: T and the
    slot size are no multiples of the 64-row cache tile or of the query block, and the cache rows past the prompt hold
    garbage (codes 0xff, norms that are not numbers) which no result may depend on.  Against the oracle
    (engine/kernels.cu:1874-1960 restated)."""
    rng = np.random.default_rng(300 + bits + H)
    R, _ = tqo.rotation()
    D, T, msl = 128, 333, 350
    ck, kn, cv, vn = hp.build_cache_oracle(rng, 1, [T], msl, Hkv, D, bits, R)
    ck[T:] = 0xFF
    cv[T:] = 0xFF
    kn.view(np.uint16)[T:] = 0x7E00
    vn.view(np.uint16)[T:] = 0x7E00
    q = rng.standard_normal((T, H * D), dtype=np.float32).astype(np.float16)
    ref, _ = tqo.prefill_attention(q, ck, cv, kn, vn, R, msl, H, Hkv, D, bits)
    got = gu.gpu_prefill_attention(q, ck, cv, kn, vn, R, msl, H, Hkv, D, bits)
    assert np.isfinite(got.astype(np.float32)).all()
    w, r = hp.assert_attention_close(got, ref, H, D, f"prefill attention tq{bits} H={H} Hkv={Hkv}")
    print(f"prefill attention tq{bits} H={H} Hkv={Hkv} T={T}: max-abs {w:.2e}, rel {r:.2e}")
    # a short prompt: fewer query tokens than one block, one cache tile
    got_s = gu.gpu_prefill_attention(q[:5], ck, cv, kn, vn, R, msl, H, Hkv, D, bits)
    hp.assert_attention_close(got_s, ref[:5], H, D, "prefill attention, 5 tokens")


def test_prefill_attention_mma_sync_form_in_a_child_process():
    """The tcgen05 form of the prefill attention is the default; the mma.sync form is selected by TQ_PREFILL_ATTN_TC=0, which
    the library reads once per process: the parity tests of the prefill attention run again in a child with it set."""
    import os
    import subprocess
    import sys
    if os.environ.get("TQ_PREFILL_ATTN_TC") == "0":
        pytest.skip("already the child")
    env = dict(os.environ, TQ_PREFILL_ATTN_TC="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_attention_gpu.py", "tests/test_fp16_gpu.py", "tests/test_engine_gpu.py",
                        "-q", "-x", "-m", "gpu", "-k", "prefill and not child", "-p", "no:cacheprovider"],
                       cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert " passed" in r.stdout
