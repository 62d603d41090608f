"""GPU parity of the kv_bits = 0 twin (fp16 cache write + GQA decode attention) against the oracle and the
committed outputs of the reference's own kernels."""
import numpy as np
import pytest
import torch

from oracle import tqo
from tests import helpers as hp

pytestmark = pytest.mark.gpu
gu = pytest.importorskip("tests.gpu_util")
from triebwerk_b200 import ops  # noqa: E402


def _fill(rng, G, lengths, msl, kv_dim):
    ck = np.zeros((G * msl, kv_dim), np.float16)
    cv = np.zeros_like(ck)
    for g, n in enumerate(lengths):
        ck[g * msl:g * msl + n] = rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16)
        cv[g * msl:g * msl + n] = rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16)
    return ck, cv


def test_cache_write_is_a_row_copy():
    rng = np.random.default_rng(0)
    G, kv_dim, msl = 5, 1024, 40
    k = rng.standard_normal((G, kv_dim), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((G, kv_dim), dtype=np.float32).astype(np.float16)
    pos = np.array([0, 39, 7, 20, 1], np.int32)
    dck = torch.zeros(G * msl, kv_dim, dtype=torch.float16, device="cuda")
    dcv = torch.zeros_like(dck)
    ops.launch_kv_cache_write_batch(dck, dcv, gu.dev(k), gu.dev(v), gu.dev(pos), msl, G, kv_dim)
    ock = np.zeros((G * msl, kv_dim), np.float16)
    ocv = np.zeros_like(ock)
    tqo.fp16_write_batch(ock, ocv, k, v, pos, msl)
    assert (gu.host(dck).view(np.uint16) == ock.view(np.uint16)).all()
    assert (gu.host(dcv).view(np.uint16) == ocv.view(np.uint16)).all()


@pytest.mark.parametrize("H", [8, 16, 32])
def test_fp16_attention_ragged(H):
    rng = np.random.default_rng(1 + H)
    Hkv, D, msl = 8, 128, 1100
    lengths = [1, 2, 31, 32, 33, 511, 512, 513, 1024, 1100]
    G = len(lengths)
    ck, cv = _fill(rng, G, lengths, msl, Hkv * D)
    # rows past the position must be ignored even when they hold NaN
    for g, n in enumerate(lengths):
        ck[g * msl + n:(g + 1) * msl] = np.float16(np.nan)
        cv[g * msl + n:(g + 1) * msl] = np.float16(np.nan)
    q = rng.standard_normal((G, H * D), dtype=np.float32).astype(np.float16)
    pos = np.array(lengths, np.int32) - 1
    ref, _ = tqo.fp16_attention_batch(q, ck, cv, pos, msl, H, Hkv, D)
    out = torch.zeros(G, H * D, dtype=torch.float16, device="cuda")
    ops.launch_gqa_attention_batch(out, gu.dev(q), gu.dev(ck), gu.dev(cv), None, gu.dev(pos), msl, G, H, Hkv, D, H * D,
                                   Hkv * D)
    worst, rel = hp.assert_attention_close(gu.host(out), ref, H, D, f"fp16 H={H}")
    print(f"fp16 H={H}: max-abs {worst:.2e}, rel {rel:.2e}")
    g = G - 1
    o1 = torch.zeros(H * D, dtype=torch.float16, device="cuda")
    ops.launch_gqa_attention(gu.dev(q[g]), gu.dev(ck[g * msl:(g + 1) * msl]), gu.dev(cv[g * msl:(g + 1) * msl]), o1, None,
                             int(pos[g]), msl, H, Hkv, D)
    r1, _ = tqo.fp16_attention_single(q[g], ck[g * msl:(g + 1) * msl], cv[g * msl:(g + 1) * msl], int(pos[g]), msl, H,
                                      Hkv, D)
    hp.assert_attention_close(gu.host(o1)[None], r1[None], H, D, "fp16 single")


def test_fp16_against_reference_kernel_outputs():
    g = hp.load_golden("ref_kernels_fp16.npz")
    if g is None:
        pytest.skip("fixture not generated yet")
    H, Hkv, D, msl = int(g["H"]), int(g["Hkv"]), int(g["D"]), int(g["msl"])
    k_steps, v_steps = hp.h(g["k_steps"]), hp.h(g["v_steps"])
    G = k_steps.shape[1]
    dck = torch.zeros(G * msl, Hkv * D, dtype=torch.float16, device="cuda")
    dcv = torch.zeros_like(dck)
    for s in range(k_steps.shape[0]):
        ops.launch_kv_cache_write_batch(dck, dcv, gu.dev(k_steps[s]), gu.dev(v_steps[s]), gu.dev(g["pos_steps"][s]), msl,
                                        G, Hkv * D)
    out = torch.zeros(G, H * D, dtype=torch.float16, device="cuda")
    ops.launch_gqa_attention_batch(out, gu.dev(hp.h(g["q"])), dck, dcv, None, gu.dev(g["final_pos"]), msl, G, H, Hkv, D,
                                   H * D, Hkv * D)
    hp.assert_attention_close(gu.host(out), hp.h(g["out"]), H, D, "fp16 vs reference kernels")


@pytest.mark.parametrize("H,Hkv", [(16, 4), (32, 4), (8, 8)])
def test_fp16_attention_many_chunks_and_wide_groups(H, Hkv):
    """Contexts of several 512-token chunks (ticketed merge), chunk tails of every length modulo the 16-token step of
    a CTA, and 4 or 8 query heads per KV head."""
    rng = np.random.default_rng(50 + H + Hkv)
    D, msl = 128, 2100
    lengths = [2100, 2049, 1537, 1025, 515, 514, 513, 17, 16, 15, 5, 4, 3]
    G = len(lengths)
    ck, cv = _fill(rng, G, lengths, msl, Hkv * D)
    q = rng.standard_normal((G, H * D), dtype=np.float32).astype(np.float16)
    pos = np.array(lengths, np.int32) - 1
    ref, _ = tqo.fp16_attention_batch(q, ck, cv, pos, msl, H, Hkv, D)
    out = torch.zeros(G, H * D, dtype=torch.float16, device="cuda")
    ops.launch_gqa_attention_batch(out, gu.dev(q), gu.dev(ck), gu.dev(cv), None, gu.dev(pos), msl, G, H, Hkv, D, H * D,
                                   Hkv * D)
    worst, rel = hp.assert_attention_close(gu.host(out), ref, H, D, f"fp16 H={H} Hkv={Hkv}")
    print(f"fp16 H={H} Hkv={Hkv}: max-abs {worst:.2e}, rel {rel:.2e}")
    # a second launch on the same workspace: tickets must have been left ready
    out2 = torch.zeros_like(out)
    ops.launch_gqa_attention_batch(out2, gu.dev(q), gu.dev(ck), gu.dev(cv), None, gu.dev(pos), msl, G, H, Hkv, D, H * D,
                                   Hkv * D)
    assert torch.equal(out, out2)


def test_fp16_prefill_attention_against_oracle_and_reference_kernel():
    """launch_gqa_prefill_attention (kv_bits = 0): query token t attends to rows 0 .. t of one sequence.  Against the
    oracle's single-sequence attention per token, and against the reference's own kernel run live when its build is
    there."""
    import ctypes as C
    import os
    rng = np.random.default_rng(77)
    H, Hkv, D, T, msl = 16, 8, 128, 70, 96
    k = rng.standard_normal((msl, Hkv * D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((msl, Hkv * D), dtype=np.float32).astype(np.float16)
    q = rng.standard_normal((T, H * D), dtype=np.float32).astype(np.float16)
    dk, dv, dq = gu.dev(k), gu.dev(v), gu.dev(q)
    out = torch.zeros(T, H * D, dtype=torch.float16, device="cuda")
    ops.launch_gqa_prefill_attention(out, dq, dk, dv, None, T, msl, H, Hkv, D, H * D, Hkv * D)
    got = gu.host(out)
    ref = np.stack([tqo.fp16_attention_single(q[t], k, v, t, msl, H, Hkv, D)[0] for t in range(T)])
    worst, rel = hp.assert_attention_close(got, ref, H, D, "fp16 prefill attention vs oracle")
    print(f"fp16 prefill attention: max-abs {worst:.2e}, rel {rel:.2e} against the oracle")
    if os.path.exists(gu.REF_SO):
        refl = C.CDLL(gu.REF_SO)
        scratch = torch.zeros(T * H * T, dtype=torch.float32, device="cuda")
        out_ref = torch.zeros_like(out)
        vp, i = C.c_void_p, C.c_int
        refl.launch_gqa_prefill_attention.restype = None
        refl.launch_gqa_prefill_attention.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, vp]
        refl.launch_gqa_prefill_attention(out_ref.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(), T,
                                          msl, H, Hkv, D, H * D, Hkv * D, torch.cuda.current_stream().cuda_stream)
        w2, _ = hp.assert_attention_close(got, gu.host(out_ref), H, D, "fp16 prefill attention vs the reference kernel")
        print(f"fp16 prefill attention: max-abs {w2:.2e} against the reference's own kernel")


@pytest.mark.parametrize("H,Hkv,T,msl", [(16, 8, 333, 350), (32, 8, 200, 200), (8, 8, 130, 192), (32, 4, 97, 100)])
def test_fp16_prefill_attention_with_query_tiles(H, Hkv, T, msl):
    """launch_gqa_prefill_attention through the kernel with the query tokens in the M dimension, at sizes that are no
    multiples of its tiles; rows past the prompt hold values that are not numbers."""
    rng = np.random.default_rng(500 + H + T)
    D = 128
    k = rng.standard_normal((msl, Hkv * D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((msl, Hkv * D), dtype=np.float32).astype(np.float16)
    k.view(np.uint16)[T:] = 0x7E00
    v.view(np.uint16)[T:] = 0x7E00
    q = rng.standard_normal((T, H * D), dtype=np.float32).astype(np.float16)
    out = torch.zeros(T, H * D, dtype=torch.float16, device="cuda")
    ops.launch_gqa_prefill_attention(out, gu.dev(q), gu.dev(k), gu.dev(v), None, T, msl, H, Hkv, D, H * D, Hkv * D)
    got = gu.host(out)
    assert np.isfinite(got.astype(np.float32)).all()
    ref = np.stack([tqo.fp16_attention_single(q[t], k, v, t, msl, H, Hkv, D)[0] for t in range(T)])
    worst, rel = hp.assert_attention_close(got, ref, H, D, f"fp16 prefill attention H={H} Hkv={Hkv} T={T}")
    print(f"fp16 prefill attention H={H} Hkv={Hkv} T={T}: max-abs {worst:.2e}, rel {rel:.2e}")
