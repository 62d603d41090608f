"""The decode step with its producer and consumer folded in (tq_engine_decode_step_produce): per-head RMS norm and
rotary embedding of the raw q / k projections run inside the query rotation and inside the append, and the inverse
rotation can be left to the consumer's weights.  Checked against the reference's OWN producer kernels run live
(qk_norm_batch_kernel + rope_batch_kernel, built unmodified under oracle/_ref) followed by the plain decode step --
cache bytes and outputs must be identical -- and against the CPU oracle's restatement of the producer."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import triebwerk_b200 as tq
from oracle import tqo
from tests import helpers as hp

pytestmark = pytest.mark.gpu
gu = pytest.importorskip("tests.gpu_util")

D = 128


def _rope_tables(rng, n_pos, rope_dim):
    half = rope_dim // 2
    inv = 1.0 / (10000.0 ** (np.arange(half, dtype=np.float64) / half))
    ang = np.arange(n_pos, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)


def _reference_producer(q, k, qw, kw, cos, sin, pos, H, Hkv, rope_dim, eps, biased):
    """q [G, q_dim], k [G, kv_dim] torch fp16 on the device -> the reference kernels' in-place results (copies)."""
    ref = C.CDLL(gu.REF_SO)
    vp, i = C.c_void_p, C.c_int
    ref.launch_qk_norm_batch.restype = None
    ref.launch_qk_norm_batch.argtypes = [vp, vp, vp, vp, i, i, i, i, C.c_float, i, i, vp, C.c_bool]
    ref.launch_rope_batch.restype = None
    ref.launch_rope_batch.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, vp]
    q, k = q.clone(), k.clone()
    G = q.shape[0]
    st = torch.cuda.current_stream().cuda_stream
    ref.launch_qk_norm_batch(q.data_ptr(), k.data_ptr(), qw.data_ptr(), kw.data_ptr(), H, Hkv, D, G, eps, H * D, Hkv * D, st, biased)
    ref.launch_rope_batch(q.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(), 0, G, H, Hkv, D, H * D,
                          Hkv * D, rope_dim, st)
    torch.cuda.synchronize()
    return q, k


@pytest.mark.parametrize("bits,H,Hkv,rope_dim,biased", [(4, 16, 8, 128, False), (2, 32, 8, 128, False), (4, 16, 4, 64, True)])
def test_fused_producer_equals_separate_kernels(bits, H, Hkv, rope_dim, biased):
    NL, eps = 3, 1e-6
    kv_dim, q_dim = Hkv * D, H * D
    lengths = [130, 1, 64, 700, 33, 257]
    G = len(lengths)
    caps = [n + 3 for n in lengths]
    rng = np.random.default_rng(500 + bits + H)
    engines = [tq.Engine(1024, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D) for _ in range(2)]
    for eng in engines:
        eng.alloc_batch(G, 1024, caps)
    for layer in range(NL):
        for g, n in enumerate(lengths):
            if n > 1:
                k = gu.dev(rng.standard_normal((n - 1, kv_dim), dtype=np.float32).astype(np.float16))
                v = gu.dev(rng.standard_normal((n - 1, kv_dim), dtype=np.float32).astype(np.float16))
                for eng in engines:
                    eng.prefill_append(layer, g, k, v, 0)
    for eng in engines:
        eng.set_positions([n - 1 for n in lengths])
    cos_h, sin_h = _rope_tables(rng, 1024, rope_dim)
    cos, sin = gu.dev(cos_h), gu.dev(sin_h)
    qw_h = (1.0 + 0.2 * rng.standard_normal((NL, D))).astype(np.float16) - (1.0 if biased else 0.0)
    kw_h = (1.0 + 0.2 * rng.standard_normal((NL, D))).astype(np.float16) - (1.0 if biased else 0.0)
    qw, kw = gu.dev(qw_h.astype(np.float16)), gu.dev(kw_h.astype(np.float16))
    pos = gu.dev(np.array([n - 1 for n in lengths], np.int32))
    for step in range(2):
        q_raw = gu.dev((3.0 * rng.standard_normal((NL, G, q_dim), dtype=np.float32)).astype(np.float16))
        k_raw = gu.dev((0.5 * rng.standard_normal((NL, G, kv_dim), dtype=np.float32)).astype(np.float16))
        v = gu.dev(rng.standard_normal((NL, G, kv_dim), dtype=np.float32).astype(np.float16))
        # separate producer: the reference's own kernels when built, else the CPU oracle's restatement
        q_post, k_post = torch.empty_like(q_raw), torch.empty_like(k_raw)
        live = os.path.exists(gu.REF_SO)
        for layer in range(NL):
            if live:
                q_post[layer], k_post[layer] = _reference_producer(q_raw[layer], k_raw[layer], qw[layer], kw[layer], cos, sin, pos,
                                                                   H, Hkv, rope_dim, eps, biased)
            oq, ok = tqo.qk_norm_rope_batch(gu.host(q_raw[layer]), gu.host(k_raw[layer]), qw_h[layer].astype(np.float16),
                                            kw_h[layer].astype(np.float16), cos_h, sin_h, gu.host(pos), H, Hkv, D, rope_dim, eps, biased)
            if live:
                # the oracle (IEEE 1/sqrt) against the reference kernels (rsqrt.approx): a normed value may land on the
                # neighbouring fp16, and a rotary pair combines two of them: rarely, and never by more than two steps
                dq = np.abs(gu.host(q_post[layer]).view(np.uint16).astype(np.int32) - oq.view(np.uint16).astype(np.int32))
                dk = np.abs(gu.host(k_post[layer]).view(np.uint16).astype(np.int32) - ok.view(np.uint16).astype(np.int32))
                assert int(dq.max()) <= 2 and int(dk.max()) <= 2, "oracle producer differs from the reference kernels by more than two fp16 steps"
                assert float((dq > 0).mean()) < 0.02 and float((dk > 0).mean()) < 0.02
            else:
                q_post[layer], k_post[layer] = gu.dev(oq), gu.dev(ok)
        out_sep, out_fused = torch.empty_like(q_raw), torch.empty_like(q_raw)
        engines[0].decode_step(q_post, k_post, v, out_sep)
        engines[1].decode_step_produce(q_raw, k_raw, v, out_fused, qw, kw, cos, sin, rope_dim, eps, biased)
        for eng in engines:
            assert eng.status() == 0
        if live:
            for layer in range(NL):
                for x, y, name in zip(engines[0].layer_cache(layer), engines[1].layer_cache(layer), ("k codes", "v codes", "k norms", "v norms")):
                    assert torch.equal(x.view(torch.uint8), y.view(torch.uint8)), f"step {step} layer {layer}: {name} differ"
            assert torch.equal(out_sep.view(torch.int16), out_fused.view(torch.int16)), "outputs differ from the separate kernels' path"
        else:
            hp.assert_attention_close(gu.host(out_fused).reshape(NL * G, q_dim), gu.host(out_sep).reshape(NL * G, q_dim), H, D, "fused producer")
        for eng in engines:
            eng.advance()
        pos += 1


def test_rotated_output_and_folded_projection():
    bits, H, Hkv, NL = 4, 16, 8, 2
    kv_dim, q_dim = Hkv * D, H * D
    lengths = [90, 300, 17]
    G = len(lengths)
    rng = np.random.default_rng(600)
    eng = tq.Engine(512, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(G, 512)
    for layer in range(NL):
        for g, n in enumerate(lengths):
            eng.prefill_append(layer, g, gu.dev(rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16)),
                               gu.dev(rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16)), 0)
    eng.set_positions(lengths)
    cos_h, sin_h = _rope_tables(rng, 512, 128)
    cos, sin = gu.dev(cos_h), gu.dev(sin_h)
    qw = gu.dev(np.ones((NL, D), np.float16))
    kw = gu.dev(np.ones((NL, D), np.float16))
    q_raw = gu.dev(rng.standard_normal((NL, G, q_dim), dtype=np.float32).astype(np.float16))
    k_raw = gu.dev(rng.standard_normal((NL, G, kv_dim), dtype=np.float32).astype(np.float16))
    v = gu.dev(rng.standard_normal((NL, G, kv_dim), dtype=np.float32).astype(np.float16))
    out, out_rot = torch.empty_like(q_raw), torch.empty_like(q_raw)
    eng.decode_step_produce(q_raw, k_raw, v, out, qw, kw, cos, sin)
    eng.decode_step_produce(q_raw, k_raw, v, out_rot, qw, kw, cos, sin, rotated_output=True)  # same token again: idempotent append
    assert eng.status() == 0
    R = tq.ops.rotation_matrix().cuda().float()
    back = (out_rot.float().view(NL, G, H, D) @ R).view(NL, G, q_dim)  # out[d] = sum_k R[k][d] * acc[k]
    err = float((back - out.float()).abs().max())
    print(f"rotated output rotated back on the host: max-abs difference {err:.2e}")
    assert err <= 2e-3
    # o_proj with R^T folded into its weights: W' * acc == W * (R^T acc)
    rows = 96
    W = gu.dev((rng.standard_normal((rows, q_dim), dtype=np.float32) / np.sqrt(q_dim)).astype(np.float16))
    Wf = torch.empty_like(W)
    st = tq.lib().tq_fold_rotation_into_projection(Wf.data_ptr(), W.data_ptr(), tq.ops.rotation_matrix().cuda().data_ptr(), rows, H,
                                                   torch.cuda.current_stream().cuda_stream)
    assert st == 0
    y_ref = out.float().view(NL * G, q_dim) @ W.float().t()
    y_fold = out_rot.float().view(NL * G, q_dim) @ Wf.float().t()
    e2 = float((y_ref - y_fold).abs().max())
    print(f"o_proj through folded weights: max-abs difference {e2:.2e} (outputs of magnitude {float(y_ref.abs().max()):.2f})")
    assert e2 <= 3e-3
