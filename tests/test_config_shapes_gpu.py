"""GPU parity at the shapes of the larger benchmark configurations, against the CPU oracle:

* config 3's shape: kv_bits=2, 32 query / 8 KV heads, sequences of 8192 tokens, a whole decode step through
  ``tq_engine_decode_step`` in the one-launch and in the two-launch form;
* config 4's shape: 32/8 heads, per-sequence (ragged) slots with contexts between 1 and 16384 tokens, kv_bits 4 and
  kv_bits 0 (the fp16 twin);
* configuration 0's generation loop at kv_bits=2 (``tests/test_engine_gpu.py`` runs it at kv_bits=4).

Every case also reports the error of the fp32 results before their final rounding to fp16, next to the fp16 one.
"""
import numpy as np
import pytest
import torch

import triebwerk_b200 as tq
from triebwerk_b200 import synth
from oracle import tqo
from tests import helpers as hp

pytestmark = pytest.mark.gpu
gu = pytest.importorskip("tests.gpu_util")

D = 128


def _oracle_single(q, k, v, R, H, Hkv, bits):
    """Oracle attention of one sequence whose tokens k, v [n, kv_dim] are all in the cache (the last one being the
    step's new token).  Returns (out fp16, out fp32)."""
    n = k.shape[0]
    if bits == 0:
        return tqo.fp16_attention_single(q, k, v, n - 1, n, H, Hkv, D)
    cq, cn = tqo.alloc_cache(1, n, Hkv, D, bits)
    vq, vn = tqo.alloc_cache(1, n, Hkv, D, bits)
    pos = np.arange(n, dtype=np.int32)
    tqo.append_tokens(cq, cn, k, R, pos, n, Hkv, D, bits)
    tqo.append_tokens(vq, vn, v, R, pos, n, Hkv, D, bits)
    return tqo.attention_single(q, cq, vq, cn, vn, R, n - 1, n, H, Hkv, D, bits)


@pytest.mark.parametrize("fused", [True, False])
def test_config3_shape_two_bit_32_heads_8192_tokens(fused):
    H, Hkv, bits, G, L, NL = 32, 8, 2, 8, 8192, 2
    kv_dim, q_dim = Hkv * D, H * D
    R = tq.ops.rotation_matrix().numpy()
    eng = tq.Engine(L, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(G, L)
    eng.set_fused(fused)
    gen = torch.Generator(device="cuda").manual_seed(3)
    scales = torch.from_numpy(synth.channel_scales(kv_dim)).cuda()
    sampled = {(0, 1), (1, 6)}  # (layer, sequence) pairs that go to the oracle
    keep = {}
    for layer in range(NL):
        for g in range(G):
            k, v = synth.torch_kv(gen, L - 1, kv_dim, scales)
            eng.prefill_append(layer, g, k, v, 0)
            if (layer, g) in sampled:
                keep[(layer, g)] = (gu.host(k), gu.host(v))
    eng.set_positions([L - 1] * G)
    k_new = torch.stack([synth.torch_kv(gen, G, kv_dim, scales)[0] for _ in range(NL)])
    v_new = torch.randn(NL, G, kv_dim, generator=gen, device="cuda").to(torch.float16)
    q = torch.randn(NL, G, q_dim, generator=gen, device="cuda").to(torch.float16)
    out = torch.empty_like(q)
    eng.enable_output_f32()
    eng.decode_step(q, k_new, v_new, out)
    assert eng.status() == 0
    out_f32 = eng.last_output_f32(NL)
    out = gu.host(out)
    for (layer, g), (kh, vh) in keep.items():
        kk = np.concatenate([kh, gu.host(k_new[layer, g:g + 1])])
        vv = np.concatenate([vh, gu.host(v_new[layer, g:g + 1])])
        ref, ref32 = _oracle_single(gu.host(q[layer, g]), kk, vv, R, H, Hkv, bits)
        w, r = hp.assert_attention_close(out[layer, g][None], ref[None], H, D, f"config-3 shape layer {layer} seq {g} fused={fused}")
        print(f"config-3 shape (2-bit, 32/8 heads, L={L}) layer {layer} seq {g} fused={fused}: fp16 max-abs {w:.2e}, rel {r:.2e}")
        if out_f32 is not None:
            e32 = float(np.abs(out_f32[layer, g].reshape(H, D) - ref32).max())
            print(f"  before the fp16 rounding: max-abs {e32:.2e}")
            assert e32 <= hp.ATTN_ABS


@pytest.mark.parametrize("bits", [4, 0])
def test_config4_shape_ragged_slots_up_to_16384(bits):
    H, Hkv, NL = 32, 8, 1
    kv_dim, q_dim = Hkv * D, H * D
    lengths = [128, 4097, 16384, 1, 33, 8000, 16383, 2049]
    G = len(lengths)
    R = tq.ops.rotation_matrix().numpy()
    eng = tq.Engine(16384, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(G, 16384, lengths)
    rng = np.random.default_rng(4)
    scales = synth.channel_scales(kv_dim)
    seqs = []
    for g, n in enumerate(lengths):
        k, v = synth.kv_batch(rng, n, kv_dim, scales)
        if n > 1:
            eng.prefill_append(0, g, gu.dev(k[:-1]), gu.dev(v[:-1]), 0)
        seqs.append((k, v))
    eng.set_positions([n - 1 for n in lengths])
    q = synth.q_batch(rng, G, q_dim)
    k_new = np.stack([s[0][-1] for s in seqs])
    v_new = np.stack([s[1][-1] for s in seqs])
    if bits != 0:
        eng.enable_output_f32()
    out = gu.host(eng.decode_layer(0, gu.dev(q), gu.dev(k_new), gu.dev(v_new)))
    assert eng.status() == 0
    out_f32 = eng.last_output_f32(1)[0] if bits != 0 else None
    worst = worst32 = 0.0
    for g, (k, v) in enumerate(seqs):
        ref, ref32 = _oracle_single(q[g], k, v, R, H, Hkv, bits)
        w, _ = hp.assert_attention_close(out[g][None], ref[None], H, D, f"config-4 shape bits={bits} seq {g} (L={lengths[g]})")
        worst = max(worst, w)
        if out_f32 is not None:
            worst32 = max(worst32, float(np.abs(out_f32[g].reshape(H, D) - ref32).max()))
    print(f"config-4 shape (32/8 heads, ragged 1..16384, kv_bits={bits}): worst fp16 max-abs {worst:.2e}"
          + (f"; before the fp16 rounding {worst32:.2e}" if out_f32 is not None else ""))
    if out_f32 is not None:
        assert worst32 <= hp.ATTN_ABS


def test_c0_generation_loop_two_bit():
    """Configuration 0's loop (16/8 heads, G=4, 100-token prompt + 512 decoded tokens) at kv_bits=2."""
    H, Hkv, G, bits = 16, 8, 4, 2
    prompt, new_tokens, msl = 100, 512, 640
    kv_dim, q_dim = Hkv * D, H * D
    rng = np.random.default_rng(0)
    scales = synth.channel_scales(kv_dim)
    R = tq.ops.rotation_matrix().numpy()
    eng = tq.Engine(msl, bits, num_layers=1, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(G, msl)
    ock, okn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    ocv, ovn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    k, v = synth.kv_batch(rng, prompt, kv_dim, scales)
    for g in range(G):
        eng.prefill_append(0, g, gu.dev(k), gu.dev(v), 0)
        tqo.append_tokens(ock[g * msl:], okn[g * msl:], k, R, np.arange(prompt, dtype=np.int32), msl, Hkv, D, bits)
        tqo.append_tokens(ocv[g * msl:], ovn[g * msl:], v, R, np.arange(prompt, dtype=np.int32), msl, Hkv, D, bits)
    eng.set_positions([prompt] * G)
    worst = 0.0
    for step in range(new_tokens):
        pos = np.full(G, prompt + step, np.int32)
        k, v = synth.kv_batch(rng, G, kv_dim, scales)
        q = synth.q_batch(rng, G, q_dim)
        out = gu.host(eng.decode_layer(0, gu.dev(q), gu.dev(k), gu.dev(v)))
        eng.advance()
        tqo.append_batch(ock, okn, k, R, pos, msl, Hkv, D, bits)
        tqo.append_batch(ocv, ovn, v, R, pos, msl, Hkv, D, bits)
        if step % 8 == 0 or step == new_tokens - 1:
            ref, _ = tqo.attention_batch(q, ock, ocv, okn, ovn, R, pos, msl, H, Hkv, D, bits)
            w, _ = hp.assert_attention_close(out, ref, H, D, f"2-bit step {step}")
            worst = max(worst, w)
    assert eng.status() == 0
    gk, gv, gkn, gvn = (gu.host(t) for t in eng.layer_cache(0))
    for got, want, name in ((gk, ock, "K"), (gv, ocv, "V")):
        a = hp.unpack_codes(got.reshape(G * msl, Hkv, -1), bits)
        b = hp.unpack_codes(want.reshape(G * msl, Hkv, -1), bits)
        n_bad = int((a != b).sum())
        print(f"C0 loop at 2-bit: {n_bad} of {G * (prompt + new_tokens) * Hkv * D} {name} coordinates differ from the oracle")
        assert n_bad <= 8
    assert np.abs(gkn.view(np.uint16).astype(np.int32) - okn.view(np.uint16).astype(np.int32)).max() <= 1
    assert np.abs(gvn.view(np.uint16).astype(np.int32) - ovn.view(np.uint16).astype(np.int32)).max() <= 1
    print(f"C0 loop at 2-bit: worst attention max-abs {worst:.2e}")
