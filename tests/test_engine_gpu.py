"""GPU tests of the engine handle (KV arena, slots, per-layer decode step, host-buffer step, CUDA graph replay)
and of the properties that hold at the benchmark's full size."""
import numpy as np
import pytest
import torch

import triebwerk_b200 as tq
from triebwerk_b200 import synth
from oracle import tqo
from tests import helpers as hp

pytestmark = pytest.mark.gpu
gu = pytest.importorskip("tests.gpu_util")


def test_c0_generation_loop_against_oracle():
    """The reference's CPU-runnable configuration: 16/8 heads, G=4, a 100-token prompt and decoded tokens up to
    context 612, kv_bits=4, one layer; every decode step is compared with the oracle run on its own cache."""
    H, Hkv, D, G, bits = 16, 8, 128, 4, 4
    prompt, new_tokens, msl = 100, 512, 640
    kv_dim, q_dim = Hkv * D, H * D
    rng = np.random.default_rng(0)
    scales = synth.channel_scales(kv_dim)
    R = tq.ops.rotation_matrix().numpy()
    eng = tq.Engine(msl, bits, num_layers=1, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(G, msl)
    ock, okn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    ocv, ovn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    # all G sequences share the prompt (GRPO rollouts of one prompt)
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
        if step % 8 == 0 or step == new_tokens - 1:  # the oracle is the slow side
            ref, _ = tqo.attention_batch(q, ock, ocv, okn, ovn, R, pos, msl, H, Hkv, D, bits)
            w, _ = hp.assert_attention_close(out, ref, H, D, f"step {step}")
            worst = max(worst, w)
    assert (eng.positions().numpy() == prompt + new_tokens).all()
    gk, gv, gkn, gvn = (gu.host(t) for t in eng.layer_cache(0))
    a = hp.unpack_codes(gk.reshape(G * msl, Hkv, -1), bits)
    b = hp.unpack_codes(ock.reshape(G * msl, Hkv, -1), bits)
    n_bad = int((a != b).sum())
    print(f"C0 loop: worst attention max-abs {worst:.2e}; {n_bad} of {G * (prompt + new_tokens) * Hkv * D} K coordinates differ from the oracle")
    assert n_bad <= 8
    assert np.abs(gkn.view(np.uint16).astype(np.int32) - okn.view(np.uint16).astype(np.int32)).max() <= 1


@pytest.mark.parametrize("bits", [4, 2, 0])
def test_ragged_slots_external_arena_and_host_step(bits):
    H, Hkv, D, NL = 32, 8, 128, 3
    kv_dim, q_dim = Hkv * D, H * D
    lengths = [130, 1, 64, 700, 33]
    caps = [n + 4 for n in lengths]
    G = len(lengths)
    rng = np.random.default_rng(1)
    R = tq.ops.rotation_matrix().numpy()
    eng = tq.Engine(1024, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    need = eng.arena_bytes(G, 1024, caps)
    assert need < eng.arena_bytes(G, 1024)
    arena = torch.empty(need + 4096, dtype=torch.uint8, device="cuda")
    canary = arena[need:]
    canary.fill_(0xA5)
    eng.set_arena(arena.data_ptr(), need, keep_alive=arena)
    eng.alloc_batch(G, 1024, caps)
    # an arena that is too small is refused, and caller memory is never replaced
    small = tq.Engine(1024, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    small.set_arena(arena.data_ptr(), 4096, keep_alive=arena)
    with pytest.raises(tq.TqError) as e:
        small.alloc_batch(G, 1024, caps)
    assert e.value.status == -2
    # fill the prompts, keep an oracle copy per sequence
    o = []
    for layer in range(NL):
        per_seq = []
        for g, n in enumerate(lengths):
            k = rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16)
            v = rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16)
            if n > 1:
                eng.prefill_append(layer, g, gu.dev(k[:-1]), gu.dev(v[:-1]), 0)
            per_seq.append((k, v))
        o.append(per_seq)
    with pytest.raises(tq.TqError):
        # sequence 1 has capacity 5 rows, rounded up to one 32-row tile: 40 tokens do not fit
        eng.prefill_append(0, 1, gu.dev(np.zeros((40, kv_dim), np.float16)), gu.dev(np.zeros((40, kv_dim), np.float16)), 0)
    with pytest.raises(tq.TqError):
        eng.set_positions([c for c in caps[:-1]] + [10 ** 6])
    eng.set_positions([n - 1 for n in lengths])
    # one decode step from host buffers: the last token of every sequence is appended by the step itself
    qh = torch.from_numpy(rng.standard_normal((NL, G, q_dim), dtype=np.float32).astype(np.float16)).pin_memory()
    kh = torch.from_numpy(np.stack([np.stack([o[l][g][0][-1] for g in range(G)]) for l in range(NL)])).pin_memory()
    vh = torch.from_numpy(np.stack([np.stack([o[l][g][1][-1] for g in range(G)]) for l in range(NL)])).pin_memory()
    outh = torch.empty(NL, G, q_dim, dtype=torch.float16).pin_memory()
    eng.decode_step_host(qh, kh, vh, outh)
    for layer in range(NL):
        for g, n in enumerate(lengths):
            k, v = o[layer][g]
            q = qh[layer, g].numpy()
            if bits == 0:
                ref, _ = tqo.fp16_attention_single(q, k, v, n - 1, n, H, Hkv, D)
            else:
                cq, cn = tqo.alloc_cache(1, n, Hkv, D, bits)
                vq, vn = tqo.alloc_cache(1, n, Hkv, D, bits)
                tqo.append_tokens(cq, cn, k, R, np.arange(n, dtype=np.int32), n, Hkv, D, bits)
                tqo.append_tokens(vq, vn, v, R, np.arange(n, dtype=np.int32), n, Hkv, D, bits)
                ref, _ = tqo.attention_single(q, cq, vq, cn, vn, R, n - 1, n, H, Hkv, D, bits)
            hp.assert_attention_close(outh[layer, g].numpy()[None], ref[None], H, D, f"bits={bits} layer {layer} seq {g}")
    torch.cuda.synchronize()
    assert (canary.cpu().numpy() == 0xA5).all(), "wrote past the end of the caller's arena"
    # sleep drops the arena, wake + alloc brings an internal one back
    eng.sleep()
    with pytest.raises(tq.TqError) as e:
        eng.alloc_batch(G, 64)
    assert e.value.status == -5
    eng.wake()
    eng.alloc_batch(2, 64)
    assert (eng.positions().numpy() == 0).all()
    eng.reset()


def test_graph_replay_equals_eager():
    """Append + attention + position increment captured once and replayed: the launch geometry does not depend
    on the (device-side) positions, as the reference's captured decode loop requires."""
    H, Hkv, D, G, bits, msl, steps = 16, 8, 128, 4, 4, 256, 48
    kv_dim, q_dim = Hkv * D, H * D
    rng = np.random.default_rng(2)
    ks = gu.dev(rng.standard_normal((steps, G, kv_dim), dtype=np.float32).astype(np.float16))
    vs = gu.dev(rng.standard_normal((steps, G, kv_dim), dtype=np.float32).astype(np.float16))
    qs = gu.dev(rng.standard_normal((steps, G, q_dim), dtype=np.float32).astype(np.float16))
    start = [0, 5, 40, 100]

    def run(use_graph):
        eng = tq.Engine(msl, bits, num_layers=1, num_heads=H, num_kv_heads=Hkv, head_dim=D)
        eng.alloc_batch(G, msl)
        eng.reset(zero_cache=True)
        eng.set_positions(start)
        k, v, q = torch.empty_like(ks[0]), torch.empty_like(vs[0]), torch.empty_like(qs[0])
        out = torch.empty_like(q)
        outs = []
        side = torch.cuda.Stream()
        graph = None
        if use_graph:
            k.copy_(ks[0]); v.copy_(vs[0]); q.copy_(qs[0])
            torch.cuda.synchronize()
            # warm-up outside the capture (module load, attribute set), then rewind the positions
            eng.decode_layer(0, q, k, v, out)
            eng.set_positions(start)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                eng.decode_layer(0, q, k, v, out)
                eng.advance()
        for s in range(steps):
            k.copy_(ks[s]); v.copy_(vs[s]); q.copy_(qs[s])
            if use_graph:
                graph.replay()
            else:
                eng.decode_layer(0, q, k, v, out)
                eng.advance()
            torch.cuda.synchronize()
            outs.append(out.clone())
        cache = [t.clone() for t in eng.layer_cache(0)]
        return torch.stack(outs), cache, eng.positions()

    o_e, c_e, p_e = run(False)
    o_g, c_g, p_g = run(True)
    assert (p_e == p_g).all() and (p_e.numpy() == np.array(start) + steps).all()
    for a, b in zip(c_e, c_g):
        assert torch.equal(a, b), "cache bytes differ between eager and graph replay"
    assert torch.equal(o_e.view(torch.int16), o_g.view(torch.int16)), "outputs differ between eager and graph replay"


def test_full_size_layer_properties():
    """One layer at the benchmark's size (64 sequences x 4096 tokens, 4-bit): sequences come in groups of four
    identical rollouts -> outputs identical within a group; two sampled sequences are checked against the oracle;
    appending the same token twice is idempotent."""
    H, Hkv, D, G, bits, msl = 16, 8, 128, 64, 4, 4096
    kv_dim, q_dim = Hkv * D, H * D
    L = 4096
    R = tq.ops.rotation_matrix().numpy()
    eng = tq.Engine(msl, bits, num_layers=1, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(G, msl)
    gen = torch.Generator(device="cuda").manual_seed(0)
    scales = torch.from_numpy(synth.channel_scales(kv_dim)).cuda()
    keep = {}
    for p in range(G // 4):
        k, v = synth.torch_kv(gen, L - 1, kv_dim, scales)
        for j in range(4):
            eng.prefill_append(0, 4 * p + j, k, v, 0)
        if p in (0, 9):
            keep[p] = (gu.host(k), gu.host(v))
    eng.set_positions([L - 1] * G)
    k_new, v_new = synth.torch_kv(gen, G // 4, kv_dim, scales)
    k_new, v_new = k_new.repeat_interleave(4, 0).contiguous(), v_new.repeat_interleave(4, 0).contiguous()
    q = torch.randn(G // 4, q_dim, generator=gen, device="cuda").to(torch.float16).repeat_interleave(4, 0).contiguous()
    out = gu.host(eng.decode_layer(0, q, k_new, v_new))
    cache1 = [t.clone() for t in eng.layer_cache(0)]
    out2 = gu.host(eng.decode_layer(0, q, k_new, v_new))  # same token at the same position again
    for a, b in zip(cache1, eng.layer_cache(0)):
        assert torch.equal(a, b), "re-appending the same token changed the cache"
    assert (out.view(np.uint16) == out2.view(np.uint16)).all()
    # The four rollouts of a prompt hold the same bytes but sit at different places of the flat tile list, so
    # their split-K partial sums are cut at different tokens: equal up to fp32 summation order, not bitwise.
    o4 = out.reshape(G // 4, 4, q_dim).astype(np.float32)
    spread = float(np.abs(o4 - o4[:, :1]).max())
    print(f"identical rollouts: largest difference between their outputs {spread:.2e}")
    assert spread <= 5e-4, "identical rollouts gave different outputs"
    for p, (kh, vh) in keep.items():
        g = 4 * p
        kk = np.concatenate([kh, gu.host(k_new[g:g + 1])])
        vv = np.concatenate([vh, gu.host(v_new[g:g + 1])])
        cq, cn = tqo.alloc_cache(1, L, Hkv, D, bits)
        vq, vn = tqo.alloc_cache(1, L, Hkv, D, bits)
        tqo.append_tokens(cq, cn, kk, R, np.arange(L, dtype=np.int32), L, Hkv, D, bits)
        tqo.append_tokens(vq, vn, vv, R, np.arange(L, dtype=np.int32), L, Hkv, D, bits)
        ref, _ = tqo.attention_single(gu.host(q[g]), cq, vq, cn, vn, R, L - 1, L, H, Hkv, D, bits)
        w, r = hp.assert_attention_close(out[g][None], ref[None], H, D, f"full-size sequence {g}")
        print(f"full-size sequence {g}: max-abs {w:.2e}, rel {r:.2e}")


@pytest.mark.parametrize("bits,H,Hkv", [(4, 16, 8), (2, 32, 8), (4, 16, 4)])
def test_fused_and_two_launch_forms_store_the_same_bytes(bits, H, Hkv):
    """One launch per layer-step (append + query rotation + attention in the attention kernel) against the
    two-launch form on the same ragged batch: identical cache bytes and norms after every step, outputs equal up
    to the order of the fp32 sums (the query rotation runs on the tensor cores in one form, as an fp32 chain in
    the other).  Several steps, so that new tokens cross tile boundaries and land in freshly started tiles."""
    D, NL = 128, 2
    kv_dim, q_dim = Hkv * D, H * D
    lengths = [130, 1, 31, 700, 33, 256, 95]
    G = len(lengths)
    steps = 4
    caps = [n + steps + 1 for n in lengths]
    rng = np.random.default_rng(7)
    engines = []
    for fused in (True, False):
        eng = tq.Engine(1024, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
        eng.alloc_batch(G, 1024, caps)
        assert eng.set_fused(fused) in (True, False)
        engines.append(eng)
    for layer in range(NL):
        for g, n in enumerate(lengths):
            k = gu.dev(rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16))
            v = gu.dev(rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16))
            for eng in engines:
                eng.prefill_append(layer, g, k, v, 0)
    for eng in engines:
        eng.set_positions(lengths)
    for step in range(steps):
        q = torch.from_numpy(rng.standard_normal((NL, G, q_dim), dtype=np.float32).astype(np.float16)).cuda()
        k = torch.from_numpy(rng.standard_normal((NL, G, kv_dim), dtype=np.float32).astype(np.float16)).cuda()
        v = torch.from_numpy(rng.standard_normal((NL, G, kv_dim), dtype=np.float32).astype(np.float16)).cuda()
        outs = []
        for eng in engines:
            out = torch.empty_like(q)
            eng.decode_step(q, k, v, out)
            outs.append(out.cpu().numpy())
            assert eng.status() == 0
        for layer in range(NL):
            a, b = engines[0].layer_cache(layer), engines[1].layer_cache(layer)
            for x, y, name in zip(a, b, ("k codes", "v codes", "k norms", "v norms")):
                assert torch.equal(x.view(torch.uint8), y.view(torch.uint8)), f"step {step} layer {layer}: {name} differ"
        hp.assert_attention_close(outs[0].reshape(NL * G, q_dim), outs[1].reshape(NL * G, q_dim), H, D,
                                  f"bits={bits} step {step}: fused against two-launch")
        for eng in engines:
            eng.advance()


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("bits", [4, 2])
def test_four_kv_heads_long_context_against_oracle(bits, fused):
    """4 KV heads make the stages small enough for a ring of four, and a context long enough that every worker
    streams several tiles walks that whole ring (stage addresses, parities, swizzle alignment of every stage)."""
    H, Hkv, D = 16, 4, 128
    kv_dim, q_dim = Hkv * D, H * D
    n, msl = 12000, 12032
    rng = np.random.default_rng(11)
    R = tq.ops.rotation_matrix().numpy()
    eng = tq.Engine(msl, bits, num_layers=1, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(1, msl)
    eng.set_fused(fused)
    k = rng.standard_normal((n + 1, kv_dim), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((n + 1, kv_dim), dtype=np.float32).astype(np.float16)
    q = rng.standard_normal((1, 1, q_dim), dtype=np.float32).astype(np.float16)
    eng.prefill_append(0, 0, gu.dev(k[:-1]), gu.dev(v[:-1]), 0)
    eng.set_positions([n])
    out = torch.empty(1, 1, q_dim, dtype=torch.float16, device="cuda")
    eng.decode_step(gu.dev(q), gu.dev(k[-1:].reshape(1, 1, kv_dim)), gu.dev(v[-1:].reshape(1, 1, kv_dim)), out)
    assert eng.status() == 0
    cq, cn = tqo.alloc_cache(1, n + 1, Hkv, D, bits)
    vq, vn = tqo.alloc_cache(1, n + 1, Hkv, D, bits)
    tqo.append_tokens(cq, cn, k, R, np.arange(n + 1, dtype=np.int32), n + 1, Hkv, D, bits)
    tqo.append_tokens(vq, vn, v, R, np.arange(n + 1, dtype=np.int32), n + 1, Hkv, D, bits)
    ref, _ = tqo.attention_single(q[0, 0], cq, vq, cn, vn, R, n, n + 1, H, Hkv, D, bits)
    hp.assert_attention_close(out.cpu().numpy().reshape(1, q_dim), ref[None], H, D, f"bits={bits} fused={fused}")


@pytest.mark.parametrize("bits,form", [(4, "whole-step"), (4, "one-launch"), (2, "two-launch"), (0, "fp16")])
def test_position_past_its_own_slot_is_refused(bits, form, monkeypatch):
    """Ragged slots of 32 and 64 rows: sequence 0 is advanced to position 32, one row past ITS slot (which would be row
    0 of sequence 1's slot).  The append must skip it, raise status 3 and leave sequence 1's rows as they were."""
    H, Hkv, D, NL = 16, 8, 128, 2
    kv_dim, q_dim = Hkv * D, H * D
    rng = np.random.default_rng(21)
    eng = tq.Engine(64, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(2, 64, [32, 64])
    eng.set_fused(form != "two-launch")
    for layer in range(NL):
        for g, n in enumerate((32, 40)):
            k = gu.dev(rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16))
            v = gu.dev(rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16))
            eng.prefill_append(layer, g, k, v, 0)
    eng.set_positions([31, 40])
    eng.advance()  # sequence 0 -> 32 = its capacity, sequence 1 -> 41
    assert eng.positions().tolist() == [32, 41]
    before = [[t.clone() for t in eng.layer_cache(layer) if t is not None] for layer in range(NL)]
    q = gu.dev(rng.standard_normal((NL, 2, q_dim), dtype=np.float32).astype(np.float16))
    k = gu.dev(rng.standard_normal((NL, 2, kv_dim), dtype=np.float32).astype(np.float16))
    v = gu.dev(rng.standard_normal((NL, 2, kv_dim), dtype=np.float32).astype(np.float16))
    out = torch.empty_like(q)
    if form == "one-launch":
        for layer in range(NL):
            eng.decode_layer(layer, q[layer], k[layer], v[layer], out[layer])
    else:
        eng.decode_step(q, k, v, out)
    assert eng.status() == 3
    for layer in range(NL):
        after = [t for t in eng.layer_cache(layer) if t is not None]
        for a, b in zip(before[layer], after):
            # rows 32 .. 72 are sequence 1's written rows (its slot starts at row 32); row 32 + 41 is its new token
            assert torch.equal(a[32:32 + 41].view(torch.uint8), b[32:32 + 41].view(torch.uint8)), "a neighbour's rows changed"
            assert not torch.equal(a[32 + 41].view(torch.uint8), b[32 + 41].view(torch.uint8)), "sequence 1's own token is missing"


def test_bounded_wait_gives_up_with_status_1():
    """A copy barrier armed for bytes that never arrive: the bounded wait runs out, the kernel reports status 1
    (a wait on a copy barrier gave up) and exits normally; the context stays usable."""
    word = torch.zeros(64, dtype=torch.int32, device="cuda")
    st = tq.lib().tq_selftest_bounded_wait(word.data_ptr(), 2000, torch.cuda.current_stream().cuda_stream)
    assert st == 1
    assert int(word[0].item()) == 0  # read and cleared
    x = torch.arange(8, device="cuda").sum().item()  # the context still works
    assert x == 28


@pytest.mark.parametrize("bits", [4, 0])
def test_sleep_keep_wake_and_sequence_blobs(bits):
    """Cache persistence: sleep_keep() + wake() bring back every sequence's rows and positions, and a decode step
    afterwards gives the bytes and outputs of an engine that never slept; a sequence exported as a blob and imported
    into another engine's slot continues there."""
    H, Hkv, D, NL = 16, 8, 128, 2
    kv_dim, q_dim = Hkv * D, H * D
    lengths = [70, 5, 33]
    caps = [96, 32, 64]
    rng = np.random.default_rng(31)
    engines = [tq.Engine(128, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D) for _ in range(2)]
    for eng in engines:
        eng.alloc_batch(3, 128, caps)
    for layer in range(NL):
        for g, n in enumerate(lengths):
            k = gu.dev(rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16))
            v = gu.dev(rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16))
            for eng in engines:
                eng.prefill_append(layer, g, k, v, 0)
    for eng in engines:
        eng.set_positions(lengths)
    a, b = engines
    blob1 = a.export_sequence(1, lengths[1])
    a.sleep_keep()
    with pytest.raises(tq.TqError):
        a.decode_layer(0, torch.zeros(3, q_dim, dtype=torch.float16, device="cuda"), torch.zeros(3, kv_dim, dtype=torch.float16, device="cuda"),
                       torch.zeros(3, kv_dim, dtype=torch.float16, device="cuda"))
    a.wake()
    a.G = 3
    assert a.positions().tolist() == lengths
    q = gu.dev(rng.standard_normal((NL, 3, q_dim), dtype=np.float32).astype(np.float16))
    k = gu.dev(rng.standard_normal((NL, 3, kv_dim), dtype=np.float32).astype(np.float16))
    v = gu.dev(rng.standard_normal((NL, 3, kv_dim), dtype=np.float32).astype(np.float16))
    outs = []
    for eng in engines:
        out = torch.empty_like(q)
        eng.decode_step(q, k, v, out)
        assert eng.status() == 0
        outs.append(out)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16)), "outputs differ after sleep_keep + wake"
    for layer in range(NL):
        for x, y in zip(a.layer_cache(layer), b.layer_cache(layer)):
            if x is None:
                continue
            base = 0
            for g, n in enumerate(lengths):  # rows 0 .. n of every slot (n = the token the step appended)
                assert torch.equal(x[base:base + n + 1].view(torch.uint8), y[base:base + n + 1].view(torch.uint8))
                base += caps[g]
    # a blob moves a sequence into another slot of another engine: sequence 1 of `a` (before the step) into slot 2 of a new one
    c = tq.Engine(128, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    c.alloc_batch(3, 128)
    c.import_sequence(2, blob1)
    assert c.positions().tolist()[2] == lengths[1]
    assert c.export_sequence(2, lengths[1]) == blob1
    other = tq.Engine(128, 2 if bits != 2 else 4, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    other.alloc_batch(1, 128)
    with pytest.raises(tq.TqError) as e:
        other.import_sequence(0, blob1)
    assert e.value.status == -4


@pytest.mark.parametrize("bits,form", [(4, "whole-step"), (4, "one-launch"), (2, "two-launch")])
def test_shared_prefix_equals_replicated_prompt(bits, form):
    """Four rollouts of one 100-token prompt (twice: eight sequences): with prefill_shared the prompt's whole tiles are
    stored once and read by all four; against an engine that holds the prompt four times, the sequences' own rows are
    byte-equal after every step and the outputs agree to the order of the split-K sums."""
    H, Hkv, D, NL = 16, 8, 128, 2
    kv_dim, q_dim = Hkv * D, H * D
    prompt, steps, G = 100, 40, 8
    P = prompt // 32 * 32
    rng = np.random.default_rng(41)
    shared = tq.Engine(256, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    plain = tq.Engine(256, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    # followers only need rows for their own tokens: the prompt's remainder and the decoded ones
    caps = [prompt + steps + 1 if g % 4 == 0 else prompt - P + steps + 1 for g in range(G)]
    shared.alloc_batch(G, 256, caps)
    plain.alloc_batch(G, 256)
    assert shared.arena_bytes(G, 256, caps) < plain.arena_bytes(G, 256, [prompt + steps + 1] * G)
    for eng in (shared, plain):
        eng.set_fused(form != "two-launch")
    for layer in range(NL):
        for g0 in (0, 4):
            k = gu.dev(rng.standard_normal((prompt, kv_dim), dtype=np.float32).astype(np.float16))
            v = gu.dev(rng.standard_normal((prompt, kv_dim), dtype=np.float32).astype(np.float16))
            shared.prefill_shared(layer, g0, 4, k, v)
            for g in range(g0, g0 + 4):
                plain.prefill_append(layer, g, k, v, 0)
    for eng in (shared, plain):
        eng.set_positions([prompt] * G)
    with pytest.raises(tq.TqError):
        shared.prefill_append(0, 1, gu.dev(np.zeros((4, kv_dim), np.float16)), gu.dev(np.zeros((4, kv_dim), np.float16)), 0)
    worst = 0.0
    for step in range(steps):
        q = gu.dev(rng.standard_normal((NL, G, q_dim), dtype=np.float32).astype(np.float16))
        k = gu.dev(rng.standard_normal((NL, G, kv_dim), dtype=np.float32).astype(np.float16))
        v = gu.dev(rng.standard_normal((NL, G, kv_dim), dtype=np.float32).astype(np.float16))
        outs = []
        for eng in (shared, plain):
            out = torch.empty_like(q)
            if form == "one-launch":
                for layer in range(NL):
                    eng.decode_layer(layer, q[layer], k[layer], v[layer], out[layer])
            else:
                eng.decode_step(q, k, v, out)
            assert eng.status() == 0
            eng.advance()
            outs.append(out.float())
        worst = max(worst, float((outs[0] - outs[1]).abs().max()))
    assert worst <= 5e-4, f"shared-prefix outputs differ from the replicated batch by {worst:.2e}"
    # own rows: sequence g of the shared engine holds tokens P.. (followers) or 0.. (owners) in its slot
    n_own = prompt + steps
    for layer in range(NL):
        base = 0
        for g in range(G):
            first = 0 if g % 4 == 0 else P
            for x, y in zip(shared.layer_cache(layer), plain.layer_cache(layer)):
                a = x[base:base + n_own - first]
                b = y[g * 256 + first:g * 256 + n_own]
                assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), f"layer {layer} sequence {g}: own rows differ"
            base += (caps[g] + 31) // 32 * 32
    # a follower exported as a blob carries its whole context, prefix included
    blob_s = shared.export_sequence(5, n_own)
    blob_p = plain.export_sequence(5, n_own)
    assert blob_s == blob_p
    print(f"shared prefix ({form}, {bits}-bit): largest output difference {worst:.2e}")


def test_attention_launch_timing_leaves_results_unchanged():
    """tq_engine_time_attention records events around the attention launch of the whole-step call: the reported time is
    positive and below the wall time of the step, the results are the same bits as without it, and switching it off
    makes the query an error."""
    import time
    H, Hkv, D, G, bits, msl, NL = 16, 8, 128, 8, 4, 512, 3
    kv_dim, q_dim = Hkv * D, H * D
    eng = tq.Engine(msl, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(G, msl)
    gen = torch.Generator(device="cuda").manual_seed(3)
    scales = torch.from_numpy(synth.channel_scales(kv_dim)).cuda()
    for layer in range(NL):
        for g in range(G):
            k, v = synth.torch_kv(gen, 300 + 7 * g, kv_dim, scales)
            eng.prefill_append(layer, g, k, v, 0)
    eng.set_positions([300 + 7 * g for g in range(G)])
    q = torch.randn(NL, G, q_dim, generator=gen, device="cuda").to(torch.float16)
    k = torch.randn(NL, G, kv_dim, generator=gen, device="cuda").to(torch.float16)
    v = torch.randn(NL, G, kv_dim, generator=gen, device="cuda").to(torch.float16)
    out_a, out_b = torch.empty_like(q), torch.empty_like(q)
    eng.decode_step(q, k, v, out_a)
    torch.cuda.synchronize()
    eng.time_attention(True)
    t0 = time.perf_counter()
    eng.decode_step(q, k, v, out_b)   # the same token at the same positions again
    ms = eng.last_attention_ms()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    assert 0.0 < ms < wall_ms
    assert torch.equal(out_a, out_b)
    eng.time_attention(False)
    with pytest.raises(Exception):
        eng.last_attention_ms()
    assert eng.status() == 0


@pytest.mark.parametrize("bits", [4, 2, 0])
def test_prefill_layer_of_a_prompt_against_oracle(bits):
    """tq_engine_prefill_layer: the cache write of a prompt and its causal self-attention (reference
    engine/engine.cpp:2110-2146) for the second sequence of a ragged batch, with the query and output stride of a gated
    model (twice the query width, the gate columns untouched)."""
    H, Hkv, D, NL = 16, 8, 128, 2
    kv_dim, q_dim = Hkv * D, H * D
    caps = [64, 224, 96]
    T = 200
    rng = np.random.default_rng(800 + bits)
    R, _ = tqo.rotation()
    eng = tq.Engine(256, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(3, 256, caps)
    k = rng.standard_normal((T, kv_dim), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((T, kv_dim), dtype=np.float32).astype(np.float16)
    q2 = rng.standard_normal((T, 2 * q_dim), dtype=np.float32).astype(np.float16)
    out = torch.full((T, 2 * q_dim), 7.0, dtype=torch.float16, device="cuda")
    eng.prefill_layer(1, 1, gu.dev(q2), gu.dev(k), gu.dev(v), out)
    got = gu.host(out)
    assert (got[:, q_dim:] == np.float16(7.0)).all(), "columns past the query heads were written"
    msl = caps[1]
    if bits == 0:
        ref = np.stack([tqo.fp16_attention_single(q2[t, :q_dim], np.pad(k, ((0, msl - T), (0, 0))), np.pad(v, ((0, msl - T), (0, 0))),
                                                  t, msl, H, Hkv, D)[0] for t in range(T)])
    else:
        ck, kn = tqo.alloc_cache(1, msl, Hkv, D, bits)
        cv, vn = tqo.alloc_cache(1, msl, Hkv, D, bits)
        pos = np.arange(T, dtype=np.int32)
        tqo.append_tokens(ck, kn, k, R, pos, msl, Hkv, D, bits)
        tqo.append_tokens(cv, vn, v, R, pos, msl, Hkv, D, bits)
        ref, _ = tqo.prefill_attention(np.ascontiguousarray(q2[:, :q_dim]), ck, cv, kn, vn, R, msl, H, Hkv, D, bits)
    w, r = hp.assert_attention_close(got[:, :q_dim], ref, H, D, f"prefill layer kv_bits={bits}")
    print(f"prefill layer kv_bits={bits}: max-abs {w:.2e}, rel {r:.2e}")
    # the neighbours' slots are untouched, and a prompt longer than the slot is refused before anything runs
    assert eng.status() == 0
    with pytest.raises(Exception):
        eng.prefill_layer(0, 0, gu.dev(q2), gu.dev(k), gu.dev(v), out)   # T = 200 > 64 rows


@pytest.mark.parametrize("bits", [4, 0])
def test_prefill_layer_batch_equals_prompt_by_prompt(bits):
    """Several prompts in one launch give the bits that the same prompts give one at a time, in dense and in ragged
    slots, and the first of them agrees with the oracle."""
    H, Hkv, D, NL, T, n = 16, 8, 128, 1, 130, 3
    kv_dim, q_dim = Hkv * D, H * D
    rng = np.random.default_rng(900 + bits)
    k = rng.standard_normal((n, T, kv_dim), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((n, T, kv_dim), dtype=np.float32).astype(np.float16)
    q = rng.standard_normal((n, T, q_dim), dtype=np.float32).astype(np.float16)
    for caps in (None, [160, 256, 192, 64]):
        eng = tq.Engine(256, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
        eng.alloc_batch(4, 256, caps)
        together = gu.host(eng.prefill_layer_batch(0, 0, gu.dev(q), gu.dev(k), gu.dev(v)))
        caches_a = [t.clone() for t in eng.layer_cache(0) if t is not None]
        eng.reset()
        single = np.stack([gu.host(eng.prefill_layer(0, i, gu.dev(q[i]), gu.dev(k[i]), gu.dev(v[i]))) for i in range(n)])
        assert (together.view(np.uint16) == single.view(np.uint16)).all()
        for a, b in zip(caches_a, [t for t in eng.layer_cache(0) if t is not None]):
            assert torch.equal(a, b)
        assert eng.status() == 0
    if bits == 4:
        R, _ = tqo.rotation()
        msl = 160
        ck, kn = tqo.alloc_cache(1, msl, Hkv, D, bits)
        cv, vn = tqo.alloc_cache(1, msl, Hkv, D, bits)
        pos = np.arange(T, dtype=np.int32)
        tqo.append_tokens(ck, kn, k[0], R, pos, msl, Hkv, D, bits)
        tqo.append_tokens(cv, vn, v[0], R, pos, msl, Hkv, D, bits)
        ref, _ = tqo.prefill_attention(q[0], ck, cv, kn, vn, R, msl, H, Hkv, D, bits)
        hp.assert_attention_close(together[0], ref, H, D, "first prompt of the batch")


def test_step_in_two_phases_equals_the_whole_step():
    """tq_engine_step_prepare + tq_engine_step_attend_layers over groups of layers give the bits (outputs and cache) of
    tq_engine_decode_step."""
    H, Hkv, D, G, bits, msl, NL = 16, 8, 128, 6, 4, 384, 5
    kv_dim, q_dim = Hkv * D, H * D
    gen = torch.Generator(device="cuda").manual_seed(11)
    scales = torch.from_numpy(synth.channel_scales(kv_dim)).cuda()
    prompts = [[synth.torch_kv(gen, 200 + 9 * g, kv_dim, scales) for g in range(G)] for _ in range(NL)]
    q = torch.randn(NL, G, q_dim, generator=gen, device="cuda").to(torch.float16)
    k = torch.randn(NL, G, kv_dim, generator=gen, device="cuda").to(torch.float16)
    v = torch.randn(NL, G, kv_dim, generator=gen, device="cuda").to(torch.float16)
    outs, caches = [], []
    for split in (False, True):
        eng = tq.Engine(msl, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
        eng.alloc_batch(G, msl)
        for layer in range(NL):
            for g in range(G):
                eng.prefill_append(layer, g, prompts[layer][g][0], prompts[layer][g][1], 0)
        eng.set_positions([200 + 9 * g for g in range(G)])
        out = torch.zeros_like(q)
        if split:
            assert eng.step_prepare(q, k, v)
            for l0, n in ((0, 2), (2, 2), (4, 1)):
                eng.step_attend_layers(l0, n, out)
        else:
            eng.decode_step(q, k, v, out)
        torch.cuda.synchronize()
        assert eng.status() == 0
        outs.append(out)
        caches.append([[t.clone() for t in eng.layer_cache(layer)] for layer in range(NL)])
    assert torch.equal(outs[0], outs[1])
    for la, lb in zip(*caches):
        for a, b in zip(la, lb):
            assert torch.equal(a, b)
