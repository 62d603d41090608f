"""CPU tests of the oracle itself: tables, quantiser, packing, rotation generator, self-consistency, and -- when
the fixtures exist -- agreement with the outputs of the reference's own kernels (tests/golden/*.npz)."""
import numpy as np
import pytest

from oracle import tqo
from tests import helpers as hp


def test_tables_monotone_and_symmetric():
    for bits in (2, 4):
        cent, bnd = tqo.tables(bits)
        assert (np.diff(cent) > 0).all() and (np.diff(bnd) > 0).all()
        assert np.allclose(cent, -cent[::-1]) and np.allclose(bnd, -bnd[::-1])
        # a Lloyd-Max bound is the midpoint of its neighbouring centroids (tables are 5-decimal literals)
        assert np.abs(bnd - 0.5 * (cent[:-1] + cent[1:])).max() < 2e-5


def test_quantize_counts_bounds_and_ties_go_up():
    for bits in (2, 4):
        cent, bnd = tqo.tables(bits)
        assert (tqo.quantize(cent, bits) == np.arange(len(cent))).all()
        assert (tqo.quantize(bnd, bits) == np.arange(1, len(cent))).all()  # value on a bound -> upper cell
        below = np.nextafter(bnd, -np.inf).astype(np.float32)
        assert (tqo.quantize(below, bits) == np.arange(0, len(cent) - 1)).all()
    assert tqo.quantize(np.array([np.nan], np.float32), 4)[0] == 15
    assert tqo.quantize(np.array([np.nan], np.float32), 2)[0] == 0
    assert tqo.quantize(np.array([-1.0, 1.0], np.float32), 4).tolist() == [0, 15]


def test_pack_roundtrip():
    rng = np.random.default_rng(1)
    for bits in (2, 4):
        codes = rng.integers(0, 1 << bits, (5, 128)).astype(np.uint8)
        assert (hp.unpack_codes(hp.pack_codes(codes, bits), bits) == codes).all()


def test_rotation_generator():
    rh, rf = tqo.rotation(42)
    # first entries of the reference generator's fp32 matrix on an x86-64 build without FMA contraction
    assert np.allclose(rf[0, :4], [0.109385304, -0.0462781675, 0.0778490305, 0.064573057], rtol=0, atol=1e-9)
    R = rh.astype(np.float32)
    assert np.abs(R @ R.T - np.eye(128)).max() < 2e-4
    assert tqo.fnv1a64(rh.tobytes()) == "cc1f4a0059e6f6c1"
    rh2, _ = tqo.rotation(43)
    assert (rh2 != rh).any()


def test_append_layout_and_norm():
    rng = np.random.default_rng(2)
    R, _ = tqo.rotation()
    G, Hkv, D, msl = 3, 8, 128, 16
    for bits in (2, 4):
        ck, kn = tqo.alloc_cache(G, msl, Hkv, D, bits)
        k = rng.standard_normal((G, Hkv * D)).astype(np.float16)
        pos = np.array([0, 5, 15], np.int32)
        rot = tqo.append_batch(ck, kn, k, R, pos, msl, Hkv, D, bits, want_rot=True)
        rows = np.arange(G) * msl + pos
        touched = np.zeros(G * msl, bool)
        touched[rows] = True
        assert (ck[~touched] == 0).all() and (kn[~touched] == 0).all()
        codes = hp.unpack_codes(ck[rows].reshape(G, Hkv, -1), bits)
        assert (codes == tqo.quantize(rot, bits)).all()
        norms = np.linalg.norm(k.astype(np.float64).reshape(G, Hkv, D), axis=-1)
        assert np.allclose(kn[rows].astype(np.float64), norms, rtol=1e-3)
        # rotated unit vectors: ||rot|| ~ 1
        assert np.allclose(np.linalg.norm(rot, axis=-1), 1.0, atol=2e-3)


def test_append_edge_vectors():
    R, _ = tqo.rotation()
    Hkv, D = 4, 128
    for bits in (2, 4):
        ck, kn = tqo.alloc_cache(1, 4, Hkv, D, bits)
        x = np.zeros((1, Hkv * D), np.float16)
        tqo.append_tokens(ck, kn, x, R, np.array([0], np.int32), 4, Hkv, D, bits)
        # all-zero vector: every rotated coordinate is 0 -> the cell whose lower bound is 0
        zero_code = 8 if bits == 4 else 2
        assert (hp.unpack_codes(ck[0], bits) == zero_code).all()
        assert (kn[0].astype(np.float32) < 2e-6).all()
        x[0, 3] = np.nan
        tqo.append_tokens(ck, kn, x, R, np.array([1], np.int32), 4, Hkv, D, bits)
        nan_code = 15 if bits == 4 else 0
        assert (hp.unpack_codes(ck[1, : D // (2 if bits == 4 else 4)], bits) == nan_code).all()


def test_token_form_equals_batched_form():
    rng = np.random.default_rng(3)
    R, _ = tqo.rotation()
    Hkv, D, msl, T = 8, 128, 8, 5
    k = rng.standard_normal((T, Hkv * D)).astype(np.float16)
    for bits in (2, 4):
        a_q, a_n = tqo.alloc_cache(1, msl, Hkv, D, bits)
        tqo.append_tokens(a_q, a_n, k, R, np.arange(T, dtype=np.int32), msl, Hkv, D, bits)
        b_q, b_n = tqo.alloc_cache(1, msl, Hkv, D, bits)
        for t in range(T):
            tqo.append_batch(b_q, b_n, k[t:t + 1], R, np.array([t], np.int32), msl, Hkv, D, bits)
        assert (a_q == b_q).all() and (a_n.view(np.uint16) == b_n.view(np.uint16)).all()


@pytest.mark.parametrize("bits", [2, 4])
def test_attention_matches_float64_model(bits):
    """The oracle's attention equals a float64 evaluation of the same formula on the dequantised cache."""
    rng = np.random.default_rng(4)
    R, _ = tqo.rotation()
    G, H, Hkv, D, msl = 3, 16, 8, 128, 80
    lengths = [1, 37, 80]
    ck, kn, cv, vn = hp.build_cache_oracle(rng, G, lengths, msl, Hkv, D, bits, R)
    q = rng.standard_normal((G, H * D)).astype(np.float16)
    pos = np.array(lengths, np.int32) - 1
    out, outf = tqo.attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
    cent, _ = tqo.tables(bits)
    Rd = R.astype(np.float64)
    Kd = cent[hp.unpack_codes(ck.reshape(G, msl, Hkv, -1), bits)].astype(np.float64) * kn.astype(np.float64).reshape(G, msl, Hkv, 1)
    Vd = cent[hp.unpack_codes(cv.reshape(G, msl, Hkv, -1), bits)].astype(np.float64) * vn.astype(np.float64).reshape(G, msl, Hkv, 1)
    qq = q.astype(np.float64).reshape(G, H, D) @ Rd.T
    for g in range(G):
        L = lengths[g]
        for hd in range(H):
            s = Kd[g, :L, hd // 2] @ qq[g, hd] / np.sqrt(128.0)
            w = np.exp(s - s.max())
            w /= w.sum() + 1e-8
            ref = (w @ Vd[g, :L, hd // 2]) @ Rd
            assert np.abs(ref - outf[g, hd]).max() < 2e-5
    # single-sequence form == batched form on the same rows
    g = 2
    o1, _ = tqo.attention_single(q[g], ck[g * msl:(g + 1) * msl], cv[g * msl:(g + 1) * msl], kn[g * msl:(g + 1) * msl],
                                 vn[g * msl:(g + 1) * msl], R, int(pos[g]), msl, H, Hkv, D, bits)
    assert (o1.view(np.uint16) == out[g].view(np.uint16)).all()
    # prefill form: query t attends 0..t == batched form with positions 0..T-1 on a shared cache
    T = 6
    qp = rng.standard_normal((T, H * D)).astype(np.float16)
    op, _ = tqo.prefill_attention(qp, ck[g * msl:(g + 1) * msl], cv[g * msl:(g + 1) * msl], kn[g * msl:(g + 1) * msl],
                                  vn[g * msl:(g + 1) * msl], R, msl, H, Hkv, D, bits)
    for t in range(T):
        o, _ = tqo.attention_single(qp[t], ck[g * msl:(g + 1) * msl], cv[g * msl:(g + 1) * msl],
                                    kn[g * msl:(g + 1) * msl], vn[g * msl:(g + 1) * msl], R, t, msl, H, Hkv, D, bits)
        assert (o.view(np.uint16) == op[t].view(np.uint16)).all()


def test_identical_sequences_give_identical_results():
    """The reference's own batch test invariant (engine/test_all.py:41-47): identical inputs -> identical outputs."""
    rng = np.random.default_rng(5)
    R, _ = tqo.rotation()
    G, H, Hkv, D, msl, L, bits = 4, 16, 8, 128, 40, 33, 4
    k = rng.standard_normal((L, Hkv * D)).astype(np.float16)
    v = rng.standard_normal((L, Hkv * D)).astype(np.float16)
    ck, kn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    cv, vn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    for g in range(G):
        tqo.append_tokens(ck[g * msl:], kn[g * msl:], k, R, np.arange(L, dtype=np.int32), msl, Hkv, D, bits)
        tqo.append_tokens(cv[g * msl:], vn[g * msl:], v, R, np.arange(L, dtype=np.int32), msl, Hkv, D, bits)
    q = np.tile(rng.standard_normal((1, H * D)).astype(np.float16), (G, 1))
    out, _ = tqo.attention_batch(q, ck, cv, kn, vn, R, np.full(G, L - 1, np.int32), msl, H, Hkv, D, bits)
    assert (out.view(np.uint16) == out[0].view(np.uint16)).all()


def test_fp16_twin_matches_float64_model():
    rng = np.random.default_rng(6)
    G, H, Hkv, D, msl = 2, 8, 4, 128, 48
    kv_dim = Hkv * D
    ck = np.zeros((G * msl, kv_dim), np.float16)
    cv = np.zeros_like(ck)
    lengths = [5, 48]
    for s in range(max(lengths)):
        k = rng.standard_normal((G, kv_dim)).astype(np.float16)
        v = rng.standard_normal((G, kv_dim)).astype(np.float16)
        pos = np.array([min(s, n - 1) for n in lengths], np.int32)
        tqo.fp16_write_batch(ck, cv, k, v, pos, msl)
    q = rng.standard_normal((G, H * D)).astype(np.float16)
    pos = np.array(lengths, np.int32) - 1
    out, outf = tqo.fp16_attention_batch(q, ck, cv, pos, msl, H, Hkv, D)
    for g in range(G):
        L = lengths[g]
        K = ck[g * msl:g * msl + L].astype(np.float64).reshape(L, Hkv, D)
        V = cv[g * msl:g * msl + L].astype(np.float64).reshape(L, Hkv, D)
        for hd in range(H):
            s = K[:, hd // 2] @ q[g].astype(np.float64).reshape(H, D)[hd] / np.sqrt(128.0)
            w = np.exp(s - s.max())
            w /= w.sum() + 1e-8
            assert np.abs(w @ V[:, hd // 2] - outf[g, hd]).max() < 2e-5
    o1, _ = tqo.fp16_attention_single(q[1], ck[msl:], cv[msl:], int(pos[1]), msl, H, Hkv, D)
    assert (o1.view(np.uint16) == out[1].view(np.uint16)).all()


# ---- the pin: outputs of the reference's own kernels on a B200 (tests/golden/make_golden.py) ----------------------------
@pytest.mark.parametrize("bits", [2, 4])
def test_oracle_against_reference_kernel_outputs(bits):
    g = hp.load_golden(f"ref_kernels_tq{bits}.npz")
    if g is None:
        pytest.skip("fixture not generated yet")
    H, Hkv, D, msl = int(g["H"]), int(g["Hkv"]), int(g["D"]), int(g["msl"])
    R = hp.h(g["R"])
    k_steps, v_steps = hp.h(g["k_steps"]), hp.h(g["v_steps"])
    G = k_steps.shape[1]
    ck, kn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    cv, vn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    rots_k = {}
    for s in range(k_steps.shape[0]):
        pos = g["pos_steps"][s]
        rk = tqo.append_batch(ck, kn, k_steps[s], R, pos, msl, Hkv, D, bits, want_rot=True)
        tqo.append_batch(cv, vn, v_steps[s], R, pos, msl, Hkv, D, bits)
        for gi in range(G):
            rots_k[(gi, int(pos[gi]))] = rk[gi]
    # codes: identical except coordinates that sit on a quantiser bound (the reference computes 1/sqrt with
    # rsqrt.approx, this oracle with a correctly rounded one); count them and bound their distance
    a = hp.unpack_codes(ck.reshape(G * msl, Hkv, -1), bits)
    b = hp.unpack_codes(g["ck"].reshape(G * msl, Hkv, -1), bits)
    bad = np.argwhere(a != b)
    worst = 0.0
    for row, hd, c in bad:
        gi, p = divmod(int(row), msl)
        if (gi, p) in rots_k:
            worst = max(worst, float(tqo.ulps_to_bound(np.array([rots_k[(gi, p)][hd, c]]), bits)[0]))
    total = int((g["pos_steps"].shape[0]) * G * Hkv * D)
    print(f"tq{bits}: {len(bad)} of {total} K coordinates differ from the reference kernels; worst distance {worst:.2f} ulp")
    assert len(bad) <= max(2, total // 20000)
    assert worst <= hp.ORACLE_ULP_SLACK
    # norms: equal or one fp16 step apart (sqrt.approx vs correctly rounded sqrt on a rounding tie)
    dn = np.abs(kn.view(np.uint16).astype(np.int32) - g["kn"].astype(np.int32))
    assert dn.max() <= 1
    # attention on the REFERENCE's cache bytes: oracle vs reference kernel output
    pos = g["final_pos"]
    out, _ = tqo.attention_batch(hp.h(g["q"]), g["ck"], g["cv"], hp.h(g["kn"]), hp.h(g["vn"]), R, pos, msl, H, Hkv, D, bits)
    hp.assert_attention_close(out, hp.h(g["out"]), H, D, "batched attention")
    sl = slice(2 * msl, 3 * msl)
    o1, _ = tqo.attention_single(hp.h(g["q"])[2], g["ck"][sl], g["cv"][sl], hp.h(g["kn"])[sl], hp.h(g["vn"])[sl], R,
                                 int(pos[2]), msl, H, Hkv, D, bits)
    hp.assert_attention_close(o1[None], hp.h(g["out_single"])[None], H, D, "single-sequence attention")
    op, _ = tqo.prefill_attention(hp.h(g["q_prefill"]), g["ck"][sl], g["cv"][sl], hp.h(g["kn"])[sl], hp.h(g["vn"])[sl],
                                  R, msl, H, Hkv, D, bits)
    hp.assert_attention_close(op, hp.h(g["out_prefill"]), H, D, "prefill attention")
    # edge vectors through the token-form append
    edges = hp.h(g["edges"])
    eq, en = tqo.alloc_cache(1, 16, Hkv, D, bits)
    tqo.append_tokens(eq, en, edges, R, np.arange(edges.shape[0], dtype=np.int32), 16, Hkv, D, bits)
    ea = hp.unpack_codes(eq, bits)
    eb = hp.unpack_codes(g["edge_codes"], bits)
    assert (ea != eb).mean() < 1e-3
    fin = np.isfinite(en.astype(np.float32)) & np.isfinite(hp.h(g["edge_norms"]).astype(np.float32))
    assert np.abs(en.view(np.uint16).astype(np.int32) - g["edge_norms"].astype(np.int32))[fin].max() <= 1


def test_oracle_fp16_against_reference_kernel_outputs():
    g = hp.load_golden("ref_kernels_fp16.npz")
    if g is None:
        pytest.skip("fixture not generated yet")
    H, Hkv, D, msl = int(g["H"]), int(g["Hkv"]), int(g["D"]), int(g["msl"])
    k_steps, v_steps = hp.h(g["k_steps"]), hp.h(g["v_steps"])
    G = k_steps.shape[1]
    ck = np.zeros((G * msl, Hkv * D), np.float16)
    cv = np.zeros_like(ck)
    for s in range(k_steps.shape[0]):
        tqo.fp16_write_batch(ck, cv, k_steps[s], v_steps[s], g["pos_steps"][s], msl)
    out, _ = tqo.fp16_attention_batch(hp.h(g["q"]), ck, cv, g["final_pos"], msl, H, Hkv, D)
    hp.assert_attention_close(out, hp.h(g["out"]), H, D, "fp16 batched attention")
    o1, _ = tqo.fp16_attention_single(hp.h(g["q"])[2], ck[2 * msl:3 * msl], cv[2 * msl:3 * msl], int(g["final_pos"][2]),
                                      msl, H, Hkv, D)
    hp.assert_attention_close(o1[None], hp.h(g["out_single"])[None], H, D, "fp16 single attention")
