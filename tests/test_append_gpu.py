"""GPU parity of the TurboQuant append, through the C ABI: against the CPU oracle (mismatches classified by
their distance to a quantiser bound), against the committed outputs of the reference's own kernels
(byte-exact) and, when the reference library travelled with the snapshot, against the reference kernels live."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import tqo
from tests import helpers as hp

pytestmark = pytest.mark.gpu
gu = pytest.importorskip("tests.gpu_util")


def _check_vs_oracle(codes_gpu, norms_gpu, codes_or, norms_or, rot, bits, rows, Hkv, what):
    a = hp.unpack_codes(codes_gpu[rows].reshape(len(rows), Hkv, -1), bits)
    b = hp.unpack_codes(codes_or[rows].reshape(len(rows), Hkv, -1), bits)
    n, worst, n1 = hp.classify_code_mismatches(a, b, rot.reshape(a.shape), bits)
    print(f"{what}: {n} of {a.size} coordinates differ from the IEEE oracle; {n1} within 1 ulp of a bound; worst {worst:.2f} ulp")
    assert n <= max(3, a.size // 50000), f"{what}: too many code mismatches ({n})"
    assert worst <= hp.ORACLE_ULP_SLACK, f"{what}: a coordinate {worst:.1f} ulp from any bound got another code"
    dn = np.abs(norms_gpu[rows].view(np.uint16).astype(np.int32) - norms_or[rows].view(np.uint16).astype(np.int32))
    assert dn.max() <= 1, f"{what}: norm differs by more than one fp16 step"
    untouched = np.ones(codes_gpu.shape[0], bool)
    untouched[rows] = False
    assert (codes_gpu[untouched] == 0).all() and (norms_gpu[untouched].view(np.uint16) == 0).all(), "wrote outside its rows"


@pytest.mark.parametrize("bits", [4, 2])
def test_batched_append_vs_oracle_c0_shape(bits):
    # 16 query / 8 KV heads, head_dim 128, G=4: the single-layer reference configuration
    rng = np.random.default_rng(0)
    R, _ = tqo.rotation()
    G, Hkv, D, msl = 4, 8, 128, 640
    scales = np.exp(np.random.default_rng(1).normal(0, 0.5, Hkv * D)).astype(np.float32)
    pos = np.array([100, 101, 350, 611], np.int32)
    k = (rng.standard_normal((G, Hkv * D), dtype=np.float32) * scales).astype(np.float16)
    cq, cn = gu.gpu_append_batch(k, R, pos, msl, Hkv, D, bits)
    oq, on = tqo.alloc_cache(G, msl, Hkv, D, bits)
    rot = tqo.append_batch(oq, on, k, R, pos, msl, Hkv, D, bits, want_rot=True)
    rows = np.arange(G) * msl + pos
    _check_vs_oracle(cq, cn, oq, on, rot, bits, rows, Hkv, f"batched tq{bits}")


@pytest.mark.parametrize("bits", [4, 2])
def test_token_append_many_vectors_vs_oracle(bits):
    rng = np.random.default_rng(2)
    R, _ = tqo.rotation()
    Hkv, D, T = 8, 128, 1500  # 12000 head vectors, 1.5 M coordinates
    k = (rng.standard_normal((T, Hkv * D), dtype=np.float32) * rng.lognormal(0, 0.5, Hkv * D).astype(np.float32)).astype(np.float16)
    pos = rng.permutation(T).astype(np.int32)  # scattered destinations
    cq, cn = gu.gpu_append_tokens(k, R, pos, T, Hkv, D, bits)
    oq, on = tqo.alloc_cache(1, T, Hkv, D, bits)
    rot = tqo.append_tokens(oq, on, k, R, pos, T, Hkv, D, bits, want_rot=True)
    # rot is indexed by token; reorder to row order for the classifier
    rot_rows = np.zeros_like(rot)
    rot_rows[pos] = rot
    a = hp.unpack_codes(cq.reshape(T, Hkv, -1), bits)
    b = hp.unpack_codes(oq.reshape(T, Hkv, -1), bits)
    n, worst, n1 = hp.classify_code_mismatches(a, b, rot_rows, bits)
    print(f"token tq{bits}: {n} of {a.size} coordinates differ; {n1} within 1 ulp; worst {worst:.2f} ulp")
    assert n <= max(3, a.size // 50000) and worst <= hp.ORACLE_ULP_SLACK
    assert np.abs(cn.view(np.uint16).astype(np.int32) - on.view(np.uint16).astype(np.int32)).max() <= 1


@pytest.mark.parametrize("bits", [4, 2])
def test_append_bytes_equal_reference_kernel_outputs(bits):
    """Byte-exact against what the reference's own kernels wrote on a B200 (committed fixture)."""
    g = hp.load_golden(f"ref_kernels_tq{bits}.npz")
    if g is None:
        pytest.skip("fixture not generated yet")
    Hkv, D, msl = int(g["Hkv"]), int(g["D"]), int(g["msl"])
    R = hp.h(g["R"])
    k_steps, v_steps = hp.h(g["k_steps"]), hp.h(g["v_steps"])
    G = k_steps.shape[1]
    ck = cn = cv = vn = None
    for s in range(k_steps.shape[0]):
        ck, cn = gu.gpu_append_batch(k_steps[s], R, g["pos_steps"][s], msl, Hkv, D, bits, ck, cn)
        cv, vn = gu.gpu_append_batch(v_steps[s], R, g["pos_steps"][s], msl, Hkv, D, bits, cv, vn)
    assert (ck == g["ck"]).all(), f"{int((ck != g['ck']).sum())} K code bytes differ from the reference kernels"
    assert (cv == g["cv"]).all()
    assert (cn.view(np.uint16) == g["kn"]).all() and (vn.view(np.uint16) == g["vn"]).all()
    edges = hp.h(g["edges"])
    eq, en = gu.gpu_append_tokens(edges, R, np.arange(edges.shape[0]), 16, Hkv, D, bits)
    assert (eq == g["edge_codes"]).all(), "edge vectors (zero, one-hot, +-65504, subnormal, NaN ...) differ"
    assert (en.view(np.uint16) == g["edge_norms"]).all()


@pytest.mark.parametrize("bits", [4, 2])
def test_fused_append_equals_separate_launchers_and_rotates_q(bits):
    import triebwerk_b200 as tq
    from triebwerk_b200 import ops
    rng = np.random.default_rng(3)
    R, Rf = tqo.rotation()
    G, H, Hkv, D, msl = 5, 16, 8, 128, 64
    kv_dim, q_dim = Hkv * D, H * D
    vpb = 4 if bits == 2 else 2
    k = rng.standard_normal((G, kv_dim)).astype(np.float16)
    v = rng.standard_normal((G, kv_dim)).astype(np.float16)
    q = rng.standard_normal((G, q_dim)).astype(np.float16)
    pos = np.array([0, 63, 7, 31, 32], np.int32)
    ck1, kn1 = gu.gpu_append_batch(k, R, pos, msl, Hkv, D, bits)
    cv1, vn1 = gu.gpu_append_batch(v, R, pos, msl, Hkv, D, bits)
    ws = ops.new_workspace(G, H)
    dck = torch.zeros(G * msl, kv_dim // vpb, dtype=torch.uint8, device="cuda")
    dcv = torch.zeros_like(dck)
    dkn = torch.zeros(G * msl, Hkv, dtype=torch.float16, device="cuda")
    dvn = torch.zeros_like(dkn)
    ops.append_decode(dck, dkn, dcv, dvn, gu.dev(k), gu.dev(v), gu.dev(q), gu.dev(R), gu.dev(pos), msl, H, Hkv, bits, ws)
    assert (gu.host(dck) == ck1).all() and (gu.host(dcv) == cv1).all()
    assert (gu.host(dkn).view(np.uint16) == kn1.view(np.uint16)).all()
    assert (gu.host(dvn).view(np.uint16) == vn1.view(np.uint16)).all()
    # the rotated queries sit after the 256-byte header of the workspace, scaled by log2(e)/sqrt(128)
    qrot = gu.host(ws)[256:256 + G * H * D * 4].view(np.float32).reshape(G, H, D)
    want = (q.astype(np.float64).reshape(G, H, D) @ R.astype(np.float64).T) * (np.log2(np.e) / np.sqrt(128.0))
    assert np.abs(qrot - want).max() < 2e-5
    assert ops.workspace_status(ws) == 0


def test_append_rejects_bad_arguments():
    import triebwerk_b200 as tq
    L = tq.lib()
    ws = tq.ops.new_workspace(2, 16)
    t = torch.zeros(16, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    pos = torch.zeros(2, dtype=torch.int32, device="cuda")
    # head_dim 64 is unsupported, kv_bits 3 is an argument error, missing workspace is reported
    assert L.tq_append_decode(p, p, p, p, p, p, None, p, pos.data_ptr(), None, 8, 2, 16, 8, 64, 1024, 512, 4, ws.data_ptr(), ws.numel(), None) == -4
    assert L.tq_append_decode(p, p, p, p, p, p, None, p, pos.data_ptr(), None, 8, 2, 16, 8, 128, 2048, 1024, 3, ws.data_ptr(), ws.numel(), None) == -1
    assert L.tq_append_decode(p, p, p, p, p, p, None, p, pos.data_ptr(), None, 8, 2, 16, 8, 128, 2048, 1024, 4, None, 0, None) == -3
    assert L.tq_append_decode(p, p, p, p, p, p, None, p, pos.data_ptr(), None, 8, 2, 16, 8, 128, 2048, 1024, 4, ws.data_ptr(), 128, None) == -3


def test_out_of_range_position_sets_status_and_writes_nothing():
    from triebwerk_b200 import ops
    rng = np.random.default_rng(4)
    R, _ = tqo.rotation()
    G, H, Hkv, D, msl, bits = 2, 16, 8, 128, 16, 4
    k = rng.standard_normal((G, Hkv * D)).astype(np.float16)
    ws = ops.new_workspace(G, H)
    dck = torch.zeros(G * msl, Hkv * D // 2, dtype=torch.uint8, device="cuda")
    dkn = torch.zeros(G * msl, Hkv, dtype=torch.float16, device="cuda")
    pos = np.array([3, 16], np.int32)  # 16 == capacity: out of range
    ops.append_decode(dck, dkn, None, None, gu.dev(k), None, None, gu.dev(R), gu.dev(pos), msl, H, Hkv, bits, ws)
    assert ops.workspace_status(ws) == 3
    assert ops.workspace_status(ws) == 0  # reading clears it
    c = gu.host(dck)
    assert c[3].any() and not c[msl:].any()


@pytest.mark.parametrize("bits", [4, 2])
def test_append_equals_reference_kernels_live(bits):
    """Same inputs through the reference's own kernels (compiled unmodified for sm_100a) in this process."""
    if not os.path.exists(gu.REF_SO):
        pytest.skip("reference kernel library not present in this snapshot")
    ref = C.CDLL(gu.REF_SO)
    ref.launch_turbo_kv_quantize.restype = None
    rng = np.random.default_rng(5)
    R, _ = tqo.rotation()
    Hkv, D, T = 8, 128, 4096
    k = (rng.standard_normal((T, Hkv * D), dtype=np.float32) * rng.lognormal(0, 0.5, Hkv * D).astype(np.float32)).astype(np.float16)
    pos = np.arange(T, dtype=np.int32)
    vpb = 4 if bits == 2 else 2
    rq = torch.zeros(T, Hkv * D // vpb, dtype=torch.uint8, device="cuda")
    rn = torch.zeros(T, Hkv, dtype=torch.float16, device="cuda")
    dk, dR, dp = gu.dev(k), gu.dev(R), gu.dev(pos)
    vp = lambda t: C.c_void_p(t.data_ptr())
    ref.launch_turbo_kv_quantize(vp(rq), vp(rn), vp(dk), vp(dR), vp(dp), C.c_int(T), C.c_int(T), C.c_int(Hkv), C.c_int(D),
                                 C.c_int(Hkv * D), C.c_int(bits), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    mq, mn = gu.gpu_append_tokens(k, R, pos, T, Hkv, D, bits)
    rqh, rnh = gu.host(rq), gu.host(rn)
    nbad = int((mq != rqh).sum())
    print(f"tq{bits}: {nbad} of {mq.size} code bytes differ from the live reference kernels over {T * Hkv * D} coordinates")
    assert nbad == 0
    assert (mn.view(np.uint16) == rnh.view(np.uint16)).all()


@pytest.mark.parametrize("bits,Hkv,T", [(4, 8, 2048), (2, 8, 1000), (4, 4, 777), (2, 4, 300)])
def test_tensor_core_prefill_append_equals_the_chain_kernel_and_the_oracle(bits, Hkv, T):
    """Whole prompts take the tcgen05 kernel (rotation on the tensor cores, exact fp32 chain for coordinates near a
    decision bound); single tokens take the chain kernel.  Same inputs through both, token by token for the chain
    kernel: every stored byte must agree, including an all-zero vector (all of its coordinates sit ON the bound 0),
    huge values, a NaN vector and the ragged last tile; a seeded subset is also checked against the oracle."""
    import triebwerk_b200 as tq
    H, D = 16, 128
    kv_dim = Hkv * D
    rng = np.random.default_rng(21)
    k = rng.standard_normal((T, kv_dim), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((T, kv_dim), dtype=np.float32).astype(np.float16)
    k[3, :D] = 0
    k[5, D:2 * D] *= np.float16(300.0)
    v[7, :D] = np.float16(np.nan)
    v[9, :D] = np.float16(6e-8)  # subnormal inputs
    k[100:140] = 0               # a stretch of padding: all-zero vectors take their constant codes without any exact chain
    v[120:130, D:] = np.float16(-0.0)
    msl = T + 32
    eng_tc = tq.Engine(msl, bits, num_layers=1, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng_ch = tq.Engine(msl, bits, num_layers=1, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng_tc.alloc_batch(1, msl)
    eng_ch.alloc_batch(1, msl)
    kd, vd = gu.dev(k), gu.dev(v)
    eng_tc.prefill_append(0, 0, kd, vd, 3)          # one call: T * Hkv >= 512 vectors -> tensor-core kernel
    step = 32 // Hkv                                 # fewer than 512 vectors per call -> chain kernel
    for t0 in range(0, T, step):
        eng_ch.prefill_append(0, 0, kd[t0:t0 + step], vd[t0:t0 + step], 3 + t0)
    assert eng_tc.status() == 0 and eng_ch.status() == 0
    for a, b, name in zip(eng_tc.layer_cache(0), eng_ch.layer_cache(0), ("k codes", "v codes", "k norms", "v norms")):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), f"{name} differ between the two kernels"
    R = tq.ops.rotation_matrix().numpy()
    n = min(T, 64)
    cq, cn = tqo.alloc_cache(1, n + 3, Hkv, D, bits)
    tqo.append_tokens(cq, cn, k[:n], R, np.arange(3, n + 3, dtype=np.int32), n + 3, Hkv, D, bits)
    got = eng_tc.layer_cache(0)[0].cpu().numpy().reshape(msl, -1)[3:n + 3]
    ref = cq.reshape(n + 3, -1)[3:n + 3]
    bad = int((got != ref).sum())
    assert bad <= hp.ORACLE_ULP_SLACK, f"{bad} packed bytes differ from the oracle"


@pytest.mark.parametrize("bits,ragged", [(4, False), (2, True)])
def test_batched_prefill_append_equals_per_sequence_calls(bits, ragged):
    """Several prompts in one launch (tensor-core kernel over [n_seq][T][kv_dim]) against one call per sequence: the same
    bytes in every slot, dense and per-sequence (ragged) slots, at a non-zero first position, leaving the neighbouring
    sequences untouched."""
    import triebwerk_b200 as tq
    H, Hkv, D, T, G = 16, 8, 128, 70, 5
    kv_dim = Hkv * D
    rng = np.random.default_rng(3)
    k = gu.dev(rng.standard_normal((3, T, kv_dim), dtype=np.float32).astype(np.float16))
    v = gu.dev(rng.standard_normal((3, T, kv_dim), dtype=np.float32).astype(np.float16))
    caps = [200, 90, 100, 96, 300] if ragged else None
    engines = []
    for _ in range(2):
        e = tq.Engine(320, bits, num_layers=1, num_heads=H, num_kv_heads=Hkv, head_dim=D)
        e.alloc_batch(G, 320, caps)
        engines.append(e)
    engines[0].prefill_append_batch(0, 1, k, v, 9)
    for i in range(3):
        engines[1].prefill_append(0, 1 + i, k[i], v[i], 9)
    assert engines[0].status() == 0 and engines[1].status() == 0
    for a, b, name in zip(engines[0].layer_cache(0), engines[1].layer_cache(0), ("k codes", "v codes", "k norms", "v norms")):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), f"{name} differ"
    assert int(engines[0].layer_cache(0)[0].view(torch.uint8).ne(0).sum()) > 0
    with pytest.raises(tq.TqError):
        engines[0].prefill_append_batch(0, 3, k, v, 0)  # sequences 3, 4, 5: one too many


def test_tensor_core_prefill_append_thread_load_form_in_a_child_process():
    """Where a tensor map over the input can be had, the tcgen05 append takes its vectors by tensor-map copies; the
    thread-load form (unaligned inputs, a head count that does not divide 128, the producer form) is selected for every
    call by TQ_PREFILL_TMA=0, which the library reads once per process: the append parity tests of the tensor-core
    kernel run again in a child with it set."""
    import os
    import subprocess
    import sys
    if os.environ.get("TQ_PREFILL_TMA") == "0":
        pytest.skip("already the child")
    env = dict(os.environ, TQ_PREFILL_TMA="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_append_gpu.py", "tests/test_engine_gpu.py", "-q", "-x", "-m", "gpu",
                        "-k", "(tensor_core or batched_prefill or prefill_layer or whole) and not child", "-p", "no:cacheprovider"],
                       cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert " passed" in r.stdout


@pytest.mark.parametrize("bits,Hkv,T", [(4, 2, 700), (4, 16, 130), (2, 32, 67), (4, 3, 400), (2, 1, 1200)])
def test_token_append_other_head_counts_vs_oracle(bits, Hkv, T):
    """The reference's token-form launcher takes any number of KV heads.  Head counts that divide 128 reach the tensor
    cores' operand tile by tensor-map copies whose box is (128 / Hkv tokens) x (Hkv heads); the others, here 3, through
    thread loads.  Scattered destinations, ragged last tiles; checked against the oracle."""
    rng = np.random.default_rng(5 + Hkv)
    R, _ = tqo.rotation()
    D = 128
    k = (rng.standard_normal((T, Hkv * D), dtype=np.float32) * rng.lognormal(0, 0.5, Hkv * D).astype(np.float32)).astype(np.float16)
    pos = rng.permutation(T).astype(np.int32)
    cq, cn = gu.gpu_append_tokens(k, R, pos, T, Hkv, D, bits)
    oq, on = tqo.alloc_cache(1, T, Hkv, D, bits)
    rot = tqo.append_tokens(oq, on, k, R, pos, T, Hkv, D, bits, want_rot=True)
    rot_rows = np.zeros_like(rot)
    rot_rows[pos] = rot
    a = hp.unpack_codes(cq.reshape(T, Hkv, -1), bits)
    b = hp.unpack_codes(oq.reshape(T, Hkv, -1), bits)
    n, worst, n1 = hp.classify_code_mismatches(a, b, rot_rows, bits)
    print(f"token tq{bits}, {Hkv} heads: {n} of {a.size} coordinates differ; {n1} within 1 ulp; worst {worst:.2f} ulp")
    assert n <= max(3, a.size // 50000) and worst <= hp.ORACLE_ULP_SLACK
    assert np.abs(cn.view(np.uint16).astype(np.int32) - on.view(np.uint16).astype(np.int32)).max() <= 1
