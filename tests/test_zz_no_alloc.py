"""GPU test of tq_decode_attention_static, the decode-attention entry point that allocates nothing (its scratch is a
fixed device array inside the library).  It is called through the C ABI twice in a row, with different queries and
positions, and each result is compared with what the regular launcher (launch_turbo_gqa_attention_batch) returns for
the same inputs.  Runs last so that a failure here cannot hide any other test; it also passes on its own in a fresh
process, where its first call is the one that looks the array's address up."""
import numpy as np
import pytest
import torch

from oracle import tqo
from tests import helpers as hp

pytestmark = pytest.mark.gpu
gu = pytest.importorskip("tests.gpu_util")


def _static_attention(L, q, dck, dcv, dkn, dvn, dR, pos, msl, H, Hkv, D, bits):
    G = q.shape[0]
    out = torch.zeros(G, H * D, dtype=torch.float16, device="cuda")
    dq, dpos = gu.dev(q), gu.dev(np.asarray(pos, np.int32))
    st = L.tq_decode_attention_static(out.data_ptr(), dq.data_ptr(), dck.data_ptr(), dcv.data_ptr(), dkn.data_ptr(),
                                      dvn.data_ptr(), dR.data_ptr(), dpos.data_ptr(), dck.shape[0], msl, G, H, Hkv, D,
                                      H * D, Hkv * D, bits, torch.cuda.current_stream().cuda_stream)
    assert st == 0, f"tq_decode_attention_static returned {st}"
    return gu.host(out)


@pytest.mark.parametrize("bits", [4, 2])
def test_static_scratch_variant_matches_regular_entry_point(bits):
    import triebwerk_b200 as tq
    L = tq.lib()
    rng = np.random.default_rng(100 + bits)
    R, _ = tqo.rotation()
    G, H, Hkv, D, msl = 6, 16, 8, 128, 1536
    lengths = [1, 33, 700, 1536, 1100, 257]
    ck, kn, cv, vn = hp.build_cache_oracle(rng, G, lengths, msl, Hkv, D, bits, R)
    dck, dcv, dkn, dvn, dR = (gu.dev(x) for x in (ck, cv, kn, vn, R))
    # two calls in a row on the shared scratch: different queries, different positions (shorter the second time)
    calls = [(rng.standard_normal((G, H * D), dtype=np.float32).astype(np.float16), np.array(lengths) - 1),
             (rng.standard_normal((G, H * D), dtype=np.float32).astype(np.float16), np.array([0, 10, 31, 900, 32, 256]))]
    for n, (q, pos) in enumerate(calls):
        got = _static_attention(L, q, dck, dcv, dkn, dvn, dR, pos, msl, H, Hkv, D, bits)
        want = gu.gpu_attention_batch(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits)
        worst, rel = hp.assert_attention_close(got, want, H, D, f"static scratch, call {n}, tq{bits}")
        same = float((got.view(np.uint16) == want.view(np.uint16)).mean())
        print(f"tq{bits} call {n}: max-abs {worst:.2e}, rel {rel:.2e}, {100 * same:.2f}% of outputs bit-identical")
        ref, _ = tqo.attention_batch(q, ck, cv, kn, vn, R, pos.astype(np.int32), msl, H, Hkv, D, bits)
        hp.assert_attention_close(got, ref, H, D, f"static scratch vs oracle, call {n}, tq{bits}")
    # no kernel of the two calls gave up on a wait or refused its shared-memory layout
    assert L.tq_static_status(torch.cuda.current_stream().cuda_stream) == 0


def test_static_scratch_variant_refuses_oversized_requests():
    import triebwerk_b200 as tq
    L = tq.lib()
    t = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    # 512 sequences x 32 heads needs far more than the built-in 20 MiB: refused with TQ_ERR_CAPACITY, nothing launched
    assert L.tq_workspace_bytes(512, 32) > (20 << 20)
    st = L.tq_decode_attention_static(p, p, p, p, p, p, p, p, 512 * 64, 64, 512, 32, 8, 128, 32 * 128, 8 * 128, 4, None)
    assert st == -2
    torch.cuda.synchronize()
