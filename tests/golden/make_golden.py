"""Generates tests/golden/ref_kernels_*.npz by running the REFERENCE's own CUDA kernels on a GPU.

The reference (BY571/triebwerk) holds no golden vectors for its TurboQuant path, so the pin is made from
its kernels themselves: oracle/Makefile compiles engine/kernels.cu unmodified (with the reference's own
--use_fast_math) for sm_100a into oracle/_ref/libtriebwerk_ref_kernels.so, and this script drives the
launchers of that library (engine/kernels.cu:1963-2028, :737-752, :1351-1357) on seeded inputs and stores inputs and
outputs.  Run on a GPU machine from the repository root:

    python tests/golden/make_golden.py --out new_golden

then copy the .npz files into tests/golden/.  The CPU oracle and the CUDA library are both tested against
these files.  Rotation bytes come from the oracle's restatement of the reference generator and are stored
in the fixture, so every consumer uses the same R.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import tqo  # noqa: E402

REF_SO = os.path.join(ROOT, "oracle", "_ref", "libtriebwerk_ref_kernels.so")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def p(t):
    return C.c_void_p(t.data_ptr())


def edge_vectors(kv_dim, rng):
    """Rows for the edge cases of the append: zero vector, one-hot, huge, tiny, NaN, constant."""
    rows = np.zeros((8, kv_dim), np.float32)
    rows[1, ::128] = 1.0
    rows[2] = 65504.0
    rows[2, 1::2] = -65504.0
    rows[3] = 6e-8
    rows[4] = rng.standard_normal(kv_dim)
    rows[4, 5] = np.nan
    rows[5] = 1.0
    rows[6] = rng.standard_normal(kv_dim) * 1e-3
    rows[7] = rng.standard_normal(kv_dim) * 100.0
    return rows.astype(np.float16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="new_golden")
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    ref = C.CDLL(REF_SO)
    for name in ("launch_turbo_kv_quantize", "launch_turbo_kv_quantize_batch", "launch_turbo_gqa_attention_batch",
                 "launch_turbo_gqa_attention", "launch_turbo_gqa_prefill_attention", "launch_kv_cache_write_batch",
                 "launch_gqa_attention_batch", "launch_gqa_attention"):
        getattr(ref, name).restype = None
    i = C.c_int
    null = C.c_void_p(0)

    H, Hkv, D = 8, 4, 128
    q_dim, kv_dim = H * D, Hkv * D
    final_pos = np.array([0, 17, 40], np.int32)
    G, msl = len(final_pos), 48
    dummy = msl - 1  # finished sequences keep writing here; never attended
    rng = np.random.default_rng(0)
    scales = np.exp(np.random.default_rng(1).normal(0.0, 0.5, kv_dim)).astype(np.float32)
    S = int(final_pos.max()) + 1
    k_steps = (rng.standard_normal((S, G, kv_dim), dtype=np.float32) * scales).astype(np.float16)
    v_steps = rng.standard_normal((S, G, kv_dim), dtype=np.float32).astype(np.float16)
    pos_steps = np.stack([np.where(s <= final_pos, s, dummy) for s in range(S)]).astype(np.int32)
    q = rng.standard_normal((G, q_dim), dtype=np.float32).astype(np.float16)
    Tq = 8
    q_prefill = rng.standard_normal((Tq, q_dim), dtype=np.float32).astype(np.float16)
    edges = edge_vectors(kv_dim, rng)
    R, _ = tqo.rotation(42)
    dR = dev(R)

    for bits in (4, 2):
        vpb = 4 if bits == 2 else 2
        kvp = kv_dim // vpb
        ck = torch.zeros(G * msl, kvp, dtype=torch.uint8, device="cuda")
        cv = torch.zeros_like(ck)
        kn = torch.zeros(G * msl, Hkv, dtype=torch.float16, device="cuda")
        vn = torch.zeros_like(kn)
        for s in range(S):
            dpos = dev(pos_steps[s])
            dk, dv = dev(k_steps[s]), dev(v_steps[s])
            ref.launch_turbo_kv_quantize_batch(p(ck), p(kn), p(dk), p(dR), p(dpos), i(msl), i(G), i(Hkv), i(D),
                                               i(kv_dim), i(bits), null)
            ref.launch_turbo_kv_quantize_batch(p(cv), p(vn), p(dv), p(dR), p(dpos), i(msl), i(G), i(Hkv), i(D),
                                               i(kv_dim), i(bits), null)
        torch.cuda.synchronize()
        # batched decode attention
        dq = dev(q)
        out = torch.zeros(G, q_dim, dtype=torch.float16, device="cuda")
        scratch = torch.zeros(max(G, Tq) * H * msl, dtype=torch.float32, device="cuda")
        dfinal = dev(final_pos)
        ref.launch_turbo_gqa_attention_batch(p(out), p(dq), p(ck), p(cv), p(kn), p(vn), p(dR), p(scratch), p(dfinal),
                                             i(msl), i(G), i(H), i(Hkv), i(D), i(q_dim), i(kv_dim), i(bits), null)
        # single-sequence form on the rows of sequence 2
        g2 = 2
        sl = slice(g2 * msl, (g2 + 1) * msl)
        ck1, cv1 = ck[sl].contiguous(), cv[sl].contiguous()
        kn1, vn1 = kn[sl].contiguous(), vn[sl].contiguous()
        out1 = torch.zeros(q_dim, dtype=torch.float16, device="cuda")
        dq1 = dq[g2].contiguous()
        ref.launch_turbo_gqa_attention(p(dq1), p(ck1), p(cv1), p(kn1), p(vn1), p(dR), p(out1), p(scratch),
                                       i(int(final_pos[g2])), i(msl), i(H), i(Hkv), i(D), i(bits), null)
        # causal prefill attention: Tq queries over the first Tq rows of sequence 2
        outp = torch.zeros(Tq, q_dim, dtype=torch.float16, device="cuda")
        dqp = dev(q_prefill)
        ref.launch_turbo_gqa_prefill_attention(p(outp), p(dqp), p(ck1), p(cv1), p(kn1), p(vn1), p(dR), p(scratch),
                                               i(Tq), i(msl), i(H), i(Hkv), i(D), i(q_dim), i(kv_dim), i(bits), null)
        # token-form append of the edge vectors into a fresh single-sequence cache
        ne = edges.shape[0]
        cke = torch.zeros(16, kvp, dtype=torch.uint8, device="cuda")
        kne = torch.zeros(16, Hkv, dtype=torch.float16, device="cuda")
        dposE = dev(np.arange(ne, dtype=np.int32))
        dE = dev(edges)
        ref.launch_turbo_kv_quantize(p(cke), p(kne), p(dE), p(dR), p(dposE), i(16), i(ne), i(Hkv), i(D), i(kv_dim),
                                     i(bits), null)
        torch.cuda.synchronize()
        np.savez_compressed(
            os.path.join(args.out, f"ref_kernels_tq{bits}.npz"),
            bits=bits, H=H, Hkv=Hkv, D=D, msl=msl, final_pos=final_pos, R=R.view(np.uint16),
            k_steps=k_steps.view(np.uint16), v_steps=v_steps.view(np.uint16), pos_steps=pos_steps,
            q=q.view(np.uint16), q_prefill=q_prefill.view(np.uint16), edges=edges.view(np.uint16),
            ck=ck.cpu().numpy(), cv=cv.cpu().numpy(), kn=kn.cpu().numpy().view(np.uint16),
            vn=vn.cpu().numpy().view(np.uint16), out=out.cpu().numpy().view(np.uint16),
            out_single=out1.cpu().numpy().view(np.uint16), out_prefill=outp.cpu().numpy().view(np.uint16),
            edge_codes=cke.cpu().numpy(), edge_norms=kne.cpu().numpy().view(np.uint16))
        print("wrote", bits)

    # fp16 twin
    ckf = torch.zeros(G * msl, kv_dim, dtype=torch.float16, device="cuda")
    cvf = torch.zeros_like(ckf)
    for s in range(S):
        dk, dv, dpos = dev(k_steps[s]), dev(v_steps[s]), dev(pos_steps[s])  # named: they must outlive the launch
        ref.launch_kv_cache_write_batch(p(ckf), p(cvf), p(dk), p(dv), p(dpos), i(msl), i(G), i(kv_dim), null)
        torch.cuda.synchronize()
    outf = torch.zeros(G, q_dim, dtype=torch.float16, device="cuda")
    scratch = torch.zeros(G * H * msl, dtype=torch.float32, device="cuda")
    dq = dev(q)
    dfinal = dev(final_pos)
    ref.launch_gqa_attention_batch(p(outf), p(dq), p(ckf), p(cvf), p(scratch), p(dfinal), i(msl), i(G), i(H),
                                   i(Hkv), i(D), i(q_dim), i(kv_dim), null)
    g2 = 2
    outf1 = torch.zeros(q_dim, dtype=torch.float16, device="cuda")
    ck1 = ckf[g2 * msl:(g2 + 1) * msl].contiguous()
    cv1 = cvf[g2 * msl:(g2 + 1) * msl].contiguous()
    dq1 = dq[g2].contiguous()
    ref.launch_gqa_attention(p(dq1), p(ck1), p(cv1), p(outf1), p(scratch), i(int(final_pos[g2])),
                             i(msl), i(H), i(Hkv), i(D), null)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(args.out, "ref_kernels_fp16.npz"), H=H, Hkv=Hkv, D=D, msl=msl,
                        final_pos=final_pos, k_steps=k_steps.view(np.uint16), v_steps=v_steps.view(np.uint16),
                        pos_steps=pos_steps, q=q.view(np.uint16), out=outf.cpu().numpy().view(np.uint16),
                        out_single=outf1.cpu().numpy().view(np.uint16))
    print("wrote fp16")


if __name__ == "__main__":
    main()
