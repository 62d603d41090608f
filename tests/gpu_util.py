"""Helpers for the -m gpu tests: numpy <-> device, and thin drivers over the C-ABI launchers."""
from __future__ import annotations

import os

import numpy as np
import torch

import triebwerk_b200 as tq
from triebwerk_b200 import ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libtriebwerk_ref_kernels.so")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def gpu_append_batch(kv_buf, R, positions, msl, Hkv, D, bits, ck=None, kn=None):
    """launch_turbo_kv_quantize_batch on numpy inputs; returns (codes, norms) numpy."""
    G, kv_dim = kv_buf.shape
    vpb = 4 if bits == 2 else 2
    dck = dev(ck) if ck is not None else torch.zeros(G * msl, kv_dim // vpb, dtype=torch.uint8, device="cuda")
    dkn = dev(kn) if kn is not None else torch.zeros(G * msl, Hkv, dtype=torch.float16, device="cuda")
    ops.launch_turbo_kv_quantize_batch(dck, dkn, dev(kv_buf), dev(R), dev(np.asarray(positions, np.int32)), msl, G,
                                       Hkv, D, kv_dim, bits)
    return host(dck), host(dkn)


def gpu_append_tokens(kv_buf, R, positions, msl, Hkv, D, bits):
    T, kv_dim = kv_buf.shape
    vpb = 4 if bits == 2 else 2
    dck = torch.zeros(msl, kv_dim // vpb, dtype=torch.uint8, device="cuda")
    dkn = torch.zeros(msl, Hkv, dtype=torch.float16, device="cuda")
    ops.launch_turbo_kv_quantize(dck, dkn, dev(kv_buf), dev(R), dev(np.asarray(positions, np.int32)), msl, T, Hkv, D,
                                 kv_dim, bits)
    return host(dck), host(dkn)


def gpu_attention_batch(q, ck, cv, kn, vn, R, positions, msl, H, Hkv, D, bits):
    G, q_dim = q.shape
    out = torch.zeros(G, q_dim, dtype=torch.float16, device="cuda")
    ops.launch_turbo_gqa_attention_batch(out, dev(q), dev(ck), dev(cv), dev(kn), dev(vn), dev(R), None,
                                         dev(np.asarray(positions, np.int32)), msl, G, H, Hkv, D, q_dim, Hkv * D, bits)
    return host(out)


def gpu_attention_single(q, ck, cv, kn, vn, R, pos, msl, H, Hkv, D, bits):
    out = torch.zeros(H * D, dtype=torch.float16, device="cuda")
    ops.launch_turbo_gqa_attention(dev(q), dev(ck), dev(cv), dev(kn), dev(vn), dev(R), out, None, int(pos), msl, H, Hkv,
                                   D, bits)
    return host(out)


def gpu_prefill_attention(q, ck, cv, kn, vn, R, msl, H, Hkv, D, bits):
    T, q_dim = q.shape
    out = torch.zeros(T, q_dim, dtype=torch.float16, device="cuda")
    ops.launch_turbo_gqa_prefill_attention(out, dev(q), dev(ck), dev(cv), dev(kn), dev(vn), dev(R), None, T, msl, H,
                                           Hkv, D, q_dim, Hkv * D, bits)
    return host(out)


def compat_status_clear():
    """Device status word of the compat workspace is not reachable from here; the launchers' host status is."""
    return tq.lib().tq_last_compat_status()
