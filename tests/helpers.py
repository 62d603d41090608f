"""Shared helpers of the test-suite: oracle-built caches, code comparison with boundary classification, and
the attention tolerance of the specification."""
from __future__ import annotations

import os

import numpy as np

from oracle import tqo

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerances of the specification: codes bit-exact except coordinates within 1 fp32 ulp of a quantiser bound
# (counted and reported); attention outputs within max-abs 2e-3 and relative 1e-2 in fp16.
ATTN_ABS = 2e-3
ATTN_REL = 1e-2
# Against the IEEE oracle (which uses correctly rounded 1/sqrt where the GPU uses rsqrt.approx, <= 2 ulp off)
# a coordinate can sit up to a few ulps from a bound and still legitimately land on the other side.
ORACLE_ULP_SLACK = 8.0


def h(a):
    return np.ascontiguousarray(a).view(np.float16) if a.dtype == np.uint16 else a


def load_golden(name):
    path = os.path.join(GOLDEN, name)
    if not os.path.exists(path):
        return None
    return dict(np.load(path))


def unpack_codes(packed: np.ndarray, bits: int) -> np.ndarray:
    """[..., nbytes] uint8 -> [..., nbytes*vpb] codes in coordinate order."""
    if bits == 4:
        parts = [packed & 0xF, packed >> 4]
    else:
        parts = [(packed >> s) & 3 for s in (0, 2, 4, 6)]
    return np.stack(parts, axis=-1).reshape(*packed.shape[:-1], -1)


def pack_codes(codes: np.ndarray, bits: int) -> np.ndarray:
    vpb = 2 if bits == 4 else 4
    c = codes.reshape(*codes.shape[:-1], -1, vpb).astype(np.uint8)
    out = np.zeros(c.shape[:-1], np.uint8)
    for j in range(vpb):
        out |= c[..., j] << (bits * j)
    return out


def build_cache_oracle(rng, G, lengths, msl, Hkv, D, bits, R, scales=None):
    """Caches filled by the oracle's token-form append with seeded inputs.  Returns (ck, kn, cv, vn)."""
    kv_dim = Hkv * D
    if scales is None:
        scales = np.ones(kv_dim, np.float32)
    ck, kn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    cv, vn = tqo.alloc_cache(G, msl, Hkv, D, bits)
    for g, n in enumerate(lengths):
        if n <= 0:
            continue
        k = (rng.standard_normal((n, kv_dim), dtype=np.float32) * scales).astype(np.float16)
        v = rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16)
        pos = np.arange(n, dtype=np.int32)
        tqo.append_tokens(ck[g * msl:], kn[g * msl:], k, R, pos, msl, Hkv, D, bits)
        tqo.append_tokens(cv[g * msl:], vn[g * msl:], v, R, pos, msl, Hkv, D, bits)
    return ck, kn, cv, vn


def classify_code_mismatches(codes_a: np.ndarray, codes_b: np.ndarray, rot_b: np.ndarray, bits: int):
    """codes_* [...,128] unpacked; rot_b the oracle's rotated coordinates.  Returns (n_mismatch, max ulp distance
    of a mismatching coordinate from its nearest bound, n within 1 ulp)."""
    bad = codes_a != codes_b
    n = int(bad.sum())
    if n == 0:
        return 0, 0.0, 0
    ulps = tqo.ulps_to_bound(rot_b[bad], bits)
    return n, float(ulps.max()), int((ulps <= 1.0).sum())


def fp16_spacing(x: np.ndarray) -> np.ndarray:
    return np.spacing(np.abs(x).astype(np.float16)).astype(np.float32)


def assert_attention_close(got16: np.ndarray, ref16: np.ndarray, num_heads: int, head_dim: int = 128, what=""):
    """got/ref: fp16 [n, num_heads*head_dim].  max-abs <= 2e-3 (or one fp16 spacing of the reference value where
    fp16 itself is coarser than that, |x| >= 4) and per-head relative L2 error <= 1e-2."""
    a = got16.astype(np.float32).reshape(-1, num_heads, head_dim)
    b = ref16.astype(np.float32).reshape(-1, num_heads, head_dim)
    assert np.isfinite(a).all(), f"{what}: non-finite output"
    err = np.abs(a - b)
    bar = np.maximum(ATTN_ABS, fp16_spacing(b))
    worst = float(err.max())
    assert (err <= bar).all(), f"{what}: max-abs error {worst:.3e} exceeds {ATTN_ABS} (at {np.argwhere(err > bar)[:4].tolist()})"
    num = np.linalg.norm(a - b, axis=-1)
    den = np.maximum(np.linalg.norm(b, axis=-1), 1e-3)
    rel = float((num / den).max())
    assert rel <= ATTN_REL, f"{what}: relative error {rel:.3e} exceeds {ATTN_REL}"
    return worst, rel
