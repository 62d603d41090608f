"""numpy front end of the CPU oracle (oracle/tq_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the cpu_baseline /
--impl reference legs of bench.py.  The product package never imports it.

All arrays cross as numpy: fp16 data as ``np.float16`` (viewed as uint16 bits at the C boundary), codes as
``np.uint8``, positions as ``np.int32``.  Cache layouts are the reference's
(engine/kernels.cu:1563-1636): codes ``[G*max_seq_len][kv_dim/vpb]``, norms ``[G*max_seq_len][Hkv]``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtq_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle (g++) if the shared object is missing or older than its source."""
    src = os.path.join(_HERE, "tq_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.tqo_half_to_float.restype = C.c_float
        _lib.tqo_half_to_float.argtypes = [C.c_uint16]
        _lib.tqo_float_to_half.restype = C.c_uint16
        _lib.tqo_float_to_half.argtypes = [C.c_float]
        _lib.tqo_quantize.restype = C.c_int
        _lib.tqo_quantize.argtypes = [C.c_float, C.c_int]
        _lib.tqo_centroid.restype = C.c_float
        _lib.tqo_centroid.argtypes = [C.c_int, C.c_int]
        _lib.tqo_ulps_to_bound.restype = C.c_float
        _lib.tqo_ulps_to_bound.argtypes = [C.c_float, C.c_int]
        _lib.tqo_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _h(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def num_threads() -> int:
    return int(lib().tqo_num_threads())


def set_num_threads(n: int) -> None:
    lib().tqo_set_num_threads(C.c_int(n))


def vpb(bits: int) -> int:
    return 4 if bits == 2 else 2


def tables(bits: int):
    n = 16 if bits == 4 else 4
    cent = np.zeros(n, np.float32)
    bnd = np.zeros(n - 1, np.float32)
    lib().tqo_tables(C.c_int(bits), _p(cent), _p(bnd))
    return cent, bnd


def rotation(seed: int = 42, d: int = 128):
    """(R fp16 [d,d], R fp32 [d,d]) from the reference's generator (engine/engine.cpp:364-392)."""
    rh = np.zeros((d, d), np.float16)
    rf = np.zeros((d, d), np.float32)
    lib().tqo_rotation_generate(C.c_uint32(seed), C.c_int(d), _p(rh), _p(rf))
    return rh, rf


def quantize(values: np.ndarray, bits: int) -> np.ndarray:
    v = np.ascontiguousarray(values, np.float32).ravel()
    f = lib().tqo_quantize
    return np.array([f(float(x), bits) for x in v], np.uint8).reshape(np.shape(values))


def ulps_to_bound(values: np.ndarray, bits: int) -> np.ndarray:
    v = np.ascontiguousarray(values, np.float32).ravel()
    f = lib().tqo_ulps_to_bound
    return np.array([f(float(x), bits) for x in v], np.float32).reshape(np.shape(values))


def alloc_cache(G: int, max_seq_len: int, num_kv_heads: int, head_dim: int, bits: int):
    kvp = num_kv_heads * head_dim // vpb(bits)
    return (np.zeros((G * max_seq_len, kvp), np.uint8), np.zeros((G * max_seq_len, num_kv_heads), np.float16))


def append_batch(cache_q, cache_norms, kv_buf, R, positions, max_seq_len, num_kv_heads, head_dim, bits,
                 want_rot=False):
    """One new token per sequence (engine/kernels.cu:1563-1636).  kv_buf: [G, kv_dim] fp16.  In place."""
    kv_buf = _h(kv_buf)
    G, kv_dim = kv_buf.shape
    positions = np.ascontiguousarray(positions, np.int32)
    rot = np.zeros((G, num_kv_heads, head_dim), np.float32) if want_rot else None
    lib().tqo_append_batch(_p(cache_q), _p(cache_norms), _p(kv_buf), _p(_h(R)), _p(positions), C.c_int(max_seq_len),
                           C.c_int(G), C.c_int(num_kv_heads), C.c_int(head_dim), C.c_int(kv_dim), C.c_int(bits),
                           _p(rot))
    return rot


def append_tokens(cache_q, cache_norms, kv_buf, R, positions, max_seq_len, num_kv_heads, head_dim, bits,
                  want_rot=False):
    """Token-form append into a single-sequence cache (engine/kernels.cu:1482-1560).  kv_buf: [T, kv_dim]."""
    kv_buf = _h(kv_buf)
    T, kv_dim = kv_buf.shape
    positions = np.ascontiguousarray(positions, np.int32)
    rot = np.zeros((T, num_kv_heads, head_dim), np.float32) if want_rot else None
    lib().tqo_append_tokens(_p(cache_q), _p(cache_norms), _p(kv_buf), _p(_h(R)), _p(positions),
                            C.c_int(max_seq_len), C.c_int(T), C.c_int(num_kv_heads), C.c_int(head_dim),
                            C.c_int(kv_dim), C.c_int(bits), _p(rot))
    return rot


def attention_batch(q, ck, cv, kn, vn, R, positions, max_seq_len, num_heads, num_kv_heads, head_dim, bits):
    """Batched decode attention (engine/kernels.cu:1641-1776).  q: [G, q_dim] fp16 -> (out fp16, out fp32)."""
    q = _h(q)
    G, q_dim = q.shape
    positions = np.ascontiguousarray(positions, np.int32)
    out = np.zeros((G, q_dim), np.float16)
    outf = np.zeros((G, num_heads, head_dim), np.float32)
    lib().tqo_attention_batch(_p(out), _p(outf), _p(q), _p(ck), _p(cv), _p(_h(kn)), _p(_h(vn)), _p(_h(R)),
                              _p(positions), C.c_int(max_seq_len), C.c_int(G), C.c_int(num_heads),
                              C.c_int(num_kv_heads), C.c_int(head_dim), C.c_int(q_dim),
                              C.c_int(num_kv_heads * head_dim), C.c_int(bits))
    return out, outf


def attention_single(q, ck, cv, kn, vn, R, pos, max_seq_len, num_heads, num_kv_heads, head_dim, bits):
    """Single-sequence decode attention (engine/kernels.cu:1779-1870).  q: [num_heads*head_dim]."""
    q = _h(q)
    out = np.zeros(num_heads * head_dim, np.float16)
    outf = np.zeros((num_heads, head_dim), np.float32)
    lib().tqo_attention_single(_p(out), _p(outf), _p(q), _p(ck), _p(cv), _p(_h(kn)), _p(_h(vn)), _p(_h(R)),
                               C.c_int(pos), C.c_int(max_seq_len), C.c_int(num_heads), C.c_int(num_kv_heads),
                               C.c_int(head_dim), C.c_int(bits))
    return out, outf


def prefill_attention(q, ck, cv, kn, vn, R, max_seq_len, num_heads, num_kv_heads, head_dim, bits):
    """Causal prefill attention over a single-sequence packed cache (engine/kernels.cu:1874-1960)."""
    q = _h(q)
    T, q_dim = q.shape
    out = np.zeros((T, q_dim), np.float16)
    outf = np.zeros((T, num_heads, head_dim), np.float32)
    lib().tqo_prefill_attention(_p(out), _p(outf), _p(q), _p(ck), _p(cv), _p(_h(kn)), _p(_h(vn)), _p(_h(R)),
                                C.c_int(T), C.c_int(max_seq_len), C.c_int(num_heads), C.c_int(num_kv_heads),
                                C.c_int(head_dim), C.c_int(q_dim), C.c_int(num_kv_heads * head_dim), C.c_int(bits))
    return out, outf


def fp16_write_batch(cache_k, cache_v, k, v, positions, max_seq_len):
    k = _h(k)
    v = _h(v)
    G, kv_dim = k.shape
    positions = np.ascontiguousarray(positions, np.int32)
    lib().tqo_fp16_write_batch(_p(cache_k), _p(cache_v), _p(k), _p(v), _p(positions), C.c_int(max_seq_len),
                               C.c_int(G), C.c_int(kv_dim))


def fp16_attention_batch(q, ck, cv, positions, max_seq_len, num_heads, num_kv_heads, head_dim):
    q = _h(q)
    G, q_dim = q.shape
    positions = np.ascontiguousarray(positions, np.int32)
    out = np.zeros((G, q_dim), np.float16)
    outf = np.zeros((G, num_heads, head_dim), np.float32)
    lib().tqo_fp16_attention_batch(_p(out), _p(outf), _p(q), _p(_h(ck)), _p(_h(cv)), _p(positions),
                                   C.c_int(max_seq_len), C.c_int(G), C.c_int(num_heads), C.c_int(num_kv_heads),
                                   C.c_int(head_dim), C.c_int(q_dim), C.c_int(num_kv_heads * head_dim))
    return out, outf


def fp16_attention_single(q, ck, cv, pos, max_seq_len, num_heads, num_kv_heads, head_dim):
    q = _h(q)
    out = np.zeros(num_heads * head_dim, np.float16)
    outf = np.zeros((num_heads, head_dim), np.float32)
    lib().tqo_fp16_attention_single(_p(out), _p(outf), _p(q), _p(_h(ck)), _p(_h(cv)), C.c_int(pos),
                                    C.c_int(max_seq_len), C.c_int(num_heads), C.c_int(num_kv_heads),
                                    C.c_int(head_dim))
    return out, outf


def fnv1a64(data: bytes) -> str:
    h = 0xCBF29CE484222325
    for b in data:
        h ^= b
        h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return f"{h:016x}"


def qk_norm_rope_batch(q, k, q_w, k_w, cos_table, sin_table, positions, num_heads, num_kv_heads, head_dim, rope_dim,
                       eps=1e-6, biased=False):
    """Per-head RMS norm and rotary embedding of the step's q [G, q_dim] and k [G, kv_dim] (fp16), as the reference's
    qk_norm_batch_kernel + rope_batch_kernel (engine/kernels.cu:880-962).  Returns new arrays."""
    q, k = _h(q).copy(), _h(k).copy()
    G, q_dim = q.shape
    kv_dim = k.shape[1]
    positions = np.ascontiguousarray(positions, np.int32)
    lib().tqo_qk_norm_rope_batch(_p(q), _p(k), _p(_h(q_w)), _p(_h(k_w)), _p(_h(cos_table)), _p(_h(sin_table)), _p(positions),
                                 C.c_int(G), C.c_int(num_heads), C.c_int(num_kv_heads), C.c_int(head_dim), C.c_int(q_dim),
                                 C.c_int(kv_dim), C.c_int(rope_dim), C.c_float(eps), C.c_int(int(biased)))
    return q, k
