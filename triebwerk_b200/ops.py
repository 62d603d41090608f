"""Python mirrors of the reference's kernel launchers for this path, same names and argument order
(BY571/triebwerk engine/kernels.cu:1963-2028 and :737-752, :1351-1357), taking torch CUDA tensors where the
reference takes device pointers.  Each call forwards to the identically named extern "C" symbol of
libtriebwerk_b200.so on torch's current stream.  The `attn_scratch` argument of the reference is accepted
and ignored.
"""
from __future__ import annotations

import torch

from ._lib import TqError, check, lib


def _ptr(t):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device, contiguous tensors only"
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _raise_compat(where):
    st = lib().tq_last_compat_status()
    if st != 0:
        raise TqError(st, where)


def launch_turbo_kv_quantize(cache_q, cache_norms, kv_buf, rotation, positions, max_seq_len, num_tokens,
                             num_kv_heads, head_dim, kv_dim, bits):
    lib().launch_turbo_kv_quantize(_ptr(cache_q), _ptr(cache_norms), _ptr(kv_buf), _ptr(rotation), _ptr(positions),
                                   max_seq_len, num_tokens, num_kv_heads, head_dim, kv_dim, bits, _stream())
    _raise_compat("launch_turbo_kv_quantize")


def launch_turbo_kv_quantize_batch(cache_q, cache_norms, kv_buf, rotation, positions, max_seq_len, G, num_kv_heads,
                                   head_dim, kv_dim, bits):
    lib().launch_turbo_kv_quantize_batch(_ptr(cache_q), _ptr(cache_norms), _ptr(kv_buf), _ptr(rotation),
                                         _ptr(positions), max_seq_len, G, num_kv_heads, head_dim, kv_dim, bits,
                                         _stream())
    _raise_compat("launch_turbo_kv_quantize_batch")


def launch_turbo_gqa_attention_batch(out, q, ck_q, cv_q, k_norms, v_norms, rotation, attn_scratch, pos, msl, G,
                                     num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits):
    lib().launch_turbo_gqa_attention_batch(_ptr(out), _ptr(q), _ptr(ck_q), _ptr(cv_q), _ptr(k_norms), _ptr(v_norms),
                                           _ptr(rotation), _ptr(attn_scratch), _ptr(pos), msl, G, num_heads,
                                           num_kv_heads, head_dim, q_dim, kv_dim, bits, _stream())
    _raise_compat("launch_turbo_gqa_attention_batch")


def launch_turbo_gqa_attention(q, ck_q, cv_q, k_norms, v_norms, rotation, output, attn_scratch, pos, msl, num_heads,
                               num_kv_heads, head_dim, bits):
    lib().launch_turbo_gqa_attention(_ptr(q), _ptr(ck_q), _ptr(cv_q), _ptr(k_norms), _ptr(v_norms), _ptr(rotation),
                                     _ptr(output), _ptr(attn_scratch), int(pos), msl, num_heads, num_kv_heads,
                                     head_dim, bits, _stream())
    _raise_compat("launch_turbo_gqa_attention")


def launch_turbo_gqa_prefill_attention(out, q, ck_q, cv_q, k_norms, v_norms, rotation, attn_scratch, T, msl,
                                       num_heads, num_kv_heads, head_dim, q_dim, kv_dim, bits):
    lib().launch_turbo_gqa_prefill_attention(_ptr(out), _ptr(q), _ptr(ck_q), _ptr(cv_q), _ptr(k_norms),
                                             _ptr(v_norms), _ptr(rotation), _ptr(attn_scratch), T, msl, num_heads,
                                             num_kv_heads, head_dim, q_dim, kv_dim, bits, _stream())
    _raise_compat("launch_turbo_gqa_prefill_attention")


def launch_kv_cache_write_batch(ck, cv, k, v, pos, msl, G, kv_dim):
    lib().launch_kv_cache_write_batch(_ptr(ck), _ptr(cv), _ptr(k), _ptr(v), _ptr(pos), msl, G, kv_dim, _stream())
    _raise_compat("launch_kv_cache_write_batch")


def launch_gqa_attention_batch(out, q, ck, cv, attn_scratch, pos, msl, G, num_heads, num_kv_heads, head_dim, q_dim,
                               kv_dim):
    lib().launch_gqa_attention_batch(_ptr(out), _ptr(q), _ptr(ck), _ptr(cv), _ptr(attn_scratch), _ptr(pos), msl, G,
                                     num_heads, num_kv_heads, head_dim, q_dim, kv_dim, _stream())
    _raise_compat("launch_gqa_attention_batch")


def launch_gqa_attention(q, k_cache, v_cache, output, attn_scratch, pos, max_seq_len, num_heads, num_kv_heads,
                         head_dim):
    lib().launch_gqa_attention(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(output), _ptr(attn_scratch), int(pos),
                               max_seq_len, num_heads, num_kv_heads, head_dim, _stream())
    _raise_compat("launch_gqa_attention")


# ---- native entry points ---------------------------------------------------------------------------------------------
def launch_gqa_prefill_attention(out, q, ck, cv, attn_scratch, T, msl, num_heads, num_kv_heads, head_dim, q_dim, kv_dim):
    """Causal prefill attention over an fp16 cache (reference engine/kernels.cu:1359-1362)."""
    lib().launch_gqa_prefill_attention(_ptr(out), _ptr(q), _ptr(ck), _ptr(cv), _ptr(attn_scratch), T, msl, num_heads,
                                       num_kv_heads, head_dim, q_dim, kv_dim, _stream())
    _raise_compat("launch_gqa_prefill_attention")


def rotation_matrix(seed: int = 42) -> torch.Tensor:
    """The engine's 128x128 fp16 rotation (reference engine/engine.cpp:364-392) as a CPU tensor."""
    out = torch.empty(128, 128, dtype=torch.float16)
    check(lib().tq_rotation_generate(seed, out.data_ptr()), "tq_rotation_generate")
    return out


def workspace_bytes(G: int, num_heads: int) -> int:
    return int(lib().tq_workspace_bytes(G, num_heads))


def new_workspace(G: int, num_heads: int, device="cuda") -> torch.Tensor:
    return torch.zeros(workspace_bytes(G, num_heads), dtype=torch.uint8, device=device)


def append_decode(ck_q, k_norms, cv_q, v_norms, k_buf, v_buf, q, rotation, positions, max_seq_len, num_heads,
                  num_kv_heads, bits, workspace, row_base=None, head_dim=128):
    G = positions.numel()
    q_dim = num_heads * head_dim if q is None else q.shape[-1]
    check(lib().tq_append_decode(_ptr(ck_q), _ptr(k_norms), _ptr(cv_q), _ptr(v_norms), _ptr(k_buf), _ptr(v_buf),
                                 _ptr(q), _ptr(rotation), _ptr(positions), _ptr(row_base), max_seq_len, G, num_heads,
                                 num_kv_heads, head_dim, q_dim, num_kv_heads * head_dim, bits, _ptr(workspace),
                                 workspace.numel(), _stream()), "tq_append_decode")


def decode_attention(out, ck_q, cv_q, k_norms, v_norms, rotation, positions, max_seq_len, num_heads, num_kv_heads,
                     bits, workspace, row_base=None, total_rows=None, head_dim=128):
    G = positions.numel()
    if total_rows is None:
        total_rows = ck_q.shape[0]
    check(lib().tq_decode_attention(_ptr(out), _ptr(ck_q), _ptr(cv_q), _ptr(k_norms), _ptr(v_norms), _ptr(rotation),
                                    _ptr(positions), -1, _ptr(row_base), total_rows, max_seq_len, G, num_heads,
                                    num_kv_heads, head_dim, out.shape[-1], num_kv_heads * head_dim, bits,
                                    _ptr(workspace), workspace.numel(), _stream()), "tq_decode_attention")


def workspace_status(workspace) -> int:
    return int(lib().tq_workspace_status(_ptr(workspace), _stream()))
