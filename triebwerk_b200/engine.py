"""Host mirror of the reference's ``jetson_engine.Engine`` for the KV-cache path.

Same constructor and the same names for what this path owns -- ``Engine(max_seq_len=1024, kv_bits=0)``,
``kv_bits()``, ``reset()``, ``set_arena(data_ptr, size)``, ``sleep()``, ``wake()`` (reference
engine/engine_py.cpp:21-26,40-41,95-106; engine/engine.cpp:300-317,893-1022,1609-1620) -- plus the calls the
reference makes internally per layer (``alloc_batch``, the append and the attention of
``forward_layer_batch``, engine/engine.cpp:1338,1979-2006).  Model execution (weights, sampling,
``generate_batch``) is not part of this library and raises ``NotImplementedError``.

All state lives in the C library (``tq_engine_*``); this class only holds the handle.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from ._lib import ModelShape, StepProducer, check, lib

QWEN3_0_6B = dict(num_layers=28, num_heads=16, num_kv_heads=8, head_dim=128)
QWEN3_8B = dict(num_layers=36, num_heads=32, num_kv_heads=8, head_dim=128)


class Engine:
    def __init__(self, max_seq_len: int = 1024, kv_bits: int = 0, *, num_layers: int = 28, num_heads: int = 16,
                 num_kv_heads: int = 8, head_dim: int = 128):
        self._h = C.c_void_p()
        self.shape = ModelShape(num_layers, num_heads, num_kv_heads, head_dim)
        check(lib().tq_engine_create(C.byref(self.shape), max_seq_len, kv_bits, C.byref(self._h)), "Engine()")
        self.max_seq_len = max_seq_len
        self._arena_ref = None
        self.G = 0

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                lib().tq_engine_destroy(h)
            except Exception:
                pass

    # ---- reference surface ------------------------------------------------------------------------------------------
    def kv_bits(self) -> int:
        return int(lib().tq_engine_kv_bits(self._h))

    def set_fused(self, on: bool) -> bool:
        """One launch per layer and step (default) or the two-launch form; returns the previous setting."""
        r = int(lib().tq_engine_set_fused(self._h, int(bool(on))))
        check(min(r, 0), "set_fused")
        return bool(r)

    def reset(self, zero_cache: bool = True) -> None:
        check(lib().tq_engine_reset(self._h, int(zero_cache), self._stream()), "reset")

    def set_arena(self, data_ptr: int, size: int, keep_alive=None) -> None:
        """Use caller-owned device memory (e.g. ``tensor.data_ptr()``) as the KV arena."""
        check(lib().tq_engine_set_arena(self._h, data_ptr, size), "set_arena")
        self._arena_ref = keep_alive

    def sleep(self) -> None:
        check(lib().tq_engine_sleep(self._h), "sleep")
        self._arena_ref = None
        self.G = 0

    def wake(self) -> None:
        check(lib().tq_engine_wake(self._h), "wake")

    def sleep_keep(self) -> None:
        """sleep() that keeps every sequence's written rows and the positions in host memory; wake() (library-owned
        arena) or the next alloc_batch of the same shape (caller-owned arena) brings them back."""
        check(lib().tq_engine_sleep_keep(self._h), "sleep_keep")
        self._arena_ref = None

    def export_sequence(self, seq: int, n_tokens: int) -> bytes:
        """Rows 0 .. n_tokens-1 of sequence `seq`, all layers, as a self-describing blob in the on-cache byte layout."""
        n = int(lib().tq_engine_sequence_blob_bytes(self._h, n_tokens))
        buf = (C.c_ubyte * n)()
        check(lib().tq_engine_export_sequence(self._h, seq, n_tokens, buf, n, self._stream()), "export_sequence")
        return bytes(buf)

    def import_sequence(self, seq: int, blob: bytes) -> None:
        """A blob from export_sequence into slot `seq`; the slot's position becomes the blob's token count."""
        buf = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
        check(lib().tq_engine_import_sequence(self._h, seq, buf, len(blob), self._stream()), "import_sequence")

    def model_config(self) -> dict:
        s = self.shape
        return dict(num_layers=s.num_layers, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim)

    def generate_batch(self, *a, **k):
        raise NotImplementedError("model execution is outside this library; it provides the KV-cache path only")

    generate = decode_token = prefill = load_weights = load_weights_gguf = load_config = generate_batch

    # ---- the per-layer path -------------------------------------------------------------------------------------------------
    def arena_bytes(self, G: int, max_seq_len: int, capacities: Optional[Sequence[int]] = None) -> int:
        return int(lib().tq_engine_arena_bytes(self._h, G, max_seq_len, self._caps(capacities, G)))

    def alloc_batch(self, G: int, max_seq_len: int, capacities: Optional[Sequence[int]] = None) -> None:
        check(lib().tq_engine_alloc_batch(self._h, G, max_seq_len, self._caps(capacities, G)), "alloc_batch")
        self.G = G
        self.batch_max_seq_len = max_seq_len

    def set_positions(self, positions: Sequence[int]) -> None:
        arr = (C.c_int * len(positions))(*[int(p) for p in positions])
        check(lib().tq_engine_set_positions(self._h, arr, len(positions), self._stream()), "set_positions")
        torch.cuda.current_stream().synchronize()  # arr is host memory owned by this frame

    def positions(self) -> torch.Tensor:
        """The device positions as a CPU tensor (copy)."""
        return self._view_i32(lib().tq_engine_positions(self._h), self.G).cpu()

    def status(self) -> int:
        """Device status word (0 = fine); reading clears it."""
        return int(lib().tq_engine_status(self._h, self._stream()))

    def advance(self) -> None:
        check(lib().tq_engine_advance(self._h, self._stream()), "advance")

    def set_rotation(self, r_half: torch.Tensor) -> None:
        r = r_half.detach().to("cpu", torch.float16).contiguous()
        assert r.shape == (128, 128)
        check(lib().tq_engine_set_rotation(self._h, r.data_ptr(), self._stream()), "set_rotation")

    def decode_layer(self, layer: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Append k/v [G, kv_dim] at the current positions of `layer`, then attend with q [G, q_dim]."""
        if out is None:
            out = torch.empty_like(q)
        for t in (q, k, v, out):
            assert t.is_cuda and t.is_contiguous() and t.dtype == torch.float16
        check(lib().tq_engine_decode_layer(self._h, layer, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                           self._stream()), "decode_layer")
        return out

    def attend_layer(self, layer: int, out: torch.Tensor) -> torch.Tensor:
        """Attention only, on the queries rotated by the last decode_layer call (packed modes)."""
        check(lib().tq_engine_attend_layer(self._h, layer, out.data_ptr(), self._stream()), "attend_layer")
        return out

    def attend_step(self, out: torch.Tensor) -> torch.Tensor:
        """attend_layer for every layer, out [layers, G, q_dim] (one C call, used to time the attention kernel)."""
        check(lib().tq_engine_attend_step(self._h, out.data_ptr(), self._stream()), "attend_step")
        return out

    def decode_step(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """All layers of one decode step on device buffers [layers, G, dim]."""
        for t in (q, k, v, out):
            assert t.is_cuda and t.is_contiguous() and t.dtype == torch.float16
        check(lib().tq_engine_decode_step(self._h, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                          self._stream()), "decode_step")
        return out

    def decode_step_produce(self, q_raw, k_raw, v, out, q_norm_weight, k_norm_weight, rope_cos, rope_sin, rope_dim=128,
                            eps=1e-6, biased=False, rotated_output=False):
        """decode_step on the projections' RAW outputs: per-head RMS norm (weights [layers, 128]) and rotary embedding
        (tables [positions, rope_dim / 2]) are applied inside the step; rotated_output leaves R^T to the consumer."""
        for t in (q_raw, k_raw, v, out, q_norm_weight, k_norm_weight, rope_cos, rope_sin):
            assert t.is_cuda and t.is_contiguous() and t.dtype == torch.float16
        prod = StepProducer(q_norm_weight.data_ptr(), k_norm_weight.data_ptr(), rope_cos.data_ptr(), rope_sin.data_ptr(),
                            int(rope_dim), float(eps), int(bool(biased)), int(bool(rotated_output)))
        check(lib().tq_engine_decode_step_produce(self._h, q_raw.data_ptr(), k_raw.data_ptr(), v.data_ptr(), out.data_ptr(),
                                                  C.byref(prod), self._stream()), "decode_step_produce")
        return out

    def decode_layers(self, first_layer: int, n_layers: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                      out: torch.Tensor) -> torch.Tensor:
        """The layers first_layer .. first_layer + n_layers - 1 of a decode step; q/k/v/out are the whole-step buffers
        [layers, G, dim] (the call addresses the blocks of its layers itself)."""
        for t in (q, k, v, out):
            assert t.is_cuda and t.is_contiguous() and t.dtype == torch.float16 and t.shape[0] == self.shape.num_layers
        check(lib().tq_engine_decode_layers(self._h, first_layer, n_layers, q[first_layer].data_ptr(), k[first_layer].data_ptr(),
                                            v[first_layer].data_ptr(), out[first_layer].data_ptr(), self._stream()), "decode_layers")
        return out

    def step_prepare(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
        """First phase of decode_step: every layer's append and query rotation.  False when the engine cannot split the
        step (fp16 cache, one launch per layer): use decode_layers then."""
        for t in (q, k, v):
            assert t.is_cuda and t.is_contiguous() and t.dtype == torch.float16 and t.shape[0] == self.shape.num_layers
        r = lib().tq_engine_step_prepare(self._h, q.data_ptr(), k.data_ptr(), v.data_ptr(), self._stream())
        if r == -4:  # TQ_ERR_UNSUPPORTED
            return False
        check(r, "step_prepare")
        return True

    def step_attend_layers(self, first_layer: int, n_layers: int, out: torch.Tensor) -> torch.Tensor:
        """Second phase: attention and merge of a group of layers; out is the whole-step buffer [layers, G, q_dim]."""
        assert out.is_cuda and out.is_contiguous() and out.dtype == torch.float16 and out.shape[0] == self.shape.num_layers
        check(lib().tq_engine_step_attend_layers(self._h, first_layer, n_layers, out[first_layer].data_ptr(), self._stream()),
              "step_attend_layers")
        return out

    def time_attention(self, on: bool = True) -> None:
        """Record CUDA events around the attention launch of the whole-step calls (measurement aid)."""
        check(lib().tq_engine_time_attention(self._h, int(bool(on))), "time_attention")

    def last_attention_ms(self) -> float:
        """Duration of the attention launch of the most recent whole-step call (after time_attention())."""
        import ctypes as C
        ms = C.c_float()
        check(lib().tq_engine_last_attention_ms(self._h, C.byref(ms)), "last_attention_ms")
        return float(ms.value)

    def enable_output_f32(self, on: bool = True) -> None:
        """Also keep the attention results as fp32, before their rounding to fp16 (error reports; packed modes)."""
        check(lib().tq_engine_output_f32(self._h, int(bool(on))), "output_f32")

    def last_output_f32(self, n_layers: int = 1, first_layer: int = 0):
        """numpy [n_layers, G, num_heads, head_dim] fp32 results of the last step (after enable_output_f32)."""
        import numpy as np
        s = self.shape
        out = np.empty((n_layers, self.G, s.num_heads, s.head_dim), np.float32)
        check(lib().tq_engine_read_output_f32(self._h, out.ctypes.data, first_layer, n_layers, self._stream()), "read_output_f32")
        return out

    def prefill_layer(self, layer: int, seq: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor = None):
        """One layer of a prompt's prefill (reference engine/engine.cpp:2110-2146): k/v [T, kv_dim] into positions 0..T-1 of
        the sequence's slot, then causal attention of q [T, q_stride] over them; returns out [T, q_stride]."""
        for t in (q, k, v):
            assert t.is_cuda and t.is_contiguous() and t.dtype == torch.float16
        if out is None:
            out = torch.empty_like(q)
        check(lib().tq_engine_prefill_layer(self._h, layer, seq, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                            k.shape[0], q.shape[1], self._stream()), "prefill_layer")
        return out

    def prefill_layer_batch(self, layer: int, first_seq: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor = None):
        """prefill_layer for the prompts of several sequences at once: q [n, T, q_stride], k/v [n, T, kv_dim]."""
        for t in (q, k, v):
            assert t.is_cuda and t.is_contiguous() and t.dtype == torch.float16 and t.dim() == 3
        if out is None:
            out = torch.empty_like(q)
        check(lib().tq_engine_prefill_layer_batch(self._h, layer, first_seq, k.shape[0], q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                  out.data_ptr(), k.shape[1], q.shape[2], self._stream()), "prefill_layer_batch")
        return out

    def prefill_append(self, layer: int, seq: int, k: torch.Tensor, v: torch.Tensor, first_pos: int = 0) -> None:
        """Token-form append of k/v [T, kv_dim] for one sequence (reference engine/engine.cpp:2121-2130)."""
        assert k.is_cuda and v.is_cuda and k.is_contiguous() and v.is_contiguous()
        check(lib().tq_engine_prefill_append(self._h, layer, seq, k.data_ptr(), v.data_ptr(), first_pos, k.shape[0],
                                             self._stream()), "prefill_append")

    def prefill_shared(self, layer: int, first_seq: int, n_seq: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """One prompt k/v [T, kv_dim] for the sequences first_seq .. first_seq + n_seq - 1: its whole tiles are stored once
        (in the slot of first_seq) and read by all of them; see tq_engine_prefill_shared."""
        assert k.is_cuda and v.is_cuda and k.is_contiguous() and v.is_contiguous() and k.shape == v.shape
        check(lib().tq_engine_prefill_shared(self._h, layer, first_seq, n_seq, k.data_ptr(), v.data_ptr(), k.shape[0],
                                             self._stream()), "prefill_shared")

    def prefill_append_batch(self, layer: int, first_seq: int, k: torch.Tensor, v: torch.Tensor, first_pos: int = 0) -> None:
        """Token-form append of k/v [n_seq, T, kv_dim] for the sequences first_seq .. first_seq + n_seq - 1 in one launch."""
        assert k.is_cuda and v.is_cuda and k.is_contiguous() and v.is_contiguous() and k.dim() == 3 and k.shape == v.shape
        check(lib().tq_engine_prefill_append_batch(self._h, layer, first_seq, k.shape[0], k.data_ptr(), v.data_ptr(), first_pos,
                                                   k.shape[1], self._stream()), "prefill_append_batch")

    def decode_step_host(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
                         out_host: torch.Tensor) -> torch.Tensor:
        """A whole decode step from host (ideally pinned) buffers [layers, G, dim]; returns out_host."""
        for t in (q_host, k_host, v_host, out_host):
            assert not t.is_cuda and t.is_contiguous() and t.dtype == torch.float16
        check(lib().tq_engine_decode_step_host(self._h, q_host.data_ptr(), k_host.data_ptr(), v_host.data_ptr(),
                                               out_host.data_ptr(), self._stream()), "decode_step_host")
        return out_host

    def layer_cache(self, layer: int):
        """Views of one layer's cache: (k_codes, v_codes, k_norms, v_norms) as torch tensors over arena memory."""
        k, v, kn, vn = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
        rows = C.c_longlong()
        check(lib().tq_engine_layer_ptrs(self._h, layer, C.byref(k), C.byref(v), C.byref(kn), C.byref(vn),
                                         C.byref(rows)), "layer_ptrs")
        s = self.shape
        kv_dim = s.num_kv_heads * s.head_dim
        bits = self.kv_bits()
        if bits == 0:
            return (self._view(k.value, (rows.value, kv_dim), torch.float16),
                    self._view(v.value, (rows.value, kv_dim), torch.float16), None, None)
        kvp = kv_dim // (4 if bits == 2 else 2)
        return (self._view(k.value, (rows.value, kvp), torch.uint8), self._view(v.value, (rows.value, kvp), torch.uint8),
                self._view(kn.value, (rows.value, s.num_kv_heads), torch.float16),
                self._view(vn.value, (rows.value, s.num_kv_heads), torch.float16))

    # ---- helpers ------------------------------------------------------------------------------------------------------------
    @staticmethod
    def _stream():
        return torch.cuda.current_stream().cuda_stream

    @staticmethod
    def _caps(capacities, G):
        if capacities is None:
            return None
        assert len(capacities) == G
        return (C.c_int * G)(*[int(c) for c in capacities])

    @staticmethod
    def _view(ptr: int, shape, dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= d
        nbytes = n * torch.empty(0, dtype=dtype).element_size()

        class _Mem:  # __cuda_array_interface__ lets torch wrap foreign device memory without copying
            __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}

        return torch.as_tensor(_Mem(), device="cuda").view(dtype).view(*shape)

    @classmethod
    def _view_i32(cls, ptr, n):
        return cls._view(ptr, (n,), torch.int32)
