#!/usr/bin/env python
"""Benchmark of the TurboQuant KV-cache decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1|c3|c4|...]

One *step* is one full decode step of the named workload: for every attention layer, append the new K/V token
of every sequence to the packed cache (normalise, rotate, quantise, pack) and run GQA decode attention over
the whole context.  Default workload `c1`: 28 layers, 16 query / 8 KV heads, head_dim 128, 64 sequences
(16 prompts x 4 rollouts, rollouts share their first 100 tokens) at context 4096, kv_bits=4 -- 7.75 GB of cache
per GPU, read once per step.  Inputs are seeded synthetic tensors with the reference configuration's shapes
and value distributions (no model weights or datasets are available offline).

Reported on ONE JSON line (rank 0): `value` = algorithmic cache+I/O bytes of a step over all GPUs / device
time of a step with inputs resident in HBM; `e2e` = the same through the host-buffer C-ABI call
(pinned host q/k/v in, attention outputs back out, both copies inside the timed region); `roofline` for the
attention kernel (its share of the step, see the key's comment below); `cpu_baseline` = the CPU oracle (a port of
the reference's kernel arithmetic -- the reference has no CPU implementation) on a bounded sample; `sustained` =
the same step looped for two seconds with the clocks sampled; `configs` = the other benchmark configurations
measured in the same run (config 3 sharded over the N GPUs, config 4 at kv_bits 4 and 0).

With N > 1 (torchrun) every rank owns its own 64 sequences (sequences are independent: weak scaling, no
data-path collective) and the per-sequence outputs are gathered inside the timed region, one group of layers at a
time on a side stream: by copy-engine copies into every peer's buffer (triebwerk_b200.sharded.PeerCopyGatherer), or over
NCCL (LayerGroupGatherer; TQ_BENCH_GATHER=nccl); after the timed region a small ragged
batch is run both unsharded and sharded + gathered on every rank and compared (`gather_check`).
`--impl reference` times the CPU port with all host threads on rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: layers, H, Hkv, G, context, bits, prompt
    "c1": dict(layers=28, H=16, Hkv=8, G=64, L=4096, bits=4, prompt=100,
               desc="Qwen3-0.6B shape decode step: 28 layers, 64 seq x ctx 4096, kv_bits=4"),
    "c3": dict(layers=36, H=32, Hkv=8, G=32, L=8192, bits=2, prompt=100,
               desc="Qwen3-8B shape decode step: 36 layers, 32 seq per GPU x ctx 8192, kv_bits=2"),
    "c3full": dict(layers=36, H=32, Hkv=8, G=256, L=8192, bits=2, prompt=100, strong=True,
                   desc="config 3 in full: Qwen3-8B shape, 36 layers, 256 seq x ctx 8192, kv_bits=2, sequences divided among the GPUs"),
    "c4f16": dict(layers=8, H=32, Hkv=8, G=128, L=16384, bits=0, prompt=100, ragged=True,
                  desc="config 4 at kv_bits=0 (fp16 cache, 4096 B per token): 8 of the 36 layers (all 36 would need 157 GB per GPU), one "
                       "GPU's share (LPT by tokens, 1 of 8) of 1024 sequences with context ~ U{128..16384}"),
    "c1l4": dict(layers=4, H=16, Hkv=8, G=64, L=4096, bits=4, prompt=100,
                 desc="4 of the 28 layers of c1 (same per-layer shape; for profiler captures): 64 seq x ctx 4096, kv_bits=4"),
    "c2": dict(layers=4, H=16, Hkv=8, G=16, L=2048, bits=4, prompt=2048, append_only=True,
               desc="prefill append only (a slice of config 2: 16 of 512 sequences x 2048 tokens, 4 of 28 layers, K and V, kv_bits=4)"),
    "c2full": dict(layers=28, H=16, Hkv=8, G=512, L=2048, bits=4, prompt=2048, append_only=True, batch=32,
                   desc="config 2 in full, prefill append: 512 sequences x 2048 tokens x 28 layers (K and V, kv_bits=4), streamed through "
                        "in batches of 32 prompts, one launch per batch and layer; 31 GB of cache written"),
    "c2attn": dict(layers=4, H=16, Hkv=8, G=1, L=2048, bits=4, prompt=2048, prefill_attention=True,
                   desc="causal prefill attention over the packed cache of one 2048-token prompt of config 2 (16/8 heads, kv_bits=4), "
                        "4 of the 28 layers, one launcher call per layer"),
    "c2prefill": dict(layers=4, H=16, Hkv=8, G=32, L=2048, bits=4, prompt=2048, prefill_attention=True, batch=32,
                      desc="prefill of config 2's prompts through the engine handle: 32 of the 512 prompts x 2048 tokens, 4 of the 28 layers; "
                           "per layer one cache-write launch (tcgen05) and one causal-attention launch for all 32 prompts, kv_bits=4"),
    "c2attn8k": dict(layers=4, H=16, Hkv=8, G=1, L=8192, bits=4, prompt=8192, prefill_attention=True,
                     desc="causal prefill attention over the packed cache of one 8192-token prompt (16/8 heads, kv_bits=4), 4 layers"),
    "c4": dict(layers=36, H=32, Hkv=8, G=128, L=16384, bits=4, prompt=100, ragged=True,
               desc="Qwen3-8B shape, ragged decode step: 36 layers, one GPU's share (LPT by tokens, 1 of 8) of 1024 sequences with "
                    "context ~ U{128..16384}, kv_bits=4"),
    "c1f16": dict(layers=8, H=16, Hkv=8, G=64, L=4096, bits=0, prompt=100,
                  desc="kv_bits=0 twin of c1 (fp16 cache, 4096 B per token): 8 of 28 layers, 64 seq x ctx 4096"),
    "c3l4": dict(layers=4, H=32, Hkv=8, G=32, L=8192, bits=2, prompt=100,
                 desc="4 of the 36 layers of c3 (same per-layer shape; for profiler captures): 32 seq x ctx 8192, kv_bits=2"),
    "c1f16l2": dict(layers=2, H=16, Hkv=8, G=64, L=4096, bits=0, prompt=100,
                    desc="2 layers of c1f16 (same per-layer shape; for profiler captures): fp16 cache, 64 seq x ctx 4096"),
    "small": dict(layers=4, H=16, Hkv=8, G=16, L=2048, bits=4, prompt=100,
                  desc="reduced case for profiler captures: 4 layers, 16 seq x ctx 2048, kv_bits=4"),
}
D = 128
METRIC = "decode-attn HBM GB/s over 4-bit KV (% of ~8 TB/s); append tokens/s"


def ragged_lengths(w, rank):
    """Config 4's contexts: 1024 lengths ~ U{128..16384} from default_rng(0), split over 8 GPUs by longest-processing-
    time on tokens; this rank's share."""
    from triebwerk_b200.partition import lpt_partition
    lengths = np.random.default_rng(0).integers(128, 16385, size=1024)
    share = lpt_partition([int(x) for x in lengths], 8)[rank % 8]
    return [int(lengths[i]) for i in share]


def algorithmic_bytes(w, attention_only=False):
    """Bytes one step must move, per GPU: every cache byte of the context once (GQA sharing does not count
    twice), q in / out out, R once per layer; plus, for the append, the new K/V vectors in and codes+norm out."""
    vpb = 4 if w["bits"] == 2 else 2
    kvp = w["Hkv"] * D // vpb
    tokens = sum(w["lengths"]) if "lengths" in w else w["G"] * w["L"]
    if w["bits"] == 0:  # fp16 twin: 2 bytes per coordinate, no norms, no rotation
        per_layer = tokens * 4 * w["Hkv"] * D + 4 * w["G"] * w["H"] * D
        per_layer_append = w["G"] * w["Hkv"] * 2 * 512
        return per_layer if attention_only else w["layers"] * (per_layer + per_layer_append)
    per_layer_attn = tokens * (2 * kvp + 4 * w["Hkv"]) + 4 * w["G"] * w["H"] * D + 32768
    per_vec = 256 + D // vpb + 2
    per_layer_append = w["G"] * w["Hkv"] * 2 * per_vec
    if attention_only:
        return per_layer_attn
    return w["layers"] * (per_layer_attn + per_layer_append)


class ClockSampler:
    """SM clock and clock-event reasons of one GPU, sampled every few milliseconds by a thread during the timed
    region.  Read-only NVML queries; nothing is set."""
    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))

    def __init__(self, torch_index, period_s=0.005):
        self.period = period_s
        self.sm, self.bits, self.power = [], 0, []
        self.max_mhz = None
        self.thread = None
        self.stop_flag = threading.Event()
        self.nv = self.handle = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(torch_index).uuid)
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(torch_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = self.handle = None

    def _loop(self):
        nv, h = self.nv, self.handle
        reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                self.bits |= int(reasons(h))
                self.power.append(nv.nvmlDeviceGetPowerUsage(h) / 1000.0)
            except Exception:
                pass
            self.stop_flag.wait(self.period)

    def start(self):
        if self.handle is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        if self.thread is None:
            return out
        self.stop_flag.set()
        self.thread.join(timeout=2)
        if self.sm:
            out.update(sm_mhz=statistics.median(self.sm), sm_min_mhz=min(self.sm), samples=len(self.sm),
                       reasons=[name for bit, name in self.REASONS if self.bits & bit],
                       power_w_max=max(self.power) if self.power else None)
        return out


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle (a port of the reference kernels' arithmetic) on the host cores
# ------------------------------------------------------------------------------------------------------------------------
class CpuPort:
    """Decode steps of ONE layer of the workload on the CPU oracle (all host threads OpenMP gives it)."""

    def __init__(self, w, seed=0):
        from oracle import tqo
        from triebwerk_b200 import synth
        self.tqo, self.synth, self.w = tqo, synth, w
        self.cores = tqo.num_threads()
        G, L, Hkv, bits = w["G"], w["L"], w["Hkv"], w["bits"]
        kv_dim = Hkv * D
        self.rng = rng = np.random.default_rng(seed)
        self.R, _ = tqo.rotation()
        vpb = 4 if bits == 2 else 2
        # The sample's cache holds random code bytes and plausible norms: the CPU cost of attention does not depend
        # on the values, and quantising 64 x 4096 tokens on the CPU first would take longer than the sample itself.
        self.ck = rng.integers(0, 256, (G * L, kv_dim // vpb), dtype=np.uint8)
        self.cv = rng.integers(0, 256, (G * L, kv_dim // vpb), dtype=np.uint8)
        self.kn = (11.3 + rng.standard_normal((G * L, Hkv), dtype=np.float32)).astype(np.float16)
        self.vn = (11.3 + rng.standard_normal((G * L, Hkv), dtype=np.float32)).astype(np.float16)
        self.scales = synth.channel_scales(kv_dim)
        self.pos = np.full(G, L - 1, np.int32)

    def run(self, seconds):
        """Returns (GB/s by the GPU arm's algorithmic-byte formula, description, seconds per layer-step)."""
        w, tqo = self.w, self.tqo
        G, L, H, Hkv, bits = w["G"], w["L"], w["H"], w["Hkv"], w["bits"]
        per_layer = algorithmic_bytes(w) / w["layers"]
        t_total, n = 0.0, 0
        while t_total < seconds or n < 1:
            k, v = self.synth.kv_batch(self.rng, G, Hkv * D, self.scales)
            q = self.synth.q_batch(self.rng, G, H * D)
            t0 = time.perf_counter()
            tqo.append_batch(self.ck, self.kn, k, self.R, self.pos, L, Hkv, D, bits)
            tqo.append_batch(self.cv, self.vn, v, self.R, self.pos, L, Hkv, D, bits)
            tqo.attention_batch(q, self.ck, self.cv, self.kn, self.vn, self.R, self.pos, L, H, Hkv, D, bits)
            t_total += time.perf_counter() - t0
            n += 1
        sec = t_total / n
        sample = f"1 of {w['layers']} layers x all {G} sequences at context {L}: {n} layer-steps in {t_total:.1f} s"
        return per_layer / sec / 1e9, sample, sec


def workload_config(w, world, kv_bits=None):
    """The `config` object both arms print: the same keys, so that the two lines can be compared key by key."""
    vpb = 4 if w["bits"] == 2 else 2
    per_layer_mb = (sum(w["lengths"]) if "lengths" in w else w["G"] * w["L"]) * (
        4 * w["Hkv"] * D if w["bits"] == 0 else 2 * w["Hkv"] * D // vpb + 4 * w["Hkv"]) / 1e6
    return {"workload": w["desc"], "kv_bits": w["bits"] if kv_bits is None else kv_bits, "sequences_per_gpu": w["G"],
            "context": w["L"] if "lengths" not in w else "ragged, %d tokens" % sum(w["lengths"]), "layers": w["layers"],
            "l2": "inputs larger than L2 (one layer's cache is %.0f MB, 126 MB L2)" % per_layer_mb,
            "parallelism": f"sequence-sharded x{world}" if world > 1 else "1 GPU"}


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    from oracle import tqo
    # a launcher may export OMP_NUM_THREADS=1 to every rank; this arm runs on rank 0 alone and takes every host core
    tqo.set_num_threads(len(os.sched_getaffinity(0)))
    port = CpuPort(w)
    NL = w["layers"]

    def one_step():
        """All layers of a decode step: the one-layer sample run once per layer (every layer has the same shape and
        cost; the cache holds random codes, see CpuPort)."""
        t = 0.0
        for _ in range(NL):
            _, _, sec = port.run(0.0)
            t += sec
        return t

    for _ in range(min(1, args.warmup)):
        port.run(0.0)  # pages the library and the cache in; CPU timings need no more warm-up than that
    secs = [one_step() for _ in range(max(1, args.steps))]
    sec = float(np.mean(secs))
    value = algorithmic_bytes(w) / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8 codes, f32 math",
        "data": "synthetic", "config": workload_config(w, 1),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": port.cores, "kind": "port",
                         "sample": "CPU port of the reference kernels' arithmetic (the reference ships no CPU implementation of "
                                   f"this path); every step runs all {NL} layers x {w['G']} sequences at context {w['L']} (append K, "
                                   "append V, attention), one layer after the other on the same random-code cache"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------------------------
def build_engine(w, device_seed):
    import torch
    import triebwerk_b200 as tq
    from triebwerk_b200 import synth
    G, L, H, Hkv, bits, NL = w["G"], w["L"], w["H"], w["Hkv"], w["bits"], w["layers"]
    kv_dim = Hkv * D
    eng = tq.Engine(L, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    gen = torch.Generator(device="cuda").manual_seed(device_seed)
    scales = torch.from_numpy(synth.channel_scales(kv_dim)).cuda()
    if w.get("ragged"):
        # per-sequence slots: the arena holds the sum of the contexts, not G x the longest one
        lengths = w["lengths"]
        eng.alloc_batch(G, L, lengths)
        pool_k, pool_v = synth.torch_kv(gen, L, kv_dim, scales)  # one random pool, sliced per sequence and layer
        for layer in range(NL):
            for g, n in enumerate(lengths):
                off = (37 * layer + 101 * g) % 64
                if n > 1:
                    eng.prefill_append(layer, g, pool_k[off:off + n - 1] if off + n - 1 <= L else pool_k[:n - 1],
                                       pool_v[off:off + n - 1] if off + n - 1 <= L else pool_v[:n - 1], 0)
        eng.set_positions([n - 1 for n in lengths])
        torch.cuda.synchronize()
        return eng, gen, scales
    eng.alloc_batch(G, L)
    prompt = w["prompt"]
    # The cache is produced by the library's own append (prefill form), not filled with random bytes.
    for layer in range(NL):
        for g0 in range(0, G, 4):
            kp, vp = synth.torch_kv(gen, prompt, kv_dim, scales)  # prompt shared by the 4 rollouts
            for g in range(g0, min(g0 + 4, G)):
                eng.prefill_append(layer, g, kp, vp, 0)
                kd, vd = synth.torch_kv(gen, L - 1 - prompt, kv_dim, scales)
                eng.prefill_append(layer, g, kd, vd, prompt)
    eng.set_positions([L - 1] * G)
    torch.cuda.synchronize()
    return eng, gen, scales


def measure_append(args, w, rank, local_rank):
    """Config 2's shape: whole prompts appended to the packed cache (token-mode append kernel), nothing attended.
    One step = every sequence's 2048 tokens through the layers of the slice.  Returns the figures of the timed steps."""
    import torch
    import triebwerk_b200 as tq
    from triebwerk_b200 import synth

    torch.cuda.set_device(local_rank)
    G, T, H, Hkv, bits, NL = w["G"], w["L"], w["H"], w["Hkv"], w["bits"], w["layers"]
    kv_dim = Hkv * D
    eng = tq.Engine(T, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(G, T)
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    scales = torch.from_numpy(synth.channel_scales(kv_dim)).cuda()
    B = w.get("batch", G)  # prompts per launch: the K/V of one batch (reused for every layer and batch) are the step's input
    kp, vp = synth.torch_kv(gen, B * T, kv_dim, scales)
    kp, vp = kp.view(B, T, kv_dim), vp.view(B, T, kv_dim)
    per_sequence = os.environ.get("TQ_BENCH_PREFILL_PER_SEQUENCE", "0") != "0"

    def step():
        for first in range(0, G, B):
            for layer in range(NL):
                if per_sequence:  # one launch per sequence and layer, as the reference's prefill loop does
                    for g in range(B):
                        eng.prefill_append(layer, first + g, kp[g], vp[g], 0)
                else:             # one launch per layer for all the prompts of the batch
                    eng.prefill_append_batch(layer, first, kp, vp, 0)

    big = G * T * NL > 1 << 24
    for _ in range(1 if big else max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    steps = max(1, min(args.steps, 3 if big else 10))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()  # a profiler started with its capture off sees exactly the timed steps
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    assert eng.status() == 0
    vectors = NL * G * T * 2 * Hkv
    vpb = 4 if bits == 2 else 2
    bytes_step = vectors * (256 + D // vpb + 2)
    del eng, kp, vp
    torch.cuda.empty_cache()
    return {"ms": ms, "steps": steps, "warmup": 1 if big else max(3, args.warmup), "vectors": vectors, "bytes_step": bytes_step,
            "clocks": clocks, "per_sequence": per_sequence, "launches": steps * NL * (G if per_sequence else G // B), "vpb": vpb}


def run_append_only(args, w, rank, world, local_rank):
    r = measure_append(args, w, rank, local_rank)
    ms, steps, vectors, bytes_step, clocks, per_sequence, vpb = (r[k] for k in ("ms", "steps", "vectors", "bytes_step", "clocks",
                                                                                "per_sequence", "vpb"))
    Hkv, bits = w["Hkv"], w["bits"]
    peak, peak_kind = measured_peaks()
    value = bytes_step / (ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": r["warmup"],
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 in, tcgen05 f16 x f16 -> f32 (+ exact f32 chain near bounds), u8 codes", "data": "synthetic",
        "config": {"workload": w["desc"], "kv_bits": bits, "l2": "every step rewrites %.0f MB of cache" % (vectors * (D // vpb + 2) / 1e6)},
        "head_vectors_per_s": vectors / (ms * 1e-3),
        "append_tokens_per_s_28_layers": vectors / (ms * 1e-3) / (28 * 2 * Hkv),
        "fp32_tflops": vectors * 2 * D * D / (ms * 1e-3) / 1e12,
        "gpu_launches": r["launches"],
        "roofline": {"kernel": "prefill_append_tc_kernel (tcgen05)", "bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s",
                     "frac": value / peak, "peak_kind": peak_kind, "traffic": None,
                     "note": ("one launch per sequence and layer (2048 tokens = 256 tiles = one wave): launch and set-up bound"
                              if per_sequence else "one launch per layer for all prompts; instruction-issue bound, not HBM bound")},
        "clocks": clocks,
    }
    print(json.dumps(line))


def run_prefill_attention(args, w, rank, world, local_rank):
    """Prefill attention of whole prompts through the reference's launcher symbol (launch_turbo_gqa_prefill_attention):
    one step = every layer's causal attention of the prompt over its own packed cache."""
    import torch
    import triebwerk_b200 as tq
    from triebwerk_b200 import ops, synth

    torch.cuda.set_device(local_rank)
    T, H, Hkv, bits, NL = w["L"], w["H"], w["Hkv"], w["bits"], w["layers"]
    B = w.get("batch", 0)   # > 0: that many prompts per launch through the engine handle (cache write + attention)
    kv_dim, q_dim = Hkv * D, H * D
    eng = tq.Engine(T, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
    eng.alloc_batch(max(1, B), T)
    gen = torch.Generator(device="cuda").manual_seed(4321)
    scales = torch.from_numpy(synth.channel_scales(kv_dim)).cuda()
    if B:
        kp, vp = synth.torch_kv(gen, B * T, kv_dim, scales)
        kp, vp = kp.view(B, T, kv_dim), vp.view(B, T, kv_dim)
        qb = torch.randn(B, T, q_dim, generator=gen, device="cuda").to(torch.float16)
        outb = torch.empty_like(qb)

        def step():
            for layer in range(NL):
                eng.prefill_layer_batch(layer, 0, qb, kp, vp, outb)
    else:
        for layer in range(NL):
            kp, vp = synth.torch_kv(gen, T, kv_dim, scales)
            eng.prefill_append(layer, 0, kp, vp, 0)
        caches = [eng.layer_cache(layer) for layer in range(NL)]
        R = ops.rotation_matrix().cuda()
        q = torch.randn(NL, T, q_dim, generator=gen, device="cuda").to(torch.float16)
        out = torch.empty_like(q)

        def step():
            for layer in range(NL):
                ck, cv, kn, vn = caches[layer]
                ops.launch_turbo_gqa_prefill_attention(out[layer], q[layer], ck, cv, kn, vn, R, None, T, T, H, Hkv, D, q_dim, kv_dim, bits)

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    steps = max(1, min(args.steps, 20))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    NP = max(1, B)
    flops = NP * NL * 2.0 * 2.0 * D * H * T * (T + 1) / 2.0          # QK^T and PV over the causal half
    vpb = 4 if bits == 2 else 2
    bytes_step = NP * NL * (T * (2 * Hkv * D // vpb + 4 * Hkv) + 4 * T * q_dim + (4 * T * kv_dim if B else 0))
    tf_peak = None
    try:
        tf_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        tf_peak = 1590.0
    tfs = flops / (ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": bytes_step / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": 1, "steps": steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8 codes -> f16 tiles, f16 mma.sync, f32 accumulate", "data": "synthetic",
        "config": {"workload": w["desc"], "kv_bits": bits, "l2": "each step reads every layer's cache and queries again (one prompt fits L2: compute bound)"},
        "us_per_layer": ms * 1e3 / NL, "us_per_prompt_and_layer": ms * 1e3 / NL / NP, "causal_tflops": tfs,
        "gpu_launches": steps * NL * (2 if B else 1),   # (cache write +) attention, one launch each per layer
        "roofline": {"kernel": f"prefill_attention_kernel<{bits}> (mma.sync)", "bound": "tensor",
                     "achieved": tfs, "peak": tf_peak, "unit": "TFLOP/s", "frac": tfs / tf_peak,
                     "peak_kind": "measured cuBLAS bf16 (tcgen05); this kernel issues mma.sync", "traffic": None},
        "clocks": clocks,
    }
    print(json.dumps(line))


def decode_inputs(w, gen, scales):
    """Step inputs resident in HBM: q, k, v [layers, G, dim] fp16 and the output buffer."""
    import torch
    from triebwerk_b200 import synth
    G, H, Hkv, NL = w["G"], w["H"], w["Hkv"], w["layers"]
    kv_dim, q_dim = Hkv * D, H * D
    k_dev = torch.empty(NL, G, kv_dim, dtype=torch.float16, device="cuda")
    v_dev = torch.empty_like(k_dev)
    for layer in range(NL):
        k_dev[layer], v_dev[layer] = synth.torch_kv(gen, G, kv_dim, scales)
    q_dev = torch.randn(NL, G, q_dim, generator=gen, device="cuda").to(torch.float16)
    return q_dev, k_dev, v_dev, torch.empty_like(q_dev)


def make_gatherer(plan, groups, row_shape):
    """The exchange of the per-sequence outputs: copy-engine copies into the peers' buffers (TQ_BENCH_GATHER=peer, the
    default) or NCCL all-gathers (=nccl, and whenever the peer buffers cannot be set up).  Returns (gatherer, kind)."""
    from triebwerk_b200 import sharded
    if os.environ.get("TQ_BENCH_GATHER", "peer") == "peer":
        try:
            return sharded.PeerCopyGatherer(plan, groups, row_shape), "peer_copy"
        except RuntimeError as e:   # raised on every rank together (the set-up is collective)
            sys.stderr.write(f"peer-copy exchange unavailable, using NCCL: {e}\n")
    return sharded.LayerGroupGatherer(plan, groups), "nccl"


def measure_decode(args, w, rank, world, local_rank, steps, warmup, full=True):
    """Builds the workload's cache on this rank and times its decode step.  full: also the host-buffer (e2e) path, the
    two-second sustained loop and the clocks; otherwise only the device-timed step (the extra configurations)."""
    import torch
    import torch.distributed as dist
    from triebwerk_b200 import sharded

    if w.get("ragged"):
        w = dict(w, lengths=ragged_lengths(w, rank))
        w["G"] = len(w["lengths"])
    if w.get("strong"):
        w = dict(w, G=w["G"] // world)  # the configuration's sequences divided among the ranks
    G, L, H, Hkv, bits, NL = w["G"], w["L"], w["H"], w["Hkv"], w["bits"], w["layers"]
    kv_dim, q_dim = Hkv * D, H * D
    eng, gen, scales = build_engine(w, 1234 + rank)
    q_dev, k_dev, v_dev, out_dev = decode_inputs(w, gen, scales)

    # N > 1: the per-sequence outputs of all ranks are gathered (NCCL) one group of layers at a time on a side stream
    # while the next group is computed; the groups are set by TQ_BENCH_GATHER_GROUPS (default 3: two groups of layers, then the
    # last, then the last one, whose exchange is the only one left exposed)
    gat, groups, gat_kind = None, [(0, NL)], None
    if world > 1:
        n_groups = int(os.environ.get("TQ_BENCH_GATHER_GROUPS", "3"))
        groups = sharded.layer_groups(NL, n_groups)
        gat, gat_kind = make_gatherer(sharded.contiguous_partition(world * G, world), groups, (q_dim,))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_compute():
        eng.decode_step(q_dev, k_dev, v_dev, out_dev)

    def step_device():
        if gat is None:
            return step_compute()
        split = eng.step_prepare(q_dev, k_dev, v_dev)   # every layer's append and query rotation first, once
        for gi, (l0, l1) in enumerate(groups):
            if split:
                eng.step_attend_layers(l0, l1 - l0, out_dev)
            else:
                eng.decode_layers(l0, l1 - l0, q_dev, k_dev, v_dev, out_dev)
            gat.gather(gi, out_dev[l0:l1])
        gat.finish()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / n

    for _ in range(max(3, warmup)):
        step_device()
    barrier()
    if full:
        # The step looped for two seconds first: the timed steps that follow run on a GPU that is already as warm
        # (and as power-capped) as a long decode loop makes it, not on a cold burst.  Nothing is set, only sampled.
        hot = ClockSampler(local_rank, period_s=0.02) if rank == 0 else None
        n_hot = max(steps, int(2000.0 / max(timed(step_device, 3), 1e-3)) + 1)
        if hot:
            hot.start()
        ms_hot = timed(step_device, n_hot)
        hc = hot.stop() if hot else None
        sustained = {"seconds": ms_hot * n_hot / 1e3, "steps": n_hot, "ms_per_step": ms_hot,
                     "value": world * algorithmic_bytes(w) / (ms_hot * 1e-3) / 1e9, "clocks": hc,
                     "ms_x_mhz": (ms_hot * hc["sm_mhz"]) if hc and hc.get("sm_mhz") else None,
                     "note": "runs directly before the timed steps; the timed steps inherit its clocks"}
    sampler = ClockSampler(local_rank) if (rank == 0 and full) else None
    if sampler:
        sampler.start()
    torch.cuda.profiler.start()  # a profiler started with its capture off sees exactly the timed steps
    ms_step = timed(step_device, steps)
    torch.cuda.profiler.stop()
    clocks = sampler.stop() if sampler else None
    res = {"w": w, "ms_step": ms_step, "clocks": clocks, "bytes_step": algorithmic_bytes(w)}
    # the step without the exchange (for the kernel's own launch duration at N > 1)
    res["ms_compute"] = ms_step if world == 1 else timed(step_compute, steps)
    # the attention launch alone: CUDA events recorded by the library on the launching stream directly before and after it
    # (whole-step form of the packed modes), averaged over steps that follow the timed ones at once
    res["ms_attn_launch"] = None
    if full and bits != 0 and os.environ.get("TQ_WHOLE_STEP", "1") != "0" and os.environ.get("TQ_FUSED", "1") != "0":
        eng.time_attention(True)
        samples = []
        for _ in range(max(10, min(steps, 50))):
            step_compute()
            samples.append(eng.last_attention_ms())
        eng.time_attention(False)
        res["ms_attn_launch"] = sum(samples) / len(samples)

    res["variants"] = None
    if full and world == 1 and bits != 0 and res["ms_attn_launch"]:
        # the step that takes the projections' raw outputs (per-head RMS norm and rotary embedding inside it), and the
        # same with the inverse rotation left to the consumer's weights
        nw_q = (1.0 + 0.1 * torch.randn(NL, D, generator=gen, device="cuda")).to(torch.float16)
        nw_k = (1.0 + 0.1 * torch.randn(NL, D, generator=gen, device="cuda")).to(torch.float16)
        ang = torch.arange(L, device="cuda", dtype=torch.float32)[:, None] * (1e6 ** (-torch.arange(D // 2, device="cuda", dtype=torch.float32) / (D // 2)))[None]
        rc, rs = ang.cos().to(torch.float16).contiguous(), ang.sin().to(torch.float16).contiguous()
        var = {}
        for name, rot_out in (("produce", False), ("produce_rotated_output", True)):
            fn = lambda: eng.decode_step_produce(q_dev, k_dev, v_dev, out_dev, nw_q, nw_k, rc, rs, D, 1e-6, False, rot_out)
            for _ in range(3):
                fn()
            var[name] = {"ms_per_step": timed(fn, max(10, min(steps, 50)))}
        var["note"] = ("tq_engine_decode_step_produce on the same workload: QK-norm and rotary embedding of the reference's "
                       "launch_qk_norm_batch + launch_rope_batch happen inside the step's own four launches")
        res["variants"] = var
    if full:
        q_host, k_host, v_host = (t.cpu().pin_memory() for t in (q_dev, k_dev, v_dev))
        out_host = torch.empty(NL, G, q_dim, dtype=torch.float16).pin_memory()

        def step_host():
            eng.decode_step_host(q_host, k_host, v_host, out_host)

        for _ in range(2):
            step_host()
        res["ms_e2e"] = timed(step_host, max(1, steps))
        res["sustained"] = sustained
    status = eng.status()
    assert status == 0, f"device status word is {status}: a kernel gave up on a bounded wait or saw a bad position"
    res["gather"] = gat_kind
    if gat_kind == "peer_copy":
        assert gat.status() == 0, "a wait for the peers' copies ran out of time"
        gat.close()
    del eng, q_dev, k_dev, v_dev, out_dev
    torch.cuda.empty_cache()
    return res


def gather_check(rank, world):
    """A small ragged batch run twice on every rank: all sequences on this GPU, and only this rank's shard
    (sharded.shard_plan) with the outputs gathered (make_gatherer).  Returns the largest
    difference between the two results and whether the shard's cache bytes equal the unsharded run's."""
    import torch
    import torch.distributed as dist
    import triebwerk_b200 as tq
    from triebwerk_b200 import sharded, synth

    H, Hkv, NL, bits, msl = 16, 8, 3, 4, 768
    kv_dim, q_dim = Hkv * D, H * D
    lengths = [int(x) for x in np.random.default_rng(5).integers(40, 700, size=13)]
    n_seq = len(lengths)
    plan = sharded.shard_plan(lengths, world)
    gen = torch.Generator(device="cuda").manual_seed(99)  # the same data on every rank
    scales = torch.from_numpy(synth.channel_scales(kv_dim)).cuda()
    prompts = [[synth.torch_kv(gen, n - 1, kv_dim, scales) for n in lengths] for _ in range(NL)]
    k_new = torch.stack([synth.torch_kv(gen, n_seq, kv_dim, scales)[0] for _ in range(NL)])
    v_new = torch.randn(NL, n_seq, kv_dim, generator=gen, device="cuda").to(torch.float16)
    q = torch.randn(NL, n_seq, q_dim, generator=gen, device="cuda").to(torch.float16)

    def run(ids):
        eng = tq.Engine(msl, bits, num_layers=NL, num_heads=H, num_kv_heads=Hkv, head_dim=D)
        eng.alloc_batch(len(ids), msl, [lengths[i] for i in ids])
        for layer in range(NL):
            for j, i in enumerate(ids):
                eng.prefill_append(layer, j, prompts[layer][i][0], prompts[layer][i][1], 0)
        eng.set_positions([lengths[i] - 1 for i in ids])
        idx = torch.as_tensor(ids, device="cuda", dtype=torch.long)
        out = torch.empty(NL, len(ids), q_dim, dtype=torch.float16, device="cuda")
        eng.decode_step(q[:, idx].contiguous(), k_new[:, idx].contiguous(), v_new[:, idx].contiguous(), out)
        rows = []  # the written rows of every sequence, all four arrays
        for layer in range(NL):
            arrays = eng.layer_cache(layer)
            base = 0
            per_seq = []
            for i in ids:
                cap = (lengths[i] + 31) // 32 * 32
                per_seq.append([a[base:base + lengths[i]].clone() for a in arrays])
                base += cap
            rows.append(per_seq)
        assert eng.status() == 0
        return out, rows

    out_all, rows_all = run(list(range(n_seq)))
    mine = plan[rank]
    out_loc, rows_loc = run(mine)
    groups = sharded.layer_groups(NL, 2)
    gat, kind = make_gatherer(plan, groups, (q_dim,))
    for gi, (l0, l1) in enumerate(groups):
        gat.gather(gi, out_loc[l0:l1].contiguous())
    gat.finish()
    torch.cuda.synchronize()
    got = gat.result()
    if kind == "peer_copy":
        assert gat.status() == 0, "a wait for the peers' copies ran out of time"
        gat.close()
    diff = float((got.float() - out_all.float()).abs().max())
    same = all(torch.equal(a, b) for layer in range(NL) for j, i in enumerate(mine)
               for a, b in zip(rows_loc[layer][j], rows_all[layer][i]))
    t = torch.tensor([diff, 0.0 if same else 1.0], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"max_abs": float(t[0].item()), "cache_bytes_equal": bool(t[1].item() == 0.0), "sequences": n_seq,
            "layers": NL, "shards": [len(p) for p in plan], "exchange": kind}


def run_ours(args, w, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    steps, warmup = args.steps, max(3, args.warmup)
    res = measure_decode(args, w, rank, world, local_rank, steps, warmup, full=True)
    w = res["w"]
    G, L, H, Hkv, bits, NL = w["G"], w["L"], w["H"], w["Hkv"], w["bits"], w["layers"]
    kv_dim, q_dim = Hkv * D, H * D
    ms_step = res["ms_step"]

    # The other benchmark configurations, measured in the same run (device-timed step only).
    extras = {}
    if args.workload == "c1" and not args.no_extras:
        for key, name in (("c3", "c3full"), ("c4_4bit", "c4"), ("c4_fp16", "c4f16")):
            r = measure_decode(args, WORKLOADS[name], rank, world, local_rank, 5, 3, full=False)
            we = r["w"]
            val = world * r["bytes_step"] / (r["ms_step"] * 1e-3) / 1e9
            extras[key] = {"workload": we["desc"], "kv_bits": we["bits"], "sequences_per_gpu": we["G"],
                           "tokens_per_gpu": sum(we["lengths"]) if "lengths" in we else we["G"] * we["L"], "layers": we["layers"],
                           "scaling": "strong" if we.get("strong") else "weak", "ms_per_step": r["ms_step"],
                           "ms_per_step_without_gather": r["ms_compute"], "value": val, "unit": "GB/s",
                           "frac_of_measured_hbm_per_gpu": val / world / measured_peaks()[0]}
        if world == 1:  # the prompt append of config 2 (a slice: 16 prompts x 2048 tokens, 4 layers), tcgen05 kernel
            wa = WORKLOADS["c2"]
            ra = measure_append(args, wa, rank, local_rank)
            val = ra["bytes_step"] / (ra["ms"] * 1e-3) / 1e9
            extras["c2_prefill_append"] = {"workload": wa["desc"], "kv_bits": wa["bits"], "ms_per_step": ra["ms"], "value": val, "unit": "GB/s",
                                           "head_vectors_per_s": ra["vectors"] / (ra["ms"] * 1e-3),
                                           "frac_of_measured_hbm_per_gpu": val / measured_peaks()[0]}
    check = gather_check(rank, world) if world > 1 else None
    if rank != 0:
        return
    bytes_step = res["bytes_step"]
    value = world * bytes_step / (ms_step * 1e-3) / 1e9
    e2e = world * bytes_step / (res["ms_e2e"] * 1e-3) / 1e9
    peak, peak_kind = measured_peaks()
    fused = os.environ.get("TQ_FUSED", "1") != "0" and bits != 0
    whole = fused and os.environ.get("TQ_WHOLE_STEP", "1") != "0"
    # The dominant kernel.  Whole-step form (default, packed modes): ONE attention launch streams all layers; its
    # duration is measured with CUDA events recorded directly around it (tq_engine_time_attention).  Other forms: the
    # step holds small launches beside the attention, so the kernel's time per layer is bounded above by the device
    # time of the step / layers, which is then what is reported (at N > 1: of the step without the exchange).
    kernel_bytes = bytes_step // NL
    attn_ms = res["ms_compute"] / NL
    timed_by = "step time / layers (upper bound: the step's other launches are included)"
    if res.get("ms_attn_launch"):
        kernel_bytes = algorithmic_bytes(w, attention_only=True)
        attn_ms = res["ms_attn_launch"] / NL
        timed_by = "CUDA events on the launching stream directly around the attention launch, mean over the steps after the timed ones"
    achieved = kernel_bytes / (attn_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8 codes, f16 mma, f32 accumulate" if bits else "f16 cache, f32 math", "data": "synthetic",
        "config": workload_config(w, world),
        "pct_of_8TBs": 100.0 * value / world / 8000.0,
        "append_tokens_per_s": world * G / (ms_step * 1e-3),
        "e2e": {"value": e2e, "unit": "GB/s", "ms_per_step": res["ms_e2e"],
                "h2d_bytes_per_step": int(world * NL * G * (q_dim + 2 * kv_dim) * 2),
                "d2h_bytes_per_step": int(world * NL * G * q_dim * 2)},
        # kernels of this library launched inside the timed region (none of anybody else's but NCCL's at N > 1)
        "gpu_launches": int(steps * ((4 if world == 1 else 2 + 2 * len(sharded_groups(NL, world))) if whole else NL * (1 if fused else 2))),
        "roofline": {"kernel": "fp16_cache_write_kernel + fp16_decode_attention_kernel" if bits == 0 else
                     f"decode_attention_kernel<{bits}>" + (" (whole-step form: one launch streams all layers; per layer)" if whole else
                                                           " (one launch per layer: append + query rotation + attention)" if fused else ""),
                     "bound": "hbm", "achieved": achieved, "peak": peak, "timed_by": timed_by,
                     "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "frac_of_8TBs": achieved / 8000.0,
                     "us_per_launch": attn_ms * 1e3 * (NL if whole else 1), "us_per_layer": attn_ms * 1e3,
                     "algorithmic_bytes_per_launch": kernel_bytes * (NL if whole else 1), "algorithmic_bytes_per_layer": kernel_bytes,
                     "traffic": (lambda t: t * (NL if whole else 1) if t else None)(TRAFFIC_PER_LAYER.get(args.workload))},
        "clocks": res["clocks"],
        "sustained": res["sustained"],
    }
    if res.get("variants"):
        line["step_variants"] = res["variants"]
    if world > 1:
        line["exchange"] = {"kind": res.get("gather"), "layer_groups": len(sharded_groups(NL, world)),
                            "ms_per_step_without_exchange": res["ms_compute"],
                            "bytes_per_rank_and_step": int(NL * G * q_dim * 2),
                            "note": "peer_copy: copy-engine copies into every peer's buffer + flag words; nccl: all_gather_into_tensor"}
    if extras:
        line["configs"] = extras
    if check is not None:
        line["gather_check"] = check
    if args.cpu_seconds > 0 and world == 1:
        from oracle import tqo
        tqo.set_num_threads(len(os.sched_getaffinity(0)))
        port = CpuPort(w)
        gbs, sample, _ = port.run(args.cpu_seconds)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": port.cores, "kind": "port", "sample": sample}
    print(json.dumps(line))


def sharded_groups(n_layers, world):
    from triebwerk_b200 import sharded
    return [(0, n_layers)] if world == 1 else sharded.layer_groups(n_layers, int(os.environ.get("TQ_BENCH_GATHER_GROUPS", "3")))


# dram__bytes_read.sum + dram__bytes_write.sum of the attention kernel PER LAYER from the ncu captures summarised under
# profiles/ (a capture covers a launch over 4 layers of the same per-layer shape), or absent while no capture exists.
TRAFFIC_PER_LAYER = {
    "c1": 281445338, "c1l4": 281445338,   # 4-layer launch: 1111.2 MB read + 14.6 MB written
    "c3l4": 148555328, "c3": 148555328,   # 4-layer launch of 32 sequences x 8192, 2-bit: 573.9 MB read + 20.4 MB written
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="length of the CPU-baseline sample (0 = skip)")
    ap.add_argument("--no-extras", action="store_true", help="default workload only: skip the other configurations")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if w.get("append_only") or w.get("prefill_attention"):
            if rank == 0:
                (run_append_only if w.get("append_only") else run_prefill_attention)(args, w, rank, world, local_rank)
        else:
            run_ours(args, w, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
