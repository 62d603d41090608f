"""CPU tests of the C-ABI library: it loads without a GPU, exports every symbol the header declares, and its
host-only entry points (rotation generator, sizing, argument checks) behave.  No kernel is launched here."""
import ctypes as C
import os
import re

import numpy as np

import triebwerk_b200 as tq
from triebwerk_b200._lib import ModelShape
from oracle import tqo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "triebwerk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b((?:launch|tq)_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    L = tq.lib()
    declared = header_functions()
    assert len(declared) >= 35
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in include/triebwerk_b200.h but not exported"
    assert sorted(tq.SYMBOLS) == declared, "the loader's symbol list and the header disagree"


def test_reference_launcher_names_present():
    # the nine launcher symbols the reference's engine.cpp declares for this path (engine/engine.cpp:128-140,164)
    L = tq.lib()
    for name in ["launch_turbo_kv_quantize", "launch_turbo_kv_quantize_batch", "launch_turbo_gqa_attention_batch",
                 "launch_turbo_gqa_attention", "launch_turbo_gqa_prefill_attention", "launch_kv_cache_write_batch",
                 "launch_gqa_attention_batch", "launch_gqa_attention"]:
        assert hasattr(L, name)


def test_rotation_bytes_equal_oracle_generator():
    r = tq.ops.rotation_matrix(42).numpy()
    rh, _ = tqo.rotation(42)
    assert (r.view(np.uint16) == rh.view(np.uint16)).all()
    r7 = tq.ops.rotation_matrix(7).numpy()
    rh7, _ = tqo.rotation(7)
    assert (r7.view(np.uint16) == rh7.view(np.uint16)).all()


def test_status_strings_and_version():
    L = tq.lib()
    assert L.tq_version() >= 100
    assert L.tq_status_string(0) == b"ok"
    for code in range(-7, 0):
        assert L.tq_status_string(code) not in (None, b"", b"ok")


def test_workspace_bytes_grow_with_batch():
    L = tq.lib()
    a = L.tq_workspace_bytes(4, 16)
    b = L.tq_workspace_bytes(64, 16)
    c = L.tq_workspace_bytes(64, 32)
    assert 0 < a < b < c
    assert L.tq_workspace_bytes(0, 16) == 0


def _engine(kv_bits, layers=2, H=16, Hkv=8, D=128, msl=64):
    h = C.c_void_p()
    shape = ModelShape(layers, H, Hkv, D)
    st = tq.lib().tq_engine_create(C.byref(shape), msl, kv_bits, C.byref(h))
    return st, h


def test_engine_create_argument_checks():
    L = tq.lib()
    st, h = _engine(4)
    assert st == 0 and L.tq_engine_kv_bits(h) == 4
    L.tq_engine_destroy(h)
    st, h = _engine(3)  # unsupported kv_bits falls back to fp16 like the reference constructor
    assert st == 0 and L.tq_engine_kv_bits(h) == 0
    L.tq_engine_destroy(h)
    st, _ = _engine(4, D=64)
    assert st == -4
    st, _ = _engine(4, H=15)
    assert st == -1
    st, _ = _engine(4, msl=0)
    assert st == -1


def test_arena_sizing_matches_layout():
    L = tq.lib()
    G, msl, layers, Hkv, D = 4, 256, 3, 8, 128
    for bits, row_bytes, norm_bytes in ((4, 512, 16), (2, 256, 16), (0, 2048, 0)):
        st, h = _engine(bits, layers=layers)
        assert st == 0
        total = L.tq_engine_arena_bytes(h, G, msl, None)
        cache = layers * 2 * G * msl * (row_bytes + norm_bytes)
        assert total >= cache
        # what is not cache (positions, workspace, staging) does not scale with the context length
        total2 = L.tq_engine_arena_bytes(h, G, 2 * msl, None)
        grow = total2 - total
        assert cache <= grow <= cache + (1 << 20) + (4 * G * 16 * 4 * 132 if bits == 0 else 0)
        # ragged capacities: rounded up to 32 rows each
        caps = (C.c_int * G)(1, 33, 64, 250)
        ragged = L.tq_engine_arena_bytes(h, G, msl, caps)
        assert ragged < total
        L.tq_engine_destroy(h)


def test_calls_before_alloc_report_state_errors():
    L = tq.lib()
    st, h = _engine(4)
    assert L.tq_engine_advance(h, None) == -5
    assert L.tq_engine_layer_ptrs(h, 0, None, None, None, None, None) == -5
    assert L.tq_engine_layer_ptrs(h, 99, None, None, None, None, None) == -1
    assert L.tq_engine_set_arena(h, None, 0) == -1
    assert L.tq_engine_set_arena(h, 0x1001, 4096) == -1  # arena must be 256-byte aligned
    L.tq_engine_destroy(h)


def test_reference_engine_links_against_this_library_for_the_path():
    """The reference's engine.cpp, compiled to an object where it lies (headers only, nothing is run), leaves a set of
    launch_* symbols undefined.  Every one of them that belongs to this path must be exported by libtriebwerk_b200.so,
    and the header's prototype must have the parameter list of the reference's own declaration (half* <-> void*,
    cudaStream_t <-> tq_stream_t).  Symbol tables and declaration text only."""
    import re
    import subprocess
    import tempfile
    ref = os.path.join(os.path.dirname(ROOT), "reference", "engine", "engine.cpp")
    if not os.path.exists(ref):
        pytest.skip("the reference tree is not present on this machine")
    with tempfile.TemporaryDirectory() as tmp:
        obj = os.path.join(tmp, "engine_ref.o")
        r = subprocess.run(["g++", "-std=c++17", "-c", "-I/usr/local/cuda/include", "-I" + os.path.dirname(ref), ref, "-o", obj],
                           capture_output=True, text=True)
        if r.returncode != 0:
            pytest.skip("the reference engine.cpp does not compile here: " + r.stderr[-200:])
        undefined = {ln.split()[-1] for ln in subprocess.check_output(["nm", "-u", obj], text=True).splitlines() if " launch_" in ln}
    path = {s for s in undefined if "turbo" in s} | (undefined & {
        "launch_gqa_attention", "launch_gqa_attention_batch", "launch_gqa_prefill_attention", "launch_kv_cache_write_batch"})
    assert len(path) == 9, sorted(path)
    import triebwerk_b200
    exported = {ln.split()[-1] for ln in subprocess.check_output(["nm", "-D", "--defined-only", triebwerk_b200._lib.LIB_PATH], text=True).splitlines()}
    assert path <= exported, f"not exported: {sorted(path - exported)}"

    def params(text, name):
        m = re.search(r"void\s+" + name + r"\s*\(([^;{]*?)\)\s*[;{]", text, re.S)
        assert m, name
        out = []
        for prm in m.group(1).split(","):
            prm = re.sub(r"=.*", "", prm).strip()
            ptr = "*" in prm
            base = "int" if re.search(r"\bint\b", prm) and not ptr else ("float*" if "float" in prm else ("int*" if re.search(r"\bint\b", prm) else
                   ("stream" if "tream" in prm and not ptr else ("ptr" if ptr else prm.split()[0]))))
            out.append(base)
        return out

    ref_text = open(ref).read()
    hdr_text = open(os.path.join(ROOT, "include", "triebwerk_b200.h")).read()
    for name in sorted(path):
        assert params(ref_text, name) == params(hdr_text, name), name
