"""The C-ABI library loads, exports every symbol the header declares, and validates arguments
before touching the device (these tests run without a GPU)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "rustorch_attn.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rt_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from rustorch_b200 import build, _lib
    build.build()
    return _lib.lib()


def test_header_symbols_are_exported_and_bound(lib):
    from rustorch_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.PROTOTYPES, f"{n} has no ctypes prototype"
    assert sorted(_lib.PROTOTYPES) == names


def test_version_and_error_strings(lib):
    from rustorch_b200 import _lib
    assert lib.rt_attn_version() >= 100
    for code in range(-13, 1):
        assert len(_lib.error_string(code)) > 0
    assert "dim" in _lib.error_string(_lib.RT_ERR_ZERO_DIM)


def test_validation_happens_before_any_device_work(lib):
    """Every one of these returns its validation code on a machine without a GPU."""
    from rustorch_b200 import _lib as L
    buf = (ctypes.c_float * 64)()
    p = ctypes.addressof(buf)
    z = ctypes.c_void_p
    assert lib.rt_attn_prefill_bf16(p, p, p, p, None, 1, 1, 4, 0, 0, None, None, 0, -1.0, None) == L.RT_ERR_ZERO_DIM
    assert lib.rt_attn_prefill_bf16(p, p, p, p, None, 1, 1, 4, 96, 0, None, None, 0, -1.0, None) == L.RT_ERR_UNSUPPORTED
    assert lib.rt_attn_prefill_bf16(p, p, p, p, None, 2, 4, 0, 128, 0, None, None, 0, -1.0, None) == L.RT_OK
    assert lib.rt_attn_prefill_bf16(None, p, p, p, None, 1, 1, 4, 128, 0, None, None, 0, -1.0, None) == L.RT_ERR_NULL_POINTER
    assert lib.rt_attn_prefill_bf16(p + 2, p, p, p, None, 1, 1, 4, 128, 0, None, None, 0, -1.0, None) == L.RT_ERR_ALIGNMENT
    assert lib.rt_attn_prefill_bf16(p, p, p, p, None, 1, 1, 4, 128, 6, None, None, 0, -1.0, None) == L.RT_ERR_UNSUPPORTED
    fp = ctypes.cast(p, ctypes.POINTER(ctypes.c_float))
    f = lib.rt_flash_forward_f32_host
    assert f(fp, 0, fp, 0, fp, 0, fp, 0, 1, 1, 4, 0, 0, None, 0, 0) == L.RT_ERR_ZERO_DIM
    assert f(fp, 32, fp, 16, fp, 32, fp, 32, 1, 1, 4, 8, 0, None, 0, 0) == L.RT_ERR_BUFFER_SHAPE
    assert f(fp, 32, fp, 32, fp, 32, fp, 31, 1, 1, 4, 8, 0, None, 0, 0) == L.RT_ERR_OUTPUT_SHAPE
    keep = (ctypes.c_uint8 * 3)(1, 1, 1)
    assert f(fp, 16, fp, 16, fp, 16, fp, 16, 1, 1, 4, 4, 2, keep, 3, 0) == L.RT_ERR_MASK_LEN
    assert f(fp, 0, fp, 0, fp, 0, fp, 0, 2, 4, 0, 16, 0, None, 0, 0) == L.RT_OK  # empty seq
    g = lib.rt_gqa_forward_f32_host
    assert g(fp, 20, fp, 8, fp, 8, fp, 20, 1, 5, 2, 1, 1, 4) == L.RT_ERR_HEAD_COUNT
    assert g(fp, 7, fp, 8, fp, 8, fp, 16, 1, 4, 2, 1, 1, 4) == L.RT_ERR_WRONG_INPUT_LEN
    d = lib.rt_gqa_decode_bf16
    assert d(p, p, p, p, None, None, 1, 5, 2, 128, 64, None, 3, 0, -1, -1.0, None, 0, None) == L.RT_ERR_HEAD_COUNT
    assert d(p, p, p, p, None, None, 1, 4, 2, 128, 64, None, 65, 0, -1, -1.0, None, 0, None) == L.RT_ERR_BAD_LENGTH
    assert d(p, p, p, p, None, None, 1, 4, 2, 96, 64, None, 3, 0, -1, -1.0, None, 0, None) == L.RT_ERR_UNSUPPORTED
    assert d(p, p, p, None, None, None, 1, 4, 2, 128, 64, None, 3, 0, -1, -1.0, None, 0, None) == L.RT_ERR_NULL_POINTER
    assert d(p, p, p, p, None, None, 1, 4, 2, 128, 4096, None, 3, 0, -1, -1.0, None, 0, None) == L.RT_ERR_WORKSPACE
    assert lib.rt_gqa_decode_workspace_bytes(1, 4, 2, 128, 64) == 0
    # n_chunks records of B*Hq rows x (D+1) floats, then one int32 completion counter per (sequence, KV head)
    ws = lib.rt_gqa_decode_workspace_bytes(2, 32, 8, 128, 8192) - 2 * 8 * 4
    assert ws > 0 and ws % (2 * 32 * 129 * 4) == 0 and 8 <= ws // (2 * 32 * 129 * 4) <= 64
    assert lib.rt_gqa_decode_workspace_bytes(64, 32, 8, 128, 8192) == 8 * 64 * 32 * 129 * 4 + 64 * 8 * 4  # 1024-token chunks
    assert lib.rt_attn_merge_partials(p, p, 2, 4, 0, p, None, None, None) == L.RT_ERR_ZERO_DIM
    assert lib.rt_attn_merge_partials(p, p, 2, 4, 8, None, None, None, None) == L.RT_ERR_NULL_POINTER
    assert lib.rt_kv_append_bf16(p, p, p, p, 1, 2, 128, 64, 64, None, None) == L.RT_ERR_BAD_LENGTH
    assert lib.rt_debug_tc_selftest(None, p, p, p, p, 128, None) == L.RT_ERR_NULL_POINTER
    assert lib.rt_rope_kv_append_bf16(p, p, p, p, p, p, 1, 4, 2, 127, 64, 3, None, 0, None) == L.RT_ERR_UNSUPPORTED
    assert lib.rt_rope_kv_append_bf16(p, p, p, p, p, p, 1, 4, 2, 128, 64, 64, None, 0, None) == L.RT_ERR_BAD_LENGTH
    assert lib.rt_rope_kv_append_bf16(p, p, p, p, p, None, 1, 4, 2, 128, 64, 3, None, 0, None) == L.RT_ERR_NULL_POINTER
    assert lib.rt_attn_merge_records(None, 2, 4, 8, p, None, None, None) == L.RT_ERR_NULL_POINTER
    assert lib.rt_gqa_decode_record_bf16(p, p, p, None, 1, 4, 2, 128, 64, None, 3, 0, -1, -1.0, None, 0, None) == L.RT_ERR_NULL_POINTER
    assert lib.rt_gqa_decode_online_bf16_static(p, p, p, p, 32, 8, 10, 128, 1 << 20, None) == L.RT_ERR_STATIC_SCRATCH


def test_python_mirror_validates_like_the_reference():
    import numpy as np
    import rustorch_b200 as rt
    z = lambda n: np.zeros(n, dtype=np.float32)
    with pytest.raises(rt.ZeroDim):
        rt.flash_forward(rt.AttentionShape.new(1, 1, 4, 0), z(0), z(0), z(0), z(0))
    with pytest.raises(rt.BufferShapeMismatch) as e:
        rt.flash_forward(rt.AttentionShape.new(1, 1, 4, 8), z(32), z(16), z(32), z(32))
    assert (e.value.which, e.value.expected, e.value.got) == ("k", 32, 16)
    with pytest.raises(rt.PaddingLengthMismatch):
        rt.flash_forward_masked(rt.AttentionShape.new(1, 1, 4, 4), z(16), z(16), z(16), rt.Mask.padding([1, 1, 1]), z(16))
    with pytest.raises(rt.HeadCountMismatch):
        rt.gqa_forward_f32(z(20), z(8), z(8), z(20), 1, 5, 2, 1, 1, 4)
    with pytest.raises(rt.WrongInputLen):
        rt.gqa_forward_f32(z(7), z(8), z(8), z(16), 1, 4, 2, 1, 1, 4)
    # mask truth tables (mask.rs:92-157)
    assert not rt.Mask.none().is_masked(0, 5)
    c = rt.Mask.causal()
    assert c.is_masked(1, 2) and not c.is_masked(2, 2) and not c.is_masked(3, 1)
    pm = rt.Mask.padding([True, False, True])
    assert pm.is_masked(0, 1) and not pm.is_masked(0, 0) and not pm.is_masked(0, 7)
    rt.Mask.padding([]).validate(0)
    s = rt.AttentionShape.new(2, 3, 5, 7)
    assert (s.br, s.bc, s.buffer_len()) == (64, 64, 210)


def test_product_does_not_import_the_oracle():
    """The shipped package must never route through the CPU oracle."""
    pkg = os.path.join(ROOT, "rustorch_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"


def _split_args(text):
    """Top-level comma split of an argument list (no nested parentheses in these signatures)."""
    text = text.strip()
    return [a for a in (x.strip() for x in text.split(",")) if a] if text and text != "void" else []


def test_rust_binding_matches_the_header():
    """rust/attn_ffi.rs (the extern "C" block a maintainer drops into crates/rustorch-cuda/src/) declares exactly
    the functions of include/rustorch_attn.h with the same number of arguments, and rust/build.rs compiles exactly
    the translation units the in-tree build compiles."""
    import re
    from rustorch_b200 import _lib as L
    from rustorch_b200 import build
    rs = open(os.path.join(ROOT, "rust", "attn_ffi.rs")).read()
    rust = {m.group(1): len(_split_args(m.group(2)))
            for m in re.finditer(r"pub fn (\w+)\(([^)]*)\)\s*(?:->\s*[^;]+)?;", rs, re.S)}
    hdr = open(os.path.join(ROOT, "include", "rustorch_attn.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    c = {m.group(1): len(_split_args(m.group(2)))
         for m in re.finditer(r"\b(rt_\w+)\s*\(([^)]*)\)\s*;", hdr, re.S)}
    assert set(rust) == set(c), (sorted(set(c) - set(rust)), sorted(set(rust) - set(c)))
    for name, n in c.items():
        assert rust[name] == n, f"{name}: {rust[name]} arguments in rust/attn_ffi.rs, {n} in the header"
        assert len(L.PROTOTYPES[name][1]) == n, f"{name}: ctypes prototype has {len(L.PROTOTYPES[name][1])} arguments"
    b = open(os.path.join(ROOT, "rust", "build.rs")).read()
    listed = re.search(r"const SOURCES: &\[&str\] = &\[(.*?)\];", b, re.S).group(1)
    assert [s.strip().strip('"') for s in listed.split(",") if s.strip()] == build.SOURCES
    # the wrappers call only declared symbols
    wrappers = open(os.path.join(ROOT, "rust", "attention.rs")).read()
    for name in set(re.findall(r"\b(rt_\w+)\(", wrappers)):
        assert name in rust, name
