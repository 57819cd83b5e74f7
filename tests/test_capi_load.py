"""CPU: the C-ABI shared object builds, loads and exports every symbol include/splitd_attn.h declares;
argument validation that needs no GPU returns the documented status codes."""
import ctypes
import os
import re

import pytest

from splitd_flash_attn import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "splitd_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(splitd_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = _capi.load_library()
    declared = _declared_symbols()
    assert "splitd_fwd" in declared and "splitd_bwd" in declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/splitd_attn.h but not exported"
    assert set(_capi.EXPORTED_SYMBOLS) <= set(declared)


def test_version_and_error_string():
    lib = _capi.load_library()
    assert b"sm_100a" in lib.splitd_version()


def test_param_struct_matches_header_field_order():
    text = open(os.path.join(ROOT, "include", "splitd_attn.h")).read()
    body = text[text.index("typedef struct {") : text.index("} splitd_params;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for decl in body.split(";"):
        decl = decl.replace("typedef struct {", "").strip()
        if not decl:
            continue
        for part in decl.split(","):
            m = re.search(r"([A-Za-z_][A-Za-z0-9_]*)\s*(\[\d+\])?\s*$", part.strip())
            names.append(m.group(1))
    assert names == [f[0] for f in _capi.SplitdParams._fields_]


def test_invalid_arguments_are_rejected_without_a_gpu():
    lib = _capi.load_library()
    assert lib.splitd_fwd(None, None) == -1
    p = _capi.SplitdParams()
    assert lib.splitd_fwd(ctypes.byref(p), None) == -1  # NULL tensors
    assert b"NULL" in lib.splitd_last_error()
    p.q = p.k = p.v = p.o = 1 << 20
    p.head_dim = 384
    assert lib.splitd_fwd(ctypes.byref(p), None) == -1
    assert b"head_dim == 512" in lib.splitd_last_error()
    p.head_dim = 512
    p.heads_q, p.heads_kv = 6, 4
    assert lib.splitd_fwd(ctypes.byref(p), None) == -1
    assert b"heads_q" in lib.splitd_last_error()
    p.heads_q, p.heads_kv, p.batch, p.seqlen_q, p.seqlen_k = 8, 2, 1, 16, 16
    p.softmax_scale = 0.0
    assert lib.splitd_fwd(ctypes.byref(p), None) == -1
    p.softmax_scale = 0.1
    p.dtype = _capi.SPLITD_DTYPE_FP16
    p.dout = p.dq = p.dk = p.dv = p.lse = p.dpsum = p.lse_log2 = 1 << 20
    assert lib.splitd_bwd(ctypes.byref(p), None) == -2  # fp16 backward unsupported
