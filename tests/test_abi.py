"""The C-ABI library loads, exports what include/jq.h declares, and rejects
bad arguments on the host before anything is launched (no GPU needed)."""
import ctypes
import os
import re

import numpy as np

from if_i_could_turn_back_time_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "jq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(jq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared_functions()
    assert "jq_gemv_e2m1" in names and "jq_gemv_gf4" in names and "jq_gemv_grouped" in names
    lib = ctypes.CDLL(_lib.lib_path())
    for n in names:
        assert hasattr(lib, n), f"{n} declared in jq.h but not exported"
    assert sorted(_lib.exported_symbols()) == names, "ctypes table and jq.h disagree"


def test_version_and_error_text():
    lib = _lib.load()
    assert lib.jq_version() == 100
    assert _lib.strerror(0) == "ok"
    for code in range(-8, 0):
        assert _lib.strerror(code) not in ("", "unknown status")
    assert "unknown" in _lib.strerror(-999)


def test_host_side_validation_needs_no_gpu():
    lib = _lib.load()
    buf = np.zeros(4096, dtype=np.uint8)
    p = buf.ctypes.data  # 64-byte aligned host address: only used for argument checks
    assert p % 16 == 0
    # null pointers
    assert lib.jq_gemv_e2m1(None, p, p, None, p, 8, 64, 1, 32, 0, 0, 0, None, 0, None) == -1
    assert lib.jq_gemv_gf4(p, p, None, p, None, p, 8, 128, 1, 128, 0, 0, 0, None, 0, None) == -1
    # shapes: K not a multiple of g, g not a multiple of 32, e2m1 without groups
    assert lib.jq_gemv_e2m1(p, p, p, None, p, 8, 100, 1, 32, 0, 0, 0, None, 0, None) == -2
    assert lib.jq_gemv_e2m1(p, p, p, None, p, 8, 64, 1, 16, 0, 0, 0, None, 0, None) == -2
    assert lib.jq_gemv_e2m1(p, p, p, None, p, 8, 64, 1, 0, 0, 0, 0, None, 0, None) == -2
    assert lib.jq_gemv_e2m1(p, p, p, None, p, 0, 64, 1, 32, 0, 0, 0, None, 0, None) == -2
    assert lib.jq_gemv_e2m1(p, p, p, None, p, 8, 64, 0, 32, 0, 0, 0, None, 0, None) == -2
    # rotation block other than 128, or K not a multiple of it
    assert lib.jq_gemv_e2m1(p, p, p, None, p, 8, 64, 1, 32, 64, 0, 0, None, 0, None) == -5
    assert lib.jq_gemv_e2m1(p, p, p, None, p, 8, 64, 1, 32, 128, 0, 0, None, 0, None) == -2
    # misaligned packed weights
    assert lib.jq_gemv_e2m1(p + 4, p, p, None, p, 8, 64, 1, 32, 0, 0, 0, None, 0, None) == -3
    # element types
    assert lib.jq_gemv_e2m1(p, p, p, None, p, 8, 64, 1, 32, 0, 7, 0, None, 0, None) == -4
    # dequant / fwht
    assert lib.jq_dequant_e2m1(None, p, p, 8, 64, 32, None) == -1
    assert lib.jq_dequant_gf4(p, None, p, p, 8, 64, 32, None) == -1
    assert lib.jq_fwht_block(p, p, 1, 100, 128, 0, None) == -2
    assert lib.jq_fwht_block(p, p, 1, 128, 64, 0, None) == -5


def test_host_packer_argument_checks():
    lib = _lib.load()
    W = np.zeros((2, 64), dtype=np.float32)
    q = np.zeros((2, 32), dtype=np.uint8)
    s = np.zeros((2, 2), dtype=np.uint16)
    assert lib.jq_pack_e2m1_host(None, 2, 64, 32, q.ctypes.data, s.ctypes.data, 1) == -1
    assert lib.jq_pack_e2m1_host(W.ctypes.data, 2, 64, 48, q.ctypes.data, s.ctypes.data, 1) == -2
    assert lib.jq_pack_gf4_host(W.ctypes.data, 2, 64, 32, q.ctypes.data, None, s.ctypes.data, 1) == -1
    assert lib.jq_rotate_weights_host(W.ctypes.data, 2, 64, 128, 1) == -2
