"""Host-side checks that need no GPU: the shared library loads, exports every symbol the header
declares and every C++ launcher name the reference's dispatcher binds, rejects bad arguments before
touching the device, and its host weight quantizers are bit-identical to the checker."""
import ctypes as C
import os
import re
import subprocess

import numpy as np

import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "ppml_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ppml_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    from proteinpredictmachinelearning_b200 import _lib
    declared = _header_symbols()
    assert len(declared) >= 24
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ppml_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes prototype"
    assert sorted(_lib.SIGNATURES) == declared


def test_library_exports_reference_launcher_names(lib):
    from proteinpredictmachinelearning_b200 import LIB_PATH
    want = open(os.path.join(ROOT, "tests", "golden", "reference_launcher_symbols.txt")).read().split()
    have = set(subprocess.check_output(["nm", "-D", "--defined-only", LIB_PATH], text=True).split())
    missing = [w for w in want if w not in have]
    assert not missing, missing


def test_bad_arguments_are_rejected_on_the_host(lib):
    assert lib.ppml_b200_mul_mat_f32(None, None, None, 4, 4, 4, None, 0, 0, None) == 1
    assert lib.ppml_b200_mul_mat_f32(C.c_void_p(16), C.c_void_p(16), C.c_void_p(16), 0, 4, 4, None, 0, 0, None) == 1
    assert lib.ppml_b200_mul_mat_f32(C.c_void_p(16), C.c_void_p(16), C.c_void_p(16), 4, 4, 4, None, 9, 0, None) == 1
    taken = C.c_int(5)
    p = C.c_void_p(16)
    assert lib.ppml_b200_mul_mat_q8(p, p, p, 8, 8, 48, 2, 1, None, None, 0, C.byref(taken), None) == 2   # K % 32
    assert taken.value == 0
    assert lib.ppml_b200_mul_mat_q8(p, p, p, 8, 8, 64, 7, 1, None, None, 0, None, None) == 5             # weight type
    assert lib.ppml_b200_mul_mat_q8(None, p, p, 8, 8, 64, 2, 1, None, None, 0, None, None) == 1
    assert lib.ppml_b200_flash_attn_forward(None, p, p, p, None, p, None, 0, None) == 1
    assert lib.ppml_b200_tri_mul(p, p, p, 0, 1, 1, 1, 1, 1.0, 1, 0, None) == 1
    assert lib.ppml_b200_out_prod(p, p, p, 4, 3, 1, 1, 5, 2, 1, 1, 4, 5, 1, 1, 0, None) == 1             # K mismatch
    assert lib.ppml_b200_quantize_rows_q8_1(p, p, 33, None) == 1
    assert lib.ppml_b200_q8_0r_bytes(64) == 68
    # entries without a counterpart in the reference follow the same conventions
    assert lib.ppml_b200_flash_attn_forward_16(None, 8, 0, p, p, p, None, p, None, 1, 0, None) == 1
    assert lib.ppml_b200_outer_prod_mean_slabs(p, p, p, 0, 4, 4, 4, 1, 1.0, 0, None) == 1
    assert lib.ppml_b200_outer_prod_mean_slabs(p, None, p, 2, 4, 4, 4, 1, 1.0, 0, None) == 1
    assert lib.ppml_b200_tri_mul_16(p, p, None, 1, 1, 1, 1, 1, 1.0, 1, 1, 0, None) == 1
    # the form of the tensor-core Q8 product: forced one-pass, forced two-pass, per shape (long K, few token tiles)
    try:
        lib.ppml_b200_set_q8_two_pass(0)
        assert lib.ppml_b200_q8_kernel_launches(256, 408, 1024) == 1
        lib.ppml_b200_set_q8_two_pass(1)
        assert lib.ppml_b200_q8_kernel_launches(256, 65536, 128) == 2
    finally:
        lib.ppml_b200_set_q8_two_pass(-1)


def test_host_weight_quantizer_bit_exact(oracle, lib):
    from proteinpredictmachinelearning_b200 import ops
    w, _ = cases.q8_case(64, 1, 256, seed=2)
    w[3, :32] = 0.0
    q = ops.quantize_q8_0_host(w)
    assert np.array_equal(q, oracle.quantize_q8_0(w))
    assert np.array_equal(ops.repack_q8_0_host(q), oracle.repack_q8_0(q))


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from proteinpredictmachinelearning_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        _lib.load()
    except ImportError as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("load() must raise when the library is missing")
