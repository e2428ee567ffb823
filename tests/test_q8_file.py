"""Q8_0 weights on disk (csrc/q8_file.cpp).

CPU: the container is the reference's GGUF dialect -- a file of fp32 tensors written here is read back by the
reference's own load_gguf (compiled into oracle/_ref where the reference tree is present), layout hash included; the
Q8_0 blocks in a file equal quantize_q8_0_host of the checker bit for bit; malformed input is refused.
GPU: a Q8_0 tensor loaded from a file arrives in device memory as exactly the planar Q8_0R bytes the checker's
quantize + repack give (both the device-repack and the host-repack route), and the Q8 product on it matches."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

import cases
from checkers import have_ref, load_ref


def _write(lib, path, tensors):
    """tensors: [(name, array[rows, cols] fp32, as_q8)]"""
    n = len(tensors)
    names = (C.c_char_p * n)(*[t[0].encode() for t in tensors])
    arrs = [np.ascontiguousarray(t[1], np.float32) for t in tensors]
    ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in arrs])
    rows = (C.c_int64 * n)(*[a.shape[0] for a in arrs])
    cols = (C.c_int64 * n)(*[a.shape[1] for a in arrs])
    q8 = (C.c_int * n)(*[int(t[2]) for t in tensors])
    return lib.ppml_b200_q8_file_write(path.encode(), n, names, ptrs, rows, cols, q8)


def _tensors():
    r = np.random.default_rng(6)
    return [("msa.row.q.weight", (r.standard_normal((256, 256)) * 0.02).astype(np.float32), True),
            ("msa.row.q.bias", r.standard_normal((1, 256)).astype(np.float32), False),
            ("pair.tri.out.weight", (r.standard_normal((128, 128)) * 0.02).astype(np.float32), False),
            ("msa2pair.left.weight", (r.standard_normal((16, 256)) * 0.02).astype(np.float32), True)]


def test_file_round_trip_on_the_host(lib, oracle, tmp_path):
    path = str(tmp_path / "weights.gguf")
    ts = _tensors()
    assert _write(lib, path, ts) == 0
    raw = open(path, "rb").read()
    assert struct.unpack("<II", raw[:8]) == (0x46554747, 3)
    h = lib.ppml_b200_q8_file_open(path.encode())
    assert h
    try:
        assert lib.ppml_b200_q8_file_count(h) == len(ts)
        hexbuf = C.create_string_buffer(17)
        assert lib.ppml_b200_q8_file_layout_hash(h, hexbuf) == 0 and len(hexbuf.value) == 16
        for i, (name, arr, q8) in enumerate(ts):
            assert lib.ppml_b200_q8_file_find(h, name.encode()) == i
            nm = C.create_string_buffer(64)
            rows, cols, isq = C.c_int64(), C.c_int64(), C.c_int()
            assert lib.ppml_b200_q8_file_info(h, i, nm, 64, C.byref(rows), C.byref(cols), C.byref(isq)) == 0
            assert (nm.value.decode(), rows.value, cols.value, isq.value) == (name, arr.shape[0], arr.shape[1], int(q8))
            nbytes = lib.ppml_b200_q8_file_nbytes(h, i)
            assert nbytes == (arr.size // 32 * 34 if q8 else arr.size * 4)
        assert lib.ppml_b200_q8_file_find(h, b"nope") == -1
    finally:
        lib.ppml_b200_q8_file_close(h)
    # the Q8_0 blocks in the file are the checker's, bit for bit (offsets are absolute and 32-byte aligned)
    blocks = oracle.quantize_q8_0(ts[0][1]).tobytes()
    assert raw.count(blocks) == 1 and raw.index(blocks) % 32 == 0
    # refusals
    assert _write(lib, path, [("w", np.zeros((4, 48), np.float32), True)]) == 2        # blocks would straddle rows
    assert lib.ppml_b200_q8_file_open(str(tmp_path / "missing.gguf").encode()) is None
    bad = str(tmp_path / "bad.gguf")
    open(bad, "wb").write(b"GGUF" + raw[4:40])                                            # cut short
    assert lib.ppml_b200_q8_file_open(bad.encode()) is None


@pytest.mark.skipif(not have_ref(), reason="oracle/_ref not built (needs the reference tree)")
def test_reference_reader_accepts_the_container(lib, tmp_path):
    """A file of fp32 tensors written here goes through the reference's load_gguf: header, metadata, tensor infos,
    alignment, absolute offsets and the layout hash are what that reader expects."""
    ref = load_ref()
    path = str(tmp_path / "f32.gguf")
    ts = [(n, a, False) for (n, a, _) in _tensors()]
    assert _write(lib, path, ts) == 0
    n = len(ts)
    names = (C.c_char_p * n)(*[t[0].encode() for t in ts])
    rows = (C.c_int64 * n)(*[t[1].shape[0] for t in ts])
    cols = (C.c_int64 * n)(*[t[1].shape[1] for t in ts])
    outs = [np.empty_like(t[1]) for t in ts]
    optrs = (C.c_void_p * n)(*[o.ctypes.data for o in outs])
    ref.ref_gguf_load.argtypes = [C.c_char_p, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_void_p)]
    assert ref.ref_gguf_load(path.encode(), n, names, rows, cols, optrs) == 0
    for (_, a, _), o in zip(ts, outs):
        assert np.array_equal(a, o)
    # a renamed tensor no longer matches the stored layout hash: the reference's reader refuses
    wrong = (C.c_char_p * n)(*([b"other.name"] + [t[0].encode() for t in ts[1:]]))
    assert ref.ref_gguf_load(path.encode(), n, wrong, rows, cols, optrs) == 1


@pytest.mark.gpu
@pytest.mark.parametrize("device_repack", [True, False])
def test_load_into_device_memory_as_q8_0r(lib, oracle, tmp_path, device_repack):
    torch = pytest.importorskip("torch")
    from proteinpredictmachinelearning_b200 import PATH_UMMA, ops
    path = str(tmp_path / "weights.gguf")
    ts = _tensors()
    assert _write(lib, path, ts) == 0
    h = lib.ppml_b200_q8_file_open(path.encode())
    assert h
    try:
        for i, (name, arr, q8) in enumerate(ts):
            nbytes = lib.ppml_b200_q8_file_nbytes(h, i)
            dst = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
            scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda") if device_repack else None
            rc = lib.ppml_b200_q8_file_load(h, i, C.c_void_p(dst.data_ptr()), None if scratch is None else C.c_void_p(scratch.data_ptr()), None)
            assert rc == 0
            got = dst.cpu().numpy()
            if q8:
                assert np.array_equal(got, oracle.repack_q8_0(oracle.quantize_q8_0(arr)))
            else:
                assert np.array_equal(got.view(np.float32).reshape(arr.shape), arr)
            if name == "msa.row.q.weight":
                _, x = cases.q8_case(256, 408, 256, seed=2)
                c, taken = ops.mul_mat_q8_cuda(dst, torch.from_numpy(x).cuda(), 256, path=PATH_UMMA)
                assert taken == 1 and cases.rel_err(c.cpu().numpy(), oracle.mul_mat_q8(got, x, 256)) <= 1e-5
    finally:
        lib.ppml_b200_q8_file_close(h)
    # the device repack alone, against the host one
    blocks = oracle.quantize_q8_0(ts[0][1])
    out = torch.zeros(blocks.size, dtype=torch.uint8, device="cuda")
    src = torch.from_numpy(blocks).cuda()
    assert lib.ppml_b200_repack_q8_0(C.c_void_p(src.data_ptr()), blocks.size // 34, C.c_void_p(out.data_ptr()), None) == 0
    assert np.array_equal(out.cpu().numpy(), oracle.repack_q8_0(blocks))
