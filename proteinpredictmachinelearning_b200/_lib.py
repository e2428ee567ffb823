"""ctypes binding of libppml_b200.so (built in-tree by build.py).  There is no fallback: if the
library is missing or does not load, importing this module raises."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libppml_b200.so")

PATH_AUTO, PATH_SIMT, PATH_UMMA = 0, 1, 2
TF32_ROUND, TF32_TMA, TF32_TRUNCATE = 0, 1, 2
NOALLOC_SCRATCH_BYTES = 4 << 20      # PPML_B200_NOALLOC_SCRATCH_BYTES


class FlashCfg(C.Structure):
    _fields_ = [("B", C.c_int), ("h", C.c_int), ("L", C.c_int), ("d", C.c_int), ("causal", C.c_int),
                ("scale", C.c_float), ("softmax_eps", C.c_float), ("Br", C.c_int), ("Bc", C.c_int)]


_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float

# name -> (restype, argtypes): every symbol include/ppml_b200.h declares
SIGNATURES = {
    "ppml_b200_version": (C.c_char_p, []),
    "ppml_b200_hw_supported": (_i, [C.POINTER(_i), C.POINTER(_i)]),
    "ppml_b200_device_status": (_i, [C.POINTER(_i)]),
    "ppml_b200_mul_mat_f32": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _i, _i, _vp]),
    "ppml_b200_mul_mat_f32_fused": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "ppml_b200_row_stats": (_i, [_vp, _vp, _i64, _i, _f, _vp]),
    "ppml_b200_layernorm_fold": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "ppml_b200_mul_mat_f16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp]),
    "ppml_b200_mul_mat_bf16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp]),
    "ppml_b200_mul_mat_f32_as_bf16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp]),
    "ppml_b200_bf16_shadow_invalidate": (None, [_vp]),
    "ppml_b200_cast_f32_to_f16": (_i, [_vp, _vp, _i64, _vp]),
    "ppml_b200_cast_f32_to_bf16": (_i, [_vp, _vp, _i64, _vp]),
    "ppml_b200_mul_mat_q8": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _i, C.POINTER(_i), _vp]),
    "ppml_b200_mul_mat_q8_noalloc": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "ppml_b200_quantize_rows_q8_1": (_i, [_vp, _vp, _i64, _vp]),
    "ppml_b200_dequantize_q8_0": (_i, [_vp, _vp, _i64, _vp]),
    "ppml_b200_dequantize_q8_1": (_i, [_vp, _vp, _i64, _vp]),
    "ppml_b200_quantize_q8_0_host": (_i, [_vp, _vp, _i64]),
    "ppml_b200_repack_q8_0_host": (_i, [_vp, _i64, _vp]),
    "ppml_b200_quantize_q8_0r": (_i, [_vp, _vp, _i64, _vp]),
    "ppml_b200_q8_0r_bytes": (_i64, [_i64]),
    "ppml_b200_repack_q8_0": (_i, [_vp, _i64, _vp, _vp]),
    "ppml_b200_q8_file_write": (_i, [C.c_char_p, _i, C.POINTER(C.c_char_p), C.POINTER(_vp), C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i)]),
    "ppml_b200_q8_file_open": (_vp, [C.c_char_p]),
    "ppml_b200_q8_file_close": (None, [_vp]),
    "ppml_b200_q8_file_count": (_i, [_vp]),
    "ppml_b200_q8_file_find": (_i, [_vp, C.c_char_p]),
    "ppml_b200_q8_file_info": (_i, [_vp, _i, C.c_char_p, _i, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i)]),
    "ppml_b200_q8_file_nbytes": (_i64, [_vp, _i]),
    "ppml_b200_q8_file_layout_hash": (_i, [_vp, C.c_char_p]),
    "ppml_b200_q8_file_load": (_i, [_vp, _i, _vp, _vp, _vp]),
    "ppml_b200_flash_attn_forward": (_i, [C.POINTER(FlashCfg), _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "ppml_b200_flash_attn_backward": (_i, [C.POINTER(FlashCfg), _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ppml_b200_flash_attn_forward_ex": (_i, [C.POINTER(FlashCfg), _i, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "ppml_b200_flash_attn_forward_16": (_i, [C.POINTER(FlashCfg), _i, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "ppml_b200_flash_attn_forward_tokens": (_i, [C.POINTER(FlashCfg), _i, _i64, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _i64, _i, _vp, _i64, _vp, _i, _vp]),
    "ppml_b200_out_prod": (_i, [_vp, _vp, _vp] + [_i64] * 12 + [_i, _vp]),
    "ppml_b200_tri_mul": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _f, _i, _i, _vp]),
    "ppml_b200_outer_prod_mean": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _f, _i, _vp]),
    "ppml_b200_tri_mul_16": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _f, _i, _i, _i, _vp]),
    "ppml_b200_outer_prod_mean_16": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _f, _i, _i, _vp]),
    "ppml_b200_set_q8_two_pass": (None, [_i]),
    "ppml_b200_q8_kernel_launches": (_i, [_i, _i, _i]),
    "ppml_b200_outer_prod_mean_slabs": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _f, _i, _vp]),
    "ppml_b200_peer_flag_bytes": (_i, []),
    "ppml_b200_peer_alloc": (_vp, [_i64]),
    "ppml_b200_peer_free": (None, [_vp]),
    "ppml_b200_peer_export": (_i, [_vp, _vp]),
    "ppml_b200_peer_open": (_vp, [_vp]),
    "ppml_b200_peer_close": (None, [_vp]),
    "ppml_b200_peer_all_gather": (_i, [_vp, C.POINTER(_vp), _i64, _i, _i, C.POINTER(_vp), _i, _vp]),
    "ppml_b200_peer_transpose": (_i, [_vp, C.POINTER(_vp), _i, _i, _i, _i, _i, C.POINTER(_vp), _i, _vp]),
    "ppml_b200_mulmat_stats_begin": (None, [_i, _i, _i]),
    "ppml_b200_mulmat_stats_end": (None, [C.c_char_p]),
    "ppml_b200_mulmat_stats_dump": (_i, [C.c_char_p, _i]),
}

_lib = None


def load():
    """Loads the shared library once and attaches the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m proteinpredictmachinelearning_b200.build` "
            "(there is no CPU or PyTorch fallback for this path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
