"""ctypes binding of libbitnet_b200.so (the C ABI in include/bitnet_b200.h).

There is no CPU or PyTorch fallback: if the shared library is missing, importing this
module raises, and every wrapper raises on a non-zero status from the library.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libbitnet_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m bitnet_b200.build` "
        "(needs nvcc; there is no fallback implementation)"
    )

lib = ctypes.CDLL(LIB_PATH)

_vp, _i, _i64, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

# every symbol the headers under include/ declare: name -> (restype, argtypes)
SIGNATURES = {
    "bitnet_last_status": (_i, []),
    "bitnet_status_string": (ctypes.c_char_p, [_i]),
    "bitnet_last_cuda_error": (ctypes.c_char_p, []),
    "bitnet_init": (_i, []),
    "bitnet_attention_decode": (_i, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "bitnet_sample_top_p": (_i, [_vp, _i64, _i, _i, _f, _f, ctypes.c_uint64, _vp, _vp, _vp, _vp, _vp]),
    "bitlinear_int8xint2": (None, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "bitlinear_int8xint2_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "bitlinear_int8xint2_noalloc_error": (_i, [_i]),
    "bitnet_linear_w2a8": (_i, [_vp, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _vp, ctypes.POINTER(_i), _i, _i, _i, _i, _vp]),
    "bitnet_linear_w2a8_add_quant": (_i, [_vp, _i64, _vp, _vp, _vp, _f, _i, _i, _i, _vp, _i64, _vp, _f, _vp, _i64, _vp, _vp, _vp]),
    "bitnet_quant_input": (_i, [_vp, _i64, _vp, _f, _vp, _i64, _vp, _vp, _vp, _i, _i, _vp]),
    "bitnet_quant_input_glu": (_i, [_vp, _i64, _vp, _f, _vp, _i64, _vp, _vp, _vp, _i, _i, _vp]),
    "bitnet_decoder_create": (_vp, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "bitnet_decoder_step": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "bitnet_decoder_step_sync": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "bitnet_decoder_bench_linears": (_i, [_vp, _vp, _vp]),
    "bitnet_decoder_read_trace": (_i, [_vp, _vp, _i]),
    "bitnet_decoder_set_attention_tap": (_i, [_vp, _vp]),
    "bitnet_decoder_error_flag": (_i, [_vp]),
    "bitnet_decoder_clear_error": (_i, [_vp]),
    "bitnet_decoder_kernels_per_step": (_i, [_vp]),
    "bitnet_workspace_error": (_i, [_i]),
    "bitnet_tp_area_bytes": (ctypes.c_size_t, [_vp, _i]),
    "bitnet_tp_area_create": (_i, [ctypes.c_size_t, _vp, _vp]),
    "bitnet_tp_area_open": (_i, [_vp, _vp]),
    "bitnet_tp_area_close": (_i, [_vp]),
    "bitnet_tp_area_free": (_i, [_vp]),
    "bitnet_decoder_set_wait_limit": (_i, [_vp, ctypes.c_double]),
    "bitnet_decoder_create_tp": (_vp, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "bitnet_decoder_destroy": (None, [_vp]),
    "bitnet_w2t_bytes": (ctypes.c_size_t, [_i, _i]),
    "bitnet_pack_ternary": (_i, [_vp, _vp, _i, _i, _vp]),
    "bitnet_pack_from_i2s": (_i, [_vp, _vp, _i, _i, _vp]),
    "bitnet_pack_from_ref_int2": (_i, [_vp, _vp, _i, _i, _vp]),
    "bitnet_unpack_ternary": (_i, [_vp, _vp, _i, _i, _vp]),
    "quantize_i2_s": (ctypes.c_size_t, [_vp, _vp, _i64, _i64, _vp]),
    "ggml_bitnet_init": (None, []),
    "ggml_bitnet_free": (None, []),
    "ggml_bitnet_can_mul_mat": (ctypes.c_bool, [_vp, _vp, _vp]),
    "ggml_bitnet_mul_mat_get_wsize": (ctypes.c_size_t, [_vp, _vp, _vp]),
    "ggml_bitnet_mul_mat_task_init": (None, [_vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "ggml_bitnet_mul_mat_task_compute": (None, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "ggml_bitnet_transform_tensor": (None, [_vp]),
    "ggml_bitnet_mul_mat": (None, [_vp, _vp]),
    "ggml_bitnet_get_type_bits": (_i, [_i]),
    "ggml_bitnet_set_n_threads": (None, [_i]),
    "ggml_preprocessor": (None, [_i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "ggml_qgemm_lut": (None, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ggml_vec_dot_i2_i8_s": (None, [_i, _vp, ctypes.c_size_t, _vp, ctypes.c_size_t, _vp, ctypes.c_size_t, _i]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here = the library lacks a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


class BitnetError(RuntimeError):
    pass


def check(status: int | None = None) -> None:
    """Raises BitnetError unless the library's last status (or `status`) is 0."""
    st = lib.bitnet_last_status() if status is None else status
    if st != 0:
        msg = lib.bitnet_status_string(st).decode()
        if st == 3:
            msg += ": " + lib.bitnet_last_cuda_error().decode()
        raise BitnetError(f"libbitnet_b200: {msg} (status {st})")


def ptr(t) -> ctypes.c_void_p:
    """Device (or host) address of a torch tensor, NULL for None."""
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> ctypes.c_void_p:
    import torch

    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
