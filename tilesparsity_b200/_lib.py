"""ctypes binding of libtilesparse.so (the C ABI declared in include/tilesparse.h).

The library is the product: there is no Python or CPU fallback.  If the shared object is missing
the import of this module raises, and every compute call raises `TileSparseError` when the C ABI
reports a failure.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtilesparse.so")

TS_OK = 0
TS_ERR_INVALID, TS_ERR_CUDA, TS_ERR_TIMEOUT, TS_ERR_UNSUPPORTED, TS_ERR_NOMEM = 1, 2, 3, 4, 5
TS_DTYPE_F16, TS_DTYPE_BF16, TS_DTYPE_F32 = 0, 1, 2
TS_INDEX_ABSOLUTE, TS_INDEX_RELATIVE = 0, 1
MASK_MODES = {"tw1": 0, "tw2": 1, "tw1m": 2, "tw2m": 3, "bert_type2": 4, "bert_type7": 5, "bert_type8": 6,
              "topk_l1": 7, "tw_cols_rows": 8}


PATTERN_MODES = {"ew": 0, "vw": 1, "bw": 2}


class TileSparseError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libtilesparse error {code}: {message}")
        self.code = code


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python tilesparsity_b200/build.py` "
            "(there is no fallback implementation)")
    return C.CDLL(LIB_PATH)


lib = _load()

class Epilogue(C.Structure):
    """ts_epilogue_t"""
    _fields_ = [("alpha", C.c_float), ("beta", C.c_float), ("bias_dev", C.c_void_p), ("activation", C.c_int),
                ("n_peers", C.c_int), ("peer_ct", C.c_void_p * 7), ("multicast_ct", C.c_void_p)]


ACTIVATIONS = {None: 0, "none": 0, "relu": 1, "gelu": 2}

_i32p = C.POINTER(C.c_int32)
_i64p = C.POINTER(C.c_int64)
_vp = C.c_void_p

# name -> (restype, argtypes); every symbol include/tilesparse.h declares.
SIGNATURES = {
    "ts_version": (C.c_int, []),
    "ts_last_error": (C.c_int, [C.c_char_p, C.c_int]),
    "ts_layer_create": (C.c_int, [C.POINTER(_vp), C.c_int, C.c_int, C.c_int, C.c_int]),
    "ts_layer_destroy": (C.c_int, [_vp]),
    "ts_layer_set_tiles": (C.c_int, [_vp, C.c_int, _i32p, _i32p, _i32p, _i32p, C.c_int]),
    "ts_layer_pack_weights": (C.c_int, [_vp, _vp, C.c_int64, C.c_int, _vp]),
    "ts_layer_get_packed": (C.c_int, [_vp, _vp, _i64p, _i64p]),
    "ts_layer_stats": (C.c_int, [_vp, _i64p, _i64p, _i64p, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "ts_masked_gemm": (C.c_int, [_vp, C.c_int, _vp, C.c_int64, _vp, C.c_int64, C.c_float, C.c_float, _vp]),
    "ts_masked_gemm_ex": (C.c_int, [_vp, C.c_int, _vp, C.c_int64, _vp, C.c_int64, C.POINTER(Epilogue), _vp]),
    "ts_masked_gemm_simt": (C.c_int, [_vp, C.c_int, _vp, C.c_int64, _vp, C.c_int64, C.c_float, C.c_float, _vp]),
    "ts_masked_gemm_host": (C.c_int, [_vp, C.c_int, _vp, _vp, C.c_float, C.c_float, _vp]),
    "ts_masked_gemm_host_async": (C.c_int, [_vp, C.c_int, _vp, _vp, C.c_float, C.c_float, _vp]),
    "ts_masked_gemm_host_wait": (C.c_int, [_vp, _vp]),
    "ts_layer_check": (C.c_int, [_vp, _vp]),
    "ts_layer_schedule_stats": (C.c_int, [_vp, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "ts_conv_geometry": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                   _i64p, _i64p]),
    "ts_layer_set_conv": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int]),
    "ts_conv_pack_input": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, C.c_int64, _vp]),
    "ts_conv_repack": (C.c_int, [_vp, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, C.c_int64, _vp]),
    "ts_masked_conv": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, _vp, C.c_int64, _vp, C.c_int64, C.POINTER(Epilogue), _vp]),
    "ts_conv_unpack_output": (C.c_int, [_vp, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp]),
    "ts_layer_set_unit_rows": (C.c_int, [_vp, C.c_int]),
    "ts_layer_set_split_k": (C.c_int, [_vp, C.c_int]),
    "ts_plan_split": (C.c_int, [C.c_int, _i32p, _i32p, C.c_int64, C.c_int, C.c_int, _i32p]),
    "ts_plan_schedule": (C.c_int, [C.c_int, _i32p, _i32p, C.c_int64, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int),
                                   C.POINTER(C.c_int), C.POINTER(C.c_int), _i32p, C.c_int, C.POINTER(C.c_float)]),
    "ts_stream_gemm_nn": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_float, _vp, _vp, C.c_float, _vp, C.c_int,
                                    C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(_vp), C.POINTER(_vp),
                                    C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int, _vp]),
    "ts_build_tw_mask": (C.c_int, [C.c_int, C.c_int, C.POINTER(_vp), C.POINTER(C.c_int), C.POINTER(C.c_int), _i64p,
                                   C.c_int, C.c_double, C.c_int, C.c_double, C.POINTER(_vp), _i64p, C.POINTER(_vp),
                                   C.POINTER(_vp), _vp]),
    "ts_build_tw_mask_f64": (C.c_int, [C.c_int, C.c_int, C.POINTER(_vp), C.POINTER(C.c_int), C.POINTER(C.c_int), _i64p,
                                       C.c_int, C.c_double, C.POINTER(_vp), _i64p, C.POINTER(_vp), _vp]),
    "ts_taylor_accumulate": (C.c_int, [_vp, _vp, _vp, C.c_int64, _vp]),
    "ts_mask_result_layer": (C.c_int, [_vp, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "ts_mask_result_copy": (C.c_int, [_vp, C.c_int, _i32p, _i32p, _i32p, _i32p, _i32p]),
    "ts_mask_result_thresholds": (C.c_int, [_vp, C.POINTER(C.c_double)]),
    "ts_mask_result_destroy": (C.c_int, [_vp]),
    "ts_order_statistics": (C.c_int, [_vp, C.c_int64, C.c_int64, C.c_int64, C.POINTER(C.c_float), _vp]),
    "ts_build_pattern_mask": (C.c_int, [C.c_int, C.c_int, C.POINTER(_vp), C.POINTER(C.c_int), C.POINTER(C.c_int), _i64p,
                                        C.c_double, C.POINTER(_vp), _i64p, C.POINTER(C.c_double), _vp]),
    "ts_percentile_f32": (C.c_int, [_vp, C.c_int64, C.c_double, C.c_int, C.POINTER(C.c_double), _vp]),
    "ts_tw1_row_keep_noalloc": (C.c_int, [_vp, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_double, C.c_int, _vp,
                                          C.POINTER(C.c_double), _vp]),
    "ts_residual_gemm": (C.c_int, [C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp, _vp, C.c_int64, _vp, C.c_int64,
                                   C.c_float, _vp]),
    "ts_transpose16": (C.c_int, [_vp, C.c_int64, _vp, C.c_int64, C.c_int, C.c_int, _vp]),
    "ts_shard_plan": (C.c_int, [C.c_int, _i64p, C.c_int, _i32p]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    buf = C.create_string_buffer(1024)
    lib.ts_last_error(buf, 1024)
    return buf.value.decode("utf-8", "replace")


def check(code: int) -> None:
    if code != TS_OK:
        raise TileSparseError(code, last_error())
