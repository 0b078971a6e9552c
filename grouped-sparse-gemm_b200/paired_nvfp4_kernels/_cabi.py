"""ctypes binding of libpaired_nvfp4_b200.so (the C ABI declared in include/paired_nvfp4_b200.h).

There is no fallback: if the shared library is missing or does not load, importing this module
raises ImportError telling the user to build it.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpaired_nvfp4_b200.so")

ABI_VERSION = 2

_p = ctypes.c_void_p
_i = ctypes.c_int
_i64 = ctypes.c_int64
_f = ctypes.c_float

# name -> (restype, argtypes); mirrors include/paired_nvfp4_b200.h one to one
SIGNATURES = {
    "pnv_abi_version": (_i, []),
    "pnv_last_error": (ctypes.c_char_p, []),
    "pnv_group_mm_device_status": (_i, [ctypes.POINTER(_i)]),
    "pnv_selftest_bounded_wait": (_i, [ctypes.POINTER(_i)]),
    "pnv_physical_dims": (_i, [_i, _i] + [ctypes.POINTER(_i)] * 4),
    "pnv_sf_numel": (_i64, [_i, _i, _i]),
    "pnv_compress": (_i, [_p, _p, _i, _i, _i, _p, _p, _p, _p]),
    "pnv_quant_act": (_i, [_p, _p, _i, _p, _i, _i, _i, _p, _p, _i, _p]),
    "pnv_silu_mul_quant_act": (_i, [_p, _p, _i, _p, _i, _i, _i, _i, _i, _f, _f, _p, _p, _i, _p]),
    "pnv_scatter_quant_act": (_i, [_p, _p, _p, _p, _p, _i, _i64, _i, _i, _i, _p, _p, _i, _p]),
    "pnv_dispatch_plan_scratch_ints": (_i64, [_i64, _i]),
    "pnv_dispatch_plan": (_i, [_p, _i, _i64, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p]),
    "pnv_dispatch_plan_strided": (_i, [_p, _i, _i64, _i64, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p]),
    "pnv_wire_row_bytes": (_i64, [_i]),
    "pnv_pack_wire_rows": (_i, [_p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _p, _p]),
    "pnv_pack_wire_rows_parts": (_i, [_p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _p, _p]),
    "pnv_scatter_fp4_wire": (_i, [_p, _p, _p, _i, _i, _i, _p, _p, _i, _p]),
    "pnv_dispatch_plan_noalloc_max_scratch_ints": (_i64, []),
    "pnv_dispatch_plan_noalloc": (_i, [_p, _i, _i64, _i, _i, _i, _i, _p, _p, _p, _p, _p]),
    "pnv_scatter_quant_act_planned": (_i, [_p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _p, _p, _i, _p]),
    "pnv_quant_rows": (_i, [_p, _p, _i64, _i, _p, _p, _i, _p]),
    "pnv_scatter_fp4_planned": (_i, [_p, _p, _p, _p, _i, _i, _i, _p, _p, _i, _p]),
    "pnv_moe_finalize": (_i, [_p, _p, _p, _p, _i64, _i, _i, _p]),
    "pnv_gather_rows": (_i, [_p, _p, _i64, _i64, _p, _p]),
    "pnv_set_silu_table": (_i, [_i]),
    "pnv_gated_act": (_i, [_p, _i64, _i, _i, _i, _f, _f, _p, _p]),
    "pnv_group_mm_num_configs": (_i, []),
    "pnv_group_mm_config_name": (ctypes.c_char_p, [_i]),
    "pnv_group_mm_workspace_bytes": (_i64, [_i, _i, _i, _i]),
    "pnv_group_mm": (_i, [_p] * 8 + [_i] * 9 + [_p, _i64, _p]),
    "pnv_group_mm_rows": (_i, [_p] * 9 + [_i] * 9 + [_p, _i64, _p]),
    "pnv_peer_buffer_alloc": (_i, [_i64, _p, _p]),
    "pnv_peer_buffer_open": (_i, [_p, _p]),
    "pnv_peer_buffer_close": (_i, [_p]),
    "pnv_peer_buffer_free": (_i, [_p]),
    "pnv_zero_rows": (_i, [_p, _p, _i64, _i64, _p]),
    "pnv_zero_rows_parts": (_i, [_p, _i, _i64, _p, _i64, _p]),
    "pnv_group_mm_rows_parts": (_i, [_p, _i, _i64] + [_p] * 8 + [_i] * 9 + [_p, _i64, _p]),
    "pnv_group_mm_swiglu_num_configs": (_i, []),
    "pnv_group_mm_swiglu_config_name": (ctypes.c_char_p, [_i]),
    "pnv_group_mm_swiglu_quant": (_i, [_p] * 10 + [_i] * 9 + [_f, _f, _i, _i, _p, _i64, _p]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python grouped-sparse-gemm_b200/build.py` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these ops.")
    try:
        lib = ctypes.CDLL(LIB_PATH)
    except OSError as exc:  # pragma: no cover
        raise ImportError(f"could not load {LIB_PATH}: {exc}") from exc
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means a stale build
        fn.restype = res
        fn.argtypes = args
    if lib.pnv_abi_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI version {lib.pnv_abi_version()}, expected {ABI_VERSION}")
    return lib


lib = _load()


def check(rc):
    """Turn a non-zero status into the RuntimeError the reference's TORCH_CHECK would raise."""
    if rc != 0:
        raise RuntimeError(lib.pnv_last_error().decode("utf-8", "replace"))


def physical_dims(features, k):
    out = [_i() for _ in range(4)]
    check(lib.pnv_physical_dims(features, k, *[ctypes.byref(o) for o in out]))
    return tuple(o.value for o in out)


def sf_numel(rows, k, groups):
    return int(lib.pnv_sf_numel(rows, k, groups))


def group_mm_swiglu_config_names():
    return [lib.pnv_group_mm_swiglu_config_name(i).decode() for i in range(lib.pnv_group_mm_swiglu_num_configs())]


def group_mm_config_names():
    return [lib.pnv_group_mm_config_name(i).decode() for i in range(lib.pnv_group_mm_num_configs())]
