"""ctypes binding of libminiattn.so (the C ABI in include/miniattn.h).

There is no CPU fallback and no other backend: if the library is missing or fails to
load, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libminiattn.so"

OK, EINVAL, EUNSUPPORTED, ECUDA, EDEVICE_WAIT = 0, -1, -2, -3, -4
FP16, BF16 = 0, 1
KERNEL_AUTO, KERNEL_SIMPLE, KERNEL_WS = 0, 1, 2
KERNELS = {"auto": KERNEL_AUTO, "simple": KERNEL_SIMPLE, "ws": KERNEL_WS}


class FwdParams(C.Structure):
    """Mirror of ``MiniAttnFwdParams``."""

    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
        ("lse", C.c_void_p), ("status", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3),
        ("v_stride", C.c_int64 * 3), ("o_stride", C.c_int64 * 3),
        ("q_pos0", C.c_int64), ("k_pos0", C.c_int64),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32),
        ("Nq", C.c_int32), ("Nk", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32),
        ("softmax_scale", C.c_float), ("kernel", C.c_int32),
        ("carry", C.c_void_p), ("carry_in", C.c_int32), ("carry_out", C.c_int32),
        ("carry_tile0", C.c_int32), ("carry_tiles", C.c_int32),
    ]


class Int8Params(C.Structure):
    """Mirror of ``MiniAttnInt8Params``."""

    _fields_ = [
        ("fwd", FwdParams), ("q8", C.c_void_p), ("k8", C.c_void_p), ("q_scale", C.c_void_p),
        ("k_scale", C.c_void_p), ("k_partial", C.c_void_p), ("k_mean", C.c_void_p),
    ]


class MergeParams(C.Structure):
    """Mirror of ``MiniAttnMergeParams``."""

    _fields_ = [
        ("acc_o", C.c_void_p), ("acc_lse", C.c_void_p), ("part_o", C.c_void_p),
        ("part_lse", C.c_void_p), ("out", C.c_void_p),
        ("rows", C.c_int64), ("D", C.c_int32), ("dtype", C.c_int32), ("init", C.c_int32),
        ("out_rows_per_slab", C.c_int64), ("out_slab_stride", C.c_int64),
    ]


class PlanInfo(C.Structure):
    """Mirror of ``MiniAttnPlanInfo``."""

    _fields_ = [
        ("split", C.c_int32), ("sm_count", C.c_int32), ("n_ctas", C.c_int64),
        ("n_whole", C.c_int32), ("n_pieces", C.c_int32), ("n_cut_items", C.c_int32), ("n_slots", C.c_int32),
        ("scratch_bytes", C.c_int64), ("est_plain", C.c_float), ("est_balanced", C.c_float),
        ("head_group", C.c_int32),
    ]


class PlanPiece(C.Structure):
    """Mirror of ``MiniAttnPlanPiece``."""

    _fields_ = [
        ("item", C.c_int32), ("t0", C.c_int32), ("t1", C.c_int32),
        ("part", C.c_int32), ("nparts", C.c_int32), ("slot", C.c_int32),
    ]


def _load() -> C.CDLL:
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python mini-attention_b200/build.py` "
            "(needs nvcc; there is no fallback path)"
        )
    lib = C.CDLL(str(_LIB_PATH))
    lib.miniattn_fwd.argtypes = [C.POINTER(FwdParams), C.c_void_p]
    lib.miniattn_fwd.restype = C.c_int
    lib.miniattn_fwd_balanced.argtypes = [C.POINTER(FwdParams), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.miniattn_fwd_balanced.restype = C.c_int
    lib.miniattn_fwd_balanced_scratch_bytes.argtypes = [C.POINTER(FwdParams)]
    lib.miniattn_fwd_balanced_scratch_bytes.restype = C.c_int64
    lib.miniattn_fwd_carry_bytes.argtypes = [C.POINTER(FwdParams)]
    lib.miniattn_fwd_carry_bytes.restype = C.c_int64
    lib.miniattn_plan_fwd.argtypes = [C.POINTER(FwdParams), C.c_int, C.POINTER(PlanInfo),
                                      C.POINTER(PlanPiece), C.c_int32]
    lib.miniattn_plan_fwd.restype = C.c_int
    lib.miniattn_fwd_int8qk_balanced.argtypes = [C.POINTER(Int8Params), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.miniattn_fwd_int8qk_balanced.restype = C.c_int
    for name in ("miniattn_quant_qk_int8", "miniattn_quant_qk_int8_static", "miniattn_fwd_int8qk"):
        getattr(lib, name).argtypes = [C.POINTER(Int8Params), C.c_void_p]
        getattr(lib, name).restype = C.c_int
    lib.miniattn_merge_partials.argtypes = [C.POINTER(MergeParams), C.c_void_p]
    lib.miniattn_merge_partials.restype = C.c_int
    lib.miniattn_selftest_wait.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p]
    lib.miniattn_selftest_wait.restype = C.c_int
    lib.miniattn_check_status.argtypes = [C.c_int32]
    lib.miniattn_check_status.restype = C.c_int
    lib.miniattn_version.restype = C.c_char_p
    lib.miniattn_last_error_string.restype = C.c_char_p
    return lib


lib = _load()


def last_error() -> str:
    return lib.miniattn_last_error_string().decode()


def check(rc: int, what: str) -> None:
    """Turn a negative return code into the exception the reference raises (RuntimeError
    from TORCH_CHECK, kernels/flash_attn/cuda/sm_120/kernel/flash_attention.cu:41-80)."""
    if rc != OK:
        raise RuntimeError(f"{what} failed ({rc}): {last_error()}")
