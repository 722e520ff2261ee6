"""ctypes binding of librwkv7_b200.so (the C ABI declared in include/rwkv7_b200.h).

There is no fallback: if the library is missing the import of this module fails, and
every wrapper raises on a non-zero status code.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
# RWKV7_B200_LIB selects another build of the same library (e.g. one compiled with different tuning macros)
LIB_PATH = os.environ.get("RWKV7_B200_LIB") or os.path.join(_HERE, "librwkv7_b200.so")

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_ALIGN, ERR_CUDA, ERR_WORKSPACE = 0, -1, -2, -3, -4, -5
F16, BF16, F32 = 0, 1, 2
EPI_NONE, EPI_RELU2, EPI_ADD = 0, 1, 2

P, I, F, L = c_void_p, c_int, c_float, c_int64
PP = ctypes.POINTER(c_void_p)

# name -> (restype, argtypes); must list every symbol of include/rwkv7_b200.h
SIGNATURES = {
    "rwkv7_abi_version": (I, []),
    "rwkv7_last_error": (ctypes.c_char_p, []),
    "rwkv7_kernel_status": (I, [I]),
    "rwkv7_relu2": (I, [P, P, ctypes.c_longlong, I, P]),
    "rwkv7_affine_gemv_workspace_bytes": (ctypes.c_int64, [I, I, I]),
    "rwkv7_affine_gemv": (I, [P] * 8 + [ctypes.c_int64, I, I, I, I, I, P]),
    "rwkv7_affine_dequant": (I, [P] * 6 + [I, I, I, I, P]),
    "rwkv7_a8w8_relu2_requant": (I, [P] * 6 + [I, I, I, P]),
    "rwkv7_wkv7_update": (I, [P] * 9 + [I, I, I, I, I, P]),
    "rwkv7_wkv7_output_prepare": (I, [P] * 13 + [I, I, I, F, I, I, P]),
    "rwkv7_wkv7_output_prepare_raw": (I, [P] * 14 + [P, P, I, P, P, P, I, P, I, I, I, I, F, I, P]),
    "rwkv7_wkv7_scan": (I, [P] * 13 + [F, I, I, I, I, I, I, P]),
    "rwkv7_wkv7_scan_f16state": (I, [P] * 13 + [F, I, I, I, I, I, I, I, P, P, P]),
    "rwkv7_wkv7_output_prepare_f16state": (I, [P] * 13 + [I, I, I, F, I, I, P]),
    "rwkv7_wkv7_output_prepare_raw_f16state": (I, [P] * 14 + [P, P, I, P, P, P, I, P, P, I, I, I, I, I, F, I, P]),
    "rwkv7_wkv7_chunk_scan": (I, [P] * 9 + [I, I, I, I, I, I, I, P]),
    "rwkv7_attn_norm_mix6": (I, [P, P, P, P, PP, PP, I, I, F, I, P]),
    "rwkv7_attn_norm_mix6_pool": (I, [P, P, P, P, P, PP, PP, I, I, F, I, P]),
    "rwkv7_ffn_add_norm_mix_pool": (I, [P] * 9 + [I, I, F, I, P]),
    "rwkv7_wkv7_output_prepare_raw_pool": (I, [P] * 14 + [P, P, I, P, P, P, I, P, I, I, I, I, F, I, P]),
    "rwkv7_ffn_add_norm_mix": (I, [P] * 8 + [I, I, F, I, P]),
    "rwkv7_layer_norm": (I, [P] * 4 + [I, I, F, I, P]),
    "rwkv7_seq_shift_mix": (I, [P, P, PP, PP, P, I, I, I, I, I, I, P]),
    "rwkv7_dense_small": (I, [P] * 4 + [I, I, I, I, I, I, P]),
    "rwkv7_small_gemm_group": (I, [I, PP, PP, PP, PP, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int), I, I, P]),
    "rwkv7_prefill_state_prep": (I, [P] * 12 + [I, I, I, I, I, I, I, P]),
    "rwkv7_attn_output_prepare": (I, [P] * 9 + [I, I, I, F, I, P]),
    "rwkv7_w4g_gemv": (I, [P] * 6 + [I, I, I, I, I, I, P]),
    "rwkv7_w4g_tiled_bytes": (L, [I, I]),
    "rwkv7_w4g_repack": (I, [P] * 4 + [I, I, I, I, P]),
    "rwkv7_w4g_gemv_tiled": (I, [P] * 4 + [I, I, I, I, I, P]),
    "rwkv7_w4g_gemv_tiled_group": (I, [P] * 3 + [I, I, I, I, I, I, P]),
    "rwkv7_w8_gemv": (I, [P] * 5 + [I, I, I, I, I, P]),
    "rwkv7_w8_tiled_bytes": (L, [I, I]),
    "rwkv7_w8_repack": (I, [P, P, I, I, P]),
    "rwkv7_w8_gemv_tiled_group": (I, [P] * 5 + [I, I, I, I, I, I, P]),
    "rwkv7_w4g_dequant": (I, [P] * 4 + [I, I, I, I, P]),
    "rwkv7_w8_dequant": (I, [P] * 3 + [I, I, I, P]),
    "rwkv7_a8_quant": (I, [P, P, P, I, I, I, P]),
    "rwkv7_i8_gemm": (I, [P, P, P, I, I, I, P]),
    "rwkv7_gemm": (I, [P, P, P, P, P, I, I, I, I, I, P]),
    "rwkv7_gemm_argmax_workspace_bytes": (L, [I, I]),
    "rwkv7_gemm_argmax": (I, [P, P, P, L, P, P, I, I, I, I, P]),
    "rwkv7_a8w8_dequant": (I, [P] * 6 + [I, I, I, P]),
    "rwkv7_a8w8_workspace_bytes": (L, [I, I, I]),
    "rwkv7_a8w8_linear": (I, [P] * 7 + [L, I, I, I, I, P]),
    "rwkv7_a8w8_linear_relu2": (I, [P] * 6 + [L, I, I, I, I, P]),
    "rwkv7_tp_allreduce_max_ctas": (I, []),
    "rwkv7_tp_allreduce": (I, [P, P, PP, PP, P, I, I, I, I, ctypes.c_longlong, I, I, P]),
    "rwkv7_tp_rows_resident": (I, [I, I]),
    "rwkv7_tp_attn_norm_mix6": (I, [P, P, P, P, P, P, PP, PP, PP, P, I, I, I, I, ctypes.c_longlong, I, F, I, I, P]),
    "rwkv7_tp_ffn_add_norm_mix": (I, [P] * 9 + [PP, P, I, I, I, I, ctypes.c_longlong, I, F, I, I, P]),
    "rwkv7_a8w8_static_capacity_bytes": (L, []),
    "rwkv7_a8w8_linear_static": (I, [P] * 6 + [I, I, I, I, P]),
}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python hf-adapter_b200/build.py` "
        "(this package has no CPU or PyTorch fallback)")

lib = ctypes.CDLL(LIB_PATH)
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = the library does not export a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.rwkv7_last_error().decode("utf-8", "replace")


LAUNCHES = 0  # kernels launched through this binding (bench.py reports it as gpu_launches)


def check(status: int, what: str, kernels: int = 1) -> None:
    """Map a status code to the exception class the reference raises for the same mistake:
    shape/dtype problems are ValueError (rwkv7_hf/fused_recurrent_update.py:993-1014), the rest RuntimeError."""
    if status == OK:
        global LAUNCHES
        LAUNCHES += kernels
        return
    msg = f"{what}: {last_error()} (status {status})"
    if status in (ERR_INVALID, ERR_UNSUPPORTED, ERR_ALIGN, ERR_WORKSPACE):
        raise ValueError(msg)
    raise RuntimeError(msg)


def ptr_array(ptrs):
    arr = (c_void_p * len(ptrs))(*ptrs)
    return ctypes.cast(arr, PP), arr


def kernel_status(reset: bool = True) -> int:
    """0 unless a tensor-core kernel's bounded wait gave up since the last reset (synchronises the device)."""
    return int(lib.rwkv7_kernel_status(1 if reset else 0))
