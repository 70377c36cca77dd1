"""ctypes binding of the C-ABI launch shim (``include/axp_sm100.h``).

The shared library is built in-tree by ``csrc/Makefile`` into
``libaxp_sm100.so`` beside this file.  There is no CPU or library fallback:
if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("AXP_SM100_LIB") or os.path.join(_HERE, "libaxp_sm100.so")   # override: an alternative build of the same ABI

AXP_OK = 0
AXP_ERR_BAD_ARG = -1
AXP_ERR_UNSUPPORTED = -2
AXP_ERR_CUDA = -3
AXP_ERR_TIMEOUT = -4
AXP_ACT_NONE = 0
AXP_ACT_SILU = 1

#: every symbol ``include/axp_sm100.h`` declares
EXPORTS = (
    "axp_sm100_query",
    "axp_sm100_fnv1a64",
    "axp_sm100_gemm_fp8_blockscaled",
    "axp_sm100_gemm_bf16",
    "axp_sm100_gemm_bf16_bias_act",
    "axp_sm100_gemm_fp8_blockscaled_bias_act",
    "axp_sm100_gemm_bf16_swiglu",
    "axp_sm100_gemm_fp8_blockscaled_swiglu",
    "axp_sm100_gemm_fp8_blockscaled_swiglu_quant",
    "axp_sm100_gemm_fp8_blockscaled_quant",
    "axp_sm100_gemm_bf16_lincomb",
    "axp_sm100_gemm_fp8_blockscaled_lincomb",
    "axp_sm100_quantize_rows_e4m3",
    "axp_sm100_rmsnorm_quantize_rows_e4m3",
    "axp_sm100_attn_fwd_bf16",
    "axp_sm100_attn_fwd_fp8",
    "axp_sm100_attn_splitkv_scratch_bytes",
    "axp_sm100_attn_fwd_bf16_splitkv",
    "axp_sm100_attn_fwd_fp8_splitkv",
    "axp_sm100_attn_partial_bytes",
    "axp_sm100_attn_fwd_bf16_kvshard",
    "axp_sm100_attn_fwd_fp8_kvshard",
    "axp_sm100_attn_combine_partials",
    "axp_sm100_attn_splitkv_static_scratch_bytes",
    "axp_sm100_attn_fwd_bf16_splitkv_static",
    "axp_sm100_causal_mask_tile",
    "axp_sm100_selftest_bounded_wait",
    "axp_sm100_set_option",
    "axp_sm100_last_error",
)


class AxpError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"axp_sm100 error {code}: {message}")
        self.code = code


class Caps(ctypes.Structure):
    _fields_ = [
        ("realization_key", ctypes.c_uint64),
        ("op_family", ctypes.c_int32),
        ("elem_bits", ctypes.c_int32),
        ("tile_m", ctypes.c_int32),
        ("tile_n", ctypes.c_int32),
        ("tile_k", ctypes.c_int32),
        ("cta_group", ctypes.c_int32),
        ("stages", ctypes.c_int32),
        ("smem_bytes", ctypes.c_int32),
        ("tmem_columns", ctypes.c_int32),
        ("threads", ctypes.c_int32),
    ]


def build(verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a (nvcc cross-compiles without a GPU)."""
    out = subprocess.run(["make", "-C", os.path.join(_HERE, "csrc"), "-s"], capture_output=True, text=True)
    if verbose or out.returncode != 0:
        print(out.stdout)
        print(out.stderr)
    if out.returncode != 0:
        raise RuntimeError("building libaxp_sm100.so failed")
    return LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    """The loaded shim; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
                "(there is no fallback path)")
        L = ctypes.CDLL(LIB_PATH)
        i64, vp, u32p, fp = ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p
        L.axp_sm100_query.argtypes = [ctypes.c_uint64, ctypes.POINTER(Caps)]
        L.axp_sm100_query.restype = ctypes.c_int
        L.axp_sm100_fnv1a64.argtypes = [ctypes.c_char_p]
        L.axp_sm100_fnv1a64.restype = ctypes.c_uint64
        L.axp_sm100_gemm_fp8_blockscaled.argtypes = [vp, vp, fp, fp, vp, i64, i64, i64, i64, i64, i64, i64, i64, vp, u32p]
        L.axp_sm100_gemm_fp8_blockscaled.restype = ctypes.c_int
        L.axp_sm100_gemm_bf16.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, vp, u32p]
        L.axp_sm100_gemm_bf16.restype = ctypes.c_int
        L.axp_sm100_gemm_bf16_bias_act.argtypes = [vp, vp, fp, vp, i64, i64, i64, i64, i64, i64, i64, i64, ctypes.c_int, vp, u32p]
        L.axp_sm100_gemm_bf16_bias_act.restype = ctypes.c_int
        L.axp_sm100_gemm_fp8_blockscaled_bias_act.argtypes = [vp, vp, fp, fp, fp, vp, i64, i64, i64, i64, i64, i64, i64, i64,
                                                             ctypes.c_int, vp, u32p]
        L.axp_sm100_gemm_fp8_blockscaled_bias_act.restype = ctypes.c_int
        L.axp_sm100_quantize_rows_e4m3.argtypes = [vp, vp, fp, i64, i64, i64, i64, vp]
        L.axp_sm100_quantize_rows_e4m3.restype = ctypes.c_int
        L.axp_sm100_rmsnorm_quantize_rows_e4m3.argtypes = [vp, vp, ctypes.c_float, vp, fp, i64, i64, i64, i64, vp]
        L.axp_sm100_rmsnorm_quantize_rows_e4m3.restype = ctypes.c_int
        cf = ctypes.c_float
        L.axp_sm100_gemm_bf16_lincomb.argtypes = [vp, vp, vp, vp, cf, cf, i64, i64, i64, i64, i64, i64, i64, i64, i64, vp, u32p]
        L.axp_sm100_gemm_bf16_lincomb.restype = ctypes.c_int
        L.axp_sm100_gemm_fp8_blockscaled_lincomb.argtypes = [vp, vp, fp, fp, vp, vp, cf, cf, i64, i64, i64, i64, i64, i64, i64, i64, i64,
                                                             vp, u32p]
        L.axp_sm100_gemm_fp8_blockscaled_lincomb.restype = ctypes.c_int
        L.axp_sm100_gemm_bf16_swiglu.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, i64, vp, u32p]
        L.axp_sm100_gemm_bf16_swiglu.restype = ctypes.c_int
        L.axp_sm100_gemm_fp8_blockscaled_swiglu.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, i64, vp, u32p]
        L.axp_sm100_gemm_fp8_blockscaled_swiglu.restype = ctypes.c_int
        L.axp_sm100_gemm_fp8_blockscaled_swiglu_quant.argtypes = [vp, vp, vp, vp, vp, vp, vp, fp, i64, i64, i64, i64, i64, i64, i64, i64, i64, vp, u32p]
        L.axp_sm100_gemm_fp8_blockscaled_swiglu_quant.restype = ctypes.c_int
        L.axp_sm100_gemm_fp8_blockscaled_quant.argtypes = [vp, vp, fp, fp, fp, ctypes.c_int, vp, fp, i64, i64, i64, i64, i64, i64, i64, i64, vp, u32p]
        L.axp_sm100_gemm_fp8_blockscaled_quant.restype = ctypes.c_int
        L.axp_sm100_attn_fwd_bf16.argtypes = [vp, vp, vp, vp, fp, i64, i64, i64, i64, i64, ctypes.c_float,
                                              ctypes.c_int, i64, i64, vp, u32p]
        L.axp_sm100_attn_fwd_bf16.restype = ctypes.c_int
        L.axp_sm100_attn_fwd_fp8.argtypes = [vp, vp, vp, fp, fp, fp, vp, fp, i64, i64, i64, i64, i64, ctypes.c_float,
                                             ctypes.c_int, i64, i64, vp, u32p]
        L.axp_sm100_attn_fwd_fp8.restype = ctypes.c_int
        L.axp_sm100_attn_splitkv_scratch_bytes.argtypes = [i64, i64, i64]
        L.axp_sm100_attn_splitkv_scratch_bytes.restype = ctypes.c_int64
        L.axp_sm100_attn_fwd_bf16_splitkv.argtypes = [vp, vp, vp, vp, fp, i64, i64, i64, i64, i64, i64, ctypes.c_float,
                                                      ctypes.c_int, i64, vp, i64, i64, i64, vp, u32p]
        L.axp_sm100_attn_fwd_bf16_splitkv.restype = ctypes.c_int
        L.axp_sm100_attn_fwd_fp8_splitkv.argtypes = [vp, vp, vp, fp, fp, fp, vp, fp, i64, i64, i64, i64, i64, i64, ctypes.c_float,
                                                     ctypes.c_int, i64, vp, i64, i64, i64, vp, u32p]
        L.axp_sm100_attn_fwd_fp8_splitkv.restype = ctypes.c_int
        L.axp_sm100_attn_partial_bytes.argtypes = [i64, i64]
        L.axp_sm100_attn_partial_bytes.restype = ctypes.c_int64
        L.axp_sm100_attn_fwd_bf16_kvshard.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, i64, ctypes.c_float,
                                                      ctypes.c_int, i64, i64, vp, u32p]
        L.axp_sm100_attn_fwd_bf16_kvshard.restype = ctypes.c_int
        L.axp_sm100_attn_fwd_fp8_kvshard.argtypes = [vp, vp, vp, fp, fp, fp, vp, i64, i64, i64, i64, i64, i64, i64, i64, i64,
                                                     ctypes.c_float, ctypes.c_int, i64, i64, vp, u32p]
        L.axp_sm100_attn_fwd_fp8_kvshard.restype = ctypes.c_int
        L.axp_sm100_attn_combine_partials.argtypes = [vp, i64, i64, vp, fp, i64, vp]
        L.axp_sm100_attn_combine_partials.restype = ctypes.c_int
        L.axp_sm100_attn_splitkv_static_scratch_bytes.argtypes = []
        L.axp_sm100_attn_splitkv_static_scratch_bytes.restype = ctypes.c_int64
        L.axp_sm100_attn_fwd_bf16_splitkv_static.argtypes = [vp, vp, vp, vp, fp, i64, i64, i64, i64, i64, i64, ctypes.c_float,
                                                             ctypes.c_int, i64, i64, i64, vp, u32p]
        L.axp_sm100_attn_fwd_bf16_splitkv_static.restype = ctypes.c_int
        L.axp_sm100_causal_mask_tile.argtypes = [i64, i64, ctypes.c_int32, ctypes.c_int32, vp, vp, vp]
        L.axp_sm100_causal_mask_tile.restype = ctypes.c_int
        L.axp_sm100_selftest_bounded_wait.argtypes = [i64, vp, u32p]
        L.axp_sm100_selftest_bounded_wait.restype = ctypes.c_int
        L.axp_sm100_set_option.argtypes = [ctypes.c_char_p, i64]
        L.axp_sm100_set_option.restype = ctypes.c_int
        L.axp_sm100_last_error.argtypes = []
        L.axp_sm100_last_error.restype = ctypes.c_char_p
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != AXP_OK:
        raise AxpError(rc, lib().axp_sm100_last_error().decode("utf-8", "replace"))


def set_option(name: str, value: int) -> None:
    """Process-wide tuning option (0 restores the default); see ``axp_sm100_set_option``."""
    check(lib().axp_sm100_set_option(name.encode(), int(value)))


def fnv1a64(s: str) -> int:
    return int(lib().axp_sm100_fnv1a64(s.encode()))


def query(realization_key: str | int) -> Caps:
    key = fnv1a64(realization_key) if isinstance(realization_key, str) else int(realization_key)
    caps = Caps()
    check(lib().axp_sm100_query(ctypes.c_uint64(key), ctypes.byref(caps)))
    return caps
