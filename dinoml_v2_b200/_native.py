"""ctypes binding of libdinoml_b200_gguf.so (the C-ABI kernel library).

There is no CPU or PyTorch fallback: if the library has not been built for sm_100a the loader
raises, and every op in this package goes through it.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libdinoml_b200_gguf.so"

VARIANTS = {"auto": 0, "simt": 1, "mma": 2, "umma": 3, "stream": 4}
VARIANT_NAMES = {v: k for k, v in VARIANTS.items()}
DINO_DTYPE = {"float16": 1, "float32": 2, "bfloat16": 6}
ACTIVATIONS = {"silu": 1, "fast_gelu": 2}
DEQUANT_DTYPE = {"float32": 0, "float16": 1, "bfloat16": 2}

_lib = None


def variant_code(variant) -> int:
    """"mma", "stream", ... or "stream:3" (family : tuning configuration) or an int code -> the C ABI's variant code."""
    if isinstance(variant, int):
        return variant
    family, _, config = str(variant).partition(":")
    if family not in VARIANTS:
        raise ValueError(f"unknown variant {variant!r}; families: {sorted(VARIANTS)}")
    return VARIANTS[family] | (int(config) << 8 if config else 0)


class NativeLibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise NativeLibraryMissing(
            f"{LIB_PATH} is missing: build the sm_100a kernels with `python -m dinoml_v2_b200.build` "
            "(there is no CPU fallback for the GGUF quantized-linear path)")
    L = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)
    vp, i64, ci, cf = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
    L.dinoml_b200_gguf_kernel_abi_version.restype = ci
    L.dino_get_last_error.restype = ctypes.c_char_p
    L.libgguf_cuda_dequantize_rows_on_stream.argtypes = [vp, i64, i64, i64, ci, vp, vp]
    L.libgguf_cuda_dequantize_rows_on_stream.restype = ci
    L.dinoml_b200_gguf_gemm_rcr.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp]
    L.dinoml_b200_gguf_gemm_rcr.restype = ci
    L.dinoml_profile_b200_gguf_gemm_rcr.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp]
    L.dinoml_profile_b200_gguf_gemm_rcr.restype = cf
    L.dinoml_b200_gguf_gemm_rcr_workspace.argtypes = [ci, ci, ci, ci, ci, ci]
    L.dinoml_b200_gguf_gemm_rcr_workspace.restype = ctypes.c_size_t
    L.dinoml_b200_gguf_gemm_rcr_select.argtypes = [ci, ci, ci, ci, ci]
    L.dinoml_b200_gguf_gemm_rcr_select.restype = ci
    L.dinoml_b200_gguf_variant_configs.argtypes = [ci]
    L.dinoml_b200_gguf_variant_configs.restype = ci
    L.dinoml_b200_gguf_variant_supports.argtypes = [ci, ci, ci, ci, ci, ci]
    L.dinoml_b200_gguf_variant_supports.restype = ci
    L.dinoml_b200_gguf_device_status.restype = ci
    L.dinoml_b200_gguf_gemv_rcr_scatter.argtypes = [vp, vp, vp, vp, ctypes.POINTER(vp), ci, ci, ci, ci, ci, ci, vp]
    L.dinoml_b200_gguf_gemv_rcr_scatter.restype = ci
    L.dinoml_b200_gguf_gemm_rcr_scatter.argtypes = [vp, vp, vp, vp, ctypes.POINTER(vp), ci, ci, ci, ci, ci, ci, ci, vp]
    L.dinoml_b200_gguf_gemm_rcr_scatter.restype = ci
    L.dinoml_b200_gguf_dual_gemm_rcr.argtypes = [vp, vp, vp, ctypes.POINTER(vp), ci, ci, ci, ci, ci, ci, ci, ci, vp]
    L.dinoml_b200_gguf_dual_gemm_rcr.restype = ci
    L.dinoml_b200_gguf_dual_gemm_rcr_bias.argtypes = [vp, vp, vp, vp, ctypes.POINTER(vp), ci, ci, ci, ci, ci, ci, ci, ci, vp]
    L.dinoml_b200_gguf_dual_gemm_rcr_bias.restype = ci
    L.dinoml_b200_peer_exchange.argtypes = [ctypes.POINTER(vp), ci, ci, ctypes.c_uint, vp, vp, i64, ci, vp]
    L.dinoml_b200_peer_exchange.restype = ci
    L.dinoml_b200_peer_pull.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(vp), ci, ci, ctypes.c_uint, ci, i64, i64, i64, i64, ci, vp]
    L.dinoml_b200_peer_pull.restype = ci
    L.dinoml_b200_peer_exchange_ctr.argtypes = [ctypes.POINTER(vp), ci, ci, vp, vp, vp, i64, ci, vp]
    L.dinoml_b200_peer_exchange_ctr.restype = ci
    L.dinoml_b200_peer_pull_ctr.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(vp), ci, ci, vp, ci, i64, i64, i64, i64, ci, vp]
    L.dinoml_b200_peer_pull_ctr.restype = ci
    L.dinoml_b200_peer_enable_access.argtypes = [ci]
    L.dinoml_b200_peer_enable_access.restype = ci
    _lib = L
    return L


def last_error() -> str:
    return (lib().dino_get_last_error() or b"").decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}: {last_error()}")


def candidate_symbol(qtype_symbol: str, dtype: str, variant: str, *, bias: bool = False, profile: bool = False):
    """Looks up one of the per-candidate symbols, e.g. dinoml_b200_gguf_q4_k_gemm_rcr_bfloat16_mma_v1."""
    op = "gemm_rcr_bias" if bias else "gemm_rcr"
    name = f"dinoml_{'profile_' if profile else ''}b200_gguf_{qtype_symbol}_{op}_{dtype}_{variant}_v1"
    fn = getattr(lib(), name)
    vp, ci = ctypes.c_void_p, ctypes.c_int
    if profile:
        fn.argtypes, fn.restype = [vp, vp, vp, ci, ci, ci, ci, vp], ctypes.c_float
    elif bias:
        fn.argtypes, fn.restype = [vp, vp, vp, vp, ci, ci, ci, vp], ci
    else:
        fn.argtypes, fn.restype = [vp, vp, vp, ci, ci, ci, vp], ci
    return fn
