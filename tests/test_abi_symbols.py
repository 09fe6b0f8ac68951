"""CPU test: the C-ABI library builds for sm_100a, loads, and exports every symbol include/*.h declares.
No kernel is launched here."""
import ctypes
import re
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADERS = sorted((ROOT / "include").glob("*.h"))


def declared_symbols():
    names = set()
    for header in HEADERS:
        text = subprocess.run(["gcc", "-E", "-P", str(header)], capture_output=True, text=True, check=True).stdout
        names |= set(re.findall(r"\b((?:dinoml_|dino_|libgguf_cuda_)\w+)\s*\(", text))
    return sorted(names)


@pytest.fixture(scope="module")
def library():
    from dinoml_v2_b200 import _native, build
    if not _native.LIB_PATH.exists():
        if shutil.which("nvcc") is None:
            pytest.skip("nvcc not available and the library is not prebuilt")
        build.build()
    return ctypes.CDLL(str(_native.LIB_PATH))


def test_header_declares_the_expected_families():
    names = declared_symbols()
    assert "libgguf_cuda_dequantize_rows_on_stream" in names
    assert "dinoml_b200_gguf_gemm_rcr" in names
    for q in ("q8_0", "q4_k", "q6_k"):
        assert f"dinoml_b200_gguf_{q}_gemm_rcr_bfloat16_mma_v1" in names
        assert f"dinoml_b200_gguf_{q}_gemm_rcr_bias_float16_umma_v1" in names
        assert f"dinoml_profile_b200_gguf_{q}_gemm_rcr_float32_simt_v1" in names
    for name in ("dino_abi_version", "dino_module_load_deferred", "dino_module_set_encoded_constant",
                 "dino_session_create", "dino_session_run", "dino_session_benchmark"):
        assert name in names, name


def test_library_exports_every_declared_symbol(library):
    missing = [n for n in declared_symbols() if not hasattr(library, n)]
    assert not missing, missing


def test_versions_and_pure_host_entry_points(library):
    library.dinoml_b200_gguf_kernel_abi_version.restype = ctypes.c_int
    assert library.dinoml_b200_gguf_kernel_abi_version() == 1
    library.dino_abi_version.restype = ctypes.c_int
    assert library.dino_abi_version() == 7          # runtime ABI of the reference, runtime/include/dinoml/abi.h:12
    sel = library.dinoml_b200_gguf_gemm_rcr_select
    sel.argtypes = [ctypes.c_int] * 5
    assert sel(12, 6, 1, 11008, 4096) == 2           # Q4_K bf16 M=1 -> mma GEMV
    assert sel(12, 2, 1, 11008, 4096) == 1           # float32 activations -> simt
    # the shape guard without a GPU (148 SMs assumed): Q4_K M=1 with few row tiles - tile GEMV on a short K, persistent one on a long K
    assert sel(12, 6, 1, 1024, 4096) == 2 and sel(12, 6, 1, 1024, 14336) == 4
    # Q4_K M=8 with few row tiles: persistent GEMV on K = 4096, K-sliced tile GEMV on a long K
    assert sel(12, 6, 8, 1024, 4096) == 4 and sel(12, 6, 8, 256, 14336) == 2
    # the further types: persistent GEMV up to M = 8, tcgen05 GEMM above, CUDA-core kernel when rows are not 16-byte multiples
    for q, bad_k in ((2, None), (13, None), (10, 768), (11, 1024), (39, 768), (40, None)):
        assert sel(q, 6, 1, 4096, 4096) == 4 and sel(q, 6, 8, 4096, 4096) == 4 and sel(q, 6, 16, 4096, 4096) == 3, q
        assert sel(q, 2, 4, 4096, 4096) == 1, q
        if bad_k:
            assert sel(q, 6, 1, 64, bad_k) == 1 and sel(q, 6, 64, 64, bad_k) == 1, q
    # argument validation happens before any CUDA call
    f = library.dinoml_b200_gguf_gemm_rcr
    f.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 6 + [ctypes.c_void_p]
    assert f(None, None, None, None, 12, 6, 1, 16, 256, 0, None) == 1
    library.dino_get_last_error.restype = ctypes.c_char_p
    assert b"null pointer" in library.dino_get_last_error()
    d = library.libgguf_cuda_dequantize_rows_on_stream
    d.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    assert d(16, 12, 4, 100, 0, 16, None) == 3       # n_per_row not a multiple of 256
    assert d(16, 99, 4, 256, 0, 16, None) == 5
    assert d(16, 12, 0, 256, 0, 16, None) == 2


def test_host_conversions_round_like_the_reference(library):
    """float32 -> bfloat16 bits: round to nearest even, the integer formula of the reference's Python (src/dinoml/ir.py:68-73);
    bfloat16 -> float32: the 16 bits followed by 16 zeros.  Every length around the vector width, odd addresses included."""
    import numpy as np
    vp = ctypes.c_void_p
    narrow, widen = library.dino_convert_f32_to_bf16, library.dino_convert_bf16_to_f32
    for fn in (narrow, widen):
        fn.argtypes, fn.restype = [vp, vp, ctypes.c_size_t], None
    rng = np.random.Generator(np.random.PCG64(3))
    for count in (0, 1, 7, 8, 9, 31, 4096, 11009):
        x = (rng.standard_normal(count + 1) * np.float32(10.0) ** rng.integers(-20, 20, count + 1)).astype(np.float32)[1:]   # 4-byte, not 16-byte aligned
        x[: min(count, 6)] = np.array([0.0, -0.0, np.inf, -np.inf, 1.00390625, 1.01171875], np.float32)[: min(count, 6)]         # ties to even both ways
        bits = np.empty(count + 1, np.uint16)[1:]
        narrow(x.ctypes.data, bits.ctypes.data, count)
        b = x.view(np.uint32).astype(np.uint64)
        assert np.array_equal(bits, (((b + 0x7FFF + ((b >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)), count
        back = np.empty(count + 1, np.float32)[1:]
        widen(bits.ctypes.data, back.ctypes.data, count)
        assert np.array_equal(back.view(np.uint32), bits.astype(np.uint32) << 16), count
