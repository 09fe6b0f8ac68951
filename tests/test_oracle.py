"""CPU tests: the oracle against the committed golden vectors, its numpy twin, the reference's own
CPU kernel (when oracle/_ref was built) and the independent `gguf` package (when importable)."""
import numpy as np
import pytest

import oracle
from dinoml_v2_b200 import synthetic as S
from dinoml_v2_b200.gguf_blocks import QTYPES, encoded_nbytes, qtype_of, row_bytes

QT3 = ("Q8_0", "Q4_K", "Q6_K")                                  # the benchmark types (they also have a numpy twin)
QT = QT3 + ("Q4_0", "Q5_K", "Q2_K", "Q3_K", "MXFP4", "NVFP4")     # + the six further types of the reference prototype


@pytest.fixture(scope="module")
def kat(golden_dir):
    return np.load(golden_dir / "gguf_dequant_kat.npz")


@pytest.fixture(scope="module")
def gemm_golden(golden_dir):
    return np.load(golden_dir / "gemm_rcr_reference_cpu.npz")


def test_block_tables_match_reference_struct_sizes():
    # sizes pinned by the reference's own test, tests/backends/test_ck_gguf_q8_gemm_kernel.py:59,82-89
    assert (QTYPES["Q8_0"].block_bytes, QTYPES["Q4_K"].block_bytes, QTYPES["Q6_K"].block_bytes) == (34, 144, 210)
    assert [QTYPES[q].value for q in QT] == [8, 12, 14, 2, 13, 10, 11, 39, 40]
    # tools/bench_ck_gguf_q8_gemm.hip:39,46,55,65,74,83,92,99,106 (static_asserts on the block structs)
    assert [QTYPES[q].block_bytes for q in QT] == [34, 144, 210, 18, 176, 84, 110, 17, 36]
    assert [QTYPES[q].block_size for q in QT] == [32, 256, 256, 32, 256, 256, 256, 32, 64]
    assert row_bytes("Q4_K", 4096) == 2304 and row_bytes("Q6_K", 14336) == 11760 and row_bytes("Q8_0", 4096) == 4352
    assert encoded_nbytes("Q4_K", 11008, 4096) == 25_362_432
    assert encoded_nbytes("Q6_K", 4096, 14336) == 48_168_960
    assert encoded_nbytes("Q8_0", 4096, 4096) == 17_825_792
    with pytest.raises(ValueError):
        row_bytes("Q4_K", 4000)
    with pytest.raises(ValueError):
        qtype_of("IQ4_XS")


@pytest.mark.parametrize("qtype", QT)
def test_oracle_matches_golden_dequant(kat, qtype):
    blocks, k = kat[f"{qtype}_blocks"], int(kat[f"{qtype}_n_per_row"])
    assert np.array_equal(oracle.dequantize(blocks, qtype, k, "float32").view(np.uint32), kat[f"{qtype}_f32_bits"])
    assert np.array_equal(oracle.dequantize(blocks, qtype, k, "float16").view(np.uint16), kat[f"{qtype}_f16_bits"])
    assert np.array_equal(oracle.dequantize(blocks, qtype, k, "bfloat16"), kat[f"{qtype}_bf16_bits"])
    if qtype in QT3:
        assert np.array_equal(oracle.dequantize_numpy(blocks, qtype, k).view(np.uint32), kat[f"{qtype}_f32_bits"])


@pytest.mark.parametrize("qtype", QT)
def test_oracle_matches_gguf_package(qtype):
    gguf = pytest.importorskip("gguf")
    t = getattr(gguf.GGMLQuantizationType, qtype)
    k = 4 * qtype_of(qtype).block_size
    blocks = S.random_blocks(qtype, 33, k, seed=77)
    want = gguf.quants.dequantize(blocks, t).astype(np.float32)
    assert np.array_equal(oracle.dequantize(blocks, qtype, k).view(np.uint32), want.view(np.uint32))


def _reference_host_library():
    """oracle/_ref/libref_gguf_host.so: the reference's own host decode functions, lifted and built by oracle/build_ref.py
    where the reference tree is present.  Absent on a machine without that tree (the committed fixtures cover it there)."""
    import ctypes
    from pathlib import Path
    path = Path(oracle.__file__).resolve().parent / "_ref" / "libref_gguf_host.so"
    if not path.exists():
        pytest.skip("oracle/_ref/libref_gguf_host.so not built (no reference tree on this machine)")
    lib = ctypes.CDLL(str(path))
    lib.ref_half_bits_to_float.restype = ctypes.c_float
    lib.ref_half_bits_to_float.argtypes = [ctypes.c_uint16]
    lib.ref_float_to_half_bits.restype = ctypes.c_uint16
    lib.ref_float_to_half_bits.argtypes = [ctypes.c_float]
    return lib


@pytest.mark.parametrize("qtype", QT)
def test_oracle_matches_the_references_own_host_functions(qtype, kat):
    """Bit for bit against `<qtype>_value_host` and `reference_gemm_quant` of tools/bench_ck_gguf_q8_gemm.hip (compiled from the
    reference's source with -ffp-contract=off): golden edge blocks, seeded synthetic blocks and blocks of uniformly random
    BYTES (every scale bit pattern, NaN and Inf included - compared as bit patterns)."""
    import ctypes
    lib = _reference_host_library()
    q = qtype_of(qtype)
    bs, bb = ctypes.c_int(), ctypes.c_int()
    assert lib.ref_gguf_block_geometry(q.value, ctypes.byref(bs), ctypes.byref(bb)) == 0
    assert (bs.value, bb.value) == (q.block_size, q.block_bytes)
    k = 4 * q.block_size
    rng = np.random.default_rng(2024)
    for blocks in (kat[f"{qtype}_blocks"], S.random_blocks(qtype, 9, k, seed=5), rng.integers(0, 256, (7, 4 * q.block_bytes), dtype=np.uint8)):
        kk = blocks.shape[1] // q.block_bytes * q.block_size
        mine = oracle.dequantize(blocks, qtype, kk)
        ref = np.empty_like(mine)
        assert lib.ref_gguf_dequantize_rows(blocks.ctypes.data_as(ctypes.c_void_p), q.value, ctypes.c_int64(blocks.shape[0]),
                                            ctypes.c_int64(kk), ref.ctypes.data_as(ctypes.c_void_p)) == 0
        assert np.array_equal(mine.view(np.uint32), ref.view(np.uint32)), qtype
    # the quantized matmul: same accumulation order => identical bits with fp32 weights.  With f16_dequant the bench tool rounds
    # each weight through ITS float_to_half_bits, which rounds ties upward (mant + 0x1000, tools/bench_ck_gguf_q8_gemm.hip:411-437);
    # the oracle rounds to nearest even like the GPU's cvt.rn and numpy, so the two differ by one fp16 ulp on tied weights only.
    n, m = 11, 3
    blocks = S.random_blocks(qtype, n, k, seed=6)
    a = S.random_activations(m, k, 7, "float32")
    for f16 in (0, 1):
        ref = np.empty((m, n), dtype=np.float32)
        assert lib.ref_gguf_gemm_quant(a.ctypes.data_as(ctypes.c_void_p), blocks.ctypes.data_as(ctypes.c_void_p), q.value, m, n, k, f16,
                                       ref.ctypes.data_as(ctypes.c_void_p)) == 0
        mine = oracle.gemm_quant(a, blocks, qtype, n, k, round_w=f16)
        if f16 == 0:
            assert np.array_equal(mine.view(np.uint32), ref.view(np.uint32)), qtype
        else:
            assert oracle.max_errors(ref, mine)[2] <= 1e-3, qtype


def test_oracle_half_conversions_and_error_metric_match_the_reference():
    import ctypes
    lib = _reference_host_library()
    L = oracle.lib()
    L.oracle_half_to_float.restype = ctypes.c_float
    L.oracle_half_to_float.argtypes = [ctypes.c_uint16]
    for h in range(0, 65536, 7):                      # every seventh fp16 bit pattern, plus the edges
        assert np.float32(L.oracle_half_to_float(h)).view(np.uint32) == np.float32(lib.ref_half_bits_to_float(h)).view(np.uint32), h
    for h in (0, 1, 0x03ff, 0x0400, 0x7bff, 0x7c00, 0x7e00, 0x8000, 0xfbff, 0xffff):
        assert np.float32(L.oracle_half_to_float(h)).view(np.uint32) == np.float32(lib.ref_half_bits_to_float(h)).view(np.uint32), h
    # float -> half: identical wherever the value is not a tie between two halves (the tool rounds ties up, the oracle to even)
    L.oracle_float_to_half.restype = ctypes.c_uint16
    L.oracle_float_to_half.argtypes = [ctypes.c_float]
    vals = (S.random_activations(1, 2000, 8, "float32").reshape(-1) * np.float32(3.7)).astype(np.float32)
    not_tie = (vals.view(np.uint32) & 0x1fff) != 0x1000
    for v in vals[not_tie]:
        assert L.oracle_float_to_half(float(v)) == lib.ref_float_to_half_bits(float(v)), float(v)
    e = S.random_activations(1, 4096, 3, "float32").reshape(-1) * 10
    a = e + S.random_activations(1, 4096, 4, "float32").reshape(-1) * 0.01
    ma, mr = ctypes.c_float(), ctypes.c_float()
    lib.ref_gguf_max_errors(e.ctypes.data_as(ctypes.c_void_p), a.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(e.size), ctypes.byref(ma), ctypes.byref(mr))
    max_abs, rel, _ = oracle.max_errors(e, a)
    assert abs(max_abs - ma.value) <= 1e-6 * max_abs and abs(rel - mr.value) <= 1e-6 * rel


@pytest.mark.parametrize("qtype", QT3)
def test_numpy_twin_equals_c_on_random_blocks(qtype):
    k = 3 * qtype_of(qtype).block_size
    blocks = S.random_blocks(qtype, 17, k, seed=11)
    assert np.array_equal(oracle.dequantize(blocks, qtype, k).view(np.uint32),
                          oracle.dequantize_numpy(blocks, qtype, k).view(np.uint32))


def test_oracle_error_codes():
    b = S.random_blocks("Q4_K", 2, 256, seed=1)
    with pytest.raises(ValueError):
        oracle.dequantize(b, 99, 256)
    with pytest.raises(ValueError):
        oracle.dequantize(b[:, :100], "Q4_K", 100)


def test_packers_round_trip_fields():
    rng = np.random.Generator(np.random.PCG64(3))
    sc = rng.integers(0, 64, size=(5, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(5, 8), dtype=np.uint8)
    packed = S.pack_k4_scales(sc, mn)
    for j in range(8):  # the unpack of kernels/rocm/src/ck_gguf_q8_gemm.hip:143-155
        if j < 4:
            d, m = packed[:, j] & 63, packed[:, j + 4] & 63
        else:
            d = (packed[:, j + 4] & 0x0F) | ((packed[:, j - 4] >> 6) << 4)
            m = (packed[:, j + 4] >> 4) | ((packed[:, j] >> 6) << 4)
        assert np.array_equal(d, sc[:, j]) and np.array_equal(m, mn[:, j])
    # Q6_K: dequantized value recovers (q - 32) * scale * d exactly for d = 1, scale = 1
    q = rng.integers(0, 64, size=(2, 256), dtype=np.uint8)
    blk = S.pack_q6_k(np.ones(2, np.float16), np.ones((2, 16), np.int8), q).reshape(2, 210)
    assert np.array_equal(oracle.dequantize(blk, "Q6_K", 256), q.astype(np.float32) - 32)
    q4 = rng.integers(0, 16, size=(2, 256), dtype=np.uint8)
    blk = S.pack_q4_k(np.ones(2, np.float16), np.zeros(2, np.float16), np.ones((2, 8), np.uint8), np.zeros((2, 8), np.uint8), q4)
    assert np.array_equal(oracle.dequantize(blk.reshape(2, 144), "Q4_K", 256), q4.astype(np.float32))


def test_synthetic_distributions():
    b = S.random_blocks("Q4_K", 64, 1024, seed=5).reshape(64, 4, 144)
    d = b[..., 0:2].copy().view(np.float16).astype(np.float32)
    assert 0.003 < d.mean() < 0.005 and (d >= 0).all()          # E|N(0,1)|*0.005 = 0.00399
    b8 = S.random_blocks("Q8_0", 64, 1024, seed=5).reshape(64, 32, 34)
    qs = b8[..., 2:].view(np.int8)
    assert qs.min() == -127 and qs.max() == 127
    b6 = S.random_blocks("Q6_K", 64, 1024, seed=5).reshape(64, 4, 210)
    sc = b6[..., 192:208].view(np.int8)
    assert sc.min() == -64 and sc.max() == 63
    assert np.array_equal(S.random_blocks("Q6_K", 4, 512, seed=9), S.random_blocks("Q6_K", 4, 512, seed=9))


def _case_inputs(gemm_golden, i):
    qtype, dtype, m, n, k = str(gemm_golden["cases"][i]).split("|")
    return qtype, dtype, int(m), int(n), int(k), gemm_golden[f"case{i}_blocks"], gemm_golden[f"case{i}_x_f32"], \
        np.asarray(gemm_golden[f"case{i}_y"], dtype=np.float32)


def _round(x, dtype):
    if dtype == "bfloat16":
        return S.bf16_bits_to_float32(S.float32_to_bf16_bits(x))
    if dtype == "float16":
        return x.astype(np.float16).astype(np.float32)
    return x


def test_oracle_matches_reference_cpu_artifact(gemm_golden):
    """The oracle's restatement of the CPU path against outputs the reference itself produced."""
    for i in range(len(gemm_golden["cases"])):
        qtype, dtype, m, n, k, blocks, x, y_ref = _case_inputs(gemm_golden, i)
        w = oracle.dequantize(blocks, qtype, k)
        code = {"float32": 0, "float16": 1, "bfloat16": 2}[dtype]
        # (1) quantized restatement (reference_gemm_quant) with weights rounded like the dense constant
        y_q = _round(oracle.gemm_quant(_round(x, dtype), blocks, qtype, n, k, round_w=code), dtype)
        # (2) dense restatement of gemm_cpu.cpp.j2 on the storage dtype
        if dtype == "bfloat16":
            y_d = S.bf16_bits_to_float32(oracle.gemm_rcr_dense(S.float32_to_bf16_bits(x), S.float32_to_bf16_bits(w), dtype))
        elif dtype == "float16":
            y_d = oracle.gemm_rcr_dense(x.astype(np.float16), w.astype(np.float16), dtype).astype(np.float32)
        else:
            y_d = oracle.gemm_rcr_dense(x, w, dtype)
        assert np.array_equal(y_q, y_d), (i, "quantized and dense restatements must agree bit for bit")
        # the reference kernel is built with -ffast-math (vectorised sum order) => tolerance, not bits
        _, rel, norm = oracle.max_errors(y_ref, y_d)
        tol = {"float32": 1e-4, "float16": 2e-3, "bfloat16": 1.6e-2}[dtype]
        assert rel <= tol and norm <= tol, (i, qtype, dtype, rel, norm)


def test_reference_cpu_kernel_build_matches_golden(gemm_golden):
    """oracle/_ref (the reference's gemm_cpu kernel compiled from its template) vs the reference artifact."""
    import ctypes
    from pathlib import Path
    ref_dir = Path(oracle.__file__).parent / "_ref"
    lib_path = ref_dir / "libref_gemm_cpu_v3.so"
    if not lib_path.exists():
        pytest.skip("oracle/_ref not built (reference tree absent at build time)")
    L = ctypes.CDLL(str(lib_path))
    for i in range(len(gemm_golden["cases"])):
        qtype, dtype, m, n, k, blocks, x, y_ref = _case_inputs(gemm_golden, i)
        w = oracle.dequantize(blocks, qtype, k)
        if dtype == "bfloat16":
            xs, ws, ys = S.float32_to_bf16_bits(x), S.float32_to_bf16_bits(w), np.empty((m, n), np.uint16)
        elif dtype == "float16":
            xs, ws, ys = x.astype(np.float16), w.astype(np.float16), np.empty((m, n), np.float16)
        else:
            xs, ws, ys = x, w, np.empty((m, n), np.float32)
        fn = getattr(L, f"ref_gemm_rcr_{dtype}")
        fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 3
        assert fn(xs.ctypes.data, ws.ctypes.data, ys.ctypes.data, m, n, k) == 0
        got = S.bf16_bits_to_float32(ys) if dtype == "bfloat16" else ys.astype(np.float32)
        _, rel, norm = oracle.max_errors(y_ref, got)
        tol = {"float32": 1e-4, "float16": 2e-3, "bfloat16": 1.6e-2}[dtype]
        assert rel <= tol and norm <= tol, (i, rel, norm)


def test_dual_gemm_oracle_and_row_interleave():
    """silu / fast_gelu gating in float32 as the reference CPU template computes it, and the row order the fused kernels read."""
    from dinoml_v2_b200 import synthetic as S
    n, k = 16, 256
    b0, b1 = S.random_blocks("Q4_K", n, k, 1), S.random_blocks("Q4_K", n, k, 2)
    x = S.random_activations(3, k, 3, "float32")
    left = oracle.gemm_quant(x, b0, "Q4_K", n, k).astype(np.float64)
    right = oracle.gemm_quant(x, b1, "Q4_K", n, k).astype(np.float64)
    want = left / (1.0 + np.exp(-left)) * right
    got = oracle.dual_gemm_quant(x, b0, b1, "Q4_K", n, k, "silu")
    assert got.dtype == np.float32 and np.allclose(got, want, rtol=1e-5, atol=1e-6)
    gelu = 0.5 * left * (1.0 + np.tanh(0.7978845608 * left * (1.0 + 0.044715 * left * left))) * right
    assert np.allclose(oracle.dual_gemm_quant(x, b0, b1, "Q4_K", n, k, "fast_gelu"), gelu, rtol=1e-5, atol=1e-6)
    # the _bias_ forms and the B1 [1, K] broadcast (dual_gemm_cpu.cpp.j2:58-69)
    bias0, bias1 = np.linspace(-1, 1, n).astype(np.float32), np.array([0.25], dtype=np.float32)
    lb, rb = left + bias0, right[:, :1] + bias1
    want_b = lb / (1.0 + np.exp(-lb)) * rb
    got_b = oracle.dual_gemm_quant(x, b0, b1[:1], "Q4_K", n, k, "silu", bias0, bias1)
    assert got_b.shape == (3, n) and np.allclose(got_b, want_b, rtol=1e-5, atol=1e-6)
    rows0, rows1 = np.arange(16, dtype=np.uint8).reshape(16, 1), 100 + np.arange(16, dtype=np.uint8).reshape(16, 1)
    order = [0, 1, 2, 3, 4, 5, 6, 7, 100, 101, 102, 103, 104, 105, 106, 107, 8, 9, 10, 11, 12, 13, 14, 15, 108, 109, 110, 111, 112, 113, 114, 115]
    # interleave_rows8 needs torch only for tensors; numpy inputs stay on the CPU
    pytest = __import__("pytest")
    kernels = pytest.importorskip("dinoml_v2_b200.kernels")
    assert kernels.interleave_rows8(rows0, rows1).reshape(-1).tolist() == order
